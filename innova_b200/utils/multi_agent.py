"""``MultiAgentSystem``: role-typed agents that exchange messages over a star / ring / mesh / hierarchical topology, split a
task into dependent subtasks, vote, share a blackboard and are watched by a supervisor (reference:
include/oil/multi_agent.h:17-210, src/multi_agent.cpp:51-790).

Rules kept from the reference: agent 0 is the supervisor; who may talk to whom per topology; the role/keyword affinity that
picks an agent for a task; the fixed decomposition (analyze, design, [implement], [optimize], review, test, integrate) with
each subtask depending on the one before; confidence-weighted consensus; the 30 s stall limit after which the supervisor
takes a subtask back and hands it to another agent.

One deliberate difference: a plan holds the SAME ``Subtask`` objects as the system, so that finishing a subtask through
``execute_plan`` or ``run_round`` is what the dependency check of the next subtask sees. (The reference copies the subtasks
into the plan and into the ready list, so there a status change made on the copy never unblocks a dependant.) An agent may
also carry a ``worker`` callable; a subtask given to such an agent completes with the worker's return value as its result
(or fails when the worker raises) instead of by the fixed progress increments.
"""
from __future__ import annotations

import enum
import random
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional


class AgentRole(enum.IntEnum):
    SUPERVISOR = 0
    PLANNER = 1
    CODER = 2
    REVIEWER = 3
    TESTER = 4
    OPTIMIZER = 5
    CUSTOM = 6


class CommTopology(enum.IntEnum):
    STAR = 0
    RING = 1
    MESH = 2
    HIERARCHICAL = 3


class MessageType(enum.IntEnum):
    TASK_ASSIGN = 0
    TASK_RESULT = 1
    VOTE_REQUEST = 2
    VOTE_CAST = 3
    FEEDBACK = 4
    STATUS_UPDATE = 5
    ERROR_REPORT = 6
    CONFLICT_ALERT = 7
    PLAN_BROADCAST = 8
    SUBTASK_DECOMP = 9


@dataclass
class AgentMessage:
    id: int = 0
    from_agent: int = -1
    to_agent: int = -1
    type: MessageType = MessageType.STATUS_UPDATE
    content: str = ""
    timestamp: int = 0
    priority: float = 0.5
    references: List[int] = field(default_factory=list)


@dataclass
class Subtask:
    id: int = 0
    description: str = ""
    status: str = ""
    assigned_agent: int = -1
    progress: float = 0.0
    dependencies: List[int] = field(default_factory=list)
    result: str = ""
    priority: int = 0
    start_time: float = 0.0
    end_time: float = 0.0


@dataclass
class AgentMetrics:
    tasks_completed: int = 0
    tasks_failed: int = 0
    avg_quality: float = 0.0
    total_time_ms: float = 0.0
    messages_sent: int = 0
    messages_received: int = 0
    votes_cast: int = 0
    consensus_score: float = 0.0


@dataclass
class AgentState:
    agent_id: int = -1
    role: AgentRole = AgentRole.CUSTOM
    name: str = ""
    context_window: List[str] = field(default_factory=list)
    history: List[str] = field(default_factory=list)
    status: str = ""
    metrics: AgentMetrics = field(default_factory=AgentMetrics)
    active: bool = True
    tasks_assigned: int = 0
    worker: Optional[Callable[[Subtask], Optional[str]]] = None


@dataclass
class BlackboardEntry:
    key: str = ""
    value: str = ""
    author_agent: int = -1
    timestamp: int = 0
    ttl: int = -1


@dataclass
class Vote:
    voter_agent: int = -1
    proposal: str = ""
    approve: bool = False
    confidence: float = 0.0
    rationale: str = ""


@dataclass
class HierarchicalPlan:
    goal: str = ""
    high_level_steps: List[str] = field(default_factory=list)
    detailed_subtasks: List[Subtask] = field(default_factory=list)
    completed: bool = False
    overall_progress: float = 0.0


_ROLE_KEYWORDS = {
    AgentRole.PLANNER: ("plan",),
    AgentRole.CODER: ("code", "implement"),
    AgentRole.REVIEWER: ("review", "check"),
    AgentRole.TESTER: ("test", "verify"),
    AgentRole.OPTIMIZER: ("optim", "speed"),
}
_MAX_CONTEXT = 100
_STALL_MS = 30000.0


def _now_ms() -> int:
    return int(time.monotonic() * 1000)


class MultiAgentSystem:
    def __init__(self, n_agents: int, topology: CommTopology = CommTopology.STAR):
        self.topology = CommTopology(topology)
        self.agents: List[AgentState] = []
        self.message_queue: List[AgentMessage] = []
        self.subtasks: List[Subtask] = []
        self.votes: List[Vote] = []
        self.blackboard: List[BlackboardEntry] = []
        self.current_plan = HierarchicalPlan()
        self.max_queue_size = 10000
        self.communication_delay_ms = 0
        self._next_message_id = 0
        self._next_subtask_id = 0
        self._monitor_cursor = 0          # id of the first message the supervisor has not read yet
        for i in range(n_agents):
            self.add_agent(AgentRole.SUPERVISOR if i == 0 else AgentRole.CUSTOM)

    # ------------------------------------------------------------------------------------------ agents
    def _valid(self, agent_id: int) -> bool:
        return 0 <= agent_id < len(self.agents)

    def add_agent(self, role: AgentRole, name: str = "", worker: Optional[Callable[[Subtask], Optional[str]]] = None) -> int:
        aid = len(self.agents)
        role = AgentRole(role)
        self.agents.append(AgentState(agent_id=aid, role=role, name=name or f"{role.name.capitalize()}_{aid}", status="idle",
                                      worker=worker))
        return aid

    def remove_agent(self, agent_id: int) -> None:
        """Agents keep their slot (ids stay stable); a removed one is inactive and receives nothing further."""
        if self._valid(agent_id):
            self.agents[agent_id].active = False
            self.agents[agent_id].status = "removed"

    def get_agent(self, agent_id: int) -> AgentState:
        return self.agents[agent_id]

    def agent_count(self) -> int:
        return len(self.agents)

    # ------------------------------------------------------------------------------------------ messages
    def is_connected(self, a: int, b: int) -> bool:
        if a == b:
            return True
        if not (self._valid(a) and self._valid(b)):
            return False
        if self.topology == CommTopology.STAR:
            return a == 0 or b == 0
        if self.topology == CommTopology.RING:
            n = len(self.agents)
            return (a + 1) % n == b or (b + 1) % n == a
        if self.topology == CommTopology.HIERARCHICAL:
            return a == 0 or b == 0 or abs(a - b) <= 1
        return True

    def send_message(self, msg: AgentMessage) -> AgentMessage:
        msg.id = self._next_message_id
        self._next_message_id += 1
        if msg.timestamp == 0:
            msg.timestamp = _now_ms()
        self.message_queue.append(msg)
        if len(self.message_queue) > self.max_queue_size:
            del self.message_queue[: len(self.message_queue) - self.max_queue_size]
        if self._valid(msg.from_agent):
            to = self.agents[msg.to_agent].name if self._valid(msg.to_agent) else "ALL"
            self.agents[msg.from_agent].history.append(f"[{msg.timestamp}] TO {to}: {msg.content}")
        return msg

    def receive_messages(self, agent_id: int) -> List[AgentMessage]:
        """Everything in the queue addressed to the agent or to all (-1). The queue is a log: reading does not consume."""
        return [m for m in self.message_queue if m.to_agent in (agent_id, -1)]

    def broadcast(self, from_agent: int, type: MessageType, content: str) -> List[AgentMessage]:   # noqa: A002
        return [self.send_message(AgentMessage(from_agent=from_agent, to_agent=i, type=type, content=content))
                for i, a in enumerate(self.agents) if i != from_agent and a.active and self.is_connected(from_agent, i)]

    def communicate_direct(self, src: int, dst: int, content: str) -> bool:
        if not (self._valid(src) and self._valid(dst)) or not (self.agents[src].active and self.agents[dst].active):
            return False
        if not self.is_connected(src, dst):
            return False
        self.send_message(AgentMessage(from_agent=src, to_agent=dst, content=content))
        self.agents[src].metrics.messages_sent += 1
        self.agents[dst].metrics.messages_received += 1
        self._remember(dst, f"[From {self.agents[src].name}]: {content}")
        return True

    def _remember(self, agent_id: int, entry: str) -> None:
        if not self._valid(agent_id):
            return
        a = self.agents[agent_id]
        a.context_window.append(entry)
        del a.context_window[: max(0, len(a.context_window) - _MAX_CONTEXT)]
        a.history.append(entry)

    # ------------------------------------------------------------------------------------------ tasks
    def affinity(self, task: str, agent: AgentState) -> float:
        low = task.lower()
        score = 0.5 + (0.3 if any(k in low for k in _ROLE_KEYWORDS.get(agent.role, ())) else 0.0)
        if agent.metrics.tasks_completed > 0:
            score += 0.1 * min(1.0, agent.metrics.avg_quality)
        return score

    def find_best_agent_for_task(self, task: str) -> int:
        """The free, active agent with the highest affinity (lowest id on ties); -1 when everyone is busy."""
        free = [a for a in self.agents if a.active and a.status != "working"]
        return max(free, key=lambda a: (self.affinity(task, a), -a.agent_id)).agent_id if free else -1

    def assign_task(self, agent_id: int, task: str) -> None:
        if not self._valid(agent_id) or not self.agents[agent_id].active:
            return
        a = self.agents[agent_id]
        a.status = "working"
        a.tasks_assigned += 1
        a.context_window.append("TASK: " + task)
        self.send_message(AgentMessage(from_agent=0, to_agent=agent_id, type=MessageType.TASK_ASSIGN, content=task))

    def assign_task_to_role(self, role: AgentRole, task: str) -> int:
        pool = [a for a in self.agents if a.active and a.role == role]
        if not pool:
            return -1
        best = max(pool, key=lambda a: (self.affinity(task, a), -a.agent_id)).agent_id
        self.assign_task(best, task)
        return best

    def get_task_status(self, task_id: int) -> str:
        return next((st.status for st in self.subtasks if st.id == task_id), "not_found")

    def decompose_task(self, complex_task: str, max_subtasks: int) -> List[Subtask]:
        low = complex_task.lower()
        stages = ["Analyze requirements: ", "Design solution for: "]
        if any(k in low for k in ("code", "implement", "build", "write")):
            stages.append("Implement code for: ")
        if any(k in low for k in ("optim", "performance", "speed")):
            stages.append("Optimize: ")
        stages += ["Review: ", "Test: ", "Final integration: "]
        n = min(max_subtasks, len(stages))
        self.subtasks = []
        for i in range(max(0, n)):
            st = Subtask(id=self._next_subtask_id, description=stages[i] + complex_task, status="pending", priority=n - i,
                         dependencies=[self.subtasks[-1].id] if self.subtasks else [])
            self._next_subtask_id += 1
            self.subtasks.append(st)
        return self.subtasks

    def get_subtasks(self) -> List[Subtask]:
        return self.subtasks

    def _subtask(self, subtask_id: int) -> Optional[Subtask]:
        return next((st for st in self.subtasks if st.id == subtask_id), None)

    def assign_subtask(self, subtask_id: int, agent_id: int) -> None:
        st = self._subtask(subtask_id)
        if st is None:
            return
        st.assigned_agent = agent_id
        st.status = "assigned"
        if self._valid(agent_id):
            self.assign_task(agent_id, st.description)

    def assign_subtask_by_role(self, role: AgentRole, subtask_id: int) -> int:
        if self._subtask(subtask_id) is None:
            return -1
        pool = [a for a in self.agents if a.active and a.role == role and a.status != "working"]
        if not pool:
            return -1
        best = max(pool, key=lambda a: (a.metrics.avg_quality, -a.agent_id)).agent_id
        self.assign_subtask(subtask_id, best)
        return best

    def _dependencies_done(self, st: Subtask) -> bool:
        done = {o.id for o in self.subtasks if o.status == "completed"}
        return all(d in done for d in st.dependencies)

    def get_ready_subtasks(self) -> List[Subtask]:
        return [st for st in self.subtasks if st.status == "pending" and self._dependencies_done(st)]

    def _start(self, st: Subtask) -> bool:
        """pending -> in_progress on a free agent; False when nobody is free."""
        if not self._valid(st.assigned_agent):
            agent = self.find_best_agent_for_task(st.description)
            if agent < 0:
                return False
            self.assign_subtask(st.id, agent)
        st.status = "in_progress"
        st.start_time = float(_now_ms())
        return True

    def _finish(self, st: Subtask) -> None:
        st.progress, st.status, st.end_time = 1.0, "completed", float(_now_ms())
        if self._valid(st.assigned_agent):
            a = self.agents[st.assigned_agent]
            a.metrics.tasks_completed += 1
            a.metrics.total_time_ms += st.end_time - st.start_time
            a.status = "idle"
            self.update_metrics(st.assigned_agent)

    def _advance(self, st: Subtask, step: float) -> None:
        """One tick of an in-progress subtask: run the agent's worker if it has one, else add ``step`` of progress."""
        worker = self.agents[st.assigned_agent].worker if self._valid(st.assigned_agent) else None
        if worker is not None:
            try:
                out = worker(st)
            except Exception as exc:   # noqa: BLE001 - a failing worker fails its subtask, not the system
                st.status = "failed"
                st.result = f"{type(exc).__name__}: {exc}"
                self.send_message(AgentMessage(from_agent=st.assigned_agent, to_agent=0, type=MessageType.ERROR_REPORT,
                                               content=f"subtask {st.id} failed: {st.result}"))
                return
            st.result = "" if out is None else str(out)
            self.send_message(AgentMessage(from_agent=st.assigned_agent, to_agent=0, type=MessageType.TASK_RESULT,
                                           content=st.result, references=[st.id]))
            self._finish(st)
            return
        st.progress += step
        if st.progress >= 1.0 - 1e-6:
            self._finish(st)

    # ------------------------------------------------------------------------------------------ voting
    def submit_vote(self, agent_id: int, proposal: str, approve: bool, confidence: float, rationale: str = "") -> None:
        if not self._valid(agent_id):
            return
        self.votes.append(Vote(agent_id, proposal, bool(approve), float(confidence), rationale))
        self.agents[agent_id].metrics.votes_cast += 1
        self.send_message(AgentMessage(from_agent=agent_id, to_agent=-1, type=MessageType.VOTE_CAST,
                                       content=f"{'APPROVE' if approve else 'REJECT'} {proposal} confidence={confidence:.6f}"))

    def check_consensus(self, threshold: float = 0.6) -> bool:
        """Approving share of the votes, each weighted by its confidence, against ``threshold``."""
        if not self.votes or not any(a.active for a in self.agents):
            return False
        total = sum(v.confidence for v in self.votes)
        if total < 1e-10:
            return False
        ratio = sum(v.confidence for v in self.votes if v.approve) / total
        for v in self.votes:
            if self._valid(v.voter_agent):
                self.agents[v.voter_agent].metrics.consensus_score = ratio
        return ratio >= threshold

    def get_votes(self) -> List[Vote]:
        return list(self.votes)

    def reset_votes(self) -> None:
        self.votes.clear()

    # ------------------------------------------------------------------------------------------ blackboard
    def write_blackboard(self, key: str, value: str, agent_id: int, ttl: int = -1) -> None:
        entry = next((e for e in self.blackboard if e.key == key), None)
        if entry is None:
            entry = BlackboardEntry(key=key)
            self.blackboard.append(entry)
        entry.value, entry.author_agent, entry.timestamp, entry.ttl = value, agent_id, _now_ms(), ttl

    def read_blackboard(self, key: str) -> str:
        return next((e.value for e in self.blackboard if e.key == key), "")

    def search_blackboard(self, prefix: str) -> List[BlackboardEntry]:
        return [e for e in self.blackboard if e.key.startswith(prefix)]

    def cleanup_blackboard(self) -> int:
        """Drops entries whose time to live (ms, > 0) has run out; returns how many."""
        now = _now_ms()
        keep = [e for e in self.blackboard if not (e.ttl > 0 and now - e.timestamp > e.ttl)]
        dropped = len(self.blackboard) - len(keep)
        self.blackboard = keep
        return dropped

    # ------------------------------------------------------------------------------------------ plans
    def create_plan(self, goal: str, max_subtasks: int) -> HierarchicalPlan:
        plan = HierarchicalPlan(goal=goal, high_level_steps=[
            "Understand goal: " + goal, "Decompose into subtasks", "Assign to specialist agents",
            "Execute subtasks in parallel where possible", "Review and integrate results", "Verify completion"])
        plan.detailed_subtasks = self.decompose_task(goal, max_subtasks)
        self.current_plan = plan
        return plan

    def _refresh_plan(self, plan: HierarchicalPlan) -> None:
        sts = plan.detailed_subtasks
        plan.overall_progress = sum(st.progress for st in sts) / len(sts) if sts else 0.0
        plan.completed = bool(sts) and all(st.status == "completed" for st in sts)

    def execute_plan(self, plan: HierarchicalPlan) -> bool:
        """One pass over the plan: start what is ready, advance what runs by 0.1, take back what failed."""
        if plan.completed:
            return True
        for st in plan.detailed_subtasks:
            if st.status in ("pending", "assigned") and self._dependencies_done(st) and not self._start(st):
                continue
            if st.status == "in_progress":
                self._advance(st, 0.1)
            if st.status == "failed":
                self.supervisor_reassign_failed(st.id)
        self._refresh_plan(plan)
        return plan.completed

    def get_plan_progress(self, plan: HierarchicalPlan) -> float:
        return plan.overall_progress

    # ------------------------------------------------------------------------------------------ supervisor
    def supervisor_monitor(self) -> None:
        """Reads the supervisor's mail since the last call (an error report opens a conflict vote) and takes back subtasks
        that have been in progress for more than 30 s."""
        fresh = [m for m in self.message_queue if m.id >= self._monitor_cursor]
        self._monitor_cursor = self._next_message_id
        if any(m.type == MessageType.ERROR_REPORT for m in fresh):
            self.supervisor_resolve_conflicts()
        for m in fresh:
            if m.type == MessageType.STATUS_UPDATE and self._valid(m.to_agent) and self.agents[m.to_agent].active:
                a = self.agents[m.to_agent]
                if not a.context_window or not a.context_window[-1].endswith(m.content):
                    a.context_window.append(m.content)
                    del a.context_window[: max(0, len(a.context_window) - _MAX_CONTEXT)]
        now = _now_ms()
        for st in self.subtasks:
            if st.status == "in_progress" and st.start_time > 0 and now - st.start_time > _STALL_MS:
                st.status = "failed"
                self.supervisor_reassign_failed(st.id)

    def supervisor_resolve_conflicts(self) -> None:
        self.reset_votes()
        for a in self.agents:
            if a.active:
                self.submit_vote(a.agent_id, "resolve_conflict", True, 0.7, "auto-resolve")

    def supervisor_reassign_failed(self, subtask_id: int) -> int:
        """Back to pending, the old agent is told and charged a failure, and another free agent (the old one only if
        nobody else is free) gets it. Returns the new agent or -1."""
        st = self._subtask(subtask_id)
        if st is None:
            return -1
        old = st.assigned_agent
        st.assigned_agent, st.status, st.progress = -1, "pending", 0.0
        if self._valid(old):
            self.agents[old].metrics.tasks_failed += 1
            self.agents[old].status = "idle"
            self.update_metrics(old)
            self.send_message(AgentMessage(from_agent=0, to_agent=old, type=MessageType.FEEDBACK,
                                           content="Task reassigned due to failure: " + st.description))
        others = [a for a in self.agents if a.active and a.status != "working" and a.agent_id != old]
        new = (max(others, key=lambda a: (self.affinity(st.description, a), -a.agent_id)).agent_id if others
               else self.find_best_agent_for_task(st.description))
        if new >= 0:
            self.assign_subtask(st.id, new)
        return new

    def supervisor_escalate(self, issue: str) -> None:
        self.write_blackboard(f"ESCALATION_{_now_ms()}", issue, 0)
        self.broadcast(0, MessageType.CONFLICT_ALERT, "ESCALATION: " + issue)

    # ------------------------------------------------------------------------------------------ metrics
    def update_metrics(self, agent_id: int) -> None:
        if not self._valid(agent_id):
            return
        m = self.agents[agent_id].metrics
        total = m.tasks_completed + m.tasks_failed
        if total:
            m.avg_quality = m.tasks_completed / total

    def get_metrics(self, agent_id: int) -> AgentMetrics:
        return self.agents[agent_id].metrics if self._valid(agent_id) else AgentMetrics()

    def get_all_metrics(self) -> List[AgentMetrics]:
        return [a.metrics for a in self.agents]

    def metrics_summary(self) -> str:
        lines = ["=== Multi-Agent System Metrics ===", f"Agents: {len(self.agents)}",
                 f"Topology: {self.topology.name.capitalize()}", f"Subtasks: {len(self.subtasks)}",
                 f"Messages in queue: {len(self.message_queue)}", f"Blackboard entries: {len(self.blackboard)}",
                 f"Votes cast: {len(self.votes)}", ""]
        for a in self.agents:
            if a.active:
                m = a.metrics
                lines.append(f"Agent {a.agent_id} [{a.name}]: completed={m.tasks_completed} failed={m.tasks_failed} "
                             f"quality={m.avg_quality:.2f} msgs_sent={m.messages_sent} msgs_rcvd={m.messages_received} "
                             f"votes={m.votes_cast} status={a.status}")
        return "\n".join(lines) + "\n"

    # ------------------------------------------------------------------------------------------ running
    def run_round(self, max_rounds: int = 10) -> int:
        """Up to ``max_rounds`` scheduling rounds over the current plan's subtasks; returns the rounds used."""
        used = 0
        for rnd in range(max_rounds):
            used = rnd + 1
            self.supervisor_monitor()
            for st in self.get_ready_subtasks():
                self._start(st)
            for st in self.subtasks:
                if st.status == "assigned" and self._dependencies_done(st):
                    self._start(st)
                if st.status == "in_progress":
                    self._advance(st, 0.15 + (rnd % 3) * 0.05)
                if st.status == "failed":
                    self.supervisor_reassign_failed(st.id)
            self._refresh_plan(self.current_plan)
            self.write_blackboard(f"round_{rnd}_progress", f"{int(self.current_plan.overall_progress * 100)}%", 0)
            if self.current_plan.completed or not self.current_plan.detailed_subtasks:
                break
        return used

    def run_episode(self, steps: int) -> None:
        """``steps`` ticks of background chatter (each connected idle pair talks with probability 0.3, seeded per step) while
        running subtasks advance by 0.2 a tick."""
        for step in range(steps):
            self.supervisor_monitor()
            rng = random.Random(42 + step)
            for a in self.agents:
                if not a.active or a.status == "working":
                    continue
                for b in self.agents:
                    if a is b or not b.active or not self.is_connected(a.agent_id, b.agent_id):
                        continue
                    if rng.random() < 0.3:
                        self.communicate_direct(a.agent_id, b.agent_id, f"Step {step} status update from {a.name}")
            for st in self.subtasks:
                if st.status == "in_progress":
                    self._advance(st, 0.2)
            self._refresh_plan(self.current_plan)

    # ------------------------------------------------------------------------------------------ configuration
    def configure(self, topology: CommTopology) -> None:
        self.topology = CommTopology(topology)

    def set_max_queue_size(self, max_size: int) -> None:
        self.max_queue_size = int(max_size)

    def set_communication_delay(self, delay_ms: int) -> None:
        self.communication_delay_ms = int(delay_ms)

    def get_histories(self) -> List[str]:
        return ["".join(h + "\n" for h in a.history) for a in self.agents]

    @staticmethod
    def string_to_role(role: str) -> AgentRole:
        return AgentRole.__members__.get(role.upper(), AgentRole.CUSTOM) if role == role.lower() else AgentRole.CUSTOM

    @staticmethod
    def role_to_string(role: AgentRole) -> str:
        return AgentRole(role).name.capitalize()
