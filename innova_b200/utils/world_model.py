"""``WorldModel``: a learned transition / reward model over keyed states with an ensemble for uncertainty, beam-search and
sampling-based (MPC) planning, counterfactual comparison and an importance-weighted state memory (reference:
include/oil/world_model.h:17-181, src/world_model.cpp:22-636).

What is kept: the keyed ``WorldState``; the 20-name action space with an action encoded at ``hash(name) % state_dim`` (hash =
31 * h + byte); the record types; beam search keeping the ``beam_width`` best cumulative rewards per step; MPC as the best of
``n_samples`` random action sequences; disagreement = root mean squared deviation of the ensemble's predictions from their
mean; total uncertainty = 0.6 epistemic + 0.4 aleatoric; the memory scoring rules (key match, importance, recency) and the
importance refresh 0.4 recency + 0.3 access + 0.3 old weight.

What is different by design: the dynamics are a real ensemble of small residual MLPs held as stacked tensors, so one
``torch.baddbmm`` evaluates every member on every candidate; ``train_on_transitions`` fits them (Adam on state-delta and reward
errors, each member on its own bootstrap resample) instead of only updating running error statistics; and both planners
evaluate all candidates of a horizon step in ONE batched call (beam x actions, or all MPC samples) instead of one model
forward per candidate. The reference's ``predict`` calls its ensemble routine, which calls ``predict`` again without a base
case; here the ensemble is the members of one batched forward.
"""
from __future__ import annotations

import math
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Sequence, Tuple, Union

import torch


@dataclass
class StateEntry:
    key: str = ""
    value: float = 0.0


@dataclass
class WorldState:
    entries: List[StateEntry] = field(default_factory=list)
    timestamp: int = 0
    importance: float = 0.0

    def get_value(self, key: str) -> float:
        return next((e.value for e in self.entries if e.key == key), 0.0)

    def set_value(self, key: str, val: float) -> None:
        for e in self.entries:
            if e.key == key:
                e.value = float(val)
                return
        self.entries.append(StateEntry(key, float(val)))

    def get_keys(self) -> List[str]:
        return [e.key for e in self.entries]

    def to_vector(self) -> List[float]:
        return [e.value for e in self.entries]

    def from_vector(self, v: Sequence[float], keys: Sequence[str]) -> None:
        self.entries = [StateEntry(k, float(x)) for k, x in zip(keys, v)]

    def copy(self) -> "WorldState":
        return WorldState([StateEntry(e.key, e.value) for e in self.entries], self.timestamp, self.importance)


@dataclass
class Transition:
    state: WorldState = field(default_factory=WorldState)
    action: str = ""
    next_state: WorldState = field(default_factory=WorldState)
    reward: float = 0.0
    predicted_reward: float = 0.0
    prediction_error: float = 0.0
    timestamp: int = 0


@dataclass
class PlanningBeam:
    action_sequence: List[str] = field(default_factory=list)
    cumulative_reward: float = 0.0
    final_state: WorldState = field(default_factory=WorldState)
    confidence: float = 0.0


@dataclass
class PredictionResult:
    predicted_state: WorldState = field(default_factory=WorldState)
    predicted_reward: float = 0.0
    uncertainty: float = 0.0
    confidence: float = 0.0
    ensemble_predictions: List[WorldState] = field(default_factory=list)


@dataclass
class CounterfactualResult:
    actual_state: WorldState = field(default_factory=WorldState)
    counterfactual_state: WorldState = field(default_factory=WorldState)
    intervention_description: str = ""
    state_difference: float = 0.0
    reward_difference: float = 0.0


@dataclass
class MPCPlan:
    action_sequence: List[str] = field(default_factory=list)
    predicted_states: List[WorldState] = field(default_factory=list)
    predicted_rewards: List[float] = field(default_factory=list)
    total_expected_reward: float = 0.0
    planning_horizon: int = 0


@dataclass
class UncertaintyEstimate:
    epistemic_uncertainty: float = 0.0
    aleatoric_uncertainty: float = 0.0
    total_uncertainty: float = 0.0
    ensemble_size: int = 0
    disagreement_magnitude: float = 0.0


@dataclass
class StateMemoryEntry:
    state: WorldState = field(default_factory=WorldState)
    importance_weight: float = 0.0
    access_count: int = 0
    last_accessed: int = 0


@dataclass
class WorldModelStats:
    total_transitions: int = 0
    total_predictions: int = 0
    avg_prediction_error: float = 0.0
    avg_reward_prediction_error: float = 0.0
    memory_entries: int = 0
    planning_calls: int = 0
    avg_planning_time_ms: float = 0.0


ACTIONS = ("move_forward", "move_backward", "turn_left", "turn_right", "accelerate", "decelerate", "interact", "observe", "plan",
           "execute", "wait", "explore", "gather_info", "process_data", "communicate", "analyze", "construct", "deconstruct",
           "optimize", "random_walk")


def action_slot(action: str, state_dim: int) -> int:
    h = 0
    for b in action.encode("utf-8", "replace"):
        h = (h * 31 + b) & 0xFFFFFFFF
    return h % state_dim


class WorldModel:
    max_transition_buffer = 100000
    max_state_memory = 10000

    def __init__(self, model=None, state_dim: int = 64, ensemble_size: int = 5, hidden: int = 64, device: Union[str, torch.device] = "cpu",
                 seed: int = 42):
        """``model`` is an optional language model kept for callers that want it (``self.model``); the dynamics are the
        ensemble owned here. States may carry up to ``state_dim`` entries."""
        self.model, self.state_dim, self.ensemble_size, self.hidden = model, state_dim, max(1, ensemble_size), hidden
        self.device = torch.device(device)
        self.possible_actions: List[str] = list(ACTIONS)
        self.gen = torch.Generator().manual_seed(seed)
        E, I, H, O = self.ensemble_size, 2 * state_dim, hidden, state_dim + 1
        rnd = lambda *shape, scale: (torch.randn(*shape, generator=self.gen) * scale).to(self.device).requires_grad_(True)
        self.w1, self.b1 = rnd(E, I, H, scale=1.0 / math.sqrt(I)), torch.zeros(E, 1, H, device=self.device, requires_grad=True)
        self.w2, self.b2 = rnd(E, H, O, scale=0.1 / math.sqrt(H)), torch.zeros(E, 1, O, device=self.device, requires_grad=True)
        self.residual_rms = 0.0                                   # running RMS of training residuals: the aleatoric term
        self.current_state = WorldState([StateEntry("x", 0.0), StateEntry("y", 0.0), StateEntry("energy", 1.0), StateEntry("knowledge", 0.0)],
                                        0, 1.0)
        self.transition_buffer: List[Transition] = []
        self.state_memory: Deque[StateMemoryEntry] = deque()
        self.stats = WorldModelStats()

    # ------------------------------------------------------------------------------------------ tensors
    def parameters(self) -> List[torch.Tensor]:
        return [self.w1, self.b1, self.w2, self.b2]

    def _state_tensor(self, states: Sequence[WorldState]) -> torch.Tensor:
        x = torch.zeros(len(states), self.state_dim)
        for i, s in enumerate(states):
            v = s.to_vector()[: self.state_dim]
            x[i, : len(v)] = torch.tensor(v)
        return x.to(self.device)

    def _action_tensor(self, actions: Sequence[str]) -> torch.Tensor:
        a = torch.zeros(len(actions), self.state_dim)
        a[torch.arange(len(actions)), torch.tensor([action_slot(n, self.state_dim) for n in actions], dtype=torch.long)] = 1.0
        return a.to(self.device)

    def members(self, states: torch.Tensor, actions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Every member on every row: ``states`` [N, state_dim], ``actions`` one-hot [N, state_dim] -> next states
        [E, N, state_dim] (input + predicted delta) and rewards [E, N]."""
        x = torch.cat([states, actions], dim=-1)[None].expand(self.ensemble_size, -1, -1)
        out = torch.baddbmm(self.b2, torch.tanh(torch.baddbmm(self.b1, x, self.w1)), self.w2)
        return states[None] + out[..., :-1], out[..., -1]

    @staticmethod
    def _disagreement(member_states: torch.Tensor, width: int) -> torch.Tensor:
        """[E, N, D] -> [N]: RMS deviation from the ensemble mean over the first ``width`` state entries."""
        if member_states.shape[0] <= 1 or width == 0:
            return member_states.new_zeros(member_states.shape[1])
        s = member_states[..., :width]
        return (s - s.mean(0, keepdim=True)).square().mean(dim=(0, 2)).sqrt()

    def _to_state(self, vec: torch.Tensor, like: WorldState, importance: float = 0.5) -> WorldState:
        keys = like.get_keys()[: self.state_dim]
        return WorldState([StateEntry(k, float(v)) for k, v in zip(keys, vec[: len(keys)].tolist())], like.timestamp + 1, importance)

    # ------------------------------------------------------------------------------------------ prediction
    @torch.no_grad()
    def predict(self, state: WorldState, action: str) -> PredictionResult:
        ns, rw = self.members(self._state_tensor([state]), self._action_tensor([action]))
        width = min(len(state.entries), self.state_dim)
        dis = float(self._disagreement(ns, width)[0])
        unc = 1.0 - math.exp(-dis) if self.ensemble_size > 1 else 1.0
        self.stats.total_predictions += 1
        return PredictionResult(self._to_state(ns.mean(0)[0], state), float(rw.mean()), unc, 1.0 - unc,
                                [self._to_state(ns[e, 0], state) for e in range(self.ensemble_size)])

    def predict_reward(self, state: WorldState, action: str) -> float:
        return self.predict(state, action).predicted_reward

    def predict_with_uncertainty(self, state: WorldState, action: str) -> PredictionResult:
        """As ``predict`` with the uncertainty set to the raw ensemble disagreement (confidence = 1 - it, floored at 0)."""
        r = self.predict(state, action)
        if len(r.ensemble_predictions) > 1:
            r.uncertainty = self.compute_ensemble_disagreement(r.ensemble_predictions)
            r.confidence = max(0.0, 1.0 - r.uncertainty)
        return r

    def ensemble_predict(self, state: WorldState, action: str) -> List[WorldState]:
        return self.predict(state, action).ensemble_predictions

    def simulate_trajectory(self, start_state: WorldState, actions: Sequence[str]) -> List[Transition]:
        out, cur = [], start_state
        for a in actions:
            p = self.predict(cur, a)
            out.append(Transition(cur, a, p.predicted_state, 0.0, p.predicted_reward, 0.0, cur.timestamp + 1))
            cur = p.predicted_state
        return out

    # ------------------------------------------------------------------------------------------ learning
    def update_transition_model(self, transition: Transition) -> float:
        """Scores one observed transition against the current model (running error statistics, the transition's own
        ``prediction_error``); returns the state error. Use ``train_on_transitions`` to fit."""
        p = self.predict(transition.state, transition.action)
        err = self.state_distance(p.predicted_state, transition.next_state)
        rerr = abs(p.predicted_reward - transition.reward)
        n = self.stats.total_transitions
        self.stats.avg_prediction_error = (self.stats.avg_prediction_error * n + err) / (n + 1)
        self.stats.avg_reward_prediction_error = (self.stats.avg_reward_prediction_error * n + rerr) / (n + 1)
        self.stats.total_transitions = n + 1
        transition.predicted_reward, transition.prediction_error = p.predicted_reward, err
        return err

    def train_on_transitions(self, transitions: Sequence[Transition], epochs: int = 10, lr: float = 1e-2, batch_size: int = 256) -> List[float]:
        """Fits the ensemble; member e sees its own bootstrap resample of each batch (a Poisson(1) weight per sample, the
        first member unweighted). Returns the mean loss per epoch."""
        if not transitions:
            return []
        s = self._state_tensor([t.state for t in transitions])
        a = self._action_tensor([t.action for t in transitions])
        width = torch.zeros(len(transitions), self.state_dim)
        for i, t in enumerate(transitions):
            width[i, : min(len(t.next_state.entries), self.state_dim)] = 1.0
        width = width.to(self.device)
        target = self._state_tensor([t.next_state for t in transitions])
        reward = torch.tensor([t.reward for t in transitions], device=self.device)
        opt = torch.optim.Adam(self.parameters(), lr)
        history, N = [], len(transitions)
        for _ in range(epochs):
            perm = torch.randperm(N, generator=self.gen).to(self.device)
            total, batches = 0.0, 0
            for lo in range(0, N, batch_size):
                idx = perm[lo: lo + batch_size]
                ns, rw = self.members(s[idx], a[idx])
                boot = torch.poisson(torch.ones(self.ensemble_size, idx.numel()), generator=self.gen).to(self.device)
                boot[0] = 1.0
                per = ((ns - target[idx][None]).square() * width[idx][None]).sum(-1) + (rw - reward[idx][None]).square()
                loss = (per * boot).sum() / boot.sum().clamp_min(1.0)
                opt.zero_grad(set_to_none=True)
                loss.backward()
                opt.step()
                total, batches = total + float(loss.detach()), batches + 1
            history.append(total / max(1, batches))
        with torch.no_grad():
            ns, _ = self.members(s, a)
            res = ((ns.mean(0) - target).square() * width).sum() / width.sum().clamp_min(1.0)
            self.residual_rms = float(res.sqrt())
        for t in transitions:
            self.update_transition_model(t)
        return history

    # ------------------------------------------------------------------------------------------ planning
    def get_action_space(self, n_actions: int) -> List[str]:
        return self.possible_actions[: max(0, n_actions)]

    @torch.no_grad()
    def beam_search_plan(self, current_state: WorldState, horizon: int, beam_width: int = 10, n_actions: int = 10) -> PlanningBeam:
        t0 = time.perf_counter()
        actions = self.get_action_space(n_actions)
        best = PlanningBeam()
        if not actions or horizon <= 0:
            best.final_state, best.confidence = current_state.copy(), 1.0
            return best
        A = len(actions)
        act = self._action_tensor(actions)
        states = self._state_tensor([current_state])                         # [beams, D]
        rewards = torch.zeros(1, device=self.device)
        paths: List[List[int]] = [[]]
        for _ in range(horizon):
            nb = states.shape[0]
            ns, rw = self.members(states.repeat_interleave(A, 0), act.repeat(nb, 1))      # every (beam, action) pair at once
            cand_r = rewards.repeat_interleave(A) + rw.mean(0)
            keep = cand_r.topk(min(beam_width, cand_r.numel())).indices
            states, rewards = ns.mean(0)[keep], cand_r[keep]
            paths = [paths[int(k) // A] + [int(k) % A] for k in keep.tolist()]
            self.stats.total_predictions += nb * A
        best.action_sequence = [actions[i] for i in paths[0]]
        best.cumulative_reward = float(rewards[0])
        final = self._to_state(states[0], current_state)
        final.timestamp = current_state.timestamp + horizon
        best.final_state, best.confidence = final, 1.0
        self._planned(t0)
        return best

    @torch.no_grad()
    def model_predictive_control(self, current_state: WorldState, horizon: int, n_samples: int = 50) -> MPCPlan:
        """Random shooting: ``n_samples`` action sequences rolled out together, the one with the highest summed predicted
        reward wins."""
        t0 = time.perf_counter()
        plan = MPCPlan(planning_horizon=horizon)
        if horizon <= 0 or n_samples <= 0:
            return plan
        actions = self.possible_actions
        table = self._action_tensor(actions)
        choice = torch.randint(0, len(actions), (n_samples, horizon), generator=self.gen)
        states = self._state_tensor([current_state]).expand(n_samples, -1)
        traj, rews = [], []
        for h in range(horizon):
            ns, rw = self.members(states, table[choice[:, h].to(self.device)])
            states = ns.mean(0)
            traj.append(states)
            rews.append(rw.mean(0))
        self.stats.total_predictions += n_samples * horizon
        rews_t = torch.stack(rews, dim=1)                                    # [samples, horizon]
        best = int(rews_t.sum(1).argmax())
        plan.action_sequence = [actions[i] for i in choice[best].tolist()]
        plan.predicted_rewards = rews_t[best].tolist()
        plan.total_expected_reward = float(rews_t[best].sum())
        cur = current_state
        for h in range(horizon):
            cur = self._to_state(traj[h][best], cur)
            plan.predicted_states.append(cur)
        self._planned(t0)
        return plan

    def _planned(self, t0: float) -> None:
        ms = (time.perf_counter() - t0) * 1e3
        n = self.stats.planning_calls
        self.stats.avg_planning_time_ms = (self.stats.avg_planning_time_ms * n + ms) / (n + 1)
        self.stats.planning_calls = n + 1

    def plan_actions(self, current_state: WorldState, horizon: int) -> List[str]:
        return self.beam_search_plan(current_state, horizon, 5, 10).action_sequence

    def evaluate_sequence_reward(self, start: WorldState, actions: Sequence[str]) -> float:
        return sum(t.predicted_reward for t in self.simulate_trajectory(start, actions))

    # ------------------------------------------------------------------------------------------ uncertainty / counterfactuals
    def estimate_uncertainty(self, state: WorldState, action: str) -> UncertaintyEstimate:
        members = self.ensemble_predict(state, action)
        dis = self.compute_ensemble_disagreement(members)
        return UncertaintyEstimate(dis, self.residual_rms, 0.6 * dis + 0.4 * self.residual_rms, len(members), dis)

    @staticmethod
    def compute_ensemble_disagreement(predictions: Sequence[WorldState]) -> float:
        if len(predictions) <= 1:
            return 0.0
        n = len(predictions[0].entries)
        if n == 0:
            return 0.0
        vals = torch.tensor([(p.to_vector() + [0.0] * n)[:n] for p in predictions])
        return float((vals - vals.mean(0, keepdim=True)).square().mean().sqrt())

    def counterfactual_analysis(self, actual_state: WorldState, actual_action: str, counterfactual_action: str) -> CounterfactualResult:
        a, c = self.predict(actual_state, actual_action), self.predict(actual_state, counterfactual_action)
        return CounterfactualResult(a.predicted_state, c.predicted_state,
                                    f"If '{actual_action}' was replaced with '{counterfactual_action}'",
                                    self.state_distance(a.predicted_state, c.predicted_state), c.predicted_reward - a.predicted_reward)

    def batch_counterfactual(self, state: WorldState, actual_action: str, alternatives: Sequence[str]) -> List[CounterfactualResult]:
        return [self.counterfactual_analysis(state, actual_action, alt) for alt in alternatives]

    # ------------------------------------------------------------------------------------------ memory
    @staticmethod
    def state_distance(a: WorldState, b: WorldState) -> float:
        return math.sqrt(sum((x - y) ** 2 for x, y in zip(a.to_vector(), b.to_vector())))

    @staticmethod
    def cosine_similarity_vec(a: Sequence[float], b: Sequence[float]) -> float:
        n = min(len(a), len(b))
        dot = sum(a[i] * b[i] for i in range(n))
        den = math.sqrt(sum(a[i] ** 2 for i in range(n)) * sum(b[i] ** 2 for i in range(n)))
        return dot / den if den > 1e-10 else 0.0

    def store_state(self, state: WorldState, importance: float = 1.0) -> None:
        self.state_memory.append(StateMemoryEntry(state, importance, 0, state.timestamp))
        if len(self.state_memory) > self.max_state_memory:
            self.consolidate_memory(self.max_state_memory // 2)
        self.stats.memory_entries = len(self.state_memory)

    def retrieve_most_relevant(self, query: Union[str, Sequence[float]]) -> WorldState:
        """By key: 2 * |value of that key| + 0.5 * importance + 0.3 * recency. By vector: cosine similarity + 0.2 *
        importance. The winner's access count and time are updated; an empty memory returns an empty state."""
        if not self.state_memory:
            return WorldState()
        now = self.current_state.timestamp

        def score(e: StateMemoryEntry) -> float:
            if isinstance(query, str):
                hit = sum(abs(x.value) * 2.0 for x in e.state.entries if x.key == query)
                return hit + 0.5 * e.importance_weight + 0.3 / (1.0 + (now - e.last_accessed))
            return self.cosine_similarity_vec(list(query), e.state.to_vector()) + 0.2 * e.importance_weight

        best = max(self.state_memory, key=score)
        best.access_count += 1
        best.last_accessed = now
        return best.state

    def update_importance_weights(self) -> None:
        now = self.current_state.timestamp
        for e in self.state_memory:
            recency = 1.0 / (1.0 + (now - e.last_accessed) * 0.01)
            e.importance_weight = 0.4 * recency + 0.3 * min(1.0, e.access_count / 10.0) + 0.3 * e.importance_weight

    def consolidate_memory(self, target_size: int = 1000) -> None:
        if len(self.state_memory) <= target_size:
            return
        self.update_importance_weights()
        kept = sorted(self.state_memory, key=lambda e: -e.importance_weight)[:target_size]
        self.state_memory = deque(kept)
        self.stats.memory_entries = len(self.state_memory)

    def get_memory(self) -> Deque[StateMemoryEntry]:
        return self.state_memory

    # ------------------------------------------------------------------------------------------ buffers / accessors
    def add_transition(self, transition: Transition) -> None:
        self.transition_buffer.append(transition)
        if len(self.transition_buffer) > self.max_transition_buffer:
            del self.transition_buffer[: len(self.transition_buffer) - self.max_transition_buffer]
        self.stats.total_transitions += 1

    def get_transition_buffer(self) -> List[Transition]:
        return self.transition_buffer

    def get_current_state(self) -> WorldState:
        return self.current_state.copy()

    def set_current_state(self, state: WorldState) -> None:
        self.current_state = state

    def get_stats(self) -> WorldModelStats:
        return self.stats

    def reset_stats(self) -> None:
        self.stats = WorldModelStats()
