"""MultiAgentSystem: topologies, message log, task affinity and decomposition, voting, blackboard, plan execution with and
without worker callables, supervisor take-back of failed subtasks, metrics."""
import pytest

from innova_b200.utils.multi_agent import (AgentMessage, AgentRole as R, CommTopology as T, MessageType as M, MultiAgentSystem)


def _team(topology=T.MESH):
    s = MultiAgentSystem(1, topology)
    ids = {r: s.add_agent(r) for r in (R.PLANNER, R.CODER, R.REVIEWER, R.TESTER, R.OPTIMIZER)}
    return s, ids


def test_agents_and_topologies():
    s = MultiAgentSystem(4, T.STAR)
    assert s.agent_count() == 4 and s.get_agent(0).role is R.SUPERVISOR and s.get_agent(0).name == "Supervisor_0"
    assert s.get_agent(2).name == "Custom_2" and s.add_agent(R.CODER, "ada") == 4 and s.get_agent(4).name == "ada"
    assert s.is_connected(0, 3) and s.is_connected(3, 0) and not s.is_connected(1, 2) and s.is_connected(2, 2) and not s.is_connected(1, 9)
    s.configure(T.RING)
    assert s.is_connected(1, 2) and s.is_connected(4, 0) and not s.is_connected(0, 2)
    s.configure(T.HIERARCHICAL)
    assert s.is_connected(0, 3) and s.is_connected(2, 3) and not s.is_connected(1, 3)
    s.configure(T.MESH)
    assert s.is_connected(1, 3)
    s.remove_agent(3)
    assert not s.get_agent(3).active and s.get_agent(3).status == "removed" and s.agent_count() == 5
    assert not s.communicate_direct(1, 3, "hi") and not s.communicate_direct(1, 17, "hi")
    assert MultiAgentSystem.string_to_role("tester") is R.TESTER and MultiAgentSystem.string_to_role("Tester") is R.CUSTOM
    assert MultiAgentSystem.role_to_string(R.OPTIMIZER) == "Optimizer"


def test_messages_queue_and_context():
    s = MultiAgentSystem(3, T.STAR)
    assert s.communicate_direct(0, 1, "hello") and not s.communicate_direct(1, 2, "blocked by the star")
    assert s.get_metrics(0).messages_sent == 1 and s.get_metrics(1).messages_received == 1
    assert s.get_agent(1).context_window == ["[From Supervisor_0]: hello"] and "TO Custom_1: hello" in s.get_histories()[0]
    sent = s.broadcast(1, M.PLAN_BROADCAST, "plan")             # agent 1 reaches only the hub in a star
    assert [m.to_agent for m in sent] == [0] and len(s.broadcast(0, M.PLAN_BROADCAST, "plan")) == 2
    assert [m.content for m in s.receive_messages(1)] == ["hello", "plan"] and [m.id for m in s.message_queue] == [0, 1, 2, 3]
    s.send_message(AgentMessage(from_agent=2, to_agent=-1, content="to all"))
    assert s.receive_messages(1)[-1].content == "to all" and "TO ALL: to all" in s.get_histories()[2]
    s.set_max_queue_size(2)
    s.send_message(AgentMessage(from_agent=0, to_agent=1, content="x"))
    assert len(s.message_queue) == 2 and s.message_queue[-1].id == 5
    for i in range(120):
        s.communicate_direct(0, 2, f"m{i}")
    assert len(s.get_agent(2).context_window) == 100 and s.get_agent(2).context_window[-1].endswith("m119")


def test_affinity_assignment_and_decomposition():
    s, ids = _team()
    assert s.affinity("implement the parser", s.get_agent(ids[R.CODER])) == pytest.approx(0.8)
    assert s.affinity("implement the parser", s.get_agent(ids[R.TESTER])) == pytest.approx(0.5)
    assert s.find_best_agent_for_task("verify the output") == ids[R.TESTER] and s.find_best_agent_for_task("hello") == 0
    assert s.assign_task_to_role(R.CODER, "write code") == ids[R.CODER] and s.get_agent(ids[R.CODER]).status == "working"
    assert s.get_agent(ids[R.CODER]).context_window == ["TASK: write code"] and s.receive_messages(ids[R.CODER])[0].type is M.TASK_ASSIGN
    assert s.find_best_agent_for_task("implement it") != ids[R.CODER] and s.assign_task_to_role(R.CUSTOM, "x") == -1
    sts = s.decompose_task("Build a fast tokenizer and optimize its speed", 10)
    assert [st.description.split(":")[0] for st in sts] == ["Analyze requirements", "Design solution for", "Implement code for", "Optimize",
                                                            "Review", "Test", "Final integration"]
    assert sts[0].dependencies == [] and all(sts[i].dependencies == [sts[i - 1].id] for i in range(1, 7)) and sts[0].priority == 7
    assert [st.id for st in s.get_ready_subtasks()] == [sts[0].id] and s.get_task_status(sts[3].id) == "pending" and s.get_task_status(99) == "not_found"
    assert len(s.decompose_task("think", 3)) == 3 and len(s.decompose_task("think", 10)) == 5 and s.get_subtasks()[0].id == 10
    st = s.get_subtasks()[0]
    assert s.assign_subtask_by_role(R.PLANNER, st.id) == ids[R.PLANNER] and st.status == "assigned" and st.assigned_agent == ids[R.PLANNER]
    assert s.assign_subtask_by_role(R.PLANNER, st.id) == -1                      # the only planner is busy now


def test_voting_and_blackboard():
    s = MultiAgentSystem(4, T.MESH)
    assert not s.check_consensus()
    s.submit_vote(0, "merge", True, 0.9, "looks right")
    s.submit_vote(1, "merge", True, 0.3)
    s.submit_vote(2, "merge", False, 0.6)
    s.submit_vote(9, "merge", False, 1.0)                                        # unknown agent: ignored
    assert len(s.get_votes()) == 3 and s.check_consensus(0.6) and not s.check_consensus(0.7)        # 1.2 / 1.8
    assert s.get_metrics(1).votes_cast == 1 and s.get_metrics(2).consensus_score == pytest.approx(1.2 / 1.8)
    assert s.receive_messages(3)[0].type is M.VOTE_CAST and s.receive_messages(3)[0].content.startswith("APPROVE merge confidence=0.9")
    s.reset_votes()
    s.submit_vote(0, "p", True, 0.0)
    assert not s.check_consensus(0.0)
    s.supervisor_resolve_conflicts()
    assert len(s.get_votes()) == 4 and s.check_consensus(0.99)
    s.write_blackboard("plan/a", "1", 0)
    s.write_blackboard("plan/b", "2", 1)
    s.write_blackboard("plan/a", "3", 2)
    assert s.read_blackboard("plan/a") == "3" and s.read_blackboard("none") == "" and len(s.search_blackboard("plan/")) == 2
    assert s.search_blackboard("plan/")[0].author_agent == 2
    s.write_blackboard("tmp", "x", 0, ttl=5)
    s.blackboard[-1].timestamp -= 1000
    assert s.cleanup_blackboard() == 1 and s.read_blackboard("tmp") == "" and len(s.blackboard) == 2
    s.supervisor_escalate("disk full")
    assert any(e.key.startswith("ESCALATION_") and e.value == "disk full" for e in s.blackboard)
    assert s.receive_messages(2)[-1].type is M.CONFLICT_ALERT


def test_plan_runs_to_completion_by_progress_ticks():
    s, ids = _team()
    plan = s.create_plan("build the cache", 10)
    assert len(plan.high_level_steps) == 6 and len(plan.detailed_subtasks) == 6 and plan.detailed_subtasks is s.get_subtasks()
    passes = 0
    while not s.execute_plan(plan) and passes < 200:
        passes += 1
    assert plan.completed and passes == 6 * 9 and s.get_plan_progress(plan) == pytest.approx(1.0)
    by_stage = {st.description.split(":")[0]: st.assigned_agent for st in plan.detailed_subtasks}
    assert by_stage["Implement code for"] == ids[R.CODER] and by_stage["Review"] == ids[R.REVIEWER] and by_stage["Test"] == ids[R.TESTER]
    assert sum(m.tasks_completed for m in s.get_all_metrics()) == 6 and all(a.status == "idle" for a in s.agents)
    assert s.get_metrics(ids[R.CODER]).avg_quality == 1.0 and s.execute_plan(plan)
    text = s.metrics_summary()
    assert "Topology: Mesh" in text and "Subtasks: 6" in text and f"Agent {ids[R.CODER]} [Coder_2]: completed=" in text and "quality=1.00" in text


def test_run_round_workers_failures_and_reassignment():
    s = MultiAgentSystem(1, T.MESH)
    calls = []

    def flaky(st):
        calls.append(("flaky", st.id))
        raise RuntimeError("no toolchain")

    coder_bad = s.add_agent(R.CODER, "bad", worker=flaky)
    coder_ok = s.add_agent(R.CODER, "good", worker=lambda st: f"done {st.id}")
    plan = s.create_plan("implement code", 3)                    # analyze, design, implement
    assert s.run_round(50) < 50 and plan.completed and plan.overall_progress == 1.0
    first = plan.detailed_subtasks[0]                            # "implement" in every description: both coders outrank the supervisor
    assert calls == [("flaky", first.id)] and all(st.assigned_agent == coder_ok and st.result == f"done {st.id}" for st in plan.detailed_subtasks)
    assert s.get_metrics(coder_ok).tasks_completed == 3          # after one success its quality bonus keeps it ahead of the failed coder
    assert s.get_metrics(coder_bad).tasks_failed == 1 and s.get_metrics(coder_bad).avg_quality == 0.0 and s.get_agent(coder_bad).status == "idle"
    kinds = [m.type for m in s.message_queue]
    assert M.ERROR_REPORT in kinds and M.FEEDBACK in kinds and M.TASK_RESULT in kinds
    assert any(v.proposal == "resolve_conflict" for v in s.get_votes())          # the supervisor read the error report
    assert s.read_blackboard("round_0_progress").endswith("%") and s.search_blackboard("round_")
    # a stalled subtask is taken back after the 30 s limit
    s2 = MultiAgentSystem(3, T.MESH)
    s2.create_plan("think", 1)
    st = s2.get_subtasks()[0]
    s2.execute_plan(s2.current_plan)
    first = st.assigned_agent
    assert st.status == "in_progress" and first == 0
    st.start_time -= 31000
    s2.supervisor_monitor()
    assert st.status == "assigned" and st.assigned_agent not in (-1, first) and st.progress == 0.0 and s2.get_metrics(first).tasks_failed == 1


def test_episode_chatter_is_seeded_and_respects_topology():
    a, b = MultiAgentSystem(5, T.RING), MultiAgentSystem(5, T.RING)
    a.run_episode(6)
    b.run_episode(6)
    assert [(m.from_agent, m.to_agent, m.content) for m in a.message_queue] == [(m.from_agent, m.to_agent, m.content) for m in b.message_queue]
    assert a.message_queue and all(a.is_connected(m.from_agent, m.to_agent) for m in a.message_queue)
    a.create_plan("think", 2)
    a.execute_plan(a.current_plan)
    a.run_episode(5)
    assert a.get_subtasks()[0].status == "completed"


def test_coordinator_five_phase_pipeline():
    from innova_b200.utils.asi import MultiAgentCoordinator
    c = MultiAgentCoordinator()
    out = c.run_task("sort numbers", max_critic_rounds=2)
    assert out.startswith("Synthesizer: Synthesize:\nAnalyst: Analyze the task: sort numbers [no model]\n") and out.endswith(" [no model]")
    assert c.current_round == 2 and not c.converged and len(c.get_agent_history("critic")) == 2 and len(c.get_agent_history("implementer")) == 3
    calls = []

    def model(prompt):
        calls.append(prompt.split(":", 1)[0])
        return "looks right [APPROVED]" if prompt.startswith("Critic") and calls.count("Critic") == 2 else f"<{len(calls)}>"

    c2 = MultiAgentCoordinator(call_model=model)
    assert c2.run_task("x", 5) == f"<{len(calls)}>" and c2.converged and c2.current_round == 2
    assert calls == ["Analyst", "Implementer", "Verifier", "Critic", "Implementer", "Verifier", "Critic", "Synthesizer"]
    c2.clear_agent_history("critic")
    assert c2.get_agent_history("critic") == [] and c2.get_agent_history("analyst") == ["<1>"]
    c2.clear_agent_history()
    assert c2.get_agent_history("analyst") == []
