"""WorldModel: the ensemble learns a toy environment, planners pick the rewarding actions with batched evaluation,
uncertainty is larger off the training distribution, counterfactuals, state memory rules, buffers and statistics."""
import random

import pytest
import torch

from innova_b200.utils.world_model import ACTIONS, StateEntry, Transition, WorldModel, WorldState, action_slot

EFFECT = {"move_forward": ("x", 1.0, -0.1), "move_backward": ("x", -1.0, -0.1), "gather_info": ("knowledge", 0.5, 1.0),
          "wait": ("energy", -0.1, 0.0), "explore": ("y", 1.0, 0.3)}


def _state(x=0.0, y=0.0, energy=1.0, knowledge=0.0, t=0):
    return WorldState([StateEntry("x", x), StateEntry("y", y), StateEntry("energy", energy), StateEntry("knowledge", knowledge)], t, 1.0)


def _step(s, a):
    key, delta, reward = EFFECT[a]
    n = s.copy()
    n.set_value(key, s.get_value(key) + delta)
    n.timestamp = s.timestamp + 1
    return n, reward


def _data(n=600, seed=0):
    rng = random.Random(seed)
    out = []
    for _ in range(n):
        s = _state(rng.uniform(-2, 2), rng.uniform(-2, 2), rng.uniform(0, 1), rng.uniform(0, 2))
        a = rng.choice(list(EFFECT))
        nxt, r = _step(s, a)
        out.append(Transition(s, a, nxt, r))
    return out


def test_world_state_and_action_encoding():
    s = WorldState()
    s.set_value("a", 1.5)
    s.set_value("b", -2.0)
    s.set_value("a", 3.0)
    assert s.get_keys() == ["a", "b"] and s.to_vector() == [3.0, -2.0] and s.get_value("zz") == 0.0
    s.from_vector([7.0, 8.0, 9.0], ["p", "q"])
    assert s.get_keys() == ["p", "q"] and s.get_value("q") == 8.0
    c = s.copy()
    c.set_value("p", 0.0)
    assert s.get_value("p") == 7.0
    h = 0
    for ch in b"wait":
        h = (h * 31 + ch) & 0xFFFFFFFF
    assert action_slot("wait", 64) == h % 64 and len(ACTIONS) == 20 and len({action_slot(a, 64) for a in EFFECT}) == 5


def test_ensemble_learns_dynamics_and_reward():
    wm = WorldModel(state_dim=16, ensemble_size=4, hidden=48, seed=1)
    data = _data()
    before = sum(wm.update_transition_model(t) for t in data[:50]) / 50
    hist = wm.train_on_transitions(data, epochs=60, lr=2e-2)
    assert hist[-1] < 0.05 * hist[0] and wm.residual_rms < 0.15
    test = _data(50, seed=9)
    wm.reset_stats()
    after = sum(wm.update_transition_model(t) for t in test) / 50
    assert after < 0.25 and after < 0.3 * before
    st = wm.get_stats()
    assert st.total_transitions == 50 and st.avg_prediction_error == pytest.approx(after, rel=1e-4) and st.avg_reward_prediction_error < 0.15
    assert test[0].prediction_error > 0 and abs(test[0].predicted_reward - test[0].reward) < 0.3
    s = _state(0.5, -0.5, 0.8, 1.0, t=3)
    p = wm.predict(s, "gather_info")
    assert p.predicted_state.get_keys() == ["x", "y", "energy", "knowledge"] and p.predicted_state.timestamp == 4
    assert p.predicted_state.get_value("knowledge") == pytest.approx(1.5, abs=0.2) and p.predicted_reward == pytest.approx(1.0, abs=0.2)
    assert len(p.ensemble_predictions) == 4 and 0 <= p.uncertainty <= 1 and p.confidence == pytest.approx(1 - p.uncertainty)
    assert wm.predict_reward(s, "move_forward") == pytest.approx(-0.1, abs=0.2)
    traj = wm.simulate_trajectory(s, ["move_forward", "move_forward", "explore"])
    assert len(traj) == 3 and traj[2].next_state.get_value("x") == pytest.approx(2.5, abs=0.4) and traj[1].state is traj[0].next_state
    assert wm.evaluate_sequence_reward(s, ["gather_info", "gather_info"]) == pytest.approx(2.0, abs=0.4)
    # planners
    calls = []
    orig = wm.members
    wm.members = lambda a, b: calls.append(a.shape[0]) or orig(a, b)
    beam = wm.beam_search_plan(s, 3, beam_width=4, n_actions=20)
    assert calls == [20, 80, 80]                                   # one batched call per step: beams x actions rows
    assert beam.action_sequence == ["gather_info"] * 3 and beam.cumulative_reward == pytest.approx(3.0, abs=0.5)
    assert beam.final_state.get_value("knowledge") == pytest.approx(2.5, abs=0.5) and beam.final_state.timestamp == 6
    calls.clear()
    mpc = wm.model_predictive_control(s, 2, n_samples=400)
    assert calls == [400, 400] and mpc.planning_horizon == 2 and len(mpc.predicted_states) == 2 and len(mpc.predicted_rewards) == 2
    assert mpc.action_sequence == ["gather_info", "gather_info"] and mpc.total_expected_reward == pytest.approx(sum(mpc.predicted_rewards))
    wm.members = orig
    quick = wm.plan_actions(s, 2)                                   # beam 5 over the first ten actions only
    assert len(quick) == 2 and set(quick) <= set(ACTIONS[:10]) and wm.get_stats().planning_calls == 3 and wm.get_stats().avg_planning_time_ms > 0
    assert wm.beam_search_plan(s, 0).action_sequence == [] and wm.model_predictive_control(s, 0).action_sequence == []
    # uncertainty: far outside the training range the members disagree more
    near, far = wm.estimate_uncertainty(s, "wait"), wm.estimate_uncertainty(_state(40.0, -35.0, 9.0, 30.0), "wait")
    assert far.epistemic_uncertainty > 3 * near.epistemic_uncertainty and near.ensemble_size == 4
    assert near.total_uncertainty == pytest.approx(0.6 * near.epistemic_uncertainty + 0.4 * near.aleatoric_uncertainty)
    assert near.aleatoric_uncertainty == pytest.approx(wm.residual_rms) and near.disagreement_magnitude == near.epistemic_uncertainty
    pu = wm.predict_with_uncertainty(s, "wait")
    assert pu.uncertainty == pytest.approx(wm.compute_ensemble_disagreement(pu.ensemble_predictions)) and pu.confidence == pytest.approx(1 - pu.uncertainty)
    # counterfactuals
    cf = wm.counterfactual_analysis(s, "move_forward", "gather_info")
    assert cf.intervention_description == "If 'move_forward' was replaced with 'gather_info'" and cf.reward_difference == pytest.approx(1.1, abs=0.3)
    assert cf.state_difference == pytest.approx((1.0 + 0.25) ** 0.5, abs=0.3)
    many = wm.batch_counterfactual(s, "wait", ["explore", "wait"])
    assert len(many) == 2 and many[1].state_difference == 0.0 and many[1].reward_difference == 0.0


def test_disagreement_formula_and_untrained_single_member():
    a, b = _state(1.0, 0.0), _state(3.0, 0.0)
    # entries: x in {1, 3} -> deviations +-1; other three entries identical -> mean square 2/8
    assert WorldModel.compute_ensemble_disagreement([a, b]) == pytest.approx((2 / 8) ** 0.5)
    assert WorldModel.compute_ensemble_disagreement([a]) == 0.0 and WorldModel.compute_ensemble_disagreement([WorldState(), WorldState()]) == 0.0
    solo = WorldModel(state_dim=8, ensemble_size=1)
    p = solo.predict(_state(), "wait")
    assert p.uncertainty == 1.0 and p.confidence == 0.0 and len(p.ensemble_predictions) == 1
    assert solo.train_on_transitions([]) == [] and WorldModel.state_distance(a, b) == 2.0
    assert WorldModel.cosine_similarity_vec([1, 0], [0, 1]) == 0.0 and WorldModel.cosine_similarity_vec([0, 0], [1, 1]) == 0.0
    assert solo.get_current_state().get_keys() == ["x", "y", "energy", "knowledge"] and solo.get_action_space(3) == list(ACTIONS[:3])


def test_state_memory_and_buffers():
    wm = WorldModel(state_dim=8, ensemble_size=2)
    assert wm.retrieve_most_relevant("x").entries == []
    wm.store_state(_state(x=0.1, t=0), 0.2)
    wm.store_state(_state(x=5.0, t=0), 0.1)
    wm.store_state(_state(knowledge=4.0, t=0), 1.0)
    assert wm.retrieve_most_relevant("x").get_value("x") == 5.0 and wm.retrieve_most_relevant("knowledge").get_value("knowledge") == 4.0
    assert wm.retrieve_most_relevant([0.0, 0.0, 1.0, 4.0]).get_value("knowledge") == 4.0
    mem = wm.get_memory()
    assert [e.access_count for e in mem] == [0, 1, 2] and wm.get_stats().memory_entries == 3
    cur = wm.get_current_state()
    cur.timestamp = 100
    wm.set_current_state(cur)
    mem[0].last_accessed = 100                                       # fresh, never accessed
    wm.update_importance_weights()
    assert mem[0].importance_weight == pytest.approx(0.4 * 1.0 + 0.0 + 0.3 * 0.2)
    assert mem[2].importance_weight == pytest.approx(0.4 / (1 + 100 * 0.01) + 0.3 * 0.2 + 0.3 * 1.0)
    wm.consolidate_memory(2)
    assert len(wm.get_memory()) == 2 and wm.get_memory()[0].importance_weight >= wm.get_memory()[1].importance_weight
    wm.consolidate_memory(5)
    assert len(wm.get_memory()) == 2
    wm.max_state_memory = 4
    for i in range(6):
        wm.store_state(_state(x=float(i)), 0.5)
    assert len(wm.get_memory()) <= 4
    wm.max_transition_buffer = 3
    for i in range(5):
        wm.add_transition(Transition(_state(), "wait", _state(), float(i)))
    assert [t.reward for t in wm.get_transition_buffer()] == [2.0, 3.0, 4.0] and wm.get_stats().total_transitions == 5
    wm.reset_stats()
    assert wm.get_stats().total_transitions == 0 and wm.get_stats().planning_calls == 0
