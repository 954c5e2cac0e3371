"""RL trainers, evaluation metrics, HPO / NAS and log writers (reference: tests/test_rl*.cpp, tests/test_eval.cpp,
tests/test_hpo_nas.cpp) on CPU."""
import math

import torch

from innova_b200.models import DenseModel, PRESETS
from innova_b200.training import rl
from innova_b200.training import utils as U


def _model(seed=1):
    cfg = PRESETS["tiny"]()
    cfg.ste_format = ""
    return DenseModel(cfg, dtype=torch.float32, device="cpu", seed=seed), cfg


def test_gae_and_returns_match_hand_computation():
    r = torch.tensor([1.0, 0.0, 2.0])
    v = torch.tensor([0.5, 0.4, 0.3])
    adv, ret = rl.compute_gae(r, v, None, gamma=0.9, lam=0.8)
    d2 = 2.0 - 0.3
    d1 = 0.0 + 0.9 * 0.3 - 0.4
    d0 = 1.0 + 0.9 * 0.4 - 0.5
    a2, a1 = d2, d1 + 0.72 * d2
    a0 = d0 + 0.72 * a1
    assert torch.allclose(adv, torch.tensor([a0, a1, a2]), atol=1e-6) and torch.allclose(ret, adv + v)
    assert torch.allclose(rl.discounted_returns(r, 0.5), torch.tensor([1.5, 1.0, 2.0]))
    assert float(rl.kl_divergence(torch.randn(2, 3, 7), torch.zeros(2, 3, 7))) > 0
    x = torch.randn(2, 3, 7)
    assert abs(float(rl.kl_divergence(x, x))) < 1e-7


def test_dpo_increases_margin_and_ppo_step_runs():
    model, cfg = _model()
    g = torch.Generator().manual_seed(0)
    chosen = torch.randint(0, cfg.vocab_size, (4, 12), generator=g)
    rejected = torch.randint(0, cfg.vocab_size, (4, 12), generator=g)
    rejected[:, :4] = chosen[:, :4]
    dpo = rl.DPOTrainer(model, beta=0.5, lr=5e-4)
    l0, m0 = dpo.loss(chosen, rejected, prompt_len=4)
    assert abs(float(l0) - math.log(2)) < 1e-4 and float(m0.abs().max()) < 1e-4      # policy == reference
    for _ in range(8):
        dpo.train_step(chosen, rejected, prompt_len=4)
    l1, m1 = dpo.loss(chosen, rejected, prompt_len=4)
    assert float(l1) < float(l0) and float(m1.mean()) > 0
    ppo = rl.PPOTrainer(model, lr=1e-4)
    states, actions = chosen[:, :-1], chosen[:, 1:]
    with torch.no_grad():
        old = rl.sequence_log_probs(model(states).float(), actions)
        vals = ppo.values(states)
    rewards = torch.zeros_like(old)
    rewards[:, -1] = 1.0
    adv, ret = ppo.compute_gae(rewards, vals)
    out = ppo.train_step(states, actions, old, adv, ret)
    assert all(math.isfinite(v) for v in out.values()) and len(ppo.critic_parameters()) == 4


def test_rlhf_pipeline_round():
    policy, cfg = _model(2)
    backbone, _ = _model(3)
    rm = rl.RewardModel(backbone)
    pipe = rl.RLHFPipeline(policy, rm, preference_fn=lambda a, b: sum(a) >= sum(b))
    prompts = [[1, 2, 3], [4, 5, 6], [7, 8, 9], [3, 2, 1]]
    m = pipe.run(prompts, n_rounds=1, n_ppo_steps=1, max_new_tokens=4)
    assert m.rounds == 1 and len(pipe.buffer) == 4 and 0.0 <= m.reward_accuracy <= 1.0
    pipe.dpo_finetune(n_steps=2, batch_size=2)
    assert math.isfinite(pipe.metrics.dpo_loss) and 0.0 <= pipe.compute_reward_accuracy(pipe.buffer) <= 1.0


def test_eval_metrics():
    assert U.compute_bleu([1, 2, 3, 4, 5], [1, 2, 3, 4, 5]) == 1.0
    assert U.compute_bleu([1, 2, 3, 4, 5], [9, 8, 7, 6, 5, 4]) == 0.0
    assert abs(U.compute_rouge_l([1, 2, 3, 4], [1, 3, 4, 5]) - 0.75) < 1e-9
    r = U.eval_classification(torch.tensor([[2.0, 1.0], [0.0, 1.0], [3.0, 0.0], [0.0, 2.0]]), [0, 1, 1, 1])
    assert r.accuracy == 0.75 and 0 < r.f1_score < 1
    model, cfg = _model()
    toks = torch.randint(0, cfg.vocab_size, (90,), generator=torch.Generator().manual_seed(0)).tolist()
    p1 = U.eval_perplexity(model, toks, context_size=32, stride=16)
    assert p1.total_tokens == 89 and cfg.vocab_size * 0.3 < p1.perplexity < cfg.vocab_size * 3
    acc = U.eval_accuracy(model, toks, context_size=32)
    assert acc.total == 89 and 0 <= acc.accuracy <= 1
    hs = U.eval_hellaswag(model, [[1, 2, 3]] * 3, [[4, 5]] * 3, [[6, 7]] * 3)
    assert hs.total == 3
    ev = U.ModelEvaluator(model).run_all(toks)
    assert [e.task_name for e in ev] == ["perplexity", "accuracy"]


def test_hpo_nas_and_helpers(tmp_path):
    target = math.log(3e-3)
    eng = U.HPOEngine(lambda c, b: (math.log(c.lr) - target) ** 2 + c.weight_decay + 1.0 / b, seed=1)
    best_r = eng.random_search(10)[0]
    best_b = eng.bayesian_optimization(5, 15)[0]
    assert best_b.score <= best_r.score + 1e-9
    assert eng.successive_halving(9, 2)[0].score < 5 and eng.population_based_training(4, 3)[0].score < 5
    assert isinstance(eng.optimize(8, "random"), U.HPConfig)
    nas = U.NASEngine(lambda a: abs(a.params(1000) - 3_000_000) / 1e6, U.HardwareConstraints(max_params=5_000_000))
    best = nas.search(U.Architecture(128, 2, 4), 40)
    assert nas.feasible(best) and best.score <= nas.history[0].score
    sc = U.MixedPrecisionScaler(128.0, growth_interval=2)
    assert not sc.update(True) and sc.scale == 64.0 and sc.update(False) and sc.update(False) and sc.scale == 128.0
    p = torch.nn.Parameter(torch.zeros(3))
    ema = U.EMA([p], 0.5)
    p.data.fill_(2.0)
    ema.update()
    assert torch.allclose(ema.shadow[0], torch.ones(3))
    es = U.EarlyStopping(patience=2)
    assert [es.step(v) for v in (1.0, 0.9, 0.95, 0.96)] == [False, False, False, True]
    acc = U.GradientAccumulator(3)
    assert [acc.ready() for _ in range(6)] == [False, False, True, False, False, True]
    w = U.CSVLogWriter(str(tmp_path / "l.csv"), ["step", "loss"])
    w.write(step=1, loss=2.5)
    w.close()
    j = U.JSONLLogWriter(str(tmp_path / "l.jsonl"))
    j.write(step=1, loss=2.5)
    j.close()
    s = U.ScalarLogWriter(str(tmp_path / "l.tb"))
    s.add_scalar("loss", 2.5, 1)
    s.close()
    assert open(tmp_path / "l.csv").read().splitlines() == ["step,loss", "1,2.5"]
    assert open(tmp_path / "l.tb").read().startswith("loss 1 2.5")
    assert U.ProgressTracker(10).summary()["progress"] == 0.0
