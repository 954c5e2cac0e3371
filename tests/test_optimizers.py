"""Optimizer zoo and scheduler tests (reference: tests/test_optimizer.cpp, tests/test_scheduler.cpp)."""
import math

import pytest
import torch

from innova_b200.training import optimizers as O


@pytest.mark.parametrize("name", O.OPTIMIZERS)
def test_optimizer_reduces_quadratic(name):
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(16, 8))
    target = torch.randn(16, 8)
    lr = {"sgd": 0.05, "nesterov": 0.05, "lars": 0.5, "lion": 0.01, "adafactor": 0.05, "adabound": 0.05}.get(name, 0.05)
    opt = O.make_optimizer(name, [w], lr=lr, weight_decay=0.0)
    first = None
    for _ in range(200):
        loss = ((w - target) ** 2).mean()
        first = first if first is not None else float(loss.detach())
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert float(((w - target) ** 2).mean()) < 0.5 * first, name


def test_sixteen_schedulers():
    assert len(O.SCHEDULERS) == 18 and O.CosineDecayScheduler is O.CosineLR and O.LRScheduler is O.Scheduler
    warm = O.WarmupScheduler(O.CosineDecayScheduler(1.0, 100), 10, 0.1)
    assert warm(0) == pytest.approx(0.1) and warm(5) == pytest.approx(0.55) and warm(10) == pytest.approx(1.0) and warm(60) == pytest.approx(0.5)
    assert O.LambdaScheduler(lambda s: 0.5 * s)(4) == 2.0
    assert O.StepLR(1.0, 10, 0.5)(25) == 0.25
    assert O.MultiStepLR(1.0, [5, 10], 0.1)(7) == pytest.approx(0.1)
    assert O.CosineLR(1.0, 100)(50) == pytest.approx(0.5)
    assert O.CosineLR(1.0, 100, 0.1)(100) == pytest.approx(0.1)
    assert O.WarmupCosineLR(1.0, 10, 110)(4) == pytest.approx(0.5)
    assert O.WarmupCosineLR(1.0, 10, 110)(60) == pytest.approx(0.5)
    assert O.LinearLR(1.0, 100)(25) == pytest.approx(0.75)
    assert O.PolynomialLR(1.0, 100, 2.0)(50) == pytest.approx(0.25)
    assert O.InverseSqrtLR(1.0, 100)(400) == pytest.approx(0.5)
    assert O.CyclicLR(0.1, 1.0, 10)(10) == pytest.approx(1.0)
    assert O.CyclicLR(0.1, 1.0, 10)(20) == pytest.approx(0.1)
    oc = O.OneCycleLR(1.0, 100)
    assert oc(30) == pytest.approx(1.0) and oc(100) == pytest.approx(1e-4)
    assert O.CosineRestartLR(1.0, 10)(10) == pytest.approx(1.0)
    assert O.ExponentialLR(1.0, 0.5)(3) == 0.125
    pl = O.ReduceLROnPlateau(1.0, factor=0.5, patience=1)
    for m in (1.0, 1.0, 1.0):
        pl.observe(m)
    assert pl(0) == 0.5
    seq = O.SequentialLR([O.LinearLR(0.1, 10, 1.0), O.CosineLR(1.0, 100)], [10])
    assert seq(5) == pytest.approx(0.55) and seq(10) == pytest.approx(1.0)
    ch = O.ChainedLR([O.StepLR(1.0, 10, 0.5), O.ExponentialLR(1.0, 0.9)])
    assert ch(10) == pytest.approx(0.5 * 0.9 ** 10)


def test_torch_engine_trains_tiny_model():
    from innova_b200.models import DenseModel, PRESETS
    from innova_b200.training.trainer import Trainer, TrainConfig
    cfg = PRESETS["tiny"]()
    model = DenseModel(cfg, dtype=torch.float32, device="cpu", seed=1)
    eng = O.TorchOptimizerEngine(model, "lion", lr=3e-4)
    tr = Trainer(model, TrainConfig(lr=3e-4, max_steps=8), engine=eng, total_steps=8)
    torch.manual_seed(0)
    x = torch.randint(0, cfg.vocab_size, (2, 33))
    l0 = float(tr.train_step(x[:, :-1].contiguous(), x[:, 1:].contiguous()))
    for _ in range(7):
        l = float(tr.train_step(x[:, :-1].contiguous(), x[:, 1:].contiguous()))
    assert l < l0
