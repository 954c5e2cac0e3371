"""The optimizer zoo and learning-rate schedulers.

Optimizers of the reference (include/oil/optimizer.h:14-259, src/optimizer.cpp): AdamW (the fused
flat engine in ``flat_engine.py``), SGD(+Nesterov), Adam, Adamax, NAdam, RAdam, RMSProp and Adafactor
come from ``torch.optim``; Lion, Ranger, AdaBound, LAMB, LARS and NovoGrad are implemented here.
``TorchOptimizerEngine`` gives any of them the engine interface the Trainer uses (fp32 master
weights, fp32 ``main_grad`` buffers fed by the fused wgrad kernels, global-norm clip).

Schedulers (include/oil/scheduler.h:8-203): sixteen step -> learning-rate rules, composable with
``Sequential`` and ``Chained``; ``ReduceLROnPlateau`` is driven by a metric.
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence

import torch
from torch.optim import Optimizer


# ---------------------------------------------------------------------------------------------- optimizers
class Lion(Optimizer):
    def __init__(self, params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["m"] = torch.zeros_like(p)
                p.mul_(1 - g["lr"] * g["weight_decay"])
                upd = (st["m"] * b1 + p.grad * (1 - b1)).sign_()
                p.add_(upd, alpha=-g["lr"])
                st["m"].mul_(b2).add_(p.grad, alpha=1 - b2)


class AdaBound(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), final_lr=0.1, gamma=1e-3, eps=1e-8, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, final_lr=final_lr, gamma=gamma, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["t"], st["m"], st["v"] = 0, torch.zeros_like(p), torch.zeros_like(p)
                st["t"] += 1
                t = st["t"]
                grad = p.grad + g["weight_decay"] * p
                st["m"].mul_(b1).add_(grad, alpha=1 - b1)
                st["v"].mul_(b2).addcmul_(grad, grad, value=1 - b2)
                step = g["lr"] * math.sqrt(1 - b2 ** t) / (1 - b1 ** t)
                lo = g["final_lr"] * (1 - 1 / (g["gamma"] * t + 1))
                hi = g["final_lr"] * (1 + 1 / (g["gamma"] * t))
                rate = (step / (st["v"].sqrt() + g["eps"])).clamp_(lo, hi)
                p.sub_(rate * st["m"])


class Lamb(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["t"], st["m"], st["v"] = 0, torch.zeros_like(p), torch.zeros_like(p)
                st["t"] += 1
                st["m"].mul_(b1).add_(p.grad, alpha=1 - b1)
                st["v"].mul_(b2).addcmul_(p.grad, p.grad, value=1 - b2)
                mh = st["m"] / (1 - b1 ** st["t"])
                vh = st["v"] / (1 - b2 ** st["t"])
                upd = mh / (vh.sqrt() + g["eps"]) + g["weight_decay"] * p
                wn, un = p.norm(), upd.norm()
                trust = float(wn / un) if wn > 0 and un > 0 else 1.0
                p.add_(upd, alpha=-g["lr"] * trust)


class LARS(Optimizer):
    def __init__(self, params, lr=0.1, momentum=0.9, weight_decay=1e-4, trust=1e-3):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay, trust=trust))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["buf"] = torch.zeros_like(p)
                wn, gn = p.norm(), p.grad.norm()
                local = float(g["trust"] * wn / (gn + g["weight_decay"] * wn)) if wn > 0 and gn > 0 else 1.0
                upd = (p.grad + g["weight_decay"] * p) * (local * g["lr"])
                st["buf"].mul_(g["momentum"]).add_(upd)
                p.sub_(st["buf"])


class NovoGrad(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.95, 0.98), eps=1e-8, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                gsq = p.grad.pow(2).sum()
                if not st:
                    st["v"], st["m"] = gsq.clone(), torch.zeros_like(p)
                else:
                    st["v"].mul_(b2).add_(gsq, alpha=1 - b2)
                upd = p.grad / (st["v"].sqrt() + g["eps"]) + g["weight_decay"] * p
                st["m"].mul_(b1).add_(upd)
                p.add_(st["m"], alpha=-g["lr"])


class Ranger(Optimizer):
    """RAdam with Lookahead (k steps, slow-weight interpolation alpha)."""

    def __init__(self, params, lr=1e-3, betas=(0.95, 0.999), eps=1e-5, weight_decay=0.0, k=6, alpha=0.5):
        params = list(params)
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, k=k, alpha=alpha))
        self.inner = torch.optim.RAdam(self.param_groups, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        self.n = 0

    @torch.no_grad()
    def step(self):
        self.inner.step()
        self.n += 1
        for g in self.param_groups:
            if self.n % g["k"]:
                continue
            for p in g["params"]:
                st = self.state[p]
                if "slow" not in st:
                    st["slow"] = p.detach().clone()
                st["slow"].add_(p - st["slow"], alpha=g["alpha"])
                p.copy_(st["slow"])


def make_optimizer(name: str, params, lr: float, weight_decay: float = 0.0, **kw) -> Optimizer:
    n = name.lower()
    table = {
        "sgd": lambda: torch.optim.SGD(params, lr=lr, momentum=kw.get("momentum", 0.9), weight_decay=weight_decay),
        "nesterov": lambda: torch.optim.SGD(params, lr=lr, momentum=kw.get("momentum", 0.9), nesterov=True, weight_decay=weight_decay),
        "adam": lambda: torch.optim.Adam(params, lr=lr, weight_decay=weight_decay),
        "adamw": lambda: torch.optim.AdamW(params, lr=lr, weight_decay=weight_decay),
        "adamax": lambda: torch.optim.Adamax(params, lr=lr, weight_decay=weight_decay),
        "nadam": lambda: torch.optim.NAdam(params, lr=lr, weight_decay=weight_decay),
        "radam": lambda: torch.optim.RAdam(params, lr=lr, weight_decay=weight_decay),
        "rmsprop": lambda: torch.optim.RMSprop(params, lr=lr, weight_decay=weight_decay),
        "adafactor": lambda: torch.optim.Adafactor(params, lr=lr, weight_decay=weight_decay),
        "lion": lambda: Lion(params, lr=lr, weight_decay=weight_decay),
        "ranger": lambda: Ranger(params, lr=lr, weight_decay=weight_decay),
        "adabound": lambda: AdaBound(params, lr=lr, weight_decay=weight_decay),
        "lamb": lambda: Lamb(params, lr=lr, weight_decay=weight_decay),
        "lars": lambda: LARS(params, lr=lr, weight_decay=weight_decay),
        "novograd": lambda: NovoGrad(params, lr=lr, weight_decay=weight_decay),
    }
    if n not in table:
        raise ValueError(f"unknown optimizer {name!r}; known: {sorted(table)}")
    return table[n]()


OPTIMIZERS = ["sgd", "nesterov", "adam", "adamw", "adamax", "nadam", "radam", "rmsprop", "adafactor", "lion", "ranger", "adabound", "lamb", "lars",
              "novograd"]


class TorchOptimizerEngine:
    """Engine interface of the Trainer on top of any ``torch.optim`` style optimizer: fp32 master copies
    are what the optimizer updates; gradients arrive in the parameters' fp32 ``main_grad`` buffers."""

    def __init__(self, model, name: str, lr: float = 1e-3, weight_decay: float = 0.0, max_grad_norm: float = 1.0, lr_schedule=None, **kw):
        self.model, self.lr, self.max_grad_norm, self.lr_schedule = model, lr, max_grad_norm, lr_schedule
        self.entries, self.masters = [], []
        off = 0
        params = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        self.total = sum(p.numel() for _, p in params)
        dev = params[0][1].device
        self.flat_grad = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.flat_param = torch.zeros(self.total, dtype=params[0][1].dtype, device=dev)
        for n, p in params:
            k = p.numel()
            self.entries.append((n, p, off, k))
            self.flat_param[off:off + k].copy_(p.data.reshape(-1))
            p.data = self.flat_param[off:off + k].view(p.shape)
            p.main_grad = self.flat_grad[off:off + k].view(p.shape)
            m = p.detach().float().clone().requires_grad_(True)
            self.masters.append(m)
            off += k
        self.opt = make_optimizer(name, self.masters, lr, weight_decay, **kw)
        self.step_count = 0
        self.shard_lo, self.shard_hi = 0, self.total

    @property
    def master(self):
        return torch.cat([m.detach().reshape(-1) for m in self.masters])

    def _moment(self, keys):
        out = []
        for m in self.masters:
            st = self.opt.state.get(m, {})
            t = next((st[k] for k in keys if k in st and torch.is_tensor(st[k]) and st[k].shape == m.shape), None)
            out.append((t if t is not None else torch.zeros_like(m)).detach().reshape(-1).float())
        return torch.cat(out)

    @property
    def exp_avg(self):
        return self._moment(("exp_avg", "m", "momentum_buffer", "buf"))

    @property
    def exp_avg_sq(self):
        return self._moment(("exp_avg_sq", "v", "square_avg", "exp_inf"))

    def sync_master_from_params(self):
        with torch.no_grad():
            for (n, p, off, k), m in zip(self.entries, self.masters):
                m.copy_(p.detach().float())

    def current_lr(self):
        return self.lr_schedule(self.step_count) if self.lr_schedule is not None else self.lr

    def zero_grad(self):
        self.flat_grad.zero_()

    def step(self, grad_scale: float = 1.0):
        self.step_count += 1
        lr = self.current_lr()
        for g in self.opt.param_groups:
            g["lr"] = lr
        scale = grad_scale
        if self.max_grad_norm and self.max_grad_norm > 0:
            norm = float(self.flat_grad.norm()) * grad_scale
            scale *= min(1.0, self.max_grad_norm / (norm + 1e-6))
        for (n, p, off, k), m in zip(self.entries, self.masters):
            m.grad = p.main_grad.detach().float().mul(scale).view_as(m)
        self.opt.step()
        with torch.no_grad():
            for (n, p, off, k), m in zip(self.entries, self.masters):
                p.data.copy_(m.detach().to(p.dtype))
        self.flat_grad.zero_()


# ---------------------------------------------------------------------------------------------- schedulers
class Scheduler:
    def __init__(self, base_lr: float):
        self.base_lr = base_lr

    def __call__(self, step: int) -> float:
        return self.base_lr


class ConstantLR(Scheduler):
    pass


class StepLR(Scheduler):
    def __init__(self, base_lr, step_size, gamma=0.1):
        super().__init__(base_lr)
        self.step_size, self.gamma = step_size, gamma

    def __call__(self, step):
        return self.base_lr * self.gamma ** (step // self.step_size)


class MultiStepLR(Scheduler):
    def __init__(self, base_lr, milestones: Sequence[int], gamma=0.1):
        super().__init__(base_lr)
        self.milestones, self.gamma = sorted(milestones), gamma

    def __call__(self, step):
        return self.base_lr * self.gamma ** sum(step >= m for m in self.milestones)


class ExponentialLR(Scheduler):
    def __init__(self, base_lr, gamma=0.999):
        super().__init__(base_lr)
        self.gamma = gamma

    def __call__(self, step):
        return self.base_lr * self.gamma ** step


class CosineLR(Scheduler):
    def __init__(self, base_lr, total_steps, min_lr=0.0):
        super().__init__(base_lr)
        self.total, self.min_lr = max(1, total_steps), min_lr

    def __call__(self, step):
        t = min(1.0, step / self.total)
        return self.min_lr + 0.5 * (self.base_lr - self.min_lr) * (1 + math.cos(math.pi * t))


class CosineRestartLR(Scheduler):
    def __init__(self, base_lr, period, mult=1.0, min_lr=0.0):
        super().__init__(base_lr)
        self.period, self.mult, self.min_lr = period, mult, min_lr

    def __call__(self, step):
        period, s = self.period, step
        while s >= period:
            s -= period
            period = max(1, int(period * self.mult))
        return self.min_lr + 0.5 * (self.base_lr - self.min_lr) * (1 + math.cos(math.pi * s / period))


class LinearLR(Scheduler):
    def __init__(self, base_lr, total_steps, end_lr=0.0):
        super().__init__(base_lr)
        self.total, self.end_lr = max(1, total_steps), end_lr

    def __call__(self, step):
        t = min(1.0, step / self.total)
        return self.base_lr + (self.end_lr - self.base_lr) * t


class PolynomialLR(Scheduler):
    def __init__(self, base_lr, total_steps, power=2.0, end_lr=0.0):
        super().__init__(base_lr)
        self.total, self.power, self.end_lr = max(1, total_steps), power, end_lr

    def __call__(self, step):
        t = min(1.0, step / self.total)
        return (self.base_lr - self.end_lr) * (1 - t) ** self.power + self.end_lr


class WarmupCosineLR(Scheduler):
    def __init__(self, base_lr, warmup_steps, total_steps, min_lr=0.0):
        super().__init__(base_lr)
        self.warmup, self.cos = warmup_steps, CosineLR(base_lr, max(1, total_steps - warmup_steps), min_lr)

    def __call__(self, step):
        if step < self.warmup:
            return self.base_lr * (step + 1) / self.warmup
        return self.cos(step - self.warmup)


class WarmupLinearLR(Scheduler):
    def __init__(self, base_lr, warmup_steps, total_steps, end_lr=0.0):
        super().__init__(base_lr)
        self.warmup, self.lin = warmup_steps, LinearLR(base_lr, max(1, total_steps - warmup_steps), end_lr)

    def __call__(self, step):
        if step < self.warmup:
            return self.base_lr * (step + 1) / self.warmup
        return self.lin(step - self.warmup)


class InverseSqrtLR(Scheduler):
    def __init__(self, base_lr, warmup_steps=1000):
        super().__init__(base_lr)
        self.warmup = max(1, warmup_steps)

    def __call__(self, step):
        s = max(1, step)
        return self.base_lr * min(s / self.warmup, math.sqrt(self.warmup / s))


class CyclicLR(Scheduler):
    def __init__(self, base_lr, max_lr, step_size):
        super().__init__(base_lr)
        self.max_lr, self.step_size = max_lr, step_size

    def __call__(self, step):
        cycle = math.floor(1 + step / (2 * self.step_size))
        x = abs(step / self.step_size - 2 * cycle + 1)
        return self.base_lr + (self.max_lr - self.base_lr) * max(0.0, 1 - x)


class OneCycleLR(Scheduler):
    def __init__(self, max_lr, total_steps, pct_start=0.3, div=25.0, final_div=1e4):
        super().__init__(max_lr)
        self.total, self.up = max(1, total_steps), max(1, int(pct_start * total_steps))
        self.lo, self.end = max_lr / div, max_lr / final_div

    def __call__(self, step):
        if step < self.up:
            return self.lo + (self.base_lr - self.lo) * step / self.up
        t = min(1.0, (step - self.up) / max(1, self.total - self.up))
        return self.end + 0.5 * (self.base_lr - self.end) * (1 + math.cos(math.pi * t))


class ReduceLROnPlateau(Scheduler):
    def __init__(self, base_lr, factor=0.5, patience=3, min_lr=1e-8):
        super().__init__(base_lr)
        self.factor, self.patience, self.min_lr = factor, patience, min_lr
        self.best, self.bad, self.lr = float("inf"), 0, base_lr

    def observe(self, metric: float):
        if metric < self.best - 1e-8:
            self.best, self.bad = metric, 0
        else:
            self.bad += 1
            if self.bad > self.patience:
                self.lr, self.bad = max(self.min_lr, self.lr * self.factor), 0

    def __call__(self, step):
        return self.lr


class SequentialLR(Scheduler):
    def __init__(self, schedulers: List[Scheduler], milestones: Sequence[int]):
        super().__init__(schedulers[0].base_lr)
        self.schedulers, self.milestones = schedulers, list(milestones)

    def __call__(self, step):
        i, start = 0, 0
        for k, m in enumerate(self.milestones):
            if step >= m:
                i, start = k + 1, m
        return self.schedulers[i](step - start)


class ChainedLR(Scheduler):
    """Product of the members' multiplicative factors."""

    def __init__(self, schedulers: List[Scheduler]):
        super().__init__(schedulers[0].base_lr)
        self.schedulers = schedulers

    def __call__(self, step):
        lr = self.base_lr
        for s in self.schedulers:
            lr *= s(step) / s.base_lr
        return lr


class WarmupLR(Scheduler):
    """Linear ramp from ``warmup_start_lr`` to the wrapped schedule's first value over ``warmup_steps``, then the wrapped
    schedule counted from its own step 0 (reference: ``WarmupScheduler``, src/scheduler.cpp:62-70)."""

    def __init__(self, wrapped: Scheduler, warmup_steps: int, warmup_start_lr: float = 0.0):
        super().__init__(wrapped.base_lr)
        self.wrapped, self.warmup_steps, self.warmup_start_lr = wrapped, warmup_steps, warmup_start_lr

    def __call__(self, step):
        if step < self.warmup_steps:
            return self.warmup_start_lr + (self.wrapped(0) - self.warmup_start_lr) * step / self.warmup_steps
        return self.wrapped(step - self.warmup_steps)


class LambdaLR(Scheduler):
    def __init__(self, fn, base_lr: float = 1.0):
        super().__init__(base_lr)
        self.fn = fn

    def __call__(self, step):
        return self.fn(step)


# the reference's class names (include/oil/scheduler.h:8-203)
LRScheduler = Scheduler
ConstantScheduler, LinearDecayScheduler, CosineDecayScheduler, ExponentialDecayScheduler = ConstantLR, LinearLR, CosineLR, ExponentialLR
StepDecayScheduler, ReduceLROnPlateauScheduler, OneCycleScheduler, WarmupScheduler = StepLR, ReduceLROnPlateau, OneCycleLR, WarmupLR
SequentialScheduler, LambdaScheduler, ChainedScheduler, CosineWarmupRestart = SequentialLR, LambdaLR, ChainedLR, CosineRestartLR
PolyScheduler, MultiStepDecay, LinearWarmupDecay = PolynomialLR, MultiStepLR, WarmupLinearLR

SCHEDULERS = [ConstantLR, StepLR, MultiStepLR, ExponentialLR, CosineLR, CosineRestartLR, LinearLR, PolynomialLR, WarmupCosineLR, WarmupLinearLR,
              InverseSqrtLR, CyclicLR, OneCycleLR, ReduceLROnPlateau, SequentialLR, ChainedLR, WarmupLR, LambdaLR]
