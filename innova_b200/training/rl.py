"""Preference-based alignment: reward model, PPO, DPO and the RLHF loop.

Reference: ``PPOTrainer`` (clipped surrogate, value head of two linear layers on the hidden state, entropy bonus,
GAE, adaptive KL coefficient towards ``kl_target``), ``DPOTrainer`` (-log sigmoid(beta * (policy margin -
reference margin))), ``RLHFPipeline`` (generate comparisons -> train reward model -> PPO or DPO rounds) and
``RewardModel`` (pairwise Bradley-Terry loss); include/oil/trainer.h:313-437, include/oil/reward.h:10-57,
src/trainer_rl.cpp, src/trainer_rl_ops.cpp.

Models are ``DenseModel``-like: ``model(ids) -> logits [B, S, V]`` and ``model.hidden_states(ids) -> [B, S, D]``.
Everything is plain tensor code on the model's device, so on a GPU the forward/backward passes run the same fused
kernels as pre-training.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


def sequence_log_probs(logits: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """log p(ids[t] | prefix) from logits aligned with ids: [B, S, V], [B, S] -> [B, S]."""
    return torch.gather(F.log_softmax(logits.float(), -1), -1, ids.long().unsqueeze(-1)).squeeze(-1)


def compute_gae(rewards: torch.Tensor, values: torch.Tensor, dones: Optional[torch.Tensor] = None, gamma: float = 0.99, lam: float = 0.95):
    """Generalised advantage estimation over the last dimension. values has one more entry than rewards or the
    same length (bootstrap 0). Returns (advantages, returns)."""
    T = rewards.shape[-1]
    if values.shape[-1] == T:
        values = torch.cat([values, torch.zeros_like(values[..., :1])], -1)
    dones = torch.zeros_like(rewards) if dones is None else dones.to(rewards.dtype)
    adv = torch.zeros_like(rewards)
    last = torch.zeros_like(rewards[..., 0])
    for t in reversed(range(T)):
        nonterm = 1.0 - dones[..., t]
        delta = rewards[..., t] + gamma * values[..., t + 1] * nonterm - values[..., t]
        last = delta + gamma * lam * nonterm * last
        adv[..., t] = last
    return adv, adv + values[..., :T]


def discounted_returns(rewards: torch.Tensor, gamma: float = 0.99) -> torch.Tensor:
    out = torch.zeros_like(rewards)
    run = torch.zeros_like(rewards[..., 0])
    for t in reversed(range(rewards.shape[-1])):
        run = rewards[..., t] + gamma * run
        out[..., t] = run
    return out


def kl_divergence(logits_a: torch.Tensor, logits_b: torch.Tensor) -> torch.Tensor:
    """mean over positions of KL(softmax(a) || softmax(b))."""
    la, lb = F.log_softmax(logits_a.float(), -1), F.log_softmax(logits_b.float(), -1)
    return (la.exp() * (la - lb)).sum(-1).mean()


# ---------------------------------------------------------------------------------------------- reward model
class RewardModel(nn.Module):
    """Scalar reward from the last position's hidden state of a backbone."""

    def __init__(self, backbone, hidden_size: Optional[int] = None):
        super().__init__()
        self.backbone = backbone
        D = hidden_size or backbone.cfg.hidden_size
        self.head = nn.Linear(D, 1)
        nn.init.zeros_(self.head.bias)
        p = next(backbone.parameters())
        self.head.to(p.device)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        h = self.backbone.hidden_states(ids)[:, -1].float()
        return self.head(h).squeeze(-1)

    def pairwise_loss(self, chosen: torch.Tensor, rejected: torch.Tensor) -> Tuple[torch.Tensor, float]:
        rc, rr = self(chosen), self(rejected)
        return -F.logsigmoid(rc - rr).mean(), float((rc > rr).float().mean())


# ---------------------------------------------------------------------------------------------- PPO
class PPOTrainer:
    def __init__(self, policy, ref_model=None, clip_epsilon: float = 0.2, value_coef: float = 0.5, entropy_coef: float = 0.01,
                 gamma: float = 0.99, gae_lambda: float = 0.95, kl_target: float = 0.02, lr: float = 1e-5, critic_hidden: int = 256):
        self.policy = policy
        self.ref = ref_model if ref_model is not None else copy.deepcopy(policy).eval()
        for p in self.ref.parameters():
            p.requires_grad_(False)
        self.clip, self.vc, self.ec, self.gamma, self.lam, self.kl_target = clip_epsilon, value_coef, entropy_coef, gamma, gae_lambda, kl_target
        self.kl_alpha, self.last_kl = 0.1, 0.0
        D = policy.cfg.hidden_size
        dev = next(policy.parameters()).device
        self.critic = nn.Sequential(nn.Linear(D, critic_hidden), nn.Tanh(), nn.Linear(critic_hidden, 1)).to(dev)
        self.opt = torch.optim.AdamW(list(p for p in policy.parameters() if p.requires_grad) + list(self.critic.parameters()), lr=lr,
                                     weight_decay=0.0)
        self.log_cb: Optional[Callable[[float, float, float, float], None]] = None

    def critic_parameters(self):
        return list(self.critic.parameters())

    def values(self, ids: torch.Tensor) -> torch.Tensor:
        return self.critic(self.policy.hidden_states(ids).float()).squeeze(-1)

    def compute_gae(self, rewards, values, dones=None):
        return compute_gae(rewards, values, dones, self.gamma, self.lam)

    def train_step(self, states: torch.Tensor, actions: torch.Tensor, old_logprobs: torch.Tensor, advantages: torch.Tensor,
                   returns: torch.Tensor) -> dict:
        """states [B, S] token prefixes; actions [B, S] the token chosen after each prefix position."""
        logits = self.policy(states).float()
        logp = sequence_log_probs(logits, actions)
        ratio = torch.exp(logp - old_logprobs)
        adv = (advantages - advantages.mean()) / (advantages.std() + 1e-8)
        pl = -torch.min(ratio * adv, torch.clamp(ratio, 1 - self.clip, 1 + self.clip) * adv).mean()
        v = self.critic(self.policy.hidden_states(states).float()).squeeze(-1)
        vl = F.mse_loss(v, returns)
        probs = F.softmax(logits, -1)
        ent = -(probs * F.log_softmax(logits, -1)).sum(-1).mean()
        with torch.no_grad():
            ref_logits = self.ref(states).float()
        kl = kl_divergence(logits, ref_logits)
        loss = pl + self.vc * vl - self.ec * ent + self.kl_alpha * kl
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_([p for g in self.opt.param_groups for p in g["params"]], 1.0)
        self.opt.step()
        self.last_kl = float(kl.detach())
        # adaptive KL penalty: grow when the policy drifts past 1.5x the target, shrink under half of it
        if self.last_kl > 1.5 * self.kl_target:
            self.kl_alpha *= 1.5
        elif self.last_kl < 0.5 * self.kl_target:
            self.kl_alpha /= 1.5
        out = {"policy_loss": float(pl.detach()), "value_loss": float(vl.detach()), "entropy": float(ent.detach()), "kl": self.last_kl}
        if self.log_cb:
            self.log_cb(out["policy_loss"], out["value_loss"], out["entropy"], out["kl"])
        return out


# ---------------------------------------------------------------------------------------------- DPO
class DPOTrainer:
    def __init__(self, policy, ref_model=None, beta: float = 0.1, lr: float = 1e-6, optimizer=None):
        self.policy = policy
        self.ref = ref_model if ref_model is not None else copy.deepcopy(policy).eval()
        for p in self.ref.parameters():
            p.requires_grad_(False)
        self.beta, self.last_loss = beta, 0.0
        self.opt = optimizer or torch.optim.AdamW([p for p in policy.parameters() if p.requires_grad], lr=lr, weight_decay=0.0)
        self.log_cb: Optional[Callable[[float, float], None]] = None

    @staticmethod
    def _seq_logp(model, ids, prompt_len: int = 0):
        logits = model(ids[:, :-1])
        lp = sequence_log_probs(logits, ids[:, 1:])
        return lp[:, max(0, prompt_len - 1):].sum(-1)

    def loss(self, chosen: torch.Tensor, rejected: torch.Tensor, prompt_len: int = 0):
        pc, pr = self._seq_logp(self.policy, chosen, prompt_len), self._seq_logp(self.policy, rejected, prompt_len)
        with torch.no_grad():
            rc, rr = self._seq_logp(self.ref, chosen, prompt_len), self._seq_logp(self.ref, rejected, prompt_len)
        margin = (pc - pr) - (rc - rr)
        return -F.logsigmoid(self.beta * margin).mean(), margin.detach()

    def train_step(self, chosen: torch.Tensor, rejected: torch.Tensor, prompt_len: int = 0) -> float:
        loss, margin = self.loss(chosen, rejected, prompt_len)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_([p for g in self.opt.param_groups for p in g["params"]], 1.0)
        self.opt.step()
        self.last_loss = float(loss.detach())
        if self.log_cb:
            self.log_cb(self.last_loss, float(margin.mean()))
        return self.last_loss


# ---------------------------------------------------------------------------------------------- RLHF loop
@dataclass
class Comparison:
    prompt: List[int]
    chosen: List[int]
    rejected: List[int]


@dataclass
class RLHFMetrics:
    reward_accuracy: float = 0.0
    reward_loss: float = 0.0
    mean_reward: float = 0.0
    kl: float = 0.0
    dpo_loss: float = 0.0
    rounds: int = 0
    history: List[dict] = field(default_factory=list)


class RLHFPipeline:
    """generate two continuations per prompt -> rank them (``preference_fn`` or the reward model) -> fit the reward
    model on the pairs -> improve the policy with PPO (reward from the model, KL to the reference) or DPO."""

    def __init__(self, policy, reward_model: RewardModel, ref_model=None, preference_fn: Optional[Callable[[List[int], List[int]], bool]] = None,
                 max_seq: Optional[int] = None, seed: int = 0):
        self.policy, self.rm = policy, reward_model
        self.ref = ref_model if ref_model is not None else copy.deepcopy(policy).eval()
        self.preference_fn = preference_fn
        self.buffer: List[Comparison] = []
        self.metrics = RLHFMetrics()
        self.gen = torch.Generator().manual_seed(seed)
        self.max_seq = max_seq or policy.cfg.max_seq_len
        self.rm_opt = torch.optim.AdamW(self.rm.parameters(), lr=1e-4, weight_decay=0.0)
        self.ppo = PPOTrainer(policy, self.ref)
        self.dpo = DPOTrainer(policy, self.ref)
        self.device = next(policy.parameters()).device

    @torch.no_grad()
    def sample(self, prompt: Sequence[int], max_new_tokens: int, temperature: float = 1.0) -> List[int]:
        ids = list(prompt)
        for _ in range(max_new_tokens):
            x = torch.tensor([ids[-self.max_seq:]], device=self.device)
            logits = self.policy(x)[0, -1].float() / max(temperature, 1e-5)
            p = torch.softmax(logits, -1).cpu()
            ids.append(int(torch.multinomial(p, 1, generator=self.gen)))
        return ids

    def generate_comparisons(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16):
        for pr in prompts:
            a, b = self.sample(pr, max_new_tokens), self.sample(pr, max_new_tokens)
            if self.preference_fn is not None:
                a_better = self.preference_fn(a, b)
            else:
                with torch.no_grad():
                    a_better = float(self.rm(torch.tensor([a], device=self.device))) >= float(self.rm(torch.tensor([b], device=self.device)))
            ch, rj = (a, b) if a_better else (b, a)
            self.buffer.append(Comparison(list(pr), ch, rj))

    def train_reward_model(self, data: Optional[List[Comparison]] = None, epochs: int = 3, batch_size: int = 8) -> float:
        data = data if data is not None else self.buffer
        acc = 0.0
        for _ in range(epochs):
            accs = []
            for i in range(0, len(data), batch_size):
                chunk = data[i:i + batch_size]
                ch = torch.tensor([c.chosen for c in chunk], device=self.device)
                rj = torch.tensor([c.rejected for c in chunk], device=self.device)
                loss, a = self.rm.pairwise_loss(ch, rj)
                self.rm_opt.zero_grad(set_to_none=True)
                loss.backward()
                self.rm_opt.step()
                accs.append(a)
                self.metrics.reward_loss = float(loss.detach())
            acc = sum(accs) / max(1, len(accs))
        self.metrics.reward_accuracy = acc
        return acc

    def compute_reward_accuracy(self, data: List[Comparison]) -> float:
        with torch.no_grad():
            ch = torch.tensor([c.chosen for c in data], device=self.device)
            rj = torch.tensor([c.rejected for c in data], device=self.device)
            return float((self.rm(ch) > self.rm(rj)).float().mean())

    def ppo_finetune(self, prompts: Sequence[Sequence[int]], n_steps: int = 4, max_new_tokens: int = 16):
        for _ in range(n_steps):
            seqs = [self.sample(p, max_new_tokens) for p in prompts]
            ids = torch.tensor(seqs, device=self.device)
            states, actions = ids[:, :-1], ids[:, 1:]
            with torch.no_grad():
                old_lp = sequence_log_probs(self.policy(states).float(), actions)
                reward_final = self.rm(ids).float()
                values = self.ppo.values(states)
            rewards = torch.zeros_like(old_lp)
            rewards[:, -1] = reward_final
            adv, ret = compute_gae(rewards, values, None, self.ppo.gamma, self.ppo.lam)
            out = self.ppo.train_step(states, actions, old_lp, adv, ret)
            self.metrics.mean_reward, self.metrics.kl = float(reward_final.mean()), out["kl"]
            self.metrics.history.append({"reward": self.metrics.mean_reward, **out})

    def dpo_finetune(self, comparisons: Optional[List[Comparison]] = None, n_steps: int = 10, batch_size: int = 4):
        data = comparisons if comparisons is not None else self.buffer
        for s in range(n_steps):
            chunk = [data[(s * batch_size + j) % len(data)] for j in range(batch_size)]
            ch = torch.tensor([c.chosen for c in chunk], device=self.device)
            rj = torch.tensor([c.rejected for c in chunk], device=self.device)
            self.metrics.dpo_loss = self.dpo.train_step(ch, rj, prompt_len=len(chunk[0].prompt))

    def run(self, prompts: Sequence[Sequence[int]], n_rounds: int = 1, n_ppo_steps: int = 2, max_new_tokens: int = 8, use_dpo: bool = False):
        for _ in range(n_rounds):
            self.generate_comparisons(prompts, max_new_tokens)
            self.train_reward_model(epochs=1)
            if use_dpo:
                self.dpo_finetune(n_steps=n_ppo_steps)
            else:
                self.ppo_finetune(prompts, n_ppo_steps, max_new_tokens)
            self.metrics.rounds += 1
        return self.metrics
