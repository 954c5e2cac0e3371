"""Pipeline parallelism: contiguous layer stages, micro-batched GPipe and 1F1B schedules.

Reference: ``PipelineParallel`` (ceil(L / stages) layers per stage, stage 0 owns the embedding, the last stage
the final norm and LM head; GPipe micro-batching with 4 micro-batches, ``forward_1f1b`` / ``backward_1f1b``,
gradient accumulation, per-stage profile; src/pipeline.cpp:47-383) and the older ``PipelineParallelWrapper``
(src/distributed.cpp:185-215). The reference moves activations by broadcasting a ``d_model * max_seq_len`` float
buffer; here neighbouring stages exchange exactly the micro-batch's activation / gradient tensor with
point-to-point sends (NCCL over NVLink on GPUs, gloo on CPU), posted asynchronously so that a stage computes one
micro-batch while the previous one's output is in flight.
"""
from __future__ import annotations

import time
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn


def stage_bounds(num_layers: int, stages: int, stage: int):
    per = -(-num_layers // stages)
    lo = min(num_layers, stage * per)
    return lo, min(num_layers, lo + per)


class DenseStage(nn.Module):
    """The slice of a ``DenseModel`` one pipeline stage owns (built from a full model; other parts are dropped)."""

    def __init__(self, model, stage: int, stages: int):
        super().__init__()
        self.cfg = model.cfg
        self.first, self.last = stage == 0, stage == stages - 1
        lo, hi = stage_bounds(len(model.layers), stages, stage)
        self.layers = nn.ModuleList(list(model.layers[lo:hi]))
        self.tok_embeddings = model.tok_embeddings if self.first else None
        self.pos_embeddings = model.pos_embeddings if self.first else None
        self.norm = model.norm if self.last else None
        self.lm_head = model.lm_head if self.last else None
        self._model_rope = model.rope

    def forward(self, x, labels=None):
        from .. import ops
        if self.first:
            x = ops.embedding(x, self.tok_embeddings.weight, None if self.pos_embeddings is None else self.pos_embeddings.weight)
        rope = self._model_rope(x.device)
        for blk in self.layers:
            x = blk(x, rope, None)
        if not self.last:
            return x
        from ..models.dense import _ste
        h = self.norm(x)
        w = _ste(self.lm_head.weight, self.cfg)
        if labels is None:
            return ops.linear(h, w)[..., : self.cfg.vocab_size]
        return ops.lm_head_cross_entropy(h, w, labels, vocab=self.cfg.vocab_size)


class PipelineParallel:
    def __init__(self, stage_module: nn.Module, group=None, num_micro_batches: int = 4, schedule: str = "1f1b", act_shape=None,
                 act_dtype=torch.bfloat16, device=None):
        """``act_shape`` is the per-micro-batch activation shape between stages (e.g. ``[mb, seq, hidden]``)."""
        self.module, self.group = stage_module, group
        self.stages = dist.get_world_size(group) if dist.is_initialized() else 1
        self.stage = dist.get_rank(group) if dist.is_initialized() else 0
        self.num_micro, self.schedule = num_micro_batches, schedule
        self.act_shape, self.act_dtype = act_shape, act_dtype
        self.device = device if device is not None else next(stage_module.parameters()).device
        self.first, self.last = self.stage == 0, self.stage == self.stages - 1
        self.profile = {"forward_ns": 0, "backward_ns": 0, "comm_wait_ns": 0}

    def _peer(self, delta):
        r = self.stage + delta
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    # ---------------------------------------------------------------- p2p
    def _recv(self, delta):
        t = torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)
        return t, dist.irecv(t, src=self._peer(delta), group=self.group)

    def _send(self, t, delta):
        return dist.isend(t.contiguous(), dst=self._peer(delta), group=self.group)

    def _wait(self, work):
        t0 = time.perf_counter_ns()
        work.wait()
        self.profile["comm_wait_ns"] += time.perf_counter_ns() - t0

    # ---------------------------------------------------------------- one micro-batch
    def _forward_micro(self, ids_mb, labels_mb, state):
        t0 = time.perf_counter_ns()
        if self.first:
            inp = ids_mb
        else:
            buf, w = self._recv(-1)
            self._wait(w)
            inp = buf.requires_grad_(True)
        out = self.module(inp, labels_mb) if self.last else self.module(inp)
        if not self.last:
            state["sends"].append(self._send(out.detach(), +1))
        state["fwd"].append((inp, out))
        self.profile["forward_ns"] += time.perf_counter_ns() - t0
        return out

    def _backward_micro(self, state, scale):
        t0 = time.perf_counter_ns()
        inp, out = state["fwd"].pop(0)
        if self.last:
            (out * scale).backward()
        else:
            g, w = self._recv(+1)
            self._wait(w)
            out.backward(g)
        if not self.first:
            state["sends"].append(self._send(inp.grad, -1))
        self.profile["backward_ns"] += time.perf_counter_ns() - t0

    # ---------------------------------------------------------------- schedules
    def train_step(self, ids: Optional[torch.Tensor], labels: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Runs all micro-batches forward and backward (gradients accumulate in the parameters / their
        ``main_grad``). ``ids`` is used on the first stage, ``labels`` on the last. Returns the mean loss on
        the last stage, None elsewhere."""
        M = self.num_micro
        ids_mb = ids.chunk(M, 0) if (self.first and ids is not None) else [None] * M
        lab_mb = labels.chunk(M, 0) if (self.last and labels is not None) else [None] * M
        state = {"fwd": [], "sends": []}
        losses = []
        scale = 1.0 / M
        if self.schedule == "gpipe" or self.stages == 1:
            for i in range(M):
                out = self._forward_micro(ids_mb[i], lab_mb[i], state)
                if self.last:
                    losses.append(out.detach())
            for i in range(M):
                self._backward_micro(state, scale)
        else:  # 1F1B: warm-up forwards, steady one-forward-one-backward, cool-down backwards
            warm = min(M, self.stages - self.stage - 1)
            f = b = 0
            for _ in range(warm):
                out = self._forward_micro(ids_mb[f], lab_mb[f], state)
                f += 1
            while f < M:
                out = self._forward_micro(ids_mb[f], lab_mb[f], state)
                if self.last:
                    losses.append(out.detach())
                f += 1
                self._backward_micro(state, scale)
                b += 1
            while b < M:
                self._backward_micro(state, scale)
                b += 1
        for w in state["sends"]:
            self._wait(w)
        return torch.stack(losses).mean() if self.last and losses else None

    @torch.no_grad()
    def forward_only(self, ids: Optional[torch.Tensor]):
        """Inference through the stages for one batch; logits on the last stage."""
        if self.first:
            x = ids
        else:
            x, w = self._recv(-1)
            self._wait(w)
        out = self.module(x)
        if not self.last:
            self._wait(self._send(out, +1))
            return None
        return out


class PipelineParallelWrapper(PipelineParallel):
    """The older reference API name; same behaviour with the GPipe schedule."""

    def __init__(self, stage_module, group=None, num_micro_batches: int = 4, **kw):
        super().__init__(stage_module, group, num_micro_batches, schedule="gpipe", **kw)
