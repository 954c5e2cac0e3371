"""The reference's class and record names, importable from one place.

Most capabilities live in this package under the name that fits their design here (``EMA`` rather than ``ModelEMA``,
``DDPFlatEngine`` rather than ``DistributedDataParallel``, PyTorch's optimisers rather than hand-rolled ones). Code written
against the reference's headers (``include/oil/*.h``) can keep its names: ``from innova_b200.reference_names import Adam,
ModelEMA, SamplerConfig``. Two kinds of entry:

* aliases, resolved on first use so that importing this module pulls in nothing heavy: ``ALIASES`` maps the reference's
  name to ``"module:attribute"``;
* the small plain records of the reference's headers that carry options or results (``SamplerConfig``, ``StreamingConfig``,
  ``StreamConfig``, ``GenerationResult``, ``NASConfig``, ``SuccessiveHalvingConfig``, ``ZeROConfig``, ``AugmentConfig``,
  ``CurriculumState``, ``BenchmarkResult``, ``LatencyHistogram``, ``Theorem12Result``), defined here with the reference's
  field names and defaults and a method that hands them to the object that consumes them.
"""
from __future__ import annotations

import bisect
import importlib
import threading
from dataclasses import dataclass, field
from typing import Any, Dict, List

_P = "innova_b200."
ALIASES: Dict[str, str] = {
    # optimisers (include/oil/optimizer.h)
    "Optimizer": "torch.optim:Optimizer", "SGD": "torch.optim:SGD", "Adam": "torch.optim:Adam", "AdamW": "torch.optim:AdamW",
    "Adamax": "torch.optim:Adamax", "NAdam": "torch.optim:NAdam", "RAdam": "torch.optim:RAdam", "RMSProp": "torch.optim:RMSprop",
    "Adafactor": "torch.optim:Adafactor", "Adabound": _P + "training.optimizers:AdaBound",
    # autograd nodes (include/oil/autograd.h, autograd_functions.h)
    "AutogradFunction": "torch.autograd:Function", "MatMulFunction": _P + "ops.gemm:_LinearFn", "BiasAddFunction": _P + "ops.gemm:_LinearFn",
    "SiLUFunction": _P + "ops.functional:_ActFn", "GatedMulFunction": _P + "ops.functional:_ActFn", "RMSNormFunction": _P + "ops.functional:_NormFn",
    "CrossEntropyFunction": _P + "ops.functional:_CrossEntropyFn", "RotaryFunction": _P + "ops.functional:_RopeFn",
    "EmbeddingFunction": _P + "ops.functional:_EmbeddingFn", "ScaledDotProductAttentionFunction": _P + "ops.attention:_FlashAttnFn",
    "FlattenAttentionFunction": _P + "ops.attention:_FlashAttnFn",
    # model pieces (include/oil/transformer.h, tokenizer.h, moe_variants.h)
    "Tensor": "torch:Tensor", "Shape": "torch:Size", "Linear": "torch.nn:Linear", "Embedding": "torch.nn:Embedding", "Model": _P + "models.dense:DenseModel",
    "Tokenizer": _P + "utils.tokenizer:BPETokenizer", "ExpertFFN": _P + "models.moe_variants:ExpertBank",
    "ExpertParallel": _P + "parallel.expert_parallel:ExpertParallelMoE", "UNetBlock": _P + "models.generative:DiffusionUNet",
    "CrossAttentionLayerConfig": _P + "models.multimodal:FusionConfig", "MultimodalEncoderConfig": _P + "models.multimodal:FusionConfig",
    # training (include/oil/trainer.h, training_utils.h, ddp.h, fsdp.h, native_moe_trainer.h, continual_engine.h)
    "ModelEMA": _P + "training.utils:EMA", "EMAWeightAveraging": _P + "training.utils:EMA", "DistributedDataParallel": _P + "parallel.ddp:DDPFlatEngine",
    "NativeMoEConfig": _P + "training.moe_trainer:MoETrainConfig", "NativeMoEMetrics": _P + "training.moe_trainer:MoEMetrics",
    "ForgettingTask": _P + "training.continual:ForgettingBenchmark", "CompressedReplayEntry": _P + "training.continual:_ReplayEntry",
    "DatasetSplit": _P + "utils.datasets:split_dataset", "MemoryProfile": _P + "utils.telemetry_ext:MemoryTracker",
    # inference and serving (include/oil/sampler.h, kv_cache.h, production.h)
    "PagedKVCacheBase": _P + "inference.kv_cache:PagedKVCache", "ModelHTTPServer": _P + "serving.http_server:HTTPServer",
    "Plugin": _P + "serving.production:PluginManager", "ModelInfo": _P + "serving.production:ModelZoo", "Tool": _P + "utils.asi:ToolUse",
    # formats and backends (include/oil/format_registry.h, codebook.h, int8_quant.h, backend.h, gpu_compute_full.h)
    "MixDescriptor": _P + "formats.registry:MixInfo", "OIL4Codebook": _P + "formats.codebook:CodebookOIL4", "OIL8Codebook": _P + "formats.codebook:CodebookOIL8",
    "Int8QuantParams": _P + "ops.engines:QuantizeParams", "HardwareProfile": _P + "utils.backend:HardwareInfo", "KernelProfile": _P + "utils.telemetry:KernelPerf",
    "GPUFallback": _P + "utils.backend:MultiGPUManager", "Stage": _P + "parallel.expert_parallel:PipelineStage",
}


def resolve(name: str) -> Any:
    """The object that stands for the reference's ``name`` (an alias target or a record defined in this module)."""
    if name in ALIASES:
        mod, attr = ALIASES[name].split(":")
        return getattr(importlib.import_module(mod), attr)
    if name in globals() and not name.startswith("_"):
        return globals()[name]
    raise AttributeError(f"no reference name {name!r}")


def __getattr__(name: str) -> Any:
    if name in ALIASES:
        obj = resolve(name)
        globals()[name] = obj
        return obj
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return sorted(set(globals()) | set(ALIASES))


# ------------------------------------------------------------------------------------------------ option and result records
@dataclass
class SamplerConfig:
    """include/oil/sampler.h:9-15."""
    temperature: float = 1.0
    top_k: int = 40
    top_p: float = 0.9
    repetition_penalty: float = 1.0
    max_tokens: int = 2048

    def to_params(self, seed: int = 42):
        from .inference.sampler import SamplingParams
        return SamplingParams(self.temperature, self.top_k, self.top_p, self.repetition_penalty, seed)


@dataclass
class StreamingConfig:
    """include/oil/generator.h:62-73."""
    max_tokens: int = 512
    eos_id: int = 2
    temperature: float = 1.0
    top_k: int = 40
    top_p: float = 0.9
    repetition_penalty: float = 1.0
    stop_token_ids: List[int] = field(default_factory=list)
    stop_strings: List[str] = field(default_factory=list)
    stream_logprobs: bool = False
    logprobs_k: int = 5

    def to_params(self, seed: int = 42):
        return SamplerConfig(self.temperature, self.top_k, self.top_p, self.repetition_penalty, self.max_tokens).to_params(seed)

    def should_stop(self, token: int, text: str = "") -> bool:
        return token == self.eos_id or token in self.stop_token_ids or any(s and text.endswith(s) for s in self.stop_strings)


@dataclass
class StreamConfig:
    """include/oil/inference_opt.h:206-212."""
    stream: bool = False
    max_tokens: int = 512
    eos_id: int = -1
    stop_on_newline: bool = False
    stop_sequences: List[str] = field(default_factory=list)

    def should_stop(self, token: int, text: str = "") -> bool:
        return (self.eos_id >= 0 and token == self.eos_id) or (self.stop_on_newline and text.endswith("\n")) or \
            any(s and text.endswith(s) for s in self.stop_sequences)


@dataclass
class GenerationResult:
    """include/oil/generator.h:17-23."""
    token_ids: List[int] = field(default_factory=list)
    text: str = ""
    duration_sec: float = 0.0
    tokens_per_sec: int = 0
    truncated: bool = False

    @classmethod
    def from_run(cls, token_ids, text: str, duration_sec: float, max_tokens: int = 0) -> "GenerationResult":
        ids = [int(t) for t in token_ids]
        return cls(ids, text, duration_sec, int(len(ids) / duration_sec) if duration_sec > 0 else 0, bool(max_tokens) and len(ids) >= max_tokens)


@dataclass
class NASConfig:
    """include/oil/hpo_nas.h:174-182."""
    population: int = 50
    generations: int = 20
    tournament_size: int = 3
    mutation_rate: float = 0.3
    crossover_rate: float = 0.7
    hardware_aware: bool = False
    oil_native: bool = True

    def run(self, engine):
        """Evolutionary search of ``engine`` (a ``training.utils.NASEngine``) under these settings."""
        return engine.evolve(population=self.population, generations=self.generations, tournament_size=self.tournament_size,
                             mutation_rate=self.mutation_rate, crossover_rate=self.crossover_rate, hardware_aware=self.hardware_aware)


@dataclass
class SuccessiveHalvingConfig:
    """include/oil/hpo_nas.h:103-109. ``plan`` fills the per-rung schedule."""
    n_configs: int = 0
    n_rungs: int = 0
    reduction_factor: float = 3.0
    configs_per_rung: List[int] = field(default_factory=list)
    budget_per_rung: List[float] = field(default_factory=list)

    def plan(self, min_budget: float = 1.0) -> "SuccessiveHalvingConfig":
        n, b = self.n_configs, min_budget
        self.configs_per_rung, self.budget_per_rung = [], []
        for _ in range(self.n_rungs):
            self.configs_per_rung.append(max(1, int(n)))
            self.budget_per_rung.append(b)
            n, b = n / self.reduction_factor, b * self.reduction_factor
        return self

    def run(self, hpo):
        return hpo.successive_halving(self.n_configs, self.n_rungs, int(round(self.reduction_factor)))


@dataclass
class ZeROConfig:
    """include/oil/zero_offload.h:63-70."""
    enabled: bool = False
    offload_threshold_bytes: int = 0
    shard_gradients: bool = False
    shard_optimizer_states: bool = True
    pin_cpu_memory: bool = True
    cpu_buffer_size: int = 1 << 30

    @property
    def stage(self) -> int:
        return 0 if not self.enabled else (2 if self.shard_gradients else (1 if self.shard_optimizer_states else 0))

    def make_manager(self, engine):
        from .parallel.zero import ZeROOffloadManager
        return ZeROOffloadManager(engine, pool_bytes=self.cpu_buffer_size)


@dataclass
class AugmentConfig:
    """include/oil/trainer.h:58-63."""
    enabled: bool = False
    mask_prob: float = 0.0
    noise_std: float = 0.01
    replace_prob: float = 0.0


@dataclass
class CurriculumState:
    """include/oil/trainer.h:88-97: the sequence length grows linearly from 64 to 512 over the epochs."""
    current_epoch: int = 0
    total_epochs: int = 3
    seq_len_multiplier: float = 0.5

    def effective_seq_length(self) -> int:
        t = self.current_epoch / max(self.total_epochs, 1)
        return max(64, int(512 * (64 / 512.0 + t * (1.0 - 64 / 512.0))))


@dataclass
class BenchmarkResult:
    """include/oil/hpo_nas.h:95-101."""
    accuracy: float = 0.0
    loss: float = 1e10
    time_ms: float = 0.0
    param_count: int = 0
    memory_bytes: int = 0


class LatencyHistogram:
    """include/oil/production.h:32-40. Samples are kept sorted on insert, so a percentile is one index."""

    def __init__(self):
        self.samples: List[float] = []
        self._mtx = threading.Lock()

    def record(self, ms: float):
        with self._mtx:
            bisect.insort(self.samples, float(ms))

    def percentile(self, p: float) -> float:
        with self._mtx:
            if not self.samples:
                return 0.0
            i = min(len(self.samples) - 1, max(0, int(p / 100.0 * len(self.samples))))
            return self.samples[i]

    def p50(self) -> float:
        return self.percentile(50.0)

    def p95(self) -> float:
        return self.percentile(95.0)

    def p99(self) -> float:
        return self.percentile(99.0)


@dataclass
class Theorem12Result:
    """include/oil/continual_engine.h:185-202: the safety claims of the single-producer single-consumer queue.
    ``verify`` here runs the queue (``utils.core.SPSCQueue``) with one producer and one consumer thread and checks
    that every item arrives once and in order, instead of returning constants."""
    correctness_guaranteed: bool = False
    aba_free: bool = False
    no_data_race: bool = False
    proof_reference: str = ("single writer per index and release/acquire publication of head and tail; one producer and one consumer "
                            "rule out ABA; head and tail sit on separate cache lines")

    @classmethod
    def verify(cls, items: int = 20000, capacity: int = 64) -> "Theorem12Result":
        from .utils.core import SPSCQueue
        q = SPSCQueue(capacity)
        got: List[int] = []

        def produce():
            i = 0
            while i < items:
                if q.push(i):
                    i += 1

        def consume():
            while len(got) < items:
                ok, v = q.pop()
                if ok:
                    got.append(v)

        ts = [threading.Thread(target=produce), threading.Thread(target=consume)]
        for t in ts:
            t.start()
        for t in ts:
            t.join(timeout=60)
        alive = any(t.is_alive() for t in ts)
        in_order = got == list(range(items))
        return cls(in_order and not alive, len(set(got)) == len(got), in_order)
