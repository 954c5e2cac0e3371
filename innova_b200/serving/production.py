"""Production plumbing: logger, JSON application config, model zoo, plugin manager and a batching model server.

Reference: ``Logger``, ``AppConfig`` (JSON), ``PluginManager`` (dlopen + hot reload), ``ModelZoo`` and
``ModelServer`` (priority-queue batching, latency percentiles); include/oil/production.h:20-363. Plugins here are
Python modules or native libraries (``ctypes``) that export ``plugin_init``; hot reload compares modification times.
"""
from __future__ import annotations

import ctypes
import importlib.util
import json
import os
import sys
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional


class Logger:
    LEVELS = {"debug": 10, "info": 20, "warn": 30, "error": 40}

    def __init__(self, path: Optional[str] = None, level: str = "info", json_lines: bool = False):
        self.level, self.json_lines = self.LEVELS[level], json_lines
        self.f = open(path, "a") if path else sys.stderr
        self._lock = threading.Lock()

    def log(self, level: str, msg: str, **fields):
        if self.LEVELS[level] < self.level:
            return
        with self._lock:
            if self.json_lines:
                self.f.write(json.dumps({"ts": time.time(), "level": level, "msg": msg, **fields}) + "\n")
            else:
                extra = " ".join(f"{k}={v}" for k, v in fields.items())
                self.f.write(f"{time.strftime('%Y-%m-%dT%H:%M:%S')} [{level.upper():5s}] {msg} {extra}".rstrip() + "\n")
            self.f.flush()

    def debug(self, m, **k): self.log("debug", m, **k)
    def info(self, m, **k): self.log("info", m, **k)
    def warn(self, m, **k): self.log("warn", m, **k)
    def error(self, m, **k): self.log("error", m, **k)


class AppConfig:
    """Nested JSON configuration with dotted-path access and environment overrides (``INNOVA_A_B=...`` sets ``a.b``)."""

    def __init__(self, data: Optional[dict] = None):
        self.data = data or {}

    @classmethod
    def load(cls, path: str) -> "AppConfig":
        cfg = cls(json.load(open(path)))
        cfg.apply_env()
        return cfg

    def save(self, path: str):
        json.dump(self.data, open(path, "w"), indent=2)

    def get(self, key: str, default: Any = None) -> Any:
        cur = self.data
        for part in key.split("."):
            if not isinstance(cur, dict) or part not in cur:
                return default
            cur = cur[part]
        return cur

    def set(self, key: str, value: Any):
        cur = self.data
        parts = key.split(".")
        for part in parts[:-1]:
            cur = cur.setdefault(part, {})
        cur[parts[-1]] = value

    def apply_env(self, prefix: str = "INNOVA_"):
        for k, v in os.environ.items():
            if k.startswith(prefix):
                try:
                    val = json.loads(v)
                except ValueError:
                    val = v
                self.set(k[len(prefix):].lower().replace("_", "."), val)


class ModelZoo:
    """Name -> (path, metadata) registry persisted as JSON."""

    def __init__(self, index_path: Optional[str] = None):
        self.index_path = index_path
        self.models: Dict[str, dict] = {}
        if index_path and os.path.exists(index_path):
            self.models = json.load(open(index_path))

    def register(self, name: str, path: str, **meta):
        self.models[name] = {"path": path, **meta}
        if self.index_path:
            json.dump(self.models, open(self.index_path, "w"), indent=2)

    def resolve(self, name: str) -> str:
        return self.models[name]["path"]

    def list(self) -> List[str]:
        return sorted(self.models)


class PluginManager:
    def __init__(self):
        self.plugins: Dict[str, dict] = {}

    def load(self, path: str, name: Optional[str] = None):
        name = name or os.path.splitext(os.path.basename(path))[0]
        if path.endswith(".py"):
            spec = importlib.util.spec_from_file_location(f"innova_plugin_{name}", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            handle = mod
            init = getattr(mod, "plugin_init", None)
        else:
            handle = ctypes.CDLL(path)
            init = getattr(handle, "plugin_init", None)
        result = init() if init else None
        self.plugins[name] = {"path": path, "handle": handle, "mtime": os.path.getmtime(path), "init_result": result}
        return handle

    def reload_changed(self) -> List[str]:
        changed = [n for n, p in self.plugins.items() if os.path.getmtime(p["path"]) != p["mtime"]]
        for n in changed:
            self.load(self.plugins[n]["path"], n)
        return changed

    def get(self, name: str):
        return self.plugins[name]["handle"]


@dataclass(order=True)
class _Job:
    key: tuple
    prompt: Any = field(compare=False)
    max_tokens: int = field(compare=False, default=64)
    event: threading.Event = field(compare=False, default_factory=threading.Event)
    result: Any = field(compare=False, default=None)
    submitted: float = field(compare=False, default=0.0)


class ModelServer:
    """Worker thread that drains a priority queue in batches of up to ``max_batch`` and records request latency."""

    def __init__(self, generate_batch: Callable[[List[Any], int], List[Any]], max_batch: int = 8, max_wait_s: float = 0.002):
        import heapq
        self._heapq = heapq
        self.generate_batch, self.max_batch, self.max_wait_s = generate_batch, max_batch, max_wait_s
        self._q: List[_Job] = []
        self._cv = threading.Condition()
        self._stop = False
        self._seq = 0
        self.latencies: List[float] = []
        self.batches = 0
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def submit(self, prompt, max_tokens: int = 64, priority: int = 0) -> _Job:
        with self._cv:
            self._seq += 1
            job = _Job((-priority, self._seq), prompt, max_tokens, submitted=time.time())
            self._heapq.heappush(self._q, job)
            self._cv.notify()
        return job

    def generate(self, prompt, max_tokens: int = 64, priority: int = 0, timeout: Optional[float] = None):
        job = self.submit(prompt, max_tokens, priority)
        if not job.event.wait(timeout):
            raise TimeoutError("model server did not answer in time")
        return job.result

    def _loop(self):
        while True:
            with self._cv:
                while not self._q and not self._stop:
                    self._cv.wait(0.05)
                if self._stop and not self._q:
                    return
                if len(self._q) < self.max_batch:
                    self._cv.wait(self.max_wait_s)
                jobs = [self._heapq.heappop(self._q) for _ in range(min(self.max_batch, len(self._q)))]
            if not jobs:
                continue
            try:
                outs = self.generate_batch([j.prompt for j in jobs], max(j.max_tokens for j in jobs))
            except Exception as e:
                outs = [e] * len(jobs)
                self._errors = getattr(self, "_errors", 0) + len(jobs)
            now = time.time()
            self.batches += 1
            for j, o in zip(jobs, outs):
                j.result = o
                self.latencies.append(now - j.submitted)
                j.event.set()

    def latency_percentiles(self) -> Dict[str, float]:
        if not self.latencies:
            return {"p50": 0.0, "p95": 0.0, "p99": 0.0}
        s = sorted(self.latencies)
        pick = lambda q: s[min(len(s) - 1, int(q * len(s)))]
        return {"p50": pick(0.50), "p95": pick(0.95), "p99": pick(0.99)}

    def stop(self):
        with self._cv:
            self._stop = True
            self._cv.notify_all()
        self._thread.join(timeout=2)

    # -- the rest of the reference's server surface (include/oil/production.h:20-142)
    def is_running(self) -> bool:
        return self._thread.is_alive() and not self._stop

    def set_batch_size(self, bs: int) -> None:
        self.max_batch = max(1, int(bs))

    def set_queue_wait_ms(self, ms: float) -> None:
        self.max_wait_s = max(0.0, ms / 1e3)

    def submit_with_callback(self, prompt, max_tokens: int = 64, priority: int = 0,
                             callback: Optional[Callable[[Any, Any], None]] = None) -> int:
        """Queues a request and returns its id; ``callback(prompt, result)`` runs on a watcher thread once the batch that
        carried it has finished (the worker thread itself never runs user code)."""
        job = self.submit(prompt, max_tokens, priority)
        if callback is not None:
            def watch():
                job.event.wait()
                callback(prompt, job.result)
            threading.Thread(target=watch, daemon=True).start()
        return job.key[1]

    def metrics(self) -> Dict[str, float]:
        lat = self.latencies
        pct = self.latency_percentiles()
        errors = getattr(self, "_errors", 0)
        return {"total_requests": len(lat), "total_errors": errors, "batches": self.batches, "queued": len(self._q),
                "avg_latency_ms": 1e3 * sum(lat) / len(lat) if lat else 0.0, "p50_ms": 1e3 * pct["p50"], "p95_ms": 1e3 * pct["p95"],
                "p99_ms": 1e3 * pct["p99"], "avg_batch": len(lat) / self.batches if self.batches else 0.0}

    def health_json(self) -> str:
        return json.dumps({"status": "ok" if self.is_running() else "stopped", "model_loaded": self.generate_batch is not None,
                           "queued": len(self._q), "max_batch": self.max_batch})

    def metrics_json(self) -> str:
        return json.dumps(self.metrics())

    def load_model(self, loader: Callable[[], Callable[[List[Any], int], List[Any]]]) -> bool:
        """Swaps the batch function for the one ``loader`` returns; queued requests are served by the new one. False (and the
        old model kept) when the loader raises."""
        try:
            fn = loader()
        except Exception:   # noqa: BLE001 - a failed load must not take the server down
            return False
        with self._cv:
            self.generate_batch = fn
        return True

    def unload_model(self) -> None:
        def unloaded(prompts, max_tokens):
            raise RuntimeError("no model loaded")
        with self._cv:
            self.generate_batch = unloaded

    def is_model_loaded(self) -> bool:
        return getattr(self.generate_batch, "__name__", "") != "unloaded"


@dataclass
class BatchConsolidationResult:
    request_ids: List[int]
    batched_input: Any          # [B, max_len] token ids, right-padded
    batched_positions: Any      # [B, max_len] positions (0 where padded)
    seq_lens: List[int]
    offsets: List[int]          # start of each request in the concatenation of the unpadded sequences


def consolidate_batch(requests: List[tuple], pad_id: int = 0) -> BatchConsolidationResult:
    """``requests`` is [(request id, token ids)]: one right-padded id matrix with positions, the true lengths, and the offsets
    the sequences would have if packed back to back (reference: ``ModelServer::consolidate_batch``,
    include/oil/production.h:58-64,128)."""
    import torch
    lens = [len(ids) for _, ids in requests]
    width = max(lens, default=0)
    inp = torch.full((len(requests), width), pad_id, dtype=torch.long)
    pos = torch.zeros(len(requests), width, dtype=torch.long)
    offsets, run = [], 0
    for r, (_, ids) in enumerate(requests):
        inp[r, : len(ids)] = torch.as_tensor(list(ids), dtype=torch.long)
        pos[r, : len(ids)] = torch.arange(len(ids))
        offsets.append(run)
        run += len(ids)
    return BatchConsolidationResult([rid for rid, _ in requests], inp, pos, lens, offsets)
