"""Failure detection, expert re-assignment and elastic restart.

Reference: ``FaultToleranceManager`` (heartbeat thread, ``on_node_failure`` -> ``handle_node_failure`` ->
``redistribute_experts_after_failure``: the first alive node takes a failed node's experts; text checkpoint of
the node list; src/expert_parallel.cpp:792-825,1010-1178), ``ClusterConfig`` (heartbeat 1000 ms, fault timeout
5000 ms, 3 retries; include/oil/expert_parallel.h:73-75), ``CapacityAwareRouter`` and the redistribution plan.
The reference's health check always answers "healthy"; here a rank is healthy while its heartbeat key in the
rendezvous store keeps advancing.

Everything in this file runs on the host: heartbeats go through a ``torch.distributed`` key-value store, a failed
rank is one whose counter stopped for ``fault_timeout_s``, and recovery is "tear the process group down, restart
with the surviving ranks, reload the last sharded checkpoint at the new world size"
(``formats.checkpoint.load_sharded`` re-slices shards written by any world size). No GPU work is in flight when a
rank leaves: ranks check ``should_stop()`` between steps, before launching the next step's kernels.
"""
from __future__ import annotations

import json
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional


@dataclass
class ClusterConfig:
    heartbeat_interval_s: float = 1.0
    fault_timeout_s: float = 5.0
    max_retries: int = 3


class HeartbeatMonitor:
    """Every rank bumps ``hb/<rank>`` in the store from a daemon thread; ``failed_ranks`` lists ranks whose counter has
    not moved for ``fault_timeout_s``. ``store`` is any object with ``set(key, str)`` / ``get(key) -> bytes``
    (``torch.distributed.TCPStore``, ``FileStore``, ``HashStore``)."""

    def __init__(self, store, rank: int, world: int, cfg: Optional[ClusterConfig] = None, on_failure: Optional[Callable[[int], None]] = None):
        self.store, self.rank, self.world, self.cfg, self.on_failure = store, rank, world, cfg or ClusterConfig(), on_failure
        self._beat = 0
        self._last: Dict[int, tuple] = {}
        self._failed: List[int] = []
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._lock = threading.Lock()

    def beat(self):
        self._beat += 1
        self.store.set(f"hb/{self.rank}", str(self._beat))

    def _read(self, r: int) -> int:
        key = f"hb/{r}"
        try:
            # get() on a key nobody has set blocks until the store's timeout: ask first
            if hasattr(self.store, "check") and not self.store.check([key]):
                return -1
            return int(self.store.get(key))
        except Exception:
            return -1

    def poll(self, now: Optional[float] = None) -> List[int]:
        """One detection pass; returns the ranks newly declared failed."""
        now = time.monotonic() if now is None else now
        new = []
        for r in range(self.world):
            if r == self.rank or r in self._failed:
                continue
            v = self._read(r)
            last = self._last.get(r)
            if last is None or v != last[0]:
                self._last[r] = (v, now)
            elif now - last[1] >= self.cfg.fault_timeout_s:
                with self._lock:
                    self._failed.append(r)
                new.append(r)
                if self.on_failure:
                    self.on_failure(r)
        return new

    def start(self):
        def loop():
            while not self._stop.wait(self.cfg.heartbeat_interval_s):
                self.beat()
                self.poll()
        self.beat()
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def failed_ranks(self) -> List[int]:
        with self._lock:
            return list(self._failed)

    def mark_recovered(self, r: int):
        with self._lock:
            if r in self._failed:
                self._failed.remove(r)
        self._last.pop(r, None)

    def should_stop(self) -> bool:
        """True once any peer has failed: the caller finishes the current step and leaves the training loop."""
        return bool(self.failed_ranks())


@dataclass
class NodeInfo:
    node_id: int
    address: str = "127.0.0.1"
    alive: bool = True
    experts: List[int] = field(default_factory=list)
    load: float = 0.0
    capacity: float = 1.0


class FaultToleranceManager:
    """Expert placement that survives node loss."""

    def __init__(self, num_nodes: int, num_experts: int):
        per = -(-num_experts // num_nodes)
        self.nodes = [NodeInfo(n, experts=list(range(n * per, min(num_experts, (n + 1) * per)))) for n in range(num_nodes)]
        self.failed: List[int] = []
        self.events: List[dict] = []
        self._lock = threading.Lock()

    def owner_of(self, expert: int) -> int:
        for n in self.nodes:
            if n.alive and expert in n.experts:
                return n.node_id
        raise KeyError(expert)

    def on_node_failure(self, node_id: int) -> Dict[int, int]:
        """Marks the node dead and hands its experts to the first alive node (the reference's rule). Returns the
        moves {expert: new owner}."""
        with self._lock:
            if node_id in self.failed:
                return {}
            node = self.nodes[node_id]
            node.alive = False
            self.failed.append(node_id)
            target = next((n for n in self.nodes if n.alive), None)
            if target is None:
                raise RuntimeError("no node left alive")
            moves = {e: target.node_id for e in node.experts}
            target.experts.extend(node.experts)
            node.experts = []
            self.events.append({"t": time.time(), "failed": node_id, "moves": moves})
            return moves

    def on_node_recovery(self, node_id: int):
        with self._lock:
            if node_id in self.failed:
                self.failed.remove(node_id)
            self.nodes[node_id].alive = True

    def redistribution_plan(self) -> Dict[int, int]:
        """Balanced placement over the alive nodes (least loaded first): {expert: node}. Does not apply it."""
        alive = [n for n in self.nodes if n.alive]
        experts = sorted(e for n in self.nodes for e in n.experts)
        plan, load = {}, {n.node_id: 0 for n in alive}
        for e in experts:
            tgt = min(alive, key=lambda n: (load[n.node_id] / n.capacity, n.node_id))
            plan[e] = tgt.node_id
            load[tgt.node_id] += 1
        return plan

    def apply_plan(self, plan: Dict[int, int]):
        with self._lock:
            for n in self.nodes:
                n.experts = []
            for e, nid in sorted(plan.items()):
                self.nodes[nid].experts.append(e)

    # text checkpoint of the node list, like the reference's
    def checkpoint(self, path: str):
        with open(path, "w") as f:
            f.write(f"nodes {len(self.nodes)}\n")
            for n in self.nodes:
                f.write(f"{n.node_id} {n.address} {int(n.alive)} {n.capacity} {','.join(map(str, n.experts))}\n")
            f.write("failed " + ",".join(map(str, self.failed)) + "\n")

    @classmethod
    def restore(cls, path: str) -> "FaultToleranceManager":
        lines = open(path).read().splitlines()
        count = int(lines[0].split()[1])
        self = cls.__new__(cls)
        self.nodes, self.events, self._lock = [], [], threading.Lock()
        for ln in lines[1:1 + count]:
            parts = ln.split(" ")
            ex = [int(x) for x in parts[4].split(",") if x] if len(parts) > 4 else []
            self.nodes.append(NodeInfo(int(parts[0]), parts[1], parts[2] == "1", ex, 0.0, float(parts[3])))
        tail = lines[1 + count].split(" ", 1)
        self.failed = [int(x) for x in tail[1].split(",") if x] if len(tail) > 1 else []
        return self


class CapacityAwareRouter:
    """Sends a token's expert choice to the next-best expert when the preferred one (or its node) is full."""

    def __init__(self, num_experts: int, capacity_per_expert: int):
        self.E, self.cap = num_experts, capacity_per_expert
        self.load = [0] * num_experts
        self.rerouted = 0

    def reset(self):
        self.load = [0] * self.E
        self.rerouted = 0

    def route(self, ranked_experts: List[int]) -> int:
        for i, e in enumerate(ranked_experts):
            if self.load[e] < self.cap:
                self.load[e] += 1
                self.rerouted += int(i > 0)
                return e
        return -1          # dropped


def run_elastic(train_fn: Callable[[int, int], str], world_sizes: List[int], max_retries: int = 3) -> List[str]:
    """Driver for the restart loop: ``train_fn(world, attempt)`` runs (or spawns) a training segment at the given
    world size and returns "done" or "failed"; on failure the next, smaller world size in ``world_sizes`` is tried
    from the last checkpoint, at most ``max_retries`` times."""
    log = []
    attempt = 0
    for world in world_sizes:
        status = train_fn(world, attempt)
        log.append(f"{world}:{status}")
        if status == "done":
            break
        attempt += 1
        if attempt > max_retries:
            break
    return log
