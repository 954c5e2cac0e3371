"""Request gathering and the worker cap of the HTTP serving front end."""
import json
import threading
import time
import urllib.request

import pytest

from innova_b200.cli.serve import MicroBatcher
from innova_b200.serving.http_server import HTTPServer


def test_micro_batcher_gathers_concurrent_requests():
    calls = []

    def run_batch(prompts, n):
        calls.append((list(prompts), n))
        time.sleep(0.02)
        return [p.upper() + f":{n}" for p in prompts]
    mb = MicroBatcher(run_batch, max_batch=4, window_s=0.2)
    out = {}
    ts = [threading.Thread(target=lambda k=k: out.__setitem__(k, mb.submit(f"p{k}", 10 + k))) for k in range(6)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=10)
    assert out == {k: f"P{k}:{max(10 + j for j in range(6) if any(f'p{j}' in c[0] and f'p{k}' in c[0] for c in calls))}" for k in range(6)}
    assert sorted(mb.batches, reverse=True) == [4, 2] and sum(len(c[0]) for c in calls) == 6     # a full batch leaves early, the rest at the window's end
    assert mb.submit("solo", 3) == "SOLO:3" and mb.batches[-1] == 1
    mb.stop()
    with pytest.raises(RuntimeError):
        mb.submit("late", 1)


def test_micro_batcher_hands_errors_to_every_caller():
    def boom(prompts, n):
        raise ValueError("engine down")
    mb = MicroBatcher(boom, max_batch=2, window_s=0.05)
    errs = []

    def call():
        try:
            mb.submit("x", 1)
        except ValueError as e:
            errs.append(str(e))
    ts = [threading.Thread(target=call) for _ in range(2)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=10)
    assert errs == ["engine down"] * 2
    mb.stop()


def test_worker_cap_bounds_concurrency():
    srv = HTTPServer(0)
    srv.set_max_workers(2)
    live, peak, lock = [0], [0], threading.Lock()

    def gen(prompt, n, stream):
        with lock:
            live[0] += 1
            peak[0] = max(peak[0], live[0])
        time.sleep(0.05)
        with lock:
            live[0] -= 1
        return "ok"
    srv.set_generate_callback(gen)
    srv.start()
    try:
        def post():
            req = urllib.request.Request(f"http://127.0.0.1:{srv.port}/v1/completions", data=json.dumps({"prompt": "a", "max_tokens": 2}).encode(),
                                         headers={"Content-Type": "application/json"})
            assert urllib.request.urlopen(req, timeout=10).status == 200
        ts = [threading.Thread(target=post) for _ in range(6)]
        for t in ts:
            t.start()
        for t in ts:
            t.join(timeout=20)
        assert peak[0] == 2 and srv.total_requests >= 6
    finally:
        srv.stop()
