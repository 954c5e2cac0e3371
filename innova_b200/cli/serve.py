"""oil-serve: HTTP serving of a saved model (tools/serve.cpp:18-110, default port 8080; the reference's second
server binary listens on 9090, ``--port 9090`` gives the same). ``--workers`` bounds how many requests are handled at once,
``--max-tokens`` caps a generation, and ``--batch-size N`` (N > 1) gathers non-streamed requests that arrive within a few
milliseconds of one another into one batched generation."""
from __future__ import annotations

import argparse
import sys
import time


class MicroBatcher:
    """Gathers calls of ``submit(prompt, n)`` from many request threads into calls of ``run_batch(prompts, n_max) -> texts``:
    the first waiting request opens a window of ``window_s``; the batch leaves when the window closes or ``max_batch``
    requests are waiting. Each caller blocks until its own text is ready; a failing batch raises in every caller of it."""

    def __init__(self, run_batch, max_batch: int, window_s: float = 0.005):
        import threading
        self.run_batch, self.max_batch, self.window_s = run_batch, max(1, max_batch), window_s
        self._cv = threading.Condition()
        self._pending = []
        self._stop = False
        self.batches = []                       # sizes of the batches run so far
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def submit(self, prompt: str, n: int) -> str:
        import threading
        slot = {"prompt": prompt, "n": n, "done": threading.Event(), "text": None, "error": None}
        with self._cv:
            if self._stop:
                raise RuntimeError("batcher stopped")
            self._pending.append(slot)
            self._cv.notify_all()
        slot["done"].wait()
        if slot["error"] is not None:
            raise slot["error"]
        return slot["text"]

    def _loop(self):
        while True:
            with self._cv:
                while not self._pending and not self._stop:
                    self._cv.wait()
                if self._stop and not self._pending:
                    return
                deadline = time.monotonic() + self.window_s
                while len(self._pending) < self.max_batch and not self._stop:
                    left = deadline - time.monotonic()
                    if left <= 0:
                        break
                    self._cv.wait(left)
                batch, self._pending = self._pending[: self.max_batch], self._pending[self.max_batch:]
            try:
                texts = self.run_batch([b["prompt"] for b in batch], max(b["n"] for b in batch))
                for b, t in zip(batch, texts):
                    b["text"] = t
            except Exception as e:          # handed to the waiting callers
                for b in batch:
                    b["error"] = e
            self.batches.append(len(batch))
            for b in batch:
                b["done"].set()

    def stop(self):
        with self._cv:
            self._stop = True
            self._cv.notify_all()
        self._thread.join(timeout=5)


def build_server(model_path: str, port: int = 8080, host: str = "127.0.0.1", device=None, rate_limit: float = 0.0, max_new_tokens: int = 256,
                 batch_size: int = 1, workers: int = 0):
    from ..inference.serving import EmbeddingEndpoint, InferenceEngine
    from ..serving.http_server import HTTPServer
    import threading
    # One engine = one generator = one paged KV cache whose rows a generation frees and rewrites at its start. HTTP
    # request threads and WebSocket client threads all end up here, so a generation (the whole stream, not only its
    # start), an embedding and a model swap each hold this lock from beginning to end.
    state = {"engine": InferenceEngine(model_path, device=device, max_batch=max(1, batch_size)), "lock": threading.Lock()}
    srv = HTTPServer(port, host)
    if workers > 0:
        srv.set_max_workers(workers)

    def _run_batch(prompts, n):
        with state["lock"]:
            return state["engine"].generate_batch(prompts, n)
    batcher = MicroBatcher(_run_batch, batch_size) if batch_size > 1 else None
    srv.batcher = batcher
    srv.set_model_name(model_path.rsplit("/", 1)[-1])

    def _locked_stream(prompt, n):
        with state["lock"]:
            yield from state["engine"].stream(prompt, n)

    def generate(prompt, n, stream):
        n = min(n, max_new_tokens)
        if stream:
            return _locked_stream(prompt, n)      # the lock is taken when the first piece is asked for, released with the last
        if batcher is not None:
            return batcher.submit(prompt, n)
        with state["lock"]:
            return state["engine"].generate(prompt, n)

    def embed(text):
        with state["lock"]:
            eng = state["engine"]
            return EmbeddingEndpoint(eng.model, eng.tok).embed(text).tolist()

    def load(path):
        try:
            new = InferenceEngine(path, device=device, max_batch=max(1, batch_size))       # built outside the lock: running generations are not held up
        except Exception:
            return False
        with state["lock"]:
            state["engine"] = new
            srv.set_model_name(path.rsplit("/", 1)[-1])
        return True
    srv.set_generate_callback(generate)
    srv.set_embeddings_callback(embed)
    srv.set_load_model_callback(load)
    if rate_limit > 0:
        srv.set_rate_limit(rate_limit, int(max(1, rate_limit)))
    srv.generate_for_websocket = generate
    return srv


def build_websocket(srv, port: int = 8081, host: str = "127.0.0.1"):
    """Token streaming over WebSocket next to the HTTP server (the reference's ``WebSocketHandler`` on port 8081): a client
    sends ``{"prompt": ..., "max_tokens": ...}`` and receives the pieces as text frames, then ``{"done": true}``."""
    from ..serving.websocket import WebSocketHandler
    ws = WebSocketHandler(port, host)
    ws.set_generate_callback(srv.generate_for_websocket)
    return ws


def main(argv=None):
    ap = argparse.ArgumentParser(prog="oil-serve")
    ap.add_argument("--model", required=True)
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--rate-limit", type=float, default=0.0)
    ap.add_argument("--device", default=None)
    ap.add_argument("--batch-size", type=int, default=1, help="gather up to this many non-streamed requests into one generation")
    ap.add_argument("--workers", type=int, default=4, help="requests handled at once")
    ap.add_argument("--max-tokens", type=int, default=512, help="cap on the tokens of one generation")
    ap.add_argument("--ws-port", type=int, default=0, help="also stream tokens over WebSocket on this port (0 = off; the reference uses 8081)")
    a = ap.parse_args(argv)
    srv = build_server(a.model, a.port, a.host, a.device, a.rate_limit, a.max_tokens, a.batch_size, a.workers)
    srv.start()
    print(f"serving {a.model} on http://{a.host}:{srv.port}", flush=True)
    ws = None
    if a.ws_port:
        ws = build_websocket(srv, a.ws_port, a.host)
        ws.start()
        print(f"token streaming on ws://{a.host}:{ws.port}", flush=True)
    try:
        while srv.is_running():
            time.sleep(0.5)
    except KeyboardInterrupt:
        srv.stop()
    if ws is not None:
        ws.stop()
    if srv.batcher is not None:
        srv.batcher.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
