"""oil-serve: HTTP serving of a saved model (tools/serve.cpp:18-110, default port 8080; the reference's second
server binary listens on 9090, ``--port 9090`` gives the same)."""
from __future__ import annotations

import argparse
import sys
import time


def build_server(model_path: str, port: int = 8080, host: str = "127.0.0.1", device=None, rate_limit: float = 0.0, max_new_tokens: int = 256):
    from ..inference.serving import EmbeddingEndpoint, InferenceEngine
    from ..serving.http_server import HTTPServer
    import threading
    # One engine = one generator = one paged KV cache whose rows a generation frees and rewrites at its start. HTTP
    # request threads and WebSocket client threads all end up here, so a generation (the whole stream, not only its
    # start), an embedding and a model swap each hold this lock from beginning to end.
    state = {"engine": InferenceEngine(model_path, device=device), "lock": threading.Lock()}
    srv = HTTPServer(port, host)
    srv.set_model_name(model_path.rsplit("/", 1)[-1])

    def _locked_stream(prompt, n):
        with state["lock"]:
            yield from state["engine"].stream(prompt, n)

    def generate(prompt, n, stream):
        n = min(n, max_new_tokens)
        if stream:
            return _locked_stream(prompt, n)      # the lock is taken when the first piece is asked for, released with the last
        with state["lock"]:
            return state["engine"].generate(prompt, n)

    def embed(text):
        with state["lock"]:
            eng = state["engine"]
            return EmbeddingEndpoint(eng.model, eng.tok).embed(text).tolist()

    def load(path):
        try:
            new = InferenceEngine(path, device=device)       # built outside the lock: running generations are not held up
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
    ap.add_argument("--ws-port", type=int, default=0, help="also stream tokens over WebSocket on this port (0 = off; the reference uses 8081)")
    a = ap.parse_args(argv)
    srv = build_server(a.model, a.port, a.host, a.device, a.rate_limit)
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
    return 0


if __name__ == "__main__":
    sys.exit(main())
