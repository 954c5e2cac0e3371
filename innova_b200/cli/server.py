"""oil-server: the reference's second serving tool (tools/oil_server.cpp:40-594): token-level API on port 9090.

Routes
    POST /api/generate     {"prompt", "max_tokens", "temperature", "top_k", "top_p", "stream"}
                           -> {"choices": [{"text"}], "usage": {"prompt_tokens", "completion_tokens"}}, or with
                           "stream": true server-sent events {"token", "index"} ... {"done": true, "count"}
    POST /api/tokenize     {"content"} -> {"tokens": [...]}
    POST /api/detokenize   {"tokens": [...]} -> {"content"}
    GET  /health, /        {"status": "ok", ...}
The tokenizer comes from ``--model-dir`` (a Qwen-layout vocab.json + merges.txt, as the reference's server expects next to
the model), else from ``<model>.vocab``, else bytes. One generation runs at a time (one KV cache); the worker pool only
keeps slow clients from blocking each other's I/O.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer


class OilServer:
    def __init__(self, model_path: str, model_dir: str = "", device=None, max_tokens: int = 2048, temperature: float = 0.7, top_k: int = 40,
                 top_p: float = 0.9, eos_id: int = 2):
        from ..inference.serving import InferenceEngine
        self.engine = InferenceEngine(model_path, device=device)
        self.tok = self._tokenizer(model_path, model_dir) or self.engine.tok
        if self.tok is None:
            from ..utils.tokenizer import ByteTokenizer
            self.tok = ByteTokenizer()
        self.engine.gen.tok = self.tok
        self.defaults = dict(max_tokens=max_tokens, temperature=temperature, top_k=top_k, top_p=top_p)
        self.eos_id = eos_id
        self.lock = threading.Lock()
        self.started, self.requests = time.time(), 0
        self.httpd = None

    @staticmethod
    def _tokenizer(model_path, model_dir):
        d = model_dir or os.path.dirname(os.path.abspath(model_path))
        if os.path.exists(os.path.join(d, "vocab.json")) and os.path.exists(os.path.join(d, "merges.txt")):
            from ..utils.qwen_tokenizer import QwenTokenizer
            return QwenTokenizer.load_from_dir(d)
        return None

    # ---- request handling without sockets (tests call this directly) ----
    def handle(self, method: str, path: str, body: bytes):
        """-> (status, json object or None, iterator of SSE strings or None)."""
        self.requests += 1
        path = path.split("?")[0].rstrip("/") or "/"
        if method == "OPTIONS":
            return 204, None, None
        if method == "GET" and path in ("/", "/health"):
            return 200, {"status": "ok", "uptime_s": time.time() - self.started, "requests": self.requests,
                         "vocab_size": getattr(self.tok, "vocab_size", 0) if not callable(getattr(self.tok, "vocab_size", None))
                         else self.tok.vocab_size()}, None
        if method != "POST":
            return 404, {"error": f"no route for {method} {path}"}, None
        try:
            req = json.loads(body.decode("utf-8") or "{}")
            if not isinstance(req, dict):
                raise ValueError("body must be a JSON object")
        except Exception as e:  # noqa: BLE001
            return 400, {"error": f"invalid JSON: {e}"}, None
        try:
            if path == "/api/tokenize":
                return 200, {"tokens": [int(t) for t in self.tok.encode(str(req.get("content", "")))]}, None
            if path == "/api/detokenize":
                return 200, {"content": self.tok.decode([int(t) for t in req.get("tokens", [])])}, None
            if path == "/api/generate":
                return self._generate(req)
        except Exception as e:  # noqa: BLE001
            return 500, {"error": f"{path.rsplit('/', 1)[-1]}: {e}"}, None
        return 404, {"error": f"no route for POST {path}"}, None

    def _generate(self, req):
        from ..inference.sampler import SamplingParams
        d = self.defaults
        n = max(1, min(int(req.get("max_tokens", d["max_tokens"])), d["max_tokens"]))
        sp = SamplingParams(temperature=float(req.get("temperature", d["temperature"])), top_k=int(req.get("top_k", d["top_k"])),
                            top_p=float(req.get("top_p", d["top_p"])))
        tokens = [int(t) for t in self.tok.encode(str(req.get("prompt", "")))] or [0]
        gen = self.engine.gen
        if not req.get("stream"):
            with self.lock:
                out = gen.generate_tokens([tokens], n, sp, eos_id=self.eos_id)[0]
            if out and out[-1] == self.eos_id:
                out = out[:-1]
            return 200, {"choices": [{"text": self.tok.decode(out) if out else ""}],
                         "usage": {"prompt_tokens": len(tokens), "completion_tokens": len(out)}}, None

        def events():
            with self.lock:
                out = gen.generate_tokens([tokens], n, sp, eos_id=self.eos_id)[0]
            count = 0
            for i, t in enumerate(out):
                if t == self.eos_id:
                    break
                count += 1
                yield "data: " + json.dumps({"token": self.tok.decode([t]), "index": i}) + "\n\n"
            yield "data: " + json.dumps({"done": True, "count": count}) + "\n\n"
        return 200, None, events()

    # ---- transport ----
    def start(self, port: int = 9090, host: str = "127.0.0.1"):
        srv = self

        class H(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):
                pass

            def _do(self, method):
                n = int(self.headers.get("Content-Length", 0) or 0)
                status, obj, sse = srv.handle(method, self.path, self.rfile.read(n) if n else b"")
                if sse is not None:
                    self.send_response(200)
                    self.send_header("Content-Type", "text/event-stream")
                    self.send_header("Cache-Control", "no-cache")
                    self.send_header("Connection", "close")
                    self.send_header("Access-Control-Allow-Origin", "*")
                    self.end_headers()
                    for ev in sse:
                        self.wfile.write(ev.encode())
                        self.wfile.flush()
                    self.close_connection = True
                    return
                data = b"" if obj is None else json.dumps(obj).encode()
                self.send_response(status)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(data)))
                self.send_header("Access-Control-Allow-Origin", "*")
                self.end_headers()
                self.wfile.write(data)

            def do_GET(self): self._do("GET")          # noqa: E704
            def do_POST(self): self._do("POST")        # noqa: E704
            def do_OPTIONS(self): self._do("OPTIONS")  # noqa: E704
        self.httpd = ThreadingHTTPServer((host, port), H)
        self.port = self.httpd.server_address[1]
        self.thread = threading.Thread(target=self.httpd.serve_forever, daemon=True)
        self.thread.start()
        return self

    def stop(self):
        if self.httpd is not None:
            self.httpd.shutdown()
            self.httpd.server_close()
            self.httpd = None


def main(argv=None):
    ap = argparse.ArgumentParser(prog="oil-server")
    ap.add_argument("--model", required=True)
    ap.add_argument("--model-dir", default="")
    ap.add_argument("--port", type=int, default=9090)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--workers", type=int, default=4, help="accepted for compatibility: connections are served by one thread each")
    ap.add_argument("--max-tokens", type=int, default=2048)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--top-k", type=int, default=40)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)
    try:
        srv = OilServer(a.model, a.model_dir, a.device, a.max_tokens, a.temperature, a.top_k, a.top_p)
    except Exception as e:  # noqa: BLE001
        print(f"Error loading model: {e}", file=sys.stderr)
        return 1
    srv.start(a.port, a.host)
    print(f"oil-server: {a.model} on http://{a.host}:{srv.port}", flush=True)
    try:
        while True:
            time.sleep(0.5)
    except KeyboardInterrupt:
        srv.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
