"""HTTP/1.1 model server with OpenAI-style endpoints.

Reference: ``HTTPServer`` (thread pool, JSON in/out, SSE streaming, CORS on every response, per-IP token-bucket
rate limit, model load / unload through the API; endpoints ``/v1/completions``, ``/v1/chat/completions``,
``/v1/embeddings``, ``/v1/models``, ``/health``; include/oil/http_server.h:22-149, tools/serve.cpp:18-110).
The reference hand-rolls sockets and a JSON parser; here the transport is the standard library's threading HTTP
server and generation is delegated to callbacks, exactly like the reference's ``set_generate_callback``.
"""
from __future__ import annotations

import json
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Callable, Dict, Iterable, List, Optional, Union


class RateLimiter:
    """Token bucket per client address: ``max_rps`` tokens per second, capacity ``burst``. 0 disables."""

    def __init__(self, max_requests_per_sec: float = 0, burst: int = 0):
        self.max_rps, self.burst = max_requests_per_sec, burst or int(max_requests_per_sec)
        self._buckets: Dict[str, List[float]] = {}
        self._lock = threading.Lock()

    def set_limits(self, max_requests_per_sec: float, burst: int):
        self.max_rps, self.burst = max_requests_per_sec, burst or int(max_requests_per_sec)

    def allow(self, ip: str, now: Optional[float] = None) -> bool:
        if self.max_rps <= 0:
            return True
        now = time.monotonic() if now is None else now
        with self._lock:
            tokens, last = self._buckets.get(ip, [float(self.burst), now])
            tokens = min(float(self.burst), tokens + (now - last) * self.max_rps)
            ok = tokens >= 1.0
            self._buckets[ip] = [tokens - 1.0 if ok else tokens, now]
            return ok


GenerateCallback = Callable[[str, int, bool], Union[str, Iterable[str]]]


class HTTPServer:
    def __init__(self, port: int = 8080, host: str = "127.0.0.1"):
        self.port, self.host = port, host
        self.model_name = "InNova-default"
        self.generate_cb: Optional[GenerateCallback] = None
        self.embeddings_cb: Optional[Callable[[str], List[float]]] = None
        self.load_model_cb: Optional[Callable[[str], bool]] = None
        self.unload_model_cb: Optional[Callable[[], None]] = None
        self.rate_limiter = RateLimiter()
        self.max_body_size = 4 * 1024 * 1024
        self.timeout_seconds = 30
        self.total_requests = 0
        self.total_errors = 0
        self._httpd: Optional[ThreadingHTTPServer] = None
        self._thread: Optional[threading.Thread] = None
        self._count_lock = threading.Lock()
        self.started_at = time.time()
        self._slots: Optional[threading.BoundedSemaphore] = None

    def set_max_workers(self, n: int):
        """At most ``n`` requests are handled at once; the others wait for a free slot (the reference sizes a thread pool)."""
        self._slots = threading.BoundedSemaphore(n) if n > 0 else None

    # configuration in the reference's spelling
    def set_generate_callback(self, cb): self.generate_cb = cb
    def set_embeddings_callback(self, cb): self.embeddings_cb = cb
    def set_load_model_callback(self, cb): self.load_model_cb = cb
    def set_unload_model_callback(self, cb): self.unload_model_cb = cb
    def set_rate_limit(self, rps, burst): self.rate_limiter.set_limits(rps, burst)
    def set_model_name(self, name): self.model_name = name
    def set_max_body_size(self, n): self.max_body_size = n
    def set_timeout_seconds(self, s): self.timeout_seconds = s
    def is_running(self): return self._httpd is not None

    # ------------------------------------------------------------------ request handling
    def _completion(self, prompt: str, body: dict, chat: bool):
        max_tokens = int(body.get("max_tokens", 64))
        stream = bool(body.get("stream", False))
        rid = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:12]
        created = int(time.time())
        if self.generate_cb is None:
            return 503, {"error": {"message": "no model loaded", "type": "unavailable"}}, None
        result = self.generate_cb(prompt, max_tokens, stream)

        def chunk(text, finish=None):
            if chat:
                choice = {"index": 0, "delta": {"content": text} if finish is None else {}, "finish_reason": finish}
                obj = "chat.completion.chunk"
            else:
                choice = {"index": 0, "text": text, "finish_reason": finish}
                obj = "text_completion"
            return {"id": rid, "object": obj, "created": created, "model": self.model_name, "choices": [choice]}
        if stream:
            pieces = [result] if isinstance(result, str) else result

            def events():
                for p in pieces:
                    yield "data: " + json.dumps(chunk(p)) + "\n\n"
                yield "data: " + json.dumps(chunk("", "stop")) + "\n\n"
                yield "data: [DONE]\n\n"
            return 200, None, events()
        text = result if isinstance(result, str) else "".join(result)
        usage = {"prompt_tokens": len(prompt.split()), "completion_tokens": len(text.split())}
        usage["total_tokens"] = usage["prompt_tokens"] + usage["completion_tokens"]
        if chat:
            choice = {"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": "stop"}
            obj = "chat.completion"
        else:
            choice = {"index": 0, "text": text, "finish_reason": "stop"}
            obj = "text_completion"
        return 200, {"id": rid, "object": obj, "created": created, "model": self.model_name, "choices": [choice], "usage": usage}, None

    def handle(self, method: str, path: str, body: bytes, client: str = "local"):
        """-> (status, json object or None, SSE iterator or None). Usable without sockets (tests, embedding)."""
        with self._count_lock:
            self.total_requests += 1
        path = path.split("?")[0].rstrip("/") or "/"
        if method == "OPTIONS":
            return 204, None, None
        if not self.rate_limiter.allow(client):
            return self._err(429, "rate limit exceeded")
        if method == "GET" and path == "/health":
            return 200, {"status": "ok", "model": self.model_name, "uptime_s": time.time() - self.started_at, "requests": self.total_requests,
                         "errors": self.total_errors}, None
        if method == "GET" and path == "/v1/models":
            return 200, {"object": "list", "data": [{"id": self.model_name, "object": "model", "owned_by": "innova"}]}, None
        if method != "POST":
            return self._err(404 if method == "GET" else 405, f"no route for {method} {path}")
        if len(body) > self.max_body_size:
            return self._err(413, "request body too large")
        try:
            req = json.loads(body.decode("utf-8") or "{}")
            if not isinstance(req, dict):
                raise ValueError("body must be a JSON object")
        except Exception as e:          # malformed JSON is the client's error, never the server's
            return self._err(400, f"invalid JSON: {e}")
        if path == "/v1/completions":
            prompt = req.get("prompt", "")
            prompt = prompt if isinstance(prompt, str) else " ".join(map(str, prompt))
            return self._completion(prompt, req, chat=False)
        if path == "/v1/chat/completions":
            msgs = req.get("messages", [])
            prompt = "\n".join(f"{m.get('role', 'user')}: {m.get('content', '')}" for m in msgs if isinstance(m, dict)) + "\nassistant:"
            return self._completion(prompt, req, chat=True)
        if path == "/v1/embeddings":
            if self.embeddings_cb is None:
                return self._err(503, "no embedding model loaded")
            inp = req.get("input", "")
            texts = [inp] if isinstance(inp, str) else list(inp)
            data = [{"object": "embedding", "index": i, "embedding": list(map(float, self.embeddings_cb(t)))} for i, t in enumerate(texts)]
            return 200, {"object": "list", "data": data, "model": self.model_name}, None
        if path == "/v1/models/load":
            ok = bool(self.load_model_cb and self.load_model_cb(str(req.get("path", ""))))
            return (200, {"loaded": True}, None) if ok else self._err(400, "could not load model")
        if path == "/v1/models/unload":
            if self.unload_model_cb:
                self.unload_model_cb()
            return 200, {"unloaded": True}, None
        return self._err(404, f"no route for POST {path}")

    def _err(self, status, msg):
        with self._count_lock:
            self.total_errors += 1
        return status, {"error": {"message": msg, "code": status}}, None

    # ------------------------------------------------------------------ transport
    def start(self):
        server = self

        class Handler(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):
                pass

            def _cors(self):
                self.send_header("Access-Control-Allow-Origin", "*")
                self.send_header("Access-Control-Allow-Methods", "GET, POST, OPTIONS")
                self.send_header("Access-Control-Allow-Headers", "Content-Type, Authorization")

            def _serve(self, method):
                n = int(self.headers.get("Content-Length", 0) or 0)
                body = self.rfile.read(min(n, server.max_body_size + 1)) if n else b""
                slots = server._slots
                if slots is not None:
                    slots.acquire()
                try:
                    status, obj, sse = server.handle(method, self.path, body, self.client_address[0])
                except Exception as e:
                    status, obj, sse = server._err(500, f"internal error: {e}")
                finally:
                    if slots is not None:
                        slots.release()
                if sse is not None:
                    self.send_response(200)
                    self.send_header("Content-Type", "text/event-stream")
                    self.send_header("Cache-Control", "no-cache")
                    self.send_header("Connection", "close")
                    self._cors()
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
                self._cors()
                self.end_headers()
                self.wfile.write(data)

            def do_GET(self): self._serve("GET")
            def do_POST(self): self._serve("POST")
            def do_OPTIONS(self): self._serve("OPTIONS")
        self._httpd = ThreadingHTTPServer((self.host, self.port), Handler)
        self._httpd.timeout = self.timeout_seconds
        self.port = self._httpd.server_address[1]
        self._thread = threading.Thread(target=self._httpd.serve_forever, daemon=True)
        self._thread.start()

    def stop(self):
        if self._httpd is not None:
            self._httpd.shutdown()
            self._httpd.server_close()
            self._httpd = None
