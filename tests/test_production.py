"""HTTP server, rate limiter, config, zoo, plugins and the batching model server."""
import json
import threading
import time
import urllib.error
import urllib.request

from innova_b200.serving.http_server import HTTPServer, RateLimiter
from innova_b200.serving.production import AppConfig, Logger, ModelServer, ModelZoo, PluginManager


def _server():
    s = HTTPServer(port=0)
    s.set_model_name("tiny-test")
    s.set_generate_callback(lambda prompt, n, stream: ["echo:", prompt[-5:]] if stream else "echo:" + prompt[-5:])
    s.set_embeddings_callback(lambda t: [float(len(t)), 1.0])
    return s


def test_routes_without_sockets():
    s = _server()
    assert s.handle("GET", "/health", b"")[0] == 200
    assert s.handle("GET", "/v1/models", b"")[1]["data"][0]["id"] == "tiny-test"
    st, obj, _ = s.handle("POST", "/v1/completions", json.dumps({"prompt": "hello world", "max_tokens": 3}).encode())
    assert st == 200 and obj["choices"][0]["text"] == "echo:world" and obj["object"] == "text_completion"
    st, obj, _ = s.handle("POST", "/v1/chat/completions", json.dumps({"messages": [{"role": "user", "content": "hi"}]}).encode())
    assert st == 200 and obj["choices"][0]["message"]["role"] == "assistant"
    st, obj, _ = s.handle("POST", "/v1/embeddings", json.dumps({"input": ["ab", "abcd"]}).encode())
    assert [d["embedding"][0] for d in obj["data"]] == [2.0, 4.0]
    assert s.handle("POST", "/v1/completions", b"{not json")[0] == 400          # malformed JSON: 400, never 500
    assert s.handle("POST", "/v1/completions", b"[1,2]")[0] == 400
    assert s.handle("POST", "/nope", b"{}")[0] == 404 and s.handle("GET", "/nope", b"")[0] == 404
    s.set_max_body_size(10)
    assert s.handle("POST", "/v1/completions", b"{" + b" " * 20 + b"}")[0] == 413
    st, _, sse = _server().handle("POST", "/v1/completions", json.dumps({"prompt": "abcdef", "stream": True}).encode())
    events = list(sse)
    assert st == 200 and events[-1] == "data: [DONE]\n\n" and json.loads(events[0][6:])["choices"][0]["text"] == "echo:"
    assert s.total_errors >= 4


def test_rate_limiter_token_bucket():
    rl = RateLimiter(2, 2)
    assert [rl.allow("a", now=0.0) for _ in range(3)] == [True, True, False]
    assert rl.allow("b", now=0.0) and rl.allow("a", now=0.6) and not rl.allow("a", now=0.6)
    assert RateLimiter(0).allow("x")
    s = _server()
    s.set_rate_limit(1, 1)
    assert s.handle("GET", "/health", b"", "1.2.3.4")[0] == 200 and s.handle("GET", "/health", b"", "1.2.3.4")[0] == 429


def test_real_socket_roundtrip_with_cors_and_sse():
    s = _server()
    s.start()
    try:
        base = f"http://127.0.0.1:{s.port}"
        with urllib.request.urlopen(base + "/health", timeout=5) as r:
            assert r.status == 200 and r.headers["Access-Control-Allow-Origin"] == "*"
        req = urllib.request.Request(base + "/v1/completions", data=json.dumps({"prompt": "socket"}).encode(), method="POST")
        with urllib.request.urlopen(req, timeout=5) as r:
            assert json.loads(r.read())["choices"][0]["text"] == "echo:ocket"
        req = urllib.request.Request(base + "/v1/completions", data=json.dumps({"prompt": "stream", "stream": True}).encode(), method="POST")
        with urllib.request.urlopen(req, timeout=5) as r:
            body = r.read().decode()
            assert r.headers["Content-Type"] == "text/event-stream" and body.endswith("data: [DONE]\n\n")
        try:
            urllib.request.urlopen(urllib.request.Request(base + "/v1/completions", data=b"{bad", method="POST"), timeout=5)
            assert False
        except urllib.error.HTTPError as e:
            assert e.code == 400
    finally:
        s.stop()


def test_config_zoo_plugins_logger(tmp_path, monkeypatch):
    cfg = AppConfig({"server": {"port": 8080}})
    cfg.set("model.path", "m.oil")
    assert cfg.get("server.port") == 8080 and cfg.get("model.path") == "m.oil" and cfg.get("x.y", 3) == 3
    p = tmp_path / "c.json"
    cfg.save(str(p))
    monkeypatch.setenv("INNOVA_SERVER_PORT", "9090")
    assert AppConfig.load(str(p)).get("server.port") == 9090
    zoo = ModelZoo(str(tmp_path / "zoo.json"))
    zoo.register("tiny", "/models/tiny.oil", params=1000)
    assert ModelZoo(str(tmp_path / "zoo.json")).resolve("tiny") == "/models/tiny.oil" and zoo.list() == ["tiny"]
    plug = tmp_path / "plug.py"
    plug.write_text("VALUE = 1\ndef plugin_init():\n    return 'ready'\n")
    pm = PluginManager()
    assert pm.load(str(plug)).VALUE == 1 and pm.plugins["plug"]["init_result"] == "ready"
    time.sleep(0.01)
    plug.write_text("VALUE = 2\n")
    import os
    os.utime(plug, (time.time() + 5, time.time() + 5))
    assert pm.reload_changed() == ["plug"] and pm.get("plug").VALUE == 2
    lg = Logger(str(tmp_path / "log.txt"), level="warn", json_lines=True)
    lg.info("hidden")
    lg.error("boom", code=7)
    lines = open(tmp_path / "log.txt").read().splitlines()
    assert len(lines) == 1 and json.loads(lines[0])["code"] == 7


def test_model_server_batches_and_orders_by_priority():
    seen = []

    def gen(prompts, n):
        seen.append(list(prompts))
        time.sleep(0.01)
        return [p.upper() for p in prompts]
    ms = ModelServer(gen, max_batch=4, max_wait_s=0.05)
    jobs = [ms.submit(f"p{i}", priority=i % 2) for i in range(6)]
    for j in jobs:
        assert j.event.wait(5)
    assert [j.result for j in jobs] == [f"P{i}" for i in range(6)]
    assert ms.generate("solo", timeout=5) == "SOLO"
    assert any(len(b) > 1 for b in seen) and ms.latency_percentiles()["p99"] > 0
    ms.stop()


def test_model_server_surface_metrics_callbacks_and_model_swap():
    import json
    import threading
    from innova_b200.serving.production import ModelServer, consolidate_batch
    srv = ModelServer(lambda prompts, n: [p.upper() for p in prompts], max_batch=4, max_wait_s=0.01)
    try:
        assert srv.is_running() and srv.is_model_loaded() and json.loads(srv.health_json())["status"] == "ok"
        got, done = {}, threading.Event()
        rid = srv.submit_with_callback("abc", 8, 0, lambda p, r: (got.update({p: r}), done.set()))
        assert rid >= 1 and done.wait(5) and got == {"abc": "ABC"} and srv.generate("x") == "X"
        m = json.loads(srv.metrics_json())
        assert m["total_requests"] == 2 and m["total_errors"] == 0 and m["batches"] >= 1 and m["p99_ms"] >= m["p50_ms"] >= 0
        srv.set_batch_size(2)
        srv.set_queue_wait_ms(1)
        assert srv.max_batch == 2 and srv.max_wait_s == 0.001
        assert srv.load_model(lambda: (lambda prompts, n: [p[::-1] for p in prompts])) and srv.generate("abc") == "cba"
        assert not srv.load_model(lambda: 1 / 0) and srv.generate("abc") == "cba"            # a failed load keeps the old model
        srv.unload_model()
        assert not srv.is_model_loaded() and isinstance(srv.generate("abc"), RuntimeError) and srv.metrics()["total_errors"] == 1
    finally:
        srv.stop()
    assert not srv.is_running() and json.loads(srv.health_json())["status"] == "stopped"
    b = consolidate_batch([(7, [5, 6, 7]), (9, [1]), (11, [2, 3])], pad_id=0)
    assert b.request_ids == [7, 9, 11] and b.seq_lens == [3, 1, 2] and b.offsets == [0, 3, 4]
    assert b.batched_input.tolist() == [[5, 6, 7], [1, 0, 0], [2, 3, 0]] and b.batched_positions.tolist() == [[0, 1, 2], [0, 0, 0], [0, 1, 0]]
    assert consolidate_batch([]).batched_input.shape == (0, 0)
