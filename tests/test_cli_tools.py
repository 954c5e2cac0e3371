"""oil-quantize / oil-finetune / oil-evaluate / oil-bench / oil-serve on a tiny model trained here (CPU)."""
import json
import os
import subprocess
import sys
import urllib.request

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(mod, *args):
    r = subprocess.run([sys.executable, "-m", mod, *args], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    d = tmp_path_factory.mktemp("cli")
    corpus = d / "corpus.txt"
    corpus.write_text("the quick brown fox jumps over the lazy dog. " * 200)
    model = str(d / "m.oil")
    _run("innova_b200.cli.train", "--model", model, "--data", str(corpus), "--batch-size", "4", "--seq-length", "32", "--hidden-size", "64",
         "--num-layers", "2", "--num-heads", "2", "--max-steps", "25", "--lr", "3e-3", "--device", "cpu", "--vocab-size", "256")
    return d, model, str(corpus)


def test_quantize_evaluate_finetune_bench(tiny):
    d, model, corpus = tiny
    q = str(d / "q.oil")
    res = json.loads(_run("innova_b200.cli.quantize", "--input", model, "--output", q, "--format", "OIL8", "--per-layer",
                          "lm_head=OIL16").splitlines()[-1])
    assert res["bytes_after"] < 0.5 * res["bytes_before"] and 8.0 < res["bpw"] < 14
    ev = json.loads(_run("innova_b200.cli.evaluate", "--model", model, "--data", corpus, "--context", "32", "--stride", "16", "--max-tokens",
                         "600", "--device", "cpu").splitlines()[-1])
    evq = json.loads(_run("innova_b200.cli.evaluate", "--model", q, "--data", corpus, "--context", "32", "--stride", "16", "--max-tokens", "600",
                          "--device", "cpu").splitlines()[-1])
    assert ev[0]["task_name"] == "perplexity" and ev[0]["perplexity"] < 200
    assert abs(evq[0]["perplexity"] / ev[0]["perplexity"] - 1) < 0.1          # OIL8 keeps the model
    # the remaining tasks: windowed classification scores and the ending choice from a JSONL file
    endings = d / "endings.jsonl"
    text = open(corpus, encoding="utf-8").read()
    endings.write_text("\n".join(json.dumps({"ctx": text[k:k + 24], "endings": [text[k + 24:k + 36], "zqxj#@~^|zqxj"], "label": 0}) for k in (0, 40, 80, 120)))
    full = json.loads(_run("innova_b200.cli.evaluate", "--model", model, "--data", corpus, "--context", "32", "--max-tokens", "300", "--task", "all",
                           "--batch-size", "4", "--endings", str(endings), "--device", "cpu").splitlines()[-1])
    by = {r["task_name"]: r for r in full}
    assert set(by) == {"perplexity", "accuracy", "generation", "classification", "hellaswag"}
    assert by["classification"]["total"] == 299 and 0 < by["classification"]["f1_score"] <= 1
    assert abs(by["classification"]["accuracy"] - by["classification"]["correct"] / 299) < 1e-9
    assert by["hellaswag"]["total"] == 4 and by["hellaswag"]["accuracy"] >= 0.75   # text it was trained on beats noise
    for method, out in (("full", "ft.oil"), ("rank", "a.nrad"), ("slots", "k.kexp")):
        r = json.loads(_run("innova_b200.cli.finetune", "--model", model, "--data", corpus, "--output", str(d / out), "--method", method, "--lr",
                            "1e-3", "--batch-size", "2", "--seq-length", "32", "--max-steps", "4", "--device", "cpu", "--rank", "4").splitlines()[-1])
        assert r["steps"] == 4 and os.path.exists(d / out)
    b = json.loads(_run("innova_b200.cli.bench", "--suite", "train", "--hidden-size", "64", "--num-layers", "2", "--num-heads", "2", "--vocab-size",
                        "512", "--batch-size", "2", "--seq-length", "32", "--steps", "2", "--warmup", "1", "--device", "cpu").splitlines()[-1])
    assert b["tokens_per_sec"] > 0
    n = json.loads(_run("innova_b200.cli.bench", "--suite", "native", "--hidden-size", "64", "--num-layers", "2", "--num-heads", "2", "--vocab-size",
                        "512", "--batch-size", "2", "--seq-length", "32", "--steps", "2", "--warmup", "1", "--device", "cpu").splitlines()[-1])
    assert n["phase"] == "native" and n["bits_per_weight"] < 9
    both = _run("innova_b200.cli.bench", "--kernel", "all", "--size", "64", "--inference", "--model", model, "--prompt", "the quick", "--new-tokens", "8",
                "--device", "cpu").splitlines()
    k, inf = json.loads(both[-2]), json.loads(both[-1])
    assert [r["M"] for r in k["rows"]] == [64, 128, 256, 512, 1024] and all(r["ops_linear"]["gflops"] > 0 and r["torch_matmul"]["us"] > 0 for r in k["rows"])
    assert inf["suite"] == "inference" and inf["new_tokens"] == 8 and inf["decode_tokens_per_s"] > 0


def test_serve_answers_over_http(tiny):
    d, model, corpus = tiny
    from innova_b200.cli.serve import build_server
    srv = build_server(model, port=0, device="cpu")
    srv.start()
    try:
        req = urllib.request.Request(f"http://127.0.0.1:{srv.port}/v1/completions", data=json.dumps({"prompt": "the quick", "max_tokens": 5}).encode(),
                                     method="POST")
        with urllib.request.urlopen(req, timeout=60) as r:
            obj = json.loads(r.read())
        assert obj["object"] == "text_completion" and isinstance(obj["choices"][0]["text"], str)
        req = urllib.request.Request(f"http://127.0.0.1:{srv.port}/v1/embeddings", data=json.dumps({"input": "fox"}).encode(), method="POST")
        with urllib.request.urlopen(req, timeout=60) as r:
            assert len(json.loads(r.read())["data"][0]["embedding"]) == 64
        # the same model streams tokens over WebSocket
        from innova_b200.cli.serve import build_websocket
        from innova_b200.serving.websocket import WebSocketClient
        ws = build_websocket(srv, port=0)
        ws.start()
        try:
            c = WebSocketClient("127.0.0.1", ws.port, timeout=60)
            c.send(json.dumps({"prompt": "the quick", "max_tokens": 4}))
            pieces = []
            while True:
                _, payload = c.recv()
                if payload.startswith(b"{") and json.loads(payload).get("done"):
                    break
                pieces.append(payload.decode("utf-8", "replace"))
            assert 1 <= len(pieces) <= 4
            c.close()
        finally:
            ws.stop()
    finally:
        srv.stop()


def test_serve_concurrent_requests_equal_sequential(tiny):
    """HTTP and WebSocket threads share one engine and one paged KV cache: overlapping requests (plain and streamed)
    must produce what the same requests produce one after the other."""
    import threading
    d, model, corpus = tiny
    from innova_b200.cli.serve import build_server
    srv = build_server(model, port=0, device="cpu")
    gen = srv.generate_for_websocket
    prompts = ["the quick", "lazy dog", "brown fox jumps", "over the", "dog. the", "quick brown"]
    want = [gen(p, 8, False) if i % 2 == 0 else "".join(gen(p, 8, True)) for i, p in enumerate(prompts)]
    got = [None] * len(prompts)
    errs = []

    def work(i):
        try:
            for _ in range(2):
                got[i] = gen(prompts[i], 8, False) if i % 2 == 0 else "".join(gen(prompts[i], 8, True))
        except Exception as e:  # noqa: BLE001
            errs.append(e)
    ts = [threading.Thread(target=work, args=(i,)) for i in range(len(prompts))]
    for t in ts:
        t.start()
    for t in ts:
        t.join(120)
    assert not errs, errs
    assert got == want


def test_oil_server_token_api(tiny):
    d, model, corpus = tiny
    from innova_b200.cli.server import OilServer
    srv = OilServer(model, device="cpu", max_tokens=16).start(0)
    try:
        def call(path, obj=None):
            req = urllib.request.Request(f"http://127.0.0.1:{srv.port}{path}", data=None if obj is None else json.dumps(obj).encode(),
                                         method="GET" if obj is None else "POST")
            with urllib.request.urlopen(req, timeout=60) as r:
                return r.read()
        assert json.loads(call("/health"))["status"] == "ok"
        toks = json.loads(call("/api/tokenize", {"content": "the quick"}))["tokens"]
        assert len(toks) >= 2 and json.loads(call("/api/detokenize", {"tokens": toks}))["content"] == "the quick"
        g = json.loads(call("/api/generate", {"prompt": "the quick", "max_tokens": 6, "temperature": 0.0}))
        assert g["usage"]["prompt_tokens"] == len(toks) and 0 <= g["usage"]["completion_tokens"] <= 6 and isinstance(g["choices"][0]["text"], str)
        sse = call("/api/generate", {"prompt": "the quick", "max_tokens": 6, "temperature": 0.0, "stream": True}).decode()
        events = [json.loads(l[6:]) for l in sse.splitlines() if l.startswith("data: ")]
        assert events[-1]["done"] is True and events[-1]["count"] == len(events) - 1
        assert "".join(e["token"] for e in events[:-1]) == g["choices"][0]["text"]
        st, obj, _ = srv.handle("POST", "/api/generate", b"{not json")
        assert st == 400 and "invalid JSON" in obj["error"]
        assert srv.handle("POST", "/api/nothing", b"{}")[0] == 404
    finally:
        srv.stop()


def test_adapters_edition_tools(tiny):
    import io
    from innova_b200.cli import adapters_tools as T
    d, model, corpus = tiny
    q = str(d / "q8.oil")
    _run("innova_b200.cli.quantize", "--input", model, "--output", q, "--format", "OIL8")
    out = _run("innova_b200.cli.adapters_tools", model).splitlines()          # module main = oil-dump
    assert json.loads(out[0])["tensors"] > 5 and "formats" in json.loads(out[1])
    import contextlib
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        assert T.verify_roundtrip([model]) == 0
        assert T.refcheck(["--model", q, "--reference", model, "--tokens", "24", "--device", "cpu"]) == 0
        assert T.refcheck(["--model", q, "--reference", model, "--tokens", "24", "--device", "cpu", "--max-rel-err", "1e-9"]) == 1
    lines = [json.loads(l) for l in buf.getvalue().splitlines()]
    assert lines[0]["mismatched"] == [] and lines[1]["relative_logit_error"] < 0.2 and lines[1]["top1_agreement"] > 0.7
    new = d / "new.txt"
    new.write_text("pack my box with five dozen liquor jugs. " * 60)
    adapted = str(d / "adapted.oil")
    with contextlib.redirect_stdout(io.StringIO()) as rep:
        assert T.adapt(["--model", model, "--data", str(new), "--replay", corpus, "--output", adapted, "--steps", "12", "--batch", "2", "--seq", "32",
                        "--lr", "1e-3", "--device", "cpu"]) == 0
    r = json.loads(rep.getvalue().splitlines()[-1])
    assert os.path.exists(adapted) and r["replay_buffer"] > 0 and r["old_domain_loss_after"] < r["old_domain_loss_before"] + 1.5
    chat_out = io.StringIO()
    assert T.chat([adapted, "--max-tokens", "4", "--greedy", "--device", "cpu"], stdin=io.StringIO("the quick\n/reset\nbrown\n/quit\n"), stdout=chat_out) == 0
    # the reference's short flag names, and the debug dumps after the prefill
    h_out, tr_out, dbg = str(d / "h.bin"), str(d / "t.bin"), io.StringIO()
    import contextlib
    import numpy as np
    with contextlib.redirect_stderr(dbg):
        assert T.chat([adapted, "--max-new", "2", "--temp", "0.5", "--topk", "3", "--raw", "--h-out", h_out, "--trace-out", tr_out, "--debug-logits",
                       "--device", "cpu"], stdin=io.StringIO("the quick\n"), stdout=io.StringIO()) == 0
    hv, tv = np.fromfile(h_out, np.float32), np.fromfile(tr_out, np.float32)
    assert hv.shape == tv.shape == (64,) and np.isfinite(hv).all() and not np.allclose(hv, tv)
    assert "[logits] argmax=" in dbg.getvalue() and "nan=0" in dbg.getvalue() and "[top5]" in dbg.getvalue()
    assert len(chat_out.getvalue().splitlines()) >= 2


def test_import_raw_dtypes_dedup_and_ptq(tmp_path, capsys):
    import json
    import numpy as np
    import torch
    from innova_b200.cli import adapters_tools
    from innova_b200.cli.convert import read_raw
    from innova_b200.formats import oil
    w = torch.randn(8192)
    for dt, tol in (("fp16", 1e-3), ("bf16", 1e-2), ("fp8", 0.07)):
        p = str(tmp_path / f"w.{dt}")
        t = {"fp16": w.half(), "bf16": w.bfloat16(), "fp8": w.to(torch.float8_e4m3fn)}[dt]
        t.view(torch.uint8).numpy().tofile(p)
        back = read_raw(p, dt)
        assert back.shape == w.shape and float((back - w).abs().max() / w.abs().max()) < tol
    src = str(tmp_path / "w.fp16")
    out = str(tmp_path / "m.oil")
    assert adapters_tools.import_main(["--input", src, "--output", out, "--raw-dtype", "fp16", "--to", "OIL8"]) == 0
    info = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert info["weights"] == 8192 and info["bpw"] < 10
    # identical tensors are stored once and read back under both names
    p2 = str(tmp_path / "tied.oil")
    wr = oil.OILWriter(p2)
    assert wr.add_tensor_dedup("tok_embeddings.weight", w, "OIL8") == "tok_embeddings.weight"
    one = wr.payload_bytes()
    assert wr.add_tensor_dedup("lm_head.weight", w.clone(), "OIL8") == "tok_embeddings.weight" and wr.payload_bytes() == one
    assert wr.add_tensor_dedup("other", w + 1, "OIL8") == "other" and wr.payload_bytes() > one
    assert wr.add_tensor_dedup("same_data_other_format", w, "OIL4") == "same_data_other_format"
    wr.close()
    with oil.OILReader(p2) as r:
        assert r.aliases == {"lm_head.weight": "tok_embeddings.weight"}
        assert torch.equal(r.read_tensor("lm_head.weight"), r.read_tensor("tok_embeddings.weight")) and "lm_head.weight" in r.tensor_names()
    q = str(tmp_path / "q.oil")
    assert adapters_tools.ptq(["--input", out, "--output", q, "--format", "OIL4"]) == 0
    with oil.OILReader(q) as r:
        assert r.numel("weights") == 8192
