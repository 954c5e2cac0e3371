"""WebSocket framing, handshake, streaming and broadcast over loopback sockets (CPU)."""
import json
import time

from innova_b200.serving.websocket import (OP_CLOSE, OP_PING, OP_PONG, OP_TEXT, ErrorCode, Result, WebSocketClient, WebSocketHandler,
                                           compute_accept_key, create_frame, parse_frame)


def test_accept_key_and_frames():
    assert compute_accept_key("dGhlIHNhbXBsZSBub25jZQ==") == "s3pPLMBiTxaQ9kYGzzhZRbK+xOo="      # the example of RFC 6455
    for n in (0, 5, 125, 126, 300, 70000):
        data = bytes(i & 0xFF for i in range(n))
        for mask in (None, b"\x01\x02\x03\x04"):
            fr = create_frame(data, 0x2, mask)
            payload, op, fin, used = parse_frame(fr + b"extra")
            assert payload == data and op == 0x2 and fin and used == len(fr)
            assert parse_frame(fr[:-1]) is None if n else True
    assert create_frame("Hello")[:2] == b"\x81\x05" and parse_frame(b"\x81") is None


def test_stream_ping_broadcast_close():
    ws = WebSocketHandler(port=0)
    ws.set_generate_callback(lambda prompt, n, stream: (f"{prompt}-{i} " for i in range(n)))
    ws.start()
    try:
        assert ws.is_running() and ws.port > 0
        a, b = WebSocketClient("127.0.0.1", ws.port), WebSocketClient("127.0.0.1", ws.port)
        deadline = time.time() + 5
        while ws.client_count() < 2 and time.time() < deadline:
            time.sleep(0.01)
        assert ws.client_count() == 2
        a.send(json.dumps({"prompt": "tok", "max_tokens": 3}))
        got = [a.recv() for _ in range(4)]
        assert [p.decode() for _, p in got[:3]] == ["tok-0 ", "tok-1 ", "tok-2 "] and json.loads(got[3][1]) == {"done": True}
        a.send("not json")
        assert "error" in json.loads(a.recv()[1])
        a.send(b"abc", OP_PING)
        assert a.recv() == (OP_PONG, b"abc")
        assert ws.broadcast("hello all") == 2
        assert a.recv() == (OP_TEXT, b"hello all") and b.recv() == (OP_TEXT, b"hello all")
        b.close()
        deadline = time.time() + 5
        while ws.client_count() > 1 and time.time() < deadline:
            time.sleep(0.01)
        assert ws.client_count() == 1 and ws.broadcast("x") == 1
        big = "y" * 70000
        a.send(json.dumps({"prompt": big, "max_tokens": 1}))
        assert a.recv() == (OP_TEXT, b"x")
        assert a.recv()[1].decode() == big + "-0 "
    finally:
        ws.stop()
    assert not ws.is_running()


def test_result_codes(tmp_path):
    r, v = Result.wrap(open, str(tmp_path / "missing"))
    assert r.code == ErrorCode.FILE_NOT_FOUND and not r.ok() and v is None
    r, v = Result.wrap(int, "12")
    assert r.ok() and v == 12
    assert Result.wrap(int, "x")[0].code == ErrorCode.INVALID_ARGUMENT


def test_c_api_shaped_calls(tmp_path):
    import ctypes as C
    import torch
    from innova_b200.formats import export
    from innova_b200.models import DenseModel, PRESETS
    from innova_b200.serving import capi
    assert capi.oil_model_load(str(tmp_path / "missing.oil")) == 0 and "missing.oil" in capi.oil_last_error()
    assert capi.oil_generate(12345, "x", 4) is None and "invalid handle" in capi.oil_last_error()
    p = str(tmp_path / "m.oil")
    export.save_model(DenseModel(PRESETS["tiny"](), dtype=torch.float32, device="cpu", seed=1), p)
    h = capi.oil_model_load(p, device="cpu")
    assert h > 0 and capi.oil_last_error() == ""
    out = capi.oil_generate(h, "ab", 5)
    assert isinstance(out, str) and capi.oil_generate(h, "ab", 5) == out           # greedy by default: repeatable
    fns = capi.export_c_callbacks()
    ptr = fns["oil_generate"](h, b"ab", 5)
    assert C.string_at(ptr).decode("utf-8", "replace") == out
    capi.oil_free_string(out)
    capi.oil_model_free(h)
    assert capi.oil_generate(h, "ab", 5) is None
    assert b"invalid handle" in C.string_at(fns["oil_last_error"]())


def test_oversized_frame_is_refused_from_its_header_and_early_frames_survive_the_handshake():
    import socket
    import struct
    import time
    from innova_b200.serving.websocket import OP_CLOSE, OP_TEXT, WebSocketHandler, compute_accept_key, create_frame, parse_frame
    got = []
    ws = WebSocketHandler(0, max_message=1024)
    ws.on_message = got.append
    ws.start()
    try:
        # request head and the first frame in one packet: the frame must not be lost
        s = socket.create_connection(("127.0.0.1", ws.port), timeout=5)
        key = "dGhlIHNhbXBsZSBub25jZQ=="
        s.sendall((f"GET / HTTP/1.1\r\nHost: x\r\nUpgrade: websocket\r\nConnection: Upgrade\r\nSec-WebSocket-Key: {key}\r\n"
                   "Sec-WebSocket-Version: 13\r\n\r\n").encode() + create_frame("early", OP_TEXT, mask=b"abcd"))
        data = b""
        while b"\r\n\r\n" not in data:
            data += s.recv(4096)
        assert compute_accept_key(key).encode() in data
        for _ in range(100):
            if got:
                break
            time.sleep(0.02)
        assert got == ["early"]
        # a header that announces 2^40 bytes: closed with 1009 although no payload byte was sent
        s.sendall(bytes([0x81, 0x80 | 127]) + struct.pack(">Q", 1 << 40) + b"abcd")
        buf = data.split(b"\r\n\r\n", 1)[1]
        fr = None
        while fr is None:
            chunk = s.recv(4096)
            if not chunk:
                break
            buf += chunk
            fr = parse_frame(buf)
        assert fr is not None and fr[1] == OP_CLOSE and struct.unpack(">H", fr[0][:2])[0] == 1009
        s.close()
    finally:
        ws.stop()
