"""TCPCommBackend between two endpoints on 127.0.0.1."""
import time

import torch

from innova_b200.parallel.tcp_backend import TCPCommBackend


def _pair():
    a, b = TCPCommBackend(), TCPCommBackend()
    assert a.listen(0, "127.0.0.1") and a.port > 0
    nb = b.connect("127.0.0.1", a.port)
    assert nb >= 0
    for _ in range(200):
        if a.nodes():
            break
        time.sleep(0.01)
    return a, b, a.nodes()[0], nb


def test_bytes_tensors_async_and_counters():
    a, b, na, nb = _pair()
    try:
        assert b.send(nb, b"hello world") and a.recv(na, 11) == b"hello world"
        big = torch.randn(300, 1000)
        for t in (big, torch.arange(7, dtype=torch.int64), torch.randn(4, 3).bfloat16(), torch.tensor(2.5), torch.empty(0, 5)):
            assert b.send_tensor(nb, t)
            got = a.recv_tensor(na)
            assert got.dtype == t.dtype and got.shape == t.shape and torch.equal(got, t)
        # both directions at once, asynchronously: neither side blocks the other
        x, y = torch.randn(1 << 18), torch.randn(1 << 18)
        fa = a.recv_async(na, x.numel() * 4)
        fb = b.recv_async(nb, y.numel() * 4)
        a.send_async(na, y.numpy().tobytes())
        b.send_async(nb, x.numpy().tobytes())
        a.wait_all()
        b.wait_all()
        assert fa.result() == x.numpy().tobytes() and fb.result() == y.numpy().tobytes()
        assert b.bytes_sent(nb) > big.numel() * 4 and a.bytes_received(na) == b.bytes_sent(nb)
        assert a.is_connected(na) and b.is_connected(nb)
    finally:
        a.shutdown()
        b.shutdown()


def test_peer_loss_is_reported_not_raised():
    a, b, na, nb = _pair()
    try:
        b.disconnect(nb)
        assert not b.is_connected(nb) and not b.send(nb, b"x")
        assert a.recv(na, 4) is None and not a.is_connected(na)           # the peer closed: nothing arrives, the link is marked down
        assert a.recv_tensor(na) is None and not a.send(na, b"y")
        assert b.connect("127.0.0.1", 1) == -1                             # nothing listens there
        assert a.send_async(na, b"z").result() is False and a.recv_async(na, 1).result() is None
    finally:
        a.shutdown()
        b.shutdown()
    assert a.nodes() == [] and not a.listen(-5, "127.0.0.1")
