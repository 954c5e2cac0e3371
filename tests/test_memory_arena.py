"""Native arena (bump / stack), per-thread pools and strided views (CPU)."""
import threading

import pytest
import torch

from innova_b200.utils.memory import Buffer, MemoryPool, StackAllocator, TensorView, ThreadLocalPoolRegistry


def test_bump_pool_alignment_aliasing_and_limits():
    pool = MemoryPool(1 << 16)
    a = pool.allocate((10, 3), torch.float32, zero=True)
    b = pool.allocate((100,), torch.bfloat16)
    assert a.data_ptr() % 256 == 0 and b.data_ptr() % 256 == 0 and b.data_ptr() - a.data_ptr() == 256
    a.fill_(1.0); b.fill_(2.0)
    assert float(a.sum()) == 30.0 and pool.bytes_used == 256 + 200 and pool.allocations == 2
    c = pool.allocate((4,), torch.int64, alignment=4096)
    assert (c.data_ptr() - pool.buffer.data_ptr()) % 4096 == 0
    with pytest.raises(MemoryError):
        pool.allocate((1 << 16,), torch.uint8)
    assert pool.failures == 1 and pool.bytes_wasted == pool.capacity - pool.bytes_used
    peak = pool.peak_usage
    pool.reset()
    assert pool.bytes_used == 0 and pool.peak_usage == peak
    assert pool.allocate((10, 3), torch.float32).data_ptr() == a.data_ptr()          # the same block again after the reset


def test_stack_scopes():
    st = StackAllocator(1 << 14)
    base = st.allocate((64,), torch.float32)
    with st.scope():
        x = st.allocate((256,), torch.float32)
        with st.scope():
            st.allocate((256,), torch.float32)
            inner = st.bytes_used
        assert st.bytes_used < inner
    assert st.bytes_used == 256 and st.allocate((8,), torch.float32).data_ptr() == x.data_ptr()
    with pytest.raises(RuntimeError):
        st.pop()
    assert base.numel() == 64


def test_concurrent_allocations_do_not_overlap():
    pool = MemoryPool(1 << 20)
    got = []

    def work():
        mine = [pool.allocate_bytes(300) for _ in range(200)]
        got.extend(mine)
    ts = [threading.Thread(target=work) for _ in range(8)]
    [t.start() for t in ts]; [t.join() for t in ts]
    offs = sorted(got)
    assert len(offs) == 1600 and all(b - a >= 300 for a, b in zip(offs, offs[1:])) and all(o % 256 == 0 for o in offs)


def test_thread_local_registry_and_buffer():
    reg = ThreadLocalPoolRegistry(1 << 12)
    ptrs = {}

    def work(i):
        ptrs[i] = reg.get().allocate((16,), torch.float32).data_ptr()
        assert reg.get() is reg.get()
    ts = [threading.Thread(target=work, args=(i,)) for i in range(3)]
    [t.start() for t in ts]; [t.join() for t in ts]
    assert len(set(ptrs.values())) == 3 and reg.total_used() == 3 * 64
    reg.reset_all()
    assert reg.total_used() == 0
    buf = Buffer(1000, alignment=512)
    assert buf.data_ptr() % 512 == 0 and buf.nbytes == 1000 and buf.view(torch.float32, (5, 5), 64).shape == (5, 5)


def test_tensor_view():
    base = torch.arange(24.0)
    v = TensorView(base, (2, 3, 4))
    assert v.shape == (2, 3, 4) and v.strides == (12, 4, 1) and v.is_contiguous()
    s = v.slice(1, 1, 3).transpose(0, 2)
    assert s.shape == (4, 2, 2) and not s.is_contiguous()
    assert torch.equal(s.materialize(), base.view(2, 3, 4)[:, 1:3].transpose(0, 2))
    s.tensor[0, 0, 0] = -1.0
    assert base[4] == -1.0                                   # a view, not a copy


@pytest.mark.gpu
def test_device_pool_feeds_kernels():
    from innova_b200 import ops
    pool = StackAllocator(64 << 20, device="cuda")
    with pool.scope():
        x = pool.allocate((256, 512), torch.bfloat16)
        w = pool.allocate((384, 512), torch.bfloat16)
        x.normal_(); w.normal_()
        y = ops.linear(x, w)
        assert x.is_cuda and x.data_ptr() % 256 == 0
        assert (y.float() - x.float() @ w.float().t()).abs().max() < 0.5
    assert pool.bytes_used == 0 and pool.peak_usage >= (256 + 384) * 512 * 2


def test_canary_guard_detects_out_of_range_writes():
    from innova_b200.parallel.symm import CanaryGuard
    n = 1000 * 4
    g = CanaryGuard(torch.zeros(CanaryGuard.total_bytes(n), dtype=torch.uint8), n)
    x = g.view(torch.float32, 10, 100)
    x.fill_(3.0)
    assert g.damage() is None and g.payload_offset == 256
    g.check("staging")
    g.storage[256 + n + 5] = 0                      # one byte past the payload
    assert g.damage() == ("back", 5)
    with pytest.raises(RuntimeError, match="back guard damaged at byte 5"):
        g.check("staging")
    g.arm()
    g.storage[255] = 1
    assert g.damage() == ("front", 255) and float(x.sum()) == 3000.0
