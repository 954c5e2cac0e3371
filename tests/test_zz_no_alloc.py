"""The no-allocation norm backward, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at the point of the call: they are
inside a stream capture, or inside a serving loop with a fixed memory budget, or they are a plugin
in another framework's pool. ``inv_norm_bwd_noalloc`` serves them from a static device array. This
test drives the symbol directly with ctypes (no Python wrapper in between) and checks it against
the regular entry point, twice in a row, because the static array keeps the previous call's data.
The file sorts last so that a run that stops at the first failure has already run everything else.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from innova_b200 import _native
    lib = _native.cuda()
    fn = lib.inv_norm_bwd_noalloc
    fn.argtypes = [C.c_void_p] * 9 + [C.c_int, C.c_int, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    return lib, fn


def _case(T, D, rms, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    dev = torch.device("cuda", 0)
    x = torch.randn(T, D, device=dev, generator=g).bfloat16()
    dy = torch.randn(T, D, device=dev, generator=g).bfloat16()
    gamma = (1 + 0.1 * torch.randn(D, device=dev, generator=g)).bfloat16()
    xf = x.float()
    if rms:
        mean = torch.zeros(T, device=dev)
        rstd = torch.rsqrt(xf.pow(2).mean(-1) + 1e-5)
    else:
        mean = xf.mean(-1)
        rstd = torch.rsqrt(xf.var(-1, unbiased=False) + 1e-5)
    return x, dy, gamma, mean.contiguous(), rstd.contiguous()


@pytest.mark.parametrize("rms", [0, 1])
def test_noalloc_matches_regular_entry_point_twice(rms):
    lib, noalloc = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row with different shapes: the second one finds the first one's partial sums
    for T, D, seed in [(4096, 768, 1), (777, 2048, 2)]:
        x, dy, gamma, mean, rstd = _case(T, D, rms, seed)
        dx_ref = torch.empty_like(x)
        dg_ref = torch.zeros(D, device=dev)
        db_ref = torch.zeros(D, device=dev)
        grid = lib.inv_norm_bwd_grid(T)
        scratch = torch.empty(grid * 2 * D, device=dev)
        rc = lib.inv_norm_bwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(), 0, dx_ref.data_ptr(),
                              dg_ref.data_ptr(), db_ref.data_ptr(), scratch.data_ptr(), T, D, rms, stream)
        assert rc == 0
        dx = torch.empty_like(x)
        dg = torch.zeros(D, device=dev)
        db = torch.zeros(D, device=dev)
        before = torch.cuda.memory_allocated()
        rc = noalloc(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), dg.data_ptr(),
                     db.data_ptr(), T, D, rms, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        # The caching allocator's counter cannot see a cudaMalloc made inside the library, the driver's free-byte count
        # can. The call above has loaded every kernel this shape uses (module loading is lazy and may take memory once),
        # so a repeat of the same call must leave the device's free memory exactly where it was.
        free_before = torch.cuda.mem_get_info(dev)[0]
        dg.zero_()
        db.zero_()
        rc = noalloc(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), dg.data_ptr(),
                     db.data_ptr(), T, D, rms, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_before
        tol = 2e-2
        assert float((dx.float() - dx_ref.float()).norm() / (dx_ref.float().norm() + 1e-12)) < tol
        assert float((dg - dg_ref).norm() / (dg_ref.norm() + 1e-12)) < tol
        if not rms:
            assert float((db - db_ref).norm() / (db_ref.norm() + 1e-12)) < tol


def test_noalloc_rejects_rows_wider_than_the_static_scratch():
    _, noalloc = _lib()
    dev = torch.device("cuda", 0)
    t = torch.zeros(8, 4096, device=dev, dtype=torch.bfloat16)
    f = torch.zeros(4096, device=dev)
    rc = noalloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), f.data_ptr(), f.data_ptr(), None, t.data_ptr(), f.data_ptr(), f.data_ptr(), 8, 4096,
                 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -7
    rc = noalloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), f.data_ptr(), f.data_ptr(), None, t.data_ptr(), f.data_ptr(), f.data_ptr(), 8, 100,
                 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -7
