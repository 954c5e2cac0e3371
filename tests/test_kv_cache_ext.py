"""KV-cache variants: contiguous (+int8), hierarchical paging with LRU spill, OIL4 with per-block codebooks."""
import torch

from innova_b200.inference import kv_cache_ext as K


def test_contiguous_cache_plain_and_int8():
    for q8 in (False, True):
        c = K.KVCache(2, 32, 4, 64, quantize_int8=q8)
        k, v = torch.randn(4, 5, 64), torch.randn(4, 5, 64)
        c.append(0, k, v)
        c.append(0, k[:, :2], v[:, :2])
        kk, vv = c.get(0)
        assert kk.shape == (4, 7, 64)
        tol = 0.05 if q8 else 0.0
        assert (kk[:, :5] - k).abs().max() <= tol and (vv[:, 5:] - v[:, :2]).abs().max() <= tol
        c.resize(3)
        assert c.get(0)[0].shape[1] == 3
    assert K.KVCache(2, 32, 4, 64, quantize_int8=True).nbytes() < 0.3 * K.KVCache(2, 32, 4, 64).nbytes()
    q, s = K.int8_block_quant(torch.randn(130))
    assert q.shape == (3, 64) and (K.int8_block_dequant(q, s, 130).numel() == 130)


def test_hierarchical_paging_spills_and_reloads(tmp_path):
    L, H, D = 2, 2, 8
    block_bytes = 2 * L * H * 16 * D * 4
    for make in (K.PagedKVCache4M, K.PagedKVCache1T):
        c = make(L, H, D, max_physical_bytes=3 * block_bytes, disk_path=str(tmp_path / make.__name__))
        assert c.slots == 3
        torch.manual_seed(0)
        k, v = torch.randn(L, H, 100, D), torch.randn(L, H, 100, D)
        c.append(k[:, :, :37], v[:, :, :37])
        c.append(k[:, :, 37:], v[:, :, 37:])          # 7 blocks through 3 slots: the early ones spill to disk
        st = c.stats()
        assert st["evictions"] >= 4 and st["resident_blocks"] == 3
        kk, vv = c.read(0, 100)                       # touching spilled blocks reloads them
        assert torch.equal(kk, k) and torch.equal(vv, v)
        assert c.stats()["reloads"] >= 4
        kk2, _ = c.read(90, 100)
        assert torch.equal(kk2, k[:, :, 90:100])
    assert K.PagedKVCache4M(1, 1, 8, 1 << 20).max_tokens() == 4096 * 4096 * 16
    assert K.PagedKVCache1T(1, 1, 8, 1 << 20).max_tokens() == 4096 ** 3 * 16


def test_oil4_kv_cache_per_block_codebook():
    c = K.OIL4KVCache(64)
    x = torch.randn(64 * 20) * torch.repeat_interleave(torch.rand(20) * 3 + 0.1, 64)
    c.append(x)
    y = c.read()
    rel = (y - x).norm() / x.norm()
    assert rel < 0.15 and c.nbytes() == 20 * (32 + 32)
