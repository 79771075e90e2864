"""KV append / trim on the device and the paged cache around the verify attention, against the oracle's
growing-array cache (append in the target forward, trim to the accepted prefix)."""
import numpy as np
import pytest
import torch

from oracle import dflash_oracle as O

pytestmark = pytest.mark.gpu
ATOL = 2e-2


def K():
    from swiftlm_b200 import kernels
    return kernels


def cache_cls():
    from swiftlm_b200.kv_cache import PagedKVCache
    return PagedKVCache


def bf16(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda().to(torch.bfloat16)


def rounded(x):
    return torch.from_numpy(x).to(torch.bfloat16).float().numpy()


@pytest.mark.parametrize("page_tokens", [128, 256])
def test_paged_cycles_match_the_growing_array(page_tokens):
    B, Hq, Hkv, D, T = 5, 16, 2, 256, 16
    rng = np.random.default_rng(40 + page_tokens)
    cache = cache_cls()(B, Hkv, D, page_tokens, num_pages=B * 4, max_pages=5)
    ref = O.TrimmableKVCache(B, Hkv, D)
    # prefill of different lengths per sequence (one of them empty)
    P = 200
    lens0 = np.array([200, 0, 37, 129, 64], np.int32)
    kp, vp = rounded(rng.standard_normal((B, Hkv, P, D), np.float32)), rounded(rng.standard_normal((B, Hkv, P, D), np.float32))
    cache.extend(bf16(kp), bf16(vp), lens0)
    ref.update(kp, vp)
    ref.restore(np.zeros(B), lens0)
    scale = 1.0 / 16
    for cycle in range(12):
        kn, vn = rounded(rng.standard_normal((B, Hkv, T, D), np.float32)), rounded(rng.standard_normal((B, Hkv, T, D), np.float32))
        q = rounded(rng.standard_normal((B, Hq, T, D), np.float32))
        start = np.array([ref.offset(b) for b in range(B)])
        lens_blk = cache.append_block(bf16(kn), bf16(vn))
        ref.update(kn, vn)
        np.testing.assert_array_equal(lens_blk.cpu().numpy(), start + T)
        out = cache.attend(bf16(q), scale)
        torch.cuda.synchronize()
        K().device_status()
        for b in range(B):
            want = O.verify_sdpa(q[b:b + 1], ref.k[b][None], ref.v[b][None], scale)
            assert np.abs(out[b:b + 1].float().cpu().numpy() - want).max() < ATOL
        commit = rng.integers(1, T + 1, B).astype(np.int32)           # accepted drafts + 1
        if cycle == 3:
            commit[:] = T                                            # a fully accepted block
        cache.commit(torch.from_numpy(commit).cuda())
        ref.restore(start, commit)
        if cycle % 4 == 1:
            np.testing.assert_array_equal(cache.sync(), [ref.offset(b) for b in range(B)])
    lens = cache.sync()
    for b in range(B):
        assert lens[b] == ref.offset(b)
        k, v = cache.gather(b)
        np.testing.assert_array_equal(k.float().cpu().numpy(), ref.k[b])    # byte movement: exact
        np.testing.assert_array_equal(v.float().cpu().numpy(), ref.v[b])
        assert len(cache.pages_of(b)) == -(-int(lens[b]) // page_tokens)   # unreachable pages went back to the pool
    assert cache.free_pages + sum(len(cache.pages_of(b)) for b in range(B)) == cache.num_pages
    used = [p for b in range(B) for p in cache.pages_of(b)]
    assert len(set(used)) == len(used)                                     # no page belongs to two sequences


def test_dense_cache_append_and_commit():
    B, Hkv, D, T, cap = 3, 2, 128, 16, 96
    rng = np.random.default_rng(7)
    kc = torch.zeros(B, Hkv, cap, D, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    kv_len = torch.tensor([0, 5, 40], dtype=torch.int32, device="cuda")
    out_len = torch.zeros_like(kv_len)
    kn = torch.from_numpy(rng.standard_normal((B, Hkv, T, D), np.float32)).cuda().half()
    vn = torch.from_numpy(rng.standard_normal((B, Hkv, T, D), np.float32)).cuda().half()
    K().kv_append(kn, vn, kc, vc, kv_len=kv_len, kv_len_out=out_len)
    assert out_len.tolist() == [16, 21, 56]
    for b, n in enumerate([0, 5, 40]):
        assert torch.equal(kc[b, :, n:n + T], kn[b]) and torch.equal(vc[b, :, n:n + T], vn[b])
        assert not kc[b, :, :n].any() and not kc[b, :, n + T:].any()
    K().kv_commit(kv_len, torch.tensor([1, 16, 99], dtype=torch.int32, device="cuda"))    # clamped to the block
    assert kv_len.tolist() == [1, 21, 56]
    # one length for the whole batch (no device array), fp32 rows
    kc32 = torch.zeros(B, Hkv, cap, D, device="cuda")
    vc32 = torch.zeros_like(kc32)
    K().kv_append(kn.float(), vn.float(), kc32, vc32, len_all=80)
    assert torch.equal(kc32[:, :, 80:96], kn.float()) and not kc32[:, :, :80].any()
    K().device_status()


def test_overflow_is_reported_not_written():
    from swiftlm_b200 import _lib
    B, Hkv, D, T, cap = 2, 1, 128, 16, 32
    kc = torch.zeros(B, Hkv, cap, D, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    kn = torch.ones(B, Hkv, T, D, dtype=torch.bfloat16, device="cuda")
    kv_len = torch.tensor([16, 24], dtype=torch.int32, device="cuda")      # sequence 1 has room for 8 of the 16 rows
    K().kv_append(kn, kn, kc, vc, kv_len=kv_len)
    torch.cuda.synchronize()
    with pytest.raises(_lib.DFlashError) as e:
        K().device_status()
    assert e.value.status == _lib.ERR_DEVICE_DATA
    assert kc[0, :, 16:32].all() and kc[1, :, 24:32].all() and not kc[1, :, :24].any()
    K().device_status()                                                     # the flag was cleared; the library stays usable
    # an unmapped page of a paged pool is reported the same way
    pool = torch.zeros(4, Hkv, 16, D, dtype=torch.bfloat16, device="cuda")
    table = torch.tensor([[0, -1], [1, 7]], dtype=torch.int32, device="cuda")
    K().kv_append(kn, kn, pool, torch.zeros_like(pool), kv_len=torch.tensor([8, 8], dtype=torch.int32, device="cuda"), page_table=table)
    torch.cuda.synchronize()
    with pytest.raises(_lib.DFlashError):
        K().device_status()
    assert pool[0, :, 8:].all() and pool[1, :, 8:].all() and not pool[2:].any()


def test_pool_exhaustion_and_release():
    from swiftlm_b200.kv_cache import KVCacheFull
    cache = cache_cls()(2, 1, 128, 16, num_pages=3, max_pages=4)
    kn = torch.ones(2, 1, 16, 128, dtype=torch.bfloat16, device="cuda")
    cache.append_block(kn, kn)
    cache.commit(torch.tensor([16, 16], dtype=torch.int32, device="cuda"))
    with pytest.raises(KVCacheFull):
        cache.append_block(kn, kn)                                          # needs 4 pages, the pool has 3
    cache.release(1)
    assert cache.free_pages == 1 and cache.kv_len.tolist() == [16, 0]    # sequence 0 kept the page it got before the pool ran dry
    cache.append_block(kn, kn)
    cache.commit(torch.tensor([3, 0], dtype=torch.int32, device="cuda"))
    assert cache.sync().tolist() == [19, 0]
    assert len(cache.pages_of(0)) == 2 and len(cache.pages_of(1)) == 0
