"""Device-resident data out of range, and the give-up path of the bounded waits - all without a fault or a
hang: the kernels clamp, skip and report through the device status word, and the one wait that is made to
run out is a self-test kernel's wait on a barrier that nothing arrives at."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as CO
from oracle import dflash_oracle as O

pytestmark = pytest.mark.gpu


def K():
    from swiftlm_b200 import kernels
    return kernels


def dev(x, dt=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if dt is None else t.to(dt)


def test_bounded_wait_gives_up_reports_and_the_context_stays_usable():
    from swiftlm_b200 import _lib
    L = _lib.lib()
    assert L.dflash_device_status(None) == 0
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert L.dflash_selftest_bounded_wait(300, flag.data_ptr(), None) == 0
    torch.cuda.synchronize()                                  # the kernel returned by itself
    assert int(flag.item()) == 1                              # the second warp left through the abort flag
    assert L.dflash_device_status(None) == _lib.ERR_DEVICE_TIMEOUT
    assert b"bounded wait" in L.dflash_last_error_string()
    assert L.dflash_device_status(None) == 0                  # reading clears the word
    # the context is intact: a real kernel runs and is right
    x = O.make_sdpa_inputs(2, 16, 2, 16 + 300, 256, 4100, "bf16")
    out = K().batched_sdpa_2pass(dev(x["q"], torch.bfloat16), dev(x["k"], torch.bfloat16), dev(x["v"], torch.bfloat16), float(x["scale"]))
    torch.cuda.synchronize()
    K().device_status()
    assert np.abs(out.float().cpu().numpy() - CO.verify_sdpa(x["q"], x["k"], x["v"], float(x["scale"]))).max() < 2e-2
    assert L.dflash_selftest_bounded_wait(0, None, None) == _lib.ERR_INVALID_ARG


def _paged(x, lens_true, pt, spare=2, seed=3):
    B, Hkv, N, D = x["k"].shape
    pages = (N + pt - 1) // pt
    rng = np.random.default_rng(seed)
    pool = B * pages + spare
    table = rng.permutation(pool)[:B * pages].reshape(B, pages).astype(np.int32)
    kp = np.zeros((pool, Hkv, pt, D), np.float32)
    vp = np.zeros_like(kp)
    for b in range(B):
        for pg in range(pages):
            lo, hi = pg * pt, min(N, (pg + 1) * pt)
            kp[table[b, pg], :, :hi - lo] = x["k"][b, :, lo:hi]
            vp[table[b, pg], :, :hi - lo] = x["v"][b, :, lo:hi]
    return kp, vp, table


def test_lengths_beyond_n_are_clamped_and_reported():
    """kv_len_per_seq lives on the device, so the host cannot vet it: an entry beyond N (here far beyond the page
    table's reach) must neither index the table out of bounds nor load outside the pool.  The kernel clamps it to N,
    computes the attention over N keys and raises the status word."""
    from swiftlm_b200 import _lib
    B, Hq, Hkv, D, pt = 3, 16, 2, 256, 128
    N = 16 + 600
    x = O.make_sdpa_inputs(B, Hq, Hkv, N, D, 4200, "bf16")
    kp, vp, table = _paged(x, None, pt)
    dt = torch.bfloat16
    good = np.array([N, 16 + 100, N], np.int32)
    bad = np.array([N + 100000, 16 + 100, 2 ** 30], np.int32)
    want = K().batched_sdpa_2pass(dev(x["q"], dt), dev(kp, dt), dev(vp, dt), float(x["scale"]), kv_len=good, page_table=dev(table), n_max=N)
    torch.cuda.synchronize()
    K().device_status()
    got = K().batched_sdpa_2pass(dev(x["q"], dt), dev(kp, dt), dev(vp, dt), float(x["scale"]), kv_len=bad, page_table=dev(table), n_max=N)
    torch.cuda.synchronize()
    with pytest.raises(_lib.DFlashError) as e:
        K().device_status()
    assert e.value.status == _lib.ERR_DEVICE_DATA and "kv_len_per_seq" in str(e.value)
    assert torch.equal(got, want)
    K().device_status()                                       # cleared


def test_non_positive_lengths_are_skipped_and_reported():
    from swiftlm_b200 import _lib
    B, Hq, Hkv, D = 4, 16, 2, 256
    N = 16 + 300
    x = O.make_sdpa_inputs(B, Hq, Hkv, N, D, 4201, "bf16")
    dt = torch.bfloat16
    lens = np.array([N, 0, -7, 16 + 40], np.int32)
    out = torch.full((B, Hq, 16, D), 7.0, dtype=dt, device="cuda")
    K().batched_sdpa_2pass(dev(x["q"], dt), dev(x["k"], dt), dev(x["v"], dt), float(x["scale"]), kv_len=lens, out=out)
    torch.cuda.synchronize()
    with pytest.raises(_lib.DFlashError) as e:
        K().device_status()
    assert e.value.status == _lib.ERR_DEVICE_DATA
    want = CO.verify_sdpa(x["q"], x["k"], x["v"], float(x["scale"]), kv_len=np.array([N, 16, 16, 16 + 40], np.int32))
    o = out.float().cpu().numpy()
    assert np.abs(o[[0, 3]] - want[[0, 3]]).max() < 2e-2      # the sequences with keys are right
    assert (o[[1, 2]] == 7.0).all()                           # the ones without keys were passed over


def test_page_ids_outside_the_pool_read_as_zeros_and_are_reported():
    """A stale page-table entry (negative, or at/after the pool's end) must not turn into a load outside the pool:
    the page reads as zero keys and values and the status word says so."""
    from swiftlm_b200 import _lib
    B, Hq, Hkv, D, pt = 2, 16, 2, 256, 128
    N = 16 + 496                                             # 4 pages per sequence
    x = O.make_sdpa_inputs(B, Hq, Hkv, N, D, 4202, "bf16")
    kp, vp, table = _paged(x, None, pt)
    dt = torch.bfloat16
    lens = np.full((B,), N, np.int32)
    for bad_id in (-1, kp.shape[0], 2 ** 30):
        t2 = table.copy()
        t2[1, 1] = bad_id
        got = K().batched_sdpa_2pass(dev(x["q"], dt), dev(kp, dt), dev(vp, dt), float(x["scale"]), kv_len=lens, page_table=dev(t2), n_max=N)
        torch.cuda.synchronize()
        with pytest.raises(_lib.DFlashError) as e:
            K().device_status()
        assert e.value.status == _lib.ERR_DEVICE_DATA
        # the oracle over the same keys with that page zeroed
        y = {k_: (v_.copy() if hasattr(v_, "copy") else v_) for k_, v_ in x.items()}
        y["k"][1, :, pt:2 * pt] = 0
        y["v"][1, :, pt:2 * pt] = 0
        want = CO.verify_sdpa(y["q"], y["k"], y["v"], float(y["scale"]))
        assert np.abs(got.float().cpu().numpy() - want).max() < 2e-2


def test_kv_append_never_hands_out_a_length_past_the_capacity():
    from swiftlm_b200 import _lib
    B, Hkv, T, D, cap = 2, 2, 16, 128, 40
    dt = torch.bfloat16
    k_new = torch.randn(B, Hkv, T, D, device="cuda").to(dt)
    cache_k = torch.zeros(B, Hkv, cap, D, dtype=dt, device="cuda")
    cache_v = torch.zeros_like(cache_k)
    lens = torch.tensor([10, 30], dtype=torch.int32, device="cuda")     # the second block does not fit
    out_len = torch.zeros(B, dtype=torch.int32, device="cuda")
    K().kv_append(k_new, k_new, cache_k, cache_v, kv_len=lens, kv_len_out=out_len)
    torch.cuda.synchronize()
    with pytest.raises(_lib.DFlashError) as e:
        K().device_status()
    assert e.value.status == _lib.ERR_DEVICE_DATA
    assert out_len.tolist() == [26, 40]
    assert torch.equal(cache_k[1, :, 30:40], k_new[1, :, :10])
