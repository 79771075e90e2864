"""The allocation-free attention entry point against the regular one, through the C ABI.

dflash_verify_sdpa_noalloc is for hosts that cannot hand the library a workspace (fixed memory
budget, allocator closed to plug-ins, request paths that must not reach cudaMalloc); its
split-KV partials live in a device array inside the library.  That array is shared by all calls
and keeps the previous call's contents, so the check runs two different problems back to back
and compares each with dflash_verify_sdpa given a caller-allocated workspace.  Collected last
(file name) so a failure here cannot hide another test's result."""
import numpy as np
import pytest
import torch

from oracle import dflash_oracle as O

pytestmark = pytest.mark.gpu
ATOL = 2e-2   # the tolerance of tests/test_gpu_sdpa.py


def _both(L, _lib, x, kv_len=None):
    dt = torch.bfloat16
    q = torch.from_numpy(x["q"]).cuda().to(dt)
    k = torch.from_numpy(x["k"]).cuda().to(dt)
    v = torch.from_numpy(x["v"]).cuda().to(dt)
    B, Hq, T, D = q.shape
    Hkv, N = k.shape[1], k.shape[2]
    lens = None if kv_len is None else torch.tensor(kv_len, dtype=torch.int32, device="cuda")
    lp = None if lens is None else lens.data_ptr()
    ws = torch.empty(L.dflash_verify_sdpa_workspace_bytes(B, Hq, Hkv, D, N), dtype=torch.uint8, device="cuda")
    ref = torch.empty_like(q)
    got = torch.full_like(q, float("nan"))
    scale = float(x["scale"])
    st = L.dflash_verify_sdpa(q.data_ptr(), k.data_ptr(), v.data_ptr(), None, lp, None, ref.data_ptr(), ws.data_ptr(),
                              ws.numel(), B, Hq, Hkv, T, D, N, 0, 0, 0, scale, _lib.BF16, _lib.KV_DENSE, None)
    assert st == 0, L.dflash_last_error_string()
    st = L.dflash_verify_sdpa_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), None, lp, None, got.data_ptr(),
                                      B, Hq, Hkv, T, D, N, 0, 0, 0, scale, _lib.BF16, _lib.KV_DENSE, None)
    assert st == 0, L.dflash_last_error_string()
    torch.cuda.synchronize()
    assert L.dflash_device_status(None) == 0
    return got.float().cpu().numpy(), ref.float().cpu().numpy()


def test_noalloc_entry_matches_workspace_entry_on_two_calls_in_a_row():
    from swiftlm_b200 import _lib
    L = _lib.lib()
    # first problem: many tiles per unit, every CTA leaves partials in the built-in array
    a = O.make_sdpa_inputs(4, 16, 2, 16 + 3000, 256, 7001, "bf16")
    got, ref = _both(L, _lib, a)
    assert np.isfinite(got).all() and np.abs(got - ref).max() < ATOL
    # second problem right after: other shape, ragged lengths, fewer CTAs, stale partials around
    b = O.make_sdpa_inputs(3, 8, 2, 16 + 500, 128, 7002, "bf16")
    got, ref = _both(L, _lib, b, kv_len=[516, 16, 300])
    assert np.isfinite(got).all() and np.abs(got - ref).max() < ATOL
    # and the first one again: same answer as before
    got2, ref2 = _both(L, _lib, a)
    assert np.abs(got2 - ref2).max() < ATOL


def test_noalloc_entry_validates_like_the_regular_one():
    from swiftlm_b200 import _lib
    L = _lib.lib()
    q = torch.zeros(1, 16, 16, 64, dtype=torch.bfloat16, device="cuda")
    st = L.dflash_verify_sdpa_noalloc(q.data_ptr(), q.data_ptr(), q.data_ptr(), None, None, None, q.data_ptr(),
                                      1, 16, 2, 16, 64, 64, 0, 0, 0, 0.1, _lib.BF16, _lib.KV_DENSE, None)
    assert st == _lib.ERR_UNSUPPORTED      # head_dim 64 is outside the supported set
    st = L.dflash_verify_sdpa_noalloc(None, None, None, None, None, None, None, 0, 16, 2, 16, 256, 64, 0, 0, 0, 0.1,
                                      _lib.BF16, _lib.KV_DENSE, None)
    assert st == _lib.ERR_INVALID_ARG


def test_noalloc_entry_refuses_compressed_kv_before_any_launch():
    """KV in the compressed format is expanded into scratch by the regular entry (B*Hkv*N*D*4 bytes), which the
    built-in array cannot hold: the no-alloc entry refuses the format up front, launches nothing and leaves
    the device status clean.  (Its DFLASH_ERR_WORKSPACE answer needs a GPU with more than 158 SMs to show:
    on 148 SMs every dense or paged call fits the array.)"""
    import ctypes as C

    from swiftlm_b200 import _lib
    L = _lib.lib()
    B, Hq, Hkv, D, N = 4, 16, 2, 256, 64
    q = torch.zeros(B, Hq, 16, D, dtype=torch.bfloat16, device="cuda")
    desc = _lib.TurboKV()   # never read: the format is refused first
    launches = L.dflash_launch_count()
    st = L.dflash_verify_sdpa_noalloc(q.data_ptr(), C.cast(C.pointer(desc), C.c_void_p), None, None, None, None, q.data_ptr(),
                                      B, Hq, Hkv, 16, D, N, 0, 0, 0, 0.0625, _lib.BF16, _lib.KV_TURBO3, None)
    assert st == _lib.ERR_UNSUPPORTED and b"TurboQuant" in L.dflash_last_error_string()
    assert L.dflash_launch_count() == launches
    assert L.dflash_device_status(None) == 0
