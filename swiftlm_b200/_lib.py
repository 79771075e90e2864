"""ctypes binding of libdflash_cuda.so (the C ABI declared in include/dflash_cuda.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# DFLASH_CUDA_LIB points at a library built elsewhere (for instance an instrumented build)
LIB_PATH = os.environ.get("DFLASH_CUDA_LIB") or os.path.join(_PKG, "lib", "libdflash_cuda.so")

F32, BF16, F16, U8 = 0, 1, 2, 3
KV_DENSE, KV_TURBO3 = 0, 1
OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_WORKSPACE, ERR_DEVICE_TIMEOUT, ERR_DEVICE_DATA = 0, -1, -2, -3, -4, -5, -6

_vp, _i32, _u64, _sz, _f32 = C.c_void_p, C.c_int32, C.c_uint64, C.c_size_t, C.c_float

# name -> (restype, argtypes); must list every symbol include/dflash_cuda.h declares
SIGNATURES = {
    "dflash_gated_delta_tape": (_i32, [_vp] * 11 + [_i32] * 9 + [_vp]),
    "dflash_tape_replay": (_i32, [_vp] * 7 + [_i32] * 9 + [_vp]),
    "dflash_verify_sdpa": (_i32, [_vp] * 8 + [_sz] + [_i32] * 9 + [_f32, _i32, _i32, _vp]),
    "dflash_verify_sdpa_workspace_bytes_ex": (_sz, [_i32] * 6),
    "dflash_verify_sdpa_workspace_bytes": (_sz, [_i32] * 5),
    "dflash_verify_sdpa_turbo_workspace_bytes": (_sz, [_i32] * 6),
    "dflash_verify_sdpa_noalloc": (_i32, [_vp] * 7 + [_i32] * 9 + [_f32, _i32, _i32, _vp]),
    "dflash_greedy_tokens": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "dflash_accept_lengths": (_i32, [_vp] * 5 + [_i32, _i32, _vp]),
    "dflash_gather_logits_rows": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "dflash_rebuild_conv_state": (_i32, [_vp, _vp, _vp, _i32, _vp, _i32, _i32, _i32, C.c_int64, C.POINTER(_i32), _vp]),
    "dflash_kv_append": (_i32, [_vp] * 6 + [_i32, _vp] + [_i32] * 9 + [_vp]),
    "dflash_kv_commit": (_i32, [_vp, _vp, _i32, _i32, _vp]),
    "dflash_turbo_encode": (_i32, [_vp] * 5 + [C.c_int64, _i32, _i32, _vp]),
    "dflash_turbo_decode": (_i32, [_vp] * 5 + [C.c_int64, _i32, _i32, _vp]),
    "dflash_verify_step_workspace_bytes": (_sz, [_vp]),
    "dflash_verify_step": (_i32, [_vp, _vp, _sz, _vp]),
    "dflash_partition_plan": (_i32, [_i32, _i32, C.POINTER(_i32)]),
    "dflash_device_status": (_i32, [_vp]),
    "dflash_selftest_bounded_wait": (_i32, [C.c_uint32, _vp, _vp]),
    "dflash_device_count": (_i32, []),
    "dflash_last_error_string": (C.c_char_p, []),
    "dflash_launch_count": (_u64, []),
    "dflash_version": (C.c_char_p, []),
}


class TurboKV(C.Structure):
    """dflash_turbo_kv of include/dflash_cuda.h."""
    _fields_ = [("k_packed", C.c_void_p), ("k_signs", C.c_void_p), ("k_norm", C.c_void_p), ("k_rnorm", C.c_void_p),
                ("v_packed", C.c_void_p), ("v_norm", C.c_void_p), ("k_hot", C.c_void_p), ("v_hot", C.c_void_p),
                ("n_cold", C.c_int32), ("n_hot", C.c_int32)]


class VerifyStepDesc(C.Structure):
    """dflash_verify_step_desc of include/dflash_cuda.h (field order and types must match the header)."""
    _fields_ = [("B", C.c_int32), ("T", C.c_int32),
                ("gdn_layers", C.c_int32), ("Hk", C.c_int32), ("Hv", C.c_int32), ("Dk", C.c_int32), ("Dv", C.c_int32),
                ("g_is_vector", C.c_int32), ("in_dtype", C.c_int32),
                ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("g", C.c_void_p), ("beta", C.c_void_p),
                ("state", C.c_void_p), ("y", C.c_void_p), ("state_verify", C.c_void_p), ("tape", C.c_void_p),
                ("state_rolled", C.c_void_p),
                ("conv_snapshot", C.c_void_p), ("qkv", C.c_void_p), ("conv_out", C.c_void_p),
                ("conv_keep", C.c_int32), ("conv_row_bytes", C.c_int64),
                ("attn_layers", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32), ("N", C.c_int32),
                ("attn_dtype", C.c_int32), ("kv_format", C.c_int32),
                ("attn_q", C.c_void_p), ("attn_k", C.c_void_p), ("attn_v", C.c_void_p), ("attn_out", C.c_void_p),
                ("scale", C.c_float),
                ("logits", C.c_void_p), ("suppress", C.c_void_p), ("verify_ids", C.c_void_p),
                ("V", C.c_int32), ("logits_dtype", C.c_int32),
                ("posterior", C.c_void_p), ("accept", C.c_void_p), ("next_token", C.c_void_p), ("replay_len", C.c_void_p),
                ("logits_rows", C.c_void_p)]


class DFlashError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"dflash status {status}: {message}")
        self.status = status


class DFlashUnsupported(DFlashError):
    """Shape or dtype outside the supported set (the reference returns nil or falls back)."""


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m swiftlm_b200.build` "
                "(there is no CPU fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status == OK:
        return
    msg = lib().dflash_last_error_string().decode()
    if status == ERR_UNSUPPORTED:
        raise DFlashUnsupported(status, msg)
    raise DFlashError(status, msg)
