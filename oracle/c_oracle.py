"""ctypes front end of the C oracle (oracle/dflash_oracle.c, oracle/turbo_oracle.c) and of the
compiled reference codec (oracle/_ref/libturbo_ref.so).  TEST INFRASTRUCTURE ONLY.

`load()` builds oracle/_build/liboracle.so with `make -C oracle` if it is missing.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")


def build():
    subprocess.run(["make", "-C", _HERE], check=True, stdout=subprocess.DEVNULL)


def load():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "_build", "liboracle.so")
        try:
            build()          # make is incremental: a no-op unless a source is newer than the library
        except (OSError, subprocess.CalledProcessError):
            if not os.path.exists(path):
                raise
        _LIB = C.CDLL(path)
        _LIB.oracle_num_threads.restype = C.c_int
    return _LIB


def load_ref():
    """The reference's own codec functions (None if oracle/_ref was never built)."""
    global _REF
    if _REF is None:
        path = os.path.join(_HERE, "_ref", "libturbo_ref.so")
        if not os.path.exists(path):
            return None
        _REF = C.CDLL(path)
        _REF.turbo_ref_ff16.restype = C.c_float
        _REF.turbo_ref_ff16.argtypes = [C.c_uint16]
        _REF.turbo_ref_tf16.restype = C.c_uint16
        _REF.turbo_ref_tf16.argtypes = [C.c_float]
        _REF.turbo_ref_rn.restype = C.c_float
        _REF.turbo_ref_seed.argtypes = [C.c_uint64]
        _REF.turbo_ref_nc3.argtypes = [C.c_float]
        _REF.turbo_ref_qjl_c.restype = C.c_float
        for name in ("centroids", "boundaries"):
            getattr(_REF, "turbo_ref_" + name).restype = C.POINTER(C.c_float)
        _REF.turbo_ref_signs.restype = C.POINTER(C.c_float)
    return _REF


def num_threads() -> int:
    return load().oracle_num_threads()


def use_all_cores() -> int:
    """Lets the OpenMP loops use every core this process may run on, whatever OMP_NUM_THREADS says (torchrun exports
    OMP_NUM_THREADS=1 to its ranks).  Returns the thread count."""
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    load().oracle_set_num_threads(int(cores))
    return num_threads()


def _opt(a, dtype):
    if a is None:
        return None
    return np.ascontiguousarray(a, dtype=dtype).ctypes.data_as(C.c_void_p)


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def gated_delta(q, k, v, g, beta, state, mask=None, n=None, want_tape=True, passes=False):
    """oracle_gated_delta_f32 (row-wise) or, with passes=True, the whole-state-pass variant."""
    lib = load()
    q, k, v, g, beta, state = map(_f, (q, k, v, g, beta, state))
    B, T, Hk, Dk = q.shape
    Hv, Dv = v.shape[2], v.shape[3]
    y = np.empty((B, T, Hv, Dv), np.float32)
    tape = np.empty((B, T, Hv, Dv), np.float32) if want_tape else None
    out = np.empty_like(state)
    args = [q.ctypes.data_as(C.c_void_p), k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p),
            g.ctypes.data_as(C.c_void_p), beta.ctypes.data_as(C.c_void_p),
            state.ctypes.data_as(C.c_void_p), _opt(mask, np.float32), _opt(n, np.int32),
            y.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p),
            tape.ctypes.data_as(C.c_void_p) if want_tape else None]
    dims = [C.c_int(x) for x in (B, T, Hk, Hv, Dk, Dv, int(g.ndim == 4))]
    if passes:
        scratch = np.empty_like(state)
        lib.oracle_gated_delta_passes_f32(*args, scratch.ctypes.data_as(C.c_void_p), *dims)
    else:
        lib.oracle_gated_delta_f32(*args, *dims)
    return y, out, tape


def tape_replay(tape, k, g, state, mask=None, n=None):
    lib = load()
    tape, k, g, state = map(_f, (tape, k, g, state))
    B, T, Hv, Dv = tape.shape
    Hk, Dk = k.shape[2], k.shape[3]
    out = np.empty_like(state)
    lib.oracle_tape_replay_f32(tape.ctypes.data_as(C.c_void_p), k.ctypes.data_as(C.c_void_p),
                               g.ctypes.data_as(C.c_void_p), state.ctypes.data_as(C.c_void_p),
                               _opt(mask, np.float32), _opt(n, np.int32),
                               out.ctypes.data_as(C.c_void_p),
                               *[C.c_int(x) for x in (B, T, Hk, Hv, Dk, Dv, int(g.ndim == 4))])
    return out


def verify_sdpa(q, k, v, scale, kv_len=None):
    lib = load()
    q, k, v = map(_f, (q, k, v))
    B, Hq, M, D = q.shape
    Hkv, N = k.shape[1], k.shape[2]
    assert M == 16
    out = np.empty_like(q)
    lib.oracle_verify_sdpa_f32(q.ctypes.data_as(C.c_void_p), k.ctypes.data_as(C.c_void_p),
                               v.ctypes.data_as(C.c_void_p), _opt(kv_len, np.int32),
                               out.ctypes.data_as(C.c_void_p),
                               *[C.c_int(x) for x in (B, Hq, Hkv, N, D)], C.c_float(scale))
    return out


def accept(logits, verify_ids, suppress=None):
    lib = load()
    logits = _f(logits)
    B, T, V = logits.shape
    ids = np.ascontiguousarray(verify_ids, np.int32)
    post = np.empty((B, T), np.uint32)
    acc = np.empty((B,), np.int32)
    nxt = np.empty((B,), np.int32)
    lib.oracle_accept_f32(logits.ctypes.data_as(C.c_void_p), _opt(suppress, np.uint8),
                          ids.ctypes.data_as(C.c_void_p), post.ctypes.data_as(C.c_void_p),
                          acc.ctypes.data_as(C.c_void_p), nxt.ctypes.data_as(C.c_void_p),
                          C.c_int(B), C.c_int(T), C.c_int(V))
    return post, acc, nxt


# ---- TurboQuant codec (d = 128 blocks) ----------------------------------------------------


def turbo_encode_v(x):
    """x [..., 128] fp32 -> (packed [..., 48] u8, norm [...] u16)."""
    lib = load()
    x = _f(x)
    flat = x.reshape(-1, 128)
    packed = np.empty((flat.shape[0], 48), np.uint8)
    norm = np.empty((flat.shape[0],), np.uint16)
    n16 = C.c_uint16()
    for i in range(flat.shape[0]):
        lib.turbo_encode_v(flat[i].ctypes.data_as(C.c_void_p), packed[i].ctypes.data_as(C.c_void_p),
                           C.byref(n16))
        norm[i] = n16.value
    return packed.reshape(x.shape[:-1] + (48,)), norm.reshape(x.shape[:-1])


def turbo_decode_v(packed, norm):
    lib = load()
    p = np.ascontiguousarray(packed, np.uint8).reshape(-1, 48)
    n = np.ascontiguousarray(norm, np.uint16).reshape(-1)
    out = np.empty((p.shape[0], 128), np.float32)
    for i in range(p.shape[0]):
        lib.turbo_decode_v(p[i].ctypes.data_as(C.c_void_p), C.c_uint16(int(n[i])),
                           out[i].ctypes.data_as(C.c_void_p))
    return out.reshape(np.shape(norm) + (128,))


def turbo_encode_k(x):
    """x [..., 128] -> (packed [...,48] u8, signs [...,16] u8, norm [...] u16, rnorm [...] u16)."""
    lib = load()
    x = _f(x)
    flat = x.reshape(-1, 128)
    m = flat.shape[0]
    packed = np.empty((m, 48), np.uint8)
    signs = np.empty((m, 16), np.uint8)
    norm = np.empty((m,), np.uint16)
    rnorm = np.empty((m,), np.uint16)
    a, b = C.c_uint16(), C.c_uint16()
    for i in range(m):
        lib.turbo_encode_k(flat[i].ctypes.data_as(C.c_void_p), packed[i].ctypes.data_as(C.c_void_p),
                           signs[i].ctypes.data_as(C.c_void_p), C.byref(a), C.byref(b))
        norm[i], rnorm[i] = a.value, b.value
    sh = x.shape[:-1]
    return packed.reshape(sh + (48,)), signs.reshape(sh + (16,)), norm.reshape(sh), rnorm.reshape(sh)


def turbo_decode_k(packed, signs, norm, rnorm):
    lib = load()
    p = np.ascontiguousarray(packed, np.uint8).reshape(-1, 48)
    s = np.ascontiguousarray(signs, np.uint8).reshape(-1, 16)
    n = np.ascontiguousarray(norm, np.uint16).reshape(-1)
    r = np.ascontiguousarray(rnorm, np.uint16).reshape(-1)
    out = np.empty((p.shape[0], 128), np.float32)
    for i in range(p.shape[0]):
        lib.turbo_decode_k(p[i].ctypes.data_as(C.c_void_p), s[i].ctypes.data_as(C.c_void_p),
                           C.c_uint16(int(n[i])), C.c_uint16(int(r[i])),
                           out[i].ctypes.data_as(C.c_void_p))
    return out.reshape(np.shape(norm) + (128,))
