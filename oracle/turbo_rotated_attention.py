"""Block-verify attention over TurboQuant KV without decoding a single key or value: test infrastructure.

The codec's rotation is orthogonal, so the decode of tests/test_turbo_quant.cpp (:74-75, :96-98 in the
reference tree) can be moved onto the 16 x G query rows and the output rows:

    k_n = norm_n * ( R^-1 c_n  +  (QJL_C / 128) * rnorm_n * Rq s_n )        decode of a key block
    q . k_n = norm_n * ( (R q) . c_n  +  (QJL_C / 128) * rnorm_n * (Rq^-1 q) . s_n )
    v_n = vnorm_n * R^-1 c'_n
    sum_n p_n v_n = R^-1 ( sum_n p_n vnorm_n c'_n )

with R = rot(., S1, S2), R^-1 = rot(., S2, S1), Rq = rot(., Q1, Q2), Rq^-1 = rot(., Q2, Q1) (:15-17), c the
centroid vector of the 3-bit indices and s the +-1 vector of the sign bits.  A head vector of 256 dimensions
is two independent 128-blocks.  This module states that form in NumPy so that a kernel which expands the
packed indices straight into tensor-core operands (no Walsh-Hadamard transform per key) has an oracle; the
test next to it checks the form against decode-then-attend.
"""
import os
import re

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))


def _tables():
    src = open(os.path.join(_HERE, "turbo_tables.h")).read()
    c3 = np.array([float(t.strip().rstrip("f")) for t in re.search(r"TURBO_C3\[8\] = \{([^}]*)\}", src).group(1).split(",")], np.float32)
    qjl = np.float32(float(re.search(r"TURBO_QJL_C ([0-9.eE+-]+)f", src).group(1)))
    sign = {}
    for name in ("S1", "S2", "Q1", "Q2"):
        words = [int(t.strip().rstrip("u"), 16) for t in re.search(r"TURBO_%s_NEG\[4\] = \{([^}]*)\}" % name, src).group(1).split(",")]
        sign[name] = np.array([-1.0 if (words[i >> 5] >> (i & 31)) & 1 else 1.0 for i in range(128)], np.float32)
    return c3, qjl, sign


C3, QJL_C, SIGN = _tables()


def _hadamard128():
    h = np.array([[1.0]], np.float32)
    while h.shape[0] < 128:
        h = np.block([[h, h], [h, -h]])
    return h.astype(np.float32)


H128 = _hadamard128()


def rot(x, first: str, second: str):
    """rot of :15-17 on the last axis (128): sign flips, Walsh-Hadamard transform scaled by 1/sqrt(128), sign flips."""
    x = np.asarray(x, np.float32)
    return ((x * SIGN[first]) @ H128) * np.float32(0.08838834764831845) * SIGN[second]


def _f16(bits):
    return np.asarray(bits, np.uint16).view(np.float16).astype(np.float32)


def unpack_indices(packed):
    """[..., 48] uint8 -> [..., 128] 3-bit indices (little-endian bit stream, :19-20)."""
    bits = np.unpackbits(np.asarray(packed, np.uint8), axis=-1, bitorder="little")
    b = bits.reshape(bits.shape[:-1] + (128, 3)).astype(np.int64)
    return b[..., 0] | (b[..., 1] << 1) | (b[..., 2] << 2)


def unpack_signs(signs):
    """[..., 16] uint8 -> [..., 128] of +-1."""
    bits = np.unpackbits(np.asarray(signs, np.uint8), axis=-1, bitorder="little")
    return np.where(bits > 0, 1.0, -1.0).astype(np.float32)


def verify_sdpa_rotated(q, k_enc, v_enc, scale, k_hot=None, v_hot=None):
    """Block-verify attention with the cold history in the TurboQuant format and an optional hot window.

    q [B,Hq,16,D]; k_enc = (packed [B,Hkv,Nc,D/128,48], signs [...,16], norm [...], rnorm [...]) and
    v_enc = (packed, norm) as the encoder returns them; k_hot, v_hot [B,Hkv,Nh,D] float (the newest tokens, the
    16 block keys among them).  Visibility as in Sources/DFlash/DFlashKernels.swift:614 of the reference tree:
    key n is visible to row r iff n <= N - 16 + r with N = Nc + Nh.  Returns [B,Hq,16,D] fp32.
    No key or value is decoded: scores and outputs are formed in the rotated domain."""
    q = np.asarray(q, np.float32)
    B, Hq, M, D = q.shape
    kp, ks, kn, kr = k_enc
    vp, vn = v_enc
    Hkv, Nc, nb = kn.shape[1], kn.shape[2], D // 128
    Nh = 0 if k_hot is None else k_hot.shape[2]
    N = Nc + Nh
    gqa = Hq // Hkv
    coef = np.float32(QJL_C / np.float32(128.0))
    ck = C3[unpack_indices(kp)]                                   # [B,Hkv,Nc,nb,128] centroid vectors
    sk = unpack_signs(ks)                                         # +-1
    cv = C3[unpack_indices(vp)]
    knorm, krn, vnorm = _f16(kn), _f16(kr), _f16(vn)
    out = np.zeros((B, Hq, M, D), np.float32)
    n_idx = np.arange(N)[None, :]
    visible = n_idx <= (N - M + np.arange(M)[:, None])
    for b in range(B):
        for h in range(Hq):
            hk = h // gqa
            qs = (np.float32(scale) * q[b, h]).reshape(M, nb, 128)
            q1 = rot(qs, "S1", "S2")                              # R q
            q2 = rot(qs, "Q2", "Q1")                              # Rq^-1 q
            s = np.zeros((M, N), np.float32)
            # per 128-block: norm * (q1 . c + coef * rnorm * q2 . s)
            main = np.einsum("mjd,njd->mnj", q1, ck[b, hk])       # [M,Nc,nb]
            resid = np.einsum("mjd,njd->mnj", q2, sk[b, hk])
            s[:, :Nc] = ((main + coef * krn[b, hk][None] * resid) * knorm[b, hk][None]).sum(-1)
            if Nh:
                s[:, Nc:] = (qs.reshape(M, D)) @ np.asarray(k_hot[b, hk], np.float32).T
            s = np.where(visible, s, -np.inf)
            mx = s.max(axis=-1, keepdims=True)
            p = np.exp(s - mx).astype(np.float32)
            den = p.sum(axis=-1, keepdims=True, dtype=np.float32)
            # cold values: accumulate in the rotated domain, rotate the 16 rows back once
            acc = np.einsum("mnj,njd->mjd", p[:, :Nc, None] * vnorm[b, hk][None], cv[b, hk])   # [M,nb,128]
            o = rot(acc, "S2", "S1").reshape(M, D)
            if Nh:
                o = o + p[:, Nc:] @ np.asarray(v_hot[b, hk], np.float32)
            out[b, h] = o / den
    return out
