"""Generates the committed golden vectors under tests/golden/ from the CPU oracle.

The reference ships no golden vectors for this path and cannot run where these tests run, so
the fixtures are outputs of the oracle's NumPy restatement on seeded inputs.  Inputs are
regenerated from the seed at test time (oracle.dflash_oracle.make_*_inputs); each fixture
stores the expected outputs plus a checksum of the inputs so a change in the generator shows
up as a fixture mismatch rather than a silent pass.   Run:  python tests/golden/gen_golden.py
(writes the fixtures that are missing; --force rewrites all of them).
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import dflash_oracle as O  # noqa: E402

GDN_CASES = {
    # name: (B, T, Hk, Hv, Dk, Dv, vector_gate, dtype, seed offset)
    "gdn_fp32_d128": (1, 16, 1, 2, 128, 128, False, "fp32", 1),
    "gdn_bf16_d128": (1, 16, 1, 2, 128, 128, False, "bf16", 2),
    "gdn_fp32_d64_vec": (2, 8, 2, 4, 64, 32, True, "fp32", 3),
    "gdn_fp32_profiler_shape": (1, 4, 8, 8, 64, 64, False, "fp32", 4),
    "gdn_bf16_d128_vec": (2, 16, 1, 2, 128, 128, True, "bf16", 5),
}
SDPA_CASES = {
    # name: (B, Hq, Hkv, N, D, dtype, seed offset)
    "sdpa_bf16_d256": (1, 8, 1, 16 + 300, 256, "bf16", 11),
    "sdpa_bf16_d128_gqa4": (1, 8, 2, 16 + 129, 128, "bf16", 12),
    "sdpa_fp16_d128_short": (1, 4, 4, 16, 128, "fp16", 13),
}


def digest(d):
    h = hashlib.sha256()
    for key in sorted(d):
        h.update(np.ascontiguousarray(d[key]).tobytes())
    return np.frombuffer(h.digest()[:8], np.uint8).copy()


def gdn_case(name):
    B, T, Hk, Hv, Dk, Dv, vec, dt, off = GDN_CASES[name]
    return O.make_gdn_inputs(B, T, Hk, Hv, Dk, Dv, O.BASE_SEED + off, vec, dt)


def sdpa_case(name):
    B, Hq, Hkv, N, D, dt, off = SDPA_CASES[name]
    return O.make_sdpa_inputs(B, Hq, Hkv, N, D, O.BASE_SEED + off, dt), dt


def main():
    force = "--force" in sys.argv

    def wanted(name):
        return force or not os.path.exists(os.path.join(HERE, name + ".npz"))

    for name in filter(wanted, GDN_CASES):
        x = gdn_case(name)
        y, s, tape = O.gated_delta_ops_with_tape(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"],
                                                 n_per_seq=x["n"])
        np.savez_compressed(os.path.join(HERE, name + ".npz"), inputs_digest=digest(x), n=x["n"],
                            y=y.astype(np.float32), state=s, tape=tape)
    for name in filter(wanted, SDPA_CASES):
        x, dt = sdpa_case(name)
        out = O.verify_sdpa(x["q"], x["k"], x["v"], x["scale"], in_dtype=dt)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), inputs_digest=digest(x), out=out)
    # acceptance: the worked example of the reference's doc comment
    # (Sources/DFlash/DFlashRuntime.swift:130-132) plus edge cases
    if wanted("accept_cases"):
        np.savez(os.path.join(HERE, "accept_cases.npz"),
                 drafted=np.array([[1, 2, 3], [1, 2, 3], [7, 7, 7], [4, 5, 6]], np.int32),
                 posterior=np.array([[1, 2, 5], [1, 2, 3], [0, 7, 7], [4, 9, 6]], np.int32),
                 expect=np.array([2, 3, 0, 1], np.int32))
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
