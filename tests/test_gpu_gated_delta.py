"""GPU parity of the gated-delta forward / tape replay kernels against the CPU oracle,
called through the C ABI (swiftlm_b200.kernels -> ctypes -> libdflash_cuda.so).

Tolerance: replayed states within 1e-4 relative (fp32), y within 1e-4 relative for fp32 inputs
and within one bf16/f16 rounding step otherwise; tape-slot indexing (which steps run, which
rows are zero) bit-exact."""
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle as CO
from oracle import dflash_oracle as O
from tests.golden import gen_golden as G

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
TORCH_DT = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}
STATE_RTOL = 1e-4


def K():
    from swiftlm_b200 import kernels
    return kernels


def dev(x, dt=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if dt is None else t.to(dt)


def rel(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def run_fwd(x, dtype, mask=None, use_n=True, want_tape=True):
    dt = TORCH_DT[dtype]
    y, s, tape = K().gated_delta_kernel_with_tape(
        dev(x["q"], dt), dev(x["k"], dt), dev(x["v"], dt), dev(x["g"], dt), dev(x["beta"], dt),
        dev(x["state"]), mask=None if mask is None else dev(mask),
        n_per_seq=dev(x["n"]) if use_n else None, want_tape=want_tape)
    torch.cuda.synchronize()
    K().device_status()
    return (y.float().cpu().numpy(), s.cpu().numpy(), None if tape is None else tape.cpu().numpy())


def y_tol(dtype):
    return {"fp32": 1e-4, "bf16": 1.0 / 128, "fp16": 1.0 / 1024}[dtype]


@pytest.mark.parametrize("name", sorted(G.GDN_CASES))
def test_golden_vectors(name):
    x = G.gdn_case(name)
    gold = np.load(os.path.join(GOLD, name + ".npz"))
    dtype = G.GDN_CASES[name][7]
    y, s, tape = run_fwd(x, dtype)
    assert rel(s, gold["state"]) < STATE_RTOL
    assert rel(tape, gold["tape"]) < 1e-4
    assert rel(y, gold["y"]) < y_tol(dtype)
    # slot indexing is exact: rows at or beyond the accepted length are exactly zero
    for b, n in enumerate(x["n"]):
        assert not y[b, n:].any() and not tape[b, n:].any()
        if n == 0:
            np.testing.assert_array_equal(s[b], x["state"][b])


CASES = [
    # B, T, Hk, Hv, Dk, Dv, vec, dtype
    (1, 16, 16, 32, 128, 128, False, "fp32"),     # the reference-runnable configuration
    (5, 16, 4, 8, 128, 128, False, "bf16"),
    (3, 16, 2, 4, 128, 128, False, "fp16"),
    (2, 7, 2, 2, 128, 128, False, "fp32"),        # Hk == Hv, T < 16
    (2, 16, 2, 4, 128, 128, True, "bf16"),        # vector gate
    (1, 4, 8, 8, 64, 64, False, "fp32"),          # the reference profiler's availability shape
    (2, 8, 8, 16, 128, 128, False, "bf16"),       # the reference's consistency-check shape
    (2, 16, 1, 3, 32, 48, True, "fp32"),          # odd head ratio, Dv not a power of two
    (2, 20, 2, 4, 256, 64, False, "bf16"),        # T > 16, Dk = 256
    (1, 1, 1, 4, 128, 128, False, "bf16"),        # a single step, four v-heads per qk-head (tensor-core path)
    (3, 13, 4, 4, 128, 128, False, "bf16"),       # Hk == Hv, odd T (tensor-core path, rows of K/Q/V beyond T read as zeros)
    (40, 16, 2, 4, 128, 128, False, "bf16"),      # more head-states than SMs (tensor-core path, several items per CTA)
    (3, 16, 2, 6, 128, 128, True, "fp16"),        # vector gate, three v-heads per qk-head
    (2, 11, 4, 4, 128, 128, True, "fp32"),        # vector gate, fp32 inputs, odd T
    (160, 16, 2, 4, 128, 128, True, "bf16"),      # vector gate, three items per CTA (both gate buffers reused)
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "x".join(map(str, c)))
@pytest.mark.parametrize("masked", [False, True], ids=["n_only", "mask_and_n"])
def test_forward_matches_oracle(case, masked):
    B, T, Hk, Hv, Dk, Dv, vec, dtype = case
    x = O.make_gdn_inputs(B, T, Hk, Hv, Dk, Dv, 500 + sum(case[:6]), vec, dtype)
    mask = None
    if masked:
        mask = (np.random.default_rng(9).random((B, T)) > 0.35).astype(np.float32)
    y, s, tape = run_fwd(x, dtype, mask=mask)
    yo, so, to = CO.gated_delta(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"], mask=mask, n=x["n"])
    assert rel(s, so) < STATE_RTOL
    assert rel(tape, to) < 1e-4
    assert rel(y, yo) < y_tol(dtype)
    np.testing.assert_array_equal(tape == 0, to == 0)     # which slots ran: exact


@pytest.mark.parametrize("case", CASES, ids=lambda c: "x".join(map(str, c)))
def test_tape_replay_matches_oracle_and_forward(case):
    B, T, Hk, Hv, Dk, Dv, vec, dtype = case
    x = O.make_gdn_inputs(B, T, Hk, Hv, Dk, Dv, 700 + sum(case[:6]), vec, dtype)
    dt = TORCH_DT[dtype]
    # record the tape with an unmasked forward, then replay n steps from the snapshot
    _, s_full, tape = K().gated_delta_kernel_with_tape(
        dev(x["q"], dt), dev(x["k"], dt), dev(x["v"], dt), dev(x["g"], dt), dev(x["beta"], dt), dev(x["state"]))
    s_rep = K().tape_replay_kernel(tape, dev(x["k"], dt), dev(x["g"], dt), dev(x["state"]), n_per_seq=dev(x["n"]))
    torch.cuda.synchronize()
    s_rep = s_rep.cpu().numpy()
    want = CO.tape_replay(tape.cpu().numpy(), x["k"], x["g"], x["state"], n=x["n"])
    assert rel(s_rep, want) < STATE_RTOL
    # replaying the recorded tape reproduces the masked forward's state
    _, s_fwd, _ = run_fwd(x, dtype)
    assert rel(s_rep, s_fwd) < STATE_RTOL
    # the caller's slicing contract (B = 1 slices): same result
    n0 = int(x["n"][0])
    if n0 > 0:
        sl = K().tape_replay_kernel(tape[:1, :n0].contiguous(), dev(x["k"], dt)[:1, :n0].contiguous(),
                                    dev(x["g"], dt)[:1, :n0].contiguous(), dev(x["state"])[:1])
        assert rel(sl.cpu().numpy(), s_rep[:1]) < 1e-6
    # full-length replay equals the unmasked forward's state
    s_all = K().tape_replay_kernel(tape, dev(x["k"], dt), dev(x["g"], dt), dev(x["state"]))
    assert rel(s_all.cpu().numpy(), s_full.cpu().numpy()) < STATE_RTOL


@pytest.mark.parametrize("vec", [False, True], ids=["scalar_gate", "vector_gate"])
def test_edge_lengths_and_determinism(vec):
    x = O.make_gdn_inputs(4, 16, 2, 4, 128, 128, 900, vec, "bf16")
    x["n"] = np.array([0, 16, 1, 15], np.int32)
    y, s, tape = run_fwd(x, "bf16")
    np.testing.assert_array_equal(s[0], x["state"][0])          # n = 0: identity
    assert not y[0].any()
    full = dict(x)
    yf, sf, tf = run_fwd(full, "bf16", use_n=False)
    np.testing.assert_array_equal(s[1], sf[1])                  # n = T equals the unmasked run
    np.testing.assert_array_equal(y[1], yf[1])
    y2, s2, t2 = run_fwd(x, "bf16")
    np.testing.assert_array_equal(s, s2)                        # bitwise repeatable
    np.testing.assert_array_equal(y, y2)
    np.testing.assert_array_equal(tape, t2)
    # optional tape output
    y3, s3, none = run_fwd(x, "bf16", want_tape=False)
    assert none is None
    np.testing.assert_array_equal(s, s3)


@pytest.mark.parametrize("dtype", ["bf16", "fp32"])
@pytest.mark.parametrize("regime", ["zero_gates", "tiny_gates", "small_gates", "gates_above_one", "mixed_items"])
def test_vector_gate_extreme_gates(regime, dtype):
    """Per-channel gates at the edges of the forward kernel's two routes: it folds the running gate products into k
    and q (state carried divided by the product), and takes the column-by-column route for an item whose product
    leaves [1e-12, 1e12] in any channel."""
    B, T, Hk, Hv, D = 6, 16, 2, 4, 128
    x = O.make_gdn_inputs(B, T, Hk, Hv, D, D, 930, True, dtype)
    x["n"] = np.array([16, 16, 9, 16, 1, 13], np.int32)
    g = x["g"]
    if regime == "zero_gates":            # exact zeros in some channels of some steps: those columns are cleared
        rng = np.random.default_rng(5)
        g[rng.random(g.shape) < 0.02] = 0.0
    elif regime == "tiny_gates":          # products far below the smallest normal number
        g[:] = (g * 1e-4).astype(np.float32)
    elif regime == "small_gates":         # products down to ~1e-11: still the folded route, 1 / G large
        g[:] = np.clip(g, 0.21, 1.0)
    elif regime == "gates_above_one":     # not a decay any more, but nothing in the interface forbids it
        g[:] = (g * 1.8).astype(np.float32)
    else:                                 # one sequence on the explicit route between sequences on the folded one
        g[2, 3, :, 17] = 0.0
        g[4, 0, 1, :] = 1e-20
    if dtype != "fp32":
        x["g"] = g = O._round_to(g, dtype)
    y, s, tape = run_fwd(x, dtype)
    yo, so, to = CO.gated_delta(x["q"], x["k"], x["v"], g, x["beta"], x["state"], n=x["n"])
    assert np.isfinite(s).all() and np.isfinite(y).all()
    assert rel(s, so) < STATE_RTOL
    assert rel(tape, to) < 1e-4
    assert rel(y, yo) < y_tol(dtype)
    # column by column too: a column the gates cleared holds what the later steps wrote, nothing of the old state
    col_scale = np.maximum(np.abs(so).max(axis=(0, 2), keepdims=True), 1e-30)
    assert float((np.abs(s - so) / col_scale).max()) < 1e-3


def test_in_place_state_through_c_abi():
    from swiftlm_b200 import _lib
    x = O.make_gdn_inputs(3, 16, 2, 4, 128, 128, 901, False, "bf16")
    dt = torch.bfloat16
    q, k, v, g, beta = (dev(x[n], dt) for n in ("q", "k", "v", "g", "beta"))
    state = dev(x["state"])
    n = dev(x["n"])
    y = torch.empty(3, 16, 4, 128, dtype=dt, device="cuda")
    st = _lib.lib().dflash_gated_delta_tape(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
                                          state.data_ptr(), None, n.data_ptr(), y.data_ptr(), state.data_ptr(), None,
                                          3, 16, 2, 4, 128, 128, 0, _lib.BF16, 0, None)
    assert st == 0
    torch.cuda.synchronize()
    _, so, _ = CO.gated_delta(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"], n=x["n"])
    assert rel(state.cpu().numpy(), so) < STATE_RTOL


def test_unsupported_shapes_report_errors():
    from swiftlm_b200 import _lib
    x = O.make_gdn_inputs(1, 4, 1, 1, 32, 32, 902)
    t = {k_: dev(v_) for k_, v_ in x.items()}
    with pytest.raises(_lib.DFlashUnsupported):
        K().gated_delta_kernel_with_tape(t["q"][..., :24], t["k"][..., :24], t["v"], t["g"], t["beta"], t["state"][..., :24])
    with pytest.raises(RuntimeError):
        K().tape_replay_kernel(torch.zeros(1, 4, 1, 32), torch.zeros(1, 4, 1, 32), torch.zeros(1, 4, 1), torch.zeros(1, 1, 32, 32))


def test_full_size_properties_replay_config():
    """Size-independent checks at the benchmark's scale (a slice of it: 8 sequences x 36 layers):
    linearity of the replay in (state, tape), and forward/replay agreement."""
    B, T, Hk, Hv, D = 8 * 36, 16, 16, 32, 128
    g = torch.Generator(device="cuda").manual_seed(20260330)
    q = torch.nn.functional.normalize(torch.randn(B, T, Hk, D, device="cuda", generator=g), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(torch.randn(B, T, Hk, D, device="cuda", generator=g), dim=-1).bfloat16()
    v = torch.randn(B, T, Hv, D, device="cuda", generator=g).bfloat16()
    beta = torch.sigmoid(torch.randn(B, T, Hv, device="cuda", generator=g)).bfloat16()
    gate = torch.exp(-torch.nn.functional.softplus(torch.randn(B, T, Hv, device="cuda", generator=g))).bfloat16()
    s0 = 0.02 * torch.randn(B, Hv, D, D, device="cuda", generator=g)
    n = torch.randint(0, T + 1, (8,), device="cuda", generator=g).repeat_interleave(36).int()
    y, s1, tape = K().gated_delta_kernel_with_tape(q, k, v, gate, beta, s0, n_per_seq=n)
    s_rep = K().tape_replay_kernel(tape, k, gate, s0, n_per_seq=n)
    torch.cuda.synchronize()
    err = (s_rep - s1).abs().max() / s1.abs().max()
    assert float(err) < STATE_RTOL
    # linearity: replay(a*S + S', a*tape + tape') == a*replay(S, tape) + replay(S', tape')
    s0b = 0.02 * torch.randn_like(s0)
    tape_b = torch.randn_like(tape) * 0.1
    lhs = K().tape_replay_kernel(2.0 * tape + tape_b, k, gate, 2.0 * s0 + s0b, n_per_seq=n)
    rhs = 2.0 * s_rep + K().tape_replay_kernel(tape_b, k, gate, s0b, n_per_seq=n)
    assert float((lhs - rhs).abs().max() / rhs.abs().max()) < STATE_RTOL
    # sequences with n == 0 are untouched, bit for bit
    idle = (n == 0)
    if idle.any():
        assert torch.equal(s1[idle], s0[idle])


@pytest.mark.parametrize("variant", ["large_state", "correlated_keys", "tiny_gates", "ones"])
def test_tensor_core_path_under_stress(variant):
    """The bf16 / 128 x 128 / scalar-gate path (three tensor-core products plus a triangular recurrence) on inputs
    that stress its two-term split of the state and the recurrence: O(1) states, nearly parallel keys, gates down to
    1e-3 (and exactly 0 and 1), betas of exactly 1."""
    rng = np.random.default_rng(77)
    x = O.make_gdn_inputs(4, 16, 2, 4, 128, 128, 950, False, "bf16")
    if variant == "large_state":
        x["state"] = rng.standard_normal(x["state"].shape).astype(np.float32)
    elif variant == "correlated_keys":
        base = rng.standard_normal((4, 1, 2, 128)).astype(np.float32)
        k = base + 0.15 * rng.standard_normal((4, 16, 2, 128)).astype(np.float32)
        x["k"] = O.round_bf16(k / np.linalg.norm(k, axis=-1, keepdims=True))
        x["beta"] = O.round_bf16(np.full_like(x["beta"], 0.98))
    elif variant == "tiny_gates":
        g = 10.0 ** rng.uniform(-3, 0, x["g"].shape)
        g[0, 3] = 0.0
        g[1, 5] = 1.0
        x["g"] = O.round_bf16(g.astype(np.float32))
    else:
        x["beta"] = np.ones_like(x["beta"])
        x["g"] = np.ones_like(x["g"])
    x["n"] = np.array([16, 9, 16, 3], np.int32)
    y, s, tape = run_fwd(x, "bf16")
    yo, so, to = CO.gated_delta(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"], n=x["n"])
    assert rel(s, so) < STATE_RTOL
    assert rel(tape, to) < 1e-4
    assert rel(y, yo) < y_tol("bf16")
