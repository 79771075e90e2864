"""CPU tests of the oracle itself: the independent statements of the recurrence in the
reference agree, the algebraic identities hold, the C restatement equals the NumPy one, and
both reproduce the committed golden vectors."""
import os

import numpy as np
import pytest

from oracle import c_oracle as CO
from oracle import dflash_oracle as O
from tests.golden import gen_golden as G

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


@pytest.mark.parametrize("vec", [False, True])
def test_ops_statement_matches_rowwise_statement(vec):
    x = O.make_gdn_inputs(2, 6, 2, 4, 32, 16, 101, vector_gate=vec)
    mask = (np.random.default_rng(5).random((2, 6)) > 0.4).astype(np.float32)
    a = O.gated_delta_ops_with_tape(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"], mask=mask)
    b = O.gated_delta_rowwise(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"], mask=mask)
    for u, w in zip(a, b):
        assert rel_err(u, w) < 2e-6


def test_vector_gate_matches_kimi_statement():
    x = O.make_gdn_inputs(2, 5, 3, 3, 32, 16, 102, vector_gate=True)
    y, s, _ = O.gated_delta_ops_with_tape(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"])
    yk, sk = O.kimi_gated_delta_update(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"])
    assert rel_err(y, yk) < 1e-6 and rel_err(s, sk) < 1e-6


def test_vector_gate_with_equal_lanes_equals_scalar_gate():
    x = O.make_gdn_inputs(1, 7, 2, 4, 32, 32, 103)
    gv = np.repeat(x["g"][..., None], 32, axis=-1)
    a = O.gated_delta_ops_with_tape(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"])
    b = O.gated_delta_ops_with_tape(x["q"], x["k"], x["v"], gv, x["beta"], x["state"])
    for u, w in zip(a, b):
        np.testing.assert_array_equal(u, w)


def test_accepted_length_identities():
    x = O.make_gdn_inputs(3, 8, 2, 4, 32, 32, 104)
    args = (x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"])
    full = O.gated_delta_ops_with_tape(*args)
    nT = O.gated_delta_ops_with_tape(*args, n_per_seq=np.full(3, 8))
    n0 = O.gated_delta_ops_with_tape(*args, n_per_seq=np.zeros(3, np.int32))
    for u, w in zip(full, nT):
        np.testing.assert_array_equal(u, w)
    np.testing.assert_array_equal(n0[1], x["state"])
    assert not n0[0].any() and not n0[2].any()
    # prefix property: state at n equals the state of a run truncated to n tokens
    n = np.array([3, 0, 5], np.int32)
    _, s, _ = O.gated_delta_ops_with_tape(*args, n_per_seq=n)
    for b in range(3):
        sl = [a[b:b + 1, :n[b]] for a in (x["q"], x["k"], x["v"], x["g"], x["beta"])]
        if n[b] == 0:
            np.testing.assert_array_equal(s[b], x["state"][b])
            continue
        _, sb, _ = O.gated_delta_ops_with_tape(*sl, x["state"][b:b + 1])
        np.testing.assert_array_equal(s[b:b + 1], sb)


@pytest.mark.parametrize("vec", [False, True])
def test_replay_of_recorded_tape_reproduces_forward_state(vec):
    x = O.make_gdn_inputs(2, 9, 2, 4, 32, 16, 105, vector_gate=vec)
    n = np.array([4, 9], np.int32)
    _, s_fwd, tape = O.gated_delta_ops_with_tape(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"],
                                                 n_per_seq=n)
    _, _, tape_all = O.gated_delta_ops_with_tape(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"])
    s_rep = O.tape_replay_ops(tape_all, x["k"], x["g"], x["state"], n_per_seq=n)
    assert rel_err(s_rep, s_fwd) < 1e-6
    # the caller's way: slice the first n steps (RecurrentRollbackCache.swift:115-125), B = 1
    for b in range(2):
        s1 = O.tape_replay_ops(tape_all[b:b + 1, :n[b]], x["k"][b:b + 1, :n[b]], x["g"][b:b + 1, :n[b]],
                               x["state"][b:b + 1])
        np.testing.assert_array_equal(s1, s_rep[b:b + 1])


@pytest.mark.parametrize("vec", [False, True])
def test_c_restatement_equals_numpy(vec):
    x = O.make_gdn_inputs(3, 16, 2, 4, 64, 32, 106, vector_gate=vec)
    mask = (np.random.default_rng(6).random((3, 16)) > 0.3).astype(np.float32)
    ref = O.gated_delta_ops_with_tape(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"], mask=mask,
                                      n_per_seq=x["n"])
    for passes in (False, True):
        got = CO.gated_delta(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"], mask=mask, n=x["n"],
                             passes=passes)
        for u, w in zip(got, ref):
            assert rel_err(u, w) < 5e-6
    s = CO.tape_replay(ref[2], x["k"], x["g"], x["state"], mask=mask, n=x["n"])
    s_np = O.tape_replay_ops(ref[2], x["k"], x["g"], x["state"], mask=mask, n_per_seq=x["n"])
    assert rel_err(s, s_np) < 1e-6
    assert rel_err(s, ref[1]) < 5e-6


@pytest.mark.parametrize("name", sorted(G.GDN_CASES))
def test_gdn_golden(name):
    x = G.gdn_case(name)
    gold = np.load(os.path.join(GOLD, name + ".npz"))
    np.testing.assert_array_equal(G.digest(x), gold["inputs_digest"])
    np.testing.assert_array_equal(x["n"], gold["n"])
    y, s, tape = O.gated_delta_ops_with_tape(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"],
                                             n_per_seq=x["n"])
    for got, key in ((y, "y"), (s, "state"), (tape, "tape")):
        assert rel_err(got, gold[key]) < 1e-6
    yc, sc, tc = CO.gated_delta(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"], n=x["n"])
    for got, key in ((yc, "y"), (sc, "state"), (tc, "tape")):
        assert rel_err(got, gold[key]) < 1e-5


@pytest.mark.parametrize("name", sorted(G.SDPA_CASES))
def test_sdpa_golden(name):
    x, dt = G.sdpa_case(name)
    gold = np.load(os.path.join(GOLD, name + ".npz"))
    np.testing.assert_array_equal(G.digest(x), gold["inputs_digest"])
    out = O.verify_sdpa(x["q"], x["k"], x["v"], x["scale"], in_dtype=dt)
    assert np.abs(out - gold["out"]).max() < 1e-5
    outc = CO.verify_sdpa(x["q"], x["k"], x["v"], float(x["scale"]))
    assert np.abs(outc - gold["out"]).max() < 1e-4


def test_sdpa_block_causal_rule_and_split_invariance():
    x = O.make_sdpa_inputs(1, 2, 1, 16 + 21, 32, 201, "fp32")
    full = O.verify_sdpa(x["q"], x["k"], x["v"], x["scale"])
    for blocks in (1, 4, 32):
        two = O.verify_sdpa_two_pass(x["q"], x["k"], x["v"], x["scale"], blocks)
        assert np.abs(two - full).max() < 2e-6
    # row r of the block must not see block keys r+1..15: perturbing them changes nothing
    k2, v2 = x["k"].copy(), x["v"].copy()
    N = k2.shape[2]
    r = 5
    k2[:, :, N - 16 + r + 1:] += 3.0
    v2[:, :, N - 16 + r + 1:] -= 2.0
    pert = O.verify_sdpa(x["q"], k2, v2, x["scale"])
    np.testing.assert_array_equal(pert[:, :, :r + 1], full[:, :, :r + 1])
    assert np.abs(pert[:, :, r + 1:] - full[:, :, r + 1:]).max() > 1e-3
    # N == 16: the first row sees exactly one key, so its output is that key's value
    y = O.make_sdpa_inputs(1, 1, 1, 16, 32, 202, "fp32")
    o = O.verify_sdpa(y["q"], y["k"], y["v"], y["scale"])
    np.testing.assert_allclose(o[0, 0, 0], y["v"][0, 0, 0], rtol=1e-6)


def test_sdpa_additive_mask_and_ragged_lengths():
    x = O.make_sdpa_inputs(2, 4, 2, 16 + 40, 32, 203, "bf16")
    N = x["k"].shape[2]
    mask = np.zeros((2, 4, 16, N), np.float32)
    mask[:, :, :, 3] = -np.inf          # hidden key
    mask[:, :, :, 7] = 0.5              # additive bias
    got = O.verify_sdpa(x["q"], x["k"], x["v"], x["scale"], mask=mask)
    k2 = np.delete(x["k"], 3, axis=2)
    v2 = np.delete(x["v"], 3, axis=2)
    m2 = np.delete(mask, 3, axis=3)
    ref = O.verify_sdpa(x["q"], k2, v2, x["scale"], mask=m2)
    assert np.abs(got - ref).max() < 1e-6
    lens = np.array([N, 30], np.int32)
    rag = O.verify_sdpa(x["q"], x["k"], x["v"], x["scale"], kv_len=lens)
    short = O.verify_sdpa(x["q"][1:], x["k"][1:, :, :30], x["v"][1:, :, :30], x["scale"])
    np.testing.assert_array_equal(rag[1:], short)
    ragc = CO.verify_sdpa(x["q"], x["k"], x["v"], float(x["scale"]), kv_len=lens)
    assert np.abs(ragc - rag).max() < 1e-5


def test_sdpa_eligibility_and_block_heuristic():
    assert O.sdpa_supported((1, 32, 16, 128), (1, 8, 512, 128), (1, 8, 512, 128), "bf16")
    assert not O.sdpa_supported((1, 32, 8, 128), (1, 8, 512, 128), (1, 8, 512, 128), "bf16")
    assert not O.sdpa_supported((1, 32, 16, 64), (1, 8, 512, 64), (1, 8, 512, 64), "bf16")
    assert not O.sdpa_supported((1, 32, 16, 128), (1, 8, 512, 128), (1, 8, 512, 128), "fp32")
    assert not O.sdpa_supported((1, 30, 16, 128), (1, 8, 512, 128), (1, 8, 512, 128), "fp16")
    assert O.compute_sdpa_2pass_blocks(8, 4112, "applegpu_g15d") == 128
    assert O.compute_sdpa_2pass_blocks(8, 20000, "applegpu_g15d") == 512
    assert O.compute_sdpa_2pass_blocks(8, 70000, "applegpu_g15s") == 1024
    assert O.compute_sdpa_2pass_blocks(2, 9000, "applegpu_g15d") == 256
    assert O.compute_sdpa_2pass_blocks(4, 100, "") == 64 and O.compute_sdpa_2pass_blocks(2, 100, "") == 32


def test_acceptance_known_answers():
    gold = np.load(os.path.join(GOLD, "accept_cases.npz"))
    for d, p, e in zip(gold["drafted"], gold["posterior"], gold["expect"]):
        assert O.match_acceptance_length(d, p) == e
    assert O.match_acceptance_length(np.zeros(0), np.zeros(0)) == 0
    rng = np.random.default_rng(3)
    logits = rng.standard_normal((2, 16, 50)).astype(np.float32)
    sup = np.zeros(50, np.uint8)
    sup[[4, 9]] = 1
    logits[0, 3, 4] = 100.0                     # suppressed id must never win
    logits[1, 2, 7] = logits[1, 2, 11] = 50.0   # tie -> lowest index
    post = O.greedy_tokens_with_mask(logits, sup)
    assert post[0, 3] != 4 and post[1, 2] == 7 and post.dtype == np.uint32
    ids = np.concatenate([np.full((2, 1), 1), post[:, :-1].astype(np.int64)], axis=1)
    ids[1, 6] = (ids[1, 6] + 1) % 50            # sequence 1 diverges at drafted index 5
    pc, acc, nxt = CO.accept(logits, ids, sup)
    np.testing.assert_array_equal(pc, post)
    assert list(acc) == [15, 5]
    for b in range(2):
        a, commit, staged = O.accept_block(ids[b], post[b])
        assert (a, commit, staged) == (acc[b], acc[b] + 1, nxt[b])


def test_rollback_indexing_contract():
    assert O.rollback_accepted_steps(0) == 1 and O.rollback_accepted_steps(6) == 7
    assert O.fully_accepted(15, 15) and not O.fully_accepted(3, 15) and not O.fully_accepted(0, 0)
    snap = np.arange(2 * 3 * 2).reshape(2, 3, 2)
    qkv = 100 + np.arange(2 * 16 * 2).reshape(2, 16, 2)
    for acc in (1, 5, 16):
        got = O.rebuild_conv_state(snap, qkv, acc, 4)
        cat = np.concatenate([snap, qkv], 1)
        np.testing.assert_array_equal(got, cat[:, acc:acc + 3])
        assert got.shape[1] == 3
    z = O.rebuild_conv_state(None, qkv, 1, 4)
    assert (z[:, :2] == 0).all() and (z[:, 2] == qkv[:, 0]).all()
    assert O.rebuild_conv_state(snap, qkv, 2, 1) is None


def test_torch_ops_restatement_matches_numpy_oracle():
    """The op-for-op Torch-CPU statement (timed by bench.py as the reference's CPU structure) against the NumPy one."""
    from oracle.torch_ops_oracle import gated_delta_ops_torch
    for vec in (False, True):
        x = O.make_gdn_inputs(2, 16, 2, 4, 64, 32, 77 + vec, vec)
        mask = (np.arange(16)[None, :] < x["n"][:, None]).astype(np.float32)
        y, s, tape = gated_delta_ops_torch(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"], mask)
        yo, so, to = O.gated_delta_ops_with_tape(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"], n_per_seq=x["n"])
        assert np.abs(s.numpy() - so).max() <= 1e-5 * np.abs(so).max()
        assert np.abs(y.numpy() - yo).max() <= 1e-5 * max(np.abs(yo).max(), 1e-30)
        assert np.abs(tape.numpy() - to).max() <= 1e-5 * max(np.abs(to).max(), 1e-30)
