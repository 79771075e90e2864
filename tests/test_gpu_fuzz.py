"""Shape fuzzing of the kernels against the C oracle (hypothesis, derandomised so that a run is repeatable):
small shapes over every dispatch dimension - head counts and ratios, head sizes, block lengths, both gates, step
masks together with accepted lengths, ragged KV lengths, grouping factors."""
import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from oracle import c_oracle as CO
from oracle import dflash_oracle as O

pytestmark = pytest.mark.gpu
TORCH_DT = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}
FUZZ = settings(max_examples=40, deadline=None, derandomize=True, suppress_health_check=list(HealthCheck))


def K():
    from swiftlm_b200 import kernels
    return kernels


def dev(x, dt=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if dt is None else t.to(dt)


def rel(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


@FUZZ
@given(B=st.integers(1, 5), T=st.integers(1, 24), Hk=st.integers(1, 4), ratio=st.integers(1, 3),
       Dk=st.sampled_from([32, 64, 128, 128, 128, 256]), Dv=st.sampled_from([32, 48, 128, 128]),
       vec=st.booleans(), dtype=st.sampled_from(["fp32", "bf16", "bf16", "fp16"]), masked=st.booleans(),
       use_n=st.booleans(), seed=st.integers(0, 10 ** 6))
def test_gated_delta_and_replay_fuzz(B, T, Hk, ratio, Dk, Dv, vec, dtype, masked, use_n, seed):
    Hv = Hk * ratio
    x = O.make_gdn_inputs(B, T, Hk, Hv, Dk, Dv, seed, vec, dtype)
    rng = np.random.default_rng(seed + 1)
    x["n"] = rng.integers(0, T + 1, B).astype(np.int32)
    mask = (rng.random((B, T)) > 0.3).astype(np.float32) if masked else None
    n = x["n"] if use_n else None
    dt = TORCH_DT[dtype]
    y, s, tape = K().gated_delta_kernel_with_tape(dev(x["q"], dt), dev(x["k"], dt), dev(x["v"], dt), dev(x["g"], dt),
                                                  dev(x["beta"], dt), dev(x["state"]), mask=None if mask is None else dev(mask),
                                                  n_per_seq=None if n is None else dev(n))
    s_rep = K().tape_replay_kernel(tape, dev(x["k"], dt), dev(x["g"], dt), dev(x["state"]),
                                   mask=None if mask is None else dev(mask), n_per_seq=None if n is None else dev(n))
    torch.cuda.synchronize()
    K().device_status()
    yo, so, to = CO.gated_delta(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"], mask=mask, n=n)
    assert rel(s.cpu().numpy(), so) < 1e-4
    assert rel(tape.cpu().numpy(), to) < 1e-4
    assert rel(y.float().cpu().numpy(), yo) < {"fp32": 1e-4, "bf16": 1.0 / 128, "fp16": 1.0 / 1024}[dtype]
    np.testing.assert_array_equal(tape.cpu().numpy() == 0, to == 0)
    assert rel(s_rep.cpu().numpy(), so) < 1e-4               # replaying the recorded tape gives the forward's state


@FUZZ
@given(B=st.integers(1, 6), Hkv=st.integers(1, 4), G=st.sampled_from([1, 2, 4, 8, 16]), D=st.sampled_from([128, 256]),
       n_ctx=st.integers(0, 1500), dtype=st.sampled_from(["bf16", "fp16"]), ragged=st.booleans(), seed=st.integers(0, 10 ** 6))
def test_verify_sdpa_fuzz(B, Hkv, G, D, n_ctx, dtype, ragged, seed):
    Hq = Hkv * G
    N = 16 + n_ctx
    x = O.make_sdpa_inputs(B, Hq, Hkv, N, D, seed, dtype)
    lens = None
    if ragged:
        lens = np.random.default_rng(seed + 2).integers(16, N + 1, B).astype(np.int32)
    dt = TORCH_DT[dtype]
    out = K().batched_sdpa_2pass(dev(x["q"], dt), dev(x["k"], dt), dev(x["v"], dt), float(x["scale"]), kv_len=lens)
    torch.cuda.synchronize()
    K().device_status()
    want = CO.verify_sdpa(x["q"], x["k"], x["v"], float(x["scale"]), kv_len=lens)
    assert np.abs(out.float().cpu().numpy() - want).max() < 2e-2


@settings(max_examples=16, deadline=None, derandomize=True, suppress_health_check=list(HealthCheck))
@given(B=st.integers(1, 5), Hkv=st.integers(1, 3), G=st.sampled_from([1, 4, 8, 16]), D=st.sampled_from([128, 256]),
       cold_tiles=st.integers(1, 9), n_hot=st.sampled_from([0, 16, 40, 128, 272]), dtype=st.sampled_from(["bf16", "bf16", "fp16"]),
       seed=st.integers(0, 10 ** 6))
def test_attention_over_compressed_kv_fuzz(B, Hkv, G, D, cold_tiles, n_hot, dtype, seed):
    """The fused attention over TurboQuant KV (cold history of whole 128-key tiles, any hot window) against the oracle's
    decode-then-attend."""
    Hq, n_cold = Hkv * G, 128 * cold_tiles
    N = n_cold + n_hot
    x = O.make_sdpa_inputs(B, Hq, Hkv, N, D, seed, dtype)
    dt = TORCH_DT[dtype]
    k, v, q = dev(x["k"], dt), dev(x["v"], dt), dev(x["q"], dt)
    k_enc = K().turbo_encode(k[:, :, :n_cold].contiguous(), True)
    vp, _, vn, _ = K().turbo_encode(v[:, :, :n_cold].contiguous(), False)
    out = K().batched_sdpa_turbo_kv(q, k_enc, (vp, vn), n_cold, float(x["scale"]),
                                    k_hot=k[:, :, n_cold:].contiguous() if n_hot else None,
                                    v_hot=v[:, :, n_cold:].contiguous() if n_hot else None)
    torch.cuda.synchronize()
    K().device_status()
    rnd = O.round_bf16 if dtype == "bf16" else (lambda a: a.astype(np.float16).astype(np.float32))
    p, s_, n_, r_ = CO.turbo_encode_k(x["k"][:, :, :n_cold].reshape(-1, 128))
    k_ref = np.concatenate([rnd(CO.turbo_decode_k(p, s_, n_, r_)).reshape(B, Hkv, n_cold, D), x["k"][:, :, n_cold:]], axis=2)
    p, n_ = CO.turbo_encode_v(x["v"][:, :, :n_cold].reshape(-1, 128))
    v_ref = np.concatenate([rnd(CO.turbo_decode_v(p, n_)).reshape(B, Hkv, n_cold, D), x["v"][:, :, n_cold:]], axis=2)
    want = CO.verify_sdpa(x["q"], k_ref, v_ref, float(x["scale"]))
    assert np.abs(out.float().cpu().numpy() - want).max() < 2e-2
