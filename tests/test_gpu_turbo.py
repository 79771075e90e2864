"""GPU parity of the TurboQuant 3-bit KV codec: bytes, fp16 norms and decoded floats must equal
the CPU oracle (itself pinned bit for bit against the reference's compiled codec) exactly."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as CO

pytestmark = pytest.mark.gpu


def K():
    from swiftlm_b200 import kernels
    return kernels


@pytest.mark.parametrize("is_key", [False, True], ids=["V", "K"])
def test_codec_bit_exact_against_oracle(is_key):
    rng = np.random.default_rng(31 + is_key)
    x = rng.standard_normal((300, 128)).astype(np.float32)
    x[7] = 0.0                      # zero vector: the 1e-10 guards
    x[8] *= 1e-6
    x[9] *= 1e2
    xt = torch.from_numpy(x).cuda()
    packed, signs, norm, rnorm = K().turbo_encode(xt, is_key)
    torch.cuda.synchronize()
    if is_key:
        p, s, n, r = CO.turbo_encode_k(x)
        np.testing.assert_array_equal(signs.cpu().numpy()[:, 0], s)
        np.testing.assert_array_equal(rnorm.cpu().numpy()[:, 0].view(np.uint16), r)
    else:
        p, n = CO.turbo_encode_v(x)
    np.testing.assert_array_equal(packed.cpu().numpy()[:, 0], p)
    np.testing.assert_array_equal(norm.cpu().numpy()[:, 0].view(np.uint16), n)
    dec = K().turbo_decode(packed, signs, norm, rnorm, dtype=torch.float32).cpu().numpy()
    want = CO.turbo_decode_k(p, s, n, r) if is_key else CO.turbo_decode_v(p, n)
    np.testing.assert_array_equal(dec, want)
    # quality bar of the reference's own test (SNR > 9 dB)
    good = np.ones(300, bool)
    good[7] = False
    rel = ((dec[good] - x[good]) ** 2).sum() / (x[good] ** 2).sum()
    assert rel < 0.15


def test_encode_of_an_unaligned_input_takes_the_bytewise_kernel_and_agrees():
    """The register-resident encoder needs 16-byte aligned arrays; anything else takes the byte-wise kernel.  Both
    must produce the same bytes."""
    g = torch.Generator(device="cuda").manual_seed(9)
    buf = torch.randn(2 + 70 * 128, device="cuda", generator=g)
    x_off = buf[2:].view(70, 128)                       # 8 bytes past a 16-byte boundary
    assert x_off.data_ptr() % 16 != 0
    x_al = x_off.clone()
    for is_key in (False, True):
        a = K().turbo_encode(x_off, is_key)
        b = K().turbo_encode(x_al, is_key)
        for u, v in zip(a, b):
            assert (u is None and v is None) or torch.equal(u, v)


def test_head_dim_256_is_two_blocks_and_bf16_io():
    g = torch.Generator(device="cuda").manual_seed(5)
    kv = torch.randn(2, 2, 40, 256, device="cuda", generator=g).bfloat16()
    packed, signs, norm, rnorm = K().turbo_encode(kv, True)
    assert packed.shape == (2, 2, 40, 2, 48) and signs.shape == (2, 2, 40, 2, 16) and norm.shape == (2, 2, 40, 2)
    dec = K().turbo_decode(packed, signs, norm, rnorm, dtype=torch.bfloat16)
    assert dec.shape == kv.shape
    p, s, n, r = CO.turbo_encode_k(kv.float().cpu().numpy().reshape(-1, 128))
    np.testing.assert_array_equal(packed.cpu().numpy().reshape(-1, 48), p)
    want = CO.turbo_decode_k(p, s, n, r).reshape(kv.shape)
    got = dec.float().cpu().numpy()
    assert np.abs(got - want).max() <= np.abs(want).max() / 128      # one bf16 rounding of the fp32 decode


def test_attention_over_turbo_compressed_kv():
    """KV held in the 3-bit format, expanded on the device, then block-verify attention: the result
    must match the oracle's attention over the oracle's decode of the oracle's encode (2e-2 absolute),
    and stay close to attention over the uncompressed KV (the codec's ~9 dB SNR on K and V)."""
    from oracle import dflash_oracle as O
    B, Hq, Hkv, N, D = 2, 16, 2, 16 + 1500, 256
    x = O.make_sdpa_inputs(B, Hq, Hkv, N, D, 4242, "bf16")
    k = torch.from_numpy(x["k"]).cuda().bfloat16()
    v = torch.from_numpy(x["v"]).cuda().bfloat16()
    q = torch.from_numpy(x["q"]).cuda().bfloat16()
    kp, ks, kn, kr = K().turbo_encode(k, True)
    vp, _, vn, _ = K().turbo_encode(v, False)
    k_hat = K().turbo_decode(kp, ks, kn, kr, dtype=torch.bfloat16)
    v_hat = K().turbo_decode(vp, None, vn, None, dtype=torch.bfloat16)
    out = K().batched_sdpa_2pass(q, k_hat, v_hat, float(x["scale"]))
    torch.cuda.synchronize()
    K().device_status()
    # compressed footprint: 48 + 16 + 2 + 2 bytes per 128 K values, 48 + 2 per 128 V values
    assert kp[0, 0, 0].numel() + ks[0, 0, 0].numel() + 4 * kn[0, 0, 0].numel() == (D // 128) * 68
    p, s, n, r = CO.turbo_encode_k(x["k"].reshape(-1, 128))
    k_ref = O.round_bf16(CO.turbo_decode_k(p, s, n, r)).reshape(x["k"].shape)
    p, n = CO.turbo_encode_v(x["v"].reshape(-1, 128))
    v_ref = O.round_bf16(CO.turbo_decode_v(p, n)).reshape(x["v"].shape)
    want = CO.verify_sdpa(x["q"], k_ref, v_ref, float(x["scale"]))
    assert np.abs(out.float().cpu().numpy() - want).max() < 2e-2


def _turbo_case(B, Hq, Hkv, D, n_cold, n_hot, dtype, seed):
    """Returns (fused output, decode-then-attend output on the GPU, oracle output) for one shape."""
    from oracle import dflash_oracle as O
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float16
    N = n_cold + n_hot
    x = O.make_sdpa_inputs(B, Hq, Hkv, N, D, seed, dtype)
    k = torch.from_numpy(x["k"]).cuda().to(tdt)
    v = torch.from_numpy(x["v"]).cuda().to(tdt)
    q = torch.from_numpy(x["q"]).cuda().to(tdt)
    k_enc = K().turbo_encode(k[:, :, :n_cold].contiguous(), True)
    vp, _, vn, _ = K().turbo_encode(v[:, :, :n_cold].contiguous(), False)
    k_hot = k[:, :, n_cold:].contiguous() if n_hot else None
    v_hot = v[:, :, n_cold:].contiguous() if n_hot else None
    launches0 = K().launch_count()
    fused = K().batched_sdpa_turbo_kv(q, k_enc, (vp, vn), n_cold, float(x["scale"]), k_hot=k_hot, v_hot=v_hot)
    launches = K().launch_count() - launches0
    k_hat = K().turbo_decode(*k_enc, dtype=tdt)
    v_hat = K().turbo_decode(vp, None, vn, None, dtype=tdt)
    if n_hot:
        k_hat, v_hat = torch.cat([k_hat, k_hot], dim=2), torch.cat([v_hat, v_hot], dim=2)
    two_step = K().batched_sdpa_2pass(q, k_hat, v_hat, float(x["scale"]))
    torch.cuda.synchronize()
    K().device_status()
    assert fused is not None
    # the oracle: its decode of its own encode for the cold part, the hot part as given
    rnd = O.round_bf16 if dtype == "bf16" else (lambda a: a.astype(np.float16).astype(np.float32))
    p, s_, n_, r_ = CO.turbo_encode_k(x["k"][:, :, :n_cold].reshape(-1, 128))
    k_ref = rnd(CO.turbo_decode_k(p, s_, n_, r_)).reshape(B, Hkv, n_cold, D)
    p, n_ = CO.turbo_encode_v(x["v"][:, :, :n_cold].reshape(-1, 128))
    v_ref = rnd(CO.turbo_decode_v(p, n_)).reshape(B, Hkv, n_cold, D)
    k_ref = np.concatenate([k_ref, x["k"][:, :, n_cold:]], axis=2)
    v_ref = np.concatenate([v_ref, x["v"][:, :, n_cold:]], axis=2)
    want = CO.verify_sdpa(x["q"], k_ref, v_ref, float(x["scale"]))
    return fused, two_step, want, launches


FUSED_CASES = [
    # B, Hq, Hkv, D, n_cold, n_hot, dtype
    (2, 16, 2, 256, 768, 16, "bf16"),       # the production head shape, the block as the hot window
    (2, 16, 2, 256, 768, 0, "bf16"),        # no hot window: the block's own keys are compressed too
    (2, 16, 2, 256, 768, 256, "bf16"),      # the reference's hot window of 256 tokens
    (3, 8, 2, 128, 384, 100, "bf16"),       # one 128-block per head vector, ragged hot window, GQA 4
    (1, 32, 8, 128, 1280, 16, "fp16"),      # fp16 operands, the reference bench's head shape
    (1, 16, 1, 256, 512, 16, "bf16"),       # GQA 16: two query tiles per KV head
    (40, 16, 2, 256, 1024, 16, "bf16"),     # 80 units: whole units and stream-K pieces, last finisher merges
    (20, 16, 2, 256, 896, 16, "bf16"),      # 40 units: three equal cuts per unit
    (64, 16, 2, 256, 256, 16, "bf16"),      # 128 units of three tiles
    (1, 16, 2, 256, 8192, 16, "bf16"),      # one sequence: a key range per SM, combined by the merge kernel
    (37, 16, 2, 256, 128, 16, "bf16"),      # 74 units of two tiles: two cuts per unit, merged through the partials
]


@pytest.mark.parametrize("case", FUSED_CASES, ids=lambda c: "x".join(map(str, c)))
def test_fused_attention_over_compressed_kv(case):
    """dflash_verify_sdpa with DFLASH_KV_TURBO3 on a cold history of whole 128-key tiles: the kernel expands packed
    indices and sign bits straight into its tensor-core operands (rotated domain), no decoded key or value is written.
    Checked against decode-then-attend, both the library's own two-step route and the oracle's."""
    B, Hq, Hkv, D, n_cold, n_hot, dtype = case
    fused, two_step, want, launches = _turbo_case(B, Hq, Hkv, D, n_cold, n_hot, dtype, 4343 + n_cold + n_hot + B)
    e_oracle = float(np.abs(fused.float().cpu().numpy() - want).max())
    e_two = float((fused.float() - two_step.float()).abs().max())
    print(f"\n[fused turbo attention {case}] vs oracle {e_oracle:.3e}, vs decode-then-attend on the GPU {e_two:.3e}, launches {launches}")
    assert e_oracle < 2e-2 and e_two < 2e-2
    assert launches <= 4            # rotate in, attention (+ merge), rotate out: no decode launches


@pytest.mark.parametrize("n_hot", [0, 16, 256])
def test_expanded_route_for_a_history_that_is_not_whole_tiles(n_hot):
    """A cold history that is not a multiple of 128 keys takes the expand route: same bits as decoding and concatenating
    first."""
    fused, two_step, want, _ = _turbo_case(2, 16, 2, 256, 700, n_hot if n_hot else 16, "bf16", 4343 + n_hot)
    assert torch.equal(fused, two_step)
    assert np.abs(fused.float().cpu().numpy() - want).max() < 2e-2
