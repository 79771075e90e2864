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


@pytest.mark.parametrize("n_hot", [0, 16, 256])
def test_turbo_kv_format_of_the_attention_entry_point(n_hot):
    """dflash_verify_sdpa with DFLASH_KV_TURBO3: the cold history is expanded inside the library, the hot window
    (the reference keeps the newest tokens uncompressed) is appended: same bits as decoding and concatenating first."""
    from oracle import dflash_oracle as O
    B, Hq, Hkv, D = 2, 16, 2, 256
    n_cold = 768
    N = n_cold + n_hot if n_hot else n_cold + 16
    x = O.make_sdpa_inputs(B, Hq, Hkv, N, D, 4343 + n_hot, "bf16")
    k = torch.from_numpy(x["k"]).cuda().bfloat16()
    v = torch.from_numpy(x["v"]).cuda().bfloat16()
    q = torch.from_numpy(x["q"]).cuda().bfloat16()
    cold = N - n_hot
    k_enc = K().turbo_encode(k[:, :, :cold].contiguous(), True)
    vp, _, vn, _ = K().turbo_encode(v[:, :, :cold].contiguous(), False)
    k_hot = k[:, :, cold:].contiguous() if n_hot else None
    v_hot = v[:, :, cold:].contiguous() if n_hot else None
    fused = K().batched_sdpa_turbo_kv(q, k_enc, (vp, vn), cold, float(x["scale"]), k_hot=k_hot, v_hot=v_hot)
    k_hat = K().turbo_decode(*k_enc, dtype=torch.bfloat16)
    v_hat = K().turbo_decode(vp, None, vn, None, dtype=torch.bfloat16)
    if n_hot:
        k_hat, v_hat = torch.cat([k_hat, k_hot], dim=2), torch.cat([v_hat, v_hot], dim=2)
    two_step = K().batched_sdpa_2pass(q, k_hat, v_hat, float(x["scale"]))
    torch.cuda.synchronize()
    K().device_status()
    assert fused is not None and torch.equal(fused, two_step)
    # against the oracle: its decode of its own encode for the cold part, the hot part as given
    p, s_, n_, r_ = CO.turbo_encode_k(x["k"][:, :, :cold].reshape(-1, 128))
    k_ref = O.round_bf16(CO.turbo_decode_k(p, s_, n_, r_)).reshape(B, Hkv, cold, D)
    p, n_ = CO.turbo_encode_v(x["v"][:, :, :cold].reshape(-1, 128))
    v_ref = O.round_bf16(CO.turbo_decode_v(p, n_)).reshape(B, Hkv, cold, D)
    k_ref = np.concatenate([k_ref, x["k"][:, :, cold:]], axis=2)
    v_ref = np.concatenate([v_ref, x["v"][:, :, cold:]], axis=2)
    want = CO.verify_sdpa(x["q"], k_ref, v_ref, float(x["scale"]))
    assert np.abs(fused.float().cpu().numpy() - want).max() < 2e-2
