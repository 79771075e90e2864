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
