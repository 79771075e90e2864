"""GPU tests of the rollback cache mirror (Sources/DFlash/RecurrentRollbackCache.swift:34-182): the conv-window
rebuild is byte-exact against the oracle, and rollback(n_accepted) leaves the state that a forward pass over
n_accepted + 1 steps leaves."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as CO
from oracle import dflash_oracle as O
from swiftlm_b200.rollback_cache import RecurrentRollbackCache

pytestmark = pytest.mark.gpu


def K():
    from swiftlm_b200 import kernels
    return kernels


def test_conv_window_rebuild_matches_oracle_exactly():
    c = RecurrentRollbackCache(conv_kernel_size=4)
    snap = torch.arange(2 * 3 * 8).reshape(2, 3, 8).float().cuda()
    qkv = (100 + torch.arange(2 * 16 * 8).reshape(2, 16, 8).float()).cuda()
    c.state = [snap, None]
    c.arm_rollback()
    c.record_tape(None, None, None, qkv)
    for steps in (1, 2, 7, 16, 17, 18):
        got = c.rebuild_conv_state(steps)
        want = O.rebuild_conv_state(snap.cpu().numpy(), qkv.cpu().numpy(), steps, 4)
        np.testing.assert_array_equal(got.cpu().numpy(), want)
    # per-sequence step counts: each row equals the scalar rule for its own count
    steps = torch.tensor([3, 12], dtype=torch.int32).cuda()
    got = c.rebuild_conv_state(steps)
    for b in range(2):
        want = O.rebuild_conv_state(snap.cpu().numpy()[b:b + 1], qkv.cpu().numpy()[b:b + 1], int(steps[b]), 4)
        np.testing.assert_array_equal(got[b:b + 1].cpu().numpy(), want)
    # no snapshot -> zero prefix; kernel size 1 -> no window; bf16 rows
    c2 = RecurrentRollbackCache(conv_kernel_size=4)
    c2.arm_rollback()
    c2.record_tape(None, None, None, qkv)
    np.testing.assert_array_equal(c2.rebuild_conv_state(1).cpu().numpy(), O.rebuild_conv_state(None, qkv.cpu().numpy(), 1, 4))
    c3 = RecurrentRollbackCache(conv_kernel_size=1)
    c3.arm_rollback()
    c3.record_tape(None, None, None, qkv)
    assert c3.rebuild_conv_state(1) is None
    qb = qkv.bfloat16()
    got = K().rebuild_conv_state(snap.bfloat16(), qb, 5, 3)
    want = torch.cat([snap.bfloat16(), qb], dim=1)[:, 5:8]
    assert torch.equal(got, want)


@pytest.mark.parametrize("per_sequence", [False, True])
def test_rollback_equals_forward_to_accepted_length(per_sequence):
    x = O.make_gdn_inputs(3, 16, 2, 4, 128, 128, 77, False, "bf16")
    bf = torch.bfloat16
    dev = lambda a, dt=None: (torch.from_numpy(np.ascontiguousarray(a)).cuda() if dt is None
                              else torch.from_numpy(np.ascontiguousarray(a)).cuda().to(dt))  # noqa: E731
    q, k, v, g, beta, s0 = dev(x["q"], bf), dev(x["k"], bf), dev(x["v"], bf), dev(x["g"], bf), dev(x["beta"], bf), dev(x["state"])
    conv0 = torch.randn(3, 3, 64, device="cuda").bfloat16()
    qkv = torch.randn(3, 16, 64, device="cuda").bfloat16()
    c = RecurrentRollbackCache(conv_kernel_size=4)
    c.state = [conv0, s0]
    c.arm_rollback()
    _, s_verify, tape = K().gated_delta_kernel_with_tape(q, k, v, g, beta, s0)     # the verify pass over the whole block
    c.state[1] = s_verify
    c.record_tape(tape, k, g, qkv)
    n_acc = np.array([4, 0, 15], np.int32) if per_sequence else np.array([6, 6, 6], np.int32)
    c.rollback(torch.from_numpy(n_acc).cuda() if per_sequence else 6)
    torch.cuda.synchronize()
    K().device_status()
    _, want_state, _ = CO.gated_delta(x["q"], x["k"], x["v"], x["g"], x["beta"], x["state"], n=n_acc + 1)
    got = c.state[1].cpu().numpy()
    assert np.abs(got - want_state).max() <= 1e-4 * np.abs(want_state).max()
    full = torch.cat([conv0, qkv], dim=1)
    for b in range(3):
        st = int(n_acc[b]) + 1
        assert torch.equal(c.state[0][b], full[b, st:st + 3])
    assert not c.is_armed
