"""The composed DFlash verify step (swiftlm_b200/verify_step.py) on a small hybrid stack against the
oracle's composition of the same pieces: every layer's verify output, the attention over TurboQuant KV,
acceptance (bit-exact) and the rolled-back states and conv windows."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as CO
from oracle import dflash_oracle as O

pytestmark = pytest.mark.gpu


def test_small_step_matches_oracle_composition():
    from swiftlm_b200 import kernels
    from swiftlm_b200.verify_step import StepConfig, VerifyStep
    cfg = StepConfig(batch=3, gdn_layers=3, attn_layers=1, Hk=2, Hv=4, Hq=16, Hkv=2, D=256, context=384, vocab=4096,
                     conv_dim=64)
    step = VerifyStep(cfg, torch.device("cuda", 0))
    r = step.run()
    torch.cuda.synchronize()
    kernels.device_status()
    f = lambda t: t.float().cpu().numpy()  # noqa: E731
    # acceptance: bit-exact
    post, acc, nxt = CO.accept(f(step.logits), step.verify_ids.cpu().numpy())
    np.testing.assert_array_equal(r["accept"].cpu().numpy(), acc)
    np.testing.assert_array_equal(r["next_token"].cpu().numpy(), nxt)
    replay = acc + 1
    np.testing.assert_array_equal(r["replay_len"].cpu().numpy(), replay)
    assert len(set(acc.tolist())) > 1 or cfg.batch == 1          # the synthetic drafts disagree at different places
    rel = lambda a, b: float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))  # noqa: E731
    for L, (y, s_verify, tape), s_roll, conv in zip(step.gdn, r["verify"], r["states"], r["convs"]):
        yo, so, to = CO.gated_delta(f(L["q"]), f(L["k"]), f(L["v"]), f(L["g"]), f(L["beta"]), f(L["state"]))
        assert rel(f(s_verify), so) < 1e-4 and rel(f(tape), to) < 1e-4 and rel(f(y), yo) < 1.0 / 128
        _, s_want, _ = CO.gated_delta(f(L["q"]), f(L["k"]), f(L["v"]), f(L["g"]), f(L["beta"]), f(L["state"]),
                                      n=replay.astype(np.int32))
        assert rel(f(s_roll), s_want) < 1e-4
        full = torch.cat([L["conv"], L["qkv"]], dim=1)
        for b in range(cfg.batch):
            assert torch.equal(conv[b], full[b, int(replay[b]):int(replay[b]) + cfg.conv_kernel - 1])
    a = step.attn[0]
    cold = cfg.context
    k_cold = O.round_bf16(CO.turbo_decode_k(a["kp"].cpu().numpy().reshape(-1, 48), a["ks"].cpu().numpy().reshape(-1, 16),
                                            a["kn"].cpu().numpy().reshape(-1).view(np.uint16),
                                            a["kr"].cpu().numpy().reshape(-1).view(np.uint16))).reshape(cfg.batch, cfg.Hkv, cold, cfg.D)
    v_cold = O.round_bf16(CO.turbo_decode_v(a["vp"].cpu().numpy().reshape(-1, 48),
                                            a["vn"].cpu().numpy().reshape(-1).view(np.uint16))).reshape(cfg.batch, cfg.Hkv, cold, cfg.D)
    k_ref = np.concatenate([k_cold, f(a["k_hot"])], axis=2)
    v_ref = np.concatenate([v_cold, f(a["v_hot"])], axis=2)
    want = CO.verify_sdpa(f(a["q"]), k_ref, v_ref, step.scale)
    assert np.abs(f(r["attn_out"][0]) - want).max() < 2e-2
