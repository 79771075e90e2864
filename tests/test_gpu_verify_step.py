"""The composed DFlash verify step (dflash_verify_step through swiftlm_b200/verify_step.py) against the oracle's
composition of the same pieces: every layer's verify output, the attention over TurboQuant KV, acceptance
(bit-exact), the logits rows, and the rolled-back states and conv windows.  Once on a small stack, once at the
benchmark definition's configs[4] shape (36 gated-delta + 12 attention layers, context 8192, vocabulary
151 936) on a sub-batch of its 64 sequences."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as CO
from oracle import dflash_oracle as O

pytestmark = pytest.mark.gpu


def f(t):
    return t.float().cpu().numpy()


def rel(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def check_step(cfg, attn_items):
    from swiftlm_b200 import kernels
    from swiftlm_b200.verify_step import VerifyStep
    step = VerifyStep(cfg, torch.device("cuda", 0))
    launches0 = kernels.launch_count()
    r = step.run()
    torch.cuda.synchronize()
    kernels.device_status()
    launches = kernels.launch_count() - launches0
    B, L, A, T = cfg.batch, cfg.gdn_layers, cfg.attn_layers, cfg.T
    # acceptance: bit-exact
    post, acc, nxt = CO.accept(f(step.logits), step.verify_ids.cpu().numpy())
    np.testing.assert_array_equal(r["accept"].cpu().numpy(), acc)
    np.testing.assert_array_equal(r["next_token"].cpu().numpy(), nxt)
    replay = (acc + 1).astype(np.int32)
    np.testing.assert_array_equal(r["replay_len"].cpu().numpy(), replay)
    assert len(set(acc.tolist())) > 1 or B == 1              # the synthetic drafts disagree at different places
    rows = r["logits_rows"]
    assert torch.equal(rows, torch.stack([step.logits[b, int(acc[b])] for b in range(B)]))
    # gated-delta layers: verify forward over the whole block, rollback to each sequence's replay length
    yo, so, to = CO.gated_delta(f(step.q), f(step.k), f(step.v), f(step.g), f(step.beta), f(step.state))
    e = dict(state_verify=rel(f(r["state_verify"]), so), tape=rel(f(r["tape"]), to), y=rel(f(r["y"]), yo))
    del yo, so
    n_items = np.repeat(replay, L)
    _, s_want, _ = CO.gated_delta(f(step.q), f(step.k), f(step.v), f(step.g), f(step.beta), f(step.state), n=n_items, want_tape=False)
    e["state_rolled"] = rel(f(r["states"]), s_want)
    del s_want
    full = torch.cat([step.conv, step.qkv], dim=1)
    keep = cfg.conv_kernel - 1
    for i in range(0, B * L, max(1, (B * L) // 40)):
        st = int(n_items[i])
        assert torch.equal(r["convs"][i], full[i, st:st + keep])
    # attention over the compressed history plus the block's own tokens, against decode-then-attend
    kv = step.kv
    errs = []
    for j in attn_items:
        sl = slice(j, j + 1)
        k_cold = O.round_bf16(CO.turbo_decode_k(kv["kp"][sl].cpu().numpy().reshape(-1, 48), kv["ks"][sl].cpu().numpy().reshape(-1, 16),
                                                kv["kn"][sl].cpu().numpy().reshape(-1).view(np.uint16),
                                                kv["kr"][sl].cpu().numpy().reshape(-1).view(np.uint16))).reshape(1, cfg.Hkv, cfg.context, cfg.D)
        v_cold = O.round_bf16(CO.turbo_decode_v(kv["vp"][sl].cpu().numpy().reshape(-1, 48),
                                                kv["vn"][sl].cpu().numpy().reshape(-1).view(np.uint16))).reshape(1, cfg.Hkv, cfg.context, cfg.D)
        k_ref = np.concatenate([k_cold, f(kv["kh"][sl])], axis=2)
        v_ref = np.concatenate([v_cold, f(kv["vh"][sl])], axis=2)
        want = CO.verify_sdpa(f(step.attn_q[sl]), k_ref, v_ref, step.scale)
        errs.append(float(np.abs(f(r["attn_out"][sl]) - want).max()))
    e["attention_abs"] = max(errs)
    print(f"\n[verify step B={B} L={L}+{A}] launches {launches}; errors {e}")
    assert e["state_verify"] < 1e-4 and e["tape"] < 1e-4 and e["y"] < 1.0 / 128 and e["state_rolled"] < 1e-4
    assert e["attention_abs"] < 2e-2
    assert launches <= 16                                     # a handful of launches, not one per layer
    # a second step from the same committed state gives the same bits
    again = step.run()
    torch.cuda.synchronize()
    assert torch.equal(again["states"], r["states"]) and torch.equal(again["attn_out"], r["attn_out"])


def test_small_step_matches_oracle_composition():
    from swiftlm_b200.verify_step import StepConfig
    cfg = StepConfig(batch=3, gdn_layers=3, attn_layers=2, Hk=2, Hv=4, Hq=16, Hkv=2, D=256, context=384, vocab=4096, conv_dim=64)
    check_step(cfg, attn_items=range(cfg.batch * cfg.attn_layers))


def test_config4_shape_on_a_sequence_sub_batch():
    from swiftlm_b200.verify_step import StepConfig
    cfg = StepConfig(batch=4)                                 # every other field at the benchmark definition's value
    check_step(cfg, attn_items=[0, 17, 47])


def test_step_without_the_verify_forwards_final_state():
    """state_verify = NULL: the forward writes no state; outputs, tape, rolled-back states and acceptance are the same
    bits as with it."""
    from swiftlm_b200.verify_step import StepConfig, VerifyStep
    kw = dict(batch=3, gdn_layers=3, attn_layers=2, Hk=2, Hv=4, Hq=16, Hkv=2, D=256, context=384, vocab=4096, conv_dim=64)
    dev = torch.device("cuda", 0)
    a = VerifyStep(StepConfig(**kw), dev).run()
    b = VerifyStep(StepConfig(keep_state_verify=False, **kw), dev).run()
    torch.cuda.synchronize()
    assert b["state_verify"] is None
    for name in ("y", "tape", "states", "convs", "accept", "next_token", "replay_len", "attn_out"):
        assert torch.equal(a[name], b[name]), name



def test_step_replayed_from_a_cuda_graph():
    """The step captured once into a CUDA graph and replayed over new activations, states and logits gives the bits of a
    direct call on the same inputs (the accepted lengths change from replay to replay and never leave the device)."""
    from swiftlm_b200 import kernels
    from swiftlm_b200.verify_step import StepConfig, VerifyStep
    cfg = StepConfig(batch=5, gdn_layers=3, attn_layers=2, Hk=2, Hv=4, Hq=16, Hkv=2, D=256, context=1024, vocab=4096, conv_dim=64)
    step = VerifyStep(cfg, torch.device("cuda", 0))
    step.run()                                                # attributes set, nothing left to allocate
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step.run()
    names = ("y", "tape", "states", "convs", "accept", "next_token", "replay_len", "attn_out", "logits_rows")
    g = torch.Generator(device="cuda").manual_seed(77)
    seen = set()
    for _ in range(3):
        for t in (step.q, step.k, step.v, step.attn_q, step.qkv, step.logits):
            t.copy_(torch.randn(t.shape, device="cuda", generator=g))
        step.state.copy_(0.02 * torch.randn(step.state.shape, device="cuda", generator=g))
        post = kernels.greedy_tokens_with_mask(step.logits).to(torch.int32)
        agree = torch.randint(0, cfg.T, (cfg.batch,), device="cuda", generator=g)
        ids = torch.zeros(cfg.batch, cfg.T, dtype=torch.int32, device="cuda")
        ids[:, 1:] = post[:, :-1]
        wrong = torch.arange(cfg.T - 1, device="cuda").view(1, -1) >= agree.view(-1, 1)
        ids[:, 1:][wrong] = (ids[:, 1:][wrong] + 1) % cfg.vocab
        step.verify_ids.copy_(ids)
        graph.replay()
        torch.cuda.synchronize()
        got = {n: getattr_out(step, n).clone() for n in names}
        step.run()
        torch.cuda.synchronize()
        for n in names:
            assert torch.equal(got[n], getattr_out(step, n)), n
        seen.add(tuple(step.accept.cpu().tolist()))
    kernels.device_status()
    assert len(seen) > 1                                      # the replays really ran on different acceptance patterns


def getattr_out(step, name):
    return {"states": step.state_rolled, "convs": step.conv_out}.get(name, getattr(step, name, None))
