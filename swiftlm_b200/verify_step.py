"""One DFlash verify step over a hybrid stack of gated-delta and full-attention layers, composed from
the library's kernels the way the reference's runtime composes its own
(Sources/DFlash/DFlashRuntime.swift: verify pass over the drafted block with armed rollback caches,
greedy posterior :118-128, acceptance :133-142, commit arithmetic :523-547, cache restore :188-223;
Sources/DFlash/RecurrentRollbackCache.swift:95-131 for the per-layer rollback).

Layer weights are omitted: the per-layer q/k/v/beta/g of the gated-delta layers, the queries of the
attention layers, the KV cache (held in the TurboQuant 3-bit format and expanded per layer inside the
library's workspace) and the logits are seeded synthetic tensors.  What runs per step:
  * every gated-delta layer: forward over the whole block with tape (the verify pass);
  * every attention layer: TurboQuant decode of K and V, then block-verify attention;
  * greedy posterior tokens over the vocabulary, accepted length, next token, replay length;
  * every gated-delta layer: delta-tape replay to the per-sequence replay length, conv-window rebuild;
  * with more than one rank: an all-gather of the acceptance results.
The accepted lengths never visit the host.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from . import kernels, partition


@dataclass
class StepConfig:
    batch: int = 64
    gdn_layers: int = 36
    attn_layers: int = 12
    T: int = 16
    Hk: int = 16
    Hv: int = 32
    Dk: int = 128
    Hq: int = 16
    Hkv: int = 2
    D: int = 256
    context: int = 8192
    vocab: int = 151936
    conv_dim: int = 8192          # width of the conv window rows (q, k, v channels of a layer)
    conv_kernel: int = 4
    seed: int = 20260330 + 4000


class VerifyStep:
    def __init__(self, cfg: StepConfig, device: torch.device):
        self.cfg = c = cfg
        self.device = device
        g = torch.Generator(device=device).manual_seed(c.seed)
        bf = torch.bfloat16
        rn = lambda *s: torch.randn(*s, device=device, generator=g)  # noqa: E731
        B, T = c.batch, c.T
        self.gdn: List[Dict[str, torch.Tensor]] = []
        for _ in range(c.gdn_layers):
            self.gdn.append(dict(
                q=torch.nn.functional.normalize(rn(B, T, c.Hk, c.Dk), dim=-1).to(bf),
                k=torch.nn.functional.normalize(rn(B, T, c.Hk, c.Dk), dim=-1).to(bf),
                v=rn(B, T, c.Hv, c.Dk).to(bf),
                beta=torch.sigmoid(rn(B, T, c.Hv)).to(bf),
                g=torch.exp(-torch.nn.functional.softplus(rn(B, T, c.Hv))).to(bf),
                state=0.02 * rn(B, c.Hv, c.Dk, c.Dk),
                conv=rn(B, c.conv_kernel - 1, c.conv_dim).to(bf),
                qkv=rn(B, T, c.conv_dim).to(bf)))
        N = c.context + T
        self.N = N
        self.attn: List[Dict[str, torch.Tensor]] = []
        for _ in range(c.attn_layers):
            k = rn(B, c.Hkv, N, c.D).to(bf)
            v = rn(B, c.Hkv, N, c.D).to(bf)
            # the committed context is compressed; the block's own T tokens stay dense (the hot window)
            kp, ks, kn, kr = kernels.turbo_encode(k[:, :, :c.context].contiguous(), True)
            vp, _, vn, _ = kernels.turbo_encode(v[:, :, :c.context].contiguous(), False)
            self.attn.append(dict(q=rn(B, c.Hq, T, c.D).to(bf), kp=kp, ks=ks, kn=kn, kr=kr, vp=vp, vn=vn,
                                  k_hot=k[:, :, c.context:].contiguous(), v_hot=v[:, :, c.context:].contiguous()))
            del k, v
        self.logits = rn(B, T, c.vocab).to(bf)
        # draft ids: the staged token, then drafted tokens that agree with the posterior for a random prefix
        post = kernels.greedy_tokens_with_mask(self.logits).to(torch.int64)
        agree = torch.randint(0, T, (B,), device=device, generator=g)
        ids = torch.zeros(B, T, dtype=torch.int64, device=device)
        ids[:, 1:] = post[:, :-1]
        wrong = torch.arange(T - 1, device=device).view(1, -1) >= agree.view(-1, 1)
        ids[:, 1:][wrong] = (ids[:, 1:][wrong] + 1) % c.vocab
        self.verify_ids = ids.to(torch.int32)
        self.attn_out = [torch.empty_like(a["q"]) for a in self.attn]
        self.scale = 1.0 / float(c.D) ** 0.5

    # ---- the step -----------------------------------------------------------------------------
    def run(self, world: int = 1, n_sequences_global: Optional[int] = None, events: Optional[dict] = None):
        c = self.cfg
        mark = (lambda name: events.setdefault(name, []).append(_event())) if events is not None else (lambda name: None)
        mark("start")
        verify = []
        ai = 0
        per_attn = max(c.gdn_layers // max(c.attn_layers, 1), 1)
        for li, L in enumerate(self.gdn):
            y, s_verify, tape = kernels.gated_delta_kernel_with_tape(L["q"], L["k"], L["v"], L["g"], L["beta"], L["state"])
            verify.append((y, s_verify, tape))
            if (li + 1) % per_attn == 0 and ai < c.attn_layers:
                self._attention(ai)
                ai += 1
        while ai < c.attn_layers:
            self._attention(ai)
            ai += 1
        mark("layers")
        posterior = kernels.greedy_tokens_with_mask(self.logits)
        accept, next_token, replay_len = kernels.accept_lengths(posterior, self.verify_ids)
        mark("acceptance")
        states, convs = [], []
        for L, (_, _, tape) in zip(self.gdn, verify):
            states.append(kernels.tape_replay_kernel(tape, L["k"], L["g"], L["state"], n_per_seq=replay_len))
            convs.append(kernels.rebuild_conv_state(L["conv"], L["qkv"], replay_len, c.conv_kernel - 1))
        mark("rollback")
        gathered = None
        if world > 1:
            gathered = partition.all_gather_acceptance(accept, next_token, n_sequences_global or self.cfg.batch * world)
        mark("gather")
        return dict(accept=accept, next_token=next_token, replay_len=replay_len, states=states, convs=convs,
                    verify=verify, attn_out=self.attn_out, gathered=gathered)

    def _attention(self, i: int) -> None:
        a = self.attn[i]
        kernels.batched_sdpa_turbo_kv(a["q"], (a["kp"], a["ks"], a["kn"], a["kr"]), (a["vp"], a["vn"]), self.cfg.context,
                                      self.scale, k_hot=a["k_hot"], v_hot=a["v_hot"], out=self.attn_out[i])

    def bytes_per_step(self) -> float:
        """Algorithmic HBM bytes of one step (what a fused implementation would have to move at least)."""
        c = self.cfg
        heads = c.batch * c.Hv
        gdn = c.gdn_layers * (heads * (131072 + 772 * c.T) + heads * (131072 + 642 * 8))          # verify + mean rollback
        blocks = c.batch * c.Hkv * c.context * (c.D // 128)
        attn = c.attn_layers * (blocks * (48 + 16 + 4 + 48 + 2) + 2 * c.batch * c.Hkv * c.T * c.D * 2)
        return float(gdn + attn + self.logits.numel() * 2)


def _event():
    e = torch.cuda.Event(enable_timing=True)
    e.record()
    return e
