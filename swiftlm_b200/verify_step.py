"""One DFlash verify step over a hybrid stack of gated-delta and full-attention layers: the host side of
dflash_verify_step (include/dflash_cuda.h), which composes the kernels below the C ABI the way the reference's
runtime composes its own (Sources/DFlash/DFlashRuntime.swift:499-579: verify pass over the drafted block with
armed rollback caches, greedy posterior :118-128, acceptance :133-142, commit arithmetic :523-547, cache restore
:188-223; Sources/DFlash/RecurrentRollbackCache.swift:95-131 for the per-layer rollback).

The layers of a kind are stacked into the batch axis (item = sequence * layers + layer), every buffer is
allocated once here, and a step is ONE call into the library: a handful of launches, no allocation, no host
read of the accepted lengths.  Layer weights are omitted: the per-layer q/k/v/beta/g of the gated-delta layers,
the queries of the attention layers, the KV cache (TurboQuant 3-bit cold history plus the block's own tokens
as the hot window) and the logits are seeded synthetic tensors.  With more than one rank the step ends with
the all-gather of the acceptance results and of one logits row per sequence (swiftlm_b200.partition).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib, kernels, partition


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
    turbo_kv: bool = True         # False: the same stack over dense bf16 KV
    keep_state_verify: bool = True   # False: the verify forward writes no final state (state_rolled is the result)


class VerifyStep:
    def __init__(self, cfg: StepConfig, device: torch.device):
        self.cfg = c = cfg
        self.device = device
        g = torch.Generator(device=device).manual_seed(c.seed)
        bf = torch.bfloat16
        rn = lambda *s: torch.randn(*s, device=device, generator=g)  # noqa: E731
        norm = torch.nn.functional.normalize
        B, T, L, A = c.batch, c.T, c.gdn_layers, c.attn_layers
        I = B * L                                              # gated-delta items, sequence-major
        self.q = norm(rn(I, T, c.Hk, c.Dk), dim=-1).to(bf)
        self.k = norm(rn(I, T, c.Hk, c.Dk), dim=-1).to(bf)
        self.v = rn(I, T, c.Hv, c.Dk).to(bf)
        self.beta = torch.sigmoid(rn(I, T, c.Hv)).to(bf)
        self.g = torch.exp(-torch.nn.functional.softplus(rn(I, T, c.Hv))).to(bf)
        self.state = 0.02 * rn(I, c.Hv, c.Dk, c.Dk)
        self.conv = rn(I, c.conv_kernel - 1, c.conv_dim).to(bf)
        self.qkv = rn(I, T, c.conv_dim).to(bf)
        self.y = torch.empty_like(self.v)
        self.state_verify = torch.empty_like(self.state) if c.keep_state_verify else None
        self.state_rolled = torch.empty_like(self.state)
        self.tape = torch.empty(I, T, c.Hv, c.Dk, device=device)
        self.conv_out = torch.empty_like(self.conv)
        # attention items, sequence-major: the committed context compressed, the block's own T tokens dense
        N = c.context + T
        self.N = N
        J = B * A
        self.attn_q = rn(J, c.Hq, T, c.D).to(bf)
        self.attn_out = torch.empty_like(self.attn_q)
        self.scale = 1.0 / float(c.D) ** 0.5
        self._turbo_desc = None
        if c.turbo_kv:
            enc = dict(kp=[], ks=[], kn=[], kr=[], vp=[], vn=[], kh=[], vh=[])
            chunk = max(1, min(J, 64))
            for lo in range(0, J, chunk):                      # encode in slices: the dense K/V never exist as a whole
                n = min(chunk, J - lo)
                k = rn(n, c.Hkv, N, c.D).to(bf)
                v = rn(n, c.Hkv, N, c.D).to(bf)
                kp, ks, kn, kr = kernels.turbo_encode(k[:, :, :c.context].contiguous(), True)
                vp, _, vn, _ = kernels.turbo_encode(v[:, :, :c.context].contiguous(), False)
                for name, t in (("kp", kp), ("ks", ks), ("kn", kn), ("kr", kr), ("vp", vp), ("vn", vn),
                                ("kh", k[:, :, c.context:].contiguous()), ("vh", v[:, :, c.context:].contiguous())):
                    enc[name].append(t)
                del k, v
            self.kv = {name: torch.cat(ts) for name, ts in enc.items()}
            e = self.kv
            self._turbo_desc = _lib.TurboKV(e["kp"].data_ptr(), e["ks"].data_ptr(), e["kn"].data_ptr(), e["kr"].data_ptr(),
                                            e["vp"].data_ptr(), e["vn"].data_ptr(), e["kh"].data_ptr(), e["vh"].data_ptr(),
                                            c.context, T)
        else:
            self.kv = dict(k=rn(J, c.Hkv, N, c.D).to(bf), v=rn(J, c.Hkv, N, c.D).to(bf))
        self.logits = rn(B, T, c.vocab).to(bf)
        # draft ids: the staged token, then drafted tokens that agree with the posterior for a random prefix
        post = kernels.greedy_tokens_with_mask(self.logits).to(torch.int64)
        agree = torch.randint(0, T, (B,), device=device, generator=g)
        ids = torch.zeros(B, T, dtype=torch.int64, device=device)
        ids[:, 1:] = post[:, :-1]
        wrong = torch.arange(T - 1, device=device).view(1, -1) >= agree.view(-1, 1)
        ids[:, 1:][wrong] = (ids[:, 1:][wrong] + 1) % c.vocab
        self.verify_ids = ids.to(torch.int32)
        self.posterior = torch.empty(B, T, dtype=torch.int32, device=device)
        self.accept = torch.empty(B, dtype=torch.int32, device=device)
        self.next_token = torch.empty_like(self.accept)
        self.replay_len = torch.empty_like(self.accept)
        self.logits_rows = torch.empty(B, c.vocab, dtype=bf, device=device)
        self.desc = self._describe()
        L_ = _lib.lib()
        need = L_.dflash_verify_step_workspace_bytes(C.byref(self.desc))
        self.workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=device)

    def _describe(self) -> "_lib.VerifyStepDesc":
        c = self.cfg
        p = lambda t: None if t is None else t.data_ptr()  # noqa: E731
        d = _lib.VerifyStepDesc()
        d.B, d.T = c.batch, c.T
        d.gdn_layers, d.Hk, d.Hv, d.Dk, d.Dv, d.g_is_vector, d.in_dtype = c.gdn_layers, c.Hk, c.Hv, c.Dk, c.Dk, 0, _lib.BF16
        d.q, d.k, d.v, d.g, d.beta = p(self.q), p(self.k), p(self.v), p(self.g), p(self.beta)
        d.state, d.y, d.state_verify, d.tape, d.state_rolled = p(self.state), p(self.y), p(self.state_verify), p(self.tape), p(self.state_rolled)
        d.conv_snapshot, d.qkv, d.conv_out = p(self.conv), p(self.qkv), p(self.conv_out)
        d.conv_keep, d.conv_row_bytes = c.conv_kernel - 1, c.conv_dim * 2
        d.attn_layers, d.Hq, d.Hkv, d.D, d.N, d.attn_dtype = c.attn_layers, c.Hq, c.Hkv, c.D, self.N, _lib.BF16
        d.attn_q, d.attn_out, d.scale = p(self.attn_q), p(self.attn_out), self.scale
        if self._turbo_desc is not None:
            d.kv_format = _lib.KV_TURBO3
            d.attn_k, d.attn_v = C.cast(C.pointer(self._turbo_desc), C.c_void_p), None
        else:
            d.kv_format = _lib.KV_DENSE
            d.attn_k, d.attn_v = p(self.kv["k"]), p(self.kv["v"])
        d.logits, d.suppress, d.verify_ids, d.V, d.logits_dtype = p(self.logits), None, p(self.verify_ids), c.vocab, _lib.BF16
        d.posterior, d.accept, d.next_token, d.replay_len = p(self.posterior), p(self.accept), p(self.next_token), p(self.replay_len)
        d.logits_rows = p(self.logits_rows)
        return d

    # ---- the step -----------------------------------------------------------------------------
    def run(self, world: int = 1, n_sequences_global: Optional[int] = None, events: Optional[dict] = None):
        """One step: a single call into the library (its launches are listed in the header), then, with more than one
        rank, the all-gather.  `events` receives CUDA events around the two parts."""
        mark = (lambda name: events.setdefault(name, []).append(_event())) if events is not None else (lambda name: None)
        mark("start")
        _lib.check(_lib.lib().dflash_verify_step(C.byref(self.desc), self.workspace.data_ptr(), self.workspace.numel(),
                                                 torch.cuda.current_stream().cuda_stream))
        mark("step")
        gathered = None
        if world > 1:
            gathered = partition.all_gather_acceptance(self.accept, self.next_token, n_sequences_global or self.cfg.batch * world,
                                                       logits_rows_local=self.logits_rows)
        mark("gather")
        return dict(accept=self.accept, next_token=self.next_token, replay_len=self.replay_len, states=self.state_rolled,
                    convs=self.conv_out, y=self.y, state_verify=self.state_verify, tape=self.tape, attn_out=self.attn_out,
                    logits_rows=self.logits_rows, gathered=gathered)

    def bytes_per_step(self) -> float:
        """Algorithmic HBM bytes of one step (what a fused implementation would have to move at least)."""
        c = self.cfg
        heads = c.batch * c.Hv
        verify_state = 131072 if c.keep_state_verify else 65536                                 # read, and written if kept
        gdn = c.gdn_layers * (heads * (verify_state + 772 * c.T) + heads * (131072 + 642 * 8))    # verify + mean rollback
        blocks = c.batch * c.Hkv * c.context * (c.D // 128)
        per_block = (48 + 16 + 4 + 48 + 2) if c.turbo_kv else 2 * 256
        attn = c.attn_layers * (blocks * per_block + 2 * c.batch * c.Hkv * c.T * c.D * 2)
        return float(gdn + attn + self.logits.numel() * 2)


def _event():
    e = torch.cuda.Event(enable_timing=True)
    e.record()
    return e
