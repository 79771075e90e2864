"""Torch-CPU restatement of the reference's CPU ("ops") path of the gated-delta forward, op for op.

Test infrastructure only (tests/ and the cpu_baseline leg of bench.py): it exists to time the
reference's own CPU structure with all intra-op threads, next to the row-wise C/OpenMP port.
Follows gatedDeltaOpsWithTape, Sources/DFlash/DFlashKernels.swift:409-466 of the SwiftLM tree:
heads repeated up front (:424-427), then per token five full-state passes (decay :440, kv :441,
delta :442, rank-1 update :443, output :444) and arithmetic masking (:449-453).  fp32 throughout.
"""
from __future__ import annotations

import torch


def gated_delta_ops_torch(q, k, v, g, beta, state, mask=None):
    """q,k [B,T,Hk,Dk]; v [B,T,Hv,Dv]; g [B,T,Hv] or [B,T,Hv,Dk]; beta [B,T,Hv]; state [B,Hv,Dv,Dk];
    mask [B,T] of 0/1 or None.  Returns (y [B,T,Hv,Dv], state, tape [B,T,Hv,Dv]) as fp32 CPU tensors."""
    q, k, v, g, beta = (torch.as_tensor(a, dtype=torch.float32) for a in (q, k, v, g, beta))
    S = torch.as_tensor(state, dtype=torch.float32).clone()
    T, Hk, Hv = q.shape[1], q.shape[2], v.shape[2]
    rep = Hv // Hk
    if rep > 1:                                                      # :424-427
        q = q.repeat_interleave(rep, dim=2)
        k = k.repeat_interleave(rep, dim=2)
    if mask is not None:
        mask = torch.as_tensor(mask, dtype=torch.float32)
    ys, tapes = [], []
    for t in range(T):
        decay = g[:, t, :, None, :] if g.dim() == 4 else g[:, t, :, None, None]   # :434-439
        decayed = S * decay                                          # :440
        kt = k[:, t, :, None, :]
        kv_mem = (decayed * kt).sum(dim=-1)                          # :441
        delta = (v[:, t] - kv_mem) * beta[:, t, :, None]             # :442
        new_state = decayed + kt * delta[..., None]                  # :443
        y = (new_state * q[:, t, :, None, :]).sum(dim=-1)            # :444
        if mask is not None:
            s_gate = mask[:, t, None, None, None]                    # :449
            y_gate = mask[:, t, None, None]                          # :450
            S = new_state * s_gate + S * (1 - s_gate)                # :451
            ys.append(y * y_gate)                                    # :452
            tapes.append(delta * y_gate)                             # :453
        else:
            S = new_state
            ys.append(y)
            tapes.append(delta)
    return torch.stack(ys, dim=1), S, torch.stack(tapes, dim=1)
