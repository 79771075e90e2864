"""Host-buffer entry points: the same kernels for a caller whose tensors live in host memory.

The reference's CPU path works on host arrays; a drop-in for such a caller has to move every
input to the device and every output back.  These functions do that with pinned host memory,
chunking the batch by sequence and overlapping the three legs (host->device copy, kernel,
device->host copy) on separate CUDA streams with double-buffered device staging.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from . import kernels

_INPUTS = ("q", "k", "v", "g", "beta", "state", "n")


def pin_replay_inputs(x: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Copies a dict of replay inputs (q,k,v,g,beta,state,n) into pinned host tensors."""
    out = {}
    for name in _INPUTS:
        t = x[name]
        h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        h.copy_(t)
        out[name] = h
    return out


def alloc_replay_outputs(hx: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {"y": torch.empty(hx["v"].shape, dtype=hx["v"].dtype, pin_memory=True),
            "state": torch.empty(hx["state"].shape, dtype=torch.float32, pin_memory=True)}


class _Staging:
    def __init__(self, hx, chunk, device):
        def dev(name, rows):
            t = hx[name]
            return torch.empty((rows,) + tuple(t.shape[1:]), dtype=t.dtype, device=device)
        self.inp = {name: dev(name, chunk) for name in _INPUTS}
        self.y = dev("v", chunk)
        self.state_out = dev("state", chunk)
        self.in_free = torch.cuda.Event()     # kernel that read `inp` has finished
        self.out_free = torch.cuda.Event()    # device->host copy of the outputs has finished
        self.loaded = torch.cuda.Event()
        self.computed = torch.cuda.Event()


_pipes = {}


def _chunk_schedule(B: int, chunk: int):
    """Row ranges of the pipeline's chunks: full chunks in the middle, a quarter and a half chunk at either end.  The
    first copy in and the last copy out overlap with nothing, so they are kept short; small chunks everywhere would
    pay the per-copy overheads on the whole batch."""
    edges = [chunk // 4, chunk // 2] if chunk >= 8 and B >= 4 * chunk else []
    head = [e for e in edges if e > 0]
    tail = head[::-1]
    sizes, left = list(head), B - sum(head) - sum(tail)
    while left > 0:
        sizes.append(min(chunk, left))
        left -= sizes[-1]
    sizes += tail
    out, lo = [], 0
    for n in sizes:
        out.append((lo, lo + n))
        lo += n
    assert lo == B
    return out


def gated_delta_from_host(hx: Dict[str, torch.Tensor], hout: Dict[str, torch.Tensor], chunk: int = 144) -> Tuple[int, int]:
    """Gated-delta replay with every tensor in pinned host memory.

    hx: q,k [B,T,Hk,Dk], v [B,T,Hv,Dv], g,beta [B,T,Hv] (bf16/f16/f32), state [B,Hv,Dv,Dk] fp32,
    n int32 [B].  hout: y [B,T,Hv,Dv], state [B,Hv,Dv,Dk].  Work is enqueued and the current
    stream is made to wait for it; returns (host->device bytes, device->host bytes)."""
    device = torch.device("cuda", torch.cuda.current_device())
    B = hx["q"].shape[0]
    chunk = min(chunk, B)
    key = (device.index, chunk, tuple(hx["state"].shape[1:]), tuple(hx["q"].shape[1:]), hx["q"].dtype)
    pipe = _pipes.get(key)
    if pipe is None:
        pipe = dict(stage=[_Staging(hx, chunk, device) for _ in range(2)],
                    s_in=torch.cuda.Stream(device), s_run=torch.cuda.Stream(device), s_out=torch.cuda.Stream(device))
        _pipes.clear()
        _pipes[key] = pipe
    s_in, s_run, s_out = pipe["s_in"], pipe["s_run"], pipe["s_out"]
    cur = torch.cuda.current_stream(device)
    start = torch.cuda.Event()
    start.record(cur)
    for s in (s_in, s_run, s_out):
        s.wait_event(start)
    h2d = d2h = 0
    for ci, (lo, hi) in enumerate(_chunk_schedule(B, chunk)):
        rows = hi - lo
        st = pipe["stage"][ci % 2]
        with torch.cuda.stream(s_in):
            if ci >= 2:
                s_in.wait_event(st.in_free)
            for name in _INPUTS:
                st.inp[name][:rows].copy_(hx[name][lo:hi], non_blocking=True)
                h2d += hx[name][lo:hi].numel() * hx[name].element_size()
            st.loaded.record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(st.loaded)
            if ci >= 2:
                s_run.wait_event(st.out_free)
            i = st.inp
            kernels.gated_delta_into(i["q"][:rows], i["k"][:rows], i["v"][:rows], i["g"][:rows], i["beta"][:rows],
                                     i["state"][:rows], i["n"][:rows], st.y[:rows], st.state_out[:rows])
            st.in_free.record(s_run)
            st.computed.record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(st.computed)
            hout["y"][lo:hi].copy_(st.y[:rows], non_blocking=True)
            hout["state"][lo:hi].copy_(st.state_out[:rows], non_blocking=True)
            d2h += (st.y[:rows].numel() * st.y.element_size() + st.state_out[:rows].numel() * 4)
            st.out_free.record(s_out)
    done = torch.cuda.Event()
    done.record(s_out)
    cur.wait_event(done)
    return h2d, d2h
