"""Host-side mirror of the reference's kernel entry points (`public enum DFlashKernels`,
Sources/DFlash/DFlashKernels.swift of the SwiftLM tree) on top of the C ABI.

Same names (snake_case), argument meaning, layouts and error behaviour as the Swift API:
inputs are never mutated, outputs are fresh tensors, `batched_sdpa_2pass` returns None for
shapes outside the supported set exactly where the reference returns nil.  torch is used only
for device memory and streams; every computation happens in libdflash_cuda.so.  There is no
CPU path: tensors must live on a CUDA device.
"""
from __future__ import annotations

from typing import Optional, Tuple

import ctypes as C

import torch

from . import _lib

_DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16,
       torch.uint8: _lib.U8, torch.bool: _lib.U8}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("DFlash kernels run on a CUDA device only (no CPU fallback)")


def _mask_arg(mask: Optional[torch.Tensor]):
    if mask is None:
        return None, 0
    if mask.dtype not in _DT:
        mask = mask.to(torch.float32)
    return mask.contiguous(), _DT[mask.dtype]


def _n_arg(n_per_seq, B, device):
    if n_per_seq is None:
        return None
    n = torch.as_tensor(n_per_seq, device=device).to(torch.int32).contiguous()
    if n.numel() != B:
        raise ValueError("n_per_seq must have one entry per sequence")
    return n


def gated_delta_kernel_with_tape(q, k, v, g, beta, state, mask=None, n_per_seq=None,
                                 want_tape: bool = True) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """DFlashKernels.gatedDeltaKernelWithTape (Sources/DFlash/DFlashKernels.swift:316-324).

    q,k [B,T,Hk,Dk]; v [B,T,Hv,Dv]; g [B,T,Hv] or [B,T,Hv,Dk]; beta [B,T,Hv];
    state [B,Hv,Dv,Dk] (kept in fp32); mask [B,T] optional.  Returns (y [B,T,Hv,Dv] in q's
    dtype, new state fp32, innovation tape fp32 [B,T,Hv,Dv]).
    n_per_seq (int32 [B], not in the reference signature) runs only the first n steps of each
    sequence: this is the replay of a recorded block to its accepted length.
    """
    _need_cuda(q, k, v, g, beta, state)
    B, T, Hk, Dk = q.shape
    Hv, Dv = v.shape[2], v.shape[3]
    dt = q.dtype
    if dt not in (torch.float32, torch.bfloat16, torch.float16):
        raise _lib.DFlashUnsupported(_lib.ERR_UNSUPPORTED, f"input dtype {dt}")
    q, k, v, g, beta = (x.to(dt).contiguous() for x in (q, k, v, g, beta))
    state = state.to(torch.float32).contiguous()
    mask, mdt = _mask_arg(mask)
    n = _n_arg(n_per_seq, B, q.device)
    y = torch.empty((B, T, Hv, Dv), dtype=dt, device=q.device)
    state_out = torch.empty_like(state)
    tape = torch.empty((B, T, Hv, Dv), dtype=torch.float32, device=q.device) if want_tape else None
    _lib.check(_lib.lib().dflash_gated_delta_tape(
        _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta), _ptr(state), _ptr(mask), _ptr(n),
        _ptr(y), _ptr(state_out), _ptr(tape), B, T, Hk, Hv, Dk, Dv, int(g.dim() == 4), _DT[dt], mdt,
        _stream()))
    return y, state_out, tape


def tape_replay_kernel(tape, k, g, state, mask=None, n_per_seq=None) -> torch.Tensor:
    """DFlashKernels.tapeReplayKernel (Sources/DFlash/DFlashKernels.swift:252-258).

    tape [B,T,Hv,Dv] (fp32), k [B,T,Hk,Dk], g [B,T,Hv] or [B,T,Hv,Dk], state [B,Hv,Dv,Dk].
    Returns the replayed state.  n_per_seq replays only the first n steps per sequence (what
    the reference's caller does by slicing, Sources/DFlash/RecurrentRollbackCache.swift:115-118).
    """
    _need_cuda(tape, k, g, state)
    B, T, Hv, Dv = tape.shape
    Hk, Dk = k.shape[2], k.shape[3]
    dt = k.dtype
    if dt not in (torch.float32, torch.bfloat16, torch.float16):
        raise _lib.DFlashUnsupported(_lib.ERR_UNSUPPORTED, f"input dtype {dt}")
    tape = tape.to(torch.float32).contiguous()
    k = k.contiguous()
    g = g.to(dt).contiguous()
    state = state.to(torch.float32).contiguous()
    mask, mdt = _mask_arg(mask)
    n = _n_arg(n_per_seq, B, k.device)
    out = torch.empty_like(state)
    _lib.check(_lib.lib().dflash_tape_replay(
        _ptr(tape), _ptr(k), _ptr(g), _ptr(state), _ptr(mask), _ptr(n), _ptr(out),
        B, T, Hk, Hv, Dk, Dv, int(g.dim() == 4), _DT[dt], mdt, _stream()))
    return out


_workspaces = {}


def _workspace(device, nbytes: int) -> Optional[torch.Tensor]:
    if nbytes == 0:
        return None
    key = (device.index, torch.cuda.current_stream().cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def batched_sdpa_2pass(queries, keys, values, scale: float, mask=None, kv_len=None,
                       page_table=None, out=None, n_max=None) -> Optional[torch.Tensor]:
    """DFlashKernels.batchedSDPA2Pass (Sources/DFlash/DFlashKernels.swift:737-743).

    queries [B,Hq,16,D]; keys/values [B,Hkv,N,D] (or, with page_table int32 [B,max_pages],
    page pools [num_pages,Hkv,page_tokens,D]); optional additive mask [B,Hq,16,N].
    Returns [B,Hq,16,D] in the input dtype, or None where the reference returns nil
    (query length != 16, dtype not bf16/f16, head_dim not in {128,256}, Hq % Hkv != 0).
    """
    _need_cuda(queries, keys, values)
    if queries.dim() != 4 or keys.dim() != 4 or values.dim() != 4:
        return None
    B, Hq, T, D = queries.shape
    dt = queries.dtype
    if T != 16 or dt not in (torch.bfloat16, torch.float16):
        return None
    if D not in (128, 256) or values.shape[3] != D:
        return None
    Hkv = keys.shape[1]
    if Hkv <= 0 or Hq % Hkv != 0:
        return None
    q = queries.contiguous()
    k = keys.to(dt).contiguous()
    v = values.to(dt).contiguous()
    if kv_len is not None:
        kv_len = torch.as_tensor(kv_len, device=q.device).to(torch.int32).contiguous()
    if page_table is None:
        N, page_tokens, max_pages, num_pages = keys.shape[2], 0, 0, 0
    else:
        if kv_len is None:
            raise ValueError("paged KV needs kv_len")
        page_table = page_table.to(torch.int32).contiguous()
        page_tokens, max_pages, num_pages = keys.shape[2], page_table.shape[1], keys.shape[0]
        # n_max avoids a host read of kv_len on the hot path
        N = int(n_max) if n_max is not None else int(kv_len.max())
    if mask is not None:
        mask = mask.to(dt).expand(B, Hq, 16, N).contiguous()
    if out is None:
        out = torch.empty_like(q)
    L = _lib.lib()
    ws = _workspace(q.device, L.dflash_verify_sdpa_workspace_bytes(B, Hq, Hkv, D, N))
    try:
        _lib.check(L.dflash_verify_sdpa(
            _ptr(q), _ptr(k), _ptr(v), _ptr(page_table), _ptr(kv_len), _ptr(mask), _ptr(out),
            _ptr(ws), 0 if ws is None else ws.numel(), B, Hq, Hkv, T, D, N, page_tokens, max_pages,
            num_pages, float(scale), _DT[dt], _lib.KV_DENSE, _stream()))
    except _lib.DFlashUnsupported:
        return None
    return out


def greedy_tokens_with_mask(logits: torch.Tensor, suppress_token_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """DFlashRuntime.greedyTokensWithMask (Sources/DFlash/DFlashRuntime.swift:118-128).
    logits [..., V]; returns token ids (uint32 values held in an int64-free int32 view)."""
    _need_cuda(logits)
    V = logits.shape[-1]
    flat = logits.contiguous().view(-1, V)
    sup = None
    if suppress_token_mask is not None:
        sup = suppress_token_mask.to(device=logits.device, dtype=torch.uint8).contiguous()
    post = torch.empty(flat.shape[0], dtype=torch.int32, device=logits.device)
    _lib.check(_lib.lib().dflash_greedy_tokens(_ptr(flat), _ptr(sup), _ptr(post), flat.shape[0], V,
                                              _DT[logits.dtype], _stream()))
    return post.view(logits.shape[:-1])


def accept_lengths(posterior: torch.Tensor, verify_ids: torch.Tensor):
    """DFlashRuntime.matchAcceptanceLength + the commit arithmetic
    (Sources/DFlash/DFlashRuntime.swift:133-142, :523-547), batched over sequences.
    posterior, verify_ids int32 [B,T].  Returns (accept [B], next_token [B], replay_len [B])."""
    _need_cuda(posterior, verify_ids)
    B, T = verify_ids.shape
    posterior = posterior.to(torch.int32).contiguous()
    verify_ids = verify_ids.to(torch.int32).contiguous()
    acc = torch.empty(B, dtype=torch.int32, device=posterior.device)
    nxt = torch.empty_like(acc)
    rep = torch.empty_like(acc)
    _lib.check(_lib.lib().dflash_accept_lengths(_ptr(posterior), _ptr(verify_ids), _ptr(acc), _ptr(nxt),
                                               _ptr(rep), B, T, _stream()))
    return acc, nxt, rep


def gather_logits_rows(logits: torch.Tensor, row_per_seq: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """logits [B,T,V], row_per_seq int32 [B] (the accepted count) -> [B,V]: each sequence's logits row at its accepted
    position, the row whose argmax is the next staged token (Sources/DFlash/DFlashRuntime.swift:547)."""
    _need_cuda(logits, row_per_seq)
    B, T, V = logits.shape
    logits = logits.contiguous()
    if out is None:
        out = torch.empty(B, V, dtype=logits.dtype, device=logits.device)
    _lib.check(_lib.lib().dflash_gather_logits_rows(_ptr(logits), _ptr(row_per_seq.to(torch.int32).contiguous()), _ptr(out),
                                                   B, T, V, _DT[logits.dtype], _stream()))
    return out


def turbo_decode_into(packed, signs, norm, rnorm, out: torch.Tensor) -> None:
    """turbo_decode into a caller-owned tensor (any shape holding norm.numel() * 128 values)."""
    _need_cuda(packed, norm, out)
    n = norm.numel()
    if out.numel() != n * 128 or not out.is_contiguous():
        raise _lib.DFlashError(_lib.ERR_INVALID_ARG, "turbo_decode_into: out must be contiguous with 128 values per block")
    _lib.check(_lib.lib().dflash_turbo_decode(_ptr(packed.contiguous()), _ptr(signs), _ptr(norm.contiguous()),
                                             _ptr(rnorm), _ptr(out), n, int(signs is not None), _DT[out.dtype], _stream()))


def device_status() -> None:
    """Raises if a kernel's bounded device-side wait gave up since the last check."""
    _lib.check(_lib.lib().dflash_device_status(_stream()))


def launch_count() -> int:
    return int(_lib.lib().dflash_launch_count())


def tape_replay_into(tape, k, g, state, n_per_seq, state_out, mask=None) -> None:
    """Allocation-free form of tape_replay_kernel: every buffer is supplied by the caller (contiguous, on the current
    device; tape and state fp32).  state_out may be the same tensor as state."""
    B, T, Hv, Dv = tape.shape
    Hk, Dk = k.shape[2], k.shape[3]
    mask_t, mdt = _mask_arg(mask)
    _lib.check(_lib.lib().dflash_tape_replay(
        _ptr(tape), _ptr(k), _ptr(g), _ptr(state), _ptr(mask_t), _ptr(n_per_seq), _ptr(state_out),
        B, T, Hk, Hv, Dk, Dv, int(g.dim() == 4), _DT[k.dtype], mdt, _stream()))


def kv_append(k_new, v_new, k_cache, v_cache, kv_len=None, len_all: int = 0, page_table=None, kv_len_out=None) -> None:
    """Writes the block's rows k_new / v_new [B,Hkv,T,D] behind the committed tokens of a dense cache [B,Hkv,capacity,D]
    or, with page_table int32[B,max_pages], of a page pool [pages,Hkv,page_tokens,D]: row t of sequence b lands at
    position kv_len[b] + t (len_all + t without kv_len).  kv_len_out receives kv_len + T, the length the verify
    attention sees.  Replaces the cache update before the target forward (Sources/DFlash/DFlashRuntime.swift:188-223)."""
    B, Hkv, T, D = k_new.shape
    if page_table is not None:
        num_pages, page_tokens, max_pages, capacity = k_cache.shape[0], k_cache.shape[2], page_table.shape[1], 0
    else:
        num_pages, page_tokens, max_pages, capacity = 0, 0, 0, k_cache.shape[2]
    _lib.check(_lib.lib().dflash_kv_append(
        _ptr(k_new), _ptr(v_new), _ptr(k_cache), _ptr(v_cache), _ptr(page_table), _ptr(kv_len), int(len_all),
        _ptr(kv_len_out), B, Hkv, T, D, capacity, page_tokens, max_pages, num_pages, _DT[k_new.dtype], _stream()))


def kv_commit(kv_len, commit, block: int = 16) -> None:
    """kv_len[b] += clamp(commit[b], 0, block): keeps the accepted prefix of the block just appended and
    leaves the rejected rows to be overwritten (the reference's cache.trim(offset - targetLen))."""
    _lib.check(_lib.lib().dflash_kv_commit(_ptr(kv_len), _ptr(commit), kv_len.numel(), int(block), _stream()))


def gated_delta_into(q, k, v, g, beta, state, n_per_seq, y, state_out, tape=None, mask=None) -> None:
    """Allocation-free form of gated_delta_kernel_with_tape: every buffer is supplied by the
    caller (contiguous, on the current device, dtypes as documented there).  state_out may be
    the same tensor as state."""
    B, T, Hk, Dk = q.shape
    Hv, Dv = v.shape[2], v.shape[3]
    mask_t, mdt = _mask_arg(mask)
    _lib.check(_lib.lib().dflash_gated_delta_tape(
        _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta), _ptr(state), _ptr(mask_t), _ptr(n_per_seq),
        _ptr(y), _ptr(state_out), _ptr(tape), B, T, Hk, Hv, Dk, Dv, int(g.dim() == 4), _DT[q.dtype], mdt,
        _stream()))


def batched_sdpa_turbo_kv(queries, k_enc, v_enc, n_cold: int, scale: float, k_hot=None, v_hot=None, out=None) -> Optional[torch.Tensor]:
    """Block-verify attention over KV held in the TurboQuant 3-bit format with a hot window: k_enc = (packed, signs,
    norm, rnorm) and v_enc = (packed, norm) as returned by turbo_encode for the cold history [B,Hkv,n_cold,D]; k_hot,
    v_hot [B,Hkv,n_hot,D] in the attention dtype are the newest tokens (the verify block among them).  With a cold
    history of whole 128-key tiles the library attends in the codec's rotated domain without decoding a key or value
    to global memory; otherwise it expands the cold history into its workspace and attends over the copy
    (dflash_verify_sdpa with DFLASH_KV_TURBO3)."""
    _need_cuda(queries, k_enc[0], v_enc[0])
    B, Hq, T, D = queries.shape
    dt = queries.dtype
    Hkv = k_enc[2].shape[1]
    if T != 16 or dt not in (torch.bfloat16, torch.float16) or D not in (128, 256) or Hq % Hkv != 0:
        return None
    q = queries.contiguous()
    if out is None:
        out = torch.empty_like(q)
    n_hot = 0 if k_hot is None else k_hot.shape[2]
    n_keys = n_cold + n_hot
    L = _lib.lib()
    ws = _workspace(q.device, L.dflash_verify_sdpa_turbo_workspace_bytes(B, Hq, Hkv, D, n_cold, n_hot))
    kp, ks, kn, kr = (t.contiguous() for t in k_enc)
    vp, vn = (t.contiguous() for t in v_enc)
    kh = None if k_hot is None else k_hot.to(dt).contiguous()
    vh = None if v_hot is None else v_hot.to(dt).contiguous()
    desc = _lib.TurboKV(_ptr(kp), _ptr(ks), _ptr(kn), _ptr(kr), _ptr(vp), _ptr(vn), _ptr(kh), _ptr(vh), n_cold, n_hot)
    try:
        _lib.check(L.dflash_verify_sdpa(_ptr(q), C.cast(C.pointer(desc), C.c_void_p), None, None, None, None, _ptr(out),
                                        _ptr(ws), ws.numel(), B, Hq, Hkv, T, D, n_keys, 0, 0, 0, float(scale), _DT[dt],
                                        _lib.KV_TURBO3, _stream()))
    except _lib.DFlashUnsupported:
        return None
    return out


def rebuild_conv_state(conv_snapshot: Optional[torch.Tensor], qkv: torch.Tensor, steps, keep: int) -> torch.Tensor:
    """RecurrentRollbackCache.rebuildConvState (Sources/DFlash/RecurrentRollbackCache.swift:139-158) on the device:
    concat(conv_snapshot [B,keep,C], qkv [B,T,C])[:, steps : min(steps + keep, keep + T)].  `steps` is an int
    (the reference's accepted_steps) or a device int32 tensor [B] of per-sequence step counts (keep rows each)."""
    _need_cuda(qkv)
    qkv = qkv.contiguous()
    B, T, Cdim = qkv.shape
    row_bytes = Cdim * qkv.element_size()
    snap = None if conv_snapshot is None else conv_snapshot.to(qkv.dtype).contiguous()
    rows = C.c_int32(0)
    out = torch.empty(B, keep, Cdim, dtype=qkv.dtype, device=qkv.device)
    if isinstance(steps, torch.Tensor):
        st = steps.to(torch.int32).contiguous()
        _lib.check(_lib.lib().dflash_rebuild_conv_state(_ptr(snap), _ptr(qkv), _ptr(st), 0, _ptr(out), B, T, keep,
                                                       row_bytes, C.byref(rows), _stream()))
        return out
    # scalar count: the window is [B, rows, C] with rows <= keep, written densely at the front of `out`
    end = min(int(steps) + keep, keep + T)
    n_rows = max(end - int(steps), 0)
    out = torch.empty(B, n_rows, Cdim, dtype=qkv.dtype, device=qkv.device)
    if n_rows:
        _lib.check(_lib.lib().dflash_rebuild_conv_state(_ptr(snap), _ptr(qkv), None, int(steps), _ptr(out), B, T, keep,
                                                       row_bytes, C.byref(rows), _stream()))
    return out


def turbo_encode(x: torch.Tensor, is_key: bool):
    """TurboQuant 3-bit encode of 128-dimension blocks (tests/test_turbo_quant.cpp:69-74 for V,
    :85-94 for K in the reference tree).  x [..., 128*m]; returns packed uint8 [..., m, 48],
    signs uint8 [..., m, 16] or None (V), norm and rnorm (or None) as fp16 bit patterns in int16 tensors."""
    _need_cuda(x)
    if x.shape[-1] % 128 != 0:
        raise _lib.DFlashUnsupported(_lib.ERR_UNSUPPORTED, "last dimension must be a multiple of 128")
    x = x.contiguous()
    lead = tuple(x.shape[:-1]) + (x.shape[-1] // 128,)
    n = x.numel() // 128
    packed = torch.empty(lead + (48,), dtype=torch.uint8, device=x.device)
    norm = torch.empty(lead, dtype=torch.int16, device=x.device)
    signs = torch.empty(lead + (16,), dtype=torch.uint8, device=x.device) if is_key else None
    rnorm = torch.empty(lead, dtype=torch.int16, device=x.device) if is_key else None
    _lib.check(_lib.lib().dflash_turbo_encode(_ptr(x), _ptr(packed), _ptr(signs), _ptr(norm), _ptr(rnorm), n,
                                             int(is_key), _DT[x.dtype], _stream()))
    return packed, signs, norm, rnorm


def turbo_decode(packed, signs, norm, rnorm, dtype=torch.bfloat16) -> torch.Tensor:
    """Inverse of turbo_encode (tests/test_turbo_quant.cpp:74-75 and :96-98): returns [..., 128*m]."""
    _need_cuda(packed, norm)
    is_key = signs is not None
    lead = tuple(norm.shape)
    n = norm.numel()
    out = torch.empty(lead[:-1] + (lead[-1] * 128,), dtype=dtype, device=packed.device)
    _lib.check(_lib.lib().dflash_turbo_decode(_ptr(packed.contiguous()), _ptr(signs), _ptr(norm.contiguous()),
                                             _ptr(rnorm), _ptr(out), n, int(is_key), _DT[dtype], _stream()))
    return out
