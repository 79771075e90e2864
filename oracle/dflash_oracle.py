"""CPU oracle for the DFlash speculative-verify hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in NumPy, the arithmetic of the reference's own CPU ("ops") statement of
the path.  It is the checker for the CUDA kernels; nothing in the shipped package may import it.
Only the tests, the smoke check and the benchmark's CPU-baseline leg use it.

Every function cites the reference file:line it follows (paths are relative to the SwiftLM
project root).

Pinning status
--------------
* gated-delta forward / tape replay / verify SDPA: **parity unpinned**.  The reference ships no
  golden vectors or known-answer tests for these kernels (its only numeric check compares two
  of its own implementations on unseeded inputs, tests/DFlash/DFlashProfiler.swift:215-244),
  and neither Swift, MLX nor Metal can run where this oracle runs.  The restatement is checked
  instead by (a) two independent statements of the recurrence in the reference agreeing with
  each other here (the ops fallback and the per-row Metal kernel body, plus the Kimi update),
  and (b) algebraic identities (replay of the recorded tape reproduces the forward state, n = T
  equals the unmasked run, n = 0 is the identity, SDPA is invariant to the split count).
* acceptance length: pinned by the worked example in the reference's doc comment
  (Sources/DFlash/DFlashRuntime.swift:130-132).
* TurboQuant codec: pinned against the reference's own C++ (tests/test_turbo_quant.cpp) compiled
  from where it lies into oracle/_ref/ (see oracle/Makefile).
"""
from __future__ import annotations

import numpy as np

# --------------------------------------------------------------------------------------------
# Gated-delta forward with innovation tape
# --------------------------------------------------------------------------------------------


def _repeat_heads(x: np.ndarray, hv: int) -> np.ndarray:
    """MLX.repeated(x, count: Hv/Hk, axis: 2): v-heads 2j and 2j+1 share qk-head j.

    Sources/DFlash/DFlashKernels.swift:381-385, 421-427 (ops) and :47, :126 (kernel: hv / (Hv/Hk)).
    """
    hk = x.shape[2]
    if hv == hk:
        return x
    assert hv % hk == 0
    return np.repeat(x, hv // hk, axis=2)


def _step_mask(mask, n_per_seq, B: int, T: int):
    """Combine the reference's [B,T] mask (step on iff value > 0.5,
    Sources/DFlash/DFlashKernels.swift:36, :115) with an accepted length per sequence
    (step on iff t < n).  Returns bool [B,T] or None when every step is on."""
    on = None
    if mask is not None:
        on = np.asarray(mask, dtype=np.float32).reshape(B, T) > 0.5
    if n_per_seq is not None:
        n = np.asarray(n_per_seq).reshape(B, 1)
        pref = np.arange(T).reshape(1, T) < n
        on = pref if on is None else (on & pref)
    return on


def gated_delta_ops_with_tape(q, k, v, g, beta, state, mask=None, n_per_seq=None):
    """Restates gatedDeltaOpsWithTape, Sources/DFlash/DFlashKernels.swift:409-466.

    q,k [B,T,Hk,Dk]; v [B,T,Hv,Dv]; g [B,T,Hv] (scalar gate) or [B,T,Hv,Dk] (vector gate);
    beta [B,T,Hv]; state [B,Hv,Dv,Dk].  Returns (y [B,T,Hv,Dv] fp32, state fp32, tape fp32).
    All arithmetic in fp32, no per-step rounding of the state (ops semantics, :440-458).
    A masked-off step leaves the state untouched and emits y = 0, tape = 0 (:446-453).
    """
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    g = np.asarray(g, dtype=np.float32)
    beta = np.asarray(beta, dtype=np.float32)
    S = np.array(state, dtype=np.float32, copy=True)
    B, T, Hk, Dk = q.shape
    Hv, Dv = v.shape[2], v.shape[3]
    q = _repeat_heads(q, Hv)
    k = _repeat_heads(k, Hv)
    on = _step_mask(mask, n_per_seq, B, T)
    ys, tapes = [], []
    for t in range(T):
        if g.ndim == 4:
            decay = g[:, t, :, None, :]                       # :436
        else:
            decay = g[:, t, :, None, None]                    # :438
        decayed = S * decay                                   # :440
        kt = k[:, t, :, None, :]
        kv_mem = (decayed * kt).sum(axis=-1, dtype=np.float32)           # :441
        delta = (v[:, t] - kv_mem) * beta[:, t, :, None]                 # :442
        new_state = decayed + kt * delta[..., None]                      # :443
        y = (new_state * q[:, t, :, None, :]).sum(axis=-1, dtype=np.float32)  # :444
        if on is not None:
            s_gate = on[:, t].astype(np.float32)[:, None, None, None]    # :449
            y_gate = on[:, t].astype(np.float32)[:, None, None]          # :450
            S = new_state * s_gate + S * (1.0 - s_gate)                  # :451
            ys.append(y * y_gate)                                        # :452
            tapes.append(delta * y_gate)                                 # :453
        else:
            S = new_state
            ys.append(y)
            tapes.append(delta)
    return np.stack(ys, axis=1), S, np.stack(tapes, axis=1)


def gated_delta_rowwise(q, k, v, g, beta, state, mask=None, n_per_seq=None):
    """Second, independent statement: the body of the Metal kernel, row by row
    (Sources/DFlash/DFlashKernels.swift:122-199) with InT = float (its per-step rounding,
    :183-186, is then the identity).  Masked-off steps restore the pre-decay row (:185).
    Slow; used on small shapes to cross-check gated_delta_ops_with_tape."""
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    g = np.asarray(g, dtype=np.float32)
    beta = np.asarray(beta, dtype=np.float32)
    B, T, Hk, Dk = q.shape
    Hv, Dv = v.shape[2], v.shape[3]
    S = np.array(state, dtype=np.float32, copy=True)
    y = np.zeros((B, T, Hv, Dv), np.float32)
    tape = np.zeros((B, T, Hv, Dv), np.float32)
    on = _step_mask(mask, n_per_seq, B, T)
    for b in range(B):
        for hv in range(Hv):
            hk = hv // (Hv // Hk)                                        # :126
            for t in range(T):
                if on is not None and not on[b, t]:
                    continue                                             # :165, :185
                gt = g[b, t, hv] if g.ndim == 4 else np.float32(g[b, t, hv])
                rows = S[b, hv] * gt                                     # :157
                kv = rows @ k[b, t, hk]                                  # :158, :166
                d = (v[b, t, hv] - kv) * beta[b, t, hv]                  # :167-168
                rows = rows + np.outer(d, k[b, t, hk])                   # :171
                y[b, t, hv] = rows @ q[b, t, hk]                         # :172-174
                tape[b, t, hv] = d                                       # :179
                S[b, hv] = rows
    return y, S, tape


def kimi_gated_delta_update(q, k, v, g, beta, state):
    """Third statement (vector gate, Hk == Hv): kimiGatedDeltaUpdate,
    Sources/SwiftLM/KimiLinearDFlash.swift:383-405, taking the already-activated g and beta."""
    q = np.asarray(q, np.float32); k = np.asarray(k, np.float32); v = np.asarray(v, np.float32)
    g = np.asarray(g, np.float32); beta = np.asarray(beta, np.float32)
    s = np.array(state, np.float32, copy=True)
    ys = []
    for t in range(q.shape[1]):
        s = s * g[:, t][..., None, :]                                    # :398
        kv = (s * k[:, t][..., None, :]).sum(-1, dtype=np.float32)       # :399
        d = (v[:, t] - kv) * beta[:, t][..., None]                       # :400
        s = s + k[:, t][..., None, :] * d[..., None]                     # :401
        ys.append((s * q[:, t][..., None, :]).sum(-1, dtype=np.float32))  # :402
    return np.stack(ys, 1), s


# --------------------------------------------------------------------------------------------
# Tape replay
# --------------------------------------------------------------------------------------------


def tape_replay_ops(tape, k, g, state, mask=None, n_per_seq=None):
    """Restates tapeReplayOps, Sources/DFlash/DFlashKernels.swift:371-407:
    S <- S * g_t + delta_t (x) k_t for t < T; a masked-off step keeps the old S (:399-404).

    The ops path broadcasts the mask as if B == 1 (:402); the kernel indexes mask[b*T + t]
    (:36) and that is the contract restated here (the reference's uncompiled alternative file
    does the same, Sources/DFlash/DFlashKernelsOptimized.swift:273).
    """
    tape = np.asarray(tape, np.float32)
    k = np.asarray(k, np.float32)
    g = np.asarray(g, np.float32)
    S = np.array(state, np.float32, copy=True)
    B, T, Hv, Dv = tape.shape
    k = _repeat_heads(k, Hv)                                             # :381-385
    on = _step_mask(mask, n_per_seq, B, T)
    for t in range(T):
        prev = S                                                         # :389
        if g.ndim == 4:
            decay = g[:, t, :, None, :]                                  # :392
        else:
            decay = g[:, t, :, None, None]                               # :394
        delta = tape[:, t, :, :, None]                                   # :396
        kt = k[:, t, :, None, :]                                         # :397
        S = S * decay + delta * kt                                       # :398
        if on is not None:
            S = np.where(on[:, t][:, None, None, None], S, prev)         # :402-403
    return S


# --------------------------------------------------------------------------------------------
# Rollback indexing (host contract of the caller)
# --------------------------------------------------------------------------------------------


def rollback_accepted_steps(n_accepted: int) -> int:
    """Sources/DFlash/RecurrentRollbackCache.swift:115: replay length = nAccepted + 1."""
    return int(n_accepted) + 1


def rebuild_conv_state(conv_snapshot, tape_qkv, accepted_steps: int, conv_kernel_size: int = 4):
    """Sources/DFlash/RecurrentRollbackCache.swift:139-158.

    conv_snapshot [B,keep,C] or None (zeros, :148-151); tape_qkv [B,T,C].
    Returns concat(prefix, qkv)[:, start:end] with start = accepted_steps,
    end = min(start + keep, len) (:155-157); keep = conv_kernel_size - 1 (:141)."""
    keep = conv_kernel_size - 1
    if keep <= 0:
        return None                                                      # :142
    tape_qkv = np.asarray(tape_qkv)
    if conv_snapshot is None:
        prefix = np.zeros((tape_qkv.shape[0], keep, tape_qkv.shape[-1]), tape_qkv.dtype)
    else:
        prefix = np.asarray(conv_snapshot)
    conv_input = np.concatenate([prefix, tape_qkv], axis=1)              # :154
    start = accepted_steps
    end = min(start + keep, conv_input.shape[1])                         # :156
    return conv_input[:, start:end]


def fully_accepted(acceptance_length: int, drafted_tokens: int) -> bool:
    """Sources/DFlash/DFlashRuntime.swift:194: full accept => no replay, keep verify state."""
    return drafted_tokens > 0 and acceptance_length == drafted_tokens


# --------------------------------------------------------------------------------------------
# Acceptance
# --------------------------------------------------------------------------------------------


def greedy_tokens_with_mask(logits, suppress_mask=None):
    """Sources/DFlash/DFlashRuntime.swift:118-128: argmax over the vocabulary after forcing
    suppressed ids to -1e9 (in the logits' dtype); ties -> lowest index; result uint32."""
    logits = np.asarray(logits)
    if suppress_mask is not None:
        floor = np.array(-1e9, dtype=logits.dtype)
        logits = np.where(np.asarray(suppress_mask, bool), floor, logits)
    return np.argmax(logits, axis=-1).astype(np.uint32)


def match_acceptance_length(drafted, posterior) -> int:
    """Sources/DFlash/DFlashRuntime.swift:133-142: sum(cumprod(drafted == posterior))."""
    drafted = np.asarray(drafted)
    posterior = np.asarray(posterior)
    if drafted.shape[0] == 0:
        return 0
    matches = (drafted == posterior).astype(np.int32)
    return int(np.cumprod(matches, axis=0).sum(axis=0))


def accept_block(verify_ids, posterior):
    """One cycle's bookkeeping, Sources/DFlash/DFlashRuntime.swift:523-547.

    verify_ids [T] (staged token followed by T-1 drafted), posterior [T] (greedy target tokens).
    accept = match(verify_ids[1:], posterior[:-1]); commit = 1 + accept (:544);
    next staged token = posterior[accept] (:547)."""
    verify_ids = np.asarray(verify_ids)
    posterior = np.asarray(posterior)
    accept = match_acceptance_length(verify_ids[1:], posterior[:-1])
    return accept, 1 + accept, int(posterior[accept])


class TrimmableKVCache:
    """The attention cache as the verify cycle uses it: one growing [Hkv, n, D] history per sequence.

    update() is the append of the target forward over the block; restore() follows
    restoreTargetCacheAfterAcceptance, Sources/DFlash/DFlashRuntime.swift:188-223, for a trimmable
    cache: offset > targetLen => trim(offset - targetLen), with targetLen = start + accepted
    inputs.  Per-sequence lengths (the reference runs B = 1)."""

    def __init__(self, batch: int, kv_heads: int, head_dim: int, dtype=np.float32):
        self.k = [np.zeros((kv_heads, 0, head_dim), dtype) for _ in range(batch)]
        self.v = [np.zeros((kv_heads, 0, head_dim), dtype) for _ in range(batch)]

    def offset(self, b: int) -> int:
        return self.k[b].shape[1]

    def update(self, k_new, v_new):
        """k_new, v_new [B,Hkv,T,D]: appended behind every sequence's history."""
        for b in range(len(self.k)):
            self.k[b] = np.concatenate([self.k[b], np.asarray(k_new[b], self.k[b].dtype)], axis=1)
            self.v[b] = np.concatenate([self.v[b], np.asarray(v_new[b], self.v[b].dtype)], axis=1)

    def trim(self, b: int, n: int) -> int:
        n = min(self.offset(b), max(0, int(n)))
        keep = self.offset(b) - n
        self.k[b] = self.k[b][:, :keep]
        self.v[b] = self.v[b][:, :keep]
        return n

    def restore(self, start_lens, accepted_inputs):
        """After verification: sequence b keeps start_lens[b] + accepted_inputs[b] rows (:212-218)."""
        for b in range(len(self.k)):
            target_len = int(start_lens[b]) + int(accepted_inputs[b])
            if self.offset(b) > target_len:
                self.trim(b, self.offset(b) - target_len)


# --------------------------------------------------------------------------------------------
# Block-verify SDPA
# --------------------------------------------------------------------------------------------

M_FIXED = 16  # query rows per head (Sources/DFlash/DFlashKernels.swift:755)


def finite_min(dtype_name: str) -> np.float32:
    """Limits<InT>::finite_min for the additive-mask test (:551)."""
    if dtype_name == "bf16":
        return np.float32(-3.3895313892515355e38)
    if dtype_name == "fp16":
        return np.float32(-65504.0)
    return np.finfo(np.float32).min


def verify_sdpa(q, k, v, scale, mask=None, kv_len=None, in_dtype="bf16"):
    """softmax(scale * Q K^T + M) V with the block-causal visibility rule of the reference's
    kernel: key n is visible to query row r iff n <= N - 16 + r, N counting the 16 block keys
    (Sources/DFlash/DFlashKernels.swift:614).  fp32 scores and accumulation (:618-633).

    q [B,Hq,16,D]; k,v [B,Hkv,N,D]; KV head = q_head // (Hq/Hkv) (:575).
    mask: optional additive [B,Hq,16,N]; entries < finite_min(in_dtype) hide the key (:551),
    otherwise the value is added to the score (:553).
    kv_len: optional per-sequence N_b <= N (keys beyond N_b do not exist for sequence b).
    Returns fp32 [B,Hq,16,D]; rows with no visible key return zeros (:711 guard).
    """
    q = np.asarray(q, np.float32)
    k = np.asarray(k, np.float32)
    v = np.asarray(v, np.float32)
    B, Hq, M, D = q.shape
    Hkv, N = k.shape[1], k.shape[2]
    assert M == M_FIXED and Hq % Hkv == 0
    gqa = Hq // Hkv
    out = np.zeros((B, Hq, M, v.shape[3]), np.float32)
    fmin = finite_min(in_dtype)
    for b in range(B):
        Nb = int(kv_len[b]) if kv_len is not None else N
        n_idx = np.arange(Nb)[None, :]
        r_idx = np.arange(M)[:, None]
        visible = n_idx <= (Nb - M + r_idx)                               # :614
        for h in range(Hq):
            hk = h // gqa                                                 # :575
            qs = np.float32(scale) * q[b, h]                              # :593-595
            s = qs @ k[b, hk, :Nb].T                                      # :618-622
            use = visible.copy()
            if mask is not None:
                mv = np.asarray(mask[b, h, :, :Nb], np.float32)
                use &= mv >= fmin                                         # :551
                s = s + mv                                                # :553
            s = np.where(use, s, -np.inf)
            mx = s.max(axis=-1, keepdims=True)
            mx = np.where(np.isfinite(mx), mx, 0.0)
            p = np.where(use, np.exp(s - mx), 0.0).astype(np.float32)
            den = p.sum(axis=-1, keepdims=True, dtype=np.float32)
            o = p @ v[b, hk, :Nb]
            out[b, h] = np.where(den == 0.0, o, o / np.where(den == 0.0, 1.0, den))  # :711
    return out


def verify_sdpa_two_pass(q, k, v, scale, blocks: int, in_dtype="bf16", round_partials=False):
    """Literal restatement of the two-pass structure: pass 1 gives block i the keys
    n = i, i + blocks, ... (:603) with a running max initialised to finite_min(float) (:600)
    and an online softmax (:625-633); pass 2 is the log-sum-exp merge (:687-711).
    round_partials=True rounds partial O to the input dtype between passes as the reference
    does (:647).  Used to check split-count invariance; small shapes only."""
    q = np.asarray(q, np.float32); k = np.asarray(k, np.float32); v = np.asarray(v, np.float32)
    B, Hq, M, D = q.shape
    Hkv, N = k.shape[1], k.shape[2]
    gqa = Hq // Hkv
    fm = np.finfo(np.float32).min
    out = np.zeros((B, Hq, M, D), np.float32)
    for b in range(B):
        for h in range(Hq):
            hk = h // gqa
            for r in range(M):
                qs = np.float32(scale) * q[b, h, r]
                part = np.zeros((blocks, D), np.float32)
                sums = np.zeros(blocks, np.float32)
                maxs = np.full(blocks, fm, np.float32)
                for blk in range(blocks):
                    mx, se, o = np.float32(fm), np.float32(0), np.zeros(D, np.float32)
                    for n in range(blk, N, blocks):
                        if n > N - M + r:
                            continue
                        sc = np.float32(qs @ k[b, hk, n])
                        nm = max(mx, sc)
                        f = np.exp(np.float32(mx - nm)); e = np.exp(np.float32(sc - nm))
                        mx = nm; se = se * f + e; o = o * f + e * v[b, hk, n]
                    if round_partials:
                        o = _round_to(o, in_dtype)
                    part[blk], sums[blk], maxs[blk] = o, se, mx
                gm = maxs.max()
                fac = np.exp(maxs - gm).astype(np.float32)
                den = np.float32((fac * sums).sum(dtype=np.float32))
                o = (fac[:, None] * part).sum(0, dtype=np.float32)
                out[b, h, r] = o if den == 0 else o / den
    return out


def compute_sdpa_2pass_blocks(gqa_factor: int, n_kv: int, device_arch: str = "") -> int:
    """Split-count heuristic of the reference, Sources/DFlash/DFlashKernels.swift:470-506
    (keyed on the last letter of the Apple GPU architecture string)."""
    devc = device_arch[-1:] if device_arch else ""
    n_simds, N = gqa_factor, n_kv
    if devc == "d":
        blocks = 128
        if n_simds <= 2 and N > 8192:
            blocks = 256
        elif n_simds >= 6:
            if 16384 <= N < 65536:
                blocks = 512
            elif N >= 65536:
                blocks = 1024
    elif devc == "s":
        blocks = 64
        if N > 1024 and n_simds > 4:
            if N <= 8192:
                blocks = 128
            elif N <= 32768:
                blocks = 256
            elif N <= 65536:
                blocks = 512
            else:
                blocks = 1024
    else:
        blocks = 64 if n_simds >= 4 else 32
    return blocks


def sdpa_supported(q_shape, k_shape, v_shape, dtype_name: str) -> bool:
    """Eligibility guards of batchedSDPA2Pass (:744-758): anything else returns nil."""
    if len(q_shape) != 4 or len(k_shape) != 4 or len(v_shape) != 4:
        return False
    if q_shape[2] != 16 or dtype_name not in ("bf16", "fp16"):
        return False
    D, V = q_shape[3], v_shape[3]
    if not (D in (128, 256) and V in (128, 256) and D == V):
        return False
    Hq, Hk = q_shape[1], k_shape[1]
    return Hk > 0 and Hq % Hk == 0


# --------------------------------------------------------------------------------------------
# dtype helpers
# --------------------------------------------------------------------------------------------


def round_bf16(x):
    """Round-to-nearest-even fp32 -> bf16 -> fp32 (what a cast to a bf16 array does)."""
    x = np.ascontiguousarray(np.asarray(x, np.float32))
    u = x.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = r.astype(np.uint32).view(np.float32)
    return np.where(np.isnan(x), x, out).reshape(x.shape)


def _round_to(x, dtype_name):
    if dtype_name == "bf16":
        return round_bf16(x)
    if dtype_name == "fp16":
        return np.asarray(x, np.float32).astype(np.float16).astype(np.float32)
    return np.asarray(x, np.float32)


# --------------------------------------------------------------------------------------------
# Seeded synthetic inputs (stand-ins for Qwen3-Next activations; distributions per config)
# --------------------------------------------------------------------------------------------

BASE_SEED = 20260330  # the seed of the reference's codec test, tests/test_turbo_quant.cpp:23


def make_gdn_inputs(B, T, Hk, Hv, Dk, Dv, seed, vector_gate=False, dtype="fp32"):
    """q,k ~ N(0,1) L2-normalised over Dk; v ~ N(0,1); beta = sigmoid(N(0,1));
    g = exp(-softplus(N(0,1))) in (0,1); S0 ~ N(0,0.02); n ~ U{0..T}.
    With dtype 'bf16' the per-token inputs are rounded to bf16 values (state stays fp32)."""
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((B, T, Hk, Dk)).astype(np.float32)
    k = rng.standard_normal((B, T, Hk, Dk)).astype(np.float32)
    q /= np.linalg.norm(q, axis=-1, keepdims=True)
    k /= np.linalg.norm(k, axis=-1, keepdims=True)
    v = rng.standard_normal((B, T, Hv, Dv)).astype(np.float32)
    beta = (1.0 / (1.0 + np.exp(-rng.standard_normal((B, T, Hv))))).astype(np.float32)
    gshape = (B, T, Hv, Dk) if vector_gate else (B, T, Hv)
    x = rng.standard_normal(gshape)
    g = np.exp(-np.log1p(np.exp(x))).astype(np.float32)
    state = (0.02 * rng.standard_normal((B, Hv, Dv, Dk))).astype(np.float32)
    n = rng.integers(0, T + 1, size=(B,)).astype(np.int32)
    if dtype != "fp32":
        q, k, v, beta, g = (_round_to(a, dtype) for a in (q, k, v, beta, g))
    return dict(q=q, k=k, v=v, g=g, beta=beta, state=state, n=n)


def make_sdpa_inputs(B, Hq, Hkv, N, D, seed, dtype="bf16"):
    """Q,K,V ~ N(0,1) rounded to the input dtype; scale = 1/sqrt(D)."""
    rng = np.random.default_rng(seed)
    q = _round_to(rng.standard_normal((B, Hq, M_FIXED, D)).astype(np.float32), dtype)
    k = _round_to(rng.standard_normal((B, Hkv, N, D)).astype(np.float32), dtype)
    v = _round_to(rng.standard_normal((B, Hkv, N, D)).astype(np.float32), dtype)
    return dict(q=q, k=k, v=v, scale=np.float32(1.0 / np.sqrt(D)))
