/* dflash_cuda.h — C ABI of the B200 (sm_100a) implementation of SwiftLM's DFlash
 * speculative-verify kernels.
 *
 * These entry points are what the Swift functions in Sources/DFlash/DFlashKernels.swift of the
 * SwiftLM tree bind to once their Metal bodies are replaced (a SwiftPM C target exposes this
 * header through a module map).  Conventions, all functions:
 *   - every pointer is a DEVICE pointer on the current CUDA device unless its name says "host";
 *   - tensors are dense, row-major, last axis contiguous, exactly the reference's layouts;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the default stream); work is
 *     stream-ordered and the call returns without synchronising;
 *   - the caller owns every buffer; the library keeps no reference after the call returns;
 *   - the return value is a dflash_status (0 = ok, negative = error); nothing aborts, nothing
 *     falls back to a CPU path.  dflash_last_error_string() describes the last failure of the
 *     calling thread.
 *   - base pointers must be 16-byte aligned (cudaMalloc gives 256).
 */
#ifndef DFLASH_CUDA_H
#define DFLASH_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  DFLASH_OK = 0,
  DFLASH_ERR_INVALID_ARG = -1,   /* null pointer, non-positive size, misaligned base pointer */
  DFLASH_ERR_UNSUPPORTED = -2,   /* shape or dtype outside the supported set (the reference returns nil / falls back) */
  DFLASH_ERR_CUDA = -3,          /* a CUDA runtime or driver call failed; see dflash_last_error_string() */
  DFLASH_ERR_WORKSPACE = -4,     /* workspace missing or smaller than *_workspace_bytes() */
  DFLASH_ERR_DEVICE_TIMEOUT = -5, /* a bounded device-side wait gave up (reported by dflash_device_status) */
  DFLASH_ERR_DEVICE_DATA = -6     /* a kernel found device-resident data out of range, e.g. a KV position beyond the
                                     cache's capacity (reported by dflash_device_status) */
} dflash_status;

typedef enum { DFLASH_F32 = 0, DFLASH_BF16 = 1, DFLASH_F16 = 2, DFLASH_U8 = 3 } dflash_dtype;

/* KV storage formats of dflash_verify_sdpa. */
typedef enum { DFLASH_KV_DENSE = 0, DFLASH_KV_TURBO3 = 1 } dflash_kv_format;

/* KV held in the TurboQuant 3-bit format (see dflash_turbo_encode below) with the reference's hot
 * window (docs/turboquant_hybrid_architecture.md:49-53 of the SwiftLM tree): the oldest n_cold
 * tokens of every (sequence, KV head) are compressed, the newest n_hot tokens (the verify block
 * among them) stay in the attention dtype; attention sees [decoded cold | hot], N = n_cold + n_hot.
 * Compressed arrays are device arrays over [B,Hkv,n_cold, D/128 blocks], each 16-byte aligned; hot
 * arrays are [B,Hkv,n_hot,D] (NULL when n_hot == 0).  With kv_format == DFLASH_KV_TURBO3 the `k` argument of
 * dflash_verify_sdpa points at one of these (in host memory) and `v` is ignored. */
typedef struct {
  const uint8_t* k_packed;   /* [blocks,48] */
  const uint8_t* k_signs;    /* [blocks,16] */
  const uint16_t* k_norm;    /* [blocks] fp16 bits */
  const uint16_t* k_rnorm;   /* [blocks] fp16 bits */
  const uint8_t* v_packed;   /* [blocks,48] */
  const uint16_t* v_norm;    /* [blocks] fp16 bits */
  const void* k_hot;         /* [B,Hkv,n_hot,D] or NULL */
  const void* v_hot;
  int32_t n_cold;
  int32_t n_hot;
} dflash_turbo_kv;

/* ---------------------------------------------------------------------------------------------
 * Gated-delta forward that records the innovation tape; with n_per_seq it is the replay of a
 * recorded (q,k,v,beta,g) block from the last committed state to the accepted length.
 * Replaces DFlashKernels.gatedDeltaKernelWithTape, Sources/DFlash/DFlashKernels.swift:316-367
 * (kernel body :122-199, CPU statement :409-466).
 *
 *   q,k      [B,T,Hk,Dk]  in_dtype          v    [B,T,Hv,Dv]  in_dtype
 *   g        [B,T,Hv] or, if g_is_vector, [B,T,Hv,Dk]  in_dtype   (the decay itself, in (0,1))
 *   beta     [B,T,Hv]     in_dtype          state_in / state_out  [B,Hv,Dv,Dk]  fp32
 *   mask     [B,T] mask_dtype or NULL: step t of sequence b runs iff mask > 0.5        (:36,:115)
 *   n_per_seq int32[B] or NULL: step t runs iff t < n_per_seq[b] (accepted length)
 *   y        [B,T,Hv,Dv]  in_dtype          tape [B,T,Hv,Dv] fp32, may be NULL
 * Per running step, per (b, hv), hk = hv / (Hv/Hk):  S *= g;  kv = S k;  delta = (v - kv) beta;
 * S += delta (x) k;  y = S q.  A step that does not run leaves S untouched and writes y = 0,
 * tape = 0.  fp32 arithmetic, no per-step rounding of the state.  state_out may alias state_in.
 * Supported: Dk % 32 == 0, Dk <= 512, Hv % Hk == 0, T <= 64; in_dtype f32 / bf16 / f16.
 */
int32_t dflash_gated_delta_tape(const void* q, const void* k, const void* v, const void* g,
                                const void* beta, const float* state_in, const void* mask,
                                const int32_t* n_per_seq, void* y, float* state_out, float* tape,
                                int32_t B, int32_t T, int32_t Hk, int32_t Hv, int32_t Dk, int32_t Dv,
                                int32_t g_is_vector, int32_t in_dtype, int32_t mask_dtype,
                                void* stream);

/* Tape replay:  S <- S * g_t + delta_t (x) k_t  for the running steps.
 * Replaces DFlashKernels.tapeReplayKernel, Sources/DFlash/DFlashKernels.swift:252-301 (kernel
 * body :43-81, CPU statement :371-407).  The caller in the reference slices the first
 * nAccepted+1 steps before the call (Sources/DFlash/RecurrentRollbackCache.swift:115-125);
 * here the same is expressed without copies by n_per_seq[b] = nAccepted_b + 1.
 *   tape [B,T,Hv,Dv] fp32;  k [B,T,Hk,Dk], g [B,T,Hv(,Dk)] in kg_dtype;  state fp32.
 * mask / n_per_seq / aliasing / supported shapes as above.
 */
int32_t dflash_tape_replay(const float* tape, const void* k, const void* g, const float* state_in,
                           const void* mask, const int32_t* n_per_seq, float* state_out, int32_t B,
                           int32_t T, int32_t Hk, int32_t Hv, int32_t Dk, int32_t Dv,
                           int32_t g_is_vector, int32_t kg_dtype, int32_t mask_dtype, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Batched block-verify attention:  out = softmax(scale * Q K^T [+ mask]) V  with the reference's
 * visibility rule: key n is visible to query row r iff n <= N_b - 16 + r, where N_b counts the
 * 16 block keys (Sources/DFlash/DFlashKernels.swift:614).
 * Replaces DFlashKernels.batchedSDPA2Pass, :737-815 (partials kernel :563-649, reduce :661-720).
 *
 *   q, out  [B,Hq,16,D]  dtype (bf16 or f16)
 *   dense KV, page_table == NULL:   k,v [B,Hkv,N,D]
 *   paged KV, page_table != NULL:   k,v [num_pages,Hkv,page_tokens,D]; page_table int32
 *           [B,max_pages]; logical token n of sequence b lives in page page_table[b][n/page_tokens]
 *           at row n % page_tokens (page_tokens a multiple of 128; not part of the reference).
 *           num_pages is the pool's page count: a table entry outside [0, num_pages) reads as
 *           zero keys/values instead of memory outside the pool, and dflash_device_status then
 *           returns DFLASH_ERR_DEVICE_DATA.  Ignored (pass 0) for dense KV.
 *   kv_len_per_seq int32[B] or NULL (every sequence has N keys); 16 <= N_b <= N.  The array is
 *           read on the device; an entry outside that range is clamped to [0, N] before any
 *           address is formed from it and reported the same way (a sequence clamped to 0 keys
 *           gets no output)
 *   mask    additive [B,Hq,16,N] dtype or NULL; a value < the most negative finite value of
 *           dtype hides the key (:551), otherwise it is added to the score (:553)
 *   workspace: dflash_verify_sdpa_workspace_bytes() bytes of device scratch (split-KV partials)
 * Supported, as the reference (:755-758): T == 16, dtype bf16/f16, D in {128,256},
 * Hq % Hkv == 0; otherwise DFLASH_ERR_UNSUPPORTED (the reference returns nil).
 */
int32_t dflash_verify_sdpa(const void* q, const void* k, const void* v, const int32_t* page_table,
                           const int32_t* kv_len_per_seq, const void* mask, void* out,
                           void* workspace, size_t workspace_bytes, int32_t B, int32_t Hq,
                           int32_t Hkv, int32_t T, int32_t D, int32_t N, int32_t page_tokens,
                           int32_t max_pages, int32_t num_pages, float scale, int32_t dtype,
                           int32_t kv_format, void* stream);

size_t dflash_verify_sdpa_workspace_bytes(int32_t B, int32_t Hq, int32_t Hkv, int32_t D, int32_t N);
/* The same for a given kv_format.  DFLASH_KV_TURBO3 takes one of two routes (no page table either way):
 *   fused   - cold history a multiple of 128 keys, no kv_len_per_seq, no mask, scale > 0: the query rows are
 *             rotated once, the attention kernel expands packed indices and sign bits into its tensor-core
 *             operands tile by tile, the output rows are rotated back; no decoded key or value reaches
 *             global memory.  Workspace: three query-sized arrays, the hot window twice, the partials.
 *   expand  - anything else: K and V are decoded into the workspace (2 * B*Hkv*N*D elements of 2 bytes) and
 *             the dense kernel attends over the copy.
 * _ex returns a size good for either route whatever n_cold is; _turbo_workspace_bytes returns what the route
 * a given (n_cold, n_hot) takes needs, which for the fused route is far less. */
size_t dflash_verify_sdpa_workspace_bytes_ex(int32_t B, int32_t Hq, int32_t Hkv, int32_t D, int32_t N, int32_t kv_format);
size_t dflash_verify_sdpa_turbo_workspace_bytes(int32_t B, int32_t Hq, int32_t Hkv, int32_t D, int32_t n_cold, int32_t n_hot);

/* Same computation as dflash_verify_sdpa for a caller that cannot supply scratch memory (a host
 * whose device-memory budget is fixed and whose allocator is closed to plug-ins, or a request path
 * that must never reach cudaMalloc).  It has no counterpart in the reference.  The split-KV
 * partials live in a 40 MiB device array that is part of the library image (every GPU that loads
 * the library holds it until exit): enough for head_dim <= 256 on up to 158 SMs; a call that needs
 * more returns DFLASH_ERR_WORKSPACE.  Dense or paged KV only: DFLASH_KV_TURBO3 is answered with
 * DFLASH_ERR_UNSUPPORTED, because that form is expanded into scratch (B*Hkv*N*D*4 bytes) before
 * attending.  Arguments are checked before the device is touched, so a bad call gets the same
 * answer as from dflash_verify_sdpa.  Nothing is allocated.  The first valid call on a device
 * resolves the array's address and loads the kernels: make it before any stream capture.  All
 * calls share the array (it keeps the previous call's contents; nothing needs clearing), so calls
 * that overlap on the GPU race: serialise them. */
int32_t dflash_verify_sdpa_noalloc(const void* q, const void* k, const void* v, const int32_t* page_table,
                                   const int32_t* kv_len_per_seq, const void* mask, void* out, int32_t B,
                                   int32_t Hq, int32_t Hkv, int32_t T, int32_t D, int32_t N,
                                   int32_t page_tokens, int32_t max_pages, int32_t num_pages, float scale,
                                   int32_t dtype, int32_t kv_format, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Acceptance bookkeeping on the device (no host round trip of the accepted length).
 * dflash_greedy_tokens replaces DFlashRuntime.greedyTokensWithMask,
 * Sources/DFlash/DFlashRuntime.swift:118-128: argmax over the vocabulary with suppressed ids
 * forced to -1e9, ties to the lowest index.  logits [rows,V] logits_dtype; suppress uint8[V] or
 * NULL; posterior uint32[rows].
 * dflash_accept_lengths replaces DFlashRuntime.matchAcceptanceLength, :133-142, and the
 * commit arithmetic :523-547: verify_ids int32[B,T] (staged token, then T-1 drafted);
 * accept[b] = number of leading i < T-1 with verify_ids[b,i+1] == posterior[b,i];
 * next_token[b] = posterior[b, accept[b]]; replay_len[b] = accept[b] + 1, the n_per_seq of the
 * replay (Sources/DFlash/RecurrentRollbackCache.swift:115).  next_token / replay_len may be NULL.
 */
int32_t dflash_greedy_tokens(const void* logits, const uint8_t* suppress, uint32_t* posterior,
                             int32_t rows, int32_t V, int32_t logits_dtype, void* stream);
int32_t dflash_accept_lengths(const uint32_t* posterior, const int32_t* verify_ids, int32_t* accept,
                              int32_t* next_token, int32_t* replay_len, int32_t B, int32_t T,
                              void* stream);
/* out[b,:] = logits[b, clamp(row_per_seq[b], 0, T-1), :]: the verify-logits row of each sequence's
 * accepted position, i.e. the row whose argmax is next_token (posterior[acceptanceLen],
 * Sources/DFlash/DFlashRuntime.swift:547), picked with the accepted count still on the device.
 * This is the logits slice a sequence-sharded step all-gathers next to the acceptance results
 * (a sampler or log-probability consumer on another rank needs that row, not the other T-1).
 * logits [B,T,V] logits_dtype; row_per_seq int32[B] (accept of dflash_accept_lengths); out [B,V]. */
int32_t dflash_gather_logits_rows(const void* logits, const int32_t* row_per_seq, void* out, int32_t B,
                                  int32_t T, int32_t V, int32_t logits_dtype, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Conv-window rebuild of the rollback cache: replaces RecurrentRollbackCache.rebuildConvState,
 * Sources/DFlash/RecurrentRollbackCache.swift:139-158.
 *   out = concat(conv_snapshot [B,keep,C], qkv [B,T,C])[:, steps : min(steps + keep, keep + T)]
 * conv_snapshot may be NULL (zeros, :150-153).  Rows are row_bytes bytes each (a multiple of 16).
 * steps_per_seq == NULL: every sequence uses steps_all and *rows_out (host) receives the window
 * length, which is shorter than keep when steps_all + keep runs past the end, as in the reference.
 * steps_per_seq != NULL (device int32[B], e.g. replay_len of dflash_accept_lengths): per-sequence
 * starts, clamped to T, keep rows each; out is [B,keep,C].
 */
int32_t dflash_rebuild_conv_state(const void* conv_snapshot, const void* qkv, const int32_t* steps_per_seq,
                                  int32_t steps_all, void* out, int32_t B, int32_t T, int32_t keep,
                                  int64_t row_bytes, int32_t* rows_out, void* stream);

/* ---------------------------------------------------------------------------------------------
 * KV cache maintenance around the verify attention, without the accepted count on the host.
 * Replaces the cache update of the target forward and the trim of restoreAfterAcceptance,
 * Sources/DFlash/DFlashRuntime.swift:188-223 (targetLen = start + accepted inputs;
 * cache.trim(offset - targetLen)).
 * dflash_kv_append writes the block's rows k_new / v_new [B,Hkv,T,D] (dtype) behind the committed
 * tokens: row t of sequence b goes to position kv_len[b] + t (kv_len == NULL: len_all + t) of
 *   a dense cache  [B,Hkv,capacity,D]                       (page_table == NULL), or
 *   a paged pool   [num_pages,Hkv,page_tokens,D] through page_table int32[B,max_pages]
 *   (the layout dflash_verify_sdpa reads).
 * kv_len_out (int32[B] or NULL, not the same array as kv_len) receives min(kv_len[b] + T, capacity),
 * the length the verify attention must be given.  A position beyond the capacity, or on a page that is
 * negative or >= num_pages, is skipped and dflash_device_status then returns
 * DFLASH_ERR_DEVICE_DATA.
 * dflash_kv_commit: kv_len[b] += clamp(commit[b], 0, T) with commit = replay_len of
 * dflash_accept_lengths (accepted drafts + 1).  Rejected rows stay in place and are overwritten
 * by the next block: the trim.
 */
int32_t dflash_kv_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                         const int32_t* page_table, const int32_t* kv_len, int32_t len_all,
                         int32_t* kv_len_out, int32_t B, int32_t Hkv, int32_t T, int32_t D,
                         int32_t capacity, int32_t page_tokens, int32_t max_pages, int32_t num_pages,
                         int32_t dtype, void* stream);
int32_t dflash_kv_commit(int32_t* kv_len, const int32_t* commit, int32_t B, int32_t T, void* stream);

/* ---------------------------------------------------------------------------------------------
 * TurboQuant 3-bit KV codec, 128-dimension blocks (a 256-dimension head vector is two blocks).
 * Follows the codec as stated in the reference's tests/test_turbo_quant.cpp: V path :69-75, K path
 * with residual sign bits :85-98, primitives :14-22 (the production encoder lives in a dependency
 * that is not part of the reference tree).  Results are bit-identical to that statement.
 *   x / out  [n_blocks,128] dtype (f32, bf16, f16)
 *   packed   uint8[n_blocks,48]  3-bit centroid indices, little-endian bit stream
 *   signs    uint8[n_blocks,16]  K only: sign bits of the rotated residual (NULL for V)
 *   norm     uint16[n_blocks]    fp16 bits: ||k|| (K) or ||v|| / ||centroid vector|| (V)
 *   rnorm    uint16[n_blocks]    K only: fp16 bits of the residual norm (NULL for V)
 * dflash_turbo_decode needs packed, signs and out 16-byte aligned.  dflash_turbo_encode takes any
 * alignment; with x, packed and signs 16-byte aligned it runs its fast kernel (same bytes).
 */
int32_t dflash_turbo_encode(const void* x, uint8_t* packed, uint8_t* signs, uint16_t* norm, uint16_t* rnorm,
                            int64_t n_blocks, int32_t is_key, int32_t in_dtype, void* stream);
int32_t dflash_turbo_decode(const uint8_t* packed, const uint8_t* signs, const uint16_t* norm,
                            const uint16_t* rnorm, void* out, int64_t n_blocks, int32_t is_key,
                            int32_t out_dtype, void* stream);

/* ---------------------------------------------------------------------------------------------
 * One DFlash verify step over a hybrid stack, a handful of launches in all.
 * Composes, below the ABI, what the reference's runtime does per speculative cycle between
 * Sources/DFlash/DFlashRuntime.swift:499 and :579: the verify forward of every gated-delta layer with
 * its tape recorded (:502, through the provider, DFlashKernelProvider.swift:9-13), the block-verify
 * attention of every attention layer, the greedy posterior and the accepted length (:513-533), the
 * commit arithmetic (:544-547) and the rollback of every gated-delta layer to the accepted length
 * (restoreTargetCacheAfterAcceptance :188-223 -> RecurrentRollbackCache.rollback,
 * RecurrentRollbackCache.swift:95-131, tape replay plus conv-window rebuild).  The reference issues one
 * kernel per layer and reads the accepted length on the host (:525-530); here the layers of a kind are
 * stacked into the batch of ONE launch (item = sequence * layers + layer, sequence-major, so a GPU owns
 * whole sequences) and the accepted length stays on the device.  Layer weights are not part of the
 * path: the per-layer tensors are the caller's.
 *
 * Launches: gated-delta forward (1), attention (1, plus its merge kernel where the split needs it),
 * greedy tokens (1), accept lengths (1), logits rows (1, optional), tape replay (1), conv windows (1).
 * Every pointer is a device pointer; outputs are written in place; `workspace` as for
 * dflash_verify_sdpa with B * attn_layers sequences (dflash_verify_step_workspace_bytes).
 */
typedef struct {
  int32_t B;                 /* sequences on this GPU */
  int32_t T;                 /* block length: 16 */
  /* ---- gated-delta layers: arrays over B * gdn_layers items ---- */
  int32_t gdn_layers, Hk, Hv, Dk, Dv, g_is_vector, in_dtype;
  const void *q, *k, *v, *g, *beta;   /* as dflash_gated_delta_tape */
  const float* state;                 /* committed states [B*gdn_layers,Hv,Dv,Dk] */
  void* y;                            /* [B*gdn_layers,T,Hv,Dv] in_dtype: the verify forward's outputs */
  float* state_verify;                /* state after all T steps (what a fully accepted block keeps).  May be NULL
                                         (bf16 inputs, Dk = Dv = 128, scalar gate, T <= 16): then it is not written and
                                         state_rolled is the result for every sequence */
  float* tape;                        /* [B*gdn_layers,T,Hv,Dv] */
  float* state_rolled;                /* state replayed to replay_len[b] steps; may alias state */
  /* conv windows of the rollback cache (may all be NULL: skipped) */
  const void* conv_snapshot;          /* [B*gdn_layers,conv_keep,C] or NULL (zeros) */
  const void* qkv;                    /* [B*gdn_layers,T,C] */
  void* conv_out;                     /* [B*gdn_layers,conv_keep,C] */
  int32_t conv_keep;
  int64_t conv_row_bytes;
  /* ---- attention layers: arrays over B * attn_layers items (0 layers: skipped) ---- */
  int32_t attn_layers, Hq, Hkv, D, N, attn_dtype, kv_format;
  const void* attn_q;                 /* [B*attn_layers,Hq,16,D] */
  const void* attn_k;                 /* dense: [B*attn_layers,Hkv,N,D]; DFLASH_KV_TURBO3: host pointer to a dflash_turbo_kv */
  const void* attn_v;
  void* attn_out;                     /* [B*attn_layers,Hq,16,D] */
  float scale;
  /* ---- acceptance ---- */
  const void* logits;                 /* [B,T,V] logits_dtype */
  const uint8_t* suppress;            /* uint8[V] or NULL */
  const int32_t* verify_ids;          /* [B,T] */
  int32_t V, logits_dtype;
  uint32_t* posterior;                /* [B,T] */
  int32_t *accept, *next_token, *replay_len;   /* [B] each */
  void* logits_rows;                  /* [B,V] logits_dtype or NULL: the row at each accepted position */
} dflash_verify_step_desc;

size_t dflash_verify_step_workspace_bytes(const dflash_verify_step_desc* desc_host);
int32_t dflash_verify_step(const dflash_verify_step_desc* desc_host, void* workspace, size_t workspace_bytes,
                           void* stream);

/* ---------------------------------------------------------------------------------------------
 * Host-side helpers.
 */
/* Splits `units` independent work units (sequences for replay, (sequence, KV head) pairs for
 * attention) over n_gpus ranks in contiguous ranges, sizes differing by at most one.
 * begin_end_host: int32[2*n_gpus] receives [begin_0,end_0,begin_1,end_1,...].  Not in the
 * reference (it is single-device). */
int32_t dflash_partition_plan(int32_t units, int32_t n_gpus, int32_t* begin_end_host);

/* Reads (and clears) the device-side status word of the current device after synchronising
 * `stream`: 0; DFLASH_ERR_DEVICE_TIMEOUT if a kernel's bounded wait gave up (every device-side
 * wait has a poll budget and the kernel returns when it runs out); DFLASH_ERR_DEVICE_DATA if a
 * kernel met device-resident data out of range (a KV position past the capacity, a page id outside
 * the pool, a kv_len_per_seq entry outside [16, N], a unit cut into more key ranges than the merge
 * takes). */
int32_t dflash_device_status(void* stream);

/* Test hook, no counterpart in the reference: launches a two-warp kernel whose first warp waits, with
 * a budget of `polls` polls (1 .. 2^20), on a barrier that nothing arrives at, and whose second warp
 * must leave through the kernel's abort flag.  Exercises the give-up path of the bounded waits
 * without faulting or hanging anything; afterwards dflash_device_status returns
 * DFLASH_ERR_DEVICE_TIMEOUT once.  left_by_flag (device int32 or NULL) is set to 1 when the second
 * warp left because of the flag. */
int32_t dflash_selftest_bounded_wait(uint32_t polls, int32_t* left_by_flag, void* stream);

int32_t dflash_device_count(void);
const char* dflash_last_error_string(void);
/* Number of kernel launches issued by this library in the calling process so far. */
uint64_t dflash_launch_count(void);
const char* dflash_version(void);

#ifdef __cplusplus
}
#endif
#endif /* DFLASH_CUDA_H */
