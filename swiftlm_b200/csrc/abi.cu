// extern "C" entry points of libdflash_cuda: argument validation, dispatch, error reporting.
// Declarations and the reference interface each one replaces: include/dflash_cuda.h.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include <cstdlib>

#include "common.cuh"
#include "ptx.cuh"

namespace dflash {

namespace {
thread_local char g_error[512] = "";
std::atomic<uint64_t> g_launches{0};
__device__ int g_status_word = 0;

constexpr int kMaxDevices = 64;
std::mutex g_dev_mutex;
int* g_status_ptr[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
}  // namespace

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
}

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!g_status_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    g_status_ptr[dev] = reinterpret_cast<int*>(p);
  }
  return g_status_ptr[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!g_sm_count[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return (EncodeTiledFn) nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

namespace {

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int32_t bad(const char* what) {
  set_error("invalid argument: %s", what);
  return DFLASH_ERR_INVALID_ARG;
}

int32_t check_gdn_shape(int B, int T, int Hk, int Hv, int Dk, int Dv, int dtype, int mask_dtype,
                        const void* mask) {
  if (B <= 0 || T <= 0 || Hk <= 0 || Hv <= 0 || Dk <= 0 || Dv <= 0) return bad("non-positive dimension");
  if (dtype != DFLASH_F32 && dtype != DFLASH_BF16 && dtype != DFLASH_F16) {
    set_error("unsupported input dtype %d", dtype);
    return DFLASH_ERR_UNSUPPORTED;
  }
  if (mask && (mask_dtype < DFLASH_F32 || mask_dtype > DFLASH_U8)) return bad("mask_dtype");
  if (Dk % 32 != 0 || Dk > 512) {
    set_error("unsupported Dk=%d (need a multiple of 32, at most 512)", Dk);
    return DFLASH_ERR_UNSUPPORTED;
  }
  if (Hv % Hk != 0) {
    set_error("unsupported heads: Hv=%d is not a multiple of Hk=%d", Hv, Hk);
    return DFLASH_ERR_UNSUPPORTED;
  }
  if (T > 64) {
    set_error("unsupported T=%d (at most 64 steps per call)", T);
    return DFLASH_ERR_UNSUPPORTED;
  }
  return DFLASH_OK;
}

}  // namespace

size_t align256(size_t x) { return (x + 255) / 256 * 256; }

// The fused attention over compressed KV takes: a cold history of whole 128-key tiles, uniform lengths, no additive mask,
// a positive scale.
bool turbo_fused_applies(const dflash_turbo_kv* t, const int32_t* kv_len_per_seq, const void* mask, float scale) {
  return t->n_cold > 0 && t->n_cold % 128 == 0 && !kv_len_per_seq && !mask && scale > 0.f && sdpa_tc_turbo_available();
}
// rotated queries (two tiles) + rotated-domain output + the hot window in the rotated domain + the split-KV partials
size_t turbo_fused_workspace_bytes(int B, int Hq, int Hkv, int D, int n_hot) {
  return 3 * align256((size_t)B * Hq * 16 * D * 2) + 2 * align256((size_t)B * Hkv * n_hot * D * 2) + sdpa_tc_scratch_bytes(D) + 256;
}

// Everything dflash_verify_sdpa can reject before it touches the device; shared with the entry point
// that brings its own scratch so that both answer a bad call the same way.
int32_t sdpa_check_args(const void* q, const void* k, const void* v, const int32_t* page_table, const void* out,
                        int32_t B, int32_t Hq, int32_t Hkv, int32_t T, int32_t D, int32_t N, int32_t page_tokens,
                        int32_t max_pages, int32_t num_pages, int32_t dtype, int32_t kv_format) {
  if (!q || !k || (!v && kv_format == DFLASH_KV_DENSE) || !out) return bad("null tensor pointer");
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || N <= 0) return bad("non-positive dimension");
  // eligibility of the reference's kernel, Sources/DFlash/DFlashKernels.swift:755-758
  if (T != 16) { set_error("unsupported query length %d (the verify block has 16 rows)", T); return DFLASH_ERR_UNSUPPORTED; }
  if (dtype != DFLASH_BF16 && dtype != DFLASH_F16) { set_error("unsupported dtype %d (bf16 or f16)", dtype); return DFLASH_ERR_UNSUPPORTED; }
  if (D != 128 && D != 256) { set_error("unsupported head_dim %d (128 or 256)", D); return DFLASH_ERR_UNSUPPORTED; }
  if (Hq % Hkv != 0) { set_error("unsupported heads: Hq=%d not a multiple of Hkv=%d", Hq, Hkv); return DFLASH_ERR_UNSUPPORTED; }
  if (N < 16) { set_error("unsupported N=%d: the 16 block keys are part of the KV", N); return DFLASH_ERR_UNSUPPORTED; }
  if (kv_format != DFLASH_KV_DENSE && kv_format != DFLASH_KV_TURBO3) { set_error("unsupported kv_format %d in dflash_verify_sdpa", kv_format); return DFLASH_ERR_UNSUPPORTED; }
  if (page_table && (page_tokens <= 0 || page_tokens % 128 != 0 || max_pages <= 0 || num_pages <= 0 ||
                     (long long)max_pages * page_tokens < N))
    return bad("paged KV needs page_tokens % 128 == 0, max_pages * page_tokens >= N and the pool's num_pages");
  if (kv_format == DFLASH_KV_DENSE && (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)))
    return bad("tensor base pointers must be 16-byte aligned");
  return DFLASH_OK;
}
}  // namespace dflash

using namespace dflash;

extern "C" {

int32_t dflash_gated_delta_tape(const void* q, const void* k, const void* v, const void* g,
                                const void* beta, const float* state_in, const void* mask,
                                const int32_t* n_per_seq, void* y, float* state_out, float* tape,
                                int32_t B, int32_t T, int32_t Hk, int32_t Hv, int32_t Dk, int32_t Dv,
                                int32_t g_is_vector, int32_t in_dtype, int32_t mask_dtype, void* stream) {
  if (!q || !k || !v || !g || !beta || !state_in || !y || !state_out) return bad("null tensor pointer");
  if (int32_t st = check_gdn_shape(B, T, Hk, Hv, Dk, Dv, in_dtype, mask_dtype, mask)) return st;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(state_in) || !aligned16(state_out) ||
      !aligned16(y) || (tape && !aligned16(tape)))
    return bad("tensor base pointers must be 16-byte aligned");
  GdnArgs a{q, k, v, g, beta, state_in, mask, n_per_seq, y, state_out, tape,
            B, T, Hk, Hv, Dk, Dv, g_is_vector ? 1 : 0, in_dtype, mask_dtype, false};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (gdn_tc_supported(a)) return launch_gdn_tc(a, s);
  if (gdn_fast_supported(a)) return launch_gdn_fast(a, s);
  return launch_gdn_generic(a, s);
}

int32_t dflash_tape_replay(const float* tape, const void* k, const void* g, const float* state_in,
                           const void* mask, const int32_t* n_per_seq, float* state_out, int32_t B,
                           int32_t T, int32_t Hk, int32_t Hv, int32_t Dk, int32_t Dv,
                           int32_t g_is_vector, int32_t kg_dtype, int32_t mask_dtype, void* stream) {
  if (!tape || !k || !g || !state_in || !state_out) return bad("null tensor pointer");
  if (int32_t st = check_gdn_shape(B, T, Hk, Hv, Dk, Dv, kg_dtype, mask_dtype, mask)) return st;
  if (!aligned16(tape) || !aligned16(k) || !aligned16(state_in) || !aligned16(state_out))
    return bad("tensor base pointers must be 16-byte aligned");
  GdnArgs a{nullptr, k, nullptr, g, nullptr, state_in, mask, n_per_seq, nullptr, state_out,
            const_cast<float*>(tape), B, T, Hk, Hv, Dk, Dv, g_is_vector ? 1 : 0, kg_dtype, mask_dtype, true};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (gdn_fast_supported(a)) return launch_gdn_fast(a, s);
  return launch_gdn_generic(a, s);
}

int32_t dflash_verify_sdpa(const void* q, const void* k, const void* v, const int32_t* page_table,
                           const int32_t* kv_len_per_seq, const void* mask, void* out, void* workspace,
                           size_t workspace_bytes, int32_t B, int32_t Hq, int32_t Hkv, int32_t T,
                           int32_t D, int32_t N, int32_t page_tokens, int32_t max_pages, int32_t num_pages,
                           float scale, int32_t dtype, int32_t kv_format, void* stream) {
  if (int32_t st = sdpa_check_args(q, k, v, page_table, out, B, Hq, Hkv, T, D, N, page_tokens, max_pages, num_pages, dtype, kv_format)) return st;
  if (kv_format == DFLASH_KV_TURBO3) {
    if (page_table) { set_error("TurboQuant KV behind a page table is not supported"); return DFLASH_ERR_UNSUPPORTED; }
    const dflash_turbo_kv* t = reinterpret_cast<const dflash_turbo_kv*>(k);
    if (t->n_cold < 0 || t->n_hot < 0 || t->n_cold + t->n_hot != N) return bad("TurboQuant KV: n_cold + n_hot must equal N");
    if (t->n_cold > 0 && (!t->k_packed || !t->k_signs || !t->k_norm || !t->k_rnorm || !t->v_packed || !t->v_norm)) return bad("null TurboQuant array");
    if (t->n_hot > 0 && (!t->k_hot || !t->v_hot || !aligned16(t->k_hot) || !aligned16(t->v_hot))) return bad("TurboQuant KV: hot window arrays missing or misaligned");
    if (!aligned16(q) || !aligned16(out)) return bad("tensor base pointers must be 16-byte aligned");
    if (turbo_fused_applies(t, kv_len_per_seq, mask, scale)) {
      // Fused: no key or value is decoded to global memory.  The query rows are rotated once (Q1 = R q, Q2 = Rq^T q), the
      // hot window is brought into the rotated domain, the attention kernel expands the packed indices and sign bits
      // into tensor-core operands tile by tile, and the output rows are rotated back.
      const size_t need = turbo_fused_workspace_bytes(B, Hq, Hkv, D, t->n_hot);
      if (!workspace || workspace_bytes < need) {
        set_error("verify_sdpa (TurboQuant KV): workspace of %zu bytes needed, %zu given", need, workspace_bytes);
        return DFLASH_ERR_WORKSPACE;
      }
      if (!aligned16(workspace)) return bad("tensor base pointers must be 16-byte aligned");
      if (!aligned16(t->k_packed) || !aligned16(t->k_signs) || !aligned16(t->k_norm) || !aligned16(t->k_rnorm) ||
          !aligned16(t->v_packed) || !aligned16(t->v_norm))
        return bad("TurboQuant arrays must be 16-byte aligned");
      uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
      const size_t q_bytes = align256((size_t)B * Hq * 16 * D * 2), hot_bytes = align256((size_t)B * Hkv * t->n_hot * D * 2);
      void *q1 = ws, *q2 = ws + q_bytes, *o_rot = ws + 2 * q_bytes, *k_rot = ws + 3 * q_bytes, *v_rot = ws + 3 * q_bytes + hot_bytes;
      uint8_t* scratch = ws + 3 * q_bytes + 2 * hot_bytes;
      cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
      if (int32_t st = launch_turbo_rotate_inputs(q, q1, q2, (long long)B * Hq * 16 * (D / 128), t->k_hot, k_rot, t->v_hot, v_rot,
                                                  (long long)B * Hkv * t->n_hot * (D / 128), dtype, s))
        return st;
      SdpaArgs a{q1, t->n_hot > 0 ? k_rot : nullptr, t->n_hot > 0 ? v_rot : nullptr, nullptr, nullptr, nullptr, o_rot, scratch,
                 workspace_bytes - (size_t)(scratch - ws), B, Hq, Hkv, D, N, 0, 0, 0, scale, dtype};
      TurboKvArgs ta{t->k_packed, t->k_signs, t->v_packed, t->k_norm, t->k_rnorm, t->v_norm, q2, t->n_cold, t->n_hot};
      if (int32_t st = launch_sdpa_tc_turbo(a, ta, s)) return st;
      return launch_turbo_unrotate_output(o_rot, out, (long long)B * Hq * 16 * (D / 128), dtype, s);
    }
    // otherwise (history not a multiple of 128 keys, ragged lengths, additive mask): expand K and V into the front of the
    // workspace, then attend over the expanded copy
    const size_t kv_elems = (size_t)B * Hkv * N * D, kv_bytes = (kv_elems * 2 + 255) / 256 * 256;
    const size_t need = 2 * kv_bytes + sdpa_workspace_bytes(B, Hq, Hkv, D, N);
    if (!workspace || workspace_bytes < need) {
      set_error("verify_sdpa (TurboQuant KV): workspace of %zu bytes needed, %zu given", need, workspace_bytes);
      return DFLASH_ERR_WORKSPACE;
    }
    if (!aligned16(workspace)) return bad("tensor base pointers must be 16-byte aligned");
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const long long pairs = (long long)B * Hkv, blocks_per_pair = (long long)t->n_cold * (D / 128);
    if (t->n_cold > 0) {   // cold history: every pair's run of blocks goes to the front of its N x D slab
      if (int32_t st = launch_turbo_decode(t->k_packed, t->k_signs, t->k_norm, t->k_rnorm, ws, pairs * blocks_per_pair, 1, dtype, s,
                                           blocks_per_pair, (long long)N * D)) return st;
      if (int32_t st = launch_turbo_decode(t->v_packed, nullptr, t->v_norm, nullptr, ws + kv_bytes, pairs * blocks_per_pair, 0, dtype, s,
                                           blocks_per_pair, (long long)N * D)) return st;
    }
    if (t->n_hot > 0) {    // hot window: copied behind the cold history
      const size_t row = (size_t)t->n_hot * D * 2, pitch = (size_t)N * D * 2, off = (size_t)t->n_cold * D * 2;
      DFLASH_CUDA_CHECK(cudaMemcpy2DAsync(ws + off, pitch, t->k_hot, row, row, (size_t)pairs, cudaMemcpyDeviceToDevice, s));
      DFLASH_CUDA_CHECK(cudaMemcpy2DAsync(ws + kv_bytes + off, pitch, t->v_hot, row, row, (size_t)pairs, cudaMemcpyDeviceToDevice, s));
    }
    return dflash_verify_sdpa(q, ws, ws + kv_bytes, nullptr, kv_len_per_seq, mask, out, ws + 2 * kv_bytes, workspace_bytes - 2 * kv_bytes,
                              B, Hq, Hkv, T, D, N, 0, 0, 0, scale, dtype, DFLASH_KV_DENSE, stream);
  }
  if (workspace && !aligned16(workspace)) return bad("tensor base pointers must be 16-byte aligned");
  SdpaArgs a{q, k, v, page_table, kv_len_per_seq, mask, out, workspace, workspace_bytes,
             B, Hq, Hkv, D, N, page_tokens, max_pages, page_table ? num_pages : 0, scale, dtype};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (sdpa_tc_supported(a)) return launch_sdpa_tc(a, s);
  return launch_sdpa_simple(a, s);
}

size_t dflash_verify_sdpa_workspace_bytes(int32_t B, int32_t Hq, int32_t Hkv, int32_t D, int32_t N) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || N <= 0) return 0;
  return sdpa_workspace_bytes(B, Hq, Hkv, D, N);
}

size_t dflash_verify_sdpa_workspace_bytes_ex(int32_t B, int32_t Hq, int32_t Hkv, int32_t D, int32_t N, int32_t kv_format) {
  const size_t base = dflash_verify_sdpa_workspace_bytes(B, Hq, Hkv, D, N);
  if (!base || kv_format != DFLASH_KV_TURBO3) return base;
  // enough for either route whatever the split into cold and hot keys: the expanded copy (2 x N keys) or the fused
  // route's rotated queries and hot window (at most N keys)
  const size_t kv_bytes = align256((size_t)B * Hkv * N * D * 2);
  const size_t fused = turbo_fused_workspace_bytes(B, Hq, Hkv, D, N);
  const size_t expand = base + 2 * kv_bytes;
  return fused > expand ? fused : expand;
}

size_t dflash_verify_sdpa_turbo_workspace_bytes(int32_t B, int32_t Hq, int32_t Hkv, int32_t D, int32_t n_cold, int32_t n_hot) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || n_cold < 0 || n_hot < 0 || n_cold + n_hot <= 0) return 0;
  dflash_turbo_kv t{};
  t.n_cold = n_cold;
  t.n_hot = n_hot;
  if (turbo_fused_applies(&t, nullptr, nullptr, 1.f)) return turbo_fused_workspace_bytes(B, Hq, Hkv, D, n_hot);
  return dflash_verify_sdpa_workspace_bytes_ex(B, Hq, Hkv, D, n_cold + n_hot, DFLASH_KV_TURBO3);
}

int32_t dflash_greedy_tokens(const void* logits, const uint8_t* suppress, uint32_t* posterior,
                             int32_t rows, int32_t V, int32_t logits_dtype, void* stream) {
  if (!logits || !posterior) return bad("null tensor pointer");
  if (rows <= 0 || V <= 0) return bad("non-positive dimension");
  return launch_greedy_tokens(logits, suppress, posterior, rows, V, logits_dtype,
                              reinterpret_cast<cudaStream_t>(stream));
}

int32_t dflash_accept_lengths(const uint32_t* posterior, const int32_t* verify_ids, int32_t* accept,
                              int32_t* next_token, int32_t* replay_len, int32_t B, int32_t T,
                              void* stream) {
  if (!posterior || !verify_ids || !accept) return bad("null tensor pointer");
  if (B <= 0 || T <= 0) return bad("non-positive dimension");
  return launch_accept_lengths(posterior, verify_ids, accept, next_token, replay_len, B, T,
                               reinterpret_cast<cudaStream_t>(stream));
}

int32_t dflash_gather_logits_rows(const void* logits, const int32_t* row_per_seq, void* out, int32_t B, int32_t T,
                                  int32_t V, int32_t logits_dtype, void* stream) {
  if (!logits || !row_per_seq || !out) return bad("null tensor pointer");
  if (B <= 0 || T <= 0 || V <= 0) return bad("non-positive dimension");
  if (logits_dtype != DFLASH_F32 && logits_dtype != DFLASH_BF16 && logits_dtype != DFLASH_F16) {
    set_error("gather_logits_rows: unsupported logits dtype %d", logits_dtype);
    return DFLASH_ERR_UNSUPPORTED;
  }
  const long long row_bytes = (long long)V * (long long)dtype_size(logits_dtype);
  if (row_bytes % 16 == 0 && (!aligned16(logits) || !aligned16(out))) return bad("tensor base pointers must be 16-byte aligned");
  return launch_gather_rows(logits, row_per_seq, out, B, T, row_bytes, reinterpret_cast<cudaStream_t>(stream));
}

int32_t dflash_turbo_encode(const void* x, uint8_t* packed, uint8_t* signs, uint16_t* norm, uint16_t* rnorm,
                            int64_t n_blocks, int32_t is_key, int32_t in_dtype, void* stream) {
  if (!x || !packed || !norm || (is_key && (!signs || !rnorm))) return bad("null tensor pointer");
  if (n_blocks <= 0) return bad("non-positive dimension");
  return launch_turbo_encode(x, packed, signs, norm, rnorm, n_blocks, is_key ? 1 : 0, in_dtype,
                             reinterpret_cast<cudaStream_t>(stream));
}

int32_t dflash_turbo_decode(const uint8_t* packed, const uint8_t* signs, const uint16_t* norm,
                            const uint16_t* rnorm, void* out, int64_t n_blocks, int32_t is_key,
                            int32_t out_dtype, void* stream) {
  if (!packed || !norm || !out || (is_key && (!signs || !rnorm))) return bad("null tensor pointer");
  if (n_blocks <= 0) return bad("non-positive dimension");
  return launch_turbo_decode(packed, signs, norm, rnorm, out, n_blocks, is_key ? 1 : 0, out_dtype,
                             reinterpret_cast<cudaStream_t>(stream));
}

int32_t dflash_partition_plan(int32_t units, int32_t n_gpus, int32_t* begin_end_host) {
  if (units < 0 || n_gpus <= 0 || !begin_end_host) return bad("partition_plan arguments");
  const int base = units / n_gpus, extra = units % n_gpus;
  int pos = 0;
  for (int r = 0; r < n_gpus; ++r) {
    const int len = base + (r < extra ? 1 : 0);
    begin_end_host[2 * r] = pos;
    begin_end_host[2 * r + 1] = pos + len;
    pos += len;
  }
  return DFLASH_OK;
}

int32_t dflash_device_status(void* stream) {
  int* word = device_status_word();
  if (!word) { set_error("no CUDA device"); return DFLASH_ERR_CUDA; }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int host = 0;
  DFLASH_CUDA_CHECK(cudaMemcpyAsync(&host, word, sizeof(int), cudaMemcpyDeviceToHost, s));
  DFLASH_CUDA_CHECK(cudaStreamSynchronize(s));
  if (host != 0) {
    DFLASH_CUDA_CHECK(cudaMemsetAsync(word, 0, sizeof(int), s));
    DFLASH_CUDA_CHECK(cudaStreamSynchronize(s));
    switch (host) {
      case kStatusKvRange:
        set_error("a KV position beyond the cache's capacity, or a page id outside the pool: kv_append skipped the row / "
                  "verify_sdpa read the page as zeros");
        return DFLASH_ERR_DEVICE_DATA;
      case kStatusKvLen:
        set_error("verify_sdpa: a kv_len_per_seq entry outside [16, N] was clamped; that sequence's output is not the attention "
                  "over its keys (no output at all for a length <= 0)");
        return DFLASH_ERR_DEVICE_DATA;
      case kStatusMergeRanges:
        set_error("verify_sdpa: a unit was cut into more key ranges than the merge kernel takes; its output is incomplete");
        return DFLASH_ERR_DEVICE_DATA;
      case kStatusSmemAlign:
        set_error("a kernel found its shared-memory window misaligned and did not run");
        return DFLASH_ERR_CUDA;
      default:
        set_error("a device-side bounded wait gave up (code %d)", host);
        return DFLASH_ERR_DEVICE_TIMEOUT;
    }
  }
  return DFLASH_OK;
}

int32_t dflash_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
  return n;
}

const char* dflash_last_error_string(void) { return g_error; }
uint64_t dflash_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
const char* dflash_version(void) { return "dflash-cuda 0.1 (sm_100a)"; }

}  // extern "C"
