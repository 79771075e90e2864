// Shared declarations of the DFlash CUDA library (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dflash_cuda.h"

namespace dflash {

// ---- error plumbing (abi.cu owns the storage) --------------------------------------------
void set_error(const char* fmt, ...);
void count_launch(int n = 1);
// Address of the per-device status word (a __device__ int); nullptr on failure.
int* device_status_word();
int sm_count();

// Codes a kernel leaves in the per-device status word; dflash_device_status maps them to a
// dflash_status in one place (abi.cu).  Codes below 16 are bounded waits that gave up
// (DFLASH_ERR_DEVICE_TIMEOUT) except where noted; 16 and above are device-resident data out of
// range (DFLASH_ERR_DEVICE_DATA).
enum DeviceStatusCode : int {
  kStatusGdnWait = 1,        // gated-delta kernels: an mbarrier wait gave up
  kStatusMbarWait = 2,       // attention: an mbarrier wait gave up
  kStatusExchangeWait = 3,   // attention: the two half-row softmax threads never met
  kStatusSmemAlign = 4,      // dynamic shared memory window not 1024-byte aligned (never seen)
  kStatusGroupWait = 5,      // attention: meeting point of the softmax warps
  kStatusPeerWait = 6,       // attention: the cluster partner never arrived
  kStatusMergeRanges = 7,    // merge kernel: a unit was cut into more key ranges than it takes (data, not a wait)
  kStatusSelftestWait = 8,   // dflash_selftest_bounded_wait: the wait that nothing satisfies gave up (as it must)
  kStatusKvRange = 16,       // a KV position beyond the capacity, or a page id outside the pool
  kStatusKvLen = 17,         // attention: a kv_len_per_seq entry outside [16, N] (clamped)
};

#define DFLASH_CUDA_CHECK(expr)                                                          \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess) {                                                             \
      ::dflash::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return DFLASH_ERR_CUDA;                                                            \
    }                                                                                    \
  } while (0)

#define DFLASH_LAUNCH_CHECK()                                                            \
  do {                                                                                   \
    cudaError_t _e = cudaGetLastError();                                                 \
    if (_e != cudaSuccess) {                                                             \
      ::dflash::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e), __FILE__, __LINE__); \
      return DFLASH_ERR_CUDA;                                                            \
    }                                                                                    \
  } while (0)

// ---- element access ----------------------------------------------------------------------
__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_f32(uint8_t x) { return (float)x; }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

// mask[b*T+t] > 0.5 for a mask of runtime dtype
__device__ __forceinline__ bool mask_on(const void* mask, int mask_dtype, int idx) {
  switch (mask_dtype) {
    case DFLASH_F32: return reinterpret_cast<const float*>(mask)[idx] > 0.5f;
    case DFLASH_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(mask)[idx]) > 0.5f;
    case DFLASH_F16: return __half2float(reinterpret_cast<const __half*>(mask)[idx]) > 0.5f;
    default: return reinterpret_cast<const uint8_t*>(mask)[idx] != 0;
  }
}

// Bit t set <=> step t of sequence b runs.  T <= 64.
__device__ __forceinline__ unsigned long long step_bits(const void* mask, int mask_dtype,
                                                        const int32_t* n_per_seq, int b, int T, int n_div = 1) {
  unsigned long long bits = T >= 64 ? ~0ull : ((1ull << T) - 1ull);
  if (n_per_seq) {
    int n = n_per_seq[(unsigned)b / (unsigned)n_div];
    n = n < 0 ? 0 : (n > T ? T : n);
    bits &= n >= 64 ? ~0ull : ((1ull << n) - 1ull);
  }
  if (mask) {
    unsigned long long m = 0;
    for (int t = 0; t < T; ++t) m |= (unsigned long long)mask_on(mask, mask_dtype, b * T + t) << t;
    bits &= m;
  }
  return bits;
}

inline size_t dtype_size(int dt) { return dt == DFLASH_F32 ? 4 : (dt == DFLASH_U8 ? 1 : 2); }

// ---- kernel families (defined in their own translation units) -----------------------------
struct GdnArgs {
  const void *q, *k, *v, *g, *beta;
  const float* state_in;
  const void* mask;
  const int32_t* n_per_seq;
  void* y;
  float* state_out;
  float* tape;        // forward: output (may be null); replay: input
  int B, T, Hk, Hv, Dk, Dv;
  int g_is_vector, in_dtype, mask_dtype;
  bool replay;        // true: S <- S g + tape (x) k ; false: full forward
  int n_div = 1;      // item b reads n_per_seq[b / n_div]: n_div stacked layers of a sequence share its length
};

int32_t launch_gdn_generic(const GdnArgs& a, cudaStream_t stream);
// Dk == Dv == 128, scalar gate, T <= 16: TMA-pipelined persistent kernel.
bool gdn_fast_supported(const GdnArgs& a);
int32_t launch_gdn_fast(const GdnArgs& a, cudaStream_t stream);
// Forward only, bf16 inputs, Dk == Dv == 128, scalar gate, T <= 16: the block's 16 steps as
// three tensor-core products plus a per-row triangular recurrence.
bool gdn_tc_supported(const GdnArgs& a);
int32_t launch_gdn_tc(const GdnArgs& a, cudaStream_t stream);

struct SdpaArgs {
  const void *q, *k, *v;
  const int32_t* page_table;
  const int32_t* kv_len;
  const void* mask;
  void* out;
  void* workspace;
  size_t workspace_bytes;
  int B, Hq, Hkv, D, N, page_tokens, max_pages, num_pages;
  float scale;
  int dtype;
};

// KV in the TurboQuant 3-bit format for the fused attention (sdpa_tc.cu, TURBO instantiation)
struct TurboKvArgs {
  const uint8_t *kp, *ks, *vp;        // packed indices / sign bits of the cold history
  const uint16_t *kn, *kr, *vn;       // fp16 bits of the norms
  const void* q2;                     // Rq^T q, laid out as q
  int n_cold, n_hot;
};
bool sdpa_tc_turbo_available();   // the fused compressed-KV kernel's register pool matches this build
int32_t launch_sdpa_tc_turbo(const SdpaArgs& a, const TurboKvArgs& t, cudaStream_t stream);
size_t sdpa_tc_scratch_bytes(int D);
int32_t launch_turbo_rotate_inputs(const void* q, void* q1, void* q2, long long q_blocks, const void* k_hot, void* k_rot,
                                   const void* v_hot, void* v_rot, long long hot_blocks, int dtype, cudaStream_t stream);
int32_t launch_turbo_unrotate_output(const void* o_rot, void* out, long long blocks, int dtype, cudaStream_t stream);

size_t sdpa_workspace_bytes(int B, int Hq, int Hkv, int D, int N);
// Scratch of the kernel a call will actually run on, given a workspace at least this large.
size_t sdpa_scratch_bytes_for_call(int B, int Hq, int D, float scale, bool ragged);
int32_t sdpa_check_args(const void* q, const void* k, const void* v, const int32_t* page_table, const void* out,
                        int32_t B, int32_t Hq, int32_t Hkv, int32_t T, int32_t D, int32_t N, int32_t page_tokens,
                        int32_t max_pages, int32_t num_pages, int32_t dtype, int32_t kv_format);
int32_t launch_sdpa_simple(const SdpaArgs& a, cudaStream_t stream);
bool sdpa_tc_supported(const SdpaArgs& a);
int32_t launch_sdpa_tc(const SdpaArgs& a, cudaStream_t stream);

int32_t launch_greedy_tokens(const void* logits, const uint8_t* suppress, uint32_t* posterior,
                             int rows, int V, int logits_dtype, cudaStream_t stream);
int32_t launch_accept_lengths(const uint32_t* posterior, const int32_t* verify_ids, int32_t* accept,
                              int32_t* next_token, int32_t* replay_len, int B, int T,
                              cudaStream_t stream);

int32_t launch_gather_rows(const void* logits, const int32_t* row, void* out, int B, int T, long long row_bytes,
                           cudaStream_t stream);

// steps_div: row b reads steps_per_seq[b / steps_div] (stacked layers of a sequence share its step count)
int32_t launch_conv_window(const void* conv_snapshot, const void* qkv, const int32_t* steps_per_seq, int steps_all, void* out,
                           int B, int T, int keep, long long row_bytes, int32_t* rows_out, int steps_div, cudaStream_t stream);

int32_t launch_turbo_encode(const void* x, uint8_t* packed, uint8_t* signs, uint16_t* norm, uint16_t* rnorm,
                            long long n, int is_key, int in_dtype, cudaStream_t stream);
// group_blocks > 0: output block v goes to out + (v / group_blocks) * group_stride + (v % group_blocks) * 128 elements
int32_t launch_turbo_decode(const uint8_t* packed, const uint8_t* signs, const uint16_t* norm, const uint16_t* rnorm,
                            void* out, long long n, int is_key, int out_dtype, cudaStream_t stream,
                            long long group_blocks = 0, long long group_stride = 0);

}  // namespace dflash
