// Acceptance bookkeeping on the device: greedy posterior tokens and accepted length.
//
// greedy_tokens follows DFlashRuntime.greedyTokensWithMask
// (Sources/DFlash/DFlashRuntime.swift:118-128): suppressed ids are forced to -1e9 in the
// logits' dtype, then argmax over the vocabulary, ties to the lowest index.
// accept_lengths follows matchAcceptanceLength (:133-142) and the commit arithmetic (:523-547).
// Both are pure streaming / integer work: one block per logits row with 16-byte loads.
#include "common.cuh"

namespace dflash {
namespace {

constexpr int kThreads = 512;

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int n = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int n = 8; };
template <> struct Vec<__half> { static constexpr int n = 8; };

__device__ __forceinline__ void take(float x, int i, float& best, int& arg) {
  // strict > keeps the lowest index among equals when candidates arrive in index order;
  // across threads the index tie-break is explicit.
  if (x > best || (x == best && i < arg)) { best = x; arg = i; }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) greedy_kernel(const T* __restrict__ logits,
                                                          const uint8_t* __restrict__ suppress,
                                                          uint32_t* __restrict__ posterior, int V) {
  const T* row = logits + (long long)blockIdx.x * V;
  const float floor_v = to_f32(from_f32<T>(-1e9f));
  float best = -INFINITY;
  int arg = 0x7fffffff;
  constexpr int VN = Vec<T>::n;
  const bool aligned = ((reinterpret_cast<uintptr_t>(row) & 15) == 0);
  const int vec_end = aligned ? (V / VN) * VN : 0;
  for (int i = threadIdx.x * VN; i < vec_end; i += kThreads * VN) {
    const uint4 raw = *reinterpret_cast<const uint4*>(row + i);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < VN; ++j) {
      float x = to_f32(e[j]);
      if (suppress && suppress[i + j]) x = floor_v;
      take(x, i + j, best, arg);
    }
  }
  for (int i = vec_end + threadIdx.x; i < V; i += kThreads) {
    float x = to_f32(row[i]);
    if (suppress && suppress[i]) x = floor_v;
    take(x, i, best, arg);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
    take(ob, oa, best, arg);
  }
  __shared__ float sb[kThreads / 32];
  __shared__ int sa[kThreads / 32];
  if ((threadIdx.x & 31) == 0) { sb[threadIdx.x >> 5] = best; sa[threadIdx.x >> 5] = arg; }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = threadIdx.x < kThreads / 32 ? sb[threadIdx.x] : -INFINITY;
    arg = threadIdx.x < kThreads / 32 ? sa[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      take(ob, oa, best, arg);
    }
    if (threadIdx.x == 0) posterior[blockIdx.x] = arg == 0x7fffffff ? 0u : (uint32_t)arg;
  }
}

__global__ void accept_kernel(const uint32_t* __restrict__ posterior, const int32_t* __restrict__ verify_ids,
                              int32_t* accept, int32_t* next_token, int32_t* replay_len, int B, int T) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const uint32_t* p = posterior + (long long)b * T;
  const int32_t* ids = verify_ids + (long long)b * T;
  int acc = 0;
  while (acc + 1 < T && (uint32_t)ids[acc + 1] == p[acc]) ++acc;
  accept[b] = acc;
  if (next_token) next_token[b] = (int32_t)p[acc];
  if (replay_len) replay_len[b] = acc + 1;
}

// out[b, :] = logits[b, clamp(row[b], 0, T-1), :] as raw bytes (16-byte copies where the row allows it): the
// logits row that produced a sequence's next token, picked with the accepted count still on the device.
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint8_t* __restrict__ logits, const int32_t* __restrict__ row,
                                                          uint8_t* __restrict__ out, int T, long long row_bytes) {
  const int b = blockIdx.y;
  int r = row[b];
  r = r < 0 ? 0 : (r >= T ? T - 1 : r);
  const uint8_t* src = logits + ((long long)b * T + r) * row_bytes;
  uint8_t* dst = out + (long long)b * row_bytes;
  const long long i0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 16, stride = (long long)gridDim.x * blockDim.x * 16;
  if (row_bytes % 16 == 0) {
    for (long long i = i0; i < row_bytes; i += stride) *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
  } else {
    for (long long i = i0; i < row_bytes; i += stride)
      for (int j = 0; j < 16 && i + j < row_bytes; ++j) dst[i + j] = src[i + j];
  }
}

}  // namespace

int32_t launch_gather_rows(const void* logits, const int32_t* row, void* out, int B, int T, long long row_bytes, cudaStream_t stream) {
  const int chunks = (int)((row_bytes / 16 + 255) / 256);
  gather_rows_kernel<<<dim3(chunks < 1 ? 1 : (chunks > 64 ? 64 : chunks), B), 256, 0, stream>>>(
      reinterpret_cast<const uint8_t*>(logits), row, reinterpret_cast<uint8_t*>(out), T, row_bytes);
  DFLASH_LAUNCH_CHECK();
  count_launch();
  return DFLASH_OK;
}

int32_t launch_greedy_tokens(const void* logits, const uint8_t* suppress, uint32_t* posterior, int rows,
                             int V, int logits_dtype, cudaStream_t stream) {
  switch (logits_dtype) {
    case DFLASH_F32:
      greedy_kernel<float><<<rows, kThreads, 0, stream>>>((const float*)logits, suppress, posterior, V);
      break;
    case DFLASH_BF16:
      greedy_kernel<__nv_bfloat16><<<rows, kThreads, 0, stream>>>((const __nv_bfloat16*)logits, suppress, posterior, V);
      break;
    case DFLASH_F16:
      greedy_kernel<__half><<<rows, kThreads, 0, stream>>>((const __half*)logits, suppress, posterior, V);
      break;
    default:
      set_error("greedy_tokens: unsupported logits dtype %d", logits_dtype);
      return DFLASH_ERR_UNSUPPORTED;
  }
  DFLASH_LAUNCH_CHECK();
  count_launch();
  return DFLASH_OK;
}

int32_t launch_accept_lengths(const uint32_t* posterior, const int32_t* verify_ids, int32_t* accept,
                              int32_t* next_token, int32_t* replay_len, int B, int T, cudaStream_t stream) {
  accept_kernel<<<(B + 127) / 128, 128, 0, stream>>>(posterior, verify_ids, accept, next_token, replay_len, B, T);
  DFLASH_LAUNCH_CHECK();
  count_launch();
  return DFLASH_OK;
}

}  // namespace dflash
