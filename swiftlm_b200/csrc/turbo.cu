// TurboQuant 3-bit KV codec on the GPU, 128-dimension blocks.
//
// Follows the codec as the reference states it in tests/test_turbo_quant.cpp of the SwiftLM
// tree: L2 normalisation, sign-flip / Walsh-Hadamard rotation (:14-17), nearest of 8 centroids
// by boundary search (:18), little-endian 3-bit packing (:19-20), fp16 norms by truncation
// (:21-22); V stores fp16(norm / centroid-vector norm) (:69-74); K additionally stores the sign
// bits of the QJL-rotated residual and its fp16 norm and decodes as
// (centroids rotated back + QJL_C/128 * rnorm * qrot(signs)) * norm (:85-98).
// A head vector of 256 dimensions is two independent 128-blocks.
//
// The codec is integer/byte work whose results must match the reference bit for bit, so every
// floating-point operation is performed in the reference's order with explicitly rounded
// adds and multiplies (no fused multiply-add).  One thread owns one 128-block and keeps it in
// registers, in the encoder and in the decoder; an encoder that walks the block sequentially in
// shared memory (element i of thread t at [i][t]) serves arrays that are not 16-byte aligned.
#include "common.cuh"
#include "turbo_tables.cuh"

namespace dflash {
namespace {

constexpr int kBlock = 128;
constexpr int kThreadsPerCta = 64;

__device__ __forceinline__ float sgn(const unsigned int* neg, int i) { return (neg[i >> 5] >> (i & 31)) & 1u ? -1.f : 1.f; }

struct Vec {   // a 128-vector in shared memory, strided by the CTA width
  float* p;
  __device__ __forceinline__ float& operator[](int i) const { return p[i * kThreadsPerCta]; }
};

__device__ void fwht128(const Vec& x) {   // :14
  for (int h = 1; h < kBlock; h *= 2)
    for (int i = 0; i < kBlock; i += 2 * h)
      for (int j = i; j < i + h; ++j) {
        const float a = x[j], b = x[j + h];
        x[j] = __fadd_rn(a, b);
        x[j + h] = __fsub_rn(a, b);
      }
  for (int i = 0; i < kBlock; ++i) x[i] = __fmul_rn(x[i], 0.08838834764831845f);
}
__device__ void rot(const Vec& x, const unsigned int* first, const unsigned int* second) {   // :15-17
  for (int i = 0; i < kBlock; ++i) x[i] = __fmul_rn(x[i], sgn(first, i));
  fwht128(x);
  for (int i = 0; i < kBlock; ++i) x[i] = __fmul_rn(x[i], sgn(second, i));
}
__device__ __forceinline__ int nearest3(float v) {   // :18
  int idx = 0;
#pragma unroll
  for (int i = 0; i < 7; ++i) idx += !(v < TURBO_B3[i]);
  return idx;
}
__device__ __forceinline__ uint16_t to_f16_trunc(float f) {   // :21
  const uint32_t u = __float_as_uint(f);
  const uint16_t s = (uint16_t)((u >> 16) & 0x8000u);
  const int32_t e = (int32_t)((u >> 23) & 0xFF) - 127 + 15;
  const uint32_t m = u & 0x7FFFFFu;
  if (e <= 0) return s;
  if (e >= 31) return (uint16_t)(s | 0x7C00u);
  return (uint16_t)(s | (uint16_t)(e << 10) | (uint16_t)(m >> 13));
}
__device__ __forceinline__ float from_f16_bits(uint16_t h) {   // :22
  const uint32_t s = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
  uint32_t u;
  if (!e) u = s;
  else if (e == 31) u = s | (0xFFu << 23) | m;
  else u = s | ((e + 127 - 15) << 23) | (m << 13);
  return __uint_as_float(u);
}

template <typename InT>
__global__ void __launch_bounds__(kThreadsPerCta)
turbo_encode_kernel(const InT* __restrict__ x, uint8_t* __restrict__ packed, uint8_t* __restrict__ signs,
                    uint16_t* __restrict__ norm, uint16_t* __restrict__ rnorm, long long n, int is_key) {
  extern __shared__ float sh[];
  const long long v = (long long)blockIdx.x * kThreadsPerCta + threadIdx.x;
  if (v >= n) return;
  const Vec nrm{sh + threadIdx.x};                                        // normalised input
  const Vec rotv{sh + kBlock * kThreadsPerCta + threadIdx.x};             // work vector
  const InT* src = x + v * kBlock;
  float ns = 0.f;
  for (int i = 0; i < kBlock; ++i) {
    const float f = to_f32(src[i]);
    rotv[i] = f;
    ns = __fadd_rn(ns, __fmul_rn(f, f));
  }
  const float gn = __fsqrt_rn(ns), inv = gn > 1e-10f ? __fdiv_rn(1.f, gn) : 0.f;
  for (int i = 0; i < kBlock; ++i) {
    const float f = __fmul_rn(rotv[i], inv);
    nrm[i] = f;
    rotv[i] = f;
  }
  rot(rotv, TURBO_S1_NEG, TURBO_S2_NEG);
  // 3-bit indices: pack as a little-endian bit stream (:19), 8 indices -> 3 bytes
  uint8_t* pk = packed + v * 48;
  float rs = 0.f;
  for (int g8 = 0; g8 < 16; ++g8) {
    uint32_t bits = 0;
    for (int e = 0; e < 8; ++e) {
      const int idx = nearest3(rotv[g8 * 8 + e]);
      bits |= (uint32_t)idx << (3 * e);
      rs = __fadd_rn(rs, __fmul_rn(TURBO_C3[idx], TURBO_C3[idx]));
      rotv[g8 * 8 + e] = TURBO_C3[idx];                                   // centroid vector, for the K residual
    }
    pk[3 * g8] = (uint8_t)bits;
    pk[3 * g8 + 1] = (uint8_t)(bits >> 8);
    pk[3 * g8 + 2] = (uint8_t)(bits >> 16);
  }
  if (!is_key) {
    const float rn2 = __fsqrt_rn(rs);
    norm[v] = to_f16_trunc(rn2 > 1e-10f ? __fdiv_rn(gn, rn2) : gn);        // :73
    return;
  }
  rot(rotv, TURBO_S2_NEG, TURBO_S1_NEG);                                   // inverse rotation of the centroids (:91)
  float rns = 0.f;
  for (int i = 0; i < kBlock; ++i) {
    const float r = __fsub_rn(nrm[i], rotv[i]);
    rotv[i] = r;
    rns = __fadd_rn(rns, __fmul_rn(r, r));
  }
  rot(rotv, TURBO_Q1_NEG, TURBO_Q2_NEG);                                   // :93
  uint8_t* sg = signs + v * 16;
  for (int byte = 0; byte < 16; ++byte) {
    uint32_t m = 0;
    for (int e = 0; e < 8; ++e) m |= (rotv[byte * 8 + e] >= 0.f ? 1u : 0u) << e;
    sg[byte] = (uint8_t)m;
  }
  norm[v] = to_f16_trunc(gn);
  rnorm[v] = to_f16_trunc(__fsqrt_rn(rns));
}

// ---- decode: one thread per 128-block, the block lives in registers ----------------------------
// The Walsh-Hadamard butterflies of one stage are independent of each other, so running them from
// registers in any order gives the same bits as the reference's loops; the stages keep their order.
constexpr int kDecThreads = 64;

__device__ __forceinline__ float flip(float x, unsigned int neg_word, int bit) {   // x * (+-1), exactly
  return __uint_as_float(__float_as_uint(x) ^ (((neg_word >> bit) & 1u) << 31));
}
template <int H> __device__ __forceinline__ void wht_stage(float (&x)[kBlock]) {
#pragma unroll
  for (int p = 0; p < kBlock / 2; ++p) {
    const int j = (p / H) * 2 * H + (p % H);   // the p-th butterfly of the stage
    const float a = x[j], b = x[j + H];
    x[j] = __fadd_rn(a, b);
    x[j + H] = __fsub_rn(a, b);
  }
}
__device__ __forceinline__ void rot_regs(float (&x)[kBlock], const unsigned int* first, const unsigned int* second) {
  unsigned int f[4], s[4];
#pragma unroll
  for (int w = 0; w < 4; ++w) { f[w] = first[w]; s[w] = second[w]; }
#pragma unroll
  for (int i = 0; i < kBlock; ++i) x[i] = flip(x[i], f[i >> 5], i & 31);
  wht_stage<1>(x); wht_stage<2>(x); wht_stage<4>(x); wht_stage<8>(x); wht_stage<16>(x); wht_stage<32>(x); wht_stage<64>(x);
#pragma unroll
  for (int i = 0; i < kBlock; ++i) x[i] = flip(__fmul_rn(x[i], 0.08838834764831845f), s[i >> 5], i & 31);
}

template <typename OutT> __device__ __forceinline__ void store8_out(OutT* dst, const float (&v)[8]);
template <> __device__ __forceinline__ void store8_out<float>(float* dst, const float (&v)[8]) {
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8_out<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[8]) {
  __nv_bfloat162 p[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(p);
}
template <> __device__ __forceinline__ void store8_out<__half>(__half* dst, const float (&v)[8]) {
  __half2 p[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(p);
}

template <typename OutT, bool IS_KEY>
__global__ void __launch_bounds__(kDecThreads)
turbo_decode_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ signs,
                    const uint16_t* __restrict__ norm, const uint16_t* __restrict__ rnorm, OutT* __restrict__ out,
                    long long n, long long group_blocks, long long group_stride) {
  // output block v lands at out + (v / group_blocks) * group_stride + (v % group_blocks) * 128 elements
  extern __shared__ float sh[];                      // [8][kDecThreads] centroid table, then (keys) [128][kDecThreads]
  float* c3 = sh;                                    // one copy of the 8 centroids per thread column: no bank conflicts
  for (int i = threadIdx.x; i < 8 * kDecThreads; i += kDecThreads) c3[i] = TURBO_C3[i / kDecThreads];
  __syncthreads();
  long long v = (long long)blockIdx.x * kDecThreads + threadIdx.x;
  if (v >= n) v = n - 1;                               // the tail threads redo the last block; their copy is not written out
  float* stash = sh + 8 * kDecThreads + threadIdx.x;   // element i at stash[i * kDecThreads]
  float x[kBlock];
  if (IS_KEY) {
    // residual term first: qrot(signs) * (QJL_C / 128 * rnorm), parked in shared memory (:96-98)
    const uint4 sg = *reinterpret_cast<const uint4*>(signs + v * 16);
    const unsigned int sw[4] = {sg.x, sg.y, sg.z, sg.w};
#pragma unroll
    for (int i = 0; i < kBlock; ++i) x[i] = (sw[i >> 5] >> (i & 31)) & 1u ? 1.f : -1.f;
    rot_regs(x, TURBO_Q1_NEG, TURBO_Q2_NEG);
    const float qs = __fmul_rn(__fdiv_rn(TURBO_QJL_C, 128.f), from_f16_bits(rnorm[v]));
#pragma unroll
    for (int i = 0; i < kBlock; ++i) stash[i * kDecThreads] = __fmul_rn(x[i], qs);
  }
  {
    const uint4* pk = reinterpret_cast<const uint4*>(packed + v * 48);
    const uint4 p0 = pk[0], p1 = pk[1], p2 = pk[2];
    const unsigned int w[13] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w, p2.x, p2.y, p2.z, p2.w, 0u};
#pragma unroll
    for (int i = 0; i < kBlock; ++i) {
      const int bit = 3 * i, word = bit >> 5, off = bit & 31;
      unsigned int idx = w[word] >> off;
      if (off > 29) idx |= w[word + 1] << (32 - off);
      x[i] = c3[(idx & 7u) * kDecThreads + threadIdx.x];
    }
  }
  rot_regs(x, TURBO_S2_NEG, TURBO_S1_NEG);
  const float sc = from_f16_bits(norm[v]);
  // Outputs leave through a staging area so that a warp writes whole lines: thread t parks its block at
  // t * (block bytes + 16) (the pad keeps the 16-byte pieces of neighbouring threads on different banks).
  constexpr int kRowBytes = kBlock * (int)sizeof(OutT) + 16;
  uint8_t* stage = reinterpret_cast<uint8_t*>(sh + (8 + (IS_KEY ? kBlock : 0)) * kDecThreads);
#pragma unroll
  for (int g8 = 0; g8 < kBlock / 8; ++g8) {
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int i = g8 * 8 + e;
      o[e] = IS_KEY ? __fmul_rn(__fadd_rn(x[i], stash[i * kDecThreads]), sc) : __fmul_rn(x[i], sc);
    }
    store8_out<OutT>(reinterpret_cast<OutT*>(stage + threadIdx.x * kRowBytes) + g8 * 8, o);
  }
  __syncthreads();
  constexpr int kPieces = kBlock * (int)sizeof(OutT) / 16;            // 16-byte pieces per block
  const long long first = (long long)blockIdx.x * kDecThreads;        // first block of this CTA
  const long long here = n - first < kDecThreads ? n - first : kDecThreads;
  for (int p = threadIdx.x; p < (int)here * kPieces; p += kDecThreads) {
    const int t = p / kPieces, off = p % kPieces;
    const long long blk = first + t;
    uint8_t* g = reinterpret_cast<uint8_t*>(out + (blk / group_blocks) * group_stride + (blk % group_blocks) * kBlock);
    *reinterpret_cast<uint4*>(g + off * 16) = *reinterpret_cast<const uint4*>(stage + t * kRowBytes + off * 16);
  }
}

template <typename OutT>
int32_t launch_decode_typed(const uint8_t* packed, const uint8_t* signs, const uint16_t* norm, const uint16_t* rnorm, void* out,
                            long long n, int is_key, long long group_blocks, long long group_stride, cudaStream_t stream) {
  const unsigned grid = (unsigned)((n + kDecThreads - 1) / kDecThreads);
  const size_t smem = (8 + (is_key ? kBlock : 0)) * kDecThreads * sizeof(float) + kDecThreads * (kBlock * sizeof(OutT) + 16);
  DFLASH_CUDA_CHECK(cudaFuncSetAttribute(turbo_decode_kernel<OutT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  if (is_key) {
    DFLASH_CUDA_CHECK(cudaFuncSetAttribute(turbo_decode_kernel<OutT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    turbo_decode_kernel<OutT, true><<<grid, kDecThreads, smem, stream>>>(packed, signs, norm, rnorm, (OutT*)out, n, group_blocks, group_stride);
  } else {
    turbo_decode_kernel<OutT, false><<<grid, kDecThreads, smem, stream>>>(packed, signs, norm, rnorm, (OutT*)out, n, group_blocks, group_stride);
  }
  return DFLASH_OK;
}

// ---- encode: one thread per 128-block, the block lives in registers ------------------------------
// Same statement order as turbo_encode_kernel above (the sums of squares run sequentially over i, the butterflies
// stage by stage), with the block in registers instead of strided shared memory.  The CTA's 64 blocks are first staged
// in shared memory with coalesced loads; the normalised vector a key needs again for its residual is recomputed from
// that stage (same operands, same bits) rather than kept in a second register file's worth of state.
template <typename InT> __device__ __forceinline__ void load8_in(const InT* src, float (&o)[8]);
template <> __device__ __forceinline__ void load8_in<float>(const float* src, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <> __device__ __forceinline__ void load8_in<__nv_bfloat16>(const __nv_bfloat16* src, float (&o)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(src);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
}
template <> __device__ __forceinline__ void load8_in<__half>(const __half* src, float (&o)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(src);
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
}

template <typename InT>
__global__ void __launch_bounds__(kDecThreads)
turbo_encode_regs_kernel(const InT* __restrict__ x, uint8_t* __restrict__ packed, uint8_t* __restrict__ signs,
                         uint16_t* __restrict__ norm, uint16_t* __restrict__ rnorm, long long n, int is_key) {
  extern __shared__ float sh[];
  float* c3 = sh;                                            // [8][kDecThreads]: one copy of the centroids per thread column
  constexpr int kRowBytes = kBlock * (int)sizeof(InT) + 16;  // the pad keeps neighbouring threads' 16-byte pieces on different banks
  uint8_t* stage = reinterpret_cast<uint8_t*>(sh + 8 * kDecThreads);
  for (int i = threadIdx.x; i < 8 * kDecThreads; i += kDecThreads) c3[i] = TURBO_C3[i / kDecThreads];
  const long long first = (long long)blockIdx.x * kDecThreads;
  const long long here = n - first < kDecThreads ? n - first : kDecThreads;
  constexpr int kPieces = kBlock * (int)sizeof(InT) / 16;
  for (int p = threadIdx.x; p < (int)here * kPieces; p += kDecThreads) {
    const int t = p / kPieces, off = p % kPieces;
    *reinterpret_cast<uint4*>(stage + t * kRowBytes + off * 16) =
        *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(x + (first + t) * kBlock) + off * 16);
  }
  __syncthreads();
  const long long v = first + threadIdx.x;
  if (v >= n) return;
  const InT* mine = reinterpret_cast<const InT*>(stage + threadIdx.x * kRowBytes);
  float w[kBlock];
  float ns = 0.f;
#pragma unroll
  for (int g8 = 0; g8 < kBlock / 8; ++g8) {
    float f[8];
    load8_in<InT>(mine + g8 * 8, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      w[g8 * 8 + e] = f[e];
      ns = __fadd_rn(ns, __fmul_rn(f[e], f[e]));
    }
  }
  const float gn = __fsqrt_rn(ns), inv = gn > 1e-10f ? __fdiv_rn(1.f, gn) : 0.f;
#pragma unroll
  for (int i = 0; i < kBlock; ++i) w[i] = __fmul_rn(w[i], inv);
  rot_regs(w, TURBO_S1_NEG, TURBO_S2_NEG);
  // 3-bit indices: little-endian bit stream (:19), 8 indices -> 3 bytes; the centroid vector replaces the work vector
  float rs = 0.f;
  unsigned int pk[12];
#pragma unroll
  for (int i = 0; i < 12; ++i) pk[i] = 0u;
#pragma unroll
  for (int i = 0; i < kBlock; ++i) {
    const int idx = nearest3(w[i]);
    const float c = c3[idx * kDecThreads + threadIdx.x];
    const int bit = 3 * i, word = bit >> 5, off = bit & 31;
    pk[word] |= (unsigned int)idx << off;
    if (off > 29) pk[word + 1] |= (unsigned int)idx >> (32 - off);
    rs = __fadd_rn(rs, __fmul_rn(c, c));
    w[i] = c;
  }
  uint4* pout = reinterpret_cast<uint4*>(packed + v * 48);
  pout[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
  pout[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
  pout[2] = make_uint4(pk[8], pk[9], pk[10], pk[11]);
  if (!is_key) {
    const float rn2 = __fsqrt_rn(rs);
    norm[v] = to_f16_trunc(rn2 > 1e-10f ? __fdiv_rn(gn, rn2) : gn);        // :73
    return;
  }
  rot_regs(w, TURBO_S2_NEG, TURBO_S1_NEG);                                 // inverse rotation of the centroids (:91)
  float rns = 0.f;
#pragma unroll
  for (int g8 = 0; g8 < kBlock / 8; ++g8) {
    float f[8];
    load8_in<InT>(mine + g8 * 8, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float r = __fsub_rn(__fmul_rn(f[e], inv), w[g8 * 8 + e]);      // normalised input minus its quantised image
      w[g8 * 8 + e] = r;
      rns = __fadd_rn(rns, __fmul_rn(r, r));
    }
  }
  rot_regs(w, TURBO_Q1_NEG, TURBO_Q2_NEG);                                 // :93
  unsigned int sg[4] = {0u, 0u, 0u, 0u};
#pragma unroll
  for (int i = 0; i < kBlock; ++i) sg[i >> 5] |= (w[i] >= 0.f ? 1u : 0u) << (i & 31);
  *reinterpret_cast<uint4*>(signs + v * 16) = make_uint4(sg[0], sg[1], sg[2], sg[3]);
  norm[v] = to_f16_trunc(gn);
  rnorm[v] = to_f16_trunc(__fsqrt_rn(rns));
}

template <typename InT>
int32_t launch_encode_typed(const void* x, uint8_t* packed, uint8_t* signs, uint16_t* norm, uint16_t* rnorm, long long n, int is_key,
                            cudaStream_t stream) {
  const unsigned grid = (unsigned)((n + kDecThreads - 1) / kDecThreads);
  const bool aligned = !(((uintptr_t)x | (uintptr_t)packed | (is_key ? (uintptr_t)signs : 0)) & 15);
  if (aligned) {   // the block in registers, 16-byte loads and stores
    const size_t smem = 8 * kDecThreads * sizeof(float) + kDecThreads * (kBlock * sizeof(InT) + 16);
    DFLASH_CUDA_CHECK(cudaFuncSetAttribute(turbo_encode_regs_kernel<InT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    turbo_encode_regs_kernel<InT><<<grid, kDecThreads, smem, stream>>>((const InT*)x, packed, signs, norm, rnorm, n, is_key);
  } else {         // byte-wise access, any alignment
    const size_t smem = 2 * kBlock * kThreadsPerCta * sizeof(float);
    DFLASH_CUDA_CHECK(cudaFuncSetAttribute(turbo_encode_kernel<InT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    turbo_encode_kernel<InT><<<grid, kThreadsPerCta, smem, stream>>>((const InT*)x, packed, signs, norm, rnorm, n, is_key);
  }
  return DFLASH_OK;
}

}  // namespace

int32_t launch_turbo_encode(const void* x, uint8_t* packed, uint8_t* signs, uint16_t* norm, uint16_t* rnorm,
                            long long n, int is_key, int in_dtype, cudaStream_t stream) {
  int32_t st;
  switch (in_dtype) {
    case DFLASH_F32: st = launch_encode_typed<float>(x, packed, signs, norm, rnorm, n, is_key, stream); break;
    case DFLASH_BF16: st = launch_encode_typed<__nv_bfloat16>(x, packed, signs, norm, rnorm, n, is_key, stream); break;
    case DFLASH_F16: st = launch_encode_typed<__half>(x, packed, signs, norm, rnorm, n, is_key, stream); break;
    default:
      set_error("turbo_encode: unsupported dtype %d", in_dtype);
      return DFLASH_ERR_UNSUPPORTED;
  }
  if (st != DFLASH_OK) return st;
  DFLASH_LAUNCH_CHECK();
  count_launch();
  return DFLASH_OK;
}

int32_t launch_turbo_decode(const uint8_t* packed, const uint8_t* signs, const uint16_t* norm, const uint16_t* rnorm,
                            void* out, long long n, int is_key, int out_dtype, cudaStream_t stream,
                            long long group_blocks, long long group_stride) {
  if (group_blocks <= 0) { group_blocks = n; group_stride = n * kBlock; }   // one dense run
  if (((uintptr_t)packed & 15) || (is_key && ((uintptr_t)signs & 15)) || ((uintptr_t)out & 15)) {
    set_error("turbo_decode: packed, signs and out must be 16-byte aligned");
    return DFLASH_ERR_INVALID_ARG;
  }
  int32_t st;
  switch (out_dtype) {
    case DFLASH_F32: st = launch_decode_typed<float>(packed, signs, norm, rnorm, out, n, is_key, group_blocks, group_stride, stream); break;
    case DFLASH_BF16: st = launch_decode_typed<__nv_bfloat16>(packed, signs, norm, rnorm, out, n, is_key, group_blocks, group_stride, stream); break;
    case DFLASH_F16: st = launch_decode_typed<__half>(packed, signs, norm, rnorm, out, n, is_key, group_blocks, group_stride, stream); break;
    default:
      set_error("turbo_decode: unsupported dtype %d", out_dtype);
      return DFLASH_ERR_UNSUPPORTED;
  }
  if (st != DFLASH_OK) return st;
  DFLASH_LAUNCH_CHECK();
  count_launch();
  return DFLASH_OK;
}

}  // namespace dflash
