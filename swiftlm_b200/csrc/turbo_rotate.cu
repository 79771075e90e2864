// Rotations around the attention over TurboQuant KV.
//
// The codec's rotation R = S2 . H . S1 (tests/test_turbo_quant.cpp:15 of the SwiftLM tree; H the Walsh-Hadamard
// transform scaled by 1/sqrt(128)) is orthogonal, so the decode of a key (:96-98) and of a value (:74-75) can be
// moved off the N keys and onto the 16 x G query rows and the output rows:
//     q . k_n        = norm_n ( (R q) . c_n  +  (QJL_C / 128) rnorm_n (Rq^T q) . s_n )        Rq = Q2 . H . Q1 (:17)
//     sum_n p_n v_n  = R^T ( sum_n p_n vnorm_n c'_n )
// with c the centroid vector of the 3-bit indices and s the +-1 vector of the sign bits.  The attention kernel then
// works on Q1 = R q, Q2 = Rq^T q and accumulates its output in the rotated domain; the uncompressed hot window (the
// newest tokens) is brought into the same domain by rotating its keys and values, K' = R k, V' = R v.
// This file holds those small rotations: one warp per 128-element block, four elements per lane, the first two
// butterfly stages inside a lane and the other five through warp shuffles.  The butterflies of a stage are
// independent, so the result has the bits of the reference's loops (:14).
#include "common.cuh"
#include "turbo_tables.cuh"

namespace dflash {
namespace {

enum SignSet : int { kS1 = 0, kS2 = 1, kQ1 = 2, kQ2 = 3 };

__device__ __forceinline__ const unsigned int* sign_words(int set) {
  return set == kS1 ? TURBO_S1_NEG : set == kS2 ? TURBO_S2_NEG : set == kQ1 ? TURBO_Q1_NEG : TURBO_Q2_NEG;
}
__device__ __forceinline__ float flip_if(float x, unsigned int word, int bit) {
  return __uint_as_float(__float_as_uint(x) ^ (((word >> bit) & 1u) << 31));
}

// x holds elements 4*lane .. 4*lane+3 of a 128-block: x <- second . H . first applied to it
__device__ __forceinline__ void rot_warp(float (&x)[4], int lane, int first, int second) {
  const unsigned int fw = sign_words(first)[lane >> 3], sw = sign_words(second)[lane >> 3];
  const int bit0 = (lane & 7) * 4;
#pragma unroll
  for (int e = 0; e < 4; ++e) x[e] = flip_if(x[e], fw, bit0 + e);
  {  // h = 1, 2: inside the lane
    const float a0 = __fadd_rn(x[0], x[1]), a1 = __fsub_rn(x[0], x[1]), a2 = __fadd_rn(x[2], x[3]), a3 = __fsub_rn(x[2], x[3]);
    x[0] = __fadd_rn(a0, a2); x[2] = __fsub_rn(a0, a2); x[1] = __fadd_rn(a1, a3); x[3] = __fsub_rn(a1, a3);
  }
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {   // h = 4 d: partner lane at distance d
    const bool upper = (lane & d) != 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float other = __shfl_xor_sync(0xffffffffu, x[e], d);
      x[e] = upper ? __fsub_rn(other, x[e]) : __fadd_rn(x[e], other);
    }
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) x[e] = flip_if(__fmul_rn(x[e], 0.08838834764831845f), sw, bit0 + e);
}

template <typename T> __device__ __forceinline__ void load4(const T* p, float (&x)[4]);
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&x)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  x[0] = __uint_as_float(u.x << 16); x[1] = __uint_as_float(u.x & 0xffff0000u);
  x[2] = __uint_as_float(u.y << 16); x[3] = __uint_as_float(u.y & 0xffff0000u);
}
template <> __device__ __forceinline__ void load4<__half>(const __half* p, float (&x)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
  x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float (&x)[4]);
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&x)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(x[0], x[1]), b = __floats2bfloat162_rn(x[2], x[3]);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}
template <> __device__ __forceinline__ void store4<__half>(__half* p, const float (&x)[4]) {
  const __half2 a = __floats2half2_rn(x[0], x[1]), b = __floats2half2_rn(x[2], x[3]);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

// Up to three jobs in one launch (queries, hot keys, hot values); block v of job j: out_a = rot(first_a, second_a),
// and, where out_b is given, out_b = rot(first_b, second_b) of the same input.
struct RotJob {
  const void* in;
  void* out_a;
  void* out_b;
  long long blocks;
  int first_a, second_a, first_b, second_b;
};
struct RotJobs {
  RotJob job[3];
  int n;
};

template <typename T>
__global__ void __launch_bounds__(256) turbo_rotate_kernel(const RotJobs jobs) {
  const int lane = threadIdx.x & 31;
  long long v = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  for (int j = 0; j < jobs.n; ++j) {
    const RotJob& job = jobs.job[j];
    if (v < job.blocks) {
      float x[4], y[4];
      load4<T>(reinterpret_cast<const T*>(job.in) + v * 128 + lane * 4, x);
#pragma unroll
      for (int e = 0; e < 4; ++e) y[e] = x[e];
      rot_warp(x, lane, job.first_a, job.second_a);
      store4<T>(reinterpret_cast<T*>(job.out_a) + v * 128 + lane * 4, x);
      if (job.out_b) {
        rot_warp(y, lane, job.first_b, job.second_b);
        store4<T>(reinterpret_cast<T*>(job.out_b) + v * 128 + lane * 4, y);
      }
      return;
    }
    v -= job.blocks;
  }
}

template <typename T>
int32_t launch_jobs(const RotJobs& jobs, cudaStream_t stream) {
  long long total = 0;
  for (int j = 0; j < jobs.n; ++j) total += jobs.job[j].blocks;
  if (total <= 0) return DFLASH_OK;
  const long long grid = (total + 7) / 8;
  if (grid > 0x7fffffffLL) { set_error("turbo rotation: too many blocks"); return DFLASH_ERR_UNSUPPORTED; }
  turbo_rotate_kernel<T><<<(unsigned)grid, 256, 0, stream>>>(jobs);
  DFLASH_LAUNCH_CHECK();
  count_launch();
  return DFLASH_OK;
}

}  // namespace

// Q1 = R q and Q2 = Rq^T q of every 128-block of q; K' = R k, V' = R v of the hot window (skipped when n_hot_blocks == 0).
int32_t launch_turbo_rotate_inputs(const void* q, void* q1, void* q2, long long q_blocks, const void* k_hot, void* k_rot,
                                   const void* v_hot, void* v_rot, long long hot_blocks, int dtype, cudaStream_t stream) {
  RotJobs jobs;
  jobs.n = 0;
  jobs.job[jobs.n++] = RotJob{q, q1, q2, q_blocks, kS1, kS2, kQ2, kQ1};
  if (hot_blocks > 0) {
    jobs.job[jobs.n++] = RotJob{k_hot, k_rot, nullptr, hot_blocks, kS1, kS2, 0, 0};
    jobs.job[jobs.n++] = RotJob{v_hot, v_rot, nullptr, hot_blocks, kS1, kS2, 0, 0};
  }
  return dtype == DFLASH_BF16 ? launch_jobs<__nv_bfloat16>(jobs, stream) : launch_jobs<__half>(jobs, stream);
}

// out = R^T o of every 128-block: the attention output back from the rotated domain.
int32_t launch_turbo_unrotate_output(const void* o_rot, void* out, long long blocks, int dtype, cudaStream_t stream) {
  RotJobs jobs;
  jobs.n = 1;
  jobs.job[0] = RotJob{o_rot, out, nullptr, blocks, kS2, kS1, 0, 0};
  return dtype == DFLASH_BF16 ? launch_jobs<__nv_bfloat16>(jobs, stream) : launch_jobs<__half>(jobs, stream);
}

}  // namespace dflash
