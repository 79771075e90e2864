// Gated-delta forward with tape / tape replay — shape-generic kernel.
//
// Covers every shape the reference's kernels accept (Dk a multiple of 32, any Dv, scalar or
// vector gate, any T <= 64), Sources/DFlash/DFlashKernels.swift:271,336.  One warp owns one row
// of the [Dv,Dk] state in registers (lane l holds columns l, l+32, ...), so global reads and
// writes of the state are fully coalesced; the two per-token reductions are warp shuffles.
// The Dk = Dv = 128 scalar-gate case that dominates production traffic is served by the
// TMA-pipelined kernel in gated_delta_fast.cu; this kernel is the general path.
#include "common.cuh"

namespace dflash {
namespace {

constexpr int kMaxNpt = 16;        // Dk <= 512
constexpr int kWarpsPerBlock = 4;

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

template <typename InT, bool VEC, bool REPLAY>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
gdn_generic_kernel(GdnArgs a) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const long long rows = (long long)a.B * a.Hv * a.Dv;
  if (row >= rows) return;
  const int dv = (int)(row % a.Dv);
  const int head = (int)(row / a.Dv);          // b * Hv + hv
  const int b = head / a.Hv, hv = head % a.Hv;
  const int hk = hv / (a.Hv / a.Hk);
  const int npt = a.Dk >> 5;
  const unsigned long long bits = step_bits(a.mask, a.mask_dtype, a.n_per_seq, b, a.T, a.n_div);

  const float* s_in = a.state_in + row * a.Dk;
  float* s_out = a.state_out + row * a.Dk;
  float s[kMaxNpt];
#pragma unroll
  for (int i = 0; i < kMaxNpt; ++i) s[i] = i < npt ? s_in[lane + 32 * i] : 0.f;

  const InT* qp = reinterpret_cast<const InT*>(a.q);
  const InT* kp = reinterpret_cast<const InT*>(a.k);
  const InT* vp = reinterpret_cast<const InT*>(a.v);
  const InT* gp = reinterpret_cast<const InT*>(a.g);
  const InT* bp = reinterpret_cast<const InT*>(a.beta);
  InT* yp = reinterpret_cast<InT*>(a.y);

  for (int t = 0; t < a.T; ++t) {
    const long long bt = (long long)b * a.T + t;
    const long long o_idx = (bt * a.Hv + hv) * a.Dv + dv;
    if (!((bits >> t) & 1ull)) {
      if (!REPLAY && lane == 0) {
        yp[o_idx] = from_f32<InT>(0.f);
        if (a.tape) a.tape[o_idx] = 0.f;
      }
      continue;
    }
    const InT* kt = kp + (bt * a.Hk + hk) * a.Dk;
    const InT* gvec = VEC ? gp + (bt * a.Hv + hv) * a.Dk : nullptr;
    const float gs = VEC ? 0.f : to_f32(gp[bt * a.Hv + hv]);
    float kreg[kMaxNpt];
#pragma unroll
    for (int i = 0; i < kMaxNpt; ++i) kreg[i] = i < npt ? to_f32(kt[lane + 32 * i]) : 0.f;
    if (REPLAY) {
      const float d = a.tape[o_idx];
#pragma unroll
      for (int i = 0; i < kMaxNpt; ++i)
        if (i < npt) {
          const float gi = VEC ? to_f32(gvec[lane + 32 * i]) : gs;
          s[i] = s[i] * gi + kreg[i] * d;
        }
    } else {
      const InT* qt = qp + (bt * a.Hk + hk) * a.Dk;
      float kv = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxNpt; ++i)
        if (i < npt) {
          const float gi = VEC ? to_f32(gvec[lane + 32 * i]) : gs;
          s[i] *= gi;
          kv += s[i] * kreg[i];
        }
      kv = warp_sum(kv);
      const float d = (to_f32(vp[o_idx]) - kv) * to_f32(bp[bt * a.Hv + hv]);
      float out = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxNpt; ++i)
        if (i < npt) {
          s[i] += kreg[i] * d;
          out += s[i] * to_f32(qt[lane + 32 * i]);
        }
      out = warp_sum(out);
      if (lane == 0) {
        yp[o_idx] = from_f32<InT>(out);
        if (a.tape) a.tape[o_idx] = d;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kMaxNpt; ++i)
    if (i < npt) s_out[lane + 32 * i] = s[i];
}

template <typename InT>
int32_t launch_typed(const GdnArgs& a, cudaStream_t stream) {
  const long long rows = (long long)a.B * a.Hv * a.Dv;
  const long long blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (blocks > 0x7fffffffLL) {
    set_error("gated-delta: too many state rows (%lld)", rows);
    return DFLASH_ERR_UNSUPPORTED;
  }
  dim3 grid((unsigned)blocks), block(kWarpsPerBlock * 32);
  if (a.replay) {
    if (a.g_is_vector) gdn_generic_kernel<InT, true, true><<<grid, block, 0, stream>>>(a);
    else gdn_generic_kernel<InT, false, true><<<grid, block, 0, stream>>>(a);
  } else {
    if (a.g_is_vector) gdn_generic_kernel<InT, true, false><<<grid, block, 0, stream>>>(a);
    else gdn_generic_kernel<InT, false, false><<<grid, block, 0, stream>>>(a);
  }
  DFLASH_LAUNCH_CHECK();
  count_launch();
  return DFLASH_OK;
}

}  // namespace

int32_t launch_gdn_generic(const GdnArgs& a, cudaStream_t stream) {
  switch (a.in_dtype) {
    case DFLASH_F32: return launch_typed<float>(a, stream);
    case DFLASH_BF16: return launch_typed<__nv_bfloat16>(a, stream);
    case DFLASH_F16: return launch_typed<__half>(a, stream);
    default:
      set_error("gated-delta: unsupported input dtype %d", a.in_dtype);
      return DFLASH_ERR_UNSUPPORTED;
  }
}

}  // namespace dflash
