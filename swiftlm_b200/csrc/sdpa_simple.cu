// Block-verify attention on CUDA cores: the general path of dflash_verify_sdpa.
//
// Serves what the tensor-core kernel (sdpa_tc.cu) does not take — a call without the tensor-core
// kernel's workspace, a non-positive scale, more than 4096 ragged sequences — with the exact semantics of the reference's
// two-pass kernel (Sources/DFlash/DFlashKernels.swift:563-649, :661-720): q pre-scaled,
// fp32 online softmax one key at a time, visibility n <= N_b - 16 + r, optional additive mask
// whose entries below the dtype's finite minimum hide the key, log-sum-exp merge of the
// split-KV partials, zero-sum guard on the final divide.  Differences from the reference: the
// KV range of a split is contiguous rather than strided, and partials stay fp32.
//
// Mapping: one block per (sequence, query head, split); 16 warps = the 16 query rows; lane l
// holds elements l, l+32, ... of the row's q and of its output accumulator.
#include "common.cuh"

namespace dflash {
namespace {

constexpr int kRows = 16;
constexpr int kMaxDpt = 8;  // D <= 256

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

template <typename T> __device__ __forceinline__ float finite_min_of();
template <> __device__ __forceinline__ float finite_min_of<__nv_bfloat16>() { return -3.3895313892515355e38f; }
template <> __device__ __forceinline__ float finite_min_of<__half>() { return -65504.f; }

struct SimpleParams {
  SdpaArgs a;
  int splits;
  float* part_o;   // [B*Hq*16][splits][D]
  float* part_m;   // [B*Hq*16][splits]
  float* part_l;
};

template <typename InT>
__global__ void __launch_bounds__(kRows * 32) sdpa_simple_kernel(SimpleParams p) {
  const SdpaArgs& a = p.a;
  const int lane = threadIdx.x & 31, r = threadIdx.x >> 5;
  const int bh = blockIdx.x, split = blockIdx.y;
  const int b = bh / a.Hq, h = bh % a.Hq;
  const int hk = h / (a.Hq / a.Hkv);
  const int dpt = a.D >> 5;
  int Nb = a.kv_len ? a.kv_len[b] : a.N;
  Nb = Nb < 0 ? 0 : (Nb > a.N ? a.N : Nb);   // a length outside [0, N] is clamped (the tensor-core kernel reports it)
  const int chunk = (Nb + p.splits - 1) / p.splits;
  const int n0 = split * chunk, n1 = min(Nb, n0 + chunk);
  const int last = Nb - kRows + r;  // last visible key of this row

  const InT* qrow = reinterpret_cast<const InT*>(a.q) + ((long long)bh * kRows + r) * a.D;
  float q[kMaxDpt], o[kMaxDpt];
#pragma unroll
  for (int i = 0; i < kMaxDpt; ++i) {
    q[i] = i < dpt ? a.scale * to_f32(qrow[lane + 32 * i]) : 0.f;
    o[i] = 0.f;
  }
  float mx = -3.402823466e38f, se = 0.f;
  const InT* kbase = reinterpret_cast<const InT*>(a.k);
  const InT* vbase = reinterpret_cast<const InT*>(a.v);
  const InT* mrow = a.mask ? reinterpret_cast<const InT*>(a.mask) + ((long long)bh * kRows + r) * a.N : nullptr;

  for (int n = n0; n < n1 && n <= last; ++n) {
    long long row_off;
    if (a.page_table) {
      const int page = a.page_table[(long long)b * a.max_pages + n / a.page_tokens];
      if (page < 0 || (a.num_pages > 0 && page >= a.num_pages)) continue;   // a page id outside the pool hides its keys
      row_off = (((long long)page * a.Hkv + hk) * a.page_tokens + n % a.page_tokens) * a.D;
    } else {
      row_off = (((long long)b * a.Hkv + hk) * a.N + n) * a.D;
    }
    float mval = 0.f;
    if (mrow) {
      mval = to_f32(mrow[n]);
      if (!(mval >= finite_min_of<InT>())) continue;
    }
    const InT* kr = kbase + row_off;
    float sc = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxDpt; ++i)
      if (i < dpt) sc += q[i] * to_f32(kr[lane + 32 * i]);
    sc = warp_sum(sc) + mval;
    const float nm = fmaxf(mx, sc);
    const float f = __expf(mx - nm), e = __expf(sc - nm);
    mx = nm;
    se = se * f + e;
    const InT* vr = vbase + row_off;
#pragma unroll
    for (int i = 0; i < kMaxDpt; ++i)
      if (i < dpt) o[i] = o[i] * f + e * to_f32(vr[lane + 32 * i]);
  }

  const long long orow = (long long)bh * kRows + r;
  if (p.splits == 1) {
    InT* out = reinterpret_cast<InT*>(a.out) + orow * a.D;
    const float inv = se == 0.f ? 1.f : 1.f / se;
#pragma unroll
    for (int i = 0; i < kMaxDpt; ++i)
      if (i < dpt) out[lane + 32 * i] = from_f32<InT>(o[i] * inv);
  } else {
    float* po = p.part_o + (orow * p.splits + split) * a.D;
#pragma unroll
    for (int i = 0; i < kMaxDpt; ++i)
      if (i < dpt) po[lane + 32 * i] = o[i];
    if (lane == 0) {
      p.part_m[orow * p.splits + split] = mx;
      p.part_l[orow * p.splits + split] = se;
    }
  }
}

// One warp per output row: merge the split partials (reference :687-711).
template <typename InT>
__global__ void sdpa_simple_merge_kernel(SimpleParams p, long long rows) {
  const SdpaArgs& a = p.a;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int dpt = a.D >> 5;
  float gm = -3.402823466e38f;
  for (int s = 0; s < p.splits; ++s) gm = fmaxf(gm, p.part_m[row * p.splits + s]);
  float den = 0.f, o[kMaxDpt];
#pragma unroll
  for (int i = 0; i < kMaxDpt; ++i) o[i] = 0.f;
  for (int s = 0; s < p.splits; ++s) {
    const float f = __expf(p.part_m[row * p.splits + s] - gm);
    den += f * p.part_l[row * p.splits + s];
    const float* po = p.part_o + (row * p.splits + s) * a.D;
#pragma unroll
    for (int i = 0; i < kMaxDpt; ++i)
      if (i < dpt) o[i] += f * po[lane + 32 * i];
  }
  InT* out = reinterpret_cast<InT*>(a.out) + row * a.D;
  const float inv = den == 0.f ? 1.f : 1.f / den;
#pragma unroll
  for (int i = 0; i < kMaxDpt; ++i)
    if (i < dpt) out[lane + 32 * i] = from_f32<InT>(o[i] * inv);
}

int simple_splits(int B, int Hq) {
  const int blocks = B * Hq;
  int s = (2 * 148 + blocks - 1) / blocks;
  return s < 1 ? 1 : (s > 8 ? 8 : s);
}

template <typename InT>
int32_t launch_typed(const SdpaArgs& a, cudaStream_t stream) {
  SimpleParams p;
  p.a = a;
  p.splits = simple_splits(a.B, a.Hq);
  const long long rows = (long long)a.B * a.Hq * kRows;
  if (p.splits > 1) {
    const size_t need = (size_t)rows * p.splits * (a.D + 2) * sizeof(float);
    if (!a.workspace || a.workspace_bytes < need) {
      set_error("verify_sdpa: workspace of %zu bytes needed, %zu given", need, a.workspace_bytes);
      return DFLASH_ERR_WORKSPACE;
    }
    p.part_o = reinterpret_cast<float*>(a.workspace);
    p.part_m = p.part_o + (size_t)rows * p.splits * a.D;
    p.part_l = p.part_m + (size_t)rows * p.splits;
  } else {
    p.part_o = p.part_m = p.part_l = nullptr;
  }
  sdpa_simple_kernel<InT><<<dim3(a.B * a.Hq, p.splits), kRows * 32, 0, stream>>>(p);
  DFLASH_LAUNCH_CHECK();
  count_launch();
  if (p.splits > 1) {
    const int wpb = 8;
    sdpa_simple_merge_kernel<InT><<<(unsigned)((rows + wpb - 1) / wpb), wpb * 32, 0, stream>>>(p, rows);
    DFLASH_LAUNCH_CHECK();
    count_launch();
  }
  return DFLASH_OK;
}

}  // namespace

size_t sdpa_simple_workspace_bytes(int B, int Hq, int D) {
  const int s = simple_splits(B, Hq);
  return s > 1 ? (size_t)B * Hq * kRows * s * (D + 2) * sizeof(float) : 0;
}

int32_t launch_sdpa_simple(const SdpaArgs& a, cudaStream_t stream) {
  if (a.dtype == DFLASH_BF16) return launch_typed<__nv_bfloat16>(a, stream);
  if (a.dtype == DFLASH_F16) return launch_typed<__half>(a, stream);
  set_error("verify_sdpa: dtype must be bf16 or f16");
  return DFLASH_ERR_UNSUPPORTED;
}

}  // namespace dflash
