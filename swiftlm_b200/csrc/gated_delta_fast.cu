// Gated-delta forward with tape / tape replay for the production shape: Dk = Dv = 128,
// scalar gate, T <= 16 (one DFlash verify block).  HBM-bound: the 64 KiB fp32 state of every
// (sequence, v-head) is read once and written once; everything else is small.
//
// One persistent CTA per SM, warp-specialised, with no CTA-wide barrier after set-up:
//   * 16 compute warps.  Warp w owns rows 8w..8w+7 of the state of the current work item: its
//     lanes hold 2 rows x 16 columns each (32 floats in registers), a row is spread over 8
//     adjacent lanes.  The warp streams its own rows in by TMA (four 128-byte-swizzled boxes of
//     8 rows x 32 floats, completion on the warp's own mbarrier, two items ahead), computes,
//     and writes its rows out as full 128-byte lines.  Per running step one pass over the
//     registers does the rank-1 update of the step, its output dot products and the kv dot
//     products of the next step, followed by one 3-level shuffle reduction; all arithmetic is
//     packed fp32x2 FMA on the lazily-decayed state (3 FMA per element per step).
//   * 1 producer warp.  It fetches the per-token inputs of the work item two ahead (k, q, v or
//     the recorded delta by 16-byte cp.async, only for the steps that will run; gates, betas
//     and the step mask by plain loads one item earlier), converts them to fp32 staging buffers
//     and publishes them on an mbarrier; compute warps hand a staging buffer back through a
//     second mbarrier when they are done with it.
// Work items are ordered so that consecutive items come from different sequences: accepted
// lengths differ per sequence, and mixing them keeps copy-only items (n = 0) and compute-heavy
// items (n = 16) overlapping on every SM.  Every wait is bounded; a wait that gives up sets the
// device status word and the CTA winds down.
//
// Reference semantics: Sources/DFlash/DFlashKernels.swift:122-199 (forward), :43-81 (replay),
// CPU statements :409-466 and :371-407; fp32 state without per-step rounding.
#include "common.cuh"
#include "ptx.cuh"

namespace dflash {
namespace {

constexpr int kD = 128;
constexpr int kTmax = 16;
constexpr int kComputeWarps = 16;      // each owns 8 rows of the state
constexpr int kThreads = (kComputeWarps + 1) * 32;   // + 1 producer warp
constexpr int kStages = 2;
constexpr uint32_t kStateBytes = kD * kD * 4;
constexpr uint32_t kWarpStateBytes = 8 * kD * 4;      // 8 rows

template <typename InT, bool REPLAY>
struct Layout {
  static constexpr uint32_t in_row = kD * sizeof(InT);
  static constexpr uint32_t f32_tile = kTmax * kD * 4;                            // 8 KiB
  // state: [stage][warp][box][8 rows][32 floats]
  static constexpr uint32_t state = 0;
  static constexpr uint32_t k32 = kStages * kStateBytes;                          // [stage][16][128] fp32
  static constexpr uint32_t q32 = k32 + kStages * f32_tile;                       // forward only
  static constexpr uint32_t d32 = REPLAY ? q32 : q32 + kStages * f32_tile;        // [stage][warp][16 steps][8 rows]: v / delta in; y out
  static constexpr uint32_t dout = d32 + kStages * f32_tile;                      // forward only: delta out [warp][16][8]
  static constexpr uint32_t raw_k = REPLAY ? dout : dout + f32_tile;              // producer-private raw inputs
  static constexpr uint32_t raw_q = raw_k + kTmax * in_row;                       // forward only
  static constexpr uint32_t raw_v = REPLAY ? raw_q : raw_q + kTmax * in_row;      // v (InT) or recorded delta (fp32)
  static constexpr uint32_t raw_end = raw_v + kTmax * (REPLAY ? kD * 4 : in_row);
  static constexpr uint32_t s_beta = raw_end;                    // [stage][16]
  static constexpr uint32_t s_g = s_beta + kStages * 16 * 4;     // [stage][16]
  static constexpr uint32_t s_bits = s_g + kStages * 16 * 4;     // [stage]
  static constexpr uint32_t s_abort = s_bits + 8;
  static constexpr uint32_t bar_state = s_abort + 8;                                // [stage][warp]
  static constexpr uint32_t bar_full = bar_state + 8 * kStages * kComputeWarps;     // [stage]
  static constexpr uint32_t bar_empty = bar_full + 8 * kStages;                     // [stage]
  static constexpr uint32_t total = bar_empty + 8 * kStages;
  static constexpr uint32_t alloc = total + 1024;        // room to align the base to 1024 bytes
};

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

template <typename InT>
__device__ __forceinline__ float4 load4_as_f32(const InT* src);
template <>
__device__ __forceinline__ float4 load4_as_f32<float>(const float* src) { return *reinterpret_cast<const float4*>(src); }
template <>
__device__ __forceinline__ float4 load4_as_f32<__nv_bfloat16>(const __nv_bfloat16* src) {
  const uint2 u = *reinterpret_cast<const uint2*>(src);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                     __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}
template <>
__device__ __forceinline__ float4 load4_as_f32<__half>(const __half* src) {
  const uint2 u = *reinterpret_cast<const uint2*>(src);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

template <typename OutT>
__device__ __forceinline__ void store4(OutT* dst, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* dst, float4 v) {
  __nv_bfloat162 p[2] = {__floats2bfloat162_rn(v.x, v.y), __floats2bfloat162_rn(v.z, v.w)};
  *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(p);
}
template <>
__device__ __forceinline__ void store4<__half>(__half* dst, float4 v) {
  __half2 p[2] = {__floats2half2_rn(v.x, v.y), __floats2half2_rn(v.z, v.w)};
  *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(p);
}

// Two per-row partial sums, each spread over the 8 lanes of a row group (lane bits 0-2), reduced
// in 3 shuffles: afterwards the lanes with bit0 == i hold the complete sum of row slot i.
__device__ __forceinline__ float reduce2_over8(float v0, float v1, int lane) {
  const bool b0 = lane & 1;
  float x = (b0 ? v1 : v0) + __shfl_xor_sync(0xffffffffu, b0 ? v0 : v1, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  return x;
}

// Bounded mbarrier wait that also watches the CTA's abort flag.  All lanes of the calling
// warp agree on the result.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
  bool ok = false;
  for (uint32_t i = 0; i < ptx::kWaitPolls; ++i) {
    if (ptx::mbar_try_wait(bar, parity)) { ok = true; break; }
    if ((i & 127u) == 127u) {
      if (*abort_flag) break;
      __nanosleep(64);
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  if (!ok && (threadIdx.x & 31) == 0 && !*abort_flag) {
    *abort_flag = 1;
    atomicExch(status, 1);
  }
  return ok;
}

template <typename InT, bool REPLAY>
__global__ void __launch_bounds__(kThreads, 1)
gdn_fast_kernel(const __grid_constant__ CUtensorMap state_map, const GdnArgs a, int* status) {
  using L = Layout<InT, REPLAY>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int T = a.T;
  const int rep = a.Hv / a.Hk;
  const uint32_t n_items = (uint32_t)a.B * (uint32_t)a.Hv;   // < 2^24: checked by the launcher
  const uint32_t G = gridDim.x;

  float* s_beta = reinterpret_cast<float*>(sm + L::s_beta);
  float* s_g = reinterpret_cast<float*>(sm + L::s_g);
  uint32_t* s_bits = reinterpret_cast<uint32_t*>(sm + L::s_bits);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + L::s_abort);
  uint64_t* bar_state = reinterpret_cast<uint64_t*>(sm + L::bar_state);
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(sm + L::bar_full);
  uint64_t* bar_empty = reinterpret_cast<uint64_t*>(sm + L::bar_empty);

  // item -> (sequence b, v-head hv): v-heads that share a qk-head are adjacent items, then
  // the sequence index varies fastest, the qk-head slowest.
  // (32-bit unsigned arithmetic: 64-bit division would cost hundreds of instructions per item)
  auto decode = [&](uint32_t i, int& b, int& hv) {
    const uint32_t p = i / (uint32_t)rep, sub = i - p * (uint32_t)rep;
    const uint32_t hk = p / (uint32_t)a.B;
    b = (int)(p - hk * (uint32_t)a.B);
    hv = (int)(hk * (uint32_t)rep + sub);
  };

  if (tid == 0) {
    ptx::prefetch_tensormap(&state_map);
    for (int i = 0; i < kStages * kComputeWarps; ++i) ptx::mbar_init(&bar_state[i], 1);
    for (int i = 0; i < kStages; ++i) {
      ptx::mbar_init(&bar_full[i], 1);
      ptx::mbar_init(&bar_empty[i], kComputeWarps);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();
  if (blockIdx.x >= n_items) return;

  if (w == kComputeWarps) {
    // =============================== producer warp ===============================
    const InT* gq = reinterpret_cast<const InT*>(a.q);
    const InT* gk = reinterpret_cast<const InT*>(a.k);
    const InT* gv = reinterpret_cast<const InT*>(a.v);
    const InT* gg = reinterpret_cast<const InT*>(a.g);
    const InT* gbeta = reinterpret_cast<const InT*>(a.beta);
    auto load_scalars = [&](uint32_t item, bool& on, float& g, float& beta) {
      on = false; g = 0.f; beta = 0.f;
      if (item < n_items && lane < T) {
        int b, hv;
        decode(item, b, hv);
        on = true;
        if (a.n_per_seq) on = lane < a.n_per_seq[b];
        if (on && a.mask) on = mask_on(a.mask, a.mask_dtype, b * T + lane);
        const long long bt = (long long)b * T + lane;
        g = to_f32(gg[bt * a.Hv + hv]);
        if (!REPLAY) beta = to_f32(gbeta[bt * a.Hv + hv]);
      }
    };
    bool on_c; float g_c, beta_c;
    uint32_t item = blockIdx.x;
    load_scalars(item, on_c, g_c, beta_c);
    for (int it = 0; item < n_items; ++it, item += G) {
      const int stage = it & 1;
      if (it >= kStages && !wait_bar(&bar_empty[stage], ((it >> 1) - 1) & 1, abort_flag, status)) break;
      const uint32_t bits = __ballot_sync(0xffffffffu, on_c);
      int b, hv;
      decode(item, b, hv);
      const int hk = hv / rep;
      if (lane < 16) {
        s_g[stage * 16 + lane] = g_c;
        s_beta[stage * 16 + lane] = beta_c;
      }
      if (lane == 0) s_bits[stage] = bits;
      // raw inputs of the running steps: 16-byte cp.async, one row of 128 elements per step
      constexpr int cpr = L::in_row / 16;
      for (int c = lane; c < kTmax * cpr; c += 32) {
        const int t = c / cpr, off = (c % cpr) * 16;
        if (t < T && ((bits >> t) & 1u)) {
          const long long bt = (long long)b * T + t;
          ptx::cp_async16(sm + L::raw_k + t * L::in_row + off, reinterpret_cast<const uint8_t*>(gk + (bt * a.Hk + hk) * kD) + off);
          if (!REPLAY) {
            ptx::cp_async16(sm + L::raw_q + t * L::in_row + off, reinterpret_cast<const uint8_t*>(gq + (bt * a.Hk + hk) * kD) + off);
            ptx::cp_async16(sm + L::raw_v + t * L::in_row + off, reinterpret_cast<const uint8_t*>(gv + (bt * a.Hv + hv) * kD) + off);
          }
        }
      }
      if (REPLAY) {
        constexpr int cpr4 = kD * 4 / 16;
        for (int c = lane; c < kTmax * cpr4; c += 32) {
          const int t = c / cpr4, off = (c % cpr4) * 16;
          if (t < T && ((bits >> t) & 1u))
            ptx::cp_async16(sm + L::raw_v + t * (kD * 4) + off,
                            reinterpret_cast<const uint8_t*>(a.tape + (((long long)b * T + t) * a.Hv + hv) * kD) + off);
        }
      }
      ptx::cp_async_commit();
      // gates, betas and step mask of the following item: in flight while this one is staged
      bool on_n; float g_n, beta_n;
      load_scalars(item + G, on_n, g_n, beta_n);
      ptx::cp_async_wait_all();
      __syncwarp();
      // raw -> fp32 staging of this stage; lane owns columns 4*lane .. 4*lane+3
      float* k32 = reinterpret_cast<float*>(sm + L::k32 + stage * L::f32_tile);
      float* q32 = reinterpret_cast<float*>(sm + L::q32 + stage * L::f32_tile);
      float* d32 = reinterpret_cast<float*>(sm + L::d32 + stage * L::f32_tile);
      const int c4 = 4 * lane;
      for (int t = 0; t < T; ++t) {
        if (!((bits >> t) & 1u)) continue;
        store4<float>(k32 + t * kD + c4, load4_as_f32<InT>(reinterpret_cast<const InT*>(sm + L::raw_k) + t * kD + c4));
        float* dstage = d32 + (c4 >> 3) * (kTmax * 8) + t * 8 + (c4 & 7);   // [owner warp][step][row in warp]
        if (!REPLAY) {
          store4<float>(q32 + t * kD + c4, load4_as_f32<InT>(reinterpret_cast<const InT*>(sm + L::raw_q) + t * kD + c4));
          store4<float>(dstage, load4_as_f32<InT>(reinterpret_cast<const InT*>(sm + L::raw_v) + t * kD + c4));
        } else {
          store4<float>(dstage, load4_as_f32<float>(reinterpret_cast<const float*>(sm + L::raw_v) + t * kD + c4));
        }
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bar_full[stage]);
      on_c = on_n; g_c = g_n; beta_c = beta_n;
    }
    return;
  }

  // ================================= compute warps =================================
  const int c_sub = lane & 7, r_sub = lane >> 3;   // 8 lanes share a state row; 4 row slots per warp
  const int col = 4 * c_sub;          // this thread's 4 columns inside each 32-column box
  const int my_i = lane & 1;          // row slot whose reduced sums this lane ends up holding
  const int my_r = r_sub + 4 * my_i;  // that row, relative to the warp's 8 rows
  float* dout = reinterpret_cast<float*>(sm + L::dout) + w * (kTmax * 8);

  auto issue_state = [&](uint32_t item, int stage) {   // lane 0 of the warp
    int b, hv;
    decode(item, b, hv);
    uint64_t* bar = &bar_state[stage * kComputeWarps + w];
    ptx::mbar_arrive_expect_tx(bar, kWarpStateBytes);
    const int row0 = (b * a.Hv + hv) * kD + 8 * w;
    uint8_t* dst = sm + L::state + stage * kStateBytes + w * kWarpStateBytes;
#pragma unroll
    for (int box = 0; box < 4; ++box) ptx::tma_load_2d(dst + box * 1024, &state_map, box * 32, row0, bar);
  };

  uint32_t item = blockIdx.x;
  if (lane == 0) {
    issue_state(item, 0);
    if (item + G < n_items) issue_state(item + G, 1);
  }

  for (int it = 0; item < n_items; ++it, item += G) {
    const int stage = it & 1;
    const uint32_t par = (it >> 1) & 1;
    int b_cur, hv_cur;
    decode(item, b_cur, hv_cur);
    if (!wait_bar(&bar_state[stage * kComputeWarps + w], par, abort_flag, status)) break;

    // thread (r_sub, c_sub) owns rows 8w + r_sub + 4i (i < 2) and, in each 32-column box, the
    // 4 columns of 16-byte chunk c_sub: 32 floats.  A quarter warp reads 8 distinct chunks of
    // one row, so the swizzled tile is read without bank conflicts.
    float2 S[2][4][2];
    {
      const uint8_t* src = sm + L::state + stage * kStateBytes + w * kWarpStateBytes;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int row = r_sub + 4 * i;          // row inside the warp's 8-row boxes
        const int phys = c_sub ^ row;           // 128-byte swizzle: chunk index xor (row mod 8)
#pragma unroll
        for (int box = 0; box < 4; ++box) {
          const float4 v4 = *reinterpret_cast<const float4*>(src + box * 1024 + row * 128 + phys * 16);
          S[i][box][0] = f2(v4.x, v4.y);
          S[i][box][1] = f2(v4.z, v4.w);
        }
      }
    }
    __syncwarp();
    if (lane == 0 && item + 2 * G < n_items) {
      ptx::fence_proxy_async();   // the reads above precede the asynchronous refill of the same bytes
      issue_state(item + 2 * G, stage);
    }
    if (!wait_bar(&bar_full[stage], par, abort_flag, status)) break;
    const uint32_t bits = s_bits[stage];
    const float* k32 = reinterpret_cast<const float*>(sm + L::k32 + stage * L::f32_tile);
    const float* q32 = reinterpret_cast<const float*>(sm + L::q32 + stage * L::f32_tile);
    float* d32 = reinterpret_cast<float*>(sm + L::d32 + stage * L::f32_tile) + w * (kTmax * 8);
    const float* sg = s_g + stage * 16;
    const float* sbeta = s_beta + stage * 16;

    // ---- the recurrence over the running steps ----
    // The state is carried as S = Gd * U with a running scalar Gd (product of the gates so far):
    //   kv = Gd * <U_row, k>,  delta = (v - kv) * beta,  U_row += (delta / Gd) * k,  y = Gd * <U_row, q>
    // which is 3 fused multiply-adds per state element per step instead of 4.  When Gd gets
    // small (or a gate is exactly 0) it is folded back into U, so delta / Gd never overflows.
    float Gd = 1.f;
    auto fold_gate = [&]() {  // U <- Gd * U, Gd <- 1   (uniform per work item)
      const float2 G2 = f2(Gd, Gd);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int box = 0; box < 4; ++box)
#pragma unroll
          for (int j = 0; j < 2; ++j) S[i][box][j] = __fmul2_rn(G2, S[i][box][j]);
      Gd = 1.f;
    };
    if (REPLAY) {
      for (int t = 0; t < T; ++t) {
        if (!((bits >> t) & 1u)) continue;
        Gd *= sg[t];
        if (Gd < 1e-12f) fold_gate();
        const float inv_G = __fdividef(1.f, Gd);
        const float d0 = d32[t * 8 + r_sub] * inv_G, d1 = d32[t * 8 + r_sub + 4] * inv_G;
        const float2 dd0 = f2(d0, d0), dd1 = f2(d1, d1);
#pragma unroll
        for (int box = 0; box < 4; ++box) {
          const float4 k4 = *reinterpret_cast<const float4*>(k32 + t * kD + 32 * box + col);
          const float2 kk[2] = {f2(k4.x, k4.y), f2(k4.z, k4.w)};
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            S[0][box][j] = __ffma2_rn(dd0, kk[j], S[0][box][j]);
            S[1][box][j] = __ffma2_rn(dd1, kk[j], S[1][box][j]);
          }
        }
      }
    } else if (bits != 0u) {
      // One pass over the registers per step does three things at once: the rank-1 update of
      // step t, the output dot products of step t (against q_t) and the kv dot products of
      // the NEXT running step (against its k).  The four row sums then go through a single
      // 3-level shuffle reduction, so a step costs one pass and one reduction.
      uint32_t rem = bits;
      int t = __ffs(rem) - 1;
      rem &= rem - 1;
      float d0, d1;        // delta / Gd of step t for this thread's two rows
      {
        // first running step: kv dot products on their own
        float2 acc[2][2];
#pragma unroll
        for (int i = 0; i < 2; ++i) acc[i][0] = acc[i][1] = f2(0.f, 0.f);
#pragma unroll
        for (int box = 0; box < 4; ++box) {
          const float4 k4 = *reinterpret_cast<const float4*>(k32 + t * kD + 32 * box + col);
          const float2 kk[2] = {f2(k4.x, k4.y), f2(k4.z, k4.w)};
#pragma unroll
          for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 2; ++j) acc[i][j] = __ffma2_rn(S[i][box][j], kk[j], acc[i][j]);
        }
        const float p0 = (acc[0][0].x + acc[0][0].y) + (acc[0][1].x + acc[0][1].y);
        const float p1 = (acc[1][0].x + acc[1][0].y) + (acc[1][1].x + acc[1][1].y);
        const float asum = reduce2_over8(p0, p1, lane);
        Gd = sg[t];
        const float kv = Gd * asum;
        if (Gd < 1e-12f) fold_gate();
        const float d_mine = (d32[t * 8 + my_r] - kv) * sbeta[t];
        if ((lane & 6) == 4) dout[t * 8 + my_r] = d_mine;
        const float ds = __fdividef(d_mine, Gd);
        d0 = __shfl_sync(0xffffffffu, ds, (lane & ~7) | 4);
        d1 = __shfl_sync(0xffffffffu, ds, (lane & ~7) | 5);
      }
      while (true) {
        const int tn = rem ? __ffs(rem) - 1 : -1;   // next running step, if any
        rem &= rem - 1;
        const float* kt = k32 + t * kD + col;
        const float* qt = q32 + t * kD + col;
        const float* kn = k32 + (tn < 0 ? t : tn) * kD + col;
        const float2 dd0 = f2(d0, d0), dd1 = f2(d1, d1);
        float2 acc_y[2][2], acc_a[2][2];
#pragma unroll
        for (int i = 0; i < 2; ++i) acc_y[i][0] = acc_y[i][1] = acc_a[i][0] = acc_a[i][1] = f2(0.f, 0.f);
#pragma unroll
        for (int box = 0; box < 4; ++box) {
          const float4 k4 = *reinterpret_cast<const float4*>(kt + 32 * box);
          const float4 q4 = *reinterpret_cast<const float4*>(qt + 32 * box);
          const float4 n4 = *reinterpret_cast<const float4*>(kn + 32 * box);
          const float2 kk[2] = {f2(k4.x, k4.y), f2(k4.z, k4.w)};
          const float2 qq[2] = {f2(q4.x, q4.y), f2(q4.z, q4.w)};
          const float2 nn[2] = {f2(n4.x, n4.y), f2(n4.z, n4.w)};
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            S[0][box][j] = __ffma2_rn(dd0, kk[j], S[0][box][j]);
            S[1][box][j] = __ffma2_rn(dd1, kk[j], S[1][box][j]);
            acc_y[0][j] = __ffma2_rn(S[0][box][j], qq[j], acc_y[0][j]);
            acc_y[1][j] = __ffma2_rn(S[1][box][j], qq[j], acc_y[1][j]);
            acc_a[0][j] = __ffma2_rn(S[0][box][j], nn[j], acc_a[0][j]);
            acc_a[1][j] = __ffma2_rn(S[1][box][j], nn[j], acc_a[1][j]);
          }
        }
        // 4 row sums (2 outputs, 2 next-step kv) over the 8 lanes of the row group: lanes with
        // bit 2 clear end up with y of row slot (lane & 1), lanes with bit 2 set with kv.
        float r;
        {
          const bool hi = lane & 4, b0 = lane & 1;
          const float y0 = (acc_y[0][0].x + acc_y[0][0].y) + (acc_y[0][1].x + acc_y[0][1].y);
          const float y1 = (acc_y[1][0].x + acc_y[1][0].y) + (acc_y[1][1].x + acc_y[1][1].y);
          const float a0 = (acc_a[0][0].x + acc_a[0][0].y) + (acc_a[0][1].x + acc_a[0][1].y);
          const float a1 = (acc_a[1][0].x + acc_a[1][0].y) + (acc_a[1][1].x + acc_a[1][1].y);
          const float k0 = (hi ? a0 : y0) + __shfl_xor_sync(0xffffffffu, hi ? y0 : a0, 4);
          const float k1 = (hi ? a1 : y1) + __shfl_xor_sync(0xffffffffu, hi ? y1 : a1, 4);
          r = (b0 ? k1 : k0) + __shfl_xor_sync(0xffffffffu, b0 ? k0 : k1, 1);
          r += __shfl_xor_sync(0xffffffffu, r, 2);
        }
        if ((lane & 6) == 0) d32[t * 8 + my_r] = Gd * r;   // y of step t takes the slot v_t was read from
        if (tn < 0) break;
        // lanes with bit 2 set hold <U_row, k_next>: finish step tn's delta there
        const float Gn = Gd * sg[tn];
        const float kv = Gn * r;
        Gd = Gn;
        if (Gd < 1e-12f) fold_gate();
        const float d_mine = (d32[tn * 8 + my_r] - kv) * sbeta[tn];
        if ((lane & 6) == 4) dout[tn * 8 + my_r] = d_mine;
        const float ds = __fdividef(d_mine, Gd);
        d0 = __shfl_sync(0xffffffffu, ds, (lane & ~7) | 4);
        d1 = __shfl_sync(0xffffffffu, ds, (lane & ~7) | 5);
        t = tn;
      }
    }
    if (Gd != 1.f) fold_gate();

    // ---- new state: each warp instruction writes four full 128-byte lines ----
    {
      float* obase = a.state_out + ((long long)(b_cur * a.Hv + hv_cur) * kD + 8 * w + r_sub) * kD + col;
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int box = 0; box < 4; ++box)
          *reinterpret_cast<float4*>(obase + (long long)(4 * i) * kD + 32 * box) =
              make_float4(S[i][box][0].x, S[i][box][0].y, S[i][box][1].x, S[i][box][1].y);
    }
    if (!REPLAY) {
      __syncwarp();
      const int t = lane >> 1, half = lane & 1;   // 16 steps x 2 halves of the warp's 8 rows
      if (t < T) {
        const bool on = (bits >> t) & 1u;
        const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 yv = on ? *reinterpret_cast<const float4*>(d32 + t * 8 + 4 * half) : zero;
        const long long o = (((long long)b_cur * T + t) * a.Hv + hv_cur) * kD + 8 * w + 4 * half;
        store4<InT>(reinterpret_cast<InT*>(a.y) + o, yv);
        if (a.tape) store4<float>(a.tape + o, on ? *reinterpret_cast<const float4*>(dout + t * 8 + 4 * half) : zero);
      }
    }
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(&bar_empty[stage]);   // this stage's staging buffers may be refilled
  }
}

template <typename InT, bool REPLAY>
int32_t launch_typed(const GdnArgs& a, cudaStream_t stream) {
  using L = Layout<InT, REPLAY>;
  EncodeTiledFn encode = tensor_map_encoder();
  if (!encode) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return DFLASH_ERR_CUDA;
  }
  int* status = device_status_word();
  if (!status) {
    set_error("no CUDA device");
    return DFLASH_ERR_CUDA;
  }
  const unsigned long long rows = (unsigned long long)a.B * a.Hv * kD;
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)kD, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)kD * 4};
  const cuuint32_t box[2] = {32, 8};   // one 128-byte-swizzle atom: 8 rows x 32 floats
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(a.state_in), dims, strides, box,
                            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled(state) failed with CUresult %d", (int)r);
    return DFLASH_ERR_CUDA;
  }
  auto kernel = gdn_fast_kernel<InT, REPLAY>;
  DFLASH_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::alloc));
  const long long items = (long long)a.B * a.Hv;
  const long long grid = items < (long long)sm_count() ? items : (long long)sm_count();
  kernel<<<(unsigned)grid, kThreads, L::alloc, stream>>>(map, a, status);
  DFLASH_LAUNCH_CHECK();
  count_launch();
  return DFLASH_OK;
}

}  // namespace

bool gdn_fast_supported(const GdnArgs& a) {
  if (a.Dk != kD || a.Dv != kD || a.g_is_vector || a.T > kTmax) return false;
  if ((long long)a.B * a.Hv > (1LL << 24) - 1024) return false;   // 32-bit item and TMA row arithmetic
  return a.in_dtype == DFLASH_F32 || a.in_dtype == DFLASH_BF16 || a.in_dtype == DFLASH_F16;
}

int32_t launch_gdn_fast(const GdnArgs& a, cudaStream_t stream) {
  switch (a.in_dtype) {
    case DFLASH_F32: return a.replay ? launch_typed<float, true>(a, stream) : launch_typed<float, false>(a, stream);
    case DFLASH_BF16: return a.replay ? launch_typed<__nv_bfloat16, true>(a, stream) : launch_typed<__nv_bfloat16, false>(a, stream);
    case DFLASH_F16: return a.replay ? launch_typed<__half, true>(a, stream) : launch_typed<__half, false>(a, stream);
    default: return DFLASH_ERR_UNSUPPORTED;
  }
}

}  // namespace dflash
