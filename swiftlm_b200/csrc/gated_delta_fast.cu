// Gated-delta forward with tape / tape replay for the production shape: Dk = Dv = 128,
// scalar or per-channel gate, T <= 16 (one DFlash verify block).  HBM-bound by design: the 64 KiB fp32 state of
// every (sequence, v-head) is read once and written once; everything else is small.
//
// Structure (persistent CTAs of 256 threads, two resident per SM for 16-bit inputs so that one
// CTA's load / store phases overlap the other's arithmetic):
//   * the state of the NEXT work item streams into shared memory by TMA (four 128-byte-swizzled
//     tensor tiles of 128 rows x 32 floats, completion on an mbarrier) while the current item is
//     computed from registers;
//   * the per-token inputs of the next item (k, q, v or the recorded delta) arrive by 16-byte
//     cp.async, only for the steps that will run, and are converted once to fp32 staging;
//   * each thread owns 4 rows x 16 columns of the state (64 floats in registers); a state row is
//     spread over 8 adjacent lanes and the four per-row sums of a step are reduced together in
//     4 shuffles; k stays in registers for both passes over the state;
//   * the state is carried as S = G * U with a running scalar G (product of the gates so far):
//       kv = G <U_row, k>,  delta = (v - kv) beta,  U_row += (delta / G) k,  y = G <U_row, q>
//     i.e. 3 packed fp32x2 fused multiply-adds per state element per step instead of 4; G is
//     folded back into U when it gets small (or a gate is exactly 0);
//   * with a per-channel gate (a [Dk] vector per step) the forward does the same with a vector of running products:
//     S = U diag(G_t), the products folded into the per-token vectors once per item (G_t k_t, k_t / G_t, G_t q_t), so the
//     recurrence keeps its 3 operations per element; an item whose product leaves [1e-12, 1e12] in any channel decays
//     its state column by column in the reference's own order instead (4 operations), as the replay always does, with
//     the gate rows kept in their input type in shared memory and widened as they are read;
//   * the new state leaves as full 128-byte lines; y and the tape are staged per warp and written
//     as 16-byte pieces.
// Work items are ordered so that consecutive items come from different sequences: accepted
// lengths differ per sequence, and mixing them keeps copy-only items (n = 0) and compute-heavy
// items (n = 16) overlapping on every SM.  The mbarrier wait is bounded; if it gives up the CTA
// sets the device status word and leaves.
//
// Reference semantics: Sources/DFlash/DFlashKernels.swift:122-199 (forward), :43-81 (replay),
// CPU statements :409-466 and :371-407; fp32 state without per-step rounding.
#include "common.cuh"
#include "ptx.cuh"

namespace dflash {
namespace {

constexpr int kD = 128;
constexpr int kTmax = 16;
constexpr int kThreads = 256;
constexpr uint32_t kStateBytes = kD * kD * 4;

template <typename InT, bool REPLAY, bool VEC>
struct Layout {
  static constexpr uint32_t in_row = kD * sizeof(InT);
  static constexpr uint32_t f32_tile = kTmax * kD * 4;
  static constexpr uint32_t state = 0;
  static constexpr uint32_t raw_k = kStateBytes;
  static constexpr uint32_t raw_q = raw_k + kTmax * in_row;                       // forward only
  static constexpr uint32_t raw_v = REPLAY ? raw_q : raw_q + kTmax * in_row;      // v (InT) or recorded delta (fp32)
  // per-channel gate only.  The replay reads the gate during the recurrence while the next item's inputs land: two
  // buffers.  The forward folds it into k and q before the recurrence starts: one.
  static constexpr bool kFolded = VEC && !REPLAY;
  static constexpr uint32_t raw_g = raw_v + kTmax * (REPLAY ? kD * 4 : in_row);
  static constexpr uint32_t raw_end = raw_g + (VEC ? (REPLAY ? 2 : 1) * kTmax * in_row : 0);
  static constexpr uint32_t k32 = raw_end;                                        // [16][128] fp32
  static constexpr uint32_t q32 = k32 + f32_tile;                                 // forward only
  static constexpr uint32_t d32 = REPLAY ? q32 : q32 + f32_tile;                  // [8 warps][16 steps][16 rows]: v / delta in; y out
  static constexpr uint32_t dout = d32 + f32_tile;                                // forward with a scalar gate: delta out; folded gate: k / G
  static constexpr uint32_t scal = REPLAY ? dout : dout + f32_tile;
  static constexpr uint32_t s_beta = scal;               // [3][16]
  static constexpr uint32_t s_g = s_beta + 3 * 16 * 4;   // [3][16]
  static constexpr uint32_t s_bits = s_g + 3 * 16 * 4;   // [4]
  static constexpr uint32_t s_bar = s_bits + 16;         // 8 bytes
  static constexpr uint32_t s_gt = s_bar + 16;           // folded gate only: [128] gate products of the whole block
  static constexpr uint32_t total = s_gt + (kFolded ? kD * 4 : 0);
  // Room to align the base to 1024 bytes, except where two CTAs of 16-bit inputs would no longer fit one SM with it:
  // there the kernel checks the alignment of the dynamic shared memory (it is the only shared memory of the kernel).
  static constexpr uint32_t slack = (kFolded && in_row == kD * 2) ? 0 : 1024;
  static constexpr uint32_t alloc = total + slack;
  static_assert(in_row != kD * 2 || 2 * (alloc + 1024) <= 233472, "two CTAs of 16-bit inputs per SM");
};

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }

template <typename InT> __device__ __forceinline__ void load8_as_f32(const InT* src, float (&o)[8]);
template <> __device__ __forceinline__ void load8_as_f32<float>(const float* src, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <> __device__ __forceinline__ void load8_as_f32<__nv_bfloat16>(const __nv_bfloat16* src, float (&o)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(src);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = __uint_as_float(w[i] << 16);
    o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <> __device__ __forceinline__ void load8_as_f32<__half>(const __half* src, float (&o)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(src);
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}
// four consecutive elements widened to two fp32 pairs
template <typename InT> __device__ __forceinline__ void load4_as_f32x2(const InT* src, float2 (&o)[2]);
template <> __device__ __forceinline__ void load4_as_f32x2<float>(const float* src, float2 (&o)[2]) {
  const float4 a = *reinterpret_cast<const float4*>(src);
  o[0] = make_float2(a.x, a.y);
  o[1] = make_float2(a.z, a.w);
}
template <> __device__ __forceinline__ void load4_as_f32x2<__nv_bfloat16>(const __nv_bfloat16* src, float2 (&o)[2]) {
  const uint2 u = *reinterpret_cast<const uint2*>(src);
  o[0] = make_float2(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u));
  o[1] = make_float2(__uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}
template <> __device__ __forceinline__ void load4_as_f32x2<__half>(const __half* src, float2 (&o)[2]) {
  const uint2 u = *reinterpret_cast<const uint2*>(src);
  o[0] = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
  o[1] = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
}
template <typename OutT> __device__ __forceinline__ void store8(OutT* dst, const float (&v)[8]);
template <> __device__ __forceinline__ void store8<float>(float* dst, const float (&v)[8]) {
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[8]) {
  __nv_bfloat162 p[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(p);
}
template <> __device__ __forceinline__ void store8<__half>(__half* dst, const float (&v)[8]) {
  __half2 p[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(p);
}

// Four per-row partial sums, each spread over the 8 lanes of a row group (lane bits 0-2).
// Transposed reduction in 4 shuffles: afterwards the lane with (bit0, bit1) = (i >> 1, i & 1)
// holds the complete sum of row slot i (both halves of the group hold a copy).
__device__ __forceinline__ float reduce4_over8(const float (&v)[4], int lane) {
  const bool b0 = lane & 1, b1 = lane & 2;
  const float s0 = b0 ? v[0] : v[2], s1 = b0 ? v[1] : v[3];
  const float k0 = (b0 ? v[2] : v[0]) + __shfl_xor_sync(0xffffffffu, s0, 1);
  const float k1 = (b0 ? v[3] : v[1]) + __shfl_xor_sync(0xffffffffu, s1, 1);
  float x = (b1 ? k1 : k0) + __shfl_xor_sync(0xffffffffu, b1 ? k0 : k1, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  return x;
}

template <typename InT, bool REPLAY, bool VEC>
__global__ void __launch_bounds__(kThreads, sizeof(InT) == 2 ? 2 : 1)
gdn_fast_kernel(const __grid_constant__ CUtensorMap state_map, const GdnArgs a, int* status) {
  using L = Layout<InT, REPLAY, VEC>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
  if (L::slack == 0 && sm != smem_raw) {   // no room to move the base: report and leave
    if (threadIdx.x == 0) atomicExch(status, kStatusSmemAlign);
    return;
  }
  constexpr bool kFolded = L::kFolded;

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int c_sub = lane & 7, r_sub = lane >> 3;   // 8 lanes share a state row; 4 row slots per warp
  const int T = a.T;
  const int rep = a.Hv / a.Hk;
  const uint32_t n_items = (uint32_t)a.B * (uint32_t)a.Hv;   // < 2^24: checked by the launcher
  const uint32_t G = gridDim.x;

  float* s_beta = reinterpret_cast<float*>(sm + L::s_beta);
  float* s_g = reinterpret_cast<float*>(sm + L::s_g);
  uint32_t* s_bits = reinterpret_cast<uint32_t*>(sm + L::s_bits);
  uint64_t* bar = reinterpret_cast<uint64_t*>(sm + L::s_bar);
  float* k32 = reinterpret_cast<float*>(sm + L::k32);
  float* q32 = reinterpret_cast<float*>(sm + L::q32);
  float* d32 = reinterpret_cast<float*>(sm + L::d32) + w * (kTmax * 16);   // this warp's [16 steps][16 rows]
  float* dout = reinterpret_cast<float*>(sm + L::dout) + w * (kTmax * 16);
  float* kh32 = reinterpret_cast<float*>(sm + L::dout);    // folded gate: [16][128] k / G
  float* s_gt = reinterpret_cast<float*>(sm + L::s_gt);

  const InT* gq = reinterpret_cast<const InT*>(a.q);
  const InT* gk = reinterpret_cast<const InT*>(a.k);
  const InT* gv = reinterpret_cast<const InT*>(a.v);
  const InT* gg = reinterpret_cast<const InT*>(a.g);
  const InT* gbeta = reinterpret_cast<const InT*>(a.beta);

  // item -> (sequence b, v-head hv): v-heads that share a qk-head are adjacent items, then the
  // sequence index varies fastest, the qk-head slowest.  32-bit unsigned arithmetic on purpose:
  // 64-bit division costs hundreds of instructions per item.
  auto decode = [&](uint32_t i, int& b, int& hv) {
    const uint32_t p = i / (uint32_t)rep, sub = i - p * (uint32_t)rep;
    const uint32_t hk = p / (uint32_t)a.B;
    b = (int)(p - hk * (uint32_t)a.B);
    hv = (int)(hk * (uint32_t)rep + sub);
  };
  auto step_on = [&](int b, int t) -> bool {
    bool on = true;
    if (a.n_per_seq) on = t < a.n_per_seq[(unsigned)b / (unsigned)a.n_div];
    if (on && a.mask) on = mask_on(a.mask, a.mask_dtype, b * T + t);
    return on;
  };
  // cp.async of the per-token inputs of item (b, hv) for the steps in `bits`
  auto issue_inputs = [&](int b, int hv, uint32_t bits, int gbuf) {
    const int hk = hv / rep;
    constexpr int cpr = L::in_row / 16;  // 16-byte chunks per k/q/v row
    for (int c = tid; c < kTmax * cpr; c += kThreads) {
      const int t = c / cpr, off = (c % cpr) * 16;
      if (t < T && ((bits >> t) & 1u)) {
        const long long bt = (long long)b * T + t;
        ptx::cp_async16(sm + L::raw_k + t * L::in_row + off, reinterpret_cast<const uint8_t*>(gk + (bt * a.Hk + hk) * kD) + off);
        if (VEC)
          ptx::cp_async16(sm + L::raw_g + ((kFolded ? 0 : gbuf) * kTmax + t) * L::in_row + off, reinterpret_cast<const uint8_t*>(gg + (bt * a.Hv + hv) * kD) + off);
        if (!REPLAY) {
          ptx::cp_async16(sm + L::raw_q + t * L::in_row + off, reinterpret_cast<const uint8_t*>(gq + (bt * a.Hk + hk) * kD) + off);
          ptx::cp_async16(sm + L::raw_v + t * L::in_row + off, reinterpret_cast<const uint8_t*>(gv + (bt * a.Hv + hv) * kD) + off);
        }
      }
    }
    if (REPLAY) {
      constexpr int cpr4 = kD * 4 / 16;
      for (int c = tid; c < kTmax * cpr4; c += kThreads) {
        const int t = c / cpr4, off = (c % cpr4) * 16;
        if (t < T && ((bits >> t) & 1u))
          ptx::cp_async16(sm + L::raw_v + t * (kD * 4) + off,
                          reinterpret_cast<const uint8_t*>(a.tape + (((long long)b * T + t) * a.Hv + hv) * kD) + off);
      }
    }
  };
  auto issue_state = [&](int b, int hv) {   // one thread
    ptx::mbar_arrive_expect_tx(bar, kStateBytes);
    const int row0 = (b * a.Hv + hv) * kD;
#pragma unroll
    for (int box = 0; box < 4; ++box)
      ptx::tma_load_2d(sm + L::state + box * (kD * 32 * 4), &state_map, box * 32, row0, bar);
  };

  // ---- prologue: barrier, step masks of the first two items, scalars and loads of the first ----
  if (tid == 0) {
    ptx::prefetch_tensormap(&state_map);
    ptx::mbar_init(bar, 1);
    ptx::fence_mbar_init();
  }
  uint32_t item = blockIdx.x;
  if (item >= n_items) return;
  int b_cur, hv_cur;
  decode(item, b_cur, hv_cur);
  if (w == 0) {
    bool on0 = false, on1 = false;
    if (lane < T) {
      on0 = step_on(b_cur, lane);
      if (item + G < n_items) {
        int b1, h1;
        decode(item + G, b1, h1);
        on1 = step_on(b1, lane);
      }
    }
    const uint32_t m0 = __ballot_sync(0xffffffffu, on0), m1 = __ballot_sync(0xffffffffu, on1);
    if (lane == 0) { s_bits[0] = m0; s_bits[1] = m1; }
  } else if (w == 1 && lane < T) {
    const long long bt = (long long)b_cur * T + lane;
    if (!VEC) s_g[lane] = to_f32(gg[bt * a.Hv + hv_cur]);
    if (!REPLAY) s_beta[lane] = to_f32(gbeta[bt * a.Hv + hv_cur]);
  }
  __syncthreads();
  if (tid == 0) issue_state(b_cur, hv_cur);
  issue_inputs(b_cur, hv_cur, s_bits[0], 0);
  ptx::cp_async_commit();

  const int col = 4 * c_sub;                                  // this thread's 4 columns inside each 32-column box
  const int my_i = 2 * (lane & 1) + ((lane >> 1) & 1);        // row slot whose reduced sums this lane ends up holding
  const int my_r = r_sub + 4 * my_i;                          // that row, relative to the warp's 16 rows

  uint32_t phase = 0;
  for (int it = 0;; ++it, item += G) {
    const uint32_t nxt = item + G, nxt2 = item + 2 * G;
    const bool has_next = nxt < n_items;
    int b_nxt = 0, hv_nxt = 0;
    if (has_next) decode(nxt, b_nxt, hv_nxt);

    // scalars needed one and two items ahead: issue the loads now, publish them at the end
    bool on2 = false;
    float g_next = 0.f, beta_next = 0.f;
    if (w == 0) {
      if (nxt2 < n_items && lane < T) {
        int b2, h2;
        decode(nxt2, b2, h2);
        on2 = step_on(b2, lane);
      }
    } else if (w == 1 && has_next && lane < T) {
      const long long bt = (long long)b_nxt * T + lane;
      if (!VEC) g_next = to_f32(gg[bt * a.Hv + hv_nxt]);
      if (!REPLAY) beta_next = to_f32(gbeta[bt * a.Hv + hv_nxt]);
    }

    // ---- wait for this item's state (TMA) and inputs (cp.async) ----
    const bool arrived = ptx::mbar_wait(bar, phase);
    phase ^= 1u;
    ptx::cp_async_wait_all();
    if (__syncthreads_or(!arrived)) {
      if (tid == 0) atomicExch(status, kStatusGdnWait);
      return;  // the wait budget ran out: report and leave
    }
    const uint32_t bits = s_bits[it % 3];
    const int slot = it % 3;

    // ---- inputs of the running steps -> fp32 staging; state -> registers ----
    {
      const int t = tid >> 4, seg = (tid & 15) * 8;
      if (t < T && ((bits >> t) & 1u)) {
        float x[8];
        if (!kFolded) {
          load8_as_f32<InT>(reinterpret_cast<const InT*>(sm + L::raw_k) + t * kD + seg, x);
          store8<float>(k32 + t * kD + seg, x);
        }
        float* dstage = reinterpret_cast<float*>(sm + L::d32) + (seg >> 4) * (kTmax * 16) + t * 16 + (seg & 15);
        if (!REPLAY) {
          if (!kFolded) {
            load8_as_f32<InT>(reinterpret_cast<const InT*>(sm + L::raw_q) + t * kD + seg, x);
            store8<float>(q32 + t * kD + seg, x);
          }
          load8_as_f32<InT>(reinterpret_cast<const InT*>(sm + L::raw_v) + t * kD + seg, x);
          store8<float>(dstage, x);
        } else {
          load8_as_f32<float>(reinterpret_cast<const float*>(sm + L::raw_v) + t * kD + seg, x);
          store8<float>(dstage, x);
        }
      }
    }
    // Per-channel gate, forward: the gates are folded into the per-token vectors once per item, so that the recurrence
    // is the scalar-gate one with G = 1.  With G_t the product of the gate rows of the running steps up to t and the
    // state carried as S = U diag(G_t):  kv = U (G_t k_t),  U += delta (k_t / G_t)^T,  y = U (G_t q_t),  and
    // S_T = U diag(G_T) at the end.  One thread per channel walks the steps (both halves of the CTA compute the products;
    // the lower half writes the two k tiles, the upper half q).  A product outside [1e-12, 1e12] in any channel (a gate
    // of zero, a long run of tiny gates) sends the item down the explicit route below.
    bool bad = false;
    if (kFolded) {
      const int c = tid & (kD - 1), hsel = tid >> 7;
      const InT* rg = reinterpret_cast<const InT*>(sm + L::raw_g) + c;
      const InT* rx = reinterpret_cast<const InT*>(sm + (hsel ? L::raw_q : L::raw_k)) + c;
      // all the loads first (bits has no step at or beyond T), then the chain of products
      float gv[kTmax], xv[kTmax];
#pragma unroll
      for (int t = 0; t < kTmax; ++t) {
        const bool on = (bits >> t) & 1u;
        gv[t] = on ? to_f32(rg[t * kD]) : 1.f;
        xv[t] = on ? to_f32(rx[t * kD]) : 0.f;
      }
      float Gc = 1.f, lo = 1.f, hi = 1.f;
#pragma unroll
      for (int t = 0; t < kTmax; ++t) {
        Gc *= gv[t];
        lo = fminf(lo, Gc);
        hi = fmaxf(hi, Gc);
        if ((bits >> t) & 1u) {
          if (hsel) {
            q32[t * kD + c] = xv[t] * Gc;
          } else {
            k32[t * kD + c] = xv[t] * Gc;
            kh32[t * kD + c] = __fdividef(xv[t], Gc);
          }
        }
      }
      bad = !(lo >= 1e-12f && hi <= 1e12f) || Gc != Gc;   // a product that is not a number stays one to the end
      if (!hsel) s_gt[c] = Gc;
    }
    // thread (r_sub, c_sub) owns rows 16w + r_sub + 4i (i < 4) and, in each 32-column box, the
    // 4 columns of 16-byte chunk c_sub: 64 floats.  A quarter warp reads 8 distinct chunks of
    // one row, so the swizzled tile is read without bank conflicts.
    float2 S[4][4][2];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = 16 * w + r_sub + 4 * i;
      const int phys = c_sub ^ (row & 7);  // 128-byte swizzle: chunk index xor (row mod 8)
#pragma unroll
      for (int box = 0; box < 4; ++box) {
        const float4 v4 = *reinterpret_cast<const float4*>(sm + L::state + box * (kD * 32 * 4) + row * 128 + phys * 16);
        S[i][box][0] = f2(v4.x, v4.y);
        S[i][box][1] = f2(v4.z, v4.w);
      }
    }
    // state tile and raw inputs are consumed: both may be refilled
    bool explicit_gate = false;
    if (kFolded) {
      explicit_gate = __syncthreads_or(bad);
      if (explicit_gate) {   // uniform: every step decays the state column by column; k and q as they are, the gate rows in the k / G tile
        const int c = tid & (kD - 1), hsel = tid >> 7;
        for (int t = 0; t < T; ++t) {
          if (!((bits >> t) & 1u)) continue;
          if (hsel) {
            q32[t * kD + c] = to_f32(reinterpret_cast<const InT*>(sm + L::raw_q)[t * kD + c]);
          } else {
            k32[t * kD + c] = to_f32(reinterpret_cast<const InT*>(sm + L::raw_k)[t * kD + c]);
            kh32[t * kD + c] = to_f32(reinterpret_cast<const InT*>(sm + L::raw_g)[t * kD + c]);
          }
        }
        __syncthreads();
      }
    } else {
      __syncthreads();
    }

    if (has_next) {
      if (tid == 0) issue_state(b_nxt, hv_nxt);
      issue_inputs(b_nxt, hv_nxt, s_bits[(it + 1) % 3], (it + 1) & 1);
    }
    ptx::cp_async_commit();

    // ---- the recurrence over the running steps (lazily decayed state, see the file header) ----
    float Gd = 1.f;
    for (int t = 0; t < T; ++t) {
      if (!((bits >> t) & 1u)) continue;
      float2 kk[4][2];
#pragma unroll
      for (int box = 0; box < 4; ++box) {
        const float4 k4 = *reinterpret_cast<const float4*>(k32 + t * kD + 32 * box + col);
        kk[box][0] = f2(k4.x, k4.y);
        kk[box][1] = f2(k4.z, k4.w);
      }
      // per-channel gate: this thread's 16 columns of the step's gate row, read box by box where they are used
      const InT* grow = (VEC && REPLAY) ? reinterpret_cast<const InT*>(sm + L::raw_g) + ((it & 1) * kTmax + t) * kD + col : nullptr;
      if (!VEC) Gd *= s_g[slot * 16 + t];
      if (!VEC && Gd < 1e-12f) {  // uniform per work item: U <- Gd * U, Gd <- 1
        const float2 G2 = f2(Gd, Gd);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int box = 0; box < 4; ++box)
#pragma unroll
            for (int j = 0; j < 2; ++j) S[i][box][j] = __fmul2_rn(G2, S[i][box][j]);
        Gd = 1.f;
      }
      const float inv_G = __fdividef(1.f, Gd);
      float d[4];
      if (REPLAY) {
#pragma unroll
        for (int i = 0; i < 4; ++i) d[i] = d32[t * 16 + r_sub + 4 * i] * inv_G;
#pragma unroll
        for (int box = 0; box < 4; ++box) {
          float2 gb[2];
          if (VEC) load4_as_f32x2<InT>(grow + 32 * box, gb);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 dd = f2(d[i], d[i]);
#pragma unroll
            for (int j = 0; j < 2; ++j)
              S[i][box][j] = __ffma2_rn(dd, kk[box][j], VEC ? __fmul2_rn(S[i][box][j], gb[j]) : S[i][box][j]);
          }
        }
      } else {
        const float beta = s_beta[slot * 16 + t];
        float part[4];
        if (kFolded && explicit_gate) {   // decay column by column first, as the reference does
#pragma unroll
          for (int box = 0; box < 4; ++box) {
            const float4 g4 = *reinterpret_cast<const float4*>(kh32 + t * kD + 32 * box + col);
            const float2 gb[2] = {f2(g4.x, g4.y), f2(g4.z, g4.w)};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int j = 0; j < 2; ++j) S[i][box][j] = __fmul2_rn(S[i][box][j], gb[j]);
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 acc0 = __fmul2_rn(S[i][0][0], kk[0][0]), acc1 = __fmul2_rn(S[i][0][1], kk[0][1]);
#pragma unroll
          for (int box = 1; box < 4; ++box) {
            acc0 = __ffma2_rn(S[i][box][0], kk[box][0], acc0);
            acc1 = __ffma2_rn(S[i][box][1], kk[box][1], acc1);
          }
          part[i] = (acc0.x + acc0.y) + (acc1.x + acc1.y);
        }
        const float kv = Gd * reduce4_over8(part, lane);
        const float d_mine = (d32[t * 16 + my_r] - kv) * beta;
        const float ds_mine = d_mine * inv_G;
#pragma unroll
        for (int i = 0; i < 4; ++i)  // lane holding row slot i inside this 8-lane group: bit0 = i >> 1, bit1 = i & 1
          d[i] = __shfl_sync(0xffffffffu, ds_mine, (lane & ~3) | ((i & 1) << 1) | (i >> 1));
        float2 acc[4][2];
#pragma unroll
        for (int box = 0; box < 4; ++box) {
          const float4 q4 = *reinterpret_cast<const float4*>(q32 + t * kD + 32 * box + col);
          const float2 qq[2] = {f2(q4.x, q4.y), f2(q4.z, q4.w)};
          float2 ku[2] = {kk[box][0], kk[box][1]};   // the update's k: k itself, or k / G where the gate is folded
          if (kFolded && !explicit_gate) {
            const float4 h4 = *reinterpret_cast<const float4*>(kh32 + t * kD + 32 * box + col);
            ku[0] = f2(h4.x, h4.y);
            ku[1] = f2(h4.z, h4.w);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 dd = f2(d[i], d[i]);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              S[i][box][j] = __ffma2_rn(dd, ku[j], S[i][box][j]);
              acc[i][j] = box == 0 ? __fmul2_rn(S[i][box][j], qq[j]) : __ffma2_rn(S[i][box][j], qq[j], acc[i][j]);
            }
          }
        }
        float y_part[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) y_part[i] = (acc[i][0].x + acc[i][0].y) + (acc[i][1].x + acc[i][1].y);
        const float y_mine = Gd * reduce4_over8(y_part, lane);
        if (!(lane & 4)) {  // lanes 0-3 of each 8-lane group hold the four rows' results
          d32[t * 16 + my_r] = y_mine;   // y takes the slot v was read from
          if (!VEC) dout[t * 16 + my_r] = d_mine;
          else if (a.tape)   // no staging tile in this variant: 16 lanes write the warp's 64 contiguous bytes of the step
            a.tape[(((long long)b_cur * T + t) * a.Hv + hv_cur) * kD + 16 * w + my_r] = d_mine;
        }
      }
    }
    if (kFolded && !explicit_gate) {   // S_T = U diag(G_T)
#pragma unroll
      for (int box = 0; box < 4; ++box) {
        const float4 g4 = *reinterpret_cast<const float4*>(s_gt + 32 * box + col);
        const float2 gb[2] = {f2(g4.x, g4.y), f2(g4.z, g4.w)};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 2; ++j) S[i][box][j] = __fmul2_rn(S[i][box][j], gb[j]);
      }
    }
    if (Gd != 1.f) {
      const float2 G2 = f2(Gd, Gd);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int box = 0; box < 4; ++box)
#pragma unroll
          for (int j = 0; j < 2; ++j) S[i][box][j] = __fmul2_rn(G2, S[i][box][j]);
    }

    // ---- new state: each warp instruction writes four full 128-byte lines ----
    {
      float* obase = a.state_out + ((long long)(b_cur * a.Hv + hv_cur) * kD + 16 * w + r_sub) * kD + col;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int box = 0; box < 4; ++box)
          *reinterpret_cast<float4*>(obase + (long long)(4 * i) * kD + 32 * box) =
              make_float4(S[i][box][0].x, S[i][box][0].y, S[i][box][1].x, S[i][box][1].y);
    }
    if (!REPLAY) {
      __syncwarp();
      const int t = lane >> 1, half = lane & 1;   // 16 steps x 2 halves of the warp's 16 rows
      if (t < T) {
        const bool on = (bits >> t) & 1u;
        float yv[8], dv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          yv[i] = on ? d32[t * 16 + 8 * half + i] : 0.f;
          dv[i] = (on && !VEC) ? dout[t * 16 + 8 * half + i] : 0.f;
        }
        const long long o = (((long long)b_cur * T + t) * a.Hv + hv_cur) * kD + 16 * w + 8 * half;
        store8<InT>(reinterpret_cast<InT*>(a.y) + o, yv);
        if (a.tape && (!VEC || !on)) store8<float>(a.tape + o, dv);
      }
    }

    // publish the scalars fetched at the top of the iteration
    if (w == 0) {
      const uint32_t m = __ballot_sync(0xffffffffu, on2);
      if (lane == 0) s_bits[(it + 2) % 3] = m;
    } else if (w == 1 && lane < T) {
      if (!VEC) s_g[((it + 1) % 3) * 16 + lane] = g_next;
      if (!REPLAY) s_beta[((it + 1) % 3) * 16 + lane] = beta_next;
    }
    if (!has_next) break;
    b_cur = b_nxt;
    hv_cur = hv_nxt;
  }
}

template <typename InT, bool REPLAY, bool VEC>
int32_t launch_variant(const GdnArgs& a, cudaStream_t stream) {
  using L = Layout<InT, REPLAY, VEC>;
  static_assert(sizeof(InT) != 2 || 2 * (L::alloc + 1024) <= 228 * 1024, "two CTAs of a 16-bit variant must fit one SM");
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
  const cuuint32_t box[2] = {32, (cuuint32_t)kD};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(a.state_in), dims, strides, box,
                            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled(state) failed with CUresult %d", (int)r);
    return DFLASH_ERR_CUDA;
  }
  auto kernel = gdn_fast_kernel<InT, REPLAY, VEC>;
  DFLASH_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::alloc));
  const long long items = (long long)a.B * a.Hv;
  const int per_sm = sizeof(InT) == 2 ? 2 : 1;
  const long long grid = items < (long long)sm_count() * per_sm ? items : (long long)sm_count() * per_sm;
  kernel<<<(unsigned)grid, kThreads, L::alloc, stream>>>(map, a, status);
  DFLASH_LAUNCH_CHECK();
  count_launch();
  return DFLASH_OK;
}

template <typename InT, bool REPLAY>
int32_t launch_typed(const GdnArgs& a, cudaStream_t stream) {
  return a.g_is_vector ? launch_variant<InT, REPLAY, true>(a, stream) : launch_variant<InT, REPLAY, false>(a, stream);
}

}  // namespace

bool gdn_fast_supported(const GdnArgs& a) {
  if (a.Dk != kD || a.Dv != kD || a.T > kTmax) return false;
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
