// Gated-delta forward with tape for one DFlash verify block on the tensor cores
// (Dk = Dv = 128, scalar gate, T <= 16, bf16 per-token inputs, fp32 state).
//
// The 16 steps of a block are not run one after another.  With S0 the incoming state, G_t the
// product of the gates up to step t and Gam[s,t] the product of the gates after s up to t, the
// recurrence  S <- g S;  delta = beta (v - S k);  S <- S + delta (x) k;  y = S q  unrolls to
//     kv_t    = G_t (S0 k_t) + sum_{s<t}  Gam[s,t] (k_s . k_t) delta_s
//     delta_t = beta_t (v_t - kv_t)
//     y_t     = G_t (S0 q_t) + sum_{s<=t} Gam[s,t] (k_s . q_t) delta_s
//     S_T     = G_T S0 + sum_s (Gam[s,T] delta_s) (x) k_s
// so the work on the 128 x 128 state becomes three small matrix products,
//     [S0 K^T | S0 Q^T]   128 x 128 x 32        (tcgen05, S0 split into two bf16 terms)
//     [K K^T  | K Q^T ]    16 x 128 x 32        (tcgen05, exact in fp32)
//     E K                 128 x  16 x 128       (tcgen05, E = Gam delta split into three bf16 terms)
// plus, per state row, a 16 x 16 unit-lower-triangular system (I + C) delta = r with
// C[t][s] = beta_t Gam[s,t] (k_s . k_t) and r_t = beta_t (v_t - G_t (S0 k_t)).  C is the same for the
// 128 rows of a head-state, so the scalar warp inverts it once (N = (I + C)^-1, and Z = Ckq N for the
// outputs) and every row gets delta = N r and y = G (S0 q) + Z r as independent dot products: no
// step of a row waits for the step before it.  A
// step that does not run (beyond the accepted length, or masked) gets gate 1 and beta 0: its
// delta is exactly 0, its y is forced to 0 and the state passes through it unchanged.
//
// S0 k and S0 q see S0 to 16 significant bits (2^-17 relative); the state itself is carried in
// fp32: S_T = G_T * S0 + (E K) with S0 read from the fp32 tile, and E is split exactly (24 bits).
// For a sequence with no running step the output state equals the input bit for bit.
//
// One persistent CTA per SM: eight compute warps, a scalar warp, a warp that issues the tensor-core products and a
// warp that issues the TMA loads.  Per work item (sequence, v-head), with the phases of neighbouring items interleaved:
//   load    loading warp, TMA: the fp32 state tile (four 128-byte-swizzled boxes) into one of two landing tiles,
//           issued two items ahead, as soon as the split has read the tile's previous contents: a state load is
//           in flight at all times.  K, Q rows of the block (swizzled, they are tensor-core operands as they
//           land) and V rows on a barrier of their own, also two items ahead
//   split   compute warps, two threads per state row: S0 -> two bf16 terms written to tensor memory, where they are
//           the A operand of TS-form products (nothing of the split passes through shared memory), and
//           G_T * S0 in fp32 -> the item's accumulator in tensor memory
//   mma     issuing warp: [S0 K^T | S0 Q^T] into tensor memory (first operand chunk while the split works
//           on the second); under the products the compute warps move the PREVIOUS item's finished state from
//           tensor memory to a staging tile, which a TMA store sends out
//   solve   two threads per state row, both from r: warps 0-3 form delta = N r, stage the tape rows and put
//           E into tensor memory as the A operand of the last product; warps 4-7 form y = G (S0 q) + Z r and
//           stage it over the item's V rows.  Outputs and tape leave by TMA stores after the barrier that ends the
//           solve (plain global stores from the SM are throttled while TMA traffic saturates the memory system)
//   mma     issuing warp: the accumulator += E K, then the next item's Gram products
//   tables  scalar warp: gates and betas of the item after the next fetched into registers, those of
//           the next item published; the next item's Gram rows out of tensor memory, scaled by the
//           gate products (and beta) into C and Ckq, then N (lanes 0-15, a row each) and Z (lanes
//           16-31, a row each) by one right-looking substitution over shuffles into the other table slot
// When no final state is wanted (state_out null: the verify step, whose result state is the rollback's) the
// accumulator, the E K product and the state's way out are skipped.
// Hand-offs that only one side waits for use named barriers (bar.arrive on the other side).
// Every wait is bounded; a wait that gives up sets the device status word and the CTA leaves.
//
// Reference semantics: Sources/DFlash/DFlashKernels.swift:122-199 (kernel), :409-466 (CPU statement).
#include <cuda.h>

#include "common.cuh"
#include "ptx.cuh"

#include "trace.cuh"

namespace dflash {
namespace {

constexpr int kD = 128;
constexpr int kT = 16;
constexpr int kComputeThreads = 256;
constexpr int kThreads = kComputeThreads + 96;   // + three helper warps: warp 8 scalars and tables, warp 9 tensor-core issue, warp 10 TMA loads
constexpr int kPairThreads = kComputeThreads + 32;   // participants of the compute <-> one-helper named barriers
constexpr int kTrioThreads = kComputeThreads + 64;   // compute <-> issuing and loading warps

// shared memory map (bytes); every tensor-core / TMA tile starts on a 1024-byte boundary
constexpr uint32_t kL = 0;                       // 2 x 64 KiB: landing tiles of the fp32 state [4 boxes][128 rows][32 floats]
constexpr uint32_t kY = 2 * 65536;               // 64 KiB: staging tile of the outgoing state, same layout
constexpr uint32_t kKQ = kY + 65536;             // 2 x 8 KiB: [2 chunks][32 rows: 16 k, 16 q][64]
constexpr uint32_t kV = kKQ + 2 * 8192;          // 2 x 4 KiB: [16 steps][128] bf16
constexpr uint32_t kTab = kV + 2 * 4096;         // 2 slots of coefficient tables
constexpr uint32_t kTabSlot = 2304;
constexpr uint32_t kTabKK = 0;                   //   [t][s] N = (I + C)^-1, C[t][s] = beta_t Gam[s,t] k_s.k_t (s < t), fp32
constexpr uint32_t kTabKQ = 1024;                //   [t][s] Z = Ckq N, Ckq[t][s] = Gam[s,t] k_s.q_t (s <= t)
constexpr uint32_t kTabGp = 2048;                //   [t] G_t
constexpr uint32_t kTabGe = 2048 + 64;           //   [s] Gam[s,T]
constexpr uint32_t kTabBG = 2048 + 128;          //   [t] beta_t G_t
constexpr uint32_t kScal = kTab + 2 * kTabSlot;  // 2 slots x { gate'[16], beta'[16], bits }
constexpr uint32_t kScalSlot = 160;
constexpr uint32_t kBars = kScal + 2 * kScalSlot;   // 8 mbarriers: state loads x 2, Gram, W, E K, K/Q/V loads x 2, first half of W
constexpr uint32_t kMisc = kBars + 64;              // tensor-memory base
constexpr uint32_t kSmemBytes = 226 * 1024;         // the Gram product reads 16 KiB past each K/Q chunk (rows it ignores)
static_assert(kMisc + 16 <= kSmemBytes, "shared memory map");
static_assert(kKQ + 8192 + 4096 + 16384 <= kSmemBytes, "Gram operand over-read stays inside the allocation");

constexpr uint32_t kStateBytes = 65536, kTokenBytes = 8192 + 4096;

// tensor memory columns
constexpr uint32_t kColW = 0;      // [S0 K^T | S0 Q^T]: 32
constexpr uint32_t kColGram = 32;  // 32
constexpr uint32_t kColE = 64;     // E as bf16 pairs: 3 x 8
constexpr uint32_t kColA = 96;     // S0 as bf16 pairs, the A operand of [S0 K^T | S0 Q^T]: hi 64 columns, lo 64
constexpr uint32_t kColD = 256;    // 2 x 128: the items' accumulators G_T S0 + E K
constexpr uint32_t kTmemCols = 512;

__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) |
         ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint32_t pack_rn(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// upper halves of two floats as a bf16 pair (truncation): a in the low half
__device__ __forceinline__ uint32_t pack_trunc(float a, float b) {
  return __byte_perm(__float_as_uint(a), __float_as_uint(b), 0x7632);
}
__device__ __forceinline__ float trunc16(float a) { return __uint_as_float(__float_as_uint(a) & 0xffff0000u); }

struct TcMaps {
  CUtensorMap state_in, state_out, k, q, v, y, tape;
};

__global__ void __launch_bounds__(kThreads, 1)
gdn_tc_kernel(const __grid_constant__ TcMaps maps, const GdnArgs a, int* status) {
  extern __shared__ __align__(1024) uint8_t sm[];
  if ((ptx::smem_u32(sm) & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicExch(status, kStatusSmemAlign);
    return;
  }
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const bool helper = w >= 8, aux = w == 8, mma = w == 9, ldw = w == 10;
  const int T = a.T;
  const int rep = a.Hv / a.Hk;
  const uint32_t n_items = (uint32_t)a.B * (uint32_t)a.Hv;
  // No final state wanted (the verify step, whose result state is the rollback's): nothing is accumulated into the
  // items' accumulators, no E K product, no state leaves the SM.
  const bool want_state = a.state_out != nullptr;
  const uint32_t G = gridDim.x;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kBars);   // 0,1: state loads; 2: Gram; 3: W; 4: E K; 5,6: K/Q/V loads; 7: first half of W
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + kMisc);
  const __nv_bfloat16* gg = reinterpret_cast<const __nv_bfloat16*>(a.g);
  const __nv_bfloat16* gbeta = reinterpret_cast<const __nv_bfloat16*>(a.beta);

  auto decode = [&](uint32_t i, int& b, int& hv) {   // 32-bit arithmetic on purpose
    const uint32_t p = i / (uint32_t)rep, sub = i - p * (uint32_t)rep;
    const uint32_t hk = p / (uint32_t)a.B;
    b = (int)(p - hk * (uint32_t)a.B);
    hv = (int)(hk * (uint32_t)rep + sub);
  };
  auto step_on = [&](int b, int t) -> bool {
    bool on = t < T;
    if (on && a.n_per_seq) on = t < a.n_per_seq[(unsigned)b / (unsigned)a.n_div];
    if (on && a.mask) on = mask_on(a.mask, a.mask_dtype, b * T + t);
    return on;
  };
  // scalars of item (b, hv): gate' (1 where the step does not run), beta' (0 there), step bits.
  // The helper warp fetches them into registers early and publishes them later.
  auto fetch_scalars = [&](int b, int hv, float& g, float& be, bool& on) {
    // all loads are issued before any is used: their latencies overlap
    const int t = lane < T ? lane : 0;
    const long long bt = (long long)b * T + t;
    const __nv_bfloat16 graw = gg[bt * a.Hv + hv], braw = gbeta[bt * a.Hv + hv];
    on = lane < kT && step_on(b, lane);
    g = on ? __bfloat162float(graw) : 1.f;
    be = on ? __bfloat162float(braw) : 0.f;
  };
  auto publish_scalars = [&](int slot, float g, float be, bool on) {
    const uint32_t m = __ballot_sync(0xffffffffu, on);
    float* sc = reinterpret_cast<float*>(sm + kScal + slot * kScalSlot);
    if (lane < kT) { sc[lane] = g; sc[16 + lane] = be; }
    if (lane == 0) reinterpret_cast<uint32_t*>(sc)[32] = m;
    __syncwarp();
  };
  // The boxes of an item are issued from several lanes of one warp (a single lane takes a few
  // hundred clocks per box).
  auto issue_state_load = [&](int b, int hv, int buf) {   // a whole warp
    void* bar = &bars[buf];
    if (lane == 0) ptx::mbar_arrive_expect_tx(bar, kStateBytes);
    __syncwarp();
    if (lane < 4) ptx::tma_load_2d(sm + kL + buf * 65536 + lane * 16384, &maps.state_in, lane * 32, (b * a.Hv + hv) * kD, bar);
    __syncwarp();
  };
  auto issue_token_loads = [&](int b, int hv, int buf) {   // a whole warp
    void* tbar = &bars[5 + buf];
    if (lane == 0) ptx::mbar_arrive_expect_tx(tbar, kTokenBytes);
    __syncwarp();
    const int hk = hv / rep;
    if (lane < 4) {
      const int c = lane >> 1;
      if (lane & 1) ptx::tma_load_4d(sm + kKQ + buf * 8192 + c * 4096 + 2048, &maps.q, c * 64, hk, 0, b, tbar);
      else ptx::tma_load_4d(sm + kKQ + buf * 8192 + c * 4096, &maps.k, c * 64, hk, 0, b, tbar);
    } else if (lane == 4) {
      ptx::tma_load_4d(sm + kV + buf * 4096, &maps.v, 0, hv, 0, b, tbar);
    }
    __syncwarp();
  };
  // instruction descriptors: fp32 accumulate, bf16 A and B, N >> 3, M >> 4 (and B MN-major for E K)
  constexpr uint32_t kIdescW = (1u << 4) | (1u << 7) | (1u << 10) | ((32u >> 3) << 17) | ((128u >> 4) << 24);
  constexpr uint32_t kIdescD = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
  // Gram products of the item in buffer buf: rows of [K; Q] against [K; Q]; only rows 0-15 (the k rows) are read back
  PH_DECL();
  auto issue_gram = [&](uint32_t tmem, int buf) {   // a whole warp, converged; lane 0 issues
    const uint32_t kq_addr = ptx::smem_u32(sm + kKQ + buf * 8192);
    const uint32_t leader = lane == 0;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint64_t d = make_desc(kq_addr + (kk >> 2) * 4096, 16, 1024) + 2 * (kk & 3);
      ptx::umma_ss_if(leader, tmem + kColGram, d, d, kIdescW, kk != 0);
    }
    ptx::umma_commit_if(leader, &bars[2]);
  };
  // the helper warp: Gram rows out of tensor memory, scaled by gate products (and beta), into table slot
  // The scalar warp: lane t < 16 holds row t of the Gram block K K^T (symmetric, so also its column) and lane
  // 16 + t row t of Q K^T.  Each lane scales its own row by gate products (and beta) into row t of C (lanes
  // 0-15) or of Ckq (lanes 16-31), then one right-looking substitution, the same for both halves, gives row t
  // of N = (I + C)^-1 (N (I + C) = I) and of Z = Ckq N (Z (I + C) = Ckq):
  //     acc[u] -= acc[s] C[s][u]   for s = 15 .. 1, u < s,
  // with row s of C broadcast from lane s by shuffles.  Nothing passes through shared memory but the results.
  auto build_tables = [&](uint32_t tmem, int slot) {
    uint32_t gr[32];
    ptx::tmem_ld32(tmem + kColGram, gr);   // lane t < 16: k_t.k_s (s < 16); lane 16 + t: q_t.k_s
    ptx::tmem_ld_wait();
    PH(9);
    const float* sc = reinterpret_cast<const float*>(sm + kScal + slot * kScalSlot);
    uint8_t* tab = sm + kTab + slot * kTabSlot;
    float gt[kT];
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const float4 g4 = reinterpret_cast<const float4*>(sc)[q4];
      gt[4 * q4] = g4.x; gt[4 * q4 + 1] = g4.y; gt[4 * q4 + 2] = g4.z; gt[4 * q4 + 3] = g4.w;
    }
    const int t = lane & 15;
    const bool pre = lane >= kT;
    const float beta_t = sc[16 + t];
    // row t: Gam[s,t] = g_{s+1} .. g_t, built downwards from s = t; prefix and suffix products of the gates
    float crow[kT], acc[kT];
    float gam = 1.f, g_pre = 1.f, g_suf = 1.f;
    const float scale = pre ? 1.f : beta_t;
#pragma unroll
    for (int s_ = kT - 1; s_ >= 0; --s_) {
      if (s_ < t) gam *= gt[s_ + 1 < kT ? s_ + 1 : kT - 1];
      const float wgt = s_ < t ? gam : (s_ == t && pre ? 1.f : 0.f);
      const float val = wgt * scale * __uint_as_float(gr[s_]);
      crow[s_] = val;
      acc[s_] = pre ? val : (s_ == t ? 1.f : 0.f);
      if (s_ <= t) g_pre *= gt[s_];
      else g_suf *= gt[s_];
    }
    if (!pre) {
      reinterpret_cast<float*>(tab + kTabGp)[t] = g_pre;
      reinterpret_cast<float*>(tab + kTabBG)[t] = beta_t * g_pre;
      reinterpret_cast<float*>(tab + kTabGe)[t] = g_suf;
    }
    PH(10);
#pragma unroll
    for (int s_ = kT - 1; s_ >= 1; --s_) {
      const float piv = acc[s_];
#pragma unroll
      for (int u = 0; u < s_; ++u) acc[u] = fmaf(-piv, __shfl_sync(0xffffffffu, crow[u], s_), acc[u]);
    }
    PH(11);
    float4* dst = reinterpret_cast<float4*>(tab + (pre ? kTabKQ : kTabKK)) + t * 4;
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) dst[q4] = make_float4(acc[4 * q4], acc[4 * q4 + 1], acc[4 * q4 + 2], acc[4 * q4 + 3]);
    ptx::tc_fence_before();
    __syncwarp();
  };

  // ---- prologue ----
  uint32_t item = blockIdx.x;
  if (tid == 0) {
    for (int i = 0; i < 8; ++i) ptx::mbar_init(&bars[i], 1);
    ptx::fence_mbar_init();
  }
  if (mma && lane == 0) {
    ptx::prefetch_tensormap(&maps.state_in);
    ptx::prefetch_tensormap(&maps.k);
    ptx::prefetch_tensormap(&maps.q);
    ptx::prefetch_tensormap(&maps.v);
    ptx::prefetch_tensormap(&maps.state_out);
    ptx::prefetch_tensormap(&maps.y);
    if (a.tape) ptx::prefetch_tensormap(&maps.tape);
  }
  if (aux) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  int b_cur = 0, hv_cur = 0;
  bool failed = false;
  __nv_bfloat16 h_g = __float2bfloat16(1.f), h_b = __float2bfloat16(0.f);   // scalar warp: gate / beta of the next item
  int h_n = 0;       // its accepted length, compared only when published (the load has a whole iteration to land)
  bool h_m = false;  // its mask bit
  if (item < n_items) {
    decode(item, b_cur, hv_cur);
    if (ldw) {
      issue_token_loads(b_cur, hv_cur, 0);
      issue_state_load(b_cur, hv_cur, 0);
      if (item + G < n_items) {
        int b1, hv1;
        decode(item + G, b1, hv1);
        issue_token_loads(b1, hv1, 1);
        issue_state_load(b1, hv1, 1);
      }
    } else if (mma) {
      failed = !ptx::mbar_wait(&bars[5], 0);
      ptx::tc_fence_after();
      issue_gram(tmem, 0);
      __syncwarp();
    } else if (aux) {
      float g0, be0;
      bool on0;
      fetch_scalars(b_cur, hv_cur, g0, be0, on0);
      publish_scalars(0, g0, be0, on0);
      if (item + G < n_items) {
        int b1, hv1;
        decode(item + G, b1, hv1);
        const long long bt = (long long)b1 * T + (lane < T ? lane : 0);
        h_g = gg[bt * a.Hv + hv1];
        h_b = gbeta[bt * a.Hv + hv1];
        h_n = a.n_per_seq ? a.n_per_seq[(unsigned)b1 / (unsigned)a.n_div] : T;
        h_m = lane < T && (!a.mask || mask_on(a.mask, a.mask_dtype, b1 * T + lane));
      }
      failed = !ptx::mbar_wait(&bars[2], 0);
      ptx::tc_fence_after();
      build_tables(tmem, 0);
    }
  }
  __syncthreads();   // the first item's scalars and tables are in place
  if (aux && item < n_items) asm volatile("bar.arrive 4, %0;" ::"n"(kPairThreads) : "memory");

  const int row = 32 * (w & 3) + lane;               // state row = tensor-memory lane of this thread
  const uint32_t lane_addr = (uint32_t)(32 * (w & 3)) << 16;
  const int half = (w >> 2) & 1;                      // which 64 state columns this thread handles in the output pass
  uint32_t gram_uses = 1;                             // phases of the Gram barrier consumed so far (helper warp)

  // previous item's finished state: tensor memory -> staging tile -> TMA store (compute warps)
  // The staging tile is free when this starts: the lanes that issued its previous store waited for that store's read
  // just before the barrier that ended the previous iteration.  With a tape, the previous item's tape rows left from
  // the head of the tile by a store issued AFTER that barrier: it is waited for here, and everyone is told.
  auto flush_state = [&](int dbuf, int b, int hv, uint32_t ek_parity) -> bool {
    if (a.tape && tid < 4) ptx::bulk_wait_read_all();
    bool ok = ptx::mbar_wait(&bars[4], ek_parity);
    ptx::tc_fence_after();
    if (a.tape) asm volatile("bar.sync 1, %0;" ::"n"(kComputeThreads) : "memory");
    PH(10);
    {   // both 32-column reads in flight before either is waited for
      uint32_t dr[2][32];
      ptx::tmem_ld32(tmem + lane_addr + kColD + 128 * dbuf + 64 * half, dr[0]);
      ptx::tmem_ld32(tmem + lane_addr + kColD + 128 * dbuf + 64 * half + 32, dr[1]);
      ptx::tmem_ld_wait();
#pragma unroll
      for (int bb = 0; bb < 2; ++bb)
#pragma unroll
        for (int g = 0; g < 8; ++g)
          *reinterpret_cast<uint4*>(sm + kY + (2 * half + bb) * 16384 + row * 128 + ((g ^ (row & 7)) << 4)) =
              make_uint4(dr[bb][4 * g], dr[bb][4 * g + 1], dr[bb][4 * g + 2], dr[bb][4 * g + 3]);
    }
    ptx::fence_proxy_async();
    ptx::tc_fence_before();
    asm volatile("bar.sync 1, %0;" ::"n"(kComputeThreads) : "memory");
    if (tid < 4) {   // one box per lane: a single lane takes a few hundred clocks per box
      const int row0 = (b * a.Hv + hv) * kD;
      ptx::tma_store_2d(&maps.state_out, tid * 32, row0, sm + kY + tid * 16384);
      ptx::bulk_commit_group();
    }
    PH(11);
    return ok;
  };

  int b_prev = 0, hv_prev = 0, it = 0;
  for (; item < n_items; ++it, item += G) {
    const int buf = it & 1;
    const uint32_t par = (uint32_t)it & 1u;
    const uint32_t nxt = item + G;
    const bool has_next = nxt < n_items;
    int b_nxt = 0, hv_nxt = 0;
    if (has_next) decode(nxt, b_nxt, hv_nxt);
    uint8_t* KQ = sm + kKQ + buf * 8192;
    const float* sc = reinterpret_cast<const float*>(sm + kScal + buf * kScalSlot);
    const uint8_t* tab = sm + kTab + buf * kTabSlot;

    // ---- this item's state, K, Q, V have landed ----
    if (!helper) failed = !ptx::mbar_wait(&bars[buf], (uint32_t)(it >> 1) & 1u);
    PH(0);

    // ---- split: S0 = hi + lo + (dropped 2^-17), both bf16, into tensor memory; G_T S0 -> this item's accumulator ----
    if (!helper) {
      float g_T = 1.f;
#pragma unroll
      for (int t = 0; t < kT; ++t) g_T *= sc[t];
#pragma unroll
      for (int pass = 0; pass < 2; ++pass) {
        const int box = 2 * pass + half;                // 32 state columns; pass = operand chunk (64 columns)
        float4 x4[8];
#pragma unroll
        for (int g = 0; g < 8; ++g)
          x4[g] = *reinterpret_cast<const float4*>(sm + kL + buf * 65536 + box * 16384 + row * 128 + ((g ^ (row & 7)) << 4));
        if (want_state) {
          uint32_t acc[32];
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            acc[4 * g] = __float_as_uint(g_T * x4[g].x);
            acc[4 * g + 1] = __float_as_uint(g_T * x4[g].y);
            acc[4 * g + 2] = __float_as_uint(g_T * x4[g].z);
            acc[4 * g + 3] = __float_as_uint(g_T * x4[g].w);
          }
          ptx::tmem_st32(tmem + lane_addr + kColD + 128 * buf + 32 * box, acc);
        }
        // the operand in tensor memory: a column holds two neighbouring state columns as a bf16 pair
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float x[4] = {x4[g].x, x4[g].y, x4[g].z, x4[g].w};
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            hi[2 * g + i] = pack_trunc(x[2 * i], x[2 * i + 1]);
            lo[2 * g + i] = pack_rn(x[2 * i] - trunc16(x[2 * i]), x[2 * i + 1] - trunc16(x[2 * i + 1]));
          }
        }
        ptx::tmem_st16(tmem + lane_addr + kColA + 16 * box, hi);
        ptx::tmem_st16(tmem + lane_addr + kColA + 64 + 16 * box, lo);
        if (pass == 0) {
          // the first chunk is complete: its eight products can run under the second pass (named barrier 5)
          ptx::tmem_st_wait();
          ptx::tc_fence_before();
          asm volatile("bar.arrive 5, %0;" ::"n"(kPairThreads) : "memory");
        }
      }
      ptx::tmem_st_wait();
    } else if (mma) {
      asm volatile("bar.sync 5, %0;" ::"n"(kPairThreads) : "memory");
      {
        ptx::tc_fence_after();
        const uint32_t kq_addr = ptx::smem_u32(KQ), leader = lane == 0;
#pragma unroll
        for (int sp = 0; sp < 2; ++sp)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t db = make_desc(kq_addr, 16, 1024) + 2 * kk;
            ptx::umma_ts_if(leader, tmem + kColW, tmem + kColA + 64 * sp + 8 * kk, db, kIdescW, (sp | kk) != 0);
          }
      }
      __syncwarp();
    }
    ptx::tc_fence_before();
    PH(1);
    // split -> products and next loads: the compute warps only signal, the issuing and loading warps wait (named barrier 3);
    // the scalar warp has no part in it: it only ever writes the table and scalar slots of the NEXT item
    if (mma || ldw) asm volatile("bar.sync 3, %0;" ::"n"(kTrioThreads) : "memory");
    else if (!helper) asm volatile("bar.arrive 3, %0;" ::"n"(kTrioThreads) : "memory");
    PH(2);

    if (mma) {
      // ---- issuing warp: the second chunk's products ----
      {
        ptx::tc_fence_after();
        const uint32_t kq_addr = ptx::smem_u32(KQ), leader = lane == 0;
#pragma unroll
        for (int sp = 0; sp < 2; ++sp)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t db = make_desc(kq_addr + 4096, 16, 1024) + 2 * kk;
            ptx::umma_ts_if(leader, tmem + kColW, tmem + kColA + 64 * sp + 32 + 8 * kk, db, kIdescW, 1u);
          }
        ptx::umma_commit_if(leader, &bars[3]);
      }
      __syncwarp();
      // the next item's Gram products: its K, Q rows landed an iteration ago, and the scalar warp read the
      // previous Gram block before the barrier that ended the previous iteration
      if (has_next) {
        failed = !ptx::mbar_wait(&bars[5 + (buf ^ 1)], (uint32_t)((it + 1) >> 1) & 1u) || failed;
        ptx::tc_fence_after();
        issue_gram(tmem, buf ^ 1);
        __syncwarp();
      }
    } else if (ldw) {
      // ---- loading warp: the state of the item after the next into this item's landing tile (free again) ----
      if (nxt + G < n_items) {
        int b2, hv2;
        decode(nxt + G, b2, hv2);
        issue_state_load(b2, hv2, buf);
      }
    } else if (aux) {
      // ---- scalar warp: the next item's gates, betas and step bits ----
      if (has_next) {
        const bool h_on = h_m && lane < h_n;
        publish_scalars(buf ^ 1, h_on ? __bfloat162float(h_g) : 1.f, h_on ? __bfloat162float(h_b) : 0.f, h_on);
      }
      // gates and betas of the item after the next: in registers until the next iteration publishes them
      if (nxt + G < n_items) {
        int b2, hv2;
        decode(nxt + G, b2, hv2);
        const long long bt = (long long)b2 * T + (lane < T ? lane : 0);
        h_g = gg[bt * a.Hv + hv2];
        h_b = gbeta[bt * a.Hv + hv2];
        h_n = a.n_per_seq ? a.n_per_seq[(unsigned)b2 / (unsigned)a.n_div] : T;
        h_m = lane < T && (!a.mask || mask_on(a.mask, a.mask_dtype, b2 * T + lane));
      }
      PH(8);
    } else {
      // ---- compute warps, under the helper's products: the previous item's state goes out ----
      if (want_state && it > 0 && !flush_state(buf ^ 1, b_prev, hv_prev, par ^ 1u)) failed = true;
      // this item's tables are in place (named barriers 4 and 6 alternate: the scalar warp signals the next
      // item's tables before this item's have been waited for)
      if (buf) asm volatile("bar.sync 6, %0;" ::"n"(kPairThreads) : "memory");
      else asm volatile("bar.sync 4, %0;" ::"n"(kPairThreads) : "memory");
    }
    PH(3);

    // ---- solve: two threads per state row, both from r_t = beta_t v_t - beta_t G_t (S0 k_t).  Warps 0-3 form
    //      delta = N r, build E and write the tape; warps 4-7 form y = G (S0 q) + Z r.  A step that does not run
    //      has beta' = 0, hence r = 0, and is skipped: its delta and its y are exactly 0 ----
    float outv[kT];
    if (!helper) {
      failed = !ptx::mbar_wait(&bars[3], par) || failed;
      failed = !ptx::mbar_wait(&bars[5 + buf], (uint32_t)(it >> 1) & 1u) || failed;
      ptx::tc_fence_after();
      uint32_t wr[32];
      ptx::tmem_ld32(tmem + lane_addr + kColW, wr);   // S0 k_t (t < 16), S0 q_t
      ptx::tmem_ld_wait();
      PH(9);
      const uint32_t bits = reinterpret_cast<const uint32_t*>(sc)[32];
      const __nv_bfloat16* vt = reinterpret_cast<const __nv_bfloat16*>(sm + kV + buf * 4096);
      float r[kT];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const float4 bg4 = reinterpret_cast<const float4*>(tab + kTabBG)[q4], be4 = reinterpret_cast<const float4*>(sc + 16)[q4];
        const float bgv[4] = {bg4.x, bg4.y, bg4.z, bg4.w}, bev[4] = {be4.x, be4.y, be4.z, be4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int t = 4 * q4 + e;
          r[t] = fmaf(-bgv[e], __uint_as_float(wr[t]), bev[e] * __bfloat162float(vt[t * kD + row]));
        }
      }
      // every row's r is formed: nothing reads this item's V rows any more, the outputs are staged over them
      asm volatile("bar.sync 7, %0;" ::"n"(kComputeThreads) : "memory");
      // rows 4 g4 .. 4 g4 + 3 of a lower-triangular table against r: eight independent partial sums.  A group
      // in which no step runs is skipped (uniform over the CTA); a step that does not run inside a running
      // group has r = 0 and a unit row of N: its delta comes out as exactly 0, its y is forced to 0.
      auto tri_rows = [&](const float4* table, int g4, const float (&first)[4], float (&out)[4]) {
        float a0[4] = {first[0], first[1], first[2], first[3]}, a1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4)
          if (q4 <= g4) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float4 c = table[(4 * g4 + e) * 4 + q4];
              const float cv[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
              for (int x = 0; x < 4; ++x)
                if (4 * q4 + x <= 4 * g4 + e) {
                  if (x & 1) a1[e] = fmaf(cv[x], r[4 * q4 + x], a1[e]);
                  else a0[e] = fmaf(cv[x], r[4 * q4 + x], a0[e]);
                }
            }
          }
#pragma unroll
        for (int e = 0; e < 4; ++e) out[e] = a0[e] + a1[e];
      };
      const float zero4[4] = {0.f, 0.f, 0.f, 0.f};
      if (w < 4) {
        const float4* tn = reinterpret_cast<const float4*>(tab + kTabKK);
        float (&d)[kT] = outv;
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) {
          float o[4] = {0.f, 0.f, 0.f, 0.f};
          if ((bits >> (4 * g4)) & 0xFu) tri_rows(tn, g4, zero4, o);
#pragma unroll
          for (int e = 0; e < 4; ++e) d[4 * g4 + e] = o[e];
        }
        PH(4);
        // E = Gam[s,T] delta_s, split exactly into three bf16 terms, as the A operand (pairs of steps per column)
        if (want_state) {
          const float* ge = reinterpret_cast<const float*>(tab + kTabGe);
          uint32_t er[32];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float e0 = ge[2 * c] * d[2 * c], e1 = ge[2 * c + 1] * d[2 * c + 1];
            const float r0 = e0 - trunc16(e0), r1 = e1 - trunc16(e1);
            er[c] = pack_trunc(e0, e1);
            er[8 + c] = pack_trunc(r0, r1);
            er[16 + c] = pack_rn(r0 - trunc16(r0), r1 - trunc16(r1));
            er[24 + c] = 0u;
          }
          ptx::tmem_st32(tmem + lane_addr + kColE, er);
        }
        PH(14);
        if (a.tape) {
          // the tape rows are staged at the head of the state's staging tile, once the previous state's
          // store has read it (it was issued a whole flush ago), and leave with a TMA store after the barrier
          if (tid < 4) ptx::bulk_wait_read_all();
          asm volatile("bar.sync 8, 128;" ::: "memory");
          float* stage = reinterpret_cast<float*>(sm + kY);
#pragma unroll
          for (int t = 0; t < kT; ++t) stage[t * kD + row] = d[t];
          ptx::fence_proxy_async();
        }
        ptx::tmem_st_wait();
        ptx::tc_fence_before();
      } else {
        const float4* tz = reinterpret_cast<const float4*>(tab + kTabKQ);
        const float* gp = reinterpret_cast<const float*>(tab + kTabGp);
        float (&yv)[kT] = outv;
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) {
          float o[4] = {0.f, 0.f, 0.f, 0.f};
          if ((bits >> (4 * g4)) & 0xFu) {
            const float4 gp4 = reinterpret_cast<const float4*>(gp)[g4];
            const float y0[4] = {gp4.x * __uint_as_float(wr[16 + 4 * g4]), gp4.y * __uint_as_float(wr[17 + 4 * g4]),
                                 gp4.z * __uint_as_float(wr[18 + 4 * g4]), gp4.w * __uint_as_float(wr[19 + 4 * g4])};
            tri_rows(tz, g4, y0, o);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) yv[4 * g4 + e] = ((bits >> (4 * g4 + e)) & 1u) ? o[e] : 0.f;
        }
        PH(14);
        __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(sm + kV + buf * 4096);
#pragma unroll
        for (int t = 0; t < kT; ++t) stage[t * kD + row] = __float2bfloat16_rn(yv[t]);
        ptx::fence_proxy_async();
      }
    }
    PH(5);
    // the previous state's store, issued in this iteration, has read the staging tile by now; after the barrier every
    // thread may write there again (one barrier fewer at the start of the next flush)
    if (tid < 4) ptx::bulk_wait_read_all();
    if (__syncthreads_or(failed)) { failed = true; break; }
    PH(6);

    // ---- issuing warp: accumulator += E K, then the next item's Gram products; scalar warp: its tables ----
    if (mma) {
      if (want_state) {
        ptx::tc_fence_after();
        // k rows 0-15 of both chunks as an MN-major operand: 64-column atoms 4096 bytes apart, 8-step groups 1024 apart
        const uint64_t db = make_desc(ptx::smem_u32(KQ), 4096, 1024);
        const uint32_t dcol = tmem + kColD + 128 * buf, leader = lane == 0;
        ptx::umma_ts_if(leader, dcol, tmem + kColE, db, kIdescD, 1u);
        ptx::umma_ts_if(leader, dcol, tmem + kColE + 8, db, kIdescD, 1u);
        ptx::umma_ts_if(leader, dcol, tmem + kColE + 16, db, kIdescD, 1u);
        ptx::umma_commit_if(leader, &bars[4]);
      }
      __syncwarp();
    } else if (ldw) {
      // this item's outputs leave from its V buffer
      if (lane == 0) {
        ptx::tma_store_4d(&maps.y, 0, hv_cur, 0, b_cur, sm + kV + buf * 4096);
        ptx::bulk_commit_group();
      }
      // K, Q, V of the item after the next go into this item's buffers as soon as E K has read its K rows and
      // the store above its V buffer (every other reader of them finished before the barrier above): a whole
      // iteration ahead of their use
      if (nxt + G < n_items) {
        if (want_state) failed = !ptx::mbar_wait(&bars[4], par) || failed;
        if (lane == 0) ptx::bulk_wait_read_all();
        __syncwarp();
        int b2, hv2;
        decode(nxt + G, b2, hv2);
        issue_token_loads(b2, hv2, buf);
      }
    } else if (!helper) {
      if (tid == 0 && a.tape) {   // steps past T fall outside the tensor and are dropped by the store
        ptx::tma_store_4d(&maps.tape, 0, hv_cur, 0, b_cur, sm + kY);
        ptx::bulk_commit_group();
      }
    } else if (aux && has_next) {
      // the next item's tables: its Gram products were issued behind this item's second chunk
      failed = !ptx::mbar_wait(&bars[2], gram_uses & 1u);
      ++gram_uses;
      ptx::tc_fence_after();
      PH(12);
      build_tables(tmem, buf ^ 1);
      PH(13);
      __threadfence_block();
      if (buf) asm volatile("bar.arrive 4, %0;" ::"n"(kPairThreads) : "memory");
      else asm volatile("bar.arrive 6, %0;" ::"n"(kPairThreads) : "memory");
    }
    PH(7);
    b_prev = b_cur;
    hv_prev = hv_cur;
    b_cur = b_nxt;
    hv_cur = hv_nxt;
  }
  // the last item's state
  if (want_state && !failed && it > 0 && !helper) {
    if (!flush_state((it - 1) & 1, b_prev, hv_prev, (uint32_t)(it - 1) & 1u)) failed = true;
  }

  PH_FLUSH();
  if (failed && lane == 0) atomicExch(status, kStatusGdnWait);
  if (tid < 4 || (ldw && lane == 0)) ptx::bulk_wait_all();    // shared memory must outlive the last stores
  ptx::tc_fence_before();
  __syncthreads();
  if (aux) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace

bool gdn_tc_supported(const GdnArgs& a) {
  if (a.replay || a.Dk != kD || a.Dv != kD || a.g_is_vector || a.T > kT || a.T < 1) return false;
  if (a.in_dtype != DFLASH_BF16) return false;
  if ((long long)a.B * a.Hv > (1LL << 24) - 1024) return false;
  if (a.Hv % a.Hk != 0) return false;
  // TMA needs 16-byte aligned bases
  // state_out may be null (internal callers only): no final state is produced
  const uintptr_t al = (uintptr_t)a.q | (uintptr_t)a.k | (uintptr_t)a.v | (uintptr_t)a.state_in | (uintptr_t)a.state_out |
                       (uintptr_t)a.y | (uintptr_t)a.tape;
  return (al & 15u) == 0;
}

int32_t launch_gdn_tc(const GdnArgs& a, cudaStream_t stream) {
  EncodeTiledFn encode = tensor_map_encoder();
  if (!encode) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return DFLASH_ERR_CUDA; }
  int* status = device_status_word();
  if (!status) { set_error("no CUDA device"); return DFLASH_ERR_CUDA; }
  TcMaps maps;
  const cuuint32_t ones[4] = {1, 1, 1, 1};
  auto state_map = [&](CUtensorMap* m, const float* base) {
    const cuuint64_t dims[2] = {(cuuint64_t)kD, (cuuint64_t)a.B * a.Hv * kD};
    const cuuint64_t strides[1] = {(cuuint64_t)kD * 4};
    const cuuint32_t box[2] = {32, (cuuint32_t)kD};
    return encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, ones,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  // per-token tensors [B, T, H, 128] as (d, h, t, b); one box = the 16 steps of one head (rows past T read as zeros)
  auto token_map = [&](CUtensorMap* m, const void* base, int H, int box_d, CUtensorMapSwizzle sw) {
    const cuuint64_t dims[4] = {(cuuint64_t)kD, (cuuint64_t)H, (cuuint64_t)a.T, (cuuint64_t)a.B};
    const cuuint64_t strides[3] = {(cuuint64_t)kD * 2, (cuuint64_t)H * kD * 2, (cuuint64_t)a.T * H * kD * 2};
    const cuuint32_t box[4] = {(cuuint32_t)box_d, 1, (cuuint32_t)kT, 1};
    return encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, ones,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = state_map(&maps.state_in, a.state_in);
  if (r == CUDA_SUCCESS) r = state_map(&maps.state_out, a.state_out ? a.state_out : a.state_in);   // never used when there is no output
  if (r == CUDA_SUCCESS) r = token_map(&maps.k, a.k, a.Hk, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r == CUDA_SUCCESS) r = token_map(&maps.q, a.q, a.Hk, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r == CUDA_SUCCESS) r = token_map(&maps.v, a.v, a.Hv, 128, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (r == CUDA_SUCCESS) r = token_map(&maps.y, a.y, a.Hv, 128, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (r == CUDA_SUCCESS && a.tape) {
    const cuuint64_t dims[4] = {(cuuint64_t)kD, (cuuint64_t)a.Hv, (cuuint64_t)a.T, (cuuint64_t)a.B};
    const cuuint64_t strides[3] = {(cuuint64_t)kD * 4, (cuuint64_t)a.Hv * kD * 4, (cuuint64_t)a.T * a.Hv * kD * 4};
    const cuuint32_t box[4] = {(cuuint32_t)kD, 1, (cuuint32_t)kT, 1};
    r = encode(&maps.tape, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.tape, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r); return DFLASH_ERR_CUDA; }
  DFLASH_CUDA_CHECK(cudaFuncSetAttribute(gdn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
  const long long items = (long long)a.B * a.Hv;
  const long long grid = items < (long long)sm_count() ? items : (long long)sm_count();
  gdn_tc_kernel<<<(unsigned)grid, kThreads, kSmemBytes, stream>>>(maps, a, status);
  DFLASH_LAUNCH_CHECK();
  count_launch();
  return DFLASH_OK;
}

}  // namespace dflash
