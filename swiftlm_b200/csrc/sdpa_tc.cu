// Block-verify attention on the 5th-generation tensor cores (tcgen05 + tensor memory).
//
// Shape of the problem: per (sequence, KV head) the 16 draft tokens of the G = Hq/Hkv grouped
// query heads form one M = 16*G row tile (128 rows for G = 8) that attends to N keys: every K/V
// byte is read from HBM exactly once per KV head.  At bf16 KV the shape is HBM-bound
// (128 FLOP/B), so the kernel is organised around keeping TMA loads in flight; the tensor
// pipe and the softmax run in the shadow of the loads.
//
// One persistent CTA per SM (cta_group::1, no multicast; the cluster-pair split regime below launches
// two-CTA clusters that exchange through distributed shared memory), 10 warps:
//   warp 0     TMA producer: Q tile (4 boxes of 128 rows x 64 elements) and a ring of 16 KiB
//              K / V boxes (128 keys x 64 elements, 128-byte swizzle), order K0 K1 V0 K2 V1 ...
//   warp 1     MMA issuer (one lane): S = Q K^T (128 x 128 x D, both operands in shared memory,
//              K-major) into one of two S buffers in tensor memory; O += P V with P read from
//              tensor memory (bf16, aliasing the S buffer) and V MN-major from shared memory.
//              Owns the tensor-memory allocation.
//   warps 2-9  softmax: two threads per query row (64 key columns each).  Loads its part of S,
//              adds the additive mask if there is one (a second instantiation of the kernel; the
//              thread's 64 mask values of a tile are fetched before it waits for S, rows read
//              16 bytes at a time when N is a multiple of 8; an entry below the dtype's lowest
//              finite value hides the key), applies the block-causal rule on the last tiles, keeps a running reference
//              maximum and sum, writes P (bf16) back to tensor memory, rescales O only when the
//              maximum grew by more than 2^8, and at the end of a segment normalises and stores.
// KV is split across CTAs stream-K style: the (unit, 128-key tile) pairs of the whole batch
// are cut into one contiguous range per CTA, so every CTA streams the same number of tiles.
// A range that covers a whole unit writes the output directly; the others write fp32 partials
// (unnormalised O, reference maximum, sum).  Where a unit is cut into at most kFusedMax ranges
// the CTA that finishes last merges them itself: every range publishes a per-launch tag in an
// arrival flag after its partials, then looks at the flags of the unit's other ranges; whoever
// sees them all set does the merge (two CTAs finishing together may both do it and store the same
// bytes).  Nobody waits for anybody.  Units cut into more ranges (long context, small batch) are
// merged by a second kernel with one block per 16 rows.  When the units divide the SMs well
// (units * c >= 80 % of the SMs for an integer c <= kFusedMax) every unit is cut into exactly c
// equal ranges instead, so that no CTA pays for two range epilogues.
//
// Semantics: Sources/DFlash/DFlashKernels.swift:563-649 (partials) and :661-720 (reduce):
// visibility n <= N_b - 16 + r, fp32 scores and accumulation, zero-sum guard.  Differences:
// contiguous instead of strided split ownership, fp32 instead of input-dtype partials, exp2
// with a pre-scaled exponent instead of exp.
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <random>
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"
#include "turbo_tables.cuh"

#include "trace.cuh"

namespace dflash {

size_t sdpa_simple_workspace_bytes(int B, int Hq, int D);

namespace {

constexpr int kBlockN = 128;            // keys per tile
constexpr int kRowsM = 128;             // query rows per unit tile
constexpr int kChunkBytes = 128 * 128;  // one TMA box: 128 rows x 64 16-bit elements
constexpr int kThreads = 320;          // TMA warp, MMA warp, 8 softmax warps
constexpr int kUnpackThreads = 384;    // compressed KV only: 12 more warps expand packed bytes into the rings: eight the keys (two
                                       // threads per key row), four the values
constexpr int kPvThreads = 32;         // one more warp whose lane 0 issues the P V products
// Dense: warp 0 TMA, 1 Q K^T issuer, 2-9 softmax, 10 P V issuer.  Compressed KV: 24 warps laid out by warpgroup so that
// registers can move between the roles (setmaxnreg works on whole warpgroups): warps 0-7 softmax, 8-15 key unpack,
// 16-19 value unpack, 20 TMA, 21 Q K^T issuer, 22 P V issuer, 23 idle.  The code below speaks of roles by the dense
// numbering.
template <bool TURBO> struct ThreadsOf { static constexpr int value = TURBO ? 768 : kThreads + kPvThreads; };
constexpr int kTurboIdleRole = 23;
// Registers per thread of the compressed-KV kernel: 80 at launch; the softmax warps take 112, the unpack warps and the
// last warpgroup keep 64 (256 x 112 + 384 x 64 + 128 x 64 = the launch's 61 440).
constexpr int kTurboRegsLaunch = 80, kTurboRegsSoftmax = 112, kTurboRegsUnpack = 64, kTurboRegsHelper = 64;
static_assert(256 * kTurboRegsSoftmax + 384 * kTurboRegsUnpack + 128 * kTurboRegsHelper <= 768 * kTurboRegsLaunch, "register pool");
__device__ __forceinline__ int turbo_role(int pw) {   // physical warp -> the dense numbering (11-22 unpack, 23 idle)
  return pw < 8 ? pw + 2 : (pw < 20 ? pw + 3 : (pw == 20 ? 0 : (pw == 21 ? 1 : (pw == 22 ? 10 : kTurboIdleRole))));
}
constexpr float kRescaleThreshold = 8.f;   // in log2 units
constexpr int kFusedMax = 4;               // a unit cut into at most this many ranges is merged by its last finisher

struct TcParams {
  SdpaArgs a;
  int G, R, MT;            // group size, rows per (b, kvh), 128-row tiles per (b, kvh)
  int units;               // B * Hkv * MT
  long long total_tiles;   // only valid when kv_len == nullptr
  float scale_log2;
  float inv_scale;         // additive mask values are brought to raw-score units: mask / scale
  int mask_vec;            // 1: mask rows can be read 16 bytes at a time (base 16-byte aligned, N a multiple of 8)
  int split;               // 0: stream-K ranges; c > 0: every unit cut into c equal ranges (uniform N only)
  int pair;                // 1: split == 2 and the two CTAs of a unit form a cluster that merges through
                           //    distributed shared memory (no partials in global memory)
  unsigned long long epoch;            // tag of this launch, never 0
  unsigned long long* flags;           // [2 * gridDim.x] arrival flags (hold the epoch of the launch that set them)
  int* slot_unit;          // [2 * gridDim.x]; -1: empty, or merged inside the main kernel
  float* part_o;           // [2 * gridDim.x][D / 4][128 rows][4]: a warp's 32 rows store 512 contiguous bytes
  float* part_m;           // [2 * gridDim.x][128]  (reference maximum, log2 units)
  float* part_l;           // [2 * gridDim.x][128]
  int* status;
  // ---- KV in the TurboQuant 3-bit format (the TURBO instantiation; see the unpack role in the kernel) ----
  // cold history, arrays over [B, Hkv, n_cold, D / 128 blocks]; a.q is then Q1 = R q, map_q2 covers Q2 = Rq^T q, a.k / a.v
  // are the hot window's keys and values in the rotated domain [B, Hkv, n_hot, D], and a.out receives the output in
  // the rotated domain
  const uint8_t* t_kp;     // [.., 48] 3-bit centroid indices of the keys
  const uint8_t* t_ks;     // [.., 16] sign bits of the keys' rotated residuals
  const uint16_t* t_kn;    // fp16 bits: ||k||
  const uint16_t* t_kr;    // fp16 bits: ||residual||
  const uint8_t* t_vp;     // [.., 48]
  const uint16_t* t_vn;    // fp16 bits: ||v|| / ||centroid vector||
  int n_cold;              // compressed keys per (sequence, KV head): a multiple of 128
  int tiles_cold;          // n_cold / 128; tiles at or beyond it come from the hot window
};

template <int D, bool TURBO>
struct Smem {
  static constexpr int kQChunks = D / 64;
  // even: V chunks are consumed in pairs.  Compressed KV: the second query tile takes the room of most of the ring;
  // four stages are enough there because chunks are produced by the CTA itself, a few hundred clocks ahead of their use
  static constexpr int kStages = TURBO ? 4 : ((D == 256) ? 10 : 12);
  // The ring is two rings: K chunks (consumed by the Q K^T issuer as they arrive) in the first kStagesK stages, V chunks
  // (consumed by the P V issuer once the probabilities exist) in the rest; each ring has one producer and one consumer,
  // so no role ever passes over a use of a stage
  static constexpr int kStagesK = TURBO ? 2 : 4;
  static constexpr int kStagesV = kStages - kStagesK;
  static constexpr uint32_t q = 0;
  static constexpr uint32_t q2 = kQChunks * kChunkBytes;                     // TURBO: Q2 = Rq^T q
  static constexpr uint32_t ring = (TURBO ? 2 : 1) * kQChunks * kChunkBytes;
  // TURBO: landing areas of the packed arrays of one 128-key tile
  static constexpr uint32_t stg_a = ring + kStages * kChunkBytes;            // kp [128][D/128][48] | kn [128][D/128] | kr [128][D/128]
  static constexpr uint32_t stg_a_kn = stg_a + 48 * D;
  static constexpr uint32_t stg_a_kr = stg_a_kn + 2 * D;
  static constexpr uint32_t stg_b = stg_a + 52 * D;                          // ks [128][D/128][16]
  static constexpr uint32_t stg_c = stg_b + 16 * D;                          // vp [128][D/128][48] | vn [128][D/128]
  static constexpr uint32_t stg_c_vn = stg_c + 48 * D;
  static constexpr uint32_t stg_end = stg_c + 50 * D;
  static constexpr uint32_t bars = TURBO ? stg_end : ring + kStages * kChunkBytes;
  // barrier slots (8 bytes each)
  static constexpr int b_q_full = 0, b_q_empty = 1, b_pv_done = 2, b_o_free = 3;
  static constexpr int b_s_full = 4;                 // 2
  static constexpr int b_p_full = 6;                 // 2
  static constexpr int b_kv_full = 8;                // kStages
  static constexpr int b_kv_empty = 8 + kStages;     // kStages
  static constexpr int b_peer_ready = 8 + 2 * kStages;   // the cluster partner has stopped using its ring
  static constexpr int b_peer_data = 9 + 2 * kStages;    // the partner's columns have landed here (256 arrivals)
  static constexpr int b_stg_full = 10 + 2 * kStages;    // 3 (TURBO): a landing area holds its tile
  static constexpr int b_stg_empty = 13 + 2 * kStages;   // 3 (TURBO): the unpack warps have read it (4 arrivals)
  static constexpr int b_s_free = 16 + 2 * kStages;      // 2: the product that read P from this score buffer has retired
  static constexpr int n_bars = 18 + 2 * kStages;
  static constexpr uint32_t misc = bars + 8 * n_bars;   // tmem base, abort flag, range info, group counter, merge decision
  static constexpr uint32_t xseq = misc + 64;            // exchange sequence numbers [2][2][4]
  static constexpr uint32_t xch = xseq + 64;             // exchange values [2 slots][2 halves][128 rows]
  static constexpr uint32_t total = xch + 2 * 2 * 128 * 4;
  static constexpr uint32_t alloc = total;               // the dynamic shared window starts 1024-byte aligned (checked)
  static_assert(total <= 232448, "shared memory of one CTA");
};

// ---- work decomposition -------------------------------------------------------------------
struct Segment {
  int unit;        // (b * Hkv + kvh) * MT + mt
  int b, kvh, mt;
  int n_keys;      // N_b
  int tile_lo, tile_hi, tiles_in_unit;
  int slot;        // -1: covers the whole unit, write the output directly
  long long unit_begin;   // global tile position of the unit's tile 0
};

// The decomposition: which global tile positions a CTA owns, and which CTA owns a position.
__device__ __forceinline__ void cta_range(const TcParams& p, long long total, int cta, long long& begin, long long& end) {
  if (p.split > 0) {
    const long long tpu = (p.a.N + kBlockN - 1) / kBlockN;
    const long long u = cta / p.split, k = cta % p.split;
    begin = u * tpu + tpu * k / p.split;
    end = u * tpu + tpu * (k + 1) / p.split;
  } else {
    // never more ranges than tiles (ragged lengths can leave CTAs idle): no range is empty
    const long long C = (long long)gridDim.x < total ? (long long)gridDim.x : total;
    begin = cta < C ? total * cta / C : 0;
    end = cta < C ? total * (cta + 1) / C : 0;
  }
}
__device__ __forceinline__ int cta_of(const TcParams& p, long long total, long long pos) {
  if (p.split > 0) {
    const long long tpu = (p.a.N + kBlockN - 1) / kBlockN;
    const long long u = pos / tpu, t = pos % tpu;
    return (int)(u * p.split + ((t + 1) * p.split - 1) / tpu);
  }
  const long long C = (long long)gridDim.x < total ? (long long)gridDim.x : total;
  return (int)(((pos + 1) * C - 1) / total);
}

// Keys of sequence b.  A device-resident length outside [0, N] is clamped here (and reported once per launch by
// CTA 0): nothing downstream may index the page table or the tensor maps with it unclamped.
__device__ __forceinline__ int keys_of(const TcParams& p, int b) {
  if (!p.a.kv_len) return p.a.N;
  const int n = p.a.kv_len[b];
  return n < 0 ? 0 : (n > p.a.N ? p.a.N : n);
}
__device__ __forceinline__ int tiles_of(const TcParams& p, int b) { return (keys_of(p, b) + kBlockN - 1) / kBlockN; }

// Iterates the segments of one CTA's tile range.  All roles run the same iterator.
struct SegmentIter {
  const TcParams& p;
  long long pos, end;     // global tile positions of the CTA's range
  int unit, tile;         // current unit and tile inside it
  int first;              // 1 until the first segment has been produced
  __device__ SegmentIter(const TcParams& p_, long long begin, long long end_, int unit0, int tile0)
      : p(p_), pos(begin), end(end_), unit(unit0), tile(tile0), first(1) {}
  __device__ bool next(Segment& s) {
    if (pos >= end) return false;
    const int per_b = p.a.Hkv * p.MT;
    // a sequence without keys (length clamped to 0) has no tiles and owns no tile positions: pass over its units
    while (p.a.kv_len && unit < p.units && keys_of(p, unit / per_b) == 0) unit += per_b - unit % per_b;
    if (unit >= p.units) return false;
    s.unit = unit;
    s.b = unit / per_b;
    s.kvh = (unit / p.MT) % p.a.Hkv;
    s.mt = unit % p.MT;
    s.n_keys = keys_of(p, s.b);
    s.tiles_in_unit = (s.n_keys + kBlockN - 1) / kBlockN;
    s.tile_lo = tile;
    const long long left = end - pos;
    const int avail = s.tiles_in_unit - tile;
    const int take = left < avail ? (int)left : avail;
    s.tile_hi = tile + take;
    const bool whole = (s.tile_lo == 0 && s.tile_hi == s.tiles_in_unit);
    // a CTA has at most one range that continues a unit (its first) and one that opens a unit
    // without finishing it (its last): slots 2i and 2i + 1
    s.slot = whole ? -1 : (s.tile_lo > 0 ? 2 * (int)blockIdx.x : 2 * (int)blockIdx.x + 1);
    s.unit_begin = pos - tile;
    first = 0;
    pos += take;
    tile = 0;
    unit += 1;
    return true;
  }
};

__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  // start address, leading / stride byte offsets (all >> 4), descriptor version 1, 128-byte swizzle
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) |
         ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ bool wait_or_abort(void* bar, uint32_t parity, volatile int* abort_flag, int* status) {
  return ptx::mbar_wait_or_abort(bar, parity, abort_flag, status, kStatusMbarWait);
}

__device__ __forceinline__ float fast_exp2(float x) {   // ex2.approx: exp2(-inf) = +0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void st_release_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_sc() { asm volatile("fence.sc.gpu;" ::: "memory"); }

// ---- distributed shared memory of a two-CTA cluster ----
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t peer_addr(const void* local, uint32_t rank) {   // same offset in CTA `rank` of the cluster
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(ptx::smem_u32(local)), "r"(rank));
  return r;
}
__device__ __forceinline__ void peer_arrive(uint32_t remote_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
__device__ __forceinline__ void peer_store(uint32_t remote, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void peer_store1(uint32_t remote, float a) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(a) : "memory");
}
__device__ __forceinline__ bool try_wait_cluster(void* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(ptx::smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ bool wait_peer_or_abort(void* bar, uint32_t parity, volatile int* abort_flag, int* status) {
  for (uint32_t i = 0; i < ptx::kWaitPolls; ++i) {
    if (try_wait_cluster(bar, parity)) return true;
    if ((i & 63u) == 63u) {
      if (*abort_flag) return false;
      __nanosleep(40);
    }
  }
  *abort_flag = 1;
  atomicExch(status, kStatusPeerWait);
  return false;
}


template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  const __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// This thread's 64 additive-mask values of one key tile (row `mrow`, keys n0 .. n0+63), as 32 packed pairs.
// Keys at or beyond N, and rows outside the group (mrow == nullptr), read as 0: the visibility rule hides them anyway.
template <typename InT>
__device__ __forceinline__ void load_mask64(const InT* mrow, int n0, int N, bool vec, uint32_t (&mk)[32]) {
  if (mrow && vec && n0 + 64 <= N) {
    const uint4* src = reinterpret_cast<const uint4*>(mrow + n0);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 u = __ldg(src + i);
      mk[4 * i] = u.x; mk[4 * i + 1] = u.y; mk[4 * i + 2] = u.z; mk[4 * i + 3] = u.w;
    }
  } else {
    const unsigned short* src = reinterpret_cast<const unsigned short*>(mrow);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const uint32_t lo = (mrow && n0 + 2 * i < N) ? (uint32_t)__ldg(src + n0 + 2 * i) : 0u;
      const uint32_t hi = (mrow && n0 + 2 * i + 1 < N) ? (uint32_t)__ldg(src + n0 + 2 * i + 1) : 0u;
      mk[i] = lo | (hi << 16);
    }
  }
}
template <typename InT> __device__ __forceinline__ float2 unpack2(uint32_t u);
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t u) {
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t u) {
  return __half22float2(*reinterpret_cast<const __half2*>(&u));
}
// Lowest finite value of the attention dtype: a mask entry below it (or a NaN) hides the key.
template <typename InT> __device__ __forceinline__ float mask_floor();
template <> __device__ __forceinline__ float mask_floor<__nv_bfloat16>() { return -3.3895313892515355e38f; }
template <> __device__ __forceinline__ float mask_floor<__half>() { return -65504.f; }

// ---- compressed KV: expanding one key's 64 dimensions into a row of an operand chunk -------------------------------
// A chunk is what a TMA box of the dense path is: 128 keys x 64 16-bit elements, 128 bytes per key, the eight 16-byte
// pieces of a row XOR-swizzled with the row index (CU_TENSOR_MAP_SWIZZLE_128B).  One thread writes one row.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ float f16_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

template <typename InT> __device__ __forceinline__ uint32_t pack2_rn(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2_rn<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2_rn<__half>(float a, float b) {
  const __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// 64 three-bit centroid indices (24 bytes at `src`, 8-byte aligned) -> 64 values scale * centroid in the attention
// dtype.  The eight scaled centroids are split into a table of their low bytes and one of their high bytes; four
// indices at a time select from both with byte permutes.
// `kPieces` = 8: the whole row; 4: thread `hsel` (0 or 1) of a row's pair writes pieces 4 hsel .. 4 hsel + 3 (the 32
// indices in bytes 12 hsel .. 12 hsel + 11).
template <typename InT, int kPieces = 8>
__device__ __forceinline__ void unpack_centroid_row(uint8_t* chunk, int row, const uint8_t* src, float scale, int hsel = 0) {
  uint32_t w[7];
  if (kPieces == 8) {
    const uint2 a = *reinterpret_cast<const uint2*>(src), b = *reinterpret_cast<const uint2*>(src + 8), c = *reinterpret_cast<const uint2*>(src + 16);
    w[0] = a.x; w[1] = a.y; w[2] = b.x; w[3] = b.y; w[4] = c.x; w[5] = c.y; w[6] = 0u;
  } else {
    const uint32_t* s32 = reinterpret_cast<const uint32_t*>(src + 12 * hsel);
    w[0] = s32[0]; w[1] = s32[1]; w[2] = s32[2]; w[3] = 0u; w[4] = w[5] = w[6] = 0u;
  }
  const uint32_t p0 = pack2_rn<InT>(TURBO_C3[0] * scale, TURBO_C3[1] * scale), p1 = pack2_rn<InT>(TURBO_C3[2] * scale, TURBO_C3[3] * scale);
  const uint32_t p2 = pack2_rn<InT>(TURBO_C3[4] * scale, TURBO_C3[5] * scale), p3 = pack2_rn<InT>(TURBO_C3[6] * scale, TURBO_C3[7] * scale);
  const uint32_t lo_a = prmt(p0, p1, 0x6420), lo_b = prmt(p2, p3, 0x6420), hi_a = prmt(p0, p1, 0x7531), hi_b = prmt(p2, p3, 0x7531);
  uint8_t* dst = chunk + row * 128;
  const int sw = row & 7;
#pragma unroll
  for (int pp = 0; pp < kPieces; ++pp) {         // 8 indices = 24 bits -> 8 values = 16 bytes
    const int piece = (kPieces == 8 ? 0 : 4 * hsel) + pp;
    const int bit = pp * 24, word = bit >> 5, off = bit & 31;
    const uint32_t x = off ? __funnelshift_r(w[word], w[word + 1], off) : w[word];
    // the eight 3-bit indices spread to one per nibble (a byte permute's selector spacing) in three halving steps
    const uint32_t s12 = (x & 0x00000FFFu) | ((x << 4) & 0x0FFF0000u);
    const uint32_t s6 = (s12 & 0x003F003Fu) | ((s12 << 2) & 0x3F003F00u);
    const uint32_t s3 = (s6 & 0x07070707u) | ((s6 << 1) & 0x70707070u);
    uint32_t o[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t sel = h ? (s3 >> 16) : s3;   // a permute reads the low 16 bits of its selector
      const uint32_t lo4 = prmt(lo_a, lo_b, sel), hi4 = prmt(hi_a, hi_b, sel);
      o[2 * h] = prmt(lo4, hi4, 0x5140);
      o[2 * h + 1] = prmt(lo4, hi4, 0x7362);
    }
    *reinterpret_cast<uint4*>(dst + ((piece ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}
// 64 sign bits (8 bytes at `src`) -> 64 values +-mag: bit set = +mag (tests/test_turbo_quant.cpp:97 of the SwiftLM tree)
// Thread `hsel` of a row's pair writes pieces 4 hsel .. 4 hsel + 3 (the 32 sign bits of word hsel).
template <typename InT>
__device__ __forceinline__ void unpack_sign_half_row(uint8_t* chunk, int row, const uint8_t* src, float mag, int hsel) {
  const uint32_t nw = ~reinterpret_cast<const uint32_t*>(src)[hsel];   // set bit = negative
  const uint32_t m2 = pack2_rn<InT>(mag, mag);
  uint8_t* dst = chunk + row * 128;
  const int sw = row & 7;
#pragma unroll
  for (int pp = 0; pp < 4; ++pp) {               // 8 bits -> 8 values = 16 bytes
    const int piece = 4 * hsel + pp;
    const uint32_t t = nw >> (pp * 8);
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) o[k] = m2 ^ ((t << (15 - 2 * k)) & 0x8000u) ^ ((t << (30 - 2 * k)) & 0x80000000u);
    *reinterpret_cast<uint4*>(dst + ((piece ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <typename InT, int D, bool MASK, bool TURBO>
__global__ void __launch_bounds__(ThreadsOf<TURBO>::value, 1)
sdpa_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_q2,
               const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const TcParams p) {
  using SL = Smem<D, TURBO>;
  constexpr int kNumThreads = ThreadsOf<TURBO>::value;
  constexpr int kStages = SL::kStages;
  constexpr int kQChunks = SL::kQChunks;            // 64-element chunks of the head dimension
  constexpr uint32_t kFmt = sizeof(InT) == 2 && std::is_same<InT, __nv_bfloat16>::value ? 1u : 0u;
  // instruction descriptors: fp32 accumulate, A/B format, majors, N >> 3, M >> 4
  constexpr uint32_t kIdescQK = (1u << 4) | (kFmt << 7) | (kFmt << 10) | ((kBlockN >> 3) << 17) | ((kRowsM >> 4) << 24);
  constexpr uint32_t kIdescPV = (1u << 4) | (kFmt << 7) | (kFmt << 10) | (1u << 16) | ((128u >> 3) << 17) | ((kRowsM >> 4) << 24);
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColO = 0, kColS = D;          // O: D columns; S buffers: 2 x 128 columns

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* sm = smem_raw;
  if ((ptx::smem_u32(sm) & 1023u) != 0u) {   // swizzled tiles need 1024-byte alignment; never seen violated
    if (threadIdx.x == 0) atomicExch(p.status, kStatusSmemAlign);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + SL::bars);
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(sm + SL::misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + SL::misc + 4);
  int* range_info = reinterpret_cast<int*>(sm + SL::misc + 8);   // unit0, tile0

  // Back-to-back calls (the attention of one layer after another): a launch made with programmatic stream
  // serialization may bring its CTAs onto SMs as the previous grid's CTAs leave, so that its set-up (barriers, tensor
  // memory, tensor maps) runs beside the previous grid's tail.  Nothing of the previous grid's results, of this call's
  // inputs or of the workspace is touched before griddepcontrol.wait, which returns when every earlier grid has
  // completed and its memory is visible: with per-sequence lengths (read right below) every thread waits here; else
  // the one thread that sets the CTA up waits before its first global store, and every other thread meets it at the
  // barrier that ends the set-up.  Without the launch attribute both instructions do nothing.
  const int pw = threadIdx.x >> 5, lane = threadIdx.x & 31;   // physical warp
  const int warp = TURBO ? turbo_role(pw) : pw;                // role, in the dense numbering
  const SdpaArgs& a = p.a;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (a.kv_len) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) TR_STAMP(0);
  TR_DECL();

  // ---- the CTA's tile range ----
  long long total = p.total_tiles;
  if (a.kv_len) {
    // ragged lengths: every CTA sums the per-sequence tile counts itself (B is small)
    long long sum = 0;
    bool in_range = true;
    for (int b = 0; b < a.B; ++b) {
      sum += tiles_of(p, b);
      const int n = a.kv_len[b];
      in_range = in_range && n >= 16 && n <= a.N;
    }
    total = sum * a.Hkv * p.MT;
    if (!in_range && blockIdx.x == 0 && threadIdx.x == 0) atomicExch(p.status, kStatusKvLen);
  }
  long long begin, end;
  cta_range(p, total, blockIdx.x, begin, end);

  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&map_q);
    if (TURBO) ptx::prefetch_tensormap(&map_q2);
    ptx::prefetch_tensormap(&map_k);
    ptx::prefetch_tensormap(&map_v);
    for (int i = 0; i < SL::n_bars; ++i) {
      const bool eight = (i == SL::b_o_free) || (i == SL::b_p_full) || (i == SL::b_p_full + 1);
      // compressed KV: a ring stage is filled by the four warps of one unpack group (one arrival each; for a hot tile
      // the group's first lane issues a TMA load and its arrival carries the byte count); a landing area is released
      // by the four warps of the group that reads it
      // (the keys' group has eight warps, the values' four)
      const bool k_side = TURBO && ((i >= SL::b_kv_full && i < SL::b_kv_full + SL::kStagesK) || i == SL::b_stg_empty || i == SL::b_stg_empty + 1);
      const bool v_side = TURBO && ((i >= SL::b_kv_full + SL::kStagesK && i < SL::b_kv_full + kStages) || i == SL::b_stg_empty + 2);
      ptx::mbar_init(&bars[i], i == SL::b_peer_data ? 256 : ((eight || k_side) ? 8 : (v_side ? 4 : 1)));
    }
    *abort_flag = 0;
    reinterpret_cast<volatile uint32_t*>(sm + SL::misc)[4] = 0;   // group counter
    for (int i = 0; i < 16; ++i) reinterpret_cast<volatile uint32_t*>(sm + SL::xseq)[i] = 0;
    // locate (unit, tile) of `begin`
    int unit = 0, tile = 0;
    if (!a.kv_len) {
      const int tpu = (a.N + kBlockN - 1) / kBlockN;
      unit = (int)(begin / tpu);
      tile = (int)(begin % tpu);
    } else {
      long long acc = 0;
      const int per_b = a.Hkv * p.MT;
      for (int b = 0; b < a.B; ++b) {
        const long long tb = tiles_of(p, b);
        if (begin < acc + tb * per_b) {
          const long long off = begin - acc;
          unit = b * per_b + (int)(off / tb);
          tile = (int)(off % tb);
          break;
        }
        acc += tb * per_b;
      }
    }
    range_info[0] = unit;
    range_info[1] = tile;
    ptx::fence_mbar_init();
    if (!a.kv_len) asm volatile("griddepcontrol.wait;" ::: "memory");
    // slot table: rewritten below by the softmax warps for the slots this CTA uses
    p.slot_unit[2 * blockIdx.x] = -1;
    p.slot_unit[2 * blockIdx.x + 1] = -1;
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_base_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  // The producer warp needs only what its own lane 0 set up (barriers, range): it arrives and goes
  // on to issue loads while the other warps still wait for the tensor-memory allocation.
  uint32_t tmem_base = 0;
  if (warp == 0) {
    __syncwarp();
    __threadfence_block();
    asm volatile("bar.arrive 1, %0;" ::"n"(kNumThreads) : "memory");
  } else {
    ptx::tc_fence_before();
    asm volatile("bar.sync 1, %0;" ::"n"(kNumThreads) : "memory");
    ptx::tc_fence_after();
    tmem_base = *tmem_base_slot;
  }
  const int unit0 = range_info[0], tile0 = range_info[1];
  if (threadIdx.x == 0) TR_STAMP(1);

  // Compressed KV: each warpgroup sets its register budget as the first thing in its own branch - code that paths
  // with different budgets share is compiled for the smallest of them, so the branches meet again only at the very end.
  if (warp == 0 || warp == 1 || warp == kThreads / 32 || warp == kTurboIdleRole) {
  if constexpr (TURBO) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kTurboRegsHelper));
  if (warp == 0) {
    // =================================== TMA producer ===================================
    if (lane == 0 && begin < end) {
      if constexpr (TURBO) {
        // Compressed KV: the packed arrays of a 128-key tile of the cold history land in three areas (A: key indices
        // and norms, B: key sign bits, C: value indices and norms), each refilled as soon as the unpack warps have read
        // it.  This lane never touches the ring: the unpack warps fill it, for hot tiles by issuing the TMA loads
        // themselves.  (A role that passed over some uses of a ring stage without waiting for them could get two phases
        // ahead of the stage's barrier, and a parity wait cannot tell "released" from "two uses behind".)
        SegmentIter it(p, begin, end, unit0, tile0);
        Segment s;
        uint32_t seg_idx = 0;
        bool ok = true;
        uint32_t n_stg[3] = {0, 0, 0};
        auto stage_area = [&](int area) -> bool {       // wait until the area's previous tile has been read, then expect the new one
          if (n_stg[area] > 0 && !wait_or_abort(&bars[SL::b_stg_empty + area], (n_stg[area] - 1) & 1, abort_flag, p.status)) return false;
          ptx::mbar_arrive_expect_tx(&bars[SL::b_stg_full + area], (area == 0 ? 52u : area == 1 ? 16u : 50u) * D);
          ++n_stg[area];
          return true;
        };
        auto cold_blocks = [&](const Segment& sg, int tile) -> long long {   // first 128-dimension block of the tile's keys
          return (((long long)sg.b * a.Hkv + sg.kvh) * p.n_cold + (long long)tile * kBlockN) * (D / 128);
        };
        auto stage_cold_k = [&](const Segment& sg, int tile) -> bool {
          const long long blk = cold_blocks(sg, tile);
          if (!stage_area(0)) return false;
          ptx::bulk_load(sm + SL::stg_a, p.t_kp + blk * 48, 48 * D, &bars[SL::b_stg_full + 0]);
          ptx::bulk_load(sm + SL::stg_a_kn, p.t_kn + blk, 2 * D, &bars[SL::b_stg_full + 0]);
          ptx::bulk_load(sm + SL::stg_a_kr, p.t_kr + blk, 2 * D, &bars[SL::b_stg_full + 0]);
          if (!stage_area(1)) return false;
          ptx::bulk_load(sm + SL::stg_b, p.t_ks + blk * 16, 16 * D, &bars[SL::b_stg_full + 1]);
          return true;
        };
        auto stage_cold_v = [&](const Segment& sg, int tile) -> bool {
          const long long blk = cold_blocks(sg, tile);
          if (!stage_area(2)) return false;
          ptx::bulk_load(sm + SL::stg_c, p.t_vp + blk * 48, 48 * D, &bars[SL::b_stg_full + 2]);
          ptx::bulk_load(sm + SL::stg_c_vn, p.t_vn + blk, 2 * D, &bars[SL::b_stg_full + 2]);
          return true;
        };
        while (ok && it.next(s)) {
          // Q tiles of this unit: wait until the previous segment's S = Q K^T products are done with them
          if (seg_idx > 0 && !wait_or_abort(&bars[SL::b_q_empty], (seg_idx - 1) & 1, abort_flag, p.status)) break;
          ptx::mbar_arrive_expect_tx(&bars[SL::b_q_full], 2 * kQChunks * kChunkBytes);
          for (int c = 0; c < kQChunks; ++c)
            ptx::tma_load_3d(sm + SL::q + c * kChunkBytes, &map_q, c * 64, s.mt * kRowsM, s.b * a.Hkv + s.kvh, &bars[SL::b_q_full]);
          for (int c = 0; c < kQChunks; ++c)
            ptx::tma_load_3d(sm + SL::q2 + c * kChunkBytes, &map_q2, c * 64, s.mt * kRowsM, s.b * a.Hkv + s.kvh, &bars[SL::b_q_full]);
          // per step the unpack warps want the values of tile j - 1 first, then the keys of tile j
          for (int j = s.tile_lo; ok && j <= s.tile_hi; ++j) {
            if (j > s.tile_lo && j - 1 < p.tiles_cold) ok = stage_cold_v(s, j - 1);
            if (ok && j < s.tile_hi && j < p.tiles_cold) ok = stage_cold_k(s, j);
          }
          ++seg_idx;
        }
      } else {
        // Dense KV: two cursors over the CTA's tiles, one feeding K chunks (and each unit's Q tile) to the Q K^T issuer
        // through the K ring, one feeding V chunks to the P V issuer through the V ring.  Neither blocks the other: a
        // cursor that finds its ring full (or the Q tile still in use) yields, and the lane sleeps only when both are stuck.
        constexpr int kSK = SL::kStagesK, kSV = SL::kStagesV;
        struct PageRef { int b, index, page; };
        struct Cursor {
          SegmentIter it;
          Segment s;
          bool have, done;
          int j, c;
          uint32_t fill, seg;
          PageRef ref;
        };
        Cursor ck{SegmentIter(p, begin, end, unit0, tile0), Segment{}, false, false, 0, 0, 0u, 0u, PageRef{-1, -1, 0}};
        Cursor cv{SegmentIter(p, begin, end, unit0, tile0), Segment{}, false, false, 0, 0, 0u, 0u, PageRef{-1, -1, 0}};
        bool q_pending = false;
        // one 16 KiB box of tile `tile`, head-dimension chunk c, into ring stage `stage`; paged KV: the page of a tile is
        // looked up once per cursor, not once per chunk
        auto issue_chunk = [&](const CUtensorMap* map, Cursor& cur, int stage) {
          ptx::mbar_arrive_expect_tx(&bars[SL::b_kv_full + stage], kChunkBytes);
          const int n0 = cur.j * kBlockN;
          if (a.page_table) {
            if (cur.c == 0) {
              const int index = n0 / a.page_tokens;
              if (index != cur.ref.index || cur.s.b != cur.ref.b) {
                // index < max_pages because n0 < N <= max_pages * page_tokens (host check, lengths clamped to N).
                // A page id outside the pool reads as zeros (the tensor map ends at num_pages) and is reported.
                cur.ref = PageRef{cur.s.b, index, a.page_table[(long long)cur.s.b * a.max_pages + index]};
                if ((unsigned)cur.ref.page >= (unsigned)a.num_pages) { cur.ref.page = a.num_pages; atomicExch(p.status, kStatusKvRange); }
              }
            }
            ptx::tma_load_4d(sm + SL::ring + stage * kChunkBytes, map, cur.c * 64, n0 - cur.ref.index * a.page_tokens, cur.s.kvh,
                             cur.ref.page, &bars[SL::b_kv_full + stage]);
          } else {
            ptx::tma_load_4d(sm + SL::ring + stage * kChunkBytes, map, cur.c * 64, n0, cur.s.kvh, cur.s.b, &bars[SL::b_kv_full + stage]);
          }
        };
        // advances a cursor by one chunk if its ring has room: 1 progressed, 0 has to wait, -1 finished
        auto step = [&](Cursor& cur, bool is_k) -> int {
          if (cur.done) return -1;
          if (!cur.have) {
            if (!cur.it.next(cur.s)) { cur.done = true; return -1; }
            cur.have = true;
            cur.j = cur.s.tile_lo;
            cur.c = 0;
            if (is_k) q_pending = true;
          }
          if (is_k && q_pending) {
            // Q tile of this unit: the previous segment's S = Q K^T products must be done with it
            if (cur.seg > 0 && !ptx::mbar_try_wait(&bars[SL::b_q_empty], (cur.seg - 1) & 1)) return 0;
            ptx::mbar_arrive_expect_tx(&bars[SL::b_q_full], kQChunks * kChunkBytes);
            for (int c = 0; c < kQChunks; ++c)
              ptx::tma_load_3d(sm + SL::q + c * kChunkBytes, &map_q, c * 64, cur.s.mt * kRowsM, cur.s.b * a.Hkv + cur.s.kvh, &bars[SL::b_q_full]);
            q_pending = false;
            return 1;
          }
          const int ring_n = is_k ? kSK : kSV, ring_0 = is_k ? 0 : kSK;
          const int stage = ring_0 + (int)(cur.fill % (uint32_t)ring_n);
          if (cur.fill >= (uint32_t)ring_n && !ptx::mbar_try_wait(&bars[SL::b_kv_empty + stage], ((cur.fill / (uint32_t)ring_n) - 1) & 1)) return 0;
          issue_chunk(is_k ? &map_k : &map_v, cur, stage);
          ++cur.fill;
          if (++cur.c == kQChunks) {
            cur.c = 0;
            if (++cur.j == cur.s.tile_hi) { cur.have = false; ++cur.seg; }
          }
          return 1;
        };
        uint32_t idle = 0;
        while (!(ck.done && cv.done)) {
          const int rk = step(ck, true), rv = step(cv, false);
          if (rk > 0 || rv > 0) { idle = 0; continue; }
          if (ck.done && cv.done) break;
          if ((++idle & 63u) == 63u) {
            if (*abort_flag) break;
            __nanosleep(40);
          }
          if (idle >= ptx::kWaitPolls) {   // neither ring has released a stage for the whole poll budget
            *abort_flag = 1;
            atomicExch(p.status, kStatusMbarWait);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ================================ Q K^T issuer ================================
    // This lane issues only S = Q K^T; a second lane (warp 10) issues O += P V.  One thread issuing both spent about
    // 6 K clocks per key tile (32 products, a dozen barrier waits and commits) where the products themselves take 2 K:
    // it, not HBM or the softmax, set the tile period.  The two issuers meet through barriers only: a score buffer may be
    // overwritten once the product that read P from it has retired (s_free), and P V starts when P is there (p_full).
    if (lane == 0 && begin < end) {
      constexpr int kSK = SL::kStagesK;
      SegmentIter it(p, begin, end, unit0, tile0);
      Segment s;
      uint32_t drain = 0, seg_idx = 0, tile_ctr = 0;
      bool ok = true;
      const uint32_t q_addr = ptx::smem_u32(sm + SL::q);
      while (ok && it.next(s)) {
        if (!wait_or_abort(&bars[SL::b_q_full], seg_idx & 1, abort_flag, p.status)) break;
        ptx::tc_fence_after();
        const int ntiles = s.tile_hi - s.tile_lo;
        for (int jj = 0; ok && jj < ntiles; ++jj) {
          const uint32_t t = tile_ctr + jj, buf = t & 1;
          const uint32_t d_tmem = tmem_base + kColS + buf * kBlockN;
          if (t >= 2) {   // P of tile t - 2 lived in this buffer: its product must have retired
            TR_T0();
            ok = wait_or_abort(&bars[SL::b_s_free + buf], ((t >> 1) - 1) & 1, abort_flag, p.status);
            TR_ACC(19);
            if (!ok) break;
          }
          // compressed keys: the scaled centroids against Q1, then the scaled residual signs against Q2, one accumulator
          const int n_kc = (TURBO && s.tile_lo + jj < p.tiles_cold) ? 2 * kQChunks : kQChunks;
          for (int c = 0; ok && c < n_kc; ++c) {
            const uint32_t stage = drain % kSK;
            {
              TR_T0();
              ok = wait_or_abort(&bars[SL::b_kv_full + stage], (drain / kSK) & 1, abort_flag, p.status);
              TR_ACC(17);
              if (drain == 0) TR_STAMP(2);
            }
            if (!ok) break;
            ptx::tc_fence_after();
            // descriptors differ only in the start-address field: +2 (32 bytes) per 16-element step
            const uint64_t da0 = make_desc(q_addr + (c < kQChunks ? c * kChunkBytes : SL::q2 + (c - kQChunks) * kChunkBytes), 16, 1024);
            const uint64_t db0 = make_desc(ptx::smem_u32(sm + SL::ring + stage * kChunkBytes), 16, 1024);
            {
              TR_T0();
              if (c == 0) ptx::umma_ss_first(d_tmem, da0, db0, kIdescQK);
              else ptx::umma_ss_acc(d_tmem, da0, db0, kIdescQK);
              ptx::umma_ss_acc(d_tmem, da0 + 2, db0 + 2, kIdescQK);
              ptx::umma_ss_acc(d_tmem, da0 + 4, db0 + 4, kIdescQK);
              ptx::umma_ss_acc(d_tmem, da0 + 6, db0 + 6, kIdescQK);
              ptx::umma_commit(&bars[SL::b_kv_empty + stage]);   // K chunk free once these products retire
              TR_ACC(22);
            }
            ++drain;
          }
          if (!ok) break;
          ptx::umma_commit(&bars[SL::b_s_full + buf]);
          if (jj == ntiles - 1) ptx::umma_commit(&bars[SL::b_q_empty]);   // last use of this Q tile
        }
        tile_ctr += ntiles;
        ++seg_idx;
      }
    }
  } else if (warp == kThreads / 32) {
    // ================================== P V issuer ==================================
    if (lane == 0 && begin < end) {
      constexpr int kSK = SL::kStagesK, kSV = SL::kStagesV;
      SegmentIter it(p, begin, end, unit0, tile0);
      Segment s;
      uint32_t drain = 0, seg_idx = 0, tile_ctr = 0;
      bool ok = true;
      while (ok && it.next(s)) {
        const int ntiles = s.tile_hi - s.tile_lo;
        for (int jj = 0; ok && jj < ntiles; ++jj) {
          // ---- O += P_j V_j ----
          const uint32_t t = tile_ctr + jj, buf = t & 1;
          if (jj == 0 && seg_idx > 0) {
            // first product of a segment overwrites O: the previous segment's epilogue must have read it
            ok = wait_or_abort(&bars[SL::b_o_free], (seg_idx - 1) & 1, abort_flag, p.status);
            if (!ok) break;
          }
          {
            TR_T0();
            ok = wait_or_abort(&bars[SL::b_p_full + buf], (t >> 1) & 1, abort_flag, p.status);
            TR_ACC(19);
          }
          if (!ok) break;
          ptx::tc_fence_after();
          const uint32_t p_tmem = tmem_base + kColS + buf * kBlockN;   // P (16-bit pairs) aliases S
          // Two 64-column V chunks per instruction (N = 128).  The pair sits in consecutive stages of the V ring (chunks come
          // in groups of kQChunks and the ring has an even number of stages, so a pair never straddles the wrap); the
          // descriptor's leading-dimension offset is the 16 KiB from one chunk to the next.
          for (int cp = 0; ok && cp < kQChunks / 2; ++cp) {
            const uint32_t stage = kSK + drain % kSV;
            {
              TR_T0();
              ok = wait_or_abort(&bars[SL::b_kv_full + stage], (drain / kSV) & 1, abort_flag, p.status) &&
                   wait_or_abort(&bars[SL::b_kv_full + stage + 1], (drain / kSV) & 1, abort_flag, p.status);
              TR_ACC(18);
            }
            if (!ok) break;
            ptx::tc_fence_after();
            // 16 keys per instruction: +128 (2048 bytes) in the start-address field, +8 P columns
            const uint64_t db0 = make_desc(ptx::smem_u32(sm + SL::ring + stage * kChunkBytes), kChunkBytes, 1024);
            const uint32_t o_tmem = tmem_base + kColO + cp * 128;
            {
              TR_T0();
              if (jj > 0) ptx::umma_ts_acc(o_tmem, p_tmem, db0, kIdescPV);
              else ptx::umma_ts_first(o_tmem, p_tmem, db0, kIdescPV);
#pragma unroll
              for (int kk = 1; kk < kBlockN / 16; ++kk)
                ptx::umma_ts_acc(o_tmem, p_tmem + kk * 8, db0 + (uint64_t)kk * 128, kIdescPV);
              ptx::umma_commit(&bars[SL::b_kv_empty + stage]);
              ptx::umma_commit(&bars[SL::b_kv_empty + stage + 1]);
              TR_ACC(23);
            }
            drain += 2;
          }
          if (!ok) break;
          ptx::umma_commit(&bars[SL::b_pv_done]);
          ptx::umma_commit(&bars[SL::b_s_free + buf]);
        }
        tile_ctr += ntiles;
        ++seg_idx;
      }
    }
  }
  } else if (TURBO && warp > kThreads / 32 && warp < kThreads / 32 + 1 + kUnpackThreads / 32) {
    if constexpr (TURBO) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kTurboRegsUnpack));
    // ====================================== unpack =======================================
    // Compressed KV: a group of eight warps for the keys (two threads per key row, half a row of every chunk each: the
    // keys' eight chunks per tile are the longest chain in the kernel) and a group of four for the values (one thread
    // per row).  Per cold tile a group
    // expands, from the landing areas, the key's centroid indices into D / 64 chunks scaled by the key block's norm,
    // its residual sign bits into D / 64 chunks of +-(norm * QJL_C / 128 * rnorm), and (one tile behind, as the MMA
    // warp consumes them) the value's centroid indices scaled by the value block's norm - the operands the dense
    // path gets by TMA, in the same swizzled layout, so that no decoded key or value ever exists in global memory.
    if (begin < end) {
      const int u = (int)threadIdx.x - 8 * 32;                  // physical warps 8-19
      const int t = u & 127, hsel = (u >> 7) & 1;               // key row of a chunk; which half of the row (key group)
      const bool v_group = u >= 256;                            // warps 0-7 expand keys (K ring), warps 8-11 values (V ring)
      constexpr int NB = D / 128;
      constexpr int kSK = SL::kStagesK, kSV = SL::kStagesV;
      SegmentIter it(p, begin, end, unit0, tile0);
      Segment s;
      uint32_t fill_k = 0, fill_v = 0, n_stg[3] = {0, 0, 0};
      bool ok = true;
      float nrm[NB], mag[NB];
      auto wait_all = [&](void* bar, uint32_t parity) -> bool {
        return __all_sync(0xffffffffu, wait_or_abort(bar, parity, abort_flag, p.status));
      };
      // the next stage of the K ring or of the V ring, once its consumer has released it
      auto ring_slot = [&](bool is_k, uint32_t& stage) -> bool {
        const uint32_t fill = is_k ? fill_k : fill_v, n = is_k ? kSK : kSV;
        stage = (is_k ? 0u : (uint32_t)kSK) + fill % n;
        return fill < n || wait_all(&bars[SL::b_kv_empty + stage], ((fill / n) - 1) & 1);
      };
      auto publish = [&](bool is_k, uint32_t stage) {            // this warp's 32 rows of the stage are written
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bars[SL::b_kv_full + stage]);
        if (is_k) ++fill_k; else ++fill_v;
      };
      auto release = [&](int area) {
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bars[SL::b_stg_empty + area]);
        ++n_stg[area];
      };
      auto unpack_kc = [&]() -> bool {                           // area A: the scaled centroids of the keys
        if (!wait_all(&bars[SL::b_stg_full + 0], n_stg[0] & 1)) return false;
        const uint16_t* kn = reinterpret_cast<const uint16_t*>(sm + SL::stg_a_kn);
        const uint16_t* kr = reinterpret_cast<const uint16_t*>(sm + SL::stg_a_kr);
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          nrm[j] = f16_bits_to_float(kn[t * NB + j]);
          mag[j] = nrm[j] * ((TURBO_QJL_C / 128.f) * f16_bits_to_float(kr[t * NB + j]));
        }
#pragma unroll 1
        for (int c = 0; c < kQChunks; ++c) {
          uint32_t stage;
          if (!ring_slot(true, stage)) return false;
          unpack_centroid_row<InT, 4>(sm + SL::ring + stage * kChunkBytes, t, sm + SL::stg_a + (t * NB + (c >> 1)) * 48 + (c & 1) * 24, nrm[c >> 1], hsel);
          publish(true, stage);
        }
        release(0);
        return true;
      };
      auto unpack_ks = [&]() -> bool {                           // area B: the scaled residual signs of the keys
        if (!wait_all(&bars[SL::b_stg_full + 1], n_stg[1] & 1)) return false;
#pragma unroll 1
        for (int c = 0; c < kQChunks; ++c) {
          uint32_t stage;
          if (!ring_slot(true, stage)) return false;
          unpack_sign_half_row<InT>(sm + SL::ring + stage * kChunkBytes, t, sm + SL::stg_b + (t * NB + (c >> 1)) * 16 + (c & 1) * 8, mag[c >> 1], hsel);
          publish(true, stage);
        }
        release(1);
        return true;
      };
      auto unpack_v = [&](int c0, int c1) -> bool {              // area C: value chunks c0 .. c1-1 of the tile
        if (c0 == 0 && !wait_all(&bars[SL::b_stg_full + 2], n_stg[2] & 1)) return false;
        const uint16_t* vn = reinterpret_cast<const uint16_t*>(sm + SL::stg_c_vn);
#pragma unroll 1
        for (int c = c0; c < c1; ++c) {
          uint32_t stage;
          if (!ring_slot(false, stage)) return false;
          unpack_centroid_row<InT>(sm + SL::ring + stage * kChunkBytes, t, sm + SL::stg_c + (t * NB + (c >> 1)) * 48 + (c & 1) * 24, f16_bits_to_float(vn[t * NB + (c >> 1)]));
          publish(false, stage);
        }
        if (c1 == kQChunks) release(2);
        return true;
      };
      // Chunks c0 .. c1-1 of a tile of the uncompressed hot window (rotated domain, [B, Hkv, n_hot, D]): the same
      // stages, filled by TMA.  Every warp waits for the stage and arrives once (the stage's barrier counts one arrival
      // per unpack warp); the first warp's arrival carries the byte count and its lane 0 issues the load.
      auto load_hot = [&](bool is_k, int tile, int c0, int c1) -> bool {
#pragma unroll 1
        for (int c = c0; c < c1; ++c) {
          uint32_t stage;
          if (!ring_slot(is_k, stage)) return false;
          if (lane == 0) {
            void* bar = &bars[SL::b_kv_full + stage];
            if (t == 0 && hsel == 0) {   // the group's first lane
              ptx::mbar_arrive_expect_tx(bar, kChunkBytes);
              ptx::tma_load_4d(sm + SL::ring + stage * kChunkBytes, is_k ? &map_k : &map_v, c * 64, (tile - p.tiles_cold) * kBlockN, s.kvh, s.b, bar);
            } else {
              ptx::mbar_arrive(bar);
            }
          }
          if (is_k) ++fill_k; else ++fill_v;
        }
        return true;
      };
      // The keys of tile j (K ring, landing areas A and B) and, one tile behind, the values of tile j - 1 (V ring, area C)
      // are expanded by separate groups of four warps: neither waits for the other's ring.  (One group doing both spent
      // most of a tile's time in the twelve per-chunk hand-offs, one after another.)
      while (ok && it.next(s)) {
        for (int j = s.tile_lo; ok && j <= s.tile_hi; ++j) {
          const bool has_k = j < s.tile_hi, has_v = j > s.tile_lo;
          const bool k_cold = j < p.tiles_cold, v_cold = j - 1 < p.tiles_cold;
          if (v_group) {
            if (has_v) ok = v_cold ? unpack_v(0, kQChunks) : load_hot(false, j - 1, 0, kQChunks);
          } else if (has_k) {
            ok = k_cold ? (unpack_kc() && unpack_ks()) : load_hot(true, j, 0, kQChunks);
          }
        }
      }
    }
  } else if (warp >= 2 && warp < 2 + 8) {
    if constexpr (TURBO) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kTurboRegsSoftmax));
    // ====================================== softmax ======================================
    // Two threads per query row: warps 2-5 take key columns 0-63 of every tile (and the lower
    // half of O's columns), warps 6-9 columns 64-127 (upper half).  Both warps of a pair touch
    // the same tensor-memory lane quarter.  The two partial row maxima of a tile (and the two
    // partial sums at the end of a segment) are exchanged through shared memory.
    const int wq = pw & 3;                         // tensor-memory lane quarter this (physical) warp may touch
    const int half = (warp - 2) >> 2;              // which 64 key columns / which half of O
    const int row = wq * 32 + lane;                // query row of the unit tile = tensor-memory lane
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    float* xch = reinterpret_cast<float*>(sm + SL::xch);                 // [2 slots][2 halves][128 rows]
    volatile uint32_t* xseq = reinterpret_cast<volatile uint32_t*>(sm + SL::xseq);   // [2 slots][2 halves][4 quarters]
    uint32_t xcount = 0;                            // exchanges done so far (same in both halves)
    // publish `mine`, return the partner's value for the same row; false if the partner never came
    auto exchange = [&](float mine, float& theirs) -> bool {
      const uint32_t slot = xcount & 1u;
      xch[(slot * 2 + half) * kRowsM + row] = mine;
      __syncwarp();
      __threadfence_block();
      if (lane == 0) xseq[(slot * 2 + half) * 4 + wq] = xcount + 1;
      bool got = false;
      for (uint32_t i = 0; i < ptx::kWaitPolls; ++i) {
        if (xseq[(slot * 2 + (half ^ 1)) * 4 + wq] >= xcount + 1) { got = true; break; }
        if ((i & 63u) == 63u && *abort_flag) break;
      }
      got = __all_sync(0xffffffffu, got);
      if (!got) {
        if (lane == 0 && !*abort_flag) { *abort_flag = 1; atomicExch(p.status, kStatusExchangeWait); }
        return false;
      }
      __threadfence_block();
      theirs = xch[(slot * 2 + (half ^ 1)) * kRowsM + row];
      ++xcount;
      return true;
    };
    // Meeting point of the eight softmax warps (bounded like every other wait in this kernel).
    volatile uint32_t* gctr = reinterpret_cast<volatile uint32_t*>(sm + SL::misc) + 4;
    volatile int* merge_go = reinterpret_cast<volatile int*>(sm + SL::misc) + 5;
    uint32_t gcount = 0;
    auto group_sync = [&]() -> bool {
      ++gcount;
      __syncwarp();
      if (lane == 0) {
        __threadfence_block();
        atomicAdd(const_cast<uint32_t*>(gctr), 1u);
      }
      bool got = false;
      for (uint32_t i = 0; i < ptx::kWaitPolls; ++i) {
        if (*gctr >= gcount * 8u) { got = true; break; }
        if ((i & 63u) == 63u && *abort_flag) break;
      }
      got = __all_sync(0xffffffffu, got);
      if (!got) {
        if (lane == 0 && !*abort_flag) { *abort_flag = 1; atomicExch(p.status, kStatusGroupWait); }
        return false;
      }
      __threadfence_block();
      return true;
    };
    if (begin < end) {
      SegmentIter it(p, begin, end, unit0, tile0);
      Segment s;
      uint32_t seg_idx = 0, tile_ctr = 0;
      bool ok = true;
      constexpr int kOHalf = D / 2;                 // O columns handled by this thread
      while (ok && it.next(s)) {
        const int ntiles = s.tile_hi - s.tile_lo;
        const int rr = s.mt * kRowsM + row;          // row inside the (b, kvh) group
        const int tok = rr & 15;                     // draft token index of this row
        const int last_visible = s.n_keys - 16 + tok;
        const InT* mrow = nullptr;                   // this row of the additive mask [B, Hq, 16, N]
        if (MASK && rr < p.R)
          mrow = reinterpret_cast<const InT*>(a.mask) + ((((long long)s.b * a.Hq + (long long)s.kvh * p.G + (rr >> 4)) * 16) + tok) * (long long)a.N;
        float m_ref = -INFINITY;                     // reference maximum (raw score units), same in both halves
        float l_sum = 0.f;                           // this half's share of the row sum
        for (int jj = 0; ok && jj < ntiles; ++jj) {
          const uint32_t t = tile_ctr + jj, buf = t & 1;
          const int j = s.tile_lo + jj;
          uint32_t mk[32];
          if constexpr (MASK) load_mask64<InT>(mrow, j * kBlockN + half * 64, a.N, p.mask_vec != 0, mk);   // in flight while S is computed
          {
            TR_T0();
            ok = wait_or_abort(&bars[SL::b_s_full + buf], (t >> 1) & 1, abort_flag, p.status);
            TR_ACC(20); if (threadIdx.x == 64) { if (t == 0) TR_STAMP(3); if (t < 40) TR_STAMP(24 + t); }
          }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          ptx::tc_fence_after();
          const uint32_t s_addr = tmem_base + lane_addr + kColS + buf * kBlockN;
          uint32_t sr[2][32];
          ptx::tmem_ld32(s_addr + half * 64, sr[0]);
          ptx::tmem_ld32(s_addr + half * 64 + 32, sr[1]);
          ptx::tmem_ld_wait();
          const int n_base = j * kBlockN + half * 64;
          if constexpr (MASK) {
            // softmax(scale * (s + mask / scale)): the mask joins the raw scores; an entry below the dtype's
            // lowest finite value (or a NaN) hides the key
#pragma unroll
            for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const float2 mv = unpack2<InT>(mk[q2 * 16 + (i >> 1)]);
                sr[q2][i] = __float_as_uint(mv.x >= mask_floor<InT>() ? fmaf(mv.x, p.inv_scale, __uint_as_float(sr[q2][i])) : -INFINITY);
                sr[q2][i + 1] = __float_as_uint(mv.y >= mask_floor<InT>() ? fmaf(mv.y, p.inv_scale, __uint_as_float(sr[q2][i + 1])) : -INFINITY);
              }
          }
          if (n_base + 63 > s.n_keys - 16) {        // this half touches the block keys or the end
#pragma unroll
            for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (n_base + q2 * 32 + i > last_visible) sr[q2][i] = __float_as_uint(-INFINITY);
          }
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
            for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sr[q2][i]));
          float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
          float other;
          ok = exchange(mx, other);
          if (!ok) break;
          mx = fmaxf(mx, other);
          // lazy rescale: move the reference only when the maximum grew by more than 2^8
          float factor = 1.f;
          const bool grow = (mx > m_ref) && ((mx - m_ref) * p.scale_log2 > kRescaleThreshold || m_ref == -INFINITY);
          if (grow) {
            factor = (m_ref == -INFINITY) ? 0.f : fast_exp2((m_ref - mx) * p.scale_log2);
            m_ref = mx;
          }
          const bool need_rescale = jj > 0 && __any_sync(0xffffffffu, grow);
          l_sum *= factor;
          const float neg_ref = (m_ref == -INFINITY) ? 0.f : -m_ref * p.scale_log2;
          uint32_t pr[32];
          float add4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float p0 = fast_exp2(fmaf(__uint_as_float(sr[q2][i]), p.scale_log2, neg_ref));
              const float p1 = fast_exp2(fmaf(__uint_as_float(sr[q2][i + 1]), p.scale_log2, neg_ref));
              add4[(i >> 1) & 3] += p0 + p1;
              pr[q2 * 16 + (i >> 1)] = pack2<InT>(p0, p1);
            }
          l_sum += (add4[0] + add4[1]) + (add4[2] + add4[3]);
          if (jj > 0) {
            // Every phase of the product barrier is waited for exactly once and in order (a
            // parity wait that skips a phase cannot tell "done" from "two phases behind").
            // It sits after the exponentials: the next product cannot start before the
            // previous one retires anyway, so nothing is lost by waiting here.
            TR_T0();
            ok = wait_or_abort(&bars[SL::b_pv_done], (t - 1) & 1, abort_flag, p.status);
            TR_ACC(21);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
          }
          if (need_rescale) {
            // O holds the products up to tile j-1: scale this row's half of the columns
            ptx::tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < kOHalf / 32; ++c) {
              uint32_t o[32];
              const uint32_t o_addr = tmem_base + lane_addr + kColO + half * kOHalf + c * 32;
              ptx::tmem_ld32(o_addr, o);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
              ptx::tmem_st32(o_addr, o);
            }
            ptx::tmem_st_wait();
          }
          ptx::tmem_st32(s_addr + half * 32, pr);   // P: 16-bit pairs, key 2c and 2c+1 in column c
          ptx::tmem_st_wait();
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&bars[SL::b_p_full + buf]);
        }
        if (!ok) break;
        // ---- segment epilogue: wait for the last product, then normalise / store ----
        {
          const uint32_t t_last = tile_ctr + ntiles - 1;
          if (threadIdx.x == 64) TR_STAMP(4 + 4 * (seg_idx > 0));
          ok = wait_or_abort(&bars[SL::b_pv_done], t_last & 1, abort_flag, p.status);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (threadIdx.x == 64) TR_STAMP(5 + 4 * (seg_idx > 0));
          float l_other;
          ok = exchange(l_sum, l_other);
          if (!ok) break;
          const float l_tot = half == 0 ? l_sum + l_other : l_other + l_sum;   // same order in both halves
          ptx::tc_fence_after();
          const bool valid = rr < p.R;
          if (p.pair) {
            // ---- the unit's other half of the keys is in the cluster partner: swap columns ----
            // Each thread owns two quarters of the head dimension; it keeps quarter 2*half + rank and
            // sends quarter 2*half + (1 - rank) to the same thread of the partner, whose ring buffer
            // is free once the partner has said so.
            constexpr int kQuart = D / 4;
            const uint32_t rank = cluster_rank(), peer = rank ^ 1u;
            const float m_log2 = (m_ref == -INFINITY) ? -INFINITY : m_ref * p.scale_log2;
            float* recv = reinterpret_cast<float*>(sm + SL::ring);              // [half][kQuart / 4][128 rows][4]
            ok = group_sync();                                                 // every warp is done with xch and the ring
            if (!ok) break;
            if (warp == 2 && lane == 0) peer_arrive(peer_addr(&bars[SL::b_peer_ready], peer));
            ok = wait_peer_or_abort(&bars[SL::b_peer_ready], 0, abort_flag, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (half == 0) {
              peer_store1(peer_addr(xch + row, peer), m_log2);
              peer_store1(peer_addr(xch + kRowsM + row, peer), l_tot);
            }
            {
              const int q_send = 2 * half + (int)peer;
              const uint32_t dst = peer_addr(recv + ((long long)(half * (kQuart / 4)) * kRowsM + row) * 4, peer);
#pragma unroll
              for (int c = 0; c < kQuart / 32; ++c) {
                uint32_t o[32];
                ptx::tmem_ld32(tmem_base + lane_addr + kColO + q_send * kQuart + c * 32, o);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  peer_store(dst + (uint32_t)((c * 8 + i) * kRowsM * 16), __uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]),
                             __uint_as_float(o[4 * i + 2]), __uint_as_float(o[4 * i + 3]));
              }
            }
            peer_arrive(peer_addr(&bars[SL::b_peer_data], peer));              // release: this thread's stores first
            ok = wait_peer_or_abort(&bars[SL::b_peer_data], 0, abort_flag, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            {
              // rank 0 holds the earlier keys: fixed order (rank 0, rank 1) in both CTAs
              const float m_peer = xch[row], l_peer = xch[kRowsM + row];
              const float m0 = rank == 0 ? m_log2 : m_peer, m1 = rank == 0 ? m_peer : m_log2;
              const float l0 = rank == 0 ? l_tot : l_peer, l1 = rank == 0 ? l_peer : l_tot;
              const float mmax = fmaxf(m0, m1);
              const float f0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - mmax), f1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - mmax);
              const float den = f0 * l0 + f1 * l1;
              const float inv = den == 0.f ? 1.f : 1.f / den;
              const float f_own = rank == 0 ? f0 : f1, f_oth = rank == 0 ? f1 : f0;
              const int q_keep = 2 * half + (int)rank;
              InT* orow = reinterpret_cast<InT*>(a.out) +
                          ((((long long)s.b * a.Hq + (long long)s.kvh * p.G + (rr >> 4)) * 16) + tok) * D + q_keep * kQuart;
              const float4* src = reinterpret_cast<const float4*>(recv) + (long long)(half * (kQuart / 4)) * kRowsM + row;
#pragma unroll
              for (int c = 0; c < kQuart / 32; ++c) {
                uint32_t o[32];
                ptx::tmem_ld32(tmem_base + lane_addr + kColO + q_keep * kQuart + c * 32, o);
                ptx::tmem_ld_wait();
                uint32_t w[16];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float4 v4 = src[(c * 8 + i) * kRowsM];
                  const float oth[4] = {v4.x, v4.y, v4.z, v4.w};
                  float r4[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float mine = __uint_as_float(o[4 * i + e]);
                    r4[e] = (rank == 0 ? fmaf(f_oth, oth[e], f_own * mine) : fmaf(f_own, mine, f_oth * oth[e])) * inv;
                  }
                  w[2 * i] = pack2<InT>(r4[0], r4[1]);
                  w[2 * i + 1] = pack2<InT>(r4[2], r4[3]);
                }
                if (valid) {
#pragma unroll
                  for (int i = 0; i < 4; ++i)
                    *reinterpret_cast<uint4*>(orow + c * 32 + i * 8) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
                }
              }
            }
          } else if (s.slot < 0) {
            const float inv = l_tot == 0.f ? 1.f : 1.f / l_tot;
            InT* orow = reinterpret_cast<InT*>(a.out) +
                        ((((long long)s.b * a.Hq + (long long)s.kvh * p.G + (rr >> 4)) * 16) + tok) * D + half * kOHalf;
#pragma unroll 1
            for (int c = 0; c < kOHalf / 32; ++c) {
              uint32_t o[32];
              ptx::tmem_ld32(tmem_base + lane_addr + kColO + half * kOHalf + c * 32, o);
              ptx::tmem_ld_wait();
              if (valid) {
                uint32_t w[16];
#pragma unroll
                for (int i = 0; i < 16; ++i)
                  w[i] = pack2<InT>(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  *reinterpret_cast<uint4*>(orow + c * 32 + i * 8) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
              }
            }
          } else {
            // ---- partial range: publish (O, m, l); merge here if this CTA is the unit's last finisher ----
            const float m_log2 = (m_ref == -INFINITY) ? -INFINITY : m_ref * p.scale_log2;
            float* pslot = p.part_o + (long long)s.slot * kRowsM * D;
#pragma unroll 1
            for (int c = 0; c < kOHalf / 32; c += 2) {
              uint32_t o[2][32];
              ptx::tmem_ld32(tmem_base + lane_addr + kColO + half * kOHalf + c * 32, o[0]);
              ptx::tmem_ld32(tmem_base + lane_addr + kColO + half * kOHalf + c * 32 + 32, o[1]);
              ptx::tmem_ld_wait();
              const int col4 = (half * kOHalf + c * 32) >> 2;
#pragma unroll
              for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  *reinterpret_cast<uint4*>(pslot + ((long long)(col4 + h2 * 8 + i) * kRowsM + row) * 4) =
                      make_uint4(o[h2][4 * i], o[h2][4 * i + 1], o[h2][4 * i + 2], o[h2][4 * i + 3]);
            }
            if (half == 0) {
              p.part_m[(long long)s.slot * kRowsM + row] = m_log2;
              p.part_l[(long long)s.slot * kRowsM + row] = l_tot;
            }
            // the unit's ranges live in CTAs cta_first .. cta_last
            const int cta_first = cta_of(p, total, s.unit_begin);
            const int cta_last = cta_of(p, total, s.unit_begin + s.tiles_in_unit - 1);
            const int nseg = cta_last - cta_first + 1;
            if (nseg > kFusedMax) {
              if (half == 0 && row == 0) p.slot_unit[s.slot] = s.unit;      // left to the merge kernel
            } else {
              // the group's stores are ordered before the leader's release by the meeting point
              // (block scope) followed by the leader's device-scope fence
              ok = group_sync();
              if (!ok) break;
              if (threadIdx.x == 64) TR_STAMP(6 + 4 * (seg_idx > 0));
              if (warp == 2 && lane == 0) {
                __threadfence();
                st_release_u64(p.flags + s.slot, p.epoch);
                fence_sc();
                bool all = true;
                for (int i = cta_first; i <= cta_last; ++i) {
                  const int sl = (i == cta_first) ? 2 * i + 1 : 2 * i;
                  if (sl != s.slot) all = all && (ld_acquire_u64(p.flags + sl) == p.epoch);
                }
                // The CTA that sees every range of the unit arrived merges, and clears the unit's flags: a launch
                // replayed from a CUDA graph carries the same epoch every time and must not find the flags of its
                // previous run.  (A range's owner sets its flag once per launch, before anybody can see it set, so a
                // clear never overtakes a set; a CTA that reads cleared flags leaves the merge to the one that cleared.)
                if (all)
                  for (int i = cta_first; i <= cta_last; ++i) st_release_u64(p.flags + ((i == cta_first) ? 2 * i + 1 : 2 * i), 0ull);
                *merge_go = all ? 1 : 0;
              }
              ok = group_sync();
              if (!ok) break;
              if (*merge_go) {
                // slot order = key order; this CTA's own range takes its place in the same order,
                // so the result does not depend on which CTA merges
                float f[kFusedMax], mmax = -INFINITY, den = 0.f;
                int sl[kFusedMax];
#pragma unroll
                for (int i = 0; i < kFusedMax; ++i) {
                  sl[i] = (i == 0) ? 2 * cta_first + 1 : 2 * (cta_first + i);
                  f[i] = -INFINITY;
                  if (i < nseg) {
                    f[i] = sl[i] == s.slot ? m_log2 : __ldcg(p.part_m + (long long)sl[i] * kRowsM + row);
                    mmax = fmaxf(mmax, f[i]);
                  }
                }
#pragma unroll
                for (int i = 0; i < kFusedMax; ++i) {
                  f[i] = (f[i] == -INFINITY) ? 0.f : exp2f(f[i] - mmax);
                  if (i < nseg) den += f[i] * (sl[i] == s.slot ? l_tot : __ldcg(p.part_l + (long long)sl[i] * kRowsM + row));
                }
                const float inv = den == 0.f ? 1.f : 1.f / den;
                InT* orow = reinterpret_cast<InT*>(a.out) +
                            ((((long long)s.b * a.Hq + (long long)s.kvh * p.G + (rr >> 4)) * 16) + tok) * D + half * kOHalf;
                auto store32 = [&](int c, const float (&acc)[32]) {
                  if (valid) {
                    uint32_t w[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) w[i] = pack2<InT>(acc[2 * i] * inv, acc[2 * i + 1] * inv);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                      *reinterpret_cast<uint4*>(orow + c * 32 + i * 8) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
                  }
                };
                if (nseg == 2) {
                  // the common case: the other range's columns are fetched one chunk ahead
                  const bool own_first = sl[0] == s.slot;
                  const float f_own = own_first ? f[0] : f[1], f_oth = own_first ? f[1] : f[0];
                  const float* src = p.part_o + (long long)(own_first ? sl[1] : sl[0]) * kRowsM * D;
                  float4 nxt[8];
                  auto fetch = [&](int c) {
                    const int col4 = (half * kOHalf + c * 32) >> 2;
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                      nxt[i] = __ldcg(reinterpret_cast<const float4*>(src + ((long long)(col4 + i) * kRowsM + row) * 4));
                  };
                  fetch(0);
#pragma unroll
                  for (int c = 0; c < kOHalf / 32; ++c) {
                    uint32_t o[32];
                    ptx::tmem_ld32(tmem_base + lane_addr + kColO + half * kOHalf + c * 32, o);
                    float oth[32];
#pragma unroll
                    for (int i = 0; i < 8; ++i) { oth[4 * i] = nxt[i].x; oth[4 * i + 1] = nxt[i].y; oth[4 * i + 2] = nxt[i].z; oth[4 * i + 3] = nxt[i].w; }
                    if (c + 1 < kOHalf / 32) fetch(c + 1);
                    ptx::tmem_ld_wait();
                    float acc[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                      const float mine = __uint_as_float(o[i]);
                      // slot order: 0 + f0 v0, then + f1 v1 (as the general path below computes it)
                      acc[i] = own_first ? fmaf(f_oth, oth[i], fmaf(f_own, mine, 0.f)) : fmaf(f_own, mine, fmaf(f_oth, oth[i], 0.f));
                    }
                    store32(c, acc);
                  }
                } else {
#pragma unroll 1
                  for (int c = 0; c < kOHalf / 32; ++c) {
                    uint32_t o[32];
                    ptx::tmem_ld32(tmem_base + lane_addr + kColO + half * kOHalf + c * 32, o);
                    ptx::tmem_ld_wait();
                    float acc[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc[i] = 0.f;
                    const int col4 = (half * kOHalf + c * 32) >> 2;
#pragma unroll
                    for (int g = 0; g < kFusedMax; ++g) {
                      if (g < nseg) {
                        if (sl[g] == s.slot) {
#pragma unroll
                          for (int i = 0; i < 32; ++i) acc[i] = fmaf(f[g], __uint_as_float(o[i]), acc[i]);
                        } else {
                          const float* src = p.part_o + (long long)sl[g] * kRowsM * D;
#pragma unroll
                          for (int i = 0; i < 8; ++i) {
                            const float4 v4 = __ldcg(reinterpret_cast<const float4*>(src + ((long long)(col4 + i) * kRowsM + row) * 4));
                            acc[4 * i] = fmaf(f[g], v4.x, acc[4 * i]); acc[4 * i + 1] = fmaf(f[g], v4.y, acc[4 * i + 1]);
                            acc[4 * i + 2] = fmaf(f[g], v4.z, acc[4 * i + 2]); acc[4 * i + 3] = fmaf(f[g], v4.w, acc[4 * i + 3]);
                          }
                        }
                      }
                    }
                    store32(c, acc);
                  }
                }
              }
            }
          }
          if (threadIdx.x == 64) TR_STAMP(7 + 4 * (seg_idx > 0));
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&bars[SL::b_o_free]);
        }
        tile_ctr += ntiles;
        ++seg_idx;
      }
    }
  }

  // No CTA of a pair may leave while its partner can still write into its shared memory.  Every
  // wait above is bounded, so both always get here.
  if (p.pair) cluster_sync_all();
  if (warp == 0 && lane == 0) TR_FLUSH(16, 16);
  if (warp == 1 && lane == 0) { TR_FLUSH(17, 17); TR_FLUSH(22, 22); }
  if (warp == kThreads / 32 && lane == 0) { TR_FLUSH(18, 19); TR_FLUSH(23, 23); }
  if (warp == 2 && lane == 0) TR_FLUSH(20, 21);
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) TR_STAMP(12);
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- merge of the split-KV partials ----------------------------------------------------------
// One block per (unit, 32 rows, 16 columns); the ranges of a unit are summed in slot order.
template <typename InT, int D>
__global__ void __launch_bounds__(128) sdpa_tc_merge_kernel(const TcParams p, int n_slots, int max_ranges) {
  // One CTA (4 warps) combines 32 rows x 4 float4 columns of one unit: lane = row (the partials keep the 128 rows of a float4
  // column contiguous, so a warp reads 512 contiguous bytes per range), warp = column.  A unit has at most one range
  // per CTA of the main kernel, so the limit of 320 covers every GPU with up to 320 SMs; more is reported, not dropped.
  // The per-range weights live in dynamic shared memory sized by the launcher for the most ranges a unit of this
  // launch can have (`max_ranges`, at most one per CTA of the main kernel): a fixed array for 320 ranges would be 40 KB
  // and leave room for five of these small CTAs per SM, two waves for a grid of a thousand.
  constexpr int kMaxRangesLimit = 320;
  const int kMaxRanges = max_ranges < kMaxRangesLimit ? max_ranges : kMaxRangesLimit;
  __shared__ int s_slots[kMaxRangesLimit];
  __shared__ int s_raw[2 * kMaxRangesLimit];    // copy of the slot table (two slots per CTA of the main kernel)
  extern __shared__ float s_f_raw[];
  float (*s_f)[32] = reinterpret_cast<float (*)[32]>(s_f_raw);   // per range and row: the range's maximum, then exp2(m - max over the ranges)
  __shared__ float s_red[4][32];           // per warp and row: partial maximum, then partial denominator
  __shared__ int s_count;
  // Launched with programmatic stream serialization behind the main kernel (which lets its dependents go as soon as all
  // of its CTAs are placed): the CTAs of this grid are resident when the main kernel ends; nothing is read before the wait.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int unit = blockIdx.x, rgrp = blockIdx.y, cgrp = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // Every global load of the set-up below is issued together with its neighbours (a chain of dependent loads, one
  // L2 round trip each, used to take most of this kernel's time): the slot table first, then the maxima, then the sums.
  const int n_scan = n_slots < 2 * kMaxRangesLimit ? n_slots : 2 * kMaxRangesLimit;
  for (int i = threadIdx.x; i < n_scan; i += 128) s_raw[i] = p.slot_unit[i];
  __syncthreads();
  // slots of this unit, in slot order (a fixed summation order keeps results bit-reproducible)
  if (threadIdx.x < 32) {
    int count = 0;
    for (int base = 0; base < n_scan; base += 32) {
      const int i = base + threadIdx.x;
      const bool hit = i < n_scan && s_raw[i] == unit;
      const unsigned m = __ballot_sync(0xffffffffu, hit);
      const int pos = count + __popc(m & ((1u << threadIdx.x) - 1u));
      if (hit && pos < kMaxRanges) s_slots[pos] = i;
      count += __popc(m);
    }
    if (threadIdx.x == 0) {
      s_count = count;
      if (count > kMaxRanges || n_slots > n_scan) atomicExch(p.status, kStatusMergeRanges);
    }
  }
  __syncthreads();
  const int cnt = s_count < kMaxRanges ? s_count : kMaxRanges;
  if (cnt == 0) return;   // the unit was written directly by a CTA that covered all of it
  const SdpaArgs& a = p.a;
  const int per_b = a.Hkv * p.MT;
  const int b = unit / per_b, kvh = (unit / p.MT) % a.Hkv, mt = unit % p.MT;
  const int r = rgrp * 32 + lane;                        // row of the 128-row tile
  const int rr = mt * kRowsM + r;
  // per-row weights once per CTA: warp w takes ranges w, w + 4, ...; partial results meet in shared memory and are
  // combined in warp order by everybody (the same bits in every warp and in every CTA of the unit)
  {
    float pm = -INFINITY;
    int i = warp;
    for (; i + 12 < cnt; i += 16) {
      float m[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) m[u] = __ldcg(p.part_m + (long long)s_slots[i + 4 * u] * kRowsM + r);
#pragma unroll
      for (int u = 0; u < 4; ++u) { s_f[i + 4 * u][lane] = m[u]; pm = fmaxf(pm, m[u]); }
    }
    for (; i < cnt; i += 4) {
      const float m = __ldcg(p.part_m + (long long)s_slots[i] * kRowsM + r);
      s_f[i][lane] = m;
      pm = fmaxf(pm, m);
    }
    s_red[warp][lane] = pm;
  }
  __syncthreads();
  const float mmax = fmaxf(fmaxf(s_red[0][lane], s_red[1][lane]), fmaxf(s_red[2][lane], s_red[3][lane]));
  __syncthreads();
  {
    float pd = 0.f;
    int i = warp;
    for (; i + 12 < cnt; i += 16) {
      float l[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) l[u] = __ldcg(p.part_l + (long long)s_slots[i + 4 * u] * kRowsM + r);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float m = s_f[i + 4 * u][lane];
        const float f = (m == -INFINITY) ? 0.f : exp2f(m - mmax);
        s_f[i + 4 * u][lane] = f;
        pd += f * l[u];
      }
    }
    for (; i < cnt; i += 4) {
      const float m = s_f[i][lane];
      const float f = (m == -INFINITY) ? 0.f : exp2f(m - mmax);
      s_f[i][lane] = f;
      pd += f * __ldcg(p.part_l + (long long)s_slots[i] * kRowsM + r);
    }
    s_red[warp][lane] = pd;
  }
  __syncthreads();
  if (rr >= p.R) return;
  const float den = (s_red[0][lane] + s_red[1][lane]) + (s_red[2][lane] + s_red[3][lane]);
  const float inv = den == 0.f ? 1.f : 1.f / den;
  const int c4 = cgrp * 4 + warp;                        // float4 index inside the row
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const float* src = p.part_o + ((long long)c4 * kRowsM + r) * 4;
  int i = 0;
  for (; i + 16 <= cnt; i += 16) {                        // sixteen independent loads in flight
    float4 v[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) v[u] = __ldcg(reinterpret_cast<const float4*>(src + (long long)s_slots[i + u] * kRowsM * D));
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const float f = s_f[i + u][lane];
      acc.x += f * v[u].x; acc.y += f * v[u].y; acc.z += f * v[u].z; acc.w += f * v[u].w;
    }
  }
  for (; i + 4 <= cnt; i += 4) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = __ldcg(reinterpret_cast<const float4*>(src + (long long)s_slots[i + u] * kRowsM * D));
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float f = s_f[i + u][lane];
      acc.x += f * v[u].x; acc.y += f * v[u].y; acc.z += f * v[u].z; acc.w += f * v[u].w;
    }
  }
  for (; i < cnt; ++i) {
    const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (long long)s_slots[i] * kRowsM * D));
    const float f = s_f[i][lane];
    acc.x += f * v.x; acc.y += f * v.y; acc.z += f * v.z; acc.w += f * v.w;
  }
  InT* orow = reinterpret_cast<InT*>(a.out) + ((((long long)b * a.Hq + (long long)kvh * p.G + (rr >> 4)) * 16) + (rr & 15)) * D + c4 * 4;
  *reinterpret_cast<uint2*>(orow) = make_uint2(pack2<InT>(acc.x * inv, acc.y * inv), pack2<InT>(acc.z * inv, acc.w * inv));
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

size_t tc_workspace_bytes(int D) {
  const size_t slots = 2 * (size_t)sm_count();
  return align_up(slots * sizeof(int), 256) + align_up(slots * sizeof(unsigned long long), 256) +
         slots * kRowsM * ((size_t)D + 2) * sizeof(float);
}

// Tag of a launch: arrival flags left in a workspace by earlier launches (or whatever else the
// memory held) must not compare equal to it.  Starts from a per-process random value.
unsigned long long next_epoch() {
  static std::atomic<unsigned long long> counter{[] {
    std::random_device rd;
    return (((unsigned long long)rd() << 32) ^ rd()) | 1ull;
  }()};
  unsigned long long e = counter.fetch_add(1);
  return e ? e : counter.fetch_add(1);
}

template <typename InT, int D, bool MASK, bool TURBO>
int32_t launch_typed(const SdpaArgs& a, const TurboKvArgs* turbo, cudaStream_t stream) {
  using SL = Smem<D, TURBO>;
  EncodeTiledFn encode = tensor_map_encoder();
  if (!encode) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return DFLASH_ERR_CUDA; }
  int* status = device_status_word();
  if (!status) { set_error("no CUDA device"); return DFLASH_ERR_CUDA; }
  const size_t need = tc_workspace_bytes(D);
  if (!a.workspace || a.workspace_bytes < need) {
    set_error("verify_sdpa: workspace of %zu bytes needed, %zu given", need, a.workspace_bytes);
    return DFLASH_ERR_WORKSPACE;
  }
  TcParams p;
  p.a = a;
  p.G = a.Hq / a.Hkv;
  p.R = p.G * 16;
  p.MT = (p.R + kRowsM - 1) / kRowsM;
  p.units = a.B * a.Hkv * p.MT;
  const long long tiles_per_unit = (a.N + kBlockN - 1) / kBlockN;
  p.total_tiles = tiles_per_unit * p.units;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.inv_scale = 1.f / a.scale;
  p.mask_vec = (a.mask && (reinterpret_cast<uintptr_t>(a.mask) & 15u) == 0 && a.N % 8 == 0) ? 1 : 0;
  p.status = status;
  p.t_kp = p.t_ks = p.t_vp = nullptr;
  p.t_kn = p.t_kr = p.t_vn = nullptr;
  p.n_cold = p.tiles_cold = 0;
  if (TURBO) {
    p.t_kp = turbo->kp; p.t_ks = turbo->ks; p.t_kn = turbo->kn; p.t_kr = turbo->kr; p.t_vp = turbo->vp; p.t_vn = turbo->vn;
    p.n_cold = turbo->n_cold;
    p.tiles_cold = turbo->n_cold / kBlockN;
  }
  const int n_sm = sm_count();
  long long grid = p.total_tiles < n_sm ? p.total_tiles : n_sm;   // upper bound also for ragged lengths
  if (grid < 1) grid = 1;
  // equal cuts of every unit when the units divide the SMs well, stream-K ranges otherwise
  p.split = 0;
  p.pair = 0;
  bool need_merge_kernel = true;
  if (!a.kv_len) {
    const int c = n_sm / p.units;
    constexpr int mode = -1;   // -1: choose; 0: always stream-K; > 0: equal cuts whenever they apply (for experiments, at compile time)
    // Equal cuts leave n_sm - units * c SMs idle.  With long units that costs more than stream-K's partials and merge
    // (measured: about ten key tiles' worth of time): B=60, N=16400 runs 12 % faster as stream-K, B=64, N=4112 4 % slower.
    const double idle_tiles = c >= 1 ? (double)tiles_per_unit / c * (1.0 - (double)p.units * c / n_sm) : 0.0;
    if (mode != 0 && c >= 1 && c <= kFusedMax && tiles_per_unit >= c && (long long)p.units * c * 5 >= (long long)n_sm * 4 &&
        (mode > 0 || idle_tiles < (TURBO ? 3.0 : 10.0))) {   // a compressed tile costs ~4x a dense one: idle SMs cost more than partials
      p.split = c;
      p.pair = (c == 2 && !TURBO) ? 1 : 0;   // compressed KV: the two ranges of a unit meet through the partials instead
      grid = (long long)p.units * c;
      need_merge_kernel = false;
    } else {
      // stream-K: the merge kernel is only needed if some unit is cut into more than kFusedMax ranges
      int worst = 1;
      for (int u = 0; u < p.units; ++u) {
        const long long lo = (long long)u * tiles_per_unit, hi = lo + tiles_per_unit - 1;
        const int n = (int)(((hi + 1) * grid - 1) / p.total_tiles - ((lo + 1) * grid - 1) / p.total_tiles) + 1;
        worst = n > worst ? n : worst;
      }
      need_merge_kernel = worst > kFusedMax;
    }
  }
  p.epoch = next_epoch();
  const size_t slots = 2 * (size_t)n_sm;
  uint8_t* ws = reinterpret_cast<uint8_t*>(a.workspace);
  p.slot_unit = reinterpret_cast<int*>(ws);
  p.flags = reinterpret_cast<unsigned long long*>(ws + align_up(slots * sizeof(int), 256));
  p.part_o = reinterpret_cast<float*>(ws + align_up(slots * sizeof(int), 256) + align_up(slots * sizeof(unsigned long long), 256));
  p.part_m = p.part_o + slots * kRowsM * (size_t)D;
  p.part_l = p.part_m + slots * kRowsM;

  const CUtensorMapDataType dt = std::is_same<InT, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap mq, mq2, mk, mv;
  auto encode_q = [&](CUtensorMap* m, const void* base) -> CUresult {
    // Q as (d, row in (b,kvh) group, b*Hkv+kvh): rows past the group read as zeros
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)p.R, (cuuint64_t)a.B * a.Hkv};
    const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)p.R * D * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)kRowsM, 1};
    const cuuint32_t es[3] = {1, 1, 1};
    return encode(m, dt, 3, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  {
    CUresult r = encode_q(&mq, a.q);
    if (r == CUDA_SUCCESS) r = encode_q(&mq2, TURBO ? turbo->q2 : a.q);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled(q) failed with CUresult %d", (int)r); return DFLASH_ERR_CUDA; }
  }
  auto encode_kv = [&](CUtensorMap* m, const void* base) -> CUresult {
    cuuint64_t dims[4], strides[3];
    if (a.page_table) {
      // pool [num_pages, Hkv, page_tokens, D]: a page coordinate at or beyond num_pages is filled with zeros
      dims[0] = D; dims[1] = a.page_tokens; dims[2] = a.Hkv; dims[3] = (cuuint64_t)a.num_pages;
      strides[0] = (cuuint64_t)D * 2; strides[1] = (cuuint64_t)a.page_tokens * D * 2; strides[2] = (cuuint64_t)a.Hkv * a.page_tokens * D * 2;
    } else if (TURBO) {
      // the hot window in the rotated domain, [B, Hkv, n_hot, D]; rows at or beyond n_hot read as zeros
      const cuuint64_t n_hot = turbo->n_hot > 0 ? turbo->n_hot : 1;
      dims[0] = D; dims[1] = n_hot; dims[2] = a.Hkv; dims[3] = a.B;
      strides[0] = (cuuint64_t)D * 2; strides[1] = n_hot * D * 2; strides[2] = (cuuint64_t)a.Hkv * n_hot * D * 2;
    } else {
      dims[0] = D; dims[1] = a.N; dims[2] = a.Hkv; dims[3] = a.B;
      strides[0] = (cuuint64_t)D * 2; strides[1] = (cuuint64_t)a.N * D * 2; strides[2] = (cuuint64_t)a.Hkv * a.N * D * 2;
    }
    const cuuint32_t box[4] = {64, (cuuint32_t)kBlockN, 1, 1};
    const cuuint32_t es[4] = {1, 1, 1, 1};
    return encode(m, dt, 4, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  // compressed KV without a hot window: no tile ever uses these two maps; they cover the first query tile instead
  const bool no_hot = TURBO && turbo->n_hot <= 0;
  CUresult r = no_hot ? encode_q(&mk, a.q) : encode_kv(&mk, a.k);
  if (r == CUDA_SUCCESS) r = no_hot ? encode_q(&mv, a.q) : encode_kv(&mv, a.v);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled(k/v) failed with CUresult %d", (int)r); return DFLASH_ERR_CUDA; }

  auto kernel = sdpa_tc_kernel<InT, D, MASK, TURBO>;
  constexpr int kNumThreads = ThreadsOf<TURBO>::value;
  DFLASH_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SL::alloc));
  if (p.pair) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kNumThreads);
    cfg.dynamicSmemBytes = SL::alloc;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see the top of the kernel
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    DFLASH_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, mq, mq2, mk, mv, p));
  } else {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kNumThreads);
    cfg.dynamicSmemBytes = SL::alloc;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see the top of the kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DFLASH_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, mq, mq2, mk, mv, p));
  }
  DFLASH_LAUNCH_CHECK();
  count_launch();
  if (need_merge_kernel) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.units, kRowsM / 32, D / 16);
    cfg.blockDim = dim3(128);
    const int max_ranges = (int)grid;                       // a unit has at most one range per CTA of the main kernel
    cfg.dynamicSmemBytes = (size_t)(max_ranges < 320 ? max_ranges : 320) * 32 * sizeof(float);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see the top of the merge kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DFLASH_CUDA_CHECK(cudaLaunchKernelEx(&cfg, sdpa_tc_merge_kernel<InT, D>, p, (int)(2 * grid), max_ranges));
    DFLASH_LAUNCH_CHECK();
    count_launch();
  }
  return DFLASH_OK;
}

}  // namespace

size_t sdpa_tc_scratch_bytes(int D) { return tc_workspace_bytes(D); }

size_t sdpa_workspace_bytes(int B, int Hq, int Hkv, int D, int N) {
  (void)Hkv; (void)N;
  const size_t simple = sdpa_simple_workspace_bytes(B, Hq, D);
  const size_t tc = tc_workspace_bytes(D);
  return (simple > tc ? simple : tc) + 256;
}

// What keeps a call off the tensor-core kernel apart from a missing workspace.
static bool tc_takes(int B, float scale, bool ragged) {
  if (ragged && B > 4096) return false;
  return scale > 0.f;                                // the running maximum assumes a positive scale
}

bool sdpa_tc_supported(const SdpaArgs& a) {
  if (a.D != 128 && a.D != 256) return false;
  if (a.dtype != DFLASH_BF16 && a.dtype != DFLASH_F16) return false;
  if (!tc_takes(a.B, a.scale, a.kv_len != nullptr)) return false;
  if (!a.workspace || a.workspace_bytes < tc_workspace_bytes(a.D)) return false;
  return true;
}

size_t sdpa_scratch_bytes_for_call(int B, int Hq, int D, float scale, bool ragged) {
  return tc_takes(B, scale, ragged) ? tc_workspace_bytes(D) : sdpa_simple_workspace_bytes(B, Hq, D);
}

template <typename InT, int D>
static int32_t launch_dims(const SdpaArgs& a, cudaStream_t stream) {
  return a.mask ? launch_typed<InT, D, true, false>(a, nullptr, stream) : launch_typed<InT, D, false, false>(a, nullptr, stream);
}

// Attention over KV in the TurboQuant 3-bit format without decoding it to global memory: a.q = Q1 = R q, t.q2 = Rq^T q,
// a.k / a.v = the hot window in the rotated domain (or null), a.out = the output in the rotated domain.
// The compressed-KV kernel moves registers between its warpgroups; that arithmetic holds only if the launch gives every
// thread kTurboRegsLaunch registers (a request for more than the pool holds would wait forever).  Checked once; if it
// does not hold, the caller takes the route through a decoded copy.
template <typename InT, int D>
static bool turbo_pool_ok_one() {
  cudaFuncAttributes attr;
  if (cudaFuncGetAttributes(&attr, sdpa_tc_kernel<InT, D, false, true>) != cudaSuccess) { (void)cudaGetLastError(); return false; }
  return attr.numRegs > kTurboRegsLaunch - 8 && attr.numRegs <= kTurboRegsLaunch;
}
bool sdpa_tc_turbo_available() {
  static const bool ok = turbo_pool_ok_one<__nv_bfloat16, 256>() && turbo_pool_ok_one<__nv_bfloat16, 128>() &&
                         turbo_pool_ok_one<__half, 256>() && turbo_pool_ok_one<__half, 128>();
  return ok;
}

int32_t launch_sdpa_tc_turbo(const SdpaArgs& a, const TurboKvArgs& t, cudaStream_t stream) {
  if (a.dtype == DFLASH_BF16)
    return a.D == 256 ? launch_typed<__nv_bfloat16, 256, false, true>(a, &t, stream) : launch_typed<__nv_bfloat16, 128, false, true>(a, &t, stream);
  return a.D == 256 ? launch_typed<__half, 256, false, true>(a, &t, stream) : launch_typed<__half, 128, false, true>(a, &t, stream);
}

int32_t launch_sdpa_tc(const SdpaArgs& a, cudaStream_t stream) {
  if (a.dtype == DFLASH_BF16) return a.D == 256 ? launch_dims<__nv_bfloat16, 256>(a, stream) : launch_dims<__nv_bfloat16, 128>(a, stream);
  return a.D == 256 ? launch_dims<__half, 256>(a, stream) : launch_dims<__half, 128>(a, stream);
}

}  // namespace dflash
