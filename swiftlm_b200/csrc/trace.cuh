// Development instrumentation of the two persistent kernels.  Nothing here is part of the shipped library: without
// -DDFLASH_SDPA_TRACE / -DDFLASH_GDN_TRACE every macro below expands to nothing and no symbol is defined.  With them,
// the attention kernel records per-CTA timer stamps and per-role wait accumulators, the tensor-core replay kernel
// per-warp clocks per phase, and an extern "C" reader copies the device arrays out.
#pragma once
#include <cuda_runtime.h>

// Optional timeline instrumentation (compile with -DDFLASH_SDPA_TRACE; never part of the shipped
// library): per CTA 64 words of %globaltimer stamps and clock64 wait accumulators.
#ifdef DFLASH_SDPA_TRACE
__device__ unsigned long long g_sdpa_trace[256 * 64];
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define TR_STAMP(i) do { g_sdpa_trace[blockIdx.x * 64 + (i)] = gtime(); } while (0)
#define TR_T0() const long long tr_t0_ = clock64()
#define TR_DECL() long long tr_acc_[8] = {0, 0, 0, 0, 0, 0, 0, 0}
#define TR_ACC(i) do { tr_acc_[(i) - 16] += clock64() - tr_t0_; } while (0)
#define TR_FLUSH(lo, hi) do { for (int i_ = (lo); i_ <= (hi); ++i_) g_sdpa_trace[blockIdx.x * 64 + i_] = (unsigned long long)tr_acc_[i_ - 16]; } while (0)
extern "C" int dflash_debug_trace(unsigned long long* out, int n, int clear) {
  if (clear) { static unsigned long long z[256 * 64]; return (int)cudaMemcpyToSymbol(g_sdpa_trace, z, sizeof z); }
  return (int)cudaMemcpyFromSymbol(out, g_sdpa_trace, sizeof(unsigned long long) * n);
}
#else
#define TR_STAMP(i) do {} while (0)
#define TR_T0() do {} while (0)
#define TR_ACC(i) do {} while (0)
#define TR_DECL() do {} while (0)
#define TR_FLUSH(lo, hi) do {} while (0)
#endif

// Optional phase timing (compile with -DDFLASH_GDN_TRACE; never part of the shipped library).
#ifdef DFLASH_GDN_TRACE
__device__ unsigned long long g_gdn_trace[256 * 12 * 16];
#define PH_DECL() long long ph_[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}; long long ph_t_ = clock64()
#define PH(i) do { const long long n_ = clock64(); ph_[i] += n_ - ph_t_; ph_t_ = n_; } while (0)
#define PH_FLUSH() do { if ((threadIdx.x & 31) == 0) for (int i_ = 0; i_ < 16; ++i_) g_gdn_trace[(blockIdx.x * 12 + (threadIdx.x >> 5)) * 16 + i_] = (unsigned long long)ph_[i_]; } while (0)
extern "C" int dflash_gdn_trace(unsigned long long* out, int n) { return (int)cudaMemcpyFromSymbol(out, g_gdn_trace, sizeof(unsigned long long) * n); }
#else
#define PH_DECL() do {} while (0)
#define PH(i) do {} while (0)
#define PH_FLUSH() do {} while (0)
#endif
