// Micro-benchmark of the DFlash kernels through the C ABI, timed with CUDA events.
//
// The counterpart of the reference's Sources/DFlashKernelBench/main.swift: same flags
// (--iterations N, --warmup N, --kernels tape,gdelta,sdpa, --long-ctx; main.swift:77-96), same
// shapes (B=1, T=16, Hk=8, Hv=16, Dk=Dv=128 for the recurrent kernels, main.swift:105,147;
// B=1, Hq=32, Hk=8, qLen=16, D=128, nKV in {512,2048,8192}(+16384,32768) for attention,
// main.swift:200-204), same inputs (uniform(-0.1, 0.1) in bf16, main.swift:28-30), same byte
// counts for the GB/s column (main.swift:119-124, 164-166, 220-222) and the same
// median / min / max report (main.swift:42-66).  Wall-clock around a lazy-graph evaluation
// (main.swift:33-39) becomes a pair of CUDA events on the launching stream.  --batch B scales
// the batch dimension and --cold rotates the large inputs among copies that together exceed the L2 cache (neither is in
// the reference).  The reference's "variants" and "ops" sections
// compare Metal source variants and its CPU fallback; neither exists here.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/dflash_cuda.h"

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_)); exit(1); } } while (0)
#define DF(x) do { int32_t s_ = (x); if (s_ != 0) { fprintf(stderr, "%s -> %d: %s\n", #x, s_, dflash_last_error_string()); exit(1); } } while (0)

struct Args {
  int iterations = 200, warmup = 20, batch = 1;
  std::string kernels = "tape,gdelta,sdpa";
  bool long_ctx = false;
  bool cold = false;   // rotate among copies of the inputs that together exceed the L2 cache
  bool has(const char* k) const { return ("," + kernels + ",").find(std::string(",") + k + ",") != std::string::npos; }
};

static uint64_t g_rng = 20260330ULL;
static float urand() {   // uniform(-0.1, 0.1)
  g_rng = g_rng * 6364136223846793005ULL + 1442695040888963407ULL;
  return (float)((double)(g_rng >> 11) / (double)(1ULL << 53) * 0.2 - 0.1);
}
static __nv_bfloat16* rand_bf16(size_t n, float lo_shift = 0.f) {
  std::vector<__nv_bfloat16> h(n);
  for (size_t i = 0; i < n; ++i) h[i] = __float2bfloat16(urand() + lo_shift);
  __nv_bfloat16* d;
  CK(cudaMalloc(&d, n * sizeof(__nv_bfloat16)));
  CK(cudaMemcpy(d, h.data(), n * sizeof(__nv_bfloat16), cudaMemcpyHostToDevice));
  return d;
}
static float* rand_f32(size_t n) {
  std::vector<float> h(n);
  for (size_t i = 0; i < n; ++i) h[i] = urand();
  float* d;
  CK(cudaMalloc(&d, n * sizeof(float)));
  CK(cudaMemcpy(d, h.data(), n * sizeof(float), cudaMemcpyHostToDevice));
  return d;
}

struct Result { double med, mn, mx; };
// how many copies of a working set of `bytes` exceed the L2 cache comfortably (1 when warm)
static int copies_for(const Args& a, double bytes) {
  if (!a.cold) return 1;
  const double target = 400e6;   // the L2 of a B200 holds 126 MB
  int n = (int)(target / bytes) + 1;
  return n < 2 ? 2 : (n > 256 ? 256 : n);
}
template <typename F>
static Result measure(const Args& a, F&& body) {
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  for (int i = 0; i < a.warmup; ++i) body(i);
  CK(cudaDeviceSynchronize());
  std::vector<double> s;
  for (int i = 0; i < a.iterations; ++i) {
    CK(cudaEventRecord(e0, 0));
    body(a.warmup + i);
    CK(cudaEventRecord(e1, 0));
    CK(cudaEventSynchronize(e1));
    float ms;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    s.push_back(ms * 1e-3);
  }
  std::sort(s.begin(), s.end());
  DF(dflash_device_status(nullptr));
  return {s[s.size() / 2], s.front(), s.back()};
}
static void print_result(const char* label, Result r, double bytes) {
  printf("  %-42s  med %7.1f us  min %7.1f us  max %7.1f us", label, r.med * 1e6, r.mn * 1e6, r.mx * 1e6);
  if (bytes > 0) printf("  %.1f GB/s", bytes / 1e9 / r.med);
  printf("\n");
}

static void bench_tape(const Args& a) {
  printf("\n-- Tape Replay ---------------------------------------------------------\n");
  const int B = a.batch, T = 16, Hk = 8, Hv = 16, Dk = 128, Dv = 128;
  float* tape = rand_f32((size_t)B * T * Hv * Dv);
  __nv_bfloat16* k = rand_bf16((size_t)B * T * Hk * Dk);
  __nv_bfloat16* g = rand_bf16((size_t)B * T * Hv, 0.5f);
  __nv_bfloat16* gvec = rand_bf16((size_t)B * T * Hv * Dk, 0.5f);
  const double state_bytes = (double)B * Hv * Dv * Dk * 4;   // fp32 state here (bf16 in the reference)
  const int nc = copies_for(a, state_bytes * 2);
  std::vector<float*> state(nc), out(nc);
  for (int c = 0; c < nc; ++c) {
    state[c] = rand_f32((size_t)B * Hv * Dv * Dk);
    CK(cudaMalloc(&out[c], (size_t)B * Hv * Dv * Dk * 4));
  }
  std::vector<__nv_bfloat16> hm((size_t)B * T);
  for (auto& m : hm) m = __float2bfloat16(urand() >= 0.f ? 1.f : 0.f);
  __nv_bfloat16* mask;
  CK(cudaMalloc(&mask, hm.size() * 2));
  CK(cudaMemcpy(mask, hm.data(), hm.size() * 2, cudaMemcpyHostToDevice));
  auto run = [&](int i, const void* gate, int vec, const void* m) {
    DF(dflash_tape_replay(tape, k, gate, state[i % nc], m, nullptr, out[i % nc], B, T, Hk, Hv, Dk, Dv, vec, DFLASH_BF16, DFLASH_BF16, nullptr));
  };
  print_result("scalar-g, no mask", measure(a, [&](int i) { run(i, g, 0, nullptr); }), state_bytes * 2);
  print_result("scalar-g, mask", measure(a, [&](int i) { run(i, g, 0, mask); }), state_bytes * 2);
  print_result("vec-g, no mask", measure(a, [&](int i) { run(i, gvec, 1, nullptr); }), state_bytes * 2);
  print_result("vec-g, mask", measure(a, [&](int i) { run(i, gvec, 1, mask); }), state_bytes * 2);
  for (int c = 0; c < nc; ++c) { CK(cudaFree(state[c])); CK(cudaFree(out[c])); }
}

static void bench_gdelta(const Args& a) {
  printf("\n-- GatedDelta + Tape ---------------------------------------------------\n");
  const int B = a.batch, T = 16, Hk = 8, Hv = 16, Dk = 128, Dv = 128;
  __nv_bfloat16 *q = rand_bf16((size_t)B * T * Hk * Dk), *k = rand_bf16((size_t)B * T * Hk * Dk);
  __nv_bfloat16* v = rand_bf16((size_t)B * T * Hv * Dv);
  __nv_bfloat16* g = rand_bf16((size_t)B * T * Hv, 0.5f);
  __nv_bfloat16* gvec = rand_bf16((size_t)B * T * Hv * Dk, 0.5f);
  __nv_bfloat16* beta = rand_bf16((size_t)B * T * Hv, 0.5f);
  const int nc = copies_for(a, (double)B * Hv * Dv * Dk * 4 * 2);
  std::vector<float*> state(nc), out(nc);
  for (int c = 0; c < nc; ++c) {
    state[c] = rand_f32((size_t)B * Hv * Dv * Dk);
    CK(cudaMalloc(&out[c], (size_t)B * Hv * Dv * Dk * 4));
  }
  float* tape;
  __nv_bfloat16* y;
  CK(cudaMalloc(&tape, (size_t)B * T * Hv * Dv * 4));
  CK(cudaMalloc(&y, (size_t)B * T * Hv * Dv * 2));
  std::vector<__nv_bfloat16> hm((size_t)B * T);
  for (auto& m : hm) m = __float2bfloat16(urand() >= 0.f ? 1.f : 0.f);
  __nv_bfloat16* mask;
  CK(cudaMalloc(&mask, hm.size() * 2));
  CK(cudaMemcpy(mask, hm.data(), hm.size() * 2, cudaMemcpyHostToDevice));
  // q + k + v inputs, state in + out (fp32 here), tape out (main.swift:164-166)
  const double bytes = ((double)B * T * Hk * Dk * 2 + (double)B * T * Hv * Dv) * 2 + (double)B * Hv * Dv * Dk * 4 * 2 +
                       (double)B * T * Hv * Dv * 4;
  auto run = [&](int i, const void* gate, int vec, const void* m) {
    DF(dflash_gated_delta_tape(q, k, v, gate, beta, state[i % nc], m, nullptr, y, out[i % nc], tape, B, T, Hk, Hv, Dk, Dv, vec, DFLASH_BF16,
                               DFLASH_BF16, nullptr));
  };
  print_result("scalar-g, no mask", measure(a, [&](int i) { run(i, g, 0, nullptr); }), bytes);
  print_result("scalar-g, mask", measure(a, [&](int i) { run(i, g, 0, mask); }), bytes);
  print_result("vec-g, no mask", measure(a, [&](int i) { run(i, gvec, 1, nullptr); }), bytes);
  print_result("vec-g, mask", measure(a, [&](int i) { run(i, gvec, 1, mask); }), bytes);
  for (int c = 0; c < nc; ++c) { CK(cudaFree(state[c])); CK(cudaFree(out[c])); }
}

static void bench_sdpa(const Args& a) {
  printf("\n-- Batched block-verify SDPA -------------------------------------------\n");
  const int B = a.batch, Hq = 32, Hk = 8, T = 16, D = 128;
  const float scale = 1.0f / sqrtf((float)D);
  std::vector<int> sizes = {512, 2048, 8192};
  if (a.long_ctx) { sizes.push_back(16384); sizes.push_back(32768); }
  __nv_bfloat16* q = rand_bf16((size_t)B * Hq * T * D);
  __nv_bfloat16* out;
  CK(cudaMalloc(&out, (size_t)B * Hq * T * D * 2));
  for (int n : sizes) {
    const double kv_bytes = 2.0 * B * Hk * n * D * 2;
    const int nc = copies_for(a, kv_bytes);
    std::vector<__nv_bfloat16*> k(nc), v(nc);
    for (int c = 0; c < nc; ++c) { k[c] = rand_bf16((size_t)B * Hk * n * D); v[c] = rand_bf16((size_t)B * Hk * n * D); }
    const size_t ws_bytes = dflash_verify_sdpa_workspace_bytes(B, Hq, Hk, D, n);
    void* ws;
    CK(cudaMalloc(&ws, ws_bytes));
    const double bytes = ((double)B * Hq * T * D + 2.0 * B * Hk * n * D) * 2 + (double)B * Hq * T * D * 2;   // main.swift:220-222
    char label[64];
    snprintf(label, sizeof label, "nKV=%d", n);
    print_result(label, measure(a, [&](int i) {
                   DF(dflash_verify_sdpa(q, k[i % nc], v[i % nc], nullptr, nullptr, nullptr, out, ws, ws_bytes, B, Hq, Hk, T, D, n, 0, 0, 0, scale,
                                         DFLASH_BF16, DFLASH_KV_DENSE, nullptr));
                 }), bytes);
    for (int c = 0; c < nc; ++c) { CK(cudaFree(k[c])); CK(cudaFree(v[c])); }
    CK(cudaFree(ws));
  }
}

int main(int argc, char** argv) {
  Args a;
  for (int i = 1; i < argc; ++i) {
    if (!strcmp(argv[i], "--iterations") && i + 1 < argc) a.iterations = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--warmup") && i + 1 < argc) a.warmup = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--batch") && i + 1 < argc) a.batch = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--kernels") && i + 1 < argc) a.kernels = argv[++i];
    else if (!strcmp(argv[i], "--long-ctx")) a.long_ctx = true;
    else if (!strcmp(argv[i], "--cold")) a.cold = true;
  }
  if (dflash_device_count() < 1) { fprintf(stderr, "no CUDA device (there is no CPU fallback)\n"); return 1; }
  cudaDeviceProp p;
  CK(cudaGetDeviceProperties(&p, 0));
  printf("DFlash Kernel Micro-Benchmark (%s)\n", dflash_version());
  printf("  Device:     %s, %d SMs\n  Iterations: %d  Warmup: %d  Batch: %d\n  Kernels:    %s\n  Long-ctx:   %s\n  L2:         %s\n", p.name,
         p.multiProcessorCount, a.iterations, a.warmup, a.batch, a.kernels.c_str(), a.long_ctx ? "true" : "false",
         a.cold ? "cold (inputs rotate among copies that exceed the cache)" : "warm (same buffers every iteration)");
  if (a.has("tape")) bench_tape(a);
  if (a.has("gdelta")) bench_gdelta(a);
  if (a.has("sdpa")) bench_sdpa(a);
  if (a.has("variants") || a.has("ops")) printf("\n(variants / ops: sections of the reference that compare Metal source variants and its CPU fallback; not applicable)\n");
  printf("\nDone.\n");
  return 0;
}
