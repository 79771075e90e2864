// Self-test of the C++ host layer (dflash_host.hpp) on one GPU.  It checks identities that need no
// outside reference: the replay of a recorded tape reproduces the forward state; rollback(n) leaves
// the state of a forward pass over n + 1 steps and the conv window concat(snapshot, qkv)[n+1 : n+4];
// the per-sequence rollback agrees with the scalar one; batchedSDPA2Pass returns no value outside
// its contract and equals the allocation-free entry point inside it; the paged KV cache keeps exactly the
// accepted rows and its attention equals the dense one.  Exit code 0 = all passed.
#include <cuda_bf16.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include "dflash_host.hpp"

using namespace dflash::host;

static uint64_t g_rng = 88172645463325252ULL;
static float urand() {
  g_rng ^= g_rng << 13; g_rng ^= g_rng >> 7; g_rng ^= g_rng << 17;
  return (float)((g_rng >> 11) * (1.0 / 9007199254740992.0));
}
static Tensor randBf16(std::vector<int64_t> shape, float lo, float hi) {
  size_t n = 1;
  for (auto d : shape) n *= (size_t)d;
  std::vector<__nv_bfloat16> h(n);
  for (auto& x : h) x = __float2bfloat16(lo + (hi - lo) * urand());
  return Tensor::fromHost(h.data(), shape, DType::BF16);
}
static Tensor randF32(std::vector<int64_t> shape, float lo, float hi) {
  size_t n = 1;
  for (auto d : shape) n *= (size_t)d;
  std::vector<float> h(n);
  for (auto& x : h) x = lo + (hi - lo) * urand();
  return Tensor::fromHost(h.data(), shape, DType::F32);
}
template <typename T> static std::vector<T> host(const Tensor& t) {
  std::vector<T> h(t.nbytes() / sizeof(T));
  t.toHost(h.data());
  return h;
}
static double relDiff(const std::vector<float>& a, const std::vector<float>& b) {
  double num = 0, den = 1e-30;
  for (size_t i = 0; i < a.size(); ++i) { num = std::fmax(num, std::fabs((double)a[i] - b[i])); den = std::fmax(den, std::fabs((double)b[i])); }
  return num / den;
}
static int g_failed = 0;
#define EXPECT(cond, msg) do { if (!(cond)) { printf("FAIL: %s\n", msg); ++g_failed; } else printf("ok:   %s\n", msg); } while (0)

int main() {
  try {
    if (dflash_device_count() < 1) { printf("no CUDA device\n"); return 2; }
    const int B = 3, T = 16, Hk = 2, Hv = 4, D = 128, C = 64, keep = 3;
    Tensor q = randBf16({B, T, Hk, D}, -0.09f, 0.09f), k = randBf16({B, T, Hk, D}, -0.09f, 0.09f);
    Tensor v = randBf16({B, T, Hv, D}, -1.f, 1.f), g = randBf16({B, T, Hv}, 0.3f, 0.95f), beta = randBf16({B, T, Hv}, 0.1f, 0.9f);
    Tensor s0 = randF32({B, Hv, D, D}, -0.03f, 0.03f);

    // 1. forward, then the replay of its tape
    auto [y, sT, tape] = DFlashKernels::gatedDeltaKernelWithTape(q, k, v, g, beta, s0);
    Tensor sRep = DFlashKernels::tapeReplayKernel(tape, k, g, s0);
    EXPECT(relDiff(host<float>(sRep), host<float>(sT)) < 1e-5, "replay of the recorded tape reproduces the forward state");

    // 2. rollback(n) == forward over n + 1 steps; conv window rows
    const int nAccepted = 6;
    std::vector<int32_t> steps(B, nAccepted + 1);
    Tensor stepsDev = Tensor::fromHost(steps.data(), {B}, DType::I32);
    auto [y2, sWant, tape2] = DFlashKernels::gatedDeltaKernelWithTape(q, k, v, g, beta, s0, nullptr, &stepsDev);
    Tensor conv0 = randBf16({B, keep, C}, -1.f, 1.f), qkv = randBf16({B, T, C}, -1.f, 1.f);
    RecurrentRollbackCache cache;
    cache.state[0] = conv0;
    cache.state[1] = s0;
    cache.armRollback();
    cache.state[1] = sT;                      // the verify pass moved the state on
    cache.recordTape(tape, k, g, qkv);
    EXPECT(cache.isArmed(), "armRollback arms the cache");
    cache.rollback(nAccepted);
    EXPECT(!cache.isArmed(), "rollback clears the transients");
    EXPECT(relDiff(host<float>(cache.state[1]), host<float>(sWant)) < 1e-5, "rollback(n) leaves the state of n + 1 steps");
    {
      auto hc = host<uint16_t>(conv0), hq = host<uint16_t>(qkv), got = host<uint16_t>(cache.state[0]);
      bool same = cache.state[0].dim(1) == keep;
      for (int b = 0; b < B && same; ++b)
        for (int j = 0; j < keep && same; ++j) {
          const int src = nAccepted + 1 + j;   // row of concat(conv0, qkv)
          const uint16_t* want = src < keep ? &hc[((size_t)b * keep + src) * C] : &hq[((size_t)b * T + (src - keep)) * C];
          same = std::memcmp(&got[((size_t)b * keep + j) * C], want, C * 2) == 0;
        }
      EXPECT(same, "conv window = concat(snapshot, qkv)[n+1 : n+1+keep]");
    }

    // 3. per-sequence rollback with the same counts gives the same bytes
    RecurrentRollbackCache cache2;
    cache2.state[0] = conv0;
    cache2.state[1] = s0;
    cache2.armRollback();
    cache2.recordTape(tape, k, g, qkv);
    cache2.rollbackPerSequence(stepsDev);
    EXPECT(host<float>(cache2.state[1]) == host<float>(cache.state[1]), "per-sequence rollback equals the scalar rollback (state, bitwise)");
    EXPECT(host<uint16_t>(cache2.state[0]) == host<uint16_t>(cache.state[0]), "per-sequence rollback equals the scalar rollback (conv window)");

    // 4. full accept keeps the verify state
    RecurrentRollbackCache cache3;
    cache3.state[1] = s0;
    cache3.armRollback();
    cache3.state[1] = sT;
    cache3.recordTape(tape, k, g, qkv);
    std::vector<RecurrentRollbackCache*> all{&cache3};
    restoreAfterAcceptance(all, 15, 15);
    EXPECT(cache3.state[1].data() == sT.data() && !cache3.isArmed(), "a fully accepted block keeps the verify state");
    cache3.offset = 20;
    EXPECT(cache3.trim(6) == 6 && cache3.offset == 14, "trim");

    // 5. attention: nil outside the contract, equal to the allocation-free entry inside it
    Tensor qa = randBf16({2, 16, 16, 256}, -1.f, 1.f), ka = randBf16({2, 2, 16 + 700, 256}, -1.f, 1.f), va = randBf16({2, 2, 16 + 700, 256}, -1.f, 1.f);
    auto out = DFlashKernels::batchedSDPA2Pass(qa, ka, va, 1.f / 16.f);
    EXPECT(out.has_value(), "batchedSDPA2Pass returns a value inside its contract");
    Tensor qbad = randBf16({2, 16, 8, 256}, -1.f, 1.f);
    EXPECT(!DFlashKernels::batchedSDPA2Pass(qbad, ka, va, 1.f / 16.f).has_value(), "batchedSDPA2Pass returns no value for 8 query rows");
    if (out) {
      Tensor o2 = Tensor::empty(qa.shape(), DType::BF16);
      check(dflash_verify_sdpa_noalloc(qa.data(), ka.data(), va.data(), nullptr, nullptr, nullptr, o2.data(), 2, 16, 2, 16, 256, 716, 0, 0, 0,
                                       1.f / 16.f, DFLASH_BF16, DFLASH_KV_DENSE, nullptr));
      EXPECT(host<uint16_t>(*out) == host<uint16_t>(o2), "workspace and allocation-free attention agree bitwise");
    }

    // 6. paged KV cache: append / attend / commit cycles against a dense history kept on the host
    {
      const int KB = 2, KH = 2, KD = 256, PT = 128, NP = 8, MP = 4, KT = 16;
      PagedKVCache cache(KB, KH, KD, PT, NP, MP);
      std::vector<std::vector<uint16_t>> histK(KB), histV(KB);      // per sequence: rows [n][KH][KD]
      const int commits[4][2] = {{16, 3}, {1, 16}, {9, 9}, {16, 2}};
      bool rowsOk = true, attnOk = true, lensOk = true;
      for (int cycle = 0; cycle < 4; ++cycle) {
        Tensor kn = randBf16({KB, KH, KT, KD}, -1.f, 1.f), vn = randBf16({KB, KH, KT, KD}, -1.f, 1.f);
        Tensor qn = randBf16({KB, 16, 16, KD}, -1.f, 1.f);
        const std::vector<uint16_t> hk = host<uint16_t>(kn), hv = host<uint16_t>(vn);
        for (int b = 0; b < KB; ++b)
          for (int t = 0; t < KT; ++t)
            for (int h = 0; h < KH; ++h) {
              const size_t src = (((size_t)b * KH + h) * KT + t) * KD;
              histK[b].insert(histK[b].end(), hk.begin() + src, hk.begin() + src + KD);
              histV[b].insert(histV[b].end(), hv.begin() + src, hv.begin() + src + KD);
            }
        const Tensor& lensBlk = cache.appendBlock(kn, vn);
        const std::vector<int32_t> lb = host<int32_t>(lensBlk);
        for (int b = 0; b < KB; ++b) lensOk = lensOk && lb[b] == (int32_t)(histK[b].size() / (KH * KD));
        // dense ragged attention over the host history must equal the paged one bit for bit
        int nMax = 0;
        for (int b = 0; b < KB; ++b) nMax = lb[b] > nMax ? lb[b] : nMax;
        std::vector<uint16_t> dk((size_t)KB * KH * nMax * KD, 0), dv(dk.size(), 0);
        for (int b = 0; b < KB; ++b)
          for (int n = 0; n < lb[b]; ++n)
            for (int h = 0; h < KH; ++h) {
              const size_t dst = (((size_t)b * KH + h) * nMax + n) * KD, src = ((size_t)n * KH + h) * KD;
              std::memcpy(&dk[dst], &histK[b][src], KD * 2);
              std::memcpy(&dv[dst], &histV[b][src], KD * 2);
            }
        Tensor dkT = Tensor::fromHost(dk.data(), {KB, KH, nMax, KD}, DType::BF16), dvT = Tensor::fromHost(dv.data(), {KB, KH, nMax, KD}, DType::BF16);
        Tensor dense = Tensor::empty(qn.shape(), DType::BF16);
        const size_t need = dflash_verify_sdpa_workspace_bytes(KB, 16, KH, KD, nMax);
        Tensor ws = Tensor::empty({(int64_t)need}, DType::U8);
        check(dflash_verify_sdpa(qn.data(), dkT.data(), dvT.data(), nullptr, static_cast<const int32_t*>(lensBlk.data()), nullptr, dense.data(),
                                 ws.data(), ws.nbytes(), KB, 16, KH, 16, KD, nMax, 0, 0, 0, 1.f / 16.f, DFLASH_BF16, DFLASH_KV_DENSE, nullptr));
        auto paged = cache.attend(qn, 1.f / 16.f);
        attnOk = attnOk && paged.has_value() && host<uint16_t>(*paged) == host<uint16_t>(dense);
        // commit: keep accepted + 1 rows of the block
        const int32_t cc[2] = {commits[cycle][0], commits[cycle][1]};
        cache.commit(Tensor::fromHost(cc, {KB}, DType::I32));
        for (int b = 0; b < KB; ++b) {
          histK[b].resize(histK[b].size() - (size_t)(KT - cc[b]) * KH * KD);
          histV[b].resize(histV[b].size() - (size_t)(KT - cc[b]) * KH * KD);
        }
      }
      const std::vector<int32_t> lens = cache.sync();
      const std::vector<uint16_t> pool = host<uint16_t>(cache.kPool);
      for (int b = 0; b < KB; ++b) {
        lensOk = lensOk && lens[b] == (int32_t)(histK[b].size() / (KH * KD));
        lensOk = lensOk && (int)cache.pagesOf(b).size() == (lens[b] + PT - 1) / PT;
        for (int n = 0; n < lens[b] && rowsOk; ++n)
          for (int h = 0; h < KH; ++h) {
            const size_t at = (((size_t)cache.pagesOf(b)[n / PT] * KH + h) * PT + n % PT) * KD;
            rowsOk = rowsOk && std::memcmp(&pool[at], &histK[b][((size_t)n * KH + h) * KD], KD * 2) == 0;
          }
      }
      EXPECT(lensOk, "paged KV cache: lengths and page counts follow append / commit");
      EXPECT(rowsOk, "paged KV cache: committed rows equal the host history");
      EXPECT(attnOk, "paged KV cache: attention over pages equals attention over the dense history bitwise");
      bool threw = false;
      try { cache.reserve(0, (int64_t)MP * PT + 1); } catch (const Error&) { threw = true; }
      EXPECT(threw, "paged KV cache: a sequence longer than its table is refused");
    }

    // 7. partition plan
    auto plan = partitionPlan(10, 4);
    EXPECT(plan.size() == 4 && plan[0].first == 0 && plan[3].second == 10 && plan[0].second - plan[0].first == 3, "partition plan");
    checkCuda(cudaDeviceSynchronize());
    check(dflash_device_status(nullptr));
  } catch (const Error& e) {
    printf("FAIL: exception %d: %s\n", e.status, e.what());
    return 1;
  }
  printf(g_failed ? "%d check(s) failed\n" : "all checks passed\n", g_failed);
  return g_failed ? 1 : 0;
}
