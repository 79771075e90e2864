// C++ host layer above the C ABI of libdflash_cuda: the counterpart of the Swift types that call the
// DFlash kernels in the reference.
//
//   dflash::host::DFlashKernels            Sources/DFlash/DFlashKernels.swift:252 (tapeReplayKernel), :316
//                                          (gatedDeltaKernelWithTape), :737 (batchedSDPA2Pass)
//   dflash::host::RecurrentRollbackCache   Sources/DFlash/RecurrentRollbackCache.swift:34-182
//   dflash::host::restoreAfterAcceptance   Sources/DFlash/DFlashRuntime.swift:188-223
//   dflash::host::PagedKVCache             the attention cache's update and trim around the verify pass, :188-223
//   dflash::host::partitionPlan            (no counterpart: one process per GPU)
//
// Same names, argument meaning and error behaviour: batchedSDPA2Pass returns an empty optional where
// the reference returns nil; everything else throws dflash::host::Error with the library's message.
// Tensors are device arrays with shared ownership (the reference passes MLXArray by reference and
// snapshots "by reference, no copy", :63-71).  Header only; link with -ldflash_cuda and the CUDA runtime.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

#include "../../include/dflash_cuda.h"

namespace dflash {
namespace host {

struct Error : std::runtime_error {
  int32_t status;
  Error(int32_t st, const std::string& what) : std::runtime_error(what), status(st) {}
};
inline void check(int32_t st) {
  if (st != DFLASH_OK) throw Error(st, dflash_last_error_string());
}
inline void checkCuda(cudaError_t e) {
  if (e != cudaSuccess) throw Error(DFLASH_ERR_CUDA, cudaGetErrorString(e));
}

enum class DType : int32_t { F32 = DFLASH_F32, BF16 = DFLASH_BF16, F16 = DFLASH_F16, U8 = DFLASH_U8, I32 = 100 };
inline size_t dtypeSize(DType t) { return t == DType::F32 || t == DType::I32 ? 4 : (t == DType::U8 ? 1 : 2); }

// A dense row-major device array.
class Tensor {
 public:
  Tensor() = default;
  static Tensor empty(std::vector<int64_t> shape, DType dt) {
    Tensor t;
    t.shape_ = std::move(shape);
    t.dtype_ = dt;
    void* p = nullptr;
    checkCuda(cudaMalloc(&p, t.nbytes() ? t.nbytes() : 1));
    t.storage_ = std::shared_ptr<void>(p, [](void* q) { cudaFree(q); });
    return t;
  }
  static Tensor fromHost(const void* src, std::vector<int64_t> shape, DType dt) {
    Tensor t = empty(std::move(shape), dt);
    checkCuda(cudaMemcpy(t.data(), src, t.nbytes(), cudaMemcpyHostToDevice));
    return t;
  }
  void toHost(void* dst, cudaStream_t stream = nullptr) const {
    checkCuda(cudaMemcpyAsync(dst, data(), nbytes(), cudaMemcpyDeviceToHost, stream));
    checkCuda(cudaStreamSynchronize(stream));
  }
  // The first n steps of a [B, T, ...] array as a new dense array (the reference's tape[0..., ..<n, ...]).
  Tensor firstSteps(int64_t n, cudaStream_t stream = nullptr) const {
    std::vector<int64_t> s = shape_;
    const int64_t B = s.at(0), T = s.at(1);
    s[1] = n;
    Tensor out = empty(s, dtype_);
    const size_t step = nbytes() / (size_t)(B * T);
    if (n > 0)
      checkCuda(cudaMemcpy2DAsync(out.data(), step * n, data(), step * T, step * n, B, cudaMemcpyDeviceToDevice, stream));
    return out;
  }
  bool defined() const { return (bool)storage_; }
  void* data() const { return storage_.get(); }
  DType dtype() const { return dtype_; }
  int ndim() const { return (int)shape_.size(); }
  int64_t dim(int i) const { return shape_.at(i < 0 ? i + shape_.size() : i); }
  const std::vector<int64_t>& shape() const { return shape_; }
  size_t numel() const { size_t n = 1; for (int64_t d : shape_) n *= (size_t)d; return n; }
  size_t nbytes() const { return numel() * dtypeSize(dtype_); }

 private:
  std::shared_ptr<void> storage_;
  std::vector<int64_t> shape_;
  DType dtype_ = DType::F32;
};

// ---- Sources/DFlash/DFlashKernels.swift -------------------------------------------------------
struct DFlashKernels {
  // :252.  tape [B,T,Hv,Dv] fp32, k [B,T,Hk,Dk], g [B,T,Hv] or [B,T,Hv,Dk], state [B,Hv,Dv,Dk] fp32.
  // stepsPerSequence (device int32[B], optional) replays only the first n_b steps of sequence b.
  static Tensor tapeReplayKernel(const Tensor& tape, const Tensor& k, const Tensor& g, const Tensor& state,
                                 const Tensor* mask = nullptr, const Tensor* stepsPerSequence = nullptr,
                                 cudaStream_t stream = nullptr) {
    Tensor out = Tensor::empty(state.shape(), DType::F32);
    check(dflash_tape_replay(static_cast<const float*>(tape.data()), k.data(), g.data(),
                             static_cast<const float*>(state.data()), mask ? mask->data() : nullptr,
                             stepsPerSequence ? static_cast<const int32_t*>(stepsPerSequence->data()) : nullptr,
                             static_cast<float*>(out.data()), (int32_t)k.dim(0), (int32_t)k.dim(1), (int32_t)k.dim(2),
                             (int32_t)tape.dim(2), (int32_t)k.dim(3), (int32_t)tape.dim(3), g.ndim() == 4 ? 1 : 0,
                             (int32_t)k.dtype(), mask ? (int32_t)mask->dtype() : DFLASH_F32, stream));
    return out;
  }
  // :316.  Returns (y, new state, tape).
  static std::tuple<Tensor, Tensor, Tensor> gatedDeltaKernelWithTape(const Tensor& q, const Tensor& k, const Tensor& v,
                                                                    const Tensor& g, const Tensor& beta, const Tensor& state,
                                                                    const Tensor* mask = nullptr,
                                                                    const Tensor* stepsPerSequence = nullptr,
                                                                    cudaStream_t stream = nullptr) {
    const int32_t B = (int32_t)k.dim(0), T = (int32_t)k.dim(1), Hk = (int32_t)k.dim(2), Dk = (int32_t)k.dim(3);
    const int32_t Hv = (int32_t)v.dim(2), Dv = (int32_t)v.dim(3);
    Tensor y = Tensor::empty({B, T, Hv, Dv}, q.dtype());
    Tensor newState = Tensor::empty(state.shape(), DType::F32);
    Tensor tape = Tensor::empty({B, T, Hv, Dv}, DType::F32);
    check(dflash_gated_delta_tape(q.data(), k.data(), v.data(), g.data(), beta.data(), static_cast<const float*>(state.data()),
                                  mask ? mask->data() : nullptr,
                                  stepsPerSequence ? static_cast<const int32_t*>(stepsPerSequence->data()) : nullptr, y.data(),
                                  static_cast<float*>(newState.data()), static_cast<float*>(tape.data()), B, T, Hk, Hv, Dk, Dv,
                                  g.ndim() == 4 ? 1 : 0, (int32_t)q.dtype(), mask ? (int32_t)mask->dtype() : DFLASH_F32, stream));
    return {y, newState, tape};
  }
  // :737.  queries [B,Hq,16,D], keys / values [B,Hkv,N,D].  Empty optional where the reference returns nil.
  static std::optional<Tensor> batchedSDPA2Pass(const Tensor& queries, const Tensor& keys, const Tensor& values, float scale,
                                                const Tensor* mask = nullptr, cudaStream_t stream = nullptr) {
    if (queries.ndim() != 4 || keys.ndim() != 4 || values.ndim() != 4) return std::nullopt;
    const int32_t B = (int32_t)queries.dim(0), Hq = (int32_t)queries.dim(1), T = (int32_t)queries.dim(2), D = (int32_t)queries.dim(3);
    const int32_t Hkv = (int32_t)keys.dim(1), N = (int32_t)keys.dim(2);
    const size_t need = dflash_verify_sdpa_workspace_bytes(B, Hq, Hkv, D, N);
    Tensor& ws = workspace();
    if (!ws.defined() || ws.nbytes() < need) ws = Tensor::empty({(int64_t)need}, DType::U8);
    Tensor out = Tensor::empty(queries.shape(), queries.dtype());
    const int32_t st = dflash_verify_sdpa(queries.data(), keys.data(), values.data(), nullptr, nullptr, mask ? mask->data() : nullptr,
                                          out.data(), ws.data(), ws.nbytes(), B, Hq, Hkv, T, D, N, 0, 0, 0, scale,
                                          (int32_t)queries.dtype(), DFLASH_KV_DENSE, stream);
    if (st == DFLASH_ERR_UNSUPPORTED) return std::nullopt;
    check(st);
    return out;
  }

 private:
  static Tensor& workspace() {   // caller-owned scratch of the attention kernel, grown on demand, one per thread
    static thread_local Tensor ws;
    return ws;
  }
};

// ---- Sources/DFlash/RecurrentRollbackCache.swift ----------------------------------------------
class RecurrentRollbackCache {
 public:
  static constexpr int defaultConvKernelSize = 4;   // :135
  explicit RecurrentRollbackCache(int convKernelSize = defaultConvKernelSize) : convKernelSize_(convKernelSize) {}

  Tensor state[2];   // [0] conv window [B, keep, C], [1] recurrent state [B, Hv, Dv, Dk] fp32
  int64_t offset = 0;

  bool isArmed() const { return armed_; }
  void armRollback(int /*prefixLen*/ = 0) {   // :63-71: snapshot by reference
    armed_ = true;
    tape_ = tapeK_ = tapeG_ = tapeQKV_ = Tensor();
    snapshot_[0] = state[0];
    snapshot_[1] = state[1];
    hasSnapshot_ = true;
  }
  void recordTape(const Tensor& tape, const Tensor& k, const Tensor& g, const Tensor& qkv) {   // :75-85
    tape_ = tape; tapeK_ = k; tapeG_ = g; tapeQKV_ = qkv;
  }
  // :95-131 with a host count: restore the snapshot, replay acceptedSteps = nAccepted + 1 steps, rebuild the window.
  void rollback(int nAccepted, cudaStream_t stream = nullptr) {
    if (!hasSnapshot_) { clearTransients(); return; }
    restoreSnapshot();
    if (tape_.defined() && tapeK_.defined() && tapeG_.defined() && state[1].defined()) {
      const int acceptedSteps = nAccepted + 1;   // :115
      state[1] = DFlashKernels::tapeReplayKernel(tape_.firstSteps(acceptedSteps, stream), tapeK_.firstSteps(acceptedSteps, stream),
                                                 tapeG_.firstSteps(acceptedSteps, stream), state[1], nullptr, nullptr, stream);
      state[0] = rebuildConvState(acceptedSteps, nullptr, stream);
    }
    clearTransients();
  }
  // The same with per-sequence step counts that never leave the device (replay_len of dflash_accept_lengths).
  void rollbackPerSequence(const Tensor& replaySteps, cudaStream_t stream = nullptr) {
    if (!hasSnapshot_) { clearTransients(); return; }
    restoreSnapshot();
    if (tape_.defined() && tapeK_.defined() && tapeG_.defined() && state[1].defined()) {
      state[1] = DFlashKernels::tapeReplayKernel(tape_, tapeK_, tapeG_, state[1], nullptr, &replaySteps, stream);
      state[0] = rebuildConvState(0, &replaySteps, stream);
    }
    clearTransients();
  }
  // :139-158
  Tensor rebuildConvState(int acceptedSteps, const Tensor* stepsPerSequence = nullptr, cudaStream_t stream = nullptr) const {
    if (!tapeQKV_.defined()) return state[0];
    const int keep = convKernelSize_ - 1;
    if (keep <= 0) return Tensor();
    const int32_t B = (int32_t)tapeQKV_.dim(0), T = (int32_t)tapeQKV_.dim(1);
    const int64_t C = tapeQKV_.dim(2);
    int32_t rows = keep;
    if (!stepsPerSequence) {
      const int end = acceptedSteps + keep < keep + T ? acceptedSteps + keep : keep + T;   // :156
      rows = end > acceptedSteps ? end - acceptedSteps : 0;
    }
    Tensor out = Tensor::empty({B, rows, C}, tapeQKV_.dtype());
    if (rows > 0)
      check(dflash_rebuild_conv_state(hasSnapshot_ && snapshot_[0].defined() ? snapshot_[0].data() : nullptr, tapeQKV_.data(),
                                      stepsPerSequence ? static_cast<const int32_t*>(stepsPerSequence->data()) : nullptr,
                                      acceptedSteps, out.data(), B, T, keep, C * (int64_t)dtypeSize(tapeQKV_.dtype()), &rows, stream));
    return out;
  }
  void clearTransients() {   // :163-170
    armed_ = false;
    tape_ = tapeK_ = tapeG_ = tapeQKV_ = Tensor();
    snapshot_[0] = snapshot_[1] = Tensor();
    hasSnapshot_ = false;
  }
  int64_t trim(int64_t n) {   // :175-181
    const int64_t trimmed = offset < n ? offset : n;
    offset -= trimmed;
    return trimmed;
  }

 private:
  void restoreSnapshot() {
    if (snapshot_[0].defined()) state[0] = snapshot_[0];
    if (snapshot_[1].defined()) state[1] = snapshot_[1];
  }
  int convKernelSize_;
  bool armed_ = false, hasSnapshot_ = false;
  Tensor tape_, tapeK_, tapeG_, tapeQKV_;
  Tensor snapshot_[2];
};

// Sources/DFlash/DFlashRuntime.swift:188-223: a fully accepted block keeps the verify state and only
// clears the transients (:194-202); otherwise every cache rolls back.
inline void restoreAfterAcceptance(std::vector<RecurrentRollbackCache*>& caches, int acceptanceLength, int draftedTokens,
                                   cudaStream_t stream = nullptr) {
  const bool fully = draftedTokens > 0 && acceptanceLength == draftedTokens;
  for (RecurrentRollbackCache* c : caches) {
    if (fully) c->clearTransients();
    else c->rollback(acceptanceLength, stream);
  }
}

// ---- attention KV cache around the verify pass ---------------------------------------------------
// The cache update of the target forward and the trim of restoreTargetCacheAfterAcceptance
// (Sources/DFlash/DFlashRuntime.swift:188-223) for a cache whose rows live in a page pool
// [pages, Hkv, pageTokens, D] (the layout batchedSDPA2Pass reads through a page table).  Committed lengths
// stay on the device: appendBlock -> attend -> commit never reads the accepted count.  Pages are handed out
// on the host from an upper bound of every sequence's length; sync() reads the true lengths, tightens the
// bounds and returns unreachable pages.  attend() needs pageTokens to be a multiple of 128.
class PagedKVCache {
 public:
  PagedKVCache(int32_t batch, int32_t kvHeads, int32_t headDim, int32_t pageTokens, int32_t numPages, int32_t maxPages,
               DType dtype = DType::BF16)
      : B_(batch), Hkv_(kvHeads), D_(headDim), pageTokens_(pageTokens), numPages_(numPages), maxPages_(maxPages), dtype_(dtype),
        tableHost_((size_t)batch * maxPages, -1), pages_(batch), upper_(batch, 0) {
    kPool = Tensor::empty({numPages, kvHeads, pageTokens, headDim}, dtype);
    vPool = Tensor::empty({numPages, kvHeads, pageTokens, headDim}, dtype);
    checkCuda(cudaMemset(kPool.data(), 0, kPool.nbytes()));
    checkCuda(cudaMemset(vPool.data(), 0, vPool.nbytes()));
    pageTable = Tensor::fromHost(tableHost_.data(), {batch, maxPages}, DType::I32);
    std::vector<int32_t> zeros(batch, 0);
    kvLen = Tensor::fromHost(zeros.data(), {batch}, DType::I32);
    kvLenBlock = Tensor::fromHost(zeros.data(), {batch}, DType::I32);
    for (int32_t p = numPages - 1; p >= 0; --p) free_.push_back(p);   // page 0 is handed out first
  }
  int32_t freePages() const { return (int32_t)free_.size(); }
  const std::vector<int32_t>& pagesOf(int32_t b) const { return pages_.at(b); }

  // Makes positions [0, tokens) of sequence b addressable; throws Error(DFLASH_ERR_WORKSPACE) when the pool or the table is full.
  void reserve(int32_t b, int64_t tokens) {
    const int64_t need = (tokens + pageTokens_ - 1) / pageTokens_;
    if (need > maxPages_) throw Error(DFLASH_ERR_WORKSPACE, "PagedKVCache: sequence needs more pages than its table holds");
    while ((int64_t)pages_[b].size() < need) {
      if (free_.empty()) throw Error(DFLASH_ERR_WORKSPACE, "PagedKVCache: page pool exhausted");
      const int32_t page = free_.back();
      free_.pop_back();
      tableHost_[(size_t)b * maxPages_ + pages_[b].size()] = page;
      pages_[b].push_back(page);
      dirty_ = true;
    }
  }
  // kNew, vNew [B,Hkv,T,D]: row t of sequence b goes to position kvLen[b] + t.  Returns the lengths including the block.
  const Tensor& appendBlock(const Tensor& kNew, const Tensor& vNew, cudaStream_t stream = nullptr) {
    const int32_t T = (int32_t)kNew.dim(2);
    for (int32_t b = 0; b < B_; ++b) reserve(b, upper_[b] + T);
    flushTable(stream);
    check(dflash_kv_append(kNew.data(), vNew.data(), kPool.data(), vPool.data(), static_cast<const int32_t*>(pageTable.data()),
                           static_cast<const int32_t*>(kvLen.data()), 0, static_cast<int32_t*>(kvLenBlock.data()), B_, Hkv_, T, D_, 0,
                           pageTokens_, maxPages_, numPages_, (int32_t)dtype_, stream));
    appended_ = T;
    return kvLenBlock;
  }
  // Block-verify attention of queries [B,Hq,16,D] over the committed tokens and the block just appended.
  std::optional<Tensor> attend(const Tensor& queries, float scale, cudaStream_t stream = nullptr) {
    const int32_t Hq = (int32_t)queries.dim(1);
    int64_t nMax = 0;
    for (int64_t u : upper_) nMax = u > nMax ? u : nMax;
    nMax += appended_;
    if (nMax > (int64_t)maxPages_ * pageTokens_) nMax = (int64_t)maxPages_ * pageTokens_;
    const size_t need = dflash_verify_sdpa_workspace_bytes(B_, Hq, Hkv_, D_, (int32_t)nMax);
    if (!ws_.defined() || ws_.nbytes() < need) ws_ = Tensor::empty({(int64_t)need}, DType::U8);
    Tensor out = Tensor::empty(queries.shape(), queries.dtype());
    const int32_t st = dflash_verify_sdpa(queries.data(), kPool.data(), vPool.data(), static_cast<const int32_t*>(pageTable.data()),
                                          static_cast<const int32_t*>(kvLenBlock.data()), nullptr, out.data(), ws_.data(), ws_.nbytes(),
                                          B_, Hq, Hkv_, 16, D_, (int32_t)nMax, pageTokens_, maxPages_, numPages_, scale, (int32_t)queries.dtype(),
                                          DFLASH_KV_DENSE, stream);
    if (st == DFLASH_ERR_UNSUPPORTED) return std::nullopt;
    check(st);
    return out;
  }
  // commitCount: device int32[B], accepted drafts + 1 (replay_len of dflash_accept_lengths).
  void commit(const Tensor& commitCount, cudaStream_t stream = nullptr) {
    check(dflash_kv_commit(static_cast<int32_t*>(kvLen.data()), static_cast<const int32_t*>(commitCount.data()), B_, appended_, stream));
    for (int32_t b = 0; b < B_; ++b) upper_[b] += appended_;
    appended_ = 0;
  }
  // Reads the committed lengths, tightens the host bounds and returns the pages beyond them to the pool.
  std::vector<int32_t> sync(cudaStream_t stream = nullptr) {
    std::vector<int32_t> lens(B_);
    kvLen.toHost(lens.data(), stream);
    for (int32_t b = 0; b < B_; ++b) {
      upper_[b] = lens[b];
      const int64_t keep = ((int64_t)lens[b] + pageTokens_ - 1) / pageTokens_;
      while ((int64_t)pages_[b].size() > keep) {
        free_.push_back(pages_[b].back());
        pages_[b].pop_back();
        tableHost_[(size_t)b * maxPages_ + pages_[b].size()] = -1;
        dirty_ = true;
      }
    }
    flushTable(stream);
    return lens;
  }

  Tensor kPool, vPool, pageTable, kvLen, kvLenBlock;

 private:
  void flushTable(cudaStream_t stream) {
    if (!dirty_) return;
    // pageable source: the copy has read the host table when the call returns, so it may be edited again at once
    checkCuda(cudaMemcpyAsync(pageTable.data(), tableHost_.data(), tableHost_.size() * sizeof(int32_t), cudaMemcpyHostToDevice, stream));
    dirty_ = false;
  }
  int32_t B_, Hkv_, D_, pageTokens_, numPages_, maxPages_;
  DType dtype_;
  std::vector<int32_t> tableHost_;
  std::vector<std::vector<int32_t>> pages_;
  std::vector<int64_t> upper_;
  std::vector<int32_t> free_;
  Tensor ws_;
  int32_t appended_ = 0;
  bool dirty_ = false;
};

// Contiguous [begin, end) ranges of `units` work units (sequences, or (sequence, KV head) pairs) per GPU.
inline std::vector<std::pair<int32_t, int32_t>> partitionPlan(int32_t units, int32_t nGpus) {
  std::vector<int32_t> raw(2 * (size_t)nGpus);
  check(dflash_partition_plan(units, nGpus, raw.data()));
  std::vector<std::pair<int32_t, int32_t>> out;
  for (int i = 0; i < nGpus; ++i) out.emplace_back(raw[2 * i], raw[2 * i + 1]);
  return out;
}

}  // namespace host
}  // namespace dflash
