// dflash_verify_sdpa_noalloc: block-verify attention for callers that cannot hand over scratch
// memory.
//
// dflash_verify_sdpa needs a caller-allocated workspace for its split-KV partials.  Some hosts
// cannot provide one: a runtime whose device-memory budget is fixed at start-up and whose
// allocator is off limits to plug-in code, a request path that must never reach cudaMalloc
// (an allocation can block behind other work on the device), or glue code that simply has no
// allocator to call.  For them the same kernels run on a scratch area that is part of the
// library image: a file-scope __device__ array of kScratchBytes.  Every GPU that loads the
// library carries this array until the process exits.
//
// Rules that follow from sharing one array:
//   * the first call on a device looks the array's device address up (cudaGetSymbolAddress)
//     and lets the CUDA runtime load the kernels; make that first call before any stream
//     capture starts;
//   * the array keeps whatever the previous call left in it; nothing in it has to start at
//     zero, because every launch rewrites the slot table entries and partials it later reads,
//     and the arrival flags carry a tag that is new for every launch;
//   * two calls that overlap on the GPU (different streams, or different threads) race on the
//     array: serialise them, or give the second caller dflash_verify_sdpa with its own buffer.
// The entry point allocates nothing: no cudaMalloc / cudaFree, no library routine that
// allocates.  A request whose scratch need exceeds kScratchBytes is rejected.
#include <mutex>

#include "common.cuh"

namespace dflash {
namespace {

// 40 MiB: enough for head_dim <= 256 on a GPU with up to 158 SMs (2 partial slots per SM, each
// 128 rows x (head_dim + 2) floats).
constexpr size_t kScratchBytes = 40u << 20;
static __device__ __align__(256) unsigned char g_sdpa_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_scratch_ptr[kMaxDevices] = {};

// The array's name is only a handle in host code; the kernels need its device address.
int32_t scratch_for_current_device(void** out) {
  int dev = 0;
  DFLASH_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    set_error("verify_sdpa_noalloc: device index %d out of range", dev);
    return DFLASH_ERR_INVALID_ARG;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    DFLASH_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_sdpa_scratch));
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return DFLASH_OK;
}

}  // namespace
}  // namespace dflash

extern "C" int32_t dflash_verify_sdpa_noalloc(const void* q, const void* k, const void* v,
                                              const int32_t* page_table, const int32_t* kv_len_per_seq,
                                              const void* mask, void* out, int32_t B, int32_t Hq, int32_t Hkv,
                                              int32_t T, int32_t D, int32_t N, int32_t page_tokens,
                                              int32_t max_pages, int32_t num_pages, float scale, int32_t dtype,
                                              int32_t kv_format, void* stream) {
  using namespace dflash;
  // 1. everything that can be rejected without touching the device, exactly as dflash_verify_sdpa answers it
  if (int32_t st = sdpa_check_args(q, k, v, page_table, out, B, Hq, Hkv, T, D, N, page_tokens, max_pages, num_pages,
                                   dtype, kv_format))
    return st;
  if (kv_format != DFLASH_KV_DENSE) {
    // the compressed form is expanded into scratch before attending: B*Hkv*N*D*4 bytes, which the built-in
    // area cannot hold for any realistic context
    set_error("verify_sdpa_noalloc: TurboQuant KV is not taken here (its expansion needs B*Hkv*N*D*4 bytes of scratch); "
              "use dflash_verify_sdpa with a workspace");
    return DFLASH_ERR_UNSUPPORTED;
  }
  // 2. the scratch the kernel that will run needs (the tensor-core kernel for every call it takes)
  const size_t need = sdpa_scratch_bytes_for_call(B, Hq, D, scale, kv_len_per_seq != nullptr);
  if (need > kScratchBytes) {
    set_error("verify_sdpa_noalloc: this call needs %zu bytes of scratch but the built-in area holds %zu "
              "(head_dim <= 256 on up to 158 SMs); use dflash_verify_sdpa with a workspace",
              need, (size_t)kScratchBytes);
    return DFLASH_ERR_WORKSPACE;
  }
  // 3. only now the device: the array's address (first call on this device), then the launch
  void* scratch = nullptr;
  if (int32_t st = scratch_for_current_device(&scratch)) return st;
  return dflash_verify_sdpa(q, k, v, page_table, kv_len_per_seq, mask, out, scratch, kScratchBytes, B, Hq, Hkv, T, D,
                            N, page_tokens, max_pages, num_pages, scale, dtype, kv_format, stream);
}
