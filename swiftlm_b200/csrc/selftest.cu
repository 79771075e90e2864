// dflash_selftest_bounded_wait: runs the give-up path of the kernels' bounded waits on purpose.
//
// Every device-side wait in this library has a poll budget; when it runs out the waiting role raises its
// CTA's abort flag, records a code in the per-device status word and returns, the other roles leave at their
// next poll, and dflash_device_status then answers DFLASH_ERR_DEVICE_TIMEOUT.  In normal operation no wait
// ever runs out, so this entry point makes one run out without anything going wrong on the device: a
// two-warp kernel in which warp 0 waits (with a budget of `polls` polls) on an mbarrier that nothing arrives
// at, and warp 1 waits on a second one with the full budget and has to leave through the abort flag.  It uses
// the same wait routine as the attention kernel (ptx::mbar_wait_or_abort).  No fault, no hang: the kernel
// returns after polls * ~40 ns.
#include "common.cuh"
#include "ptx.cuh"

namespace dflash {
namespace {

__global__ void __launch_bounds__(64) bounded_wait_selftest_kernel(int* status, uint32_t polls, int* left_by_flag) {
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bars[0], 1);
    ptx::mbar_init(&bars[1], 1);
    abort_flag = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    ptx::mbar_wait_or_abort(&bars[0], 0, &abort_flag, status, kStatusSelftestWait, polls);
  } else if (threadIdx.x == 32) {
    const bool ok = ptx::mbar_wait_or_abort(&bars[1], 0, &abort_flag, status, kStatusSelftestWait);
    if (!ok && abort_flag && left_by_flag) *left_by_flag = 1;
  }
}

}  // namespace
}  // namespace dflash

extern "C" int32_t dflash_selftest_bounded_wait(uint32_t polls, int32_t* left_by_flag, void* stream) {
  using namespace dflash;
  if (polls == 0 || polls > (1u << 20)) {
    set_error("selftest_bounded_wait: polls must be in [1, 2^20]");
    return DFLASH_ERR_INVALID_ARG;
  }
  int* status = device_status_word();
  if (!status) { set_error("no CUDA device"); return DFLASH_ERR_CUDA; }
  bounded_wait_selftest_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status, polls, left_by_flag);
  DFLASH_LAUNCH_CHECK();
  count_launch();
  return DFLASH_OK;
}
