// Conv-window rebuild of the rollback cache on the device.
//
// RecurrentRollbackCache.rebuildConvState (Sources/DFlash/RecurrentRollbackCache.swift:139-158):
//   conv_input = concat(conv_snapshot [B, keep, C], qkv [B, T, C]) along the step axis
//   new window = conv_input[:, steps : min(steps + keep, keep + T)]        keep = conv kernel size - 1
// with steps = accepted_steps.  Here the step count may differ per sequence (a device array), in
// which case every sequence gets keep rows and the start is clamped so that the window stays
// inside conv_input.  Pure byte movement: one block per (sequence, window row), 16-byte copies.
#include "common.cuh"

namespace dflash {
namespace {

__global__ void conv_window_kernel(const uint8_t* __restrict__ prefix, const uint8_t* __restrict__ qkv,
                                   const int32_t* __restrict__ steps_per_seq, int steps_all, uint8_t* __restrict__ out,
                                   int T, int keep, int rows_out, long long row_bytes, int steps_div) {
  const int b = blockIdx.x / rows_out, j = blockIdx.x % rows_out;
  int start = steps_per_seq ? steps_per_seq[b / steps_div] : steps_all;
  if (start < 0) start = 0;
  if (steps_per_seq && start > T) start = T;                 // keep rows must exist: the last window is qkv's tail
  const int src_row = start + j;                              // row of concat(prefix, qkv)
  const uint8_t* src = src_row < keep ? (prefix ? prefix + ((long long)b * keep + src_row) * row_bytes : nullptr)
                                      : qkv + ((long long)b * T + (src_row - keep)) * row_bytes;
  uint8_t* dst = out + ((long long)b * rows_out + j) * row_bytes;
  for (long long i = (long long)threadIdx.x * 16; i < row_bytes; i += (long long)blockDim.x * 16) {
    const uint4 v = src ? *reinterpret_cast<const uint4*>(src + i) : make_uint4(0, 0, 0, 0);   // no snapshot: zeros (:150-153)
    *reinterpret_cast<uint4*>(dst + i) = v;
  }
}

}  // namespace
}  // namespace dflash

namespace dflash {
int32_t launch_conv_window(const void* conv_snapshot, const void* qkv, const int32_t* steps_per_seq, int steps_all, void* out,
                           int B, int T, int keep, long long row_bytes, int32_t* rows_out, int steps_div, cudaStream_t stream) {
  if (!qkv || !out || B <= 0 || T <= 0 || keep <= 0 || row_bytes <= 0) {
    set_error("rebuild_conv_state: invalid argument");
    return DFLASH_ERR_INVALID_ARG;
  }
  if (row_bytes % 16 != 0 || ((uintptr_t)qkv & 15) || ((uintptr_t)out & 15) || ((uintptr_t)conv_snapshot & 15)) {
    set_error("rebuild_conv_state: rows must be multiples of 16 bytes and 16-byte aligned");
    return DFLASH_ERR_INVALID_ARG;
  }
  int rows = keep;
  if (!steps_per_seq) {
    if (steps_all < 0) { set_error("rebuild_conv_state: negative step count"); return DFLASH_ERR_INVALID_ARG; }
    const int end = steps_all + keep < keep + T ? steps_all + keep : keep + T;   // :156
    rows = end - steps_all;
    if (rows < 0) rows = 0;
  }
  if (rows_out) *rows_out = rows;
  if (rows == 0) return DFLASH_OK;
  conv_window_kernel<<<(unsigned)(B * rows), 128, 0, stream>>>(
      reinterpret_cast<const uint8_t*>(conv_snapshot), reinterpret_cast<const uint8_t*>(qkv), steps_per_seq, steps_all,
      reinterpret_cast<uint8_t*>(out), T, keep, rows, (long long)row_bytes, steps_div < 1 ? 1 : steps_div);
  DFLASH_LAUNCH_CHECK();
  count_launch();
  return DFLASH_OK;
}
}  // namespace dflash

extern "C" int32_t dflash_rebuild_conv_state(const void* conv_snapshot, const void* qkv, const int32_t* steps_per_seq,
                                             int32_t steps_all, void* out, int32_t B, int32_t T, int32_t keep,
                                             int64_t row_bytes, int32_t* rows_out, void* stream) {
  return dflash::launch_conv_window(conv_snapshot, qkv, steps_per_seq, steps_all, out, B, T, keep, (long long)row_bytes, rows_out, 1,
                                    reinterpret_cast<cudaStream_t>(stream));
}
