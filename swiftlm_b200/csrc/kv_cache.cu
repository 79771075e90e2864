// KV cache maintenance around the block-verify attention, on the device.
//
// The reference appends the verify block's 16 key/value rows to the attention cache before the
// target forward and trims the cache back to the accepted prefix afterwards
// (Sources/DFlash/DFlashRuntime.swift:188-223: targetLen = start + accepted inputs, cache.trim(offset - targetLen)).
// Here the committed length of every sequence lives in a device array, so neither step needs the
// accepted count on the host:
//   kv_append  writes row t of sequence b at position kv_len[b] + t of a dense cache [B,Hkv,N_cap,D]
//              or of a paged pool [pages,Hkv,page_tokens,D] through the sequence's page table, and
//              emits kv_len[b] + T (the length the verify attention sees);
//   kv_commit  kv_len[b] += clamp(commit[b], 0, T): the rejected rows stay where they are and are
//              overwritten by the next block, which is what trimming means for this layout.
// A position beyond the capacity or on an unmapped page is skipped and reported through the
// device status word (code kStatusKvRange).  Pure byte movement: one warp per row, 16-byte copies.
#include "common.cuh"

namespace dflash {

namespace {

constexpr int kRowsPerBlock = 8;

struct AppendParams {
  const uint8_t* k_new;
  const uint8_t* v_new;
  uint8_t* k_cache;
  uint8_t* v_cache;
  const int32_t* page_table;
  const int32_t* kv_len;
  int32_t* kv_len_out;
  int B, Hkv, T, capacity, page_tokens, max_pages, num_pages, len_all;
  int row_bytes;
  int* status;
};

__global__ void __launch_bounds__(kRowsPerBlock * 32) kv_append_kernel(const AppendParams p) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * kRowsPerBlock + (threadIdx.x >> 5);   // (b, h, t)
  const long long rows = (long long)p.B * p.Hkv * p.T;
  if (row >= rows) return;
  const int t = (int)(row % p.T);
  const int h = (int)((row / p.T) % p.Hkv);
  const int b = (int)(row / ((long long)p.T * p.Hkv));
  const int base = p.kv_len ? p.kv_len[b] : p.len_all;
  if (p.kv_len_out && h == 0 && t == 0 && lane == 0) {
    // never hand the attention a length past the cache: rows that did not fit were skipped (and reported)
    const long long want = (long long)(base < 0 ? 0 : base) + p.T;
    p.kv_len_out[b] = (int)(want < p.capacity ? want : p.capacity);
  }
  const int pos = base + t;
  long long dst_row = -1;
  if (base >= 0 && pos < p.capacity) {
    if (p.page_table) {
      const int page = p.page_table[(long long)b * p.max_pages + pos / p.page_tokens];
      if (page >= 0 && page < p.num_pages) dst_row = ((long long)page * p.Hkv + h) * p.page_tokens + pos % p.page_tokens;
    } else {
      dst_row = ((long long)b * p.Hkv + h) * p.capacity + pos;
    }
  }
  if (dst_row < 0) {
    if (lane == 0) atomicExch(p.status, kStatusKvRange);
    return;
  }
  const long long src = row * p.row_bytes, dst = dst_row * p.row_bytes;
  for (int i = lane * 16; i < p.row_bytes; i += 32 * 16) {
    *reinterpret_cast<uint4*>(p.k_cache + dst + i) = *reinterpret_cast<const uint4*>(p.k_new + src + i);
    *reinterpret_cast<uint4*>(p.v_cache + dst + i) = *reinterpret_cast<const uint4*>(p.v_new + src + i);
  }
}

__global__ void kv_commit_kernel(int32_t* kv_len, const int32_t* commit, int B, int T) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  int c = commit[b];
  c = c < 0 ? 0 : (c > T ? T : c);
  kv_len[b] += c;
}

}  // namespace
}  // namespace dflash

extern "C" int32_t dflash_kv_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                                    const int32_t* page_table, const int32_t* kv_len, int32_t len_all,
                                    int32_t* kv_len_out, int32_t B, int32_t Hkv, int32_t T, int32_t D,
                                    int32_t capacity, int32_t page_tokens, int32_t max_pages, int32_t num_pages,
                                    int32_t dtype, void* stream) {
  using namespace dflash;
  if (!k_new || !v_new || !k_cache || !v_cache || B <= 0 || Hkv <= 0 || T <= 0 || D <= 0) {
    set_error("kv_append: invalid argument");
    return DFLASH_ERR_INVALID_ARG;
  }
  if (dtype != DFLASH_BF16 && dtype != DFLASH_F16 && dtype != DFLASH_F32) {
    set_error("kv_append: unsupported dtype %d", dtype);
    return DFLASH_ERR_UNSUPPORTED;
  }
  const long long row_bytes = (long long)D * (dtype == DFLASH_F32 ? 4 : 2);
  if (row_bytes % 16 != 0 || ((uintptr_t)k_new & 15) || ((uintptr_t)v_new & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15)) {
    set_error("kv_append: rows must be multiples of 16 bytes and the arrays 16-byte aligned");
    return DFLASH_ERR_INVALID_ARG;
  }
  if (page_table) {
    if (page_tokens <= 0 || max_pages <= 0 || num_pages <= 0) { set_error("kv_append: paged cache needs page_tokens, max_pages, num_pages"); return DFLASH_ERR_INVALID_ARG; }
    if ((long long)max_pages * page_tokens > 0x7fffffffLL) { set_error("kv_append: page table too long"); return DFLASH_ERR_INVALID_ARG; }
    capacity = max_pages * page_tokens;
  } else if (capacity <= 0) {
    set_error("kv_append: dense cache needs its capacity");
    return DFLASH_ERR_INVALID_ARG;
  }
  if (!kv_len && len_all < 0) { set_error("kv_append: negative length"); return DFLASH_ERR_INVALID_ARG; }
  int* status = device_status_word();
  if (!status) { set_error("no CUDA device"); return DFLASH_ERR_CUDA; }
  AppendParams p{reinterpret_cast<const uint8_t*>(k_new), reinterpret_cast<const uint8_t*>(v_new),
                 reinterpret_cast<uint8_t*>(k_cache), reinterpret_cast<uint8_t*>(v_cache), page_table, kv_len, kv_len_out,
                 B, Hkv, T, capacity, page_tokens, max_pages, num_pages, len_all, (int)row_bytes, status};
  const long long rows = (long long)B * Hkv * T;
  const long long blocks = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
  if (blocks > 0x7fffffffLL) { set_error("kv_append: too many rows"); return DFLASH_ERR_UNSUPPORTED; }
  kv_append_kernel<<<(unsigned)blocks, kRowsPerBlock * 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  DFLASH_LAUNCH_CHECK();
  count_launch();
  return DFLASH_OK;
}

extern "C" int32_t dflash_kv_commit(int32_t* kv_len, const int32_t* commit, int32_t B, int32_t T, void* stream) {
  using namespace dflash;
  if (!kv_len || !commit || B <= 0 || T <= 0) {
    set_error("kv_commit: invalid argument");
    return DFLASH_ERR_INVALID_ARG;
  }
  kv_commit_kernel<<<(unsigned)((B + 127) / 128), 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(kv_len, commit, B, T);
  DFLASH_LAUNCH_CHECK();
  count_launch();
  return DFLASH_OK;
}
