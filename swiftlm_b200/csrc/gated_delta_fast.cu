#include "common.cuh"
namespace dflash {
bool gdn_fast_supported(const GdnArgs&) { return false; }
int32_t launch_gdn_fast(const GdnArgs&, cudaStream_t) { return DFLASH_ERR_UNSUPPORTED; }
}  // namespace dflash
