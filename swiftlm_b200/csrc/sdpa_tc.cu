#include "common.cuh"
namespace dflash {
size_t sdpa_simple_workspace_bytes(int B, int Hq, int D);
size_t sdpa_workspace_bytes(int B, int Hq, int Hkv, int D, int N) { return sdpa_simple_workspace_bytes(B, Hq, D) + 256; }
bool sdpa_tc_supported(const SdpaArgs&) { return false; }
int32_t launch_sdpa_tc(const SdpaArgs&, cudaStream_t) { return DFLASH_ERR_UNSUPPORTED; }
}  // namespace dflash
