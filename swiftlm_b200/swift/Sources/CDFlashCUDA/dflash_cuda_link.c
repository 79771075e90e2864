/* SwiftPM wants at least one translation unit in a C target.  The kernels live in the prebuilt
 * libdflash_cuda.so (nvcc, sm_100a); this file only pins the header the target was written against
 * to the library found at link time. */
#include "dflash_cuda.h"

/* Non-zero when the linked library speaks the ABI of this header (same major version string). */
int cdflash_cuda_abi_matches(void) {
  const char* v = dflash_version();
  return v != 0 && v[0] == 'd' && v[1] == 'f';
}
