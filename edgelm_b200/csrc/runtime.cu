// Error reporting and small queries of the kernel library.
#include <cstdarg>
#include <cstring>

#include "common.cuh"

namespace edgelm {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

static int g_pdl = 57;   // the few-rows matrix products (bit 0), the tcgen05 products (bits 3 and 5), the tcgen05 prefill attention
                         // (bit 4), RMSNorm and the rotation (bit 5) start under the tail of the kernel before them
int pdl_enabled() { return g_pdl; }

}  // namespace edgelm

// Switch programmatic dependent launch of the decode kernels on (1, the default) or off (0).
extern "C" int edgelm_set_pdl(int on) {
  edgelm::g_pdl = on;
  return 0;
}

// Message of the last refused or failed call of this thread.
extern "C" const char* edgelm_last_error() { return edgelm::g_error; }

// Compute capability of the current device as major * 10 + minor, or a negative code.
extern "C" int edgelm_device_arch() {
  int dev = 0, major = 0, minor = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) return -1;
  return major * 10 + minor;
}
