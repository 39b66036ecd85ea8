// Process-level pieces of the hmc_* C ABI: thread-local error text, device queries, versions.
#include <string.h>

#include "common.cuh"

namespace hmc {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace hmc

extern "C" const char* hmc_last_error(void) { return hmc::g_error; }
extern "C" int hmc_abi_version(void) { return HMC_ABI_VERSION; }
extern "C" int hmc_mega_moe_transport_version(void) { return 2; }
extern "C" int hmc_worker_queue_layout_version(void) { return 2; }
