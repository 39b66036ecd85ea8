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

namespace {
__global__ void store_words_kernel(int* __restrict__ dst, const int* __restrict__ src, long long words) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < words; i += stride) dst[i] = src[i];
  __threadfence_system();
}
}  // namespace

extern "C" int hmc_store_words(int32_t* dst, const int32_t* src, int64_t words, void* stream_ptr) {
  HMC_REQUIRE(dst != nullptr && src != nullptr && words >= 0, HMC_ERR_INVALID, "hmc_store_words: bad arguments");
  if (words == 0) return 0;
  const int blocks = static_cast<int>(words < 256 * 64 ? (words + 255) / 256 : 64);
  store_words_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(dst, src, words);
  HMC_LAUNCH_OK();
  return 0;
}
