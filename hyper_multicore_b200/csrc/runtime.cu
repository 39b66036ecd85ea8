// Process-level pieces of the hmc_* C ABI: thread-local error text, device queries, versions.
#include <string.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace hmc {

static std::atomic<long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// ------------------------------------------------------------------------------------- profiling
struct ProfileRecord {
  cudaEvent_t start, stop;
  int kind;
};
static std::atomic<int> g_profile_on{0};
static std::mutex g_profile_mutex;
static std::vector<ProfileRecord> g_profile_records;

// Events are created when profiling is switched on, not inside the measured call sequence: creating one
// costs the host microseconds the GPU would spend idle between two launches.
static std::vector<cudaEvent_t> g_profile_pool;

static cudaEvent_t take_event() {
  {
    std::lock_guard<std::mutex> lock(g_profile_mutex);
    if (!g_profile_pool.empty()) {
      cudaEvent_t e = g_profile_pool.back();
      g_profile_pool.pop_back();
      return e;
    }
  }
  cudaEvent_t e = nullptr;
  return cudaEventCreate(&e) == cudaSuccess ? e : nullptr;
}

ProfileScope::ProfileScope(int kind, cudaStream_t stream) : kind_(kind), stream_(stream), start_(nullptr), active_(false) {
  if (((g_profile_on.load(std::memory_order_relaxed) >> kind) & 1) == 0) return;
  start_ = take_event();
  if (start_ == nullptr) return;
  if (cudaEventRecord(start_, stream_) != cudaSuccess) {
    cudaEventDestroy(start_);
    return;
  }
  active_ = true;
}

ProfileScope::~ProfileScope() {
  if (!active_) return;
  cudaEvent_t stop = take_event();
  if (stop == nullptr || cudaEventRecord(stop, stream_) != cudaSuccess) {
    cudaEventDestroy(start_);
    if (stop != nullptr) cudaEventDestroy(stop);
    return;
  }
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  g_profile_records.push_back({start_, stop, kind_});
}

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
extern "C" int64_t hmc_launch_count(void) { return hmc::g_launches.load(std::memory_order_relaxed); }

extern "C" int hmc_profile_enable_kinds(uint32_t kinds_mask) {
  using namespace hmc;
  if (kinds_mask != 0) {
    std::lock_guard<std::mutex> lock(g_profile_mutex);
    while (g_profile_pool.size() < 1024) {
      cudaEvent_t e = nullptr;
      if (cudaEventCreate(&e) != cudaSuccess) break;
      g_profile_pool.push_back(e);
    }
  }
  g_profile_on.store(static_cast<int>(kinds_mask & ((1u << HMC_PROFILE_KINDS) - 1u)), std::memory_order_relaxed);
  return 0;
}

extern "C" int hmc_profile_enable(int on) { return hmc_profile_enable_kinds(on ? (1u << HMC_PROFILE_KINDS) - 1u : 0u); }

extern "C" int hmc_profile_dump(int32_t* kinds, double* start_ms, double* duration_ms, int capacity) {
  using namespace hmc;
  std::vector<ProfileRecord> records;
  {
    std::lock_guard<std::mutex> lock(g_profile_mutex);
    records.swap(g_profile_records);
  }
  int written = 0;
  for (size_t i = 0; i < records.size(); ++i) {
    const ProfileRecord& r = records[i];
    float since = 0.0f, ms = 0.0f;
    if (kinds != nullptr && written < capacity && cudaEventSynchronize(r.stop) == cudaSuccess &&
        cudaEventElapsedTime(&ms, r.start, r.stop) == cudaSuccess &&
        cudaEventElapsedTime(&since, records[0].start, r.start) == cudaSuccess) {
      kinds[written] = r.kind;
      start_ms[written] = since;
      duration_ms[written] = ms;
      ++written;
    }
  }
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  for (const ProfileRecord& r : records) {
    g_profile_pool.push_back(r.start);
    g_profile_pool.push_back(r.stop);
  }
  return written;
}

extern "C" int hmc_profile_collect(double* ms_by_kind, int64_t* calls_by_kind, int kinds) {
  using namespace hmc;
  HMC_REQUIRE(ms_by_kind != nullptr && calls_by_kind != nullptr && kinds > 0, HMC_ERR_INVALID,
              "hmc_profile_collect: bad arguments");
  for (int k = 0; k < kinds; ++k) {
    ms_by_kind[k] = 0.0;
    calls_by_kind[k] = 0;
  }
  std::vector<ProfileRecord> records;
  {
    std::lock_guard<std::mutex> lock(g_profile_mutex);
    records.swap(g_profile_records);
  }
  int rc = 0;
  for (const ProfileRecord& r : records) {
    float ms = 0.0f;
    if (cudaEventSynchronize(r.stop) != cudaSuccess || cudaEventElapsedTime(&ms, r.start, r.stop) != cudaSuccess) {
      rc = HMC_ERR_CUDA;
    } else if (r.kind >= 0 && r.kind < kinds) {
      ms_by_kind[r.kind] += ms;
      calls_by_kind[r.kind] += 1;
    }
    std::lock_guard<std::mutex> lock(g_profile_mutex);
    g_profile_pool.push_back(r.start);
    g_profile_pool.push_back(r.stop);
  }
  if (rc != 0) set_error("hmc_profile_collect: an event could not be read");
  return rc;
}

namespace {
__global__ void store_words_kernel(int* __restrict__ dst, const int* __restrict__ src, long long words) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < words; i += stride) dst[i] = src[i];
  __threadfence_system();
}
}  // namespace

namespace {
__global__ void store_words_pair_kernel(int* __restrict__ dst, const int* __restrict__ first, long long first_words,
                                        const int* __restrict__ second, long long second_words) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < first_words + second_words; i += stride)
    dst[i] = i < first_words ? first[i] : second[i - first_words];
  __threadfence_system();
}
}  // namespace

extern "C" int hmc_store_words_pair(int32_t* dst, const int32_t* first, int64_t first_words, const int32_t* second,
                                    int64_t second_words, void* stream_ptr) {
  HMC_REQUIRE(dst != nullptr && first != nullptr && second != nullptr && first_words >= 0 && second_words >= 0,
              HMC_ERR_INVALID, "hmc_store_words_pair: bad arguments");
  const long long words = first_words + second_words;
  if (words == 0) return 0;
  hmc::ProfileScope profile(HMC_PROFILE_ROUTE, static_cast<cudaStream_t>(stream_ptr));
  const int blocks = static_cast<int>(words < 256 * 64 ? (words + 255) / 256 : 64);
  store_words_pair_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(dst, first, first_words, second,
                                                                                   second_words);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_store_words(int32_t* dst, const int32_t* src, int64_t words, void* stream_ptr) {
  HMC_REQUIRE(dst != nullptr && src != nullptr && words >= 0, HMC_ERR_INVALID, "hmc_store_words: bad arguments");
  hmc::ProfileScope profile(HMC_PROFILE_ROUTE, static_cast<cudaStream_t>(stream_ptr));
  if (words == 0) return 0;
  const int blocks = static_cast<int>(words < 256 * 64 ? (words + 255) / 256 : 64);
  store_words_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(dst, src, words);
  HMC_LAUNCH_OK();
  return 0;
}
