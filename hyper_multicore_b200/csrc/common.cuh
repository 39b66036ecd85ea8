// Shared host/device helpers for the hmc_* C-ABI library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/hmc_b200.h"

namespace hmc {

// ---------------------------------------------------------------------------------------------
// Host-side error reporting: every entry point returns 0 or a negative HMC_ERR_* code and leaves
// a human-readable message retrievable with hmc_last_error(). Nothing throws, nothing syncs.
// ---------------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);

#define HMC_REQUIRE(cond, code, ...)             \
  do {                                           \
    if (!(cond)) {                               \
      ::hmc::set_error(__VA_ARGS__);             \
      return (code);                             \
    }                                            \
  } while (0)

#define HMC_CUDA_OK(expr)                                                            \
  do {                                                                               \
    cudaError_t err__ = (expr);                                                      \
    if (err__ != cudaSuccess) {                                                      \
      ::hmc::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__),    \
                       __FILE__, __LINE__);                                          \
      return HMC_ERR_CUDA;                                                           \
    }                                                                                \
  } while (0)

#define HMC_LAUNCH_OK()                                                              \
  do {                                                                               \
    cudaError_t err__ = cudaGetLastError();                                          \
    if (err__ != cudaSuccess) {                                                      \
      ::hmc::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(err__),\
                       __FILE__, __LINE__);                                          \
      return HMC_ERR_CUDA;                                                           \
    }                                                                                \
    ::hmc::count_launch();                                                           \
  } while (0)

void count_launch();  // one more kernel of this library launched (hmc_launch_count)

// Brackets the launches of one entry point with CUDA events while profiling is on (hmc_profile_enable):
// per-kind device time for callers that report where a step's time goes. Does nothing when it is off.
struct ProfileScope {
  ProfileScope(int kind, cudaStream_t stream);
  ~ProfileScope();
  int kind_;
  cudaStream_t stream_;
  cudaEvent_t start_;
  bool active_;
};

int sm_count();  // number of SMs on the current device (cached per device)
int moe_unpermute_unless(const void* permuted, const int32_t* mapping, const float* probs, int64_t num_tokens,
                         int64_t top_k, int64_t hidden, int64_t permuted_rows, void* out, int32_t* status,
                         const int32_t* skip_flag, void* stream);  // route_prep.cu

// cudaFuncAttributeMaxDynamicSharedMemorySize belongs to a (kernel, device) pair: every launch site keeps one
// PerDeviceFlag and raises the limit the first time it launches on each device ordinal.
constexpr int HMC_MAX_DEVICES = 64;
struct PerDeviceFlag {
  bool done[HMC_MAX_DEVICES];
};

template <typename Kernel>
static inline int allow_dynamic_smem(Kernel kernel, int bytes, PerDeviceFlag& flag) {
  int dev = 0;
  HMC_CUDA_OK(cudaGetDevice(&dev));
  const bool tracked = dev >= 0 && dev < HMC_MAX_DEVICES;
  if (!tracked || !flag.done[dev]) {
    HMC_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    if (tracked) flag.done[dev] = true;
  }
  return 0;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------------------------------------
// Device helpers
// ---------------------------------------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ float bf16_round(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float2 unpack_bf16x2(uint32_t v) {
  __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&v);
  return __bfloat1622float2(b);
}

__device__ __forceinline__ uint4 ld_nc_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint4 ld_16(const void* p) {
  return *reinterpret_cast<const uint4*>(p);
}

__device__ __forceinline__ void st_16(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

// Streaming 16-byte store (written once, not re-read by this kernel).
__device__ __forceinline__ void st_cs_16(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// System-scope acquire load / release add used by the peer-buffer protocol.
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Device status word layout (int32[HMC_STATUS_WORDS]); word 0 is 0 while healthy. The first
// failing thread wins the compare-and-swap and records what it was waiting for.
__device__ __forceinline__ void report_status(int* status, int code, int a, int b, int c) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = a;
    status[2] = b;
    status[3] = c;
    __threadfence();
  }
}

// Bounded poll on a local counter that peers (or other CTAs) advance. Returns false on time-out.
// With `status`, the wait also ends (false) as soon as the status words carry an error: whoever was to
// advance the counter may be the one that failed.
__device__ __forceinline__ bool wait_counter_ge(const int* counter, int expected, uint64_t budget_ns,
                                                int* observed, const int* status = nullptr) {
  int v = ld_acquire_sys(counter);
  if (v >= expected) {
    *observed = v;
    return true;
  }
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      v = ld_acquire_sys(counter);
      if (v >= expected) {
        *observed = v;
        return true;
      }
      __nanosleep(64);
    }
    if (global_timer_ns() - t0 > budget_ns) break;
    if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) break;
  }
  *observed = v;
  return false;
}

#endif  // __CUDACC__

// Result rows that leave the epilogue for their source ranks (fused combine).
struct CombineFuse {
  const long long* segment_start;       // [local_experts * ep] first row of (local expert, source)
  const long long* combine_target_off;  // [ep * local_experts]
  void* peer_data[HMC_MAX_EP];          // routed buffer of every rank
  int* peer_ctrl[HMC_MAX_EP];           // control block of every rank
  long long target_rows_limit;
  int ep;
  int local_experts;
};


}  // namespace hmc
