// Device side of the push dispatch, shared by the stand-alone dispatch kernel's callers and by the
// dispatch warps that ride inside the grouped GEMM (the GEMM that consumes the rows also sends this
// rank's rows, so the NVLink transfer overlaps the first tiles instead of preceding them).
//
// Reference: the dispatch PUT tasks and the first grouped matmul run inside one launch, wired per
// expert by event counters (hyper_multicore/ops/hyper_mega_moe/op_kernel/worker_kernel.cpp:301-366,
// hyper_multicore/ops/runtime/worker_kernel.h:141-183, hyper_multicore/tasks/gmm.py:154-160); remote
// destinations are served in rank-rotated order (hyper_multicore/scheduler/scheduler.py:27-53).
#pragma once

#include "common.cuh"

namespace hmc {

// Everything a warp needs to send rows of this rank to their owners.
struct DispatchFuse {
  const uint4* tokens;                  // [tokens, H] (with source_of_row) or expert-major [rows, H]
  const int* source_of_row;             // flat (token * top_k + slot) index of each expert-major row, or null
  const int* expert_of_row;             // global expert of each expert-major row
  const long long* dispatch_src_off;    // [experts] first source row of each expert
  const long long* dispatch_target_off; // [experts] first row of this rank's segment on the owner
  const long long* send_order_start;    // [experts + 1] prefix of the segments in sending order, or null
  long long rows;
  long long capacity_rows;
  void* peer_data[HMC_MAX_EP];          // receive buffer of every rank
  int* peer_ctrl[HMC_MAX_EP];           // control block of every rank
  const int* local_ctrl;
  const float* row_values;              // optional per-row scalar (routing probability)
  const int* value_index;
  long long value_plane_offset;
  unsigned long long budget_ns;
  int top_k;
  int vec_per_row;
  int ep;
  int rank;
  int local_experts;
  int generation;
};

#ifdef __CUDACC__

// One warp copies one row of `vec_per_row` 16-byte vectors, eight (then four) loads in flight per lane: the
// stores are posted writes (over NVLink for a remote owner), so the bytes in flight are set by the loads.
__device__ __forceinline__ void copy_row_warp(uint4* __restrict__ dst, const uint4* __restrict__ src, int vec_per_row,
                                              int lane) {
  int v = lane;
  for (; v + 224 < vec_per_row; v += 256) {
    uint4 q[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) q[u] = ld_nc_16(src + v + 32 * u);
#pragma unroll
    for (int u = 0; u < 8; ++u) st_16(dst + v + 32 * u, q[u]);
  }
  for (; v + 96 < vec_per_row; v += 128) {
    uint4 q[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) q[u] = ld_nc_16(src + v + 32 * u);
#pragma unroll
    for (int u = 0; u < 4; ++u) st_16(dst + v + 32 * u, q[u]);
  }
  for (; v < vec_per_row; v += 32) st_16(dst + v, ld_nc_16(src + v));
}

// Rows one warp sends between two counter updates. Small on purpose: the first tile of the carrying GEMM
// cannot start before one whole round of groups has been sent, and that round lasts as long as one warp
// needs for its group.
constexpr int DISPATCH_WARP_ROWS = 2;

// One warp sends its share of the rows: worker `worker` of `workers` takes every workers-th group of
// DISPATCH_WARP_ROWS rows of the sending order (send_order_start: local expert 0 of every destination,
// remote destinations first, then local expert 1, ...), so that every owner's early experts are complete
// early and their tiles overlap the rest of the transfer. After each group one release-add per expert
// advances the owners' arrival counters. Returns false when a peer never became ready (status set).
__device__ __forceinline__ bool dispatch_rows_warp(const DispatchFuse& d, int worker, int workers, int lane,
                                                   int* status) {
  if (d.rows <= 0) return true;
  const int experts = d.ep * d.local_experts;
  unsigned ready_mask = 0;  // peers seen ready for this generation (warp-uniform)
  const long long groups = (d.rows + DISPATCH_WARP_ROWS - 1) / DISPATCH_WARP_ROWS;
  for (long long group = worker; group < groups; group += workers) {
    const long long i0 = group * DISPATCH_WARP_ROWS;
    const int count = static_cast<int>(min(static_cast<long long>(DISPATCH_WARP_ROWS), d.rows - i0));
    // lane r < count owns the metadata of row r of the group
    int e = -1;
    long long j = 0, dest_row = 0, src_row = 0;
    if (lane < count) {
      j = i0 + lane;
      if (d.send_order_start != nullptr) {
        // position j of the sending order lies in segment q = le * ep + dd: the last q whose start is <= j
        int lo = 0, hi = experts - 1;
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (d.send_order_start[mid] <= j) lo = mid; else hi = mid - 1;
        }
        const int owner_of = (d.rank + 1 + lo % d.ep) % d.ep;
        const int segment_expert = owner_of * d.local_experts + lo / d.ep;
        j = d.dispatch_src_off[segment_expert] + (j - d.send_order_start[lo]);
      }
      e = (j >= 0 && j < d.rows) ? d.expert_of_row[j] : -1;
      if (e < 0 || e >= experts) {
        report_status(status, HMC_STATUS_BAD_INDEX, static_cast<int>(j), e, 0);
        e = -1;
      } else {
        dest_row = d.dispatch_target_off[e] + (j - d.dispatch_src_off[e]);
        if (dest_row < 0 || dest_row >= d.capacity_rows) {
          report_status(status, HMC_STATUS_BAD_INDEX, static_cast<int>(j), e, static_cast<int>(dest_row));
          e = -1;  // this row is not counted as delivered
        }
        src_row = d.source_of_row != nullptr ? d.source_of_row[j] / d.top_k : j;
      }
    }
    const int owner = e >= 0 ? e / d.local_experts : -1;
    // every destination of the group must have declared itself ready before anyone stores
    unsigned wanted = 0;
    for (int r = 0; r < count; ++r) {
      const int o = __shfl_sync(0xffffffffu, owner, r);
      if (o >= 0) wanted |= 1u << o;
    }
    unsigned missing = wanted & ~ready_mask;
    while (missing != 0) {
      const int p = __ffs(missing) - 1;
      int ok = 1;
      if (lane == 0) {
        int observed = 0;
        if (!wait_counter_ge(d.local_ctrl + HMC_CTRL_READY + p * HMC_CTRL_READY_STRIDE, d.generation, d.budget_ns,
                             &observed)) {
          report_status(status, HMC_STATUS_TIMEOUT_READY, p, d.generation, observed);
          ok = 0;
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) return false;
      ready_mask |= 1u << p;
      missing &= missing - 1;
    }
    for (int r = 0; r < count; ++r) {
      const int er = __shfl_sync(0xffffffffu, e, r);
      const long long sr = __shfl_sync(0xffffffffu, src_row, r);
      const long long dr = __shfl_sync(0xffffffffu, dest_row, r);
      if (er < 0) continue;
      const int o = er / d.local_experts;
      const uint4* src = d.tokens + sr * d.vec_per_row;
      uint4* dst = static_cast<uint4*>(d.peer_data[o]) + dr * d.vec_per_row;
      copy_row_warp(dst, src, d.vec_per_row, lane);
    }
    if (d.row_values != nullptr && e >= 0) {
      // the row's scalar (its routing probability) lands in the float plane behind the owner's rows
      float* plane = reinterpret_cast<float*>(static_cast<unsigned char*>(d.peer_data[owner]) + d.value_plane_offset);
      plane[dest_row] = d.row_values[d.value_index != nullptr ? d.value_index[j] : j];
    }
    // The warp barrier orders every lane's stores before the leaders' releases, which publish them to
    // the acquiring owner: one release-add per expert of the group.
    __syncwarp();
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const bool first = e >= 0 && lane == __ffs(same) - 1;
    if (first) red_release_sys_add(d.peer_ctrl[owner] + HMC_CTRL_ARRIVAL + (e % d.local_experts), __popc(same));
  }
  return true;
}

#endif  // __CUDACC__

}  // namespace hmc
