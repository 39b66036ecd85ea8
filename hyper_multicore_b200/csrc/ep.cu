// Expert-parallel transport over CUDA-IPC peer-mapped buffers (NVLink / NVSwitch).
//
// Replaces the reference's SHMEM data plane for the MoE path: the dispatch PUT task with its
// per-expert "signal ADD" (hyper_multicore/ops/hyper_mega_moe/op_kernel/worker_kernel.cpp:301-366,
// ops/common/mega_moe/transport_task.h:37-79, tasks/alltoall.py:90-157), the combine PUT
// (same files), the ready handshake before any remote write
// (ops/common/mega_moe/invocation_protocol.h:9-52) and the symmetric allocation
// (hyper_multicore/shmem/_api.py:77-182).
//
// Protocol (push mode, one process per GPU):
//   1. every rank zeroes its own arrival counters on its stream, then publishes "ready(g)" into
//      each peer's control block (generation g grows by one per operator call);
//   2. a sender polls its local copy of peer p's ready flag (bounded) before the first store to p;
//   3. rows travel as coalesced 16-byte stores through the peer pointer; after a chunk of rows the
//      CTA adds the number of rows it delivered to the owner's per-expert counter with a
//      system-scope release;
//   4. consumers (the grouped GEMM, or hmc_ep_wait) poll their local counter with acquire loads,
//      bounded, and write a status word instead of hanging when rows never arrive.
#include <string.h>

#include "common.cuh"
#include "ep_device.cuh"

namespace hmc {
namespace {

constexpr int ROWS_PER_CHUNK = 32;
constexpr int THREADS = 256;

struct PeerTable {
  void* data[HMC_MAX_EP];  // destination buffer on each peer (expert buffer or routed buffer)
  int* ctrl[HMC_MAX_EP];   // control block on each peer
};

__global__ void ep_publish_ready_kernel(PeerTable peers, int ep, int rank, int generation) {
  const int p = threadIdx.x;
  if (p < ep) st_release_sys(peers.ctrl[p] + HMC_CTRL_READY + rank * HMC_CTRL_READY_STRIDE, generation);
}

// Bounded wait until peer `p` has published `generation`; `seen` caches the answer per CTA.
__device__ __forceinline__ bool peer_ready(const int* local_ctrl, int p, int generation, uint64_t budget_ns,
                                           int* seen, int* status) {
  if (seen[p] >= generation) return true;
  int observed = 0;
  if (!wait_counter_ge(local_ctrl + HMC_CTRL_READY + p * HMC_CTRL_READY_STRIDE, generation, budget_ns, &observed)) {
    report_status(status, HMC_STATUS_TIMEOUT_READY, p, generation, observed);
    return false;
  }
  seen[p] = observed;
  return true;
}

// Dispatch: source row j (expert-major order on the source) -> owner of its expert.
//   tokens          : [num_tokens, H] when source_of_row != null (row j reads token source_of_row[j] / top_k)
//                     [rows, H] already expert-major when source_of_row == null (backward dY)
__global__ void __launch_bounds__(THREADS)
ep_dispatch_kernel(const uint4* __restrict__ tokens, const int* __restrict__ source_of_row,
                   const int* __restrict__ expert_of_row, const long long* __restrict__ dispatch_src_off,
                   const long long* __restrict__ dispatch_target_off, long long rows, int top_k, int vec_per_row,
                   int ep, int local_experts, long long capacity_rows, PeerTable peers,
                   const int* __restrict__ local_ctrl, int generation, unsigned long long budget_ns,
                   int* __restrict__ status, const float* __restrict__ row_values,
                   const int* __restrict__ value_index, long long value_plane_offset, const int* __restrict__ skip_flag,
                   int rank) {
  __shared__ int seen[HMC_MAX_EP];
  __shared__ int chunk_expert[ROWS_PER_CHUNK];
  __shared__ int failed;
  __shared__ long long first_chunk;
  if (skip_flag != nullptr && *reinterpret_cast<const volatile int*>(skip_flag) != 0) return;
  if (threadIdx.x < HMC_MAX_EP) seen[threadIdx.x] = -1;
  if (threadIdx.x == 0) {
    failed = 0;
    // The rows are expert-major, i.e. destination-major, and the grid walks them as one moving window: if every
    // rank started at row 0, all of them would send to rank 0's experts first, then to rank 1's, ... and one
    // receiver's link at a time would carry the whole group's traffic. Rank r starts with the rows of rank r + 1.
    first_chunk = ep > 1 ? dispatch_src_off[((rank + 1) % ep) * local_experts] / ROWS_PER_CHUNK : 0;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long chunks = (rows + ROWS_PER_CHUNK - 1) / ROWS_PER_CHUNK;
  for (long long turn = blockIdx.x; turn < chunks; turn += gridDim.x) {
    const long long chunk = (turn + first_chunk) % chunks;
    const long long j0 = chunk * ROWS_PER_CHUNK;
    const int count = static_cast<int>(min(static_cast<long long>(ROWS_PER_CHUNK), rows - j0));
    if (threadIdx.x < count) {
      int e = expert_of_row[j0 + threadIdx.x];
      if (e < 0 || e >= ep * local_experts) {
        report_status(status, HMC_STATUS_BAD_INDEX, static_cast<int>(j0 + threadIdx.x), e, 0);
        e = -1;
      }
      chunk_expert[threadIdx.x] = e;
    }
    __syncthreads();
    // one thread makes sure every destination of this chunk is ready before anyone stores
    if (threadIdx.x == 0) {
      for (int r = 0; r < count; ++r) {
        const int e = chunk_expert[r];
        if (e >= 0 && !peer_ready(local_ctrl, e / local_experts, generation, budget_ns, seen, status)) failed = 1;
      }
    }
    __syncthreads();
    if (failed) return;
    for (int r = warp; r < count; r += THREADS / 32) {
      const int e = chunk_expert[r];
      if (e < 0) continue;
      const long long j = j0 + r;
      const long long dest_row = dispatch_target_off[e] + (j - dispatch_src_off[e]);
      if (dest_row < 0 || dest_row >= capacity_rows) {
        if (lane == 0) report_status(status, HMC_STATUS_BAD_INDEX, static_cast<int>(j), e, static_cast<int>(dest_row));
        chunk_expert[r] = -1;  // this row is not counted as delivered
        continue;
      }
      const long long src_row = source_of_row != nullptr ? source_of_row[j] / top_k : j;
      const uint4* src = tokens + src_row * vec_per_row;
      uint4* dst = static_cast<uint4*>(peers.data[e / local_experts]) + dest_row * vec_per_row;
      copy_row_warp(dst, src, vec_per_row, lane);
      if (row_values != nullptr && lane == 0) {
        // the row's scalar (its routing probability) lands in the float plane behind the rows
        float* plane = reinterpret_cast<float*>(static_cast<unsigned char*>(peers.data[e / local_experts]) +
                                                value_plane_offset);
        plane[dest_row] = row_values[value_index != nullptr ? value_index[j] : j];
      }
    }
    __syncthreads();
    // One release-add per run of equal experts in the chunk. The barrier above orders every
    // warp's stores before this thread's release, which makes them visible to the acquirer.
    if (threadIdx.x < count) {
      const int e = chunk_expert[threadIdx.x];
      const bool first = e >= 0 && (threadIdx.x == 0 || chunk_expert[threadIdx.x - 1] != e);
      if (first) {
        int run = 1;
        while (threadIdx.x + run < count && chunk_expert[threadIdx.x + run] == e) ++run;
        red_release_sys_add(peers.ctrl[e / local_experts] + HMC_CTRL_ARRIVAL + (e % local_experts), run);
      }
    }
    __syncthreads();
  }
}

// Combine: row r of the owner's result buffer (local-expert-major, then source rank) -> the
// source's routed buffer at the row the source's own expert-major order gave it.
__global__ void __launch_bounds__(THREADS)
ep_combine_kernel(const uint4* __restrict__ results, const long long* __restrict__ segment_start,
                  const long long* __restrict__ combine_target_off, long long rows, int vec_per_row, int ep,
                  int local_experts, long long target_rows_limit, PeerTable peers,
                  const int* __restrict__ local_ctrl, int generation, unsigned long long budget_ns,
                  int* __restrict__ status, const float* __restrict__ result_values,
                  long long value_plane_offset) {
  __shared__ int seen[HMC_MAX_EP];
  __shared__ int chunk_source[ROWS_PER_CHUNK];
  __shared__ long long chunk_dest[ROWS_PER_CHUNK];
  __shared__ int failed;
  if (threadIdx.x < HMC_MAX_EP) seen[threadIdx.x] = -1;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int segments = ep * local_experts;
  const long long chunks = (rows + ROWS_PER_CHUNK - 1) / ROWS_PER_CHUNK;
  for (long long chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
    const long long r0 = chunk * ROWS_PER_CHUNK;
    const int count = static_cast<int>(min(static_cast<long long>(ROWS_PER_CHUNK), rows - r0));
    if (threadIdx.x < count) {
      const long long r = r0 + threadIdx.x;
      // last segment q (buffer order: local expert * ep + source) with segment_start[q] <= r
      int lo = 0, hi = segments - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (segment_start[mid] <= r) lo = mid; else hi = mid - 1;
      }
      const int le = lo / ep;
      const int s = lo % ep;
      const long long dest = combine_target_off[s * local_experts + le] + (r - segment_start[lo]);
      if (dest < 0 || dest >= target_rows_limit) {
        report_status(status, HMC_STATUS_BAD_INDEX, static_cast<int>(r), lo, static_cast<int>(dest));
        chunk_source[threadIdx.x] = -1;
      } else {
        chunk_source[threadIdx.x] = s;
      }
      chunk_dest[threadIdx.x] = dest;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int r = 0; r < count; ++r) {
        const int s = chunk_source[r];
        if (s >= 0 && !peer_ready(local_ctrl, s, generation, budget_ns, seen, status)) failed = 1;
      }
    }
    __syncthreads();
    if (failed) return;
    for (int r = warp; r < count; r += THREADS / 32) {
      const int s = chunk_source[r];
      if (s < 0) continue;
      const uint4* src = results + (r0 + r) * vec_per_row;
      uint4* dst = static_cast<uint4*>(peers.data[s]) + chunk_dest[r] * vec_per_row;
      copy_row_warp(dst, src, vec_per_row, lane);
      if (result_values != nullptr && lane == 0) {
        float* plane = reinterpret_cast<float*>(static_cast<unsigned char*>(peers.data[s]) + value_plane_offset);
        plane[chunk_dest[r]] = result_values[r0 + r];
      }
    }
    __syncthreads();
    if (threadIdx.x < count) {
      const int s = chunk_source[threadIdx.x];
      const bool first = s >= 0 && (threadIdx.x == 0 || chunk_source[threadIdx.x - 1] != s);
      if (first) {
        int run = 1;
        while (threadIdx.x + run < count && chunk_source[threadIdx.x + run] == s) ++run;
        red_release_sys_add(peers.ctrl[s] + HMC_CTRL_COMBINE, run);
      }
    }
    __syncthreads();
  }
}

// Count exchange: every rank stores its row into every peer's table, then waits for all rows.
__global__ void __launch_bounds__(256)
ep_exchange_counts_kernel(const int* __restrict__ counts, int h0, int h1, int h2, int h3, PeerTable peers,
                          const int* __restrict__ local_ctrl, int ep, int rank, int experts, int exchange,
                          unsigned long long budget_ns, int* __restrict__ status) {
  const long long half_words = static_cast<long long>(ep) * (experts + 4);
  const long long base = (exchange & 1) * half_words;
  for (int p = 0; p < ep; ++p) {
    int* table = static_cast<int*>(peers.data[p]) + base;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) table[static_cast<long long>(rank) * experts + e] = counts[e];
    if (threadIdx.x < 4) {
      const int h = threadIdx.x == 0 ? h0 : threadIdx.x == 1 ? h1 : threadIdx.x == 2 ? h2 : h3;
      table[static_cast<long long>(ep) * experts + rank * 4 + threadIdx.x] = h;
    }
  }
  __syncthreads();  // every store of this CTA is ordered before the releases below
  if (threadIdx.x < ep)
    st_release_sys(peers.ctrl[threadIdx.x] + HMC_CTRL_COUNTS + rank * HMC_CTRL_READY_STRIDE, exchange);
  if (threadIdx.x < ep) {
    int observed = 0;
    if (!wait_counter_ge(local_ctrl + HMC_CTRL_COUNTS + threadIdx.x * HMC_CTRL_READY_STRIDE, exchange, budget_ns,
                         &observed))
      report_status(status, HMC_STATUS_TIMEOUT_READY, threadIdx.x, exchange, observed);
  }
}

__global__ void ep_publish_source_kernel(PeerTable peers, int ep, int rank, int generation) {
  const int p = threadIdx.x;
  if (p < ep) st_release_sys(peers.ctrl[p] + HMC_CTRL_SOURCE + rank * HMC_CTRL_READY_STRIDE, generation);
}

// Pull: row r of this rank's receive layout (local-expert-major, then source rank) is fetched from the
// source's expert-major buffer. Plain (coherent) loads: the rows were written by another GPU during
// this call and become visible through the acquire of the source's flag.
__global__ void __launch_bounds__(THREADS)
ep_pull_kernel(PeerTable sources, const long long* __restrict__ source_row_off,
               const long long* __restrict__ segment_start, uint4* __restrict__ out, float* __restrict__ out_values,
               long long rows, int vec_per_row, int ep, int local_experts, long long source_rows_limit,
               long long value_plane_offset, const int* __restrict__ local_ctrl, int generation,
               unsigned long long budget_ns, int* __restrict__ status) {
  __shared__ int seen[HMC_MAX_EP];
  __shared__ int chunk_source[ROWS_PER_CHUNK];
  __shared__ long long chunk_row[ROWS_PER_CHUNK];
  __shared__ int failed;
  if (threadIdx.x < HMC_MAX_EP) seen[threadIdx.x] = -1;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int segments = ep * local_experts;
  const long long chunks = (rows + ROWS_PER_CHUNK - 1) / ROWS_PER_CHUNK;
  for (long long chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
    const long long r0 = chunk * ROWS_PER_CHUNK;
    const int count = static_cast<int>(min(static_cast<long long>(ROWS_PER_CHUNK), rows - r0));
    if (threadIdx.x < count) {
      const long long r = r0 + threadIdx.x;
      int lo = 0, hi = segments - 1;
      while (lo < hi) {  // last segment (local expert * ep + source) that starts at or before r
        const int mid = (lo + hi + 1) >> 1;
        if (segment_start[mid] <= r) lo = mid; else hi = mid - 1;
      }
      const int le = lo / ep;
      const int s = lo % ep;
      const long long src = source_row_off[s * local_experts + le] + (r - segment_start[lo]);
      if (src < 0 || src >= source_rows_limit) {
        report_status(status, HMC_STATUS_BAD_INDEX, static_cast<int>(r), lo, static_cast<int>(src));
        chunk_source[threadIdx.x] = -1;
      } else {
        chunk_source[threadIdx.x] = s;
      }
      chunk_row[threadIdx.x] = src;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int r = 0; r < count; ++r) {
        const int s = chunk_source[r];
        if (s < 0 || seen[s] >= generation) continue;
        int observed = 0;
        if (!wait_counter_ge(local_ctrl + HMC_CTRL_SOURCE + s * HMC_CTRL_READY_STRIDE, generation, budget_ns,
                             &observed)) {
          report_status(status, HMC_STATUS_TIMEOUT_READY, s, generation, observed);
          failed = 1;
          break;
        }
        seen[s] = observed;
      }
    }
    __syncthreads();
    if (failed) return;
    for (int r = warp; r < count; r += THREADS / 32) {
      const int s = chunk_source[r];
      if (s < 0) continue;
      const uint4* src = static_cast<const uint4*>(sources.data[s]) + chunk_row[r] * vec_per_row;
      uint4* dst = out + (r0 + r) * vec_per_row;
      for (int v = lane; v < vec_per_row; v += 32) st_16(dst + v, ld_16(src + v));
      if (out_values != nullptr && lane == 0) {
        const float* plane = reinterpret_cast<const float*>(static_cast<const unsigned char*>(sources.data[s]) +
                                                           value_plane_offset);
        out_values[r0 + r] = plane[chunk_row[r]];
      }
    }
    __syncthreads();
  }
}

__global__ void ep_wait_kernel(const int* counter, int expected, unsigned long long budget_ns, int* status,
                               const int* skip_flag) {
  if (skip_flag != nullptr && *reinterpret_cast<const volatile int*>(skip_flag) != 0) return;
  int seen = 0;
  if (!wait_counter_ge(counter, expected, budget_ns, &seen))
    report_status(status, HMC_STATUS_TIMEOUT_ARRIVAL, -1, expected, seen);
}

// One thread per group: bounded wait until the group's arrival counter covers its rows.
__global__ void ep_wait_groups_kernel(const int* counters, const long long* group_ends, int groups,
                                      unsigned long long budget_ns, int* status, const int* skip_flag) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= groups) return;
  if (skip_flag != nullptr && *skip_flag != 0) return;  // the call was not admitted: nothing is on its way
  const long long prev = g == 0 ? 0 : group_ends[g - 1];
  const int need = static_cast<int>(group_ends[g] - prev);
  int seen = 0;
  if (!wait_counter_ge(counters + g, need, budget_ns, &seen))
    report_status(status, HMC_STATUS_TIMEOUT_ARRIVAL, g, need, seen);
}

int fill_peers(PeerTable* table, void* const* data, void* const* ctrl, int64_t ep) {
  HMC_REQUIRE(ep >= 1 && ep <= HMC_MAX_EP, HMC_ERR_LIMIT, "expert-parallel size must be in [1, %d], got %lld",
              HMC_MAX_EP, (long long)ep);
  HMC_REQUIRE(data != nullptr && ctrl != nullptr, HMC_ERR_INVALID, "null peer table");
  memset(table, 0, sizeof(*table));
  for (int p = 0; p < ep; ++p) {
    HMC_REQUIRE(data[p] != nullptr && ctrl[p] != nullptr, HMC_ERR_INVALID, "peer %d has a null mapping", p);
    table->data[p] = data[p];
    table->ctrl[p] = static_cast<int*>(ctrl[p]);
  }
  return 0;
}

}  // namespace

// Checks an hmc_ep_dispatch_args and turns it into the device-side description used by the dispatch
// warps of the grouped GEMM (declared in grouped_gemm.cu).
int fill_dispatch(DispatchFuse* out, const hmc_ep_dispatch_args& a, const char* who) {
  PeerTable table;
  int rc = fill_peers(&table, a.peer_buffers, a.peer_ctrl, a.ep);
  if (rc != 0) return rc;
  HMC_REQUIRE(a.tokens && a.expert_of_row && a.dispatch_src_off && a.dispatch_target_off && a.local_ctrl,
              HMC_ERR_INVALID, "%s: null tensor pointer in the dispatch description", who);
  HMC_REQUIRE(a.hidden > 0 && a.hidden % 8 == 0 && aligned16(a.tokens), HMC_ERR_INVALID,
              "%s: dispatched rows must be 16-byte aligned multiples of 8 BF16 elements", who);
  HMC_REQUIRE(a.local_experts > 0 && a.local_experts <= HMC_CTRL_MAX_LOCAL_EXPERTS, HMC_ERR_LIMIT,
              "%s: local experts must be in [1, %d]", who, HMC_CTRL_MAX_LOCAL_EXPERTS);
  HMC_REQUIRE(a.rows >= 0 && a.rows < (1ll << 31) && a.top_k > 0, HMC_ERR_INVALID, "%s: bad dispatch extents", who);
  HMC_REQUIRE(a.rank >= 0 && a.rank < a.ep, HMC_ERR_INVALID, "%s: dispatch rank %lld outside [0, %lld)", who,
              (long long)a.rank, (long long)a.ep);
  HMC_REQUIRE(a.row_values == nullptr || (a.value_plane_offset >= a.capacity_rows * a.hidden * 2 &&
                                          a.value_plane_offset % 4 == 0),
              HMC_ERR_INVALID, "%s: the value plane must lie behind the rows of the receive buffer", who);
  for (int p = 0; p < a.ep; ++p) {
    HMC_REQUIRE(aligned16(a.peer_buffers[p]), HMC_ERR_INVALID, "%s: receive buffer %d is not 16-byte aligned", who, p);
    out->peer_data[p] = table.data[p];
    out->peer_ctrl[p] = table.ctrl[p];
  }
  out->tokens = static_cast<const uint4*>(a.tokens);
  out->source_of_row = a.source_of_row;
  out->expert_of_row = a.expert_of_row;
  out->dispatch_src_off = reinterpret_cast<const long long*>(a.dispatch_src_off);
  out->dispatch_target_off = reinterpret_cast<const long long*>(a.dispatch_target_off);
  out->send_order_start = reinterpret_cast<const long long*>(a.send_order_start);
  out->rows = a.rows;
  out->capacity_rows = a.capacity_rows;
  out->local_ctrl = a.local_ctrl;
  out->row_values = a.row_values;
  out->value_index = a.value_index;
  out->value_plane_offset = a.value_plane_offset;
  out->budget_ns = a.budget_ns ? a.budget_ns : 10ull * 1000 * 1000 * 1000;
  out->top_k = static_cast<int>(a.top_k);
  out->vec_per_row = static_cast<int>(a.hidden / 8);
  out->ep = static_cast<int>(a.ep);
  out->rank = static_cast<int>(a.rank);
  out->local_experts = static_cast<int>(a.local_experts);
  out->generation = a.generation;
  return 0;
}


}  // namespace hmc

using namespace hmc;

extern "C" int hmc_symm_alloc(int64_t bytes, void** out) {
  HMC_REQUIRE(out != nullptr && bytes > 0, HMC_ERR_INVALID, "hmc_symm_alloc: bad arguments");
  HMC_CUDA_OK(cudaMalloc(out, static_cast<size_t>(bytes)));
  HMC_CUDA_OK(cudaMemset(*out, 0, static_cast<size_t>(bytes)));
  return 0;
}

extern "C" int hmc_symm_free(void* ptr) {
  if (ptr != nullptr) HMC_CUDA_OK(cudaFree(ptr));
  return 0;
}

extern "C" int hmc_ipc_get_handle(void* ptr, void* handle_out_64_bytes) {
  HMC_REQUIRE(ptr != nullptr && handle_out_64_bytes != nullptr, HMC_ERR_INVALID, "hmc_ipc_get_handle: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == HMC_IPC_HANDLE_BYTES, "IPC handle size");
  cudaIpcMemHandle_t handle;
  HMC_CUDA_OK(cudaIpcGetMemHandle(&handle, ptr));
  memcpy(handle_out_64_bytes, &handle, sizeof(handle));
  return 0;
}

extern "C" int hmc_ipc_open_handle(const void* handle_64_bytes, void** out) {
  HMC_REQUIRE(handle_64_bytes != nullptr && out != nullptr, HMC_ERR_INVALID, "hmc_ipc_open_handle: null pointer");
  cudaIpcMemHandle_t handle;
  memcpy(&handle, handle_64_bytes, sizeof(handle));
  HMC_CUDA_OK(cudaIpcOpenMemHandle(out, handle, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}

extern "C" int hmc_ipc_close_handle(void* ptr) {
  if (ptr != nullptr) HMC_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return 0;
}

extern "C" int hmc_ep_publish_ready(void* const* peer_ctrl, int64_t ep, int64_t rank, int32_t generation,
                                    void* stream_ptr) {
  PeerTable table;
  int rc = fill_peers(&table, peer_ctrl, peer_ctrl, ep);
  if (rc != 0) return rc;
  HMC_REQUIRE(rank >= 0 && rank < ep, HMC_ERR_INVALID, "hmc_ep_publish_ready: rank out of range");
  ep_publish_ready_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_ptr)>>>(table, static_cast<int>(ep),
                                                                              static_cast<int>(rank), generation);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int64_t hmc_ep_exchange_table_bytes(int64_t ep, int64_t experts) {
  return 2 * ep * (experts + 4) * static_cast<int64_t>(sizeof(int));
}

extern "C" int hmc_ep_exchange_counts(const hmc_ep_exchange_args* args, void* stream_ptr) {
  HMC_REQUIRE(args != nullptr, HMC_ERR_INVALID, "hmc_ep_exchange_counts: null args");
  const hmc_ep_exchange_args& a = *args;
  ProfileScope profile(HMC_PROFILE_EP, static_cast<cudaStream_t>(stream_ptr));
  PeerTable table;
  int rc = fill_peers(&table, a.peer_tables, a.peer_ctrl, a.ep);
  if (rc != 0) return rc;
  HMC_REQUIRE(a.counts && a.local_ctrl, HMC_ERR_INVALID, "hmc_ep_exchange_counts: null tensor pointer");
  HMC_REQUIRE(a.rank >= 0 && a.rank < a.ep && a.experts > 0 && a.experts <= 4096, HMC_ERR_INVALID,
              "hmc_ep_exchange_counts: bad rank or expert count");
  HMC_REQUIRE(a.exchange > 0, HMC_ERR_INVALID, "hmc_ep_exchange_counts: exchanges are numbered from 1");
  ep_exchange_counts_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      a.counts, a.header[0], a.header[1], a.header[2], a.header[3], table, a.local_ctrl, static_cast<int>(a.ep),
      static_cast<int>(a.rank), static_cast<int>(a.experts), a.exchange,
      a.budget_ns ? a.budget_ns : 10ull * 1000 * 1000 * 1000, a.status);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_ep_publish_source(void* const* peer_ctrl, int64_t ep, int64_t rank, int32_t generation,
                                     void* stream_ptr) {
  PeerTable table;
  int rc = fill_peers(&table, peer_ctrl, peer_ctrl, ep);
  if (rc != 0) return rc;
  HMC_REQUIRE(rank >= 0 && rank < ep, HMC_ERR_INVALID, "hmc_ep_publish_source: rank out of range");
  ep_publish_source_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_ptr)>>>(table, static_cast<int>(ep),
                                                                               static_cast<int>(rank), generation);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_ep_pull(const hmc_ep_pull_args* args, void* stream_ptr) {
  HMC_REQUIRE(args != nullptr, HMC_ERR_INVALID, "hmc_ep_pull: null args");
  const hmc_ep_pull_args& a = *args;
  ProfileScope profile(HMC_PROFILE_EP, static_cast<cudaStream_t>(stream_ptr));
  if (a.rows == 0) return 0;
  PeerTable table;
  int rc = fill_peers(&table, a.peer_sources, a.peer_sources, a.ep);
  if (rc != 0) return rc;
  HMC_REQUIRE(a.source_row_off && a.segment_start && a.out && a.local_ctrl, HMC_ERR_INVALID,
              "hmc_ep_pull: null tensor pointer");
  HMC_REQUIRE(a.hidden > 0 && a.hidden % 8 == 0 && aligned16(a.out), HMC_ERR_INVALID,
              "hmc_ep_pull: rows must be 16-byte aligned multiples of 8 BF16 elements");
  HMC_REQUIRE(a.local_experts > 0 && a.rows > 0 && a.rows < (1ll << 31) && a.source_rows_limit > 0, HMC_ERR_INVALID,
              "hmc_ep_pull: bad extents");
  HMC_REQUIRE(a.out_values == nullptr || (a.value_plane_offset >= a.source_rows_limit * a.hidden * 2 &&
                                          a.value_plane_offset % 4 == 0),
              HMC_ERR_INVALID, "hmc_ep_pull: the value plane must lie behind the rows of the source buffer");
  for (int p = 0; p < a.ep; ++p)
    HMC_REQUIRE(aligned16(a.peer_sources[p]), HMC_ERR_INVALID, "hmc_ep_pull: source buffer %d is not 16-byte aligned", p);
  const long long chunks = (a.rows + ROWS_PER_CHUNK - 1) / ROWS_PER_CHUNK;
  int grid = 4 * sm_count();
  if (a.max_ctas > 0 && grid > a.max_ctas) grid = a.max_ctas;
  if (chunks < grid) grid = static_cast<int>(chunks);
  ep_pull_kernel<<<grid, THREADS, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      table, reinterpret_cast<const long long*>(a.source_row_off), reinterpret_cast<const long long*>(a.segment_start),
      static_cast<uint4*>(a.out), a.out_values, a.rows, static_cast<int>(a.hidden / 8), static_cast<int>(a.ep),
      static_cast<int>(a.local_experts), a.source_rows_limit, a.value_plane_offset, a.local_ctrl, a.generation,
      a.budget_ns ? a.budget_ns : 10ull * 1000 * 1000 * 1000, a.status);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_ep_dispatch(const hmc_ep_dispatch_args* args, void* stream_ptr) {
  HMC_REQUIRE(args != nullptr, HMC_ERR_INVALID, "hmc_ep_dispatch: null args");
  const hmc_ep_dispatch_args& a = *args;
  ProfileScope profile(HMC_PROFILE_EP, static_cast<cudaStream_t>(stream_ptr));
  if (a.rows == 0) return 0;
  PeerTable table;
  int rc = fill_peers(&table, a.peer_buffers, a.peer_ctrl, a.ep);
  if (rc != 0) return rc;
  HMC_REQUIRE(a.tokens && a.expert_of_row && a.dispatch_src_off && a.dispatch_target_off && a.local_ctrl,
              HMC_ERR_INVALID, "hmc_ep_dispatch: null tensor pointer");
  HMC_REQUIRE(a.hidden > 0 && a.hidden % 8 == 0 && aligned16(a.tokens), HMC_ERR_INVALID,
              "hmc_ep_dispatch: rows must be 16-byte aligned multiples of 8 BF16 elements");
  HMC_REQUIRE(a.local_experts > 0 && a.local_experts <= HMC_CTRL_MAX_LOCAL_EXPERTS, HMC_ERR_LIMIT,
              "hmc_ep_dispatch: local experts must be in [1, %d]", HMC_CTRL_MAX_LOCAL_EXPERTS);
  HMC_REQUIRE(a.rows > 0 && a.rows < (1ll << 31) && a.top_k > 0, HMC_ERR_INVALID, "hmc_ep_dispatch: bad extents");
  HMC_REQUIRE(a.rank >= 0 && a.rank < a.ep, HMC_ERR_INVALID, "hmc_ep_dispatch: rank %lld outside [0, %lld)", (long long)a.rank,
              (long long)a.ep);
  HMC_REQUIRE(a.row_values == nullptr || (a.value_plane_offset >= a.capacity_rows * a.hidden * 2 &&
                                          a.value_plane_offset % 4 == 0),
              HMC_ERR_INVALID, "hmc_ep_dispatch: the value plane must lie behind the rows of the receive buffer");
  const long long chunks = (a.rows + ROWS_PER_CHUNK - 1) / ROWS_PER_CHUNK;
  int grid = 4 * sm_count();
  if (a.max_ctas > 0 && grid > a.max_ctas) grid = a.max_ctas;
  if (chunks < grid) grid = static_cast<int>(chunks);
  ep_dispatch_kernel<<<grid, THREADS, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const uint4*>(a.tokens), a.source_of_row, a.expert_of_row,
      reinterpret_cast<const long long*>(a.dispatch_src_off), reinterpret_cast<const long long*>(a.dispatch_target_off),
      a.rows, static_cast<int>(a.top_k), static_cast<int>(a.hidden / 8), static_cast<int>(a.ep),
      static_cast<int>(a.local_experts), a.capacity_rows, table, a.local_ctrl, a.generation,
      a.budget_ns ? a.budget_ns : 10ull * 1000 * 1000 * 1000, a.status, a.row_values, a.value_index,
      a.value_plane_offset, a.skip_flag, static_cast<int>(a.rank));
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_ep_combine(const hmc_ep_combine_args* args, void* stream_ptr) {
  HMC_REQUIRE(args != nullptr, HMC_ERR_INVALID, "hmc_ep_combine: null args");
  const hmc_ep_combine_args& a = *args;
  ProfileScope profile(HMC_PROFILE_EP, static_cast<cudaStream_t>(stream_ptr));
  if (a.rows == 0) return 0;
  PeerTable table;
  int rc = fill_peers(&table, a.peer_buffers, a.peer_ctrl, a.ep);
  if (rc != 0) return rc;
  HMC_REQUIRE(a.results && a.segment_start && a.combine_target_off && a.local_ctrl, HMC_ERR_INVALID,
              "hmc_ep_combine: null tensor pointer");
  HMC_REQUIRE(a.hidden > 0 && a.hidden % 8 == 0 && aligned16(a.results), HMC_ERR_INVALID,
              "hmc_ep_combine: rows must be 16-byte aligned multiples of 8 BF16 elements");
  HMC_REQUIRE(a.local_experts > 0 && a.rows > 0 && a.rows < (1ll << 31), HMC_ERR_INVALID,
              "hmc_ep_combine: bad extents");
  HMC_REQUIRE(a.result_values == nullptr || (a.value_plane_offset >= a.target_rows_limit * a.hidden * 2 &&
                                             a.value_plane_offset % 4 == 0),
              HMC_ERR_INVALID, "hmc_ep_combine: the value plane must lie behind the rows of the routed buffer");
  const long long chunks = (a.rows + ROWS_PER_CHUNK - 1) / ROWS_PER_CHUNK;
  int grid = 4 * sm_count();
  if (a.max_ctas > 0 && grid > a.max_ctas) grid = a.max_ctas;
  if (chunks < grid) grid = static_cast<int>(chunks);
  ep_combine_kernel<<<grid, THREADS, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const uint4*>(a.results), reinterpret_cast<const long long*>(a.segment_start),
      reinterpret_cast<const long long*>(a.combine_target_off), a.rows, static_cast<int>(a.hidden / 8),
      static_cast<int>(a.ep), static_cast<int>(a.local_experts), a.target_rows_limit, table, a.local_ctrl,
      a.generation, a.budget_ns ? a.budget_ns : 10ull * 1000 * 1000 * 1000, a.status, a.result_values,
      a.value_plane_offset);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_ep_wait_unless(const int32_t* counter, int32_t expected, uint64_t budget_ns, int32_t* status,
                                  const int32_t* skip_flag, void* stream_ptr) {
  HMC_REQUIRE(counter != nullptr, HMC_ERR_INVALID, "hmc_ep_wait: null counter");
  ProfileScope profile(HMC_PROFILE_EP, static_cast<cudaStream_t>(stream_ptr));
  ep_wait_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      counter, expected, budget_ns ? budget_ns : 10ull * 1000 * 1000 * 1000, status, skip_flag);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_ep_wait(const int32_t* counter, int32_t expected, uint64_t budget_ns, int32_t* status,
                           void* stream_ptr) {
  return hmc_ep_wait_unless(counter, expected, budget_ns, status, nullptr, stream_ptr);
}

namespace hmc {
namespace {
// One CTA. Threads r < ep add up what rank r receives and what it routes; any excess, or any rank's
// "invalid" header word, sets the flag. Then the table, the status words and the flag go to the host mirror.
__global__ void __launch_bounds__(256)
route_guard_kernel(const int* __restrict__ table, int ep, int experts, long long capacity_rows, long long routed_limit,
                   const int* __restrict__ status_words, int* __restrict__ skip_flag, int* __restrict__ host_mirror) {
  __shared__ int flag;
  if (threadIdx.x == 0) flag = 0;
  __syncthreads();
  const int local = experts / ep;
  const int* header = table + static_cast<long long>(ep) * experts;
  for (int r = threadIdx.x; r < ep; r += blockDim.x) {
    long long received = 0, routed = 0;
    for (int s = 0; s < ep; ++s)
      for (int le = 0; le < local; ++le) received += table[static_cast<long long>(s) * experts + r * local + le];
    for (int e = 0; e < experts; ++e) routed += table[static_cast<long long>(r) * experts + e];
    if (received > capacity_rows || routed > routed_limit || header[r * 4] != 0) atomicOr(&flag, 1);
  }
  __syncthreads();
  const int value = flag;
  if (threadIdx.x == 0) *skip_flag = value;
  if (host_mirror != nullptr) {
    const int table_words = ep * (experts + 4);
    for (int i = threadIdx.x; i < table_words; i += blockDim.x) host_mirror[i] = table[i];
    if (threadIdx.x < HMC_STATUS_WORDS)
      host_mirror[table_words + threadIdx.x] = status_words != nullptr ? status_words[threadIdx.x] : 0;
    if (threadIdx.x == 0) host_mirror[table_words + HMC_STATUS_WORDS] = value;
    __threadfence_system();
  }
}
}  // namespace
}  // namespace hmc

extern "C" int hmc_route_guard(const int32_t* table, int64_t ep, int64_t experts, int64_t capacity_rows,
                               int64_t routed_limit, const int32_t* status_words, int32_t* skip_flag,
                               int32_t* host_mirror, void* stream_ptr) {
  HMC_REQUIRE(table != nullptr && skip_flag != nullptr, HMC_ERR_INVALID, "hmc_route_guard: null tensor pointer");
  HMC_REQUIRE(ep >= 1 && ep <= HMC_MAX_EP && experts > 0 && experts % ep == 0 && experts <= 65536, HMC_ERR_INVALID,
              "hmc_route_guard: experts (%lld) must be a positive multiple of ep (%lld)", (long long)experts, (long long)ep);
  HMC_REQUIRE(capacity_rows >= 0 && routed_limit >= 0, HMC_ERR_INVALID, "hmc_route_guard: negative limits");
  ProfileScope profile(HMC_PROFILE_EP, static_cast<cudaStream_t>(stream_ptr));
  hmc::route_guard_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      table, static_cast<int>(ep), static_cast<int>(experts), capacity_rows, routed_limit, status_words, skip_flag,
      host_mirror);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_ep_wait_groups_unless(const int32_t* counters, const int64_t* group_ends, int64_t groups,
                                         uint64_t budget_ns, int32_t* status, const int32_t* skip_flag, void* stream_ptr) {
  HMC_REQUIRE(counters != nullptr && group_ends != nullptr && groups > 0 && groups <= HMC_CTRL_MAX_LOCAL_EXPERTS,
              HMC_ERR_INVALID, "hmc_ep_wait_groups: bad arguments");
  ProfileScope profile(HMC_PROFILE_EP, static_cast<cudaStream_t>(stream_ptr));
  ep_wait_groups_kernel<<<static_cast<unsigned>((groups + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      counters, reinterpret_cast<const long long*>(group_ends), static_cast<int>(groups),
      budget_ns ? budget_ns : 10ull * 1000 * 1000 * 1000, status, skip_flag);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_ep_wait_groups(const int32_t* counters, const int64_t* group_ends, int64_t groups,
                                  uint64_t budget_ns, int32_t* status, void* stream_ptr) {
  return hmc_ep_wait_groups_unless(counters, group_ends, groups, budget_ns, status, nullptr, stream_ptr);
}
