// MoE route preparation and token (un)permutation: integer work is bit-exact by construction
// (stable counting sort), payload work is 16-byte vectorised row copies.
//
// Replaces, on the reference side: histogram + expert-major permutation (hyper_multicore/modules/
// mega_moe/route.py:186-211, 266-295; torch/csrc/moe_token_permute_out.cpp:50-60), offset
// descriptors (route.py:309-390, ops/common/mega_moe/utilities.asc:89-151), PermuteFromMapping
// (utilities.asc:162-209), weighted un-permutation and its gradients (route.py:1029-1051,
// torch/csrc/mega_moe_unpermute.cpp:56-65, moe_token_permute_grad.cpp:29-38) and
// ZeroEmptyExpertGrad (utilities.asc:17-54).
#include <cooperative_groups.h>
#include <cuda_bf16.h>

#include "common.cuh"

namespace hmc {
namespace {

constexpr int SORT_CHUNK = 1024;  // flat (token, slot) entries ranked by one CTA
constexpr int SORT_THREADS = 1024;

__device__ __forceinline__ long long load_index(const void* indices, int is_i64, long long i) {
  return is_i64 ? static_cast<const long long*>(indices)[i]
                : static_cast<long long>(static_cast<const int*>(indices)[i]);
}

// ---- pass 1: per-chunk histogram ---------------------------------------------------------
__global__ void __launch_bounds__(SORT_THREADS)
chunk_histogram_kernel(const void* __restrict__ indices, int is_i64, long long entries, int experts,
                       int* __restrict__ chunk_counts, int* __restrict__ status) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const long long i = static_cast<long long>(blockIdx.x) * SORT_CHUNK + threadIdx.x;
  if (i < entries) {
    const long long e = load_index(indices, is_i64, i);
    if (e >= 0 && e < experts) {
      atomicAdd(&hist[e], 1);
    } else {
      report_status(status, HMC_STATUS_BAD_INDEX, static_cast<int>(i), static_cast<int>(e), experts);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x)
    chunk_counts[static_cast<long long>(blockIdx.x) * experts + e] = hist[e];
}

// ---- pass 2: one CTA turns chunk histograms into chunk bases and expert bases -------------
// chunk_counts[c][e] becomes the first destination row of chunk c's entries for expert e.
__global__ void __launch_bounds__(1024)
chunk_scan_kernel(int* __restrict__ chunk_counts, int chunks, int experts, int* __restrict__ counts_out,
                  long long* __restrict__ ends_out, int* __restrict__ expert_of_row,
                  int* __restrict__ source_of_row, long long entries, int stage_table) {
  extern __shared__ int totals[];  // [experts] (+ [chunks * experts] when the table is staged)
  __shared__ int placed;
  // Small tables are scanned in shared memory: the serial walk over the chunks then costs shared-memory
  // latencies instead of one global round trip per chunk.
  const long long cells = static_cast<long long>(chunks) * experts;
  int* staged = stage_table ? totals + experts : nullptr;
  if (staged != nullptr) {
    for (long long i = threadIdx.x; i < cells; i += blockDim.x) staged[i] = chunk_counts[i];
    __syncthreads();
  }
  int* table = staged != nullptr ? staged : chunk_counts;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    int run = 0;
    for (int c = 0; c < chunks; ++c) {
      int* slot = table + static_cast<long long>(c) * experts + e;
      const int v = *slot;
      *slot = run;
      run += v;
    }
    totals[e] = run;
    if (counts_out != nullptr) counts_out[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // experts <= 4096: a serial scan by one thread costs microseconds and is trivially exact
    int run = 0;
    for (int e = 0; e < experts; ++e) {
      const int v = totals[e];
      totals[e] = run;
      run += v;
      if (ends_out != nullptr) ends_out[e] = run;
    }
    placed = run;
  }
  __syncthreads();
  // Rejected expert ids leave the last rows without an owner: mark them so that no consumer
  // reads a stale expert or source there.
  for (long long r = placed + threadIdx.x; r < entries; r += blockDim.x) {
    if (expert_of_row != nullptr) expert_of_row[r] = -1;
    if (source_of_row != nullptr) source_of_row[r] = -1;
  }
  if (staged != nullptr) {
    for (long long i = threadIdx.x; i < cells; i += blockDim.x)
      chunk_counts[i] = staged[i] + totals[static_cast<int>(i % experts)];
  } else {
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
      const int base = totals[e];
      for (int c = 0; c < chunks; ++c) chunk_counts[static_cast<long long>(c) * experts + e] += base;
    }
  }
}

// ---- pass 3: stable rank inside each chunk --------------------------------------------------
// Warps take turns in flat-index order; inside a warp, match_any groups equal experts and the
// lower lanes rank first, so equal experts keep their flat (token * top_k + slot) order.
__global__ void __launch_bounds__(SORT_THREADS)
chunk_rank_kernel(const void* __restrict__ indices, int is_i64, long long entries, int experts,
                  const int* __restrict__ chunk_bases, int* __restrict__ mapping,
                  int* __restrict__ source_of_row, int* __restrict__ expert_of_row) {
  extern __shared__ int cursor[];  // [experts] next free destination row per expert
  for (int e = threadIdx.x; e < experts; e += blockDim.x)
    cursor[e] = chunk_bases[static_cast<long long>(blockIdx.x) * experts + e];
  __syncthreads();
  const long long i = static_cast<long long>(blockIdx.x) * SORT_CHUNK + threadIdx.x;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  long long e = -1;
  if (i < entries) {
    e = load_index(indices, is_i64, i);
    if (e < 0 || e >= experts) e = -1;
  }
  for (int w = 0; w < SORT_THREADS / 32; ++w) {
    if (w == warp) {
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      if (e >= 0) {
        const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
        const int leader = __ffs(peers) - 1;
        int base = 0;
        if (lane == leader) {
          base = cursor[e];
          cursor[e] = base + __popc(peers);
        }
        base = __shfl_sync(peers, base, leader);
        const int dest = base + rank_in_warp;
        mapping[i] = dest;
        if (source_of_row != nullptr) source_of_row[dest] = static_cast<int>(i);
        if (expert_of_row != nullptr) expert_of_row[dest] = static_cast<int>(e);
      } else if (i < entries) {
        mapping[i] = -1;
      }
    }
    __syncthreads();
  }
}

// ---- the three passes in one cooperative launch ----------------------------------------------
// For route counts whose chunks are all resident at once (one CTA per chunk): histogram, one grid-wide
// barrier, then every CTA derives its own destination bases from the table of all chunks (a column sum over
// the chunks before it plus an exclusive scan over the experts) and ranks its entries. Same stable order as
// the three-kernel path: chunks in flat order, warps in flat order inside a chunk, lanes inside a warp.
constexpr int RANK_PARALLEL_EXPERTS = 256;  // per-warp counters of the parallel ranking fit shared memory up to here

__device__ __forceinline__ int warp_inclusive_scan(int v, int lane) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int other = __shfl_up_sync(0xffffffffu, v, d);
    if (lane >= d) v += other;
  }
  return v;
}

__global__ void __launch_bounds__(SORT_THREADS)
sort_routes_fused_kernel(const void* __restrict__ indices, int is_i64, long long entries, int experts,
                         int* __restrict__ chunk_counts, int* __restrict__ mapping, int* __restrict__ source_of_row,
                         int* __restrict__ expert_of_row, int* __restrict__ counts_out, long long* __restrict__ ends_out,
                         int* __restrict__ status) {
  extern __shared__ int smem[];   // cursor [experts], then per-warp counters [32][experts] when experts <= 256
  int* cursor = smem;
  int* warp_counts = smem + experts;
  __shared__ int warp_sums[32];
  __shared__ int pass_total;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int chunk = blockIdx.x;
  const int chunks = gridDim.x;
  const bool parallel_rank = experts <= RANK_PARALLEL_EXPERTS;

  // ---- histogram of this chunk
  for (int e = threadIdx.x; e < experts; e += blockDim.x) cursor[e] = 0;
  __syncthreads();
  const long long i = static_cast<long long>(chunk) * SORT_CHUNK + threadIdx.x;
  long long e = -1;
  if (i < entries) {
    e = load_index(indices, is_i64, i);
    if (e >= 0 && e < experts) {
      atomicAdd(&cursor[e], 1);
    } else {
      report_status(status, HMC_STATUS_BAD_INDEX, static_cast<int>(i), static_cast<int>(e), experts);
      e = -1;
    }
  }
  __syncthreads();
  for (int x = threadIdx.x; x < experts; x += blockDim.x) chunk_counts[static_cast<long long>(chunk) * experts + x] = cursor[x];
  cooperative_groups::this_grid().sync();

  // ---- destination bases of this chunk: rows of earlier experts + rows of this expert in earlier chunks
  int carry = 0;
  for (int first = 0; first < experts; first += SORT_THREADS) {
    const int x = first + threadIdx.x;
    int below = 0, total = 0;
    if (x < experts) {
      for (int c = 0; c < chunks; ++c) {
        const int v = chunk_counts[static_cast<long long>(c) * experts + x];
        total += v;
        if (c < chunk) below += v;
      }
    }
    const int incl = warp_inclusive_scan(total, lane);
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const int sum = warp_sums[lane];
      const int scanned = warp_inclusive_scan(sum, lane);
      warp_sums[lane] = scanned - sum;
      if (lane == 31) pass_total = scanned;
    }
    __syncthreads();
    if (x < experts) {
      const int expert_base = carry + warp_sums[warp] + incl - total;
      cursor[x] = expert_base + below;
      if (chunk == 0) {
        if (counts_out != nullptr) counts_out[x] = total;
        if (ends_out != nullptr) ends_out[x] = expert_base + total;
      }
    }
    carry += pass_total;
    __syncthreads();
  }
  // Rejected expert ids leave the last rows without an owner: mark them so that no consumer reads a stale
  // expert or source there (`carry` is the number of rows that were placed).
  for (long long r = carry + i; r < entries; r += static_cast<long long>(chunks) * SORT_CHUNK) {
    if (expert_of_row != nullptr) expert_of_row[r] = -1;
    if (source_of_row != nullptr) source_of_row[r] = -1;
  }

  // ---- stable rank inside the chunk
  if (parallel_rank) {
    for (int x = threadIdx.x; x < 32 * experts; x += blockDim.x) warp_counts[x] = 0;
    __syncthreads();
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int leader = __ffs(peers) - 1;
    if (e >= 0 && lane == leader) warp_counts[warp * experts + e] = __popc(peers);
    __syncthreads();
    for (int x = threadIdx.x; x < experts; x += blockDim.x) {
      int run = cursor[x];
      for (int w = 0; w < SORT_THREADS / 32; ++w) {
        const int v = warp_counts[w * experts + x];
        warp_counts[w * experts + x] = run;
        run += v;
      }
    }
    __syncthreads();
    if (e >= 0) {
      const int dest = warp_counts[warp * experts + e] + __popc(peers & ((1u << lane) - 1u));
      mapping[i] = dest;
      if (source_of_row != nullptr) source_of_row[dest] = static_cast<int>(i);
      if (expert_of_row != nullptr) expert_of_row[dest] = static_cast<int>(e);
    } else if (i < entries) {
      mapping[i] = -1;
    }
    return;
  }
  for (int w = 0; w < SORT_THREADS / 32; ++w) {
    if (w == warp) {
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      if (e >= 0) {
        const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
        const int leader = __ffs(peers) - 1;
        int base = 0;
        if (lane == leader) {
          base = cursor[e];
          cursor[e] = base + __popc(peers);
        }
        base = __shfl_sync(peers, base, leader);
        const int dest = base + rank_in_warp;
        mapping[i] = dest;
        if (source_of_row != nullptr) source_of_row[dest] = static_cast<int>(i);
        if (expert_of_row != nullptr) expert_of_row[dest] = static_cast<int>(e);
      } else if (i < entries) {
        mapping[i] = -1;
      }
    }
    __syncthreads();
  }
}

// ---- payload movement ----------------------------------------------------------------------
// One warp per destination row: out[row] = tokens[source_of_row[row] / top_k].
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ tokens, const int* __restrict__ source_of_row, long long rows,
                   int top_k, int vec_per_row, uint4* __restrict__ out) {
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int flat = source_of_row[row];
  uint4* d = out + row * vec_per_row;
  if (flat < 0) {  // a row without an owner (its route named no valid expert): defined contents, no read
    for (int v = lane; v < vec_per_row; v += 32) st_cs_16(d + v, make_uint4(0, 0, 0, 0));
    return;
  }
  const uint4* s = tokens + static_cast<long long>(flat / top_k) * vec_per_row;
  for (int v = lane; v < vec_per_row; v += 32) st_cs_16(d + v, ld_16(s + v));
}

// One warp per flat entry i: out[mapping[i]] = tokens[i / top_k], out_p[mapping[i]] = p[i].
__global__ void __launch_bounds__(256)
scatter_rows_kernel(const uint4* __restrict__ tokens, const int* __restrict__ mapping,
                    const float* __restrict__ probs, long long entries, int top_k, int vec_per_row,
                    uint4* __restrict__ out, float* __restrict__ out_probs, int* __restrict__ status) {
  const long long i = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (i >= entries) return;
  const int lane = threadIdx.x & 31;
  const int dest = mapping[i];
  if (dest < 0 || dest >= entries) {
    if (lane == 0) report_status(status, HMC_STATUS_BAD_INDEX, static_cast<int>(i), dest, 0);
    return;
  }
  const uint4* s = tokens + (i / top_k) * vec_per_row;
  uint4* d = out + static_cast<long long>(dest) * vec_per_row;
  for (int v = lane; v < vec_per_row; v += 32) st_cs_16(d + v, ld_16(s + v));
  if (lane == 0 && out_probs != nullptr) out_probs[dest] = probs[i];
}

// out[t] = sum over the token's routes, in ascending expert (= ascending row) order, of
// bf16(float(y[row]) * p), accumulated in BF16 like the golden's index_add
// (tests/common/multicore/moe_reference.py:179-180). One CTA of 128 threads per token.
constexpr int MAX_TOP_K = 64;
__global__ void __launch_bounds__(128)
unpermute_kernel(const uint4* __restrict__ y, const int* __restrict__ mapping, const float* __restrict__ probs,
                 long long tokens, int top_k, int vec_per_row, long long y_rows, uint4* __restrict__ out,
                 int* __restrict__ status, const int* __restrict__ skip_flag) {
  __shared__ int rows[MAX_TOP_K];
  __shared__ float weight[MAX_TOP_K];
  if (skip_flag != nullptr && *reinterpret_cast<const volatile int*>(skip_flag) != 0) return;  // uniform per launch
  const long long t = blockIdx.x;
  __shared__ int raw_rows[MAX_TOP_K];
  __shared__ float raw_weight[MAX_TOP_K];
  if (threadIdx.x < top_k) {  // one memory latency for all routes of the token
    raw_rows[threadIdx.x] = mapping[t * top_k + threadIdx.x];
    raw_weight[threadIdx.x] = probs != nullptr ? probs[t * top_k + threadIdx.x] : 1.0f;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // insertion sort of the (row, weight) pairs by row; top_k is small
    for (int k = 0; k < top_k; ++k) {
      int r = raw_rows[k];
      float w = raw_weight[k];
      if (r < 0 || r >= y_rows) {
        report_status(status, HMC_STATUS_BAD_INDEX, static_cast<int>(t), k, r);
        r = -1;
      }
      int j = k;
      while (j > 0 && rows[j - 1] > r) {
        rows[j] = rows[j - 1];
        weight[j] = weight[j - 1];
        --j;
      }
      rows[j] = r;
      weight[j] = w;
    }
  }
  __syncthreads();
  for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
    // Running sums as packed BF16 pairs: a BF16 add rounds the exact sum once, which is what
    // bf16(float(a) + float(b)) does, and the weighted term is the FP32 product rounded once.
    __nv_bfloat162 acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = __floats2bfloat162_rn(0.f, 0.f);
    for (int k0 = 0; k0 < top_k; k0 += 4) {
      // four rows in flight: the loads do not depend on the running sum
      uint4 q[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = k0 + i < top_k ? rows[k0 + i] : -1;
        q[i] = r >= 0 ? ld_nc_16(y + static_cast<long long>(r) * vec_per_row + v) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (k0 + i >= top_k || rows[k0 + i] < 0) continue;
        const float w = weight[k0 + i];
        const uint32_t words[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(words[j]);
          acc[j] = __hadd2(acc[j], __floats2bfloat162_rn(f.x * w, f.y * w));
        }
      }
    }
    uint4 o;
    o.x = *reinterpret_cast<const uint32_t*>(&acc[0]);
    o.y = *reinterpret_cast<const uint32_t*>(&acc[1]);
    o.z = *reinterpret_cast<const uint32_t*>(&acc[2]);
    o.w = *reinterpret_cast<const uint32_t*>(&acc[3]);
    st_cs_16(out + t * vec_per_row + v, o);
  }
}

// Backward of the weighted un-permutation. One CTA per token:
//   grad_permuted[row(t,k)] = bf16(float(dOut[t]) * p[t,k])
//   grad_probs[t,k]         = sum_h float(dOut[t,h]) * float(y[row(t,k), h])
__global__ void __launch_bounds__(128)
unpermute_grad_kernel(const uint4* __restrict__ y, const uint4* __restrict__ grad_out,
                      const int* __restrict__ mapping, const float* __restrict__ probs, long long tokens,
                      int top_k, int vec_per_row, long long permuted_rows, uint4* __restrict__ grad_permuted,
                      float* __restrict__ grad_probs, int* __restrict__ status) {
  __shared__ float partial[4][4];
  const long long t = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  // Four routes of the token at a time: dOut[t] is read once for the four, their forward rows are in flight
  // together, and one block reduction serves four dot products.
  for (int k0 = 0; k0 < top_k; k0 += 4) {
    int r[4];
    float w[4];
    float dot[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      r[i] = -1;
      w[i] = 0.f;
      if (k0 + i < top_k) {
        r[i] = mapping[t * top_k + k0 + i];
        w[i] = probs[t * top_k + k0 + i];
        if (r[i] < 0 || r[i] >= permuted_rows) {
          if (threadIdx.x == 0) report_status(status, HMC_STATUS_BAD_INDEX, static_cast<int>(t), k0 + i, r[i]);
          r[i] = -1;
        }
      }
    }
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
      const uint4 g = ld_16(grad_out + t * vec_per_row + v);
      const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
      uint4 q[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        q[i] = (y != nullptr && r[i] >= 0) ? ld_nc_16(y + static_cast<long long>(r[i]) * vec_per_row + v) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (r[i] < 0) continue;
        const uint32_t yw[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
        uint32_t ow[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 gf = unpack_bf16x2(gw[j]);
          ow[j] = pack_bf16x2(gf.x * w[i], gf.y * w[i]);
          if (y != nullptr) {
            const float2 yf = unpack_bf16x2(yw[j]);
            dot[i] += gf.x * yf.x + gf.y * yf.y;
          }
        }
        st_cs_16(grad_permuted + static_cast<long long>(r[i]) * vec_per_row + v, make_uint4(ow[0], ow[1], ow[2], ow[3]));
      }
    }
    if (grad_probs != nullptr) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float sum = warp_sum(dot[i]);
        if (lane == 0) partial[warp][i] = sum;
      }
      __syncthreads();
      if (threadIdx.x < 4 && k0 + threadIdx.x < top_k)
        grad_probs[t * top_k + k0 + threadIdx.x] =
            partial[0][threadIdx.x] + partial[1][threadIdx.x] + partial[2][threadIdx.x] + partial[3][threadIdx.x];
      __syncthreads();
    }
  }
}

// dX[t] = sum over the token's routes of dXe[row(t,k)], added the way the golden's autograd adds them:
// every expert's index_select hands the token one BF16 row, the engine accumulates those rows as the
// per-expert backward nodes run, last expert first, and every addition rounds to BF16
// (tests/common/multicore/moe_reference.py:170-181 under torch.autograd). Rows are expert-major, so
// "last expert first" is descending row order. One CTA of 128 threads per token.
__global__ void __launch_bounds__(128)
permute_grad_kernel(const uint4* __restrict__ grad_permuted, const int* __restrict__ mapping, long long tokens,
                    int top_k, int vec_per_row, long long rows, uint4* __restrict__ grad_tokens,
                    int* __restrict__ status) {
  __shared__ int order[MAX_TOP_K];
  const long long t = blockIdx.x;
  __shared__ int raw_rows[MAX_TOP_K];
  if (threadIdx.x < top_k) raw_rows[threadIdx.x] = mapping[t * top_k + threadIdx.x];  // one memory latency for all routes
  __syncthreads();
  if (threadIdx.x == 0) {
    // insertion sort by descending row; rejected entries (-1) sink to the end
    for (int k = 0; k < top_k; ++k) {
      int r = raw_rows[k];
      if (r < 0 || r >= rows) {
        report_status(status, HMC_STATUS_BAD_INDEX, static_cast<int>(t), k, r);
        r = -1;
      }
      int j = k;
      while (j > 0 && order[j - 1] < r) {
        order[j] = order[j - 1];
        --j;
      }
      order[j] = r;
    }
  }
  __syncthreads();
  for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
    __nv_bfloat162 acc[4];  // packed BF16 running sums: one rounding of the exact sum per addition
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = __floats2bfloat162_rn(0.f, 0.f);
    for (int k0 = 0; k0 < top_k; k0 += 4) {
      uint4 q[4];  // four rows in flight: the loads do not depend on the running sum
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = k0 + i < top_k ? order[k0 + i] : -1;
        q[i] = r >= 0 ? ld_nc_16(grad_permuted + static_cast<long long>(r) * vec_per_row + v) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (k0 + i >= top_k || order[k0 + i] < 0) continue;
        const uint32_t words[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j)  // the first row passes unchanged: 0 + x is exact
          acc[j] = __hadd2(acc[j], *reinterpret_cast<const __nv_bfloat162*>(&words[j]));
      }
    }
    uint4 o;
    o.x = *reinterpret_cast<const uint32_t*>(&acc[0]);
    o.y = *reinterpret_cast<const uint32_t*>(&acc[1]);
    o.z = *reinterpret_cast<const uint32_t*>(&acc[2]);
    o.w = *reinterpret_cast<const uint32_t*>(&acc[3]);
    st_cs_16(grad_tokens + t * vec_per_row + v, o);
  }
}

// Zero the gradient slices of experts whose cumulative row count did not advance.
__global__ void __launch_bounds__(256)
zero_empty_kernel(uint4* __restrict__ first, long long first_vec_per_expert, uint4* __restrict__ second,
                  long long second_vec_per_expert, const long long* __restrict__ cumulative, int experts) {
  const int e = blockIdx.y;
  const long long prev = e == 0 ? 0 : cumulative[e - 1];
  if (cumulative[e] != prev) return;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < first_vec_per_expert; v += stride)
    first[e * first_vec_per_expert + v] = zero;
  if (second != nullptr)
    for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < second_vec_per_expert; v += stride)
      second[e * second_vec_per_expert + v] = zero;
}

// Offset descriptors for push dispatch from the gathered count table counts[ep][experts]. Row units.
// One CTA; every running sum below is a warp scan over 32 table entries at a time: warp 0 lays out this
// rank's send order, warps 1 .. ep the sources' expert-major buffers, warps ep+1 .. 2*ep the destinations'
// receive buffers (the warps take these jobs round-robin when the CTA has fewer).
__device__ __forceinline__ long long warp_inclusive_scan_ll(long long v, int lane) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const long long other = __shfl_up_sync(0xffffffffu, v, d);
    if (lane >= d) v += other;
  }
  return v;
}

__global__ void __launch_bounds__(1024)
route_offsets_kernel(const int* __restrict__ counts, int ep, int experts, int rank,
                     long long* __restrict__ dispatch_src_off, long long* __restrict__ dispatch_target_off,
                     int* __restrict__ dispatch_size, long long* __restrict__ combine_src_off,
                     long long* __restrict__ combine_target_off, int* __restrict__ combine_size,
                     long long* __restrict__ group_list, long long* __restrict__ totals,
                     long long* __restrict__ recv_segment_start, long long* __restrict__ send_order_start,
                     int stage_table) {
  // Tables of up to 48 KiB are staged in shared memory: one global round trip for the whole table.
  extern __shared__ int staged[];
  const int* table = counts;
  if (stage_table) {
    for (int i = threadIdx.x; i < ep * experts; i += blockDim.x) staged[i] = counts[i];
    __syncthreads();
    table = staged;
  }
  const int local = experts / ep;
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  for (int job = threadIdx.x >> 5; job < 1 + 2 * ep; job += warps) {
    long long run = 0;
    if (job == 0) {
      if (send_order_start == nullptr) continue;
      // Order in which this rank sends its rows when the dispatch rides inside the consuming GEMM: local
      // expert 0 of every destination first (destinations rank + 1, rank + 2, ..., this rank last), then
      // local expert 1, ... so that on every owner expert 0 completes after 1 / local of the transfer and
      // its tiles run while the later experts' rows still travel. Entry q = le * ep + dd holds the first
      // position of segment (destination (rank + 1 + dd) % ep, local expert le) in that order.
      for (int q0 = 0; q0 < experts; q0 += 32) {
        const int q = q0 + lane;
        int c = 0;
        if (q < experts) {
          const int le = q / ep, dd = q % ep;
          c = table[rank * experts + ((rank + 1 + dd) % ep) * local + le];
        }
        const long long incl = warp_inclusive_scan_ll(c, lane);
        if (q < experts) send_order_start[q] = run + incl - c;
        run += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) send_order_start[experts] = run;
    } else if (job <= ep) {
      // source s: first row of expert e in its expert-major routed buffer
      const int s = job - 1;
      for (int e0 = 0; e0 < experts; e0 += 32) {
        const int e = e0 + lane;
        const int c = e < experts ? table[s * experts + e] : 0;
        const long long incl = warp_inclusive_scan_ll(c, lane);
        const long long first = run + incl - c;
        if (e < experts) {
          if (s == rank) {
            dispatch_src_off[e] = first;
            dispatch_size[e] = c;
          }
          if (e >= rank * local && e < (rank + 1) * local) {
            combine_target_off[s * local + (e - rank * local)] = first;
            combine_size[s * local + (e - rank * local)] = c;
          }
        }
        run += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (s == rank && totals != nullptr && lane == 0) totals[0] = run;  // rows this rank routes (tokens * top_k)
    } else {
      // destination d lays its receive buffer out local-expert-major, then by source rank: entry q = le * ep + s
      const int d = job - 1 - ep;
      for (int q0 = 0; q0 < experts; q0 += 32) {
        const int q = q0 + lane;
        int c = 0, le = 0, src = 0;
        if (q < experts) {
          le = q / ep;
          src = q % ep;
          c = table[src * experts + d * local + le];
        }
        const long long incl = warp_inclusive_scan_ll(c, lane);
        const long long first = run + incl - c;
        if (q < experts) {
          if (src == rank) dispatch_target_off[d * local + le] = first;
          if (d == rank) {
            combine_src_off[src * local + le] = first;
            if (recv_segment_start != nullptr) recv_segment_start[le * ep + src] = first;
            if (src == ep - 1) group_list[le] = first + c;  // rows of local experts 0 .. le
          }
        }
        run += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (d == rank && totals != nullptr && lane == 0) totals[1] = run;  // rows this rank receives
    }
  }
}

__global__ void histogram_kernel(const void* __restrict__ indices, int is_i64, long long entries, int experts,
                                 int* __restrict__ counts, int* __restrict__ status) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < entries; i += stride) {
    const long long e = load_index(indices, is_i64, i);
    if (e >= 0 && e < experts) atomicAdd(&hist[e], 1);
    else report_status(status, HMC_STATUS_BAD_INDEX, static_cast<int>(i), static_cast<int>(e), experts);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x)
    if (hist[e] != 0) atomicAdd(&counts[e], hist[e]);
}

}  // namespace
}  // namespace hmc

using namespace hmc;

static size_t fused_sort_smem(int experts) {
  return static_cast<size_t>(experts) * sizeof(int) * (experts <= RANK_PARALLEL_EXPERTS ? 33 : 1);
}

// Chunks (= CTAs) of the one-launch sort that are resident together on the current device, 0 where cooperative
// launches are not supported. Asked once per device and expert-count class.
static int fused_sort_capacity(int experts) {
  static int cached[64][2];
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  const int cls = experts <= RANK_PARALLEL_EXPERTS ? 0 : 1;
  if (cached[device][cls] == 0) {
    int cooperative = 0, per_sm = 0;
    cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, device);
    // the largest shared-memory request of the class bounds the occupancy of every member
    const size_t smem = cls == 0 ? fused_sort_smem(RANK_PARALLEL_EXPERTS) : fused_sort_smem(4096);
    if (cooperative != 0 && smem <= 48 * 1024 &&
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sort_routes_fused_kernel, SORT_THREADS, smem) == cudaSuccess &&
        per_sm > 0)
      cached[device][cls] = per_sm * sm_count();
    else
      cached[device][cls] = -1;
  }
  return cached[device][cls] > 0 ? cached[device][cls] : 0;
}

extern "C" int64_t hmc_moe_sort_workspace_bytes(int64_t entries, int64_t experts) {
  const int64_t chunks = (entries + SORT_CHUNK - 1) / SORT_CHUNK;
  return (chunks > 0 ? chunks : 1) * experts * static_cast<int64_t>(sizeof(int));
}

extern "C" int hmc_moe_histogram(const void* indices, int indices_are_i64, int64_t entries, int64_t experts,
                                 int32_t* counts, int32_t* status, void* stream_ptr) {
  ProfileScope profile(HMC_PROFILE_ROUTE, static_cast<cudaStream_t>(stream_ptr));
  HMC_REQUIRE(counts != nullptr && (entries == 0 || indices != nullptr), HMC_ERR_INVALID,
              "hmc_moe_histogram: null tensor pointer");
  HMC_REQUIRE(experts > 0 && experts <= 4096, HMC_ERR_LIMIT, "hmc_moe_histogram: experts must be in [1, 4096]");
  HMC_REQUIRE(entries >= 0 && entries < (1ll << 31), HMC_ERR_LIMIT, "hmc_moe_histogram: entries must fit in int32");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  HMC_CUDA_OK(cudaMemsetAsync(counts, 0, experts * sizeof(int), stream));
  if (entries == 0) return 0;
  int grid = static_cast<int>((entries + 255) / 256);
  if (grid > 4 * sm_count()) grid = 4 * sm_count();
  histogram_kernel<<<grid, 256, experts * sizeof(int), stream>>>(indices, indices_are_i64, entries,
                                                                 static_cast<int>(experts), counts, status);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_moe_sort_routes(const void* indices, int indices_are_i64, int64_t entries, int64_t experts,
                                   void* workspace, int64_t workspace_bytes, int32_t* mapping,
                                   int32_t* source_of_row, int32_t* expert_of_row, int32_t* counts,
                                   int64_t* cumulative, int32_t* status, void* stream_ptr) {
  ProfileScope profile(HMC_PROFILE_ROUTE, static_cast<cudaStream_t>(stream_ptr));
  HMC_REQUIRE(experts > 0 && experts <= 4096, HMC_ERR_LIMIT, "hmc_moe_sort_routes: experts must be in [1, 4096]");
  HMC_REQUIRE(entries >= 0 && entries < (1ll << 31), HMC_ERR_LIMIT,
              "hmc_moe_sort_routes: tokens * top_k must fit in int32");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (entries == 0) {
    if (counts != nullptr) HMC_CUDA_OK(cudaMemsetAsync(counts, 0, experts * sizeof(int), stream));
    if (cumulative != nullptr) HMC_CUDA_OK(cudaMemsetAsync(cumulative, 0, experts * sizeof(long long), stream));
    return 0;
  }
  HMC_REQUIRE(indices && mapping && workspace, HMC_ERR_INVALID, "hmc_moe_sort_routes: null tensor pointer");
  HMC_REQUIRE(workspace_bytes >= hmc_moe_sort_workspace_bytes(entries, experts), HMC_ERR_INVALID,
              "hmc_moe_sort_routes: workspace holds %lld bytes, %lld needed", (long long)workspace_bytes,
              (long long)hmc_moe_sort_workspace_bytes(entries, experts));
  const int chunks = static_cast<int>((entries + SORT_CHUNK - 1) / SORT_CHUNK);
  const int e = static_cast<int>(experts);
  const size_t smem = experts * sizeof(int);
  int* chunk_counts = static_cast<int*>(workspace);
  if (chunks <= fused_sort_capacity(e)) {
    // every chunk's CTA is resident at once: one cooperative launch instead of three kernels
    long long entries_arg = entries;
    int experts_arg = e;
    long long* ends = reinterpret_cast<long long*>(cumulative);
    void* params[] = {&indices, &indices_are_i64, &entries_arg, &experts_arg, &chunk_counts, &mapping, &source_of_row,
                      &expert_of_row, &counts, &ends, &status};
    HMC_CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(sort_routes_fused_kernel), dim3(chunks),
                                            dim3(SORT_THREADS), params, fused_sort_smem(e), stream));
    count_launch();
    return 0;
  }
  chunk_histogram_kernel<<<chunks, SORT_THREADS, smem, stream>>>(indices, indices_are_i64, entries, e,
                                                               chunk_counts, status);
  HMC_LAUNCH_OK();
  {
    // stage the chunk table in shared memory when it fits the default 48 KiB
    const size_t staged_bytes = smem + static_cast<size_t>(chunks) * experts * sizeof(int);
    const int stage_table = staged_bytes <= 48 * 1024;
    chunk_scan_kernel<<<1, 1024, stage_table ? staged_bytes : smem, stream>>>(
        chunk_counts, chunks, e, counts, reinterpret_cast<long long*>(cumulative), expert_of_row, source_of_row,
        entries, stage_table);
  }
  HMC_LAUNCH_OK();
  chunk_rank_kernel<<<chunks, SORT_THREADS, smem, stream>>>(indices, indices_are_i64, entries, e, chunk_counts,
                                                          mapping, source_of_row, expert_of_row);
  HMC_LAUNCH_OK();
  return 0;
}

static int check_rows(const char* what, const void* a, const void* b, int64_t hidden) {
  HMC_REQUIRE(a != nullptr && b != nullptr, HMC_ERR_INVALID, "%s: null tensor pointer", what);
  HMC_REQUIRE(hidden > 0 && hidden % 8 == 0, HMC_ERR_INVALID,
              "%s: hidden size (%lld) must be a positive multiple of 8 BF16 elements", what, (long long)hidden);
  HMC_REQUIRE(aligned16(a) && aligned16(b), HMC_ERR_INVALID, "%s: rows must be 16-byte aligned", what);
  return 0;
}

extern "C" int hmc_moe_gather_rows(const void* tokens, const int32_t* source_of_row, int64_t rows, int64_t top_k,
                                   int64_t hidden, void* out, void* stream_ptr) {
  ProfileScope profile(HMC_PROFILE_ROUTE, static_cast<cudaStream_t>(stream_ptr));
  if (rows == 0) return 0;
  int rc = check_rows("hmc_moe_gather_rows", tokens, out, hidden);
  if (rc != 0) return rc;
  HMC_REQUIRE(source_of_row != nullptr && top_k > 0, HMC_ERR_INVALID, "hmc_moe_gather_rows: bad arguments");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  gather_rows_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, stream>>>(
      static_cast<const uint4*>(tokens), source_of_row, rows, static_cast<int>(top_k), static_cast<int>(hidden / 8),
      static_cast<uint4*>(out));
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_moe_permute_from_mapping(const void* tokens, const int32_t* mapping, const float* probs,
                                            int64_t num_tokens, int64_t top_k, int64_t hidden, void* out,
                                            float* out_probs, int32_t* status, void* stream_ptr) {
  ProfileScope profile(HMC_PROFILE_ROUTE, static_cast<cudaStream_t>(stream_ptr));
  if (num_tokens == 0) return 0;
  int rc = check_rows("hmc_moe_permute_from_mapping", tokens, out, hidden);
  if (rc != 0) return rc;
  HMC_REQUIRE(mapping != nullptr && top_k > 0, HMC_ERR_INVALID, "hmc_moe_permute_from_mapping: bad arguments");
  HMC_REQUIRE((out_probs == nullptr) == (probs == nullptr), HMC_ERR_INVALID,
              "hmc_moe_permute_from_mapping: probabilities and their output go together");
  HMC_REQUIRE(num_tokens * top_k < (1ll << 31), HMC_ERR_LIMIT, "hmc_moe_permute_from_mapping: too many routes");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const long long entries = num_tokens * top_k;
  scatter_rows_kernel<<<static_cast<unsigned>((entries + 7) / 8), 256, 0, stream>>>(
      static_cast<const uint4*>(tokens), mapping, probs, entries, static_cast<int>(top_k),
      static_cast<int>(hidden / 8), static_cast<uint4*>(out), out_probs, status);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_moe_unpermute(const void* permuted, const int32_t* mapping, const float* probs,
                                 int64_t num_tokens, int64_t top_k, int64_t hidden, int64_t permuted_rows,
                                 void* out, int32_t* status, void* stream_ptr) {
  return hmc::moe_unpermute_unless(permuted, mapping, probs, num_tokens, top_k, hidden, permuted_rows, out, status, nullptr,
                                   stream_ptr);
}

// hmc_moe_unpermute that does nothing when *skip_flag is non-zero on the device (used by hmc_mega_moe).
int hmc::moe_unpermute_unless(const void* permuted, const int32_t* mapping, const float* probs, int64_t num_tokens,
                              int64_t top_k, int64_t hidden, int64_t permuted_rows, void* out, int32_t* status,
                              const int32_t* skip_flag, void* stream_ptr) {
  ProfileScope profile(HMC_PROFILE_ROUTE, static_cast<cudaStream_t>(stream_ptr));
  if (num_tokens == 0) return 0;
  int rc = check_rows("hmc_moe_unpermute", permuted, out, hidden);
  if (rc != 0) return rc;
  HMC_REQUIRE(mapping != nullptr, HMC_ERR_INVALID, "hmc_moe_unpermute: null mapping");
  HMC_REQUIRE(top_k > 0 && top_k <= MAX_TOP_K, HMC_ERR_LIMIT, "hmc_moe_unpermute: top_k must be in [1, %d]",
              MAX_TOP_K);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  unpermute_kernel<<<static_cast<unsigned>(num_tokens), 128, 0, stream>>>(
      static_cast<const uint4*>(permuted), mapping, probs, num_tokens, static_cast<int>(top_k),
      static_cast<int>(hidden / 8), permuted_rows, static_cast<uint4*>(out), status, skip_flag);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_moe_unpermute_grad(const void* permuted, const void* grad_out, const int32_t* mapping,
                                      const float* probs, int64_t num_tokens, int64_t top_k, int64_t hidden,
                                      void* grad_permuted, float* grad_probs, int32_t* status,
                                      void* stream_ptr) {
  ProfileScope profile(HMC_PROFILE_ROUTE, static_cast<cudaStream_t>(stream_ptr));
  if (num_tokens == 0) return 0;
  int rc = check_rows("hmc_moe_unpermute_grad", grad_out, grad_permuted, hidden);
  if (rc != 0) return rc;
  HMC_REQUIRE(mapping != nullptr && probs != nullptr, HMC_ERR_INVALID, "hmc_moe_unpermute_grad: null tensor pointer");
  HMC_REQUIRE((permuted == nullptr) == (grad_probs == nullptr), HMC_ERR_INVALID,
              "hmc_moe_unpermute_grad: forward outputs and grad_probs go together");
  HMC_REQUIRE(permuted == nullptr || aligned16(permuted), HMC_ERR_INVALID,
              "hmc_moe_unpermute_grad: rows must be 16-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  unpermute_grad_kernel<<<static_cast<unsigned>(num_tokens), 128, 0, stream>>>(
      static_cast<const uint4*>(permuted), static_cast<const uint4*>(grad_out), mapping, probs, num_tokens,
      static_cast<int>(top_k), static_cast<int>(hidden / 8), num_tokens * top_k, static_cast<uint4*>(grad_permuted),
      grad_probs, status);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_moe_token_permute_grad(const void* grad_permuted, const int32_t* mapping, int64_t num_tokens,
                                          int64_t top_k, int64_t hidden, void* grad_tokens, int32_t* status,
                                          void* stream_ptr) {
  ProfileScope profile(HMC_PROFILE_ROUTE, static_cast<cudaStream_t>(stream_ptr));
  if (num_tokens == 0) return 0;
  int rc = check_rows("hmc_moe_token_permute_grad", grad_permuted, grad_tokens, hidden);
  if (rc != 0) return rc;
  HMC_REQUIRE(mapping != nullptr && top_k > 0, HMC_ERR_INVALID, "hmc_moe_token_permute_grad: bad arguments");
  HMC_REQUIRE(top_k <= MAX_TOP_K, HMC_ERR_LIMIT, "hmc_moe_token_permute_grad: top_k must be in [1, %d]", MAX_TOP_K);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  permute_grad_kernel<<<static_cast<unsigned>(num_tokens), 128, 0, stream>>>(
      static_cast<const uint4*>(grad_permuted), mapping, num_tokens, static_cast<int>(top_k),
      static_cast<int>(hidden / 8), num_tokens * top_k, static_cast<uint4*>(grad_tokens), status);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_zero_empty_expert_grad(void* first, int64_t first_bytes_per_expert, void* second,
                                          int64_t second_bytes_per_expert, const int64_t* cumulative,
                                          int64_t experts, void* stream_ptr) {
  HMC_REQUIRE(first != nullptr && cumulative != nullptr && experts > 0, HMC_ERR_INVALID,
              "hmc_zero_empty_expert_grad: bad arguments");
  HMC_REQUIRE(first_bytes_per_expert % 16 == 0 && second_bytes_per_expert % 16 == 0 && aligned16(first) &&
                  (second == nullptr || aligned16(second)),
              HMC_ERR_INVALID, "hmc_zero_empty_expert_grad: expert slices must be multiples of 16 bytes");
  HMC_REQUIRE(experts <= 65535, HMC_ERR_LIMIT, "hmc_zero_empty_expert_grad: too many experts");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  dim3 grid(32, static_cast<unsigned>(experts));
  zero_empty_kernel<<<grid, 256, 0, stream>>>(static_cast<uint4*>(first), first_bytes_per_expert / 16,
                                              static_cast<uint4*>(second), second_bytes_per_expert / 16,
                                              reinterpret_cast<const long long*>(cumulative),
                                              static_cast<int>(experts));
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_route_offsets(const int32_t* counts, int64_t ep, int64_t experts, int64_t rank,
                                 int64_t* dispatch_src_off, int64_t* dispatch_target_off, int32_t* dispatch_size,
                                 int64_t* combine_src_off, int64_t* combine_target_off, int32_t* combine_size,
                                 int64_t* group_list, int64_t* totals, int64_t* recv_segment_start,
                                 int64_t* send_order_start, void* stream_ptr) {
  ProfileScope profile(HMC_PROFILE_ROUTE, static_cast<cudaStream_t>(stream_ptr));
  HMC_REQUIRE(counts && dispatch_src_off && dispatch_target_off && dispatch_size && combine_src_off &&
                  combine_target_off && combine_size && group_list,
              HMC_ERR_INVALID, "hmc_route_offsets: null tensor pointer");
  HMC_REQUIRE(ep > 0 && experts > 0 && experts % ep == 0, HMC_ERR_INVALID,
              "hmc_route_offsets: experts (%lld) must be a positive multiple of ep (%lld)", (long long)experts,
              (long long)ep);
  HMC_REQUIRE(rank >= 0 && rank < ep, HMC_ERR_INVALID, "hmc_route_offsets: rank %lld outside [0, %lld)",
              (long long)rank, (long long)ep);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const size_t table_bytes = static_cast<size_t>(ep) * experts * sizeof(int);
  const int stage_table = table_bytes <= 48 * 1024;
  const int offsets_threads = 32 * static_cast<int>(1 + 2 * ep < 32 ? 1 + 2 * ep : 32);  // one warp per running sum
  route_offsets_kernel<<<1, offsets_threads, stage_table ? table_bytes : 0, stream>>>(
      counts, static_cast<int>(ep), static_cast<int>(experts), static_cast<int>(rank),
      reinterpret_cast<long long*>(dispatch_src_off), reinterpret_cast<long long*>(dispatch_target_off),
      dispatch_size, reinterpret_cast<long long*>(combine_src_off), reinterpret_cast<long long*>(combine_target_off),
      combine_size, reinterpret_cast<long long*>(group_list), reinterpret_cast<long long*>(totals),
      reinterpret_cast<long long*>(recv_segment_start), reinterpret_cast<long long*>(send_order_start), stage_table);
  HMC_LAUNCH_OK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of hmc_moe_sort_routes.
//
// Some callers may not allocate device memory at the point where they route tokens: code that
// runs while a memory pool is frozen, plugins that were handed a fixed set of buffers by their
// host framework, or real-time loops where a cudaMalloc (which can synchronise the whole device)
// is not acceptable. For them the chunk-histogram scratch of the sort lives in this file-scope
// device array instead of a caller-provided workspace. Every GPU that loads the library holds
// the array (HMC_SORT_STATIC_BYTES) until the process exits.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) int g_sort_scratch[HMC_SORT_STATIC_BYTES / sizeof(int)];

// In host code the array's name is only a handle; the device address comes from
// cudaGetSymbolAddress, asked once per device with that device current. The cache is indexed by the
// CURRENT device (the stream passed in must belong to it), is written without a lock (two host threads
// making the first call store the same value, which is harmless) and is not dropped by cudaDeviceReset:
// a process that resets a device must not call this entry point on it again.
static int* g_sort_scratch_address[64];

extern "C" int hmc_moe_sort_routes_static(const void* indices, int indices_are_i64, int64_t entries,
                                          int64_t experts, int32_t* mapping, int32_t* source_of_row,
                                          int32_t* expert_of_row, int32_t* counts, int64_t* cumulative,
                                          int32_t* status, void* stream_ptr) {
  HMC_REQUIRE(experts > 0 && experts <= 4096, HMC_ERR_LIMIT,
              "hmc_moe_sort_routes_static: experts must be in [1, 4096]");
  HMC_REQUIRE(entries >= 0 && entries < (1ll << 31), HMC_ERR_LIMIT,
              "hmc_moe_sort_routes_static: tokens * top_k must fit in int32");
  const int64_t needed = hmc_moe_sort_workspace_bytes(entries, experts);
  HMC_REQUIRE(needed <= static_cast<int64_t>(HMC_SORT_STATIC_BYTES), HMC_ERR_LIMIT,
              "hmc_moe_sort_routes_static: %lld routes over %lld experts need %lld bytes of scratch, the built-in "
              "array holds %lld; use hmc_moe_sort_routes with a caller-provided workspace",
              (long long)entries, (long long)experts, (long long)needed, (long long)HMC_SORT_STATIC_BYTES);
  int device = 0;
  HMC_CUDA_OK(cudaGetDevice(&device));
  HMC_REQUIRE(device >= 0 && device < 64, HMC_ERR_LIMIT, "hmc_moe_sort_routes_static: device ordinal %d not supported",
              device);
  if (g_sort_scratch_address[device] == nullptr) {
    int* address = nullptr;
    HMC_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_sort_scratch));
    HMC_REQUIRE(address != nullptr, HMC_ERR_CUDA, "hmc_moe_sort_routes_static: the scratch array has no device address");
    g_sort_scratch_address[device] = address;
  }
  // Nothing in the scratch has to start at zero: the first pass writes every slot the later
  // passes read, so the previous call's contents are simply overwritten.
  return hmc_moe_sort_routes(indices, indices_are_i64, entries, experts, g_sort_scratch_address[device],
                             static_cast<int64_t>(HMC_SORT_STATIC_BYTES), mapping, source_of_row, expert_of_row,
                             counts, cumulative, status, stream_ptr);
}
