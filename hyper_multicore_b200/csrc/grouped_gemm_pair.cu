// CTA-pair variant of the grouped BF16 GEMM for row-ragged problems: two CTAs of a cluster share a
// 256 x 256 tile (tcgen05.mma.cta_group::2, M = 256). Each CTA loads its own 128 rows of A and its
// own 128 columns of B, so per k-block a CTA moves 32 KiB instead of 48 KiB and the MMA reads
// 8 KiB per instruction from each SM instead of 12 KiB from one: the shared-memory port stops
// being the limit of the one-CTA kernel. The even CTA of the pair issues every MMA; each CTA's
// TMEM holds its own 128 accumulator rows, and its own epilogue warps store them.
//
// Same math, layouts and epilogues as grouped_gemm.cu (reference: ops/hyper_mega_moe/op_kernel/
// worker_kernel.cpp:122-299, ops/hyper_mega_moe_grad/op_kernel/worker_kernel.cpp:164-195).
#include <cuda.h>

#include "common.cuh"
#include "gemm_shared.cuh"
#include "sm100.cuh"

namespace hmc {
namespace {

using namespace sm100;
using namespace gemm;

constexpr int PAIR_ROWS = 2 * BM;                 // rows of one pair tile
constexpr int HALF_B_BYTES = B_TILE_BYTES / 2;    // 128 columns of B per CTA
constexpr int PAIR_STAGE_BYTES = A_TILE_BYTES + HALF_B_BYTES;  // 32 KiB per CTA per k-block
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256;
using PairWalker = TileWalkerT<PAIR_ROWS>;

// With DISPATCH_WARPS > 0 every CTA carries extra warps that send this rank's rows to their owners while
// the producers wait, per expert, for the rows this rank receives (see grouped_gemm.cu).
template <int B_MAJOR, int DISPATCH_WARPS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS + 32 * DISPATCH_WARPS, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                         const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PAIR_STAGES * PAIR_STAGE_BYTES);
  uint64_t* full_bar = bars;                                          // used in the leader only
  uint64_t* empty_bar = bars + PAIR_STAGES;                           // one set per CTA
  uint64_t* acc_full_bar = bars + 2 * PAIR_STAGES;                    // one set per CTA
  uint64_t* acc_empty_bar = bars + 2 * PAIR_STAGES + ACC_STAGES;      // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * PAIR_STAGES + 2 * ACC_STAGES);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const long long pair = blockIdx.x >> 1;
  const long long pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < ACC_STAGES; ++s) {
      mbar_init(&acc_full_bar[s], 1);
      mbar_init(&acc_empty_bar[s], 2 * EPI_WARPS);  // every epilogue warp of both CTAs
    }
    *abort_word = 0;
    mbar_fence_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before any cross-CTA signal
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ======================================================================== TMA producer
    if (lane == 0) {
      PairWalker walker(p);
      Tile t;
      int stage = 0;
      uint32_t phase = 0;
      int ready_group = -1;
      bool ok = true;
      const int kiters = (p.k + BK - 1) / BK;
      for (long long idx = pair; ok && walker.get(idx, t); idx += pairs) {
        if (p.ready_counters != nullptr && t.group != ready_group) {
          int seen = 0;
          const int need = static_cast<int>(t.row1 - t.row0);
          if (!wait_counter_ge(p.ready_counters + t.group, need, p.ready_budget_ns, &seen, p.status)) {
            report_status(p.status, HMC_STATUS_TIMEOUT_ARRIVAL, t.group, need, seen);
            *abort_word = 1;
            ok = false;
            break;
          }
          fence_proxy_async_all();
          ready_group = t.group;
        }
        const int row = static_cast<int>(t.row0) + t.m_idx * PAIR_ROWS + static_cast<int>(rank) * BM;
        // this CTA's 128 columns of B: second half of the tile, or the `up` columns for SwiGLU
        const int n0 = p.epilogue == HMC_EPI_SWIGLU ? (rank == 0 ? t.n_idx * (BN / 2) : p.n + t.n_idx * (BN / 2))
                                                    : t.n_idx * BN + static_cast<int>(rank) * (BN / 2);
        for (int kb = 0; kb < kiters; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_word, p.pipe_budget_ns)) {
            report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 0, stage, kb);
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + stage * PAIR_STAGE_BYTES;
          uint8_t* b_dst = a_dst + A_TILE_BYTES;
          // the leader's barrier counts the bytes of both CTAs
          if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * PAIR_STAGE_BYTES);
          tma_load_2d_pair(a_dst, &tm_a, &full_bar[stage], kb * BK, row);
          if (B_MAJOR == HMC_MAJOR_MN) {
            tma_load_3d_pair(b_dst, &tm_b, &full_bar[stage], n0, kb * BK, t.group);
            tma_load_3d_pair(b_dst + CHUNK_BYTES, &tm_b, &full_bar[stage], n0 + 64, kb * BK, t.group);
          } else {
            tma_load_3d_pair(b_dst, &tm_b, &full_bar[stage], kb * BK, n0, t.group);
          }
          if (++stage == PAIR_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ======================================================================== MMA issuer (leader only)
    if (rank == 0) {
      PairWalker walker(p);
      Tile t;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      constexpr uint32_t idesc = make_idesc_f32acc(1u, PAIR_ROWS, BN, HMC_MAJOR_K, B_MAJOR);
      constexpr uint32_t B_LBO = B_MAJOR == HMC_MAJOR_MN ? CHUNK_BYTES : 16;
      constexpr uint32_t B_KSTEP = B_MAJOR == HMC_MAJOR_MN ? (16 * 128) >> 4 : 32 >> 4;
      const int kiters = (p.k + BK - 1) / BK;
      for (long long idx = pair; ok && walker.get(idx, t); idx += pairs) {
        if (!mbar_wait(&acc_empty_bar[acc], acc_phase ^ 1u, abort_word, p.pipe_budget_ns)) {
          if (lane == 0) report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 1, acc, 0);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < kiters; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_word, p.pipe_budget_ns)) {
            if (lane == 0) report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 2, stage, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (lane == 0) {
            uint8_t* a_src = smem + stage * PAIR_STAGE_BYTES;
            uint64_t da = make_smem_desc(smem_u32(a_src), 16, 1024, SWIZZLE_128B);
            uint64_t db = make_smem_desc(smem_u32(a_src + A_TILE_BYTES), B_LBO, 1024, SWIZZLE_128B);
#pragma unroll
            for (int ks = 0; ks < BK / 16; ++ks) {
              umma_bf16_pair(tmem_d, da, db, idesc, (kb > 0 || ks > 0) ? 1u : 0u);
              da += 32 >> 4;
              db += B_KSTEP;
            }
            umma_commit_pair(&empty_bar[stage]);  // frees the slot in both CTAs
            if (kb == kiters - 1) umma_commit_pair(&acc_full_bar[acc]);
          }
          __syncwarp();
          if (++stage == PAIR_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (++acc == ACC_STAGES) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else if (DISPATCH_WARPS > 0 && warp >= 2 + EPI_WARPS) {
    // ======================================================================== dispatch warps (both CTAs)
    if (p.dispatch_enabled && !launch_skipped(p))
      dispatch_rows_warp(p.dispatch, static_cast<int>(blockIdx.x) * DISPATCH_WARPS + (warp - 2 - EPI_WARPS),
                         static_cast<int>(gridDim.x) * DISPATCH_WARPS, lane, p.status);
  } else {
    // ======================================================================== epilogue (both CTAs)
    PairWalker walker(p);
    Tile t;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    for (long long idx = pair; ok && walker.get(idx, t); idx += pairs) {
      const long long out_row =
          t.row0 + static_cast<long long>(t.m_idx) * PAIR_ROWS + static_cast<long long>(rank) * BM + row_in_tile;
      const bool row_ok = out_row < t.row1;
      const int col_base = p.epilogue == HMC_EPI_SWIGLU ? t.n_idx * (BN / 2) : t.n_idx * BN;
      if (!mbar_wait(&acc_full_bar[acc], acc_phase, abort_word, p.pipe_budget_ns)) {
        if (lane == 0) report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 3, acc, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
      epilogue_rows(p, taddr, out_row, row_ok, col_base, half);
      tc_fence_before_sync();
      __syncwarp();
      // the MMA issuer lives in the leader: signal its barrier from either CTA
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty_bar[acc]), 0));
      if (++acc == ACC_STAGES) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  // Teardown: no CTA may leave while its partner can still reach into its shared memory or TMEM.
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

constexpr int PAIR_DISPATCH_WARPS = 4;  // 448 threads x 124 registers fit the register file

template <int B_MAJOR, int DISPATCH_WARPS>
int launch_pair_impl(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, int grid, cudaStream_t stream) {
  static PerDeviceFlag configured{};
  auto kernel = grouped_gemm_pair_kernel<B_MAJOR, DISPATCH_WARPS>;
  if (int rc = allow_dynamic_smem(kernel, PAIR_SMEM_BYTES, configured)) return rc;
  kernel<<<grid, NUM_THREADS + 32 * DISPATCH_WARPS, PAIR_SMEM_BYTES, stream>>>(ta, tb, p);
  HMC_LAUNCH_OK();
  return 0;
}

}  // namespace

// Called by hmc_grouped_gemm for RAGGED_M problems with enough rows per group.
int launch_grouped_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const gemm::Params& p, int b_major, int grid,
                             cudaStream_t stream) {
  grid &= ~1;  // whole pairs
  if (grid < 2) grid = 2;
  if (p.dispatch_enabled) {
    if (b_major == HMC_MAJOR_MN) return launch_pair_impl<HMC_MAJOR_MN, PAIR_DISPATCH_WARPS>(ta, tb, p, grid, stream);
    return launch_pair_impl<HMC_MAJOR_K, PAIR_DISPATCH_WARPS>(ta, tb, p, grid, stream);
  }
  if (b_major == HMC_MAJOR_MN) return launch_pair_impl<HMC_MAJOR_MN, 0>(ta, tb, p, grid, stream);
  return launch_pair_impl<HMC_MAJOR_K, 0>(ta, tb, p, grid, stream);
}

}  // namespace hmc
