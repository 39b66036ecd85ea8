// CTA-pair variant of the weight-gradient GEMM (RAGGED_K): C_g = A[r0:r1, :]^T * B[r0:r1, :] on
// 256 x 256 tiles shared by the two CTAs of a cluster (tcgen05.mma.cta_group::2, M = 256). Each CTA
// loads 128 columns of A and 128 columns of B per 64-row k-block: 32 KiB instead of the 48 KiB a
// 128 x 256 one-CTA tile needs, so a pair moves two thirds of the operand bytes for the same flops.
//
// The contraction runs over the group's rows, so the last k-block of a tile holds rows of the next
// group; they are cleared in shared memory before the MMA reads them, by each CTA in its own operands.
// Every other k-block follows the protocol of the row-ragged pair kernel: both CTAs' loads count on the
// leader's barrier. Only for a block that needs clearing the second CTA loads onto a barrier of its
// own, clears, and tells the leader (release/acquire at cluster scope) that its stage is ready.
// The leader issues every MMA; each CTA's TMEM holds its own 128 accumulator rows and its own
// epilogue warps store them.
//
// Reference math: the weight-gradient grouped matmuls of ops/hyper_mega_moe_grad/op_kernel/
// worker_kernel.cpp:164-195 (dW2 = act^T dY, dW1 = X^T dU per local expert).
#include <cuda.h>

#include "common.cuh"
#include "gemm_shared.cuh"
#include "sm100.cuh"

namespace hmc {
namespace {

using namespace sm100;
using namespace gemm;

constexpr int DW_PAIR_M = 2 * BM;                     // rows of C per pair tile
constexpr int DW_STAGE_BYTES = 4 * CHUNK_BYTES;       // 2 chunks of A + 2 chunks of B per CTA
constexpr int DW_STAGES = 6;
constexpr int DW_SMEM_BYTES = DW_STAGES * DW_STAGE_BYTES + EPI_WARPS * STORE_STAGE_BYTES + 1024 + 256;
using DwWalker = TileWalkerT<DW_PAIR_M>;

// A k-block with `left` rows of its group left holds foreign rows inside an issued 16-row step.
__device__ __forceinline__ bool block_needs_clearing(long long left) { return left < BK && (left & 15) != 0; }

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_pair_dw_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                            const __grid_constant__ CUtensorMap tm_c, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* store_stage = smem + DW_STAGES * DW_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(store_stage + EPI_WARPS * STORE_STAGE_BYTES);
  uint64_t* full_bar = bars;                                        // leader only: loads of both CTAs
  uint64_t* empty_bar = bars + DW_STAGES;                           // one set per CTA
  uint64_t* peer_bar = bars + 2 * DW_STAGES;                        // leader only: the other CTA's cleared stage is ready
  uint64_t* tail_full_bar = bars + 3 * DW_STAGES;                   // second CTA only: its own loads of a block to clear
  uint64_t* acc_full_bar = bars + 4 * DW_STAGES;                    // one set per CTA
  uint64_t* acc_empty_bar = bars + 4 * DW_STAGES + ACC_STAGES;      // leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4 * DW_STAGES + 2 * ACC_STAGES);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const long long pair = blockIdx.x >> 1;
  const long long pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < DW_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
      mbar_init(&peer_bar[s], 1);
      mbar_init(&tail_full_bar[s], 1);
    }
    for (int s = 0; s < ACC_STAGES; ++s) {
      mbar_init(&acc_full_bar[s], 1);
      mbar_init(&acc_empty_bar[s], 2 * EPI_WARPS);  // every epilogue warp of both CTAs
    }
    *abort_word = 0;
    mbar_fence_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
    prefetch_tensormap(&tm_c);
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
    // ======================================================================== TMA producer (both CTAs)
    if (lane == 0) {
      DwWalker walker(p);
      Tile t;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long idx = pair; ok && walker.get(idx, t); idx += pairs) {
        const int kiters = k_iterations(p, t);
        const int m0 = t.m_idx * DW_PAIR_M + static_cast<int>(rank) * BM;      // this CTA's 128 rows of C
        const int n0 = t.n_idx * BN + static_cast<int>(rank) * (BN / 2);       // this CTA's 128 columns of B
        for (int kb = 0; kb < kiters; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_word, p.pipe_budget_ns)) {
            report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 0, stage, kb);
            ok = false;
            break;
          }
          uint8_t* dst = smem + stage * DW_STAGE_BYTES;
          const int row = static_cast<int>(t.row0) + kb * BK;
          const long long left = t.row1 - (t.row0 + static_cast<long long>(kb) * BK);
          if (block_needs_clearing(left)) {
            // each CTA's bytes count on a barrier of its own: it has to see them before it clears
            if (rank == 0) {
              mbar_arrive_expect_tx(&full_bar[stage], DW_STAGE_BYTES);
              tma_load_2d(dst + 0 * CHUNK_BYTES, &tm_a, &full_bar[stage], m0, row);
              tma_load_2d(dst + 1 * CHUNK_BYTES, &tm_a, &full_bar[stage], m0 + 64, row);
              tma_load_2d(dst + 2 * CHUNK_BYTES, &tm_b, &full_bar[stage], n0, row);
              tma_load_2d(dst + 3 * CHUNK_BYTES, &tm_b, &full_bar[stage], n0 + 64, row);
            } else {
              mbar_arrive_expect_tx(&tail_full_bar[stage], DW_STAGE_BYTES);
              tma_load_2d(dst + 0 * CHUNK_BYTES, &tm_a, &tail_full_bar[stage], m0, row);
              tma_load_2d(dst + 1 * CHUNK_BYTES, &tm_a, &tail_full_bar[stage], m0 + 64, row);
              tma_load_2d(dst + 2 * CHUNK_BYTES, &tm_b, &tail_full_bar[stage], n0, row);
              tma_load_2d(dst + 3 * CHUNK_BYTES, &tm_b, &tail_full_bar[stage], n0 + 64, row);
            }
          } else {
            // the leader's barrier counts the bytes of both CTAs
            if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * DW_STAGE_BYTES);
            tma_load_2d_pair(dst + 0 * CHUNK_BYTES, &tm_a, &full_bar[stage], m0, row);
            tma_load_2d_pair(dst + 1 * CHUNK_BYTES, &tm_a, &full_bar[stage], m0 + 64, row);
            tma_load_2d_pair(dst + 2 * CHUNK_BYTES, &tm_b, &full_bar[stage], n0, row);
            tma_load_2d_pair(dst + 3 * CHUNK_BYTES, &tm_b, &full_bar[stage], n0 + 64, row);
          }
          if (++stage == DW_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ============================================== MMA issue (leader) + tail clearing (both CTAs)
    DwWalker walker(p);
    Tile t;
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t tail_parity = 0;  // per stage: parity of the next phase of peer_bar / tail_full_bar
    bool ok = true;
    constexpr uint32_t idesc = make_idesc_f32acc(1u, DW_PAIR_M, BN, HMC_MAJOR_MN, HMC_MAJOR_MN);
    constexpr uint32_t KSTEP = (16 * 128) >> 4;  // 16 k rows of 128 bytes
    const uint32_t leader_peer_bar = map_to_cta(smem_u32(peer_bar), 0);
    if (rank != 0) {
      // The second CTA issues nothing; it visits the blocks that need clearing, in the order in which
      // its producer loads them. A stage's barriers advance once per such block, and the stage cannot
      // be loaded again before the leader has consumed the block, so the parity bit names the block.
      for (long long idx = pair; ok && walker.get(idx, t); idx += pairs) {
        const int kiters = k_iterations(p, t);
        for (int kb = 0; kb < kiters; ++kb) {
          const long long left = t.row1 - (t.row0 + static_cast<long long>(kb) * BK);
          if (block_needs_clearing(left)) {
            const uint32_t bit = 1u << stage;
            if (!mbar_wait(&tail_full_bar[stage], (tail_parity & bit) ? 1u : 0u, abort_word, p.pipe_budget_ns)) {
              if (lane == 0) report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 5, stage, kb);
              ok = false;
              break;
            }
            tail_parity ^= bit;
            clear_tail_rows(smem + stage * DW_STAGE_BYTES, 4, static_cast<int>(left), lane);
            if (lane == 0) mbar_arrive_cluster(leader_peer_bar + static_cast<uint32_t>(stage) * 8u);
          }
          if (++stage == DW_STAGES) stage = 0;
        }
      }
    } else {
      for (long long idx = pair; ok && walker.get(idx, t); idx += pairs) {
        const int kiters = k_iterations(p, t);
        if (kiters == 0) continue;  // cold group: the epilogue writes zeros on its own
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
          uint8_t* src = smem + stage * DW_STAGE_BYTES;
          int k_steps = BK / 16;
          const long long left = t.row1 - (t.row0 + static_cast<long long>(kb) * BK);
          if (left < BK) k_steps = (static_cast<int>(left) + 15) >> 4;
          if (block_needs_clearing(left)) {
            clear_tail_rows(src, 4, static_cast<int>(left), lane);
            const uint32_t bit = 1u << stage;
            if (!mbar_wait_cluster(&peer_bar[stage], (tail_parity & bit) ? 1u : 0u, abort_word, p.pipe_budget_ns)) {
              if (lane == 0) report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 4, stage, kb);
              ok = false;
              break;
            }
            tail_parity ^= bit;
          }
          tc_fence_after_sync();
          if (lane == 0) {
            uint64_t da = make_smem_desc(smem_u32(src), CHUNK_BYTES, 1024, SWIZZLE_128B);
            uint64_t db = make_smem_desc(smem_u32(src + 2 * CHUNK_BYTES), CHUNK_BYTES, 1024, SWIZZLE_128B);
#pragma unroll
            for (int ks = 0; ks < BK / 16; ++ks) {
              if (ks < k_steps) umma_bf16_pair(tmem_d, da, db, idesc, (kb > 0 || ks > 0) ? 1u : 0u);
              da += KSTEP;
              db += KSTEP;
            }
            umma_commit_pair(&empty_bar[stage]);  // frees the slot in both CTAs
            if (kb == kiters - 1) umma_commit_pair(&acc_full_bar[acc]);
          }
          __syncwarp();
          if (++stage == DW_STAGES) {
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
  } else {
    // ======================================================================== epilogue (both CTAs)
    DwWalker walker(p);
    Tile t;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const int quarter = warp & 3;       // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;   // which half of the tile's columns this warp handles
    const int c_lo = half * (BN / 2);
    const int c_hi = c_lo + BN / 2;
    uint8_t* my_stage = store_stage + (warp - 2) * STORE_STAGE_BYTES;
    unsigned stores_issued = 0;
    const uint32_t leader_acc_empty = map_to_cta(smem_u32(acc_empty_bar), 0);
    for (long long idx = pair; ok && walker.get(idx, t); idx += pairs) {
      const int kiters = k_iterations(p, t);
      const int m_first = t.m_idx * DW_PAIR_M + static_cast<int>(rank) * BM + quarter * 32;  // this warp's rows of C
      const int col_base = t.n_idx * BN;
      if (kiters == 0) {
        // Cold group: exact zeros, no accumulator involved.
        const int m = m_first + lane;
        if (m < p.m) {
          const long long out_row = static_cast<long long>(t.group) * p.m + m;
          if (p.epilogue == HMC_EPI_STORE_F32) {
            float* dst = static_cast<float*>(p.c) + out_row * p.ldc + col_base;
            for (int c = c_lo; c < c_hi && col_base + c < p.n; c += 4)
              *reinterpret_cast<float4*>(dst + c) = make_float4(0.f, 0.f, 0.f, 0.f);
          } else {
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.c) + out_row * p.ldc + col_base;
            for (int c = c_lo; c < c_hi && col_base + c < p.n; c += 8)
              *reinterpret_cast<uint4*>(dst + c) = make_uint4(0, 0, 0, 0);
          }
        }
        continue;
      }
      if (!mbar_wait(&acc_full_bar[acc], acc_phase, abort_word, p.pipe_budget_ns)) {
        if (lane == 0) report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 3, acc, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
      epilogue_tma_boxes(p, &tm_c, taddr, my_stage, stores_issued, m_first, t.group, col_base, c_lo, c_hi, lane);
      tc_fence_before_sync();
      __syncwarp();
      // the MMA issuer lives in the leader: signal its barrier from either CTA
      if (lane == 0) mbar_arrive_cluster(leader_acc_empty + static_cast<uint32_t>(acc) * 8u);
      if (++acc == ACC_STAGES) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (stores_issued > 0 && lane == 0) bulk_wait_all();  // this thread's stores are in global memory
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

}  // namespace

// Called by hmc_grouped_gemm for RAGGED_K problems whose m is a multiple of 256. `p.m_tiles` counts
// 256-row tiles.
int launch_grouped_gemm_pair_dw(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const gemm::Params& p,
                                int grid, cudaStream_t stream) {
  static PerDeviceFlag configured{};
  if (int rc = allow_dynamic_smem(grouped_gemm_pair_dw_kernel, DW_SMEM_BYTES, configured)) return rc;
  grid &= ~1;  // whole pairs
  if (grid < 2) grid = 2;
  grouped_gemm_pair_dw_kernel<<<grid, NUM_THREADS, DW_SMEM_BYTES, stream>>>(ta, tb, tc, p);
  HMC_LAUNCH_OK();
  return 0;
}

}  // namespace hmc
