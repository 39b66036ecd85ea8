// Persistent grouped GEMM for the MoE expert FFN on sm_100a: TMA-fed shared-memory ring,
// tcgen05.mma with FP32 accumulators in TMEM (two accumulator stages), fused epilogues.
//
// Replaces the reference's per-expert Cube tasks: GMM1/GMM2 (ops/hyper_mega_moe/op_kernel/
// worker_kernel.cpp:225-299, ops/common/mega_moe/adapters/arch35/gmm/bf16_worker.h:44-85), the
// SwiGLU vector task (worker_kernel.cpp:122-223), the backward GEMMs and SwiGLUGrad
// (ops/hyper_mega_moe_grad/op_kernel/worker_kernel.cpp:164-195), and the "zero dW of cold
// experts" rule (bf16_worker.h:62-75).
//
// One CTA per SM, 320 threads: warp 0 = TMA producer, warp 1 = MMA issuer (+TMEM owner),
// warps 2..9 = epilogue (two warps per TMEM lane quarter, one column half each). Tiles are
// 128 x 256 x 64. Weight-gradient tiles leave through shared memory and TMA stores.
// With DISPATCH_WARPS > 0 the CTA carries extra warps that send this rank's rows to their owners
// (peer stores + arrival counters) while the producer waits, per expert, for the rows this rank
// receives: dispatch and the first tiles overlap inside one launch, as the reference's dispatch PUT
// tasks and GMM1 do (ops/hyper_mega_moe/op_kernel/worker_kernel.cpp:301-366).
//
//  RAGGED_M : C[r0:r1, :] = A[r0:r1, :] * B_g      rows of group g are [ends[g-1], ends[g])
//  RAGGED_K : C_g = A[r0:r1, :]^T * B[r0:r1, :]    contraction over the group's rows
#include <cuda.h>

#include "common.cuh"
#include "gemm_shared.cuh"
#include "sm100.cuh"

namespace hmc {
namespace {

using namespace sm100;
using namespace gemm;

using TileWalker = TileWalkerT<BM>;

template <int A_MAJOR, int B_MAJOR, int DISPATCH_WARPS>
__global__ void __launch_bounds__(NUM_THREADS + 32 * DISPATCH_WARPS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ CUtensorMap tm_c, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* store_stage = smem + STAGES * STAGE_BYTES;  // [EPI_WARPS][STORE_STAGE_BYTES], 1024-aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(store_stage + EPI_WARPS * STORE_STAGE_BYTES);
  uint64_t* full_bar = bars;                                 // [STAGES]
  uint64_t* empty_bar = bars + STAGES;                       // [STAGES]
  uint64_t* acc_full_bar = bars + 2 * STAGES;                // [ACC_STAGES]
  uint64_t* acc_empty_bar = bars + 2 * STAGES + ACC_STAGES;  // [ACC_STAGES]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * ACC_STAGES);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < ACC_STAGES; ++s) {
      mbar_init(&acc_full_bar[s], 1);
      mbar_init(&acc_empty_bar[s], EPI_WARPS);  // one arrival per epilogue warp
    }
    *abort_word = 0;
    mbar_fence_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
    if (p.mode == HMC_GEMM_RAGGED_K || p.tma_store) prefetch_tensormap(&tm_c);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ======================================================================== TMA producer
    if (lane == 0) {
      TileWalker walker(p);
      Tile t;
      int stage = 0;
      uint32_t phase = 0;
      int ready_group = -1;
      bool ok = true;
      for (long long idx = blockIdx.x; ok && walker.get(idx, t); idx += gridDim.x) {
        const int kiters = k_iterations(p, t);
        if (p.ready_counters != nullptr && t.group != ready_group) {
          // Rows of this group are written by peers; wait until all of them have landed, then
          // order the async-proxy (TMA) reads after the acquire.
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
        for (int kb = 0; kb < kiters; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_word, p.pipe_budget_ns)) {
            report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 0, stage, kb);
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + stage * STAGE_BYTES;
          uint8_t* b_dst = a_dst + A_TILE_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
          if (p.mode == HMC_GEMM_RAGGED_M) {
            const int row = static_cast<int>(t.row0) + t.m_idx * BM;
            // A is [rows, K] row-major: K-major operand, one 64 x 128 box.
            tma_load_2d(a_dst, &tm_a, &full_bar[stage], kb * BK, row);
            if (p.epilogue == HMC_EPI_SWIGLU) {
              // Accumulator columns [0,128) = gate columns, [128,256) = matching up columns.
              const int g0 = t.n_idx * (BN / 2);
              const int u0 = p.n + g0;
              if (B_MAJOR == HMC_MAJOR_MN) {
                tma_load_3d(b_dst + 0 * CHUNK_BYTES, &tm_b, &full_bar[stage], g0, kb * BK, t.group);
                tma_load_3d(b_dst + 1 * CHUNK_BYTES, &tm_b, &full_bar[stage], g0 + 64, kb * BK, t.group);
                tma_load_3d(b_dst + 2 * CHUNK_BYTES, &tm_b, &full_bar[stage], u0, kb * BK, t.group);
                tma_load_3d(b_dst + 3 * CHUNK_BYTES, &tm_b, &full_bar[stage], u0 + 64, kb * BK, t.group);
              } else {
                tma_load_3d(b_dst, &tm_b, &full_bar[stage], kb * BK, g0, t.group);
                tma_load_3d(b_dst + B_TILE_BYTES / 2, &tm_b, &full_bar[stage], kb * BK, u0, t.group);
              }
            } else {
              const int n0 = t.n_idx * BN;
              if (B_MAJOR == HMC_MAJOR_MN) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
                  tma_load_3d(b_dst + c * CHUNK_BYTES, &tm_b, &full_bar[stage], n0 + c * 64, kb * BK,
                              t.group);
              } else {
                tma_load_3d(b_dst, &tm_b, &full_bar[stage], kb * BK, n0, t.group);
                tma_load_3d(b_dst + B_TILE_BYTES / 2, &tm_b, &full_bar[stage], kb * BK, n0 + BN / 2,
                            t.group);
              }
            }
          } else {
            // Both operands are [rows, width] row-major, contracted over rows: MN-major chunks.
            const int row = static_cast<int>(t.row0) + kb * BK;
            const int m0 = t.m_idx * BM;
            const int n0 = t.n_idx * BN;
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_2d(a_dst + c * CHUNK_BYTES, &tm_a, &full_bar[stage], m0 + c * 64, row);
#pragma unroll
            for (int c = 0; c < 4; ++c)
              tma_load_2d(b_dst + c * CHUNK_BYTES, &tm_b, &full_bar[stage], n0 + c * 64, row);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ======================================================================== MMA issuer
    TileWalker walker(p);
    Tile t;
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    constexpr uint32_t idesc = make_idesc_f32acc(1u, BM, BN, A_MAJOR, B_MAJOR);
    // Descriptor strides. K-major: 8-row groups are 1024 B apart. MN-major: 64-wide chunks are
    // CHUNK_BYTES apart (leading), 8-row k groups are 1024 B apart (stride).
    constexpr uint32_t A_LBO = A_MAJOR == HMC_MAJOR_MN ? CHUNK_BYTES : 16;
    constexpr uint32_t B_LBO = B_MAJOR == HMC_MAJOR_MN ? CHUNK_BYTES : 16;
    constexpr uint32_t A_KSTEP = A_MAJOR == HMC_MAJOR_MN ? (16 * 128) >> 4 : 32 >> 4;
    constexpr uint32_t B_KSTEP = B_MAJOR == HMC_MAJOR_MN ? (16 * 128) >> 4 : 32 >> 4;
    for (long long idx = blockIdx.x; ok && walker.get(idx, t); idx += gridDim.x) {
      const int kiters = k_iterations(p, t);
      if (kiters == 0) continue;  // RAGGED_K cold group: the epilogue writes zeros on its own
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
        uint8_t* a_src = smem + stage * STAGE_BYTES;
        uint8_t* b_src = a_src + A_TILE_BYTES;
        int k_steps = BK / 16;
        if (p.mode == HMC_GEMM_RAGGED_K) {
          const long long left = t.row1 - (t.row0 + static_cast<long long>(kb) * BK);
          // the stage holds 2 A chunks followed by 4 B chunks
          if (left < BK) k_steps = clear_tail_rows(a_src, 6, static_cast<int>(left), lane);
        }
        if (lane == 0) {
          uint64_t da = make_smem_desc(smem_u32(a_src), A_LBO, 1024, SWIZZLE_128B);
          uint64_t db = make_smem_desc(smem_u32(b_src), B_LBO, 1024, SWIZZLE_128B);
#pragma unroll
          for (int ks = 0; ks < BK / 16; ++ks) {
            if (ks < k_steps) umma_bf16(tmem_d, da, db, idesc, (kb > 0 || ks > 0) ? 1u : 0u);
            da += A_KSTEP;
            db += B_KSTEP;
          }
          umma_commit(&empty_bar[stage]);  // frees this smem slot once the MMAs have read it
          if (kb == kiters - 1) umma_commit(&acc_full_bar[acc]);
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (++acc == ACC_STAGES) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  } else if (DISPATCH_WARPS > 0 && warp >= 2 + EPI_WARPS) {
    // ======================================================================== dispatch warps
    if (p.dispatch_enabled && !launch_skipped(p))
      dispatch_rows_warp(p.dispatch, static_cast<int>(blockIdx.x) * DISPATCH_WARPS + (warp - 2 - EPI_WARPS),
                         static_cast<int>(gridDim.x) * DISPATCH_WARPS, lane, p.status);
  } else {
    // ======================================================================== epilogue
    TileWalker walker(p);
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
    const int row_in_tile = quarter * 32 + lane;
    for (long long idx = blockIdx.x; ok && walker.get(idx, t); idx += gridDim.x) {
      const int kiters = k_iterations(p, t);
      long long out_row;
      bool row_ok;
      int col_base;
      if (p.mode == HMC_GEMM_RAGGED_M) {
        out_row = t.row0 + static_cast<long long>(t.m_idx) * BM + row_in_tile;
        row_ok = out_row < t.row1;
        col_base = p.epilogue == HMC_EPI_SWIGLU ? t.n_idx * (BN / 2) : t.n_idx * BN;
      } else {
        const int m = t.m_idx * BM + row_in_tile;
        row_ok = m < p.m;
        out_row = static_cast<long long>(t.group) * p.m + m;
        col_base = t.n_idx * BN;
      }
      if (kiters == 0) {
        // Cold group in RAGGED_K: exact zeros, no accumulator involved.
        if (row_ok) {
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
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(acc * BN);
      // A RAGGED_M tile whose 128 rows all belong to its group may use the same path: nothing past
      // the group's last row is written.
      const bool full_rows = p.tma_store && t.row0 + static_cast<long long>(t.m_idx + 1) * BM <= t.row1;
      if (p.mode == HMC_GEMM_RAGGED_K || full_rows) {
        // Weight-gradient tiles are regular [m, n] grids per group, so they leave through shared
        // memory and TMA stores (clipped at the m and n edges by the tensor map), 32 columns per box.
        // FP32 boxes are 32 columns x 128 bytes in one 4 KiB stage. BF16 boxes are 32 columns x 64 bytes:
        // the stage holds two of them, so the store of one box overlaps the packing of the next.
        const bool ragged_k = p.mode == HMC_GEMM_RAGGED_K;
        const int m0 = (ragged_k ? t.m_idx * BM : static_cast<int>(t.row0) + t.m_idx * BM) + quarter * 32;
        const int plane = ragged_k ? t.group : 0;
        epilogue_tma_boxes(p, &tm_c, taddr, my_stage, stores_issued, m0, plane, col_base, c_lo, c_hi, lane);
      } else if (p.combine_enabled) {
        // Fused combine: the rows go to the routed buffers of their source ranks. Each lane finds the
        // destination of its own row; the tile is staged in shared memory so that every store
        // instruction writes whole 128-byte pieces of four rows (NVLink-friendly), not 16 bytes of
        // thirty-two rows.
        const CombineFuse& cf = p.combine;
        unsigned long long dst_bits = 0;
        int source = -1;
        if (row_ok) {
          const long long* seg = cf.segment_start + static_cast<long long>(t.group) * cf.ep;
          int s = 0;
          for (int q = 1; q < cf.ep; ++q)
            if (seg[q] <= out_row) s = q;
          const long long dest = cf.combine_target_off[s * cf.local_experts + t.group] + (out_row - seg[s]);
          if (dest >= 0 && dest < cf.target_rows_limit) {
            source = s;
            dst_bits = reinterpret_cast<unsigned long long>(static_cast<__nv_bfloat16*>(cf.peer_data[s]) +
                                                            dest * p.ldc + col_base);
          } else {
            report_status(p.status, HMC_STATUS_BAD_INDEX, static_cast<int>(out_row), s, static_cast<int>(dest));
          }
        }
        const int sub = lane >> 3;
        const int piece = lane & 7;
#pragma unroll 1
        for (int c = c_lo; c < c_hi; c += 64) {
          if (col_base + c >= p.n) break;
          uint32_t v[32];
          uint32_t w[32];
          tmem_ld_32x32(taddr + c, v);
          tmem_ld_32x32(taddr + c + 32, w);
          tmem_ld_wait();
          uint8_t* row_base = my_stage + lane * 128;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint32_t* src = q < 4 ? v + 8 * q : w + 8 * (q - 4);
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(src[0]), __uint_as_float(src[1]));
            o.y = pack_bf16x2(__uint_as_float(src[2]), __uint_as_float(src[3]));
            o.z = pack_bf16x2(__uint_as_float(src[4]), __uint_as_float(src[5]));
            o.w = pack_bf16x2(__uint_as_float(src[6]), __uint_as_float(src[7]));
            *reinterpret_cast<uint4*>(row_base + ((q ^ (lane & 7)) << 4)) = o;
          }
          __syncwarp();
          const bool piece_ok = col_base + c + piece * 8 < p.n;
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const int r = i + sub;
            const unsigned long long base = __shfl_sync(0xffffffffu, dst_bits, r);
            if (base != 0 && piece_ok) {
              const uint4 val = *reinterpret_cast<const uint4*>(my_stage + r * 128 + ((piece ^ (r & 7)) << 4));
              st_16(reinterpret_cast<uint8_t*>(base) + c * 2 + piece * 16, val);
            }
          }
          __syncwarp();
        }
        // One release-add per destination per warp: the warp barrier orders every lane's stores
        // before the leader's release, which publishes them to the acquiring rank.
        const unsigned same = __match_any_sync(0xffffffffu, source);
        if (source >= 0 && lane == __ffs(same) - 1)
          red_release_sys_add(cf.peer_ctrl[source] + HMC_CTRL_COMBINE, __popc(same));
      } else {
        epilogue_rows(p, taddr, out_row, row_ok, col_base, half);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty_bar[acc]);
      if (++acc == ACC_STAGES) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (stores_issued > 0 && lane == 0) bulk_wait_all();  // this thread's stores are in global memory
  }

  // Teardown: everyone meets here (also after a time-out), then the allocating warp frees TMEM.
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ----------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  }
  return fn;
}

// Tensor of `rank` dims (dims[0] innermost), box with a 128-byte inner extent, 128-byte swizzle.
int make_map(CUtensorMap* out, const void* base, int rank, const cuuint64_t* dims, const cuuint32_t* box,
             bool f32 = false, bool swizzle64 = false) {
  EncodeTiledFn fn = encode_fn();
  HMC_REQUIRE(fn != nullptr, HMC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t strides[4];
  cuuint64_t acc = f32 ? 4 : 2;
  for (int i = 0; i + 1 < rank; ++i) {
    acc *= dims[i];
    strides[i] = acc;
  }
  cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                  static_cast<cuuint32_t>(rank),
                  const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  HMC_REQUIRE(r == CUDA_SUCCESS, HMC_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

constexpr int SINGLE_DISPATCH_WARPS = 2;  // 384 threads x 168 registers still fit the register file

template <int A_MAJOR, int B_MAJOR, int DISPATCH_WARPS = 0>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const Params& p, int grid,
           cudaStream_t stream) {
  static PerDeviceFlag configured{};
  auto kernel = grouped_gemm_kernel<A_MAJOR, B_MAJOR, DISPATCH_WARPS>;
  if (int rc = allow_dynamic_smem(kernel, SMEM_BYTES, configured)) return rc;
  kernel<<<grid, NUM_THREADS + 32 * DISPATCH_WARPS, SMEM_BYTES, stream>>>(ta, tb, tc, p);
  HMC_LAUNCH_OK();
  return 0;
}

}  // namespace

int launch_grouped_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const gemm::Params& p, int b_major, int grid,
                             cudaStream_t stream);
int fill_dispatch(DispatchFuse* out, const hmc_ep_dispatch_args& a, const char* who);  // ep.cu
int launch_grouped_gemm_pair_dw(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const gemm::Params& p,
                                int grid, cudaStream_t stream);

}  // namespace hmc

extern "C" int64_t hmc_grouped_gemm_combine_units(int64_t n) {
  // every (32-row, half-tile) piece of every 256-column tile reports its rows once
  return 2 * ((n + hmc::gemm::BN - 1) / hmc::gemm::BN);
}

extern "C" int hmc_grouped_gemm(const hmc_grouped_gemm_args* args, void* stream_ptr) {
  using namespace hmc;
  HMC_REQUIRE(args != nullptr, HMC_ERR_INVALID, "hmc_grouped_gemm: null args");
  const hmc_grouped_gemm_args& a = *args;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  ProfileScope profile(HMC_PROFILE_GROUPED_GEMM, stream);
  HMC_REQUIRE(a.mode == HMC_GEMM_RAGGED_M || a.mode == HMC_GEMM_RAGGED_K, HMC_ERR_INVALID,
              "hmc_grouped_gemm: unknown mode %d", a.mode);
  HMC_REQUIRE(a.epilogue >= HMC_EPI_STORE_BF16 && a.epilogue <= HMC_EPI_SWIGLU_GRAD, HMC_ERR_INVALID,
              "hmc_grouped_gemm: unknown epilogue %d", a.epilogue);
  HMC_REQUIRE(a.groups > 0 && a.rows >= 0 && a.n > 0, HMC_ERR_INVALID,
              "hmc_grouped_gemm: groups (%d) and n (%lld) must be positive, rows (%lld) non-negative",
              a.groups, (long long)a.n, (long long)a.rows);
  HMC_REQUIRE(a.rows < (1ll << 31) && a.n < (1ll << 31) && a.k < (1ll << 31) && a.m < (1ll << 31),
              HMC_ERR_INVALID, "hmc_grouped_gemm: extents must fit in int32");
  HMC_REQUIRE(a.a && a.b && (a.c || a.combine) && a.group_ends, HMC_ERR_INVALID,
              "hmc_grouped_gemm: null tensor pointer");
  HMC_REQUIRE(aligned16(a.a) && aligned16(a.b) && aligned16(a.c), HMC_ERR_INVALID,
              "hmc_grouped_gemm: tensors must be 16-byte aligned");
  HMC_REQUIRE(a.n % 8 == 0, HMC_ERR_INVALID, "hmc_grouped_gemm: n (%lld) must be a multiple of 8",
              (long long)a.n);
  if (a.rows == 0 && a.mode == HMC_GEMM_RAGGED_M && (a.dispatch == nullptr || a.dispatch->rows == 0)) return 0;

  Params p{};
  p.mode = a.mode;
  p.epilogue = a.epilogue;
  p.groups = a.groups;
  p.rows = a.rows;
  p.group_ends = reinterpret_cast<const long long*>(a.group_ends);
  p.c = a.c;
  p.aux = a.aux;
  p.ready_counters = a.ready_counters;
  p.ready_budget_ns = a.ready_budget_ns ? a.ready_budget_ns : 10ull * 1000 * 1000 * 1000;
  // The producer may wait for late rows for the whole arrival budget: the MMA and epilogue warps behind
  // it get that time on top of their own, so that a slow peer never shows up as a pipeline time-out.
  p.pipe_budget_ns = (a.pipe_budget_ns ? a.pipe_budget_ns : PIPE_BUDGET_NS) + (a.ready_counters ? p.ready_budget_ns : 0);
  p.status = a.status;
  p.skip_flag = a.skip_flag;
  p.n = static_cast<int>(a.n);
  {
    const bool swiglu_family = a.epilogue == HMC_EPI_SWIGLU || a.epilogue == HMC_EPI_SWIGLU_GRAD;
    HMC_REQUIRE(a.swiglu_clamp >= HMC_CLAMP_NONE && a.swiglu_clamp <= HMC_CLAMP_AFTER_SILU, HMC_ERR_INVALID,
                "hmc_grouped_gemm: unknown swiglu_clamp %d", a.swiglu_clamp);
    HMC_REQUIRE(swiglu_family || (a.swiglu_clamp == HMC_CLAMP_NONE && a.row_probs == nullptr && a.row_dot == nullptr),
                HMC_ERR_INVALID, "hmc_grouped_gemm: clamp and row probabilities belong to the SwiGLU epilogues");
    HMC_REQUIRE(a.swiglu_clamp == HMC_CLAMP_NONE || (a.swiglu_limit > 0.0f && a.swiglu_limit < 3.0e38f),
                HMC_ERR_INVALID, "hmc_grouped_gemm: swiglu_limit must be positive and finite");
    HMC_REQUIRE(a.row_dot == nullptr || (a.epilogue == HMC_EPI_SWIGLU_GRAD && a.row_probs != nullptr), HMC_ERR_INVALID,
                "hmc_grouped_gemm: row_dot is an output of the SwiGLU-grad epilogue with row_probs");
    p.swiglu_clamp = a.swiglu_clamp;
    p.swiglu_limit = a.swiglu_limit;
    p.row_probs = a.row_probs;
    p.row_dot = a.row_dot;
  }
  if (a.combine != nullptr) {
    const hmc_gemm_combine& cb = *a.combine;
    HMC_REQUIRE(a.mode == HMC_GEMM_RAGGED_M && a.epilogue == HMC_EPI_STORE_BF16, HMC_ERR_INVALID,
                "hmc_grouped_gemm: the fused combine belongs to RAGGED_M GEMMs with BF16 stores");
    HMC_REQUIRE(cb.ep >= 1 && cb.ep <= HMC_MAX_EP && cb.local_experts == a.groups, HMC_ERR_INVALID,
                "hmc_grouped_gemm: combine needs 1 <= ep <= %d and local_experts == groups", HMC_MAX_EP);
    HMC_REQUIRE(cb.segment_start && cb.combine_target_off && cb.peer_buffers && cb.peer_ctrl && cb.target_rows_limit > 0,
                HMC_ERR_INVALID, "hmc_grouped_gemm: null combine table");
    HMC_REQUIRE(a.n % 8 == 0, HMC_ERR_INVALID, "hmc_grouped_gemm: combined rows must be multiples of 16 bytes");
    for (int r = 0; r < cb.ep; ++r) {
      HMC_REQUIRE(cb.peer_buffers[r] != nullptr && cb.peer_ctrl[r] != nullptr && aligned16(cb.peer_buffers[r]),
                  HMC_ERR_INVALID, "hmc_grouped_gemm: peer %d has no 16-byte aligned routed buffer / control block", r);
      p.combine.peer_data[r] = cb.peer_buffers[r];
      p.combine.peer_ctrl[r] = static_cast<int*>(cb.peer_ctrl[r]);
    }
    p.combine.segment_start = reinterpret_cast<const long long*>(cb.segment_start);
    p.combine.combine_target_off = reinterpret_cast<const long long*>(cb.combine_target_off);
    p.combine.target_rows_limit = cb.target_rows_limit;
    p.combine.ep = static_cast<int>(cb.ep);
    p.combine.local_experts = static_cast<int>(cb.local_experts);
    p.combine_enabled = 1;
  }

  if (a.dispatch != nullptr && a.dispatch->rows > 0) {  // a rank without rows has nothing to send
    const hmc_ep_dispatch_args& d = *a.dispatch;
    HMC_REQUIRE(a.mode == HMC_GEMM_RAGGED_M && a.ready_counters != nullptr, HMC_ERR_INVALID,
                "hmc_grouped_gemm: a fused dispatch belongs to a RAGGED_M GEMM gated by arrival counters");
    int drc = fill_dispatch(&p.dispatch, d, "hmc_grouped_gemm");
    if (drc != 0) return drc;
    HMC_REQUIRE(d.local_experts == a.groups && d.hidden == a.k, HMC_ERR_INVALID,
                "hmc_grouped_gemm: the fused dispatch must send rows of this GEMM's k (%lld) to groups (%d) experts per rank",
                (long long)a.k, a.groups);
    HMC_REQUIRE(d.peer_buffers[d.rank] == a.a, HMC_ERR_INVALID,
                "hmc_grouped_gemm: with a fused dispatch, a must be this rank's own receive buffer");
    p.dispatch_enabled = 1;
  }

  CUtensorMap ta, tb, tc;
  int rc;
  if (a.mode == HMC_GEMM_RAGGED_M) {
    HMC_REQUIRE(a.k > 0 && a.k % 8 == 0, HMC_ERR_INVALID,
                "hmc_grouped_gemm: k (%lld) must be a positive multiple of 8", (long long)a.k);
    HMC_REQUIRE(a.a_major == HMC_MAJOR_K, HMC_ERR_INVALID,
                "hmc_grouped_gemm: RAGGED_M takes a row-major (K-major) A");
    p.k = static_cast<int>(a.k);
    const bool swiglu = a.epilogue == HMC_EPI_SWIGLU;
    const bool grad = a.epilogue == HMC_EPI_SWIGLU_GRAD;
    HMC_REQUIRE(!(swiglu || grad) || (a.aux != nullptr && aligned16(a.aux)), HMC_ERR_INVALID,
                "hmc_grouped_gemm: the SwiGLU epilogues need a 16-byte aligned aux tensor");
    const long long b_cols = swiglu ? 2 * a.n : a.n;  // width of B along N
    p.n_tiles = swiglu ? static_cast<int>((a.n + BN / 2 - 1) / (BN / 2)) : static_cast<int>((a.n + BN - 1) / BN);
    p.ldc = static_cast<int>((swiglu || grad) ? 2 * a.n : a.n);
    p.ld_aux = static_cast<int>(swiglu ? a.n : 2 * a.n);
    {
      // a rank that receives nothing still launches when it has rows to send: one row keeps the map valid
      cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.k), static_cast<cuuint64_t>(a.rows > 0 ? a.rows : 1)};
      cuuint32_t box[2] = {64, BM};
      if ((rc = make_map(&ta, a.a, 2, dims, box)) != 0) return rc;
    }
    if (a.b_major == HMC_MAJOR_MN) {  // B = [groups, K, Ncols]
      cuuint64_t dims[3] = {static_cast<cuuint64_t>(b_cols), static_cast<cuuint64_t>(a.k),
                            static_cast<cuuint64_t>(a.groups)};
      cuuint32_t box[3] = {64, BK, 1};
      if ((rc = make_map(&tb, a.b, 3, dims, box)) != 0) return rc;
    } else {  // B = [groups, Ncols, K]
      cuuint64_t dims[3] = {static_cast<cuuint64_t>(a.k), static_cast<cuuint64_t>(b_cols),
                            static_cast<cuuint64_t>(a.groups)};
      cuuint32_t box[3] = {64, BN / 2, 1};
      if ((rc = make_map(&tb, a.b, 3, dims, box)) != 0) return rc;
    }
  } else {
    HMC_REQUIRE(a.m > 0 && a.m % 8 == 0, HMC_ERR_INVALID,
                "hmc_grouped_gemm: m (%lld) must be a positive multiple of 8", (long long)a.m);
    HMC_REQUIRE(a.a_major == HMC_MAJOR_MN && a.b_major == HMC_MAJOR_MN, HMC_ERR_INVALID,
                "hmc_grouped_gemm: RAGGED_K takes row-major [rows, m] and [rows, n] operands");
    HMC_REQUIRE(a.epilogue == HMC_EPI_STORE_BF16 || a.epilogue == HMC_EPI_STORE_F32, HMC_ERR_INVALID,
                "hmc_grouped_gemm: RAGGED_K supports plain stores only");
    HMC_REQUIRE(a.ready_counters == nullptr, HMC_ERR_INVALID,
                "hmc_grouped_gemm: arrival counters apply to RAGGED_M only");
    p.m = static_cast<int>(a.m);
    p.m_tiles = static_cast<int>((a.m + BM - 1) / BM);
    p.n_tiles = static_cast<int>((a.n + BN - 1) / BN);
    p.ldc = static_cast<int>(a.n);
    // A zero-row tensor cannot be described by a tensor map; one row keeps the map valid and is
    // never read because every group then has zero k iterations.
    const cuuint64_t map_rows = static_cast<cuuint64_t>(a.rows > 0 ? a.rows : 1);
    {
      cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.m), map_rows};
      cuuint32_t box[2] = {64, BK};
      if ((rc = make_map(&ta, a.a, 2, dims, box)) != 0) return rc;
    }
    {
      cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.n), map_rows};
      cuuint32_t box[2] = {64, BK};
      if ((rc = make_map(&tb, a.b, 2, dims, box)) != 0) return rc;
    }
    {  // C = [groups, m, n]: 32-row boxes, 128 bytes wide
      const bool f32 = a.epilogue == HMC_EPI_STORE_F32;
      cuuint64_t dims[3] = {static_cast<cuuint64_t>(a.n), static_cast<cuuint64_t>(a.m),
                            static_cast<cuuint64_t>(a.groups)};
      cuuint32_t box[3] = {32u, 32, 1};  // FP32: 128-byte rows; BF16: 64-byte rows, two boxes in flight
      if ((rc = make_map(&tc, a.c, 3, dims, box, f32, !f32)) != 0) return rc;
    }
  }
  if (a.mode == HMC_GEMM_RAGGED_M) {
    tc = ta;  // unused by the kernel unless the plain-store path below is on
    const bool f32 = a.epilogue == HMC_EPI_STORE_F32;
    const bool plain = f32 || a.epilogue == HMC_EPI_STORE_BF16;
    if (plain && !p.combine_enabled && (a.n * (f32 ? 4 : 2)) % 16 == 0 && aligned16(a.c)) {
      // C = [1, rows, n] seen through the same 32-row x 128-byte boxes as the weight gradients
      cuuint64_t dims[3] = {static_cast<cuuint64_t>(a.n), static_cast<cuuint64_t>(a.rows > 0 ? a.rows : 1), 1};
      cuuint32_t box[3] = {32u, 32, 1};
      if ((rc = make_map(&tc, a.c, 3, dims, box, f32, !f32)) != 0) return rc;
      p.tma_store = 1;
    }
  }

  int grid = a.max_ctas > 0 ? a.max_ctas : sm_count();
  if (grid > sm_count()) grid = sm_count();
  if (a.mode == HMC_GEMM_RAGGED_K) {
    // CTA pairs on 256 x 256 tiles move two thirds of the operand bytes: taken whenever m splits into them
    if (a.tile_mode != HMC_TILE_SINGLE && a.m % (2 * BM) == 0 && sm_count() >= 2) {
      p.m_tiles = static_cast<int>(a.m / (2 * BM));
      const long long pair_tiles = static_cast<long long>(p.groups) * p.m_tiles * p.n_tiles;
      if (2 * pair_tiles < grid) grid = static_cast<int>(2 * pair_tiles);
      return launch_grouped_gemm_pair_dw(ta, tb, tc, p, grid, stream);
    }
    const long long tiles = static_cast<long long>(p.groups) * p.m_tiles * p.n_tiles;
    if (tiles < grid) grid = static_cast<int>(tiles);
    return launch<HMC_MAJOR_MN, HMC_MAJOR_MN>(ta, tb, tc, p, grid, stream);
  }
  // CTA pairs work on 256-row tiles: worth it once the average group fills most of one
  const bool use_pairs = a.tile_mode == HMC_TILE_PAIR || (a.tile_mode == HMC_TILE_AUTO && a.rows >= 192ll * a.groups);
  if (use_pairs && !p.combine_enabled && a.k % 8 == 0 && sm_count() >= 2)
    return launch_grouped_gemm_pair(ta, tb, p, a.b_major, grid, stream);
  if (p.dispatch_enabled) {
    if (a.b_major == HMC_MAJOR_MN)
      return launch<HMC_MAJOR_K, HMC_MAJOR_MN, SINGLE_DISPATCH_WARPS>(ta, tb, tc, p, grid, stream);
    return launch<HMC_MAJOR_K, HMC_MAJOR_K, SINGLE_DISPATCH_WARPS>(ta, tb, tc, p, grid, stream);
  }
  if (a.b_major == HMC_MAJOR_MN) return launch<HMC_MAJOR_K, HMC_MAJOR_MN>(ta, tb, tc, p, grid, stream);
  return launch<HMC_MAJOR_K, HMC_MAJOR_K>(ta, tb, tc, p, grid, stream);
}
