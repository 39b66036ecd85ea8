// Persistent grouped GEMM on MXFP8 operands: E4M3 data with one UE8M0 scale per 32 elements of
// the contraction axis, tcgen05.mma kind::mxf8f6f4.block_scale, FP32 accumulators in TMEM.
//
// Replaces the reference's MX GMM worker (hyper_multicore/ops/common/mega_moe/adapters/arch35/
// gmm/mxfp8_worker.h:15-159; layouts NN forward, NT for dA / dX, TN for dW: tasks/gmm_mxfp8.py).
//
// Same skeleton as the BF16 kernel: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner,
// warps 2..9 = epilogue. Tiles are 128 x 128 x 128 (bytes == elements for FP8); each pipeline
// stage carries the two operand tiles plus one 512-byte scale-factor atom per operand, which the
// MMA thread copies into TMEM (tcgen05.cp) right before the four K=32 instructions that use it.
// Activation rows live in the padded expert-major layout (every group starts on a 128-row
// block, padding rows are zero), so no tile, scale block or atom straddles two experts and the
// ragged contraction of the weight-gradient GEMM needs no masking.
#include <cuda.h>

#include "common.cuh"
#include "mx_gemm_shared.cuh"
#include "sm100.cuh"

namespace hmc {
namespace {

using namespace sm100;
using namespace mx;

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int STAGES = 5;
constexpr int ACC_STAGES = 2;
constexpr int STAGE_BYTES = 2 * TILE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_WARPS * STORE_STAGE_BYTES + STAGES * 2 * ATOM_BYTES + 1024 + 256;
constexpr uint32_t TMEM_SFA_COL = ACC_STAGES * BN;  // 4 columns
constexpr uint32_t TMEM_SFB_COL = TMEM_SFA_COL + 4;
using TileWalker = TileWalkerT<1>;

template <int A_MAJOR, int B_MAJOR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
               const __grid_constant__ CUtensorMap tm_c, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* store_stage = smem + STAGES * STAGE_BYTES;
  uint8_t* sf_stage = store_stage + EPI_WARPS * STORE_STAGE_BYTES;  // [STAGES][2][ATOM_BYTES]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sf_stage + STAGES * 2 * ATOM_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* acc_full_bar = bars + 2 * STAGES;
  uint64_t* acc_empty_bar = bars + 2 * STAGES + ACC_STAGES;
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
      mbar_init(&acc_empty_bar[s], EPI_WARPS);
    }
    *abort_word = 0;
    mbar_fence_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
    if (p.mode == HMC_GEMM_RAGGED_K) prefetch_tensormap(&tm_c);
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
    // ======================================================================== producer
    if (lane == 0) {
      TileWalker walker(p);
      Tile t;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long idx = blockIdx.x; ok && walker.get(idx, t); idx += gridDim.x) {
        const int kiters = k_iterations(p, t);
        for (int kb = 0; kb < kiters; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_word, PIPE_BUDGET_NS)) {
            report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 0, stage, kb);
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + stage * STAGE_BYTES;
          uint8_t* b_dst = a_dst + TILE_BYTES;
          uint8_t* sfa_dst = sf_stage + stage * 2 * ATOM_BYTES;
          uint8_t* sfb_dst = sfa_dst + ATOM_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES + 2 * ATOM_BYTES);
          if (p.mode == HMC_GEMM_RAGGED_M) {
            const int pad_block = t.pad_block0 + t.m_idx;
            tma_load_2d(a_dst, &tm_a, &full_bar[stage], kb * BK, pad_block * 128);
            if (B_MAJOR == HMC_MAJOR_MN) tma_load_3d(b_dst, &tm_b, &full_bar[stage], t.n_idx * BN, kb * BK, t.group);
            else tma_load_3d(b_dst, &tm_b, &full_bar[stage], kb * BK, t.n_idx * BN, t.group);
            bulk_load(sfa_dst, p.a_scale + (static_cast<long long>(kb) * p.pad_blocks + pad_block) * ATOM_BYTES,
                      ATOM_BYTES, &full_bar[stage]);
            bulk_load(sfb_dst,
                      p.b_scale + ((static_cast<long long>(t.group) * p.k_blocks + kb) * p.n_tiles + t.n_idx) * ATOM_BYTES,
                      ATOM_BYTES, &full_bar[stage]);
          } else {
            const int pad_block = t.pad_block0 + kb;
            tma_load_2d(a_dst, &tm_a, &full_bar[stage], t.m_idx * BM, pad_block * 128);
            tma_load_2d(b_dst, &tm_b, &full_bar[stage], t.n_idx * BN, pad_block * 128);
            bulk_load(sfa_dst, p.a_scale + (static_cast<long long>(pad_block) * p.m_tiles + t.m_idx) * ATOM_BYTES,
                      ATOM_BYTES, &full_bar[stage]);
            bulk_load(sfb_dst, p.b_scale + (static_cast<long long>(pad_block) * p.n_tiles + t.n_idx) * ATOM_BYTES,
                      ATOM_BYTES, &full_bar[stage]);
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
    // K-major: a K=32 step is 32 bytes along the 128-byte row. MN-major: 32 k-rows of 128 bytes.
    constexpr uint32_t A_KSTEP = A_MAJOR == HMC_MAJOR_MN ? (32 * 128) >> 4 : 32 >> 4;
    constexpr uint32_t B_KSTEP = B_MAJOR == HMC_MAJOR_MN ? (32 * 128) >> 4 : 32 >> 4;
    const uint32_t tmem_sfa = tmem_base + TMEM_SFA_COL;
    const uint32_t tmem_sfb = tmem_base + TMEM_SFB_COL;
    for (long long idx = blockIdx.x; ok && walker.get(idx, t); idx += gridDim.x) {
      const int kiters = k_iterations(p, t);
      if (kiters == 0) continue;
      if (!mbar_wait(&acc_empty_bar[acc], acc_phase ^ 1u, abort_word, PIPE_BUDGET_NS)) {
        if (lane == 0) report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 1, acc, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
      for (int kb = 0; kb < kiters; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase, abort_word, PIPE_BUDGET_NS)) {
          if (lane == 0) report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 2, stage, kb);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (lane == 0) {
          uint8_t* a_src = smem + stage * STAGE_BYTES;
          uint8_t* b_src = a_src + TILE_BYTES;
          uint8_t* sfa_src = sf_stage + stage * 2 * ATOM_BYTES;
          // scale atoms: un-swizzled, 8-row groups of 16 bytes are 128 bytes apart
          tmem_cp_sf(tmem_sfa, make_smem_desc(smem_u32(sfa_src), 0, 128, 0));
          tmem_cp_sf(tmem_sfb, make_smem_desc(smem_u32(sfa_src + ATOM_BYTES), 0, 128, 0));
          uint64_t da = make_smem_desc(smem_u32(a_src), A_MAJOR == HMC_MAJOR_MN ? TILE_BYTES : 16, 1024, SWIZZLE_128B);
          uint64_t db = make_smem_desc(smem_u32(b_src), B_MAJOR == HMC_MAJOR_MN ? TILE_BYTES : 16, 1024, SWIZZLE_128B);
#pragma unroll
          for (int ks = 0; ks < BK / 32; ++ks) {
            umma_mxf8(tmem_d, da, db, make_idesc_mxf8(BM, BN, A_MAJOR, B_MAJOR, ks), tmem_sfa, tmem_sfb,
                      (kb > 0 || ks > 0) ? 1u : 0u);
            da += A_KSTEP;
            db += B_KSTEP;
          }
          umma_commit(&empty_bar[stage]);
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
  } else {
    // ======================================================================== epilogue
    TileWalker walker(p);
    Tile t;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int c_lo = half * (BN / 2);
    const int c_hi = c_lo + BN / 2;
    const int row_in_tile = quarter * 32 + lane;
    uint8_t* my_stage = store_stage + (warp - 2) * STORE_STAGE_BYTES;
    bool store_pending = false;
    for (long long idx = blockIdx.x; ok && walker.get(idx, t); idx += gridDim.x) {
      const int kiters = k_iterations(p, t);
      const int col_base = t.n_idx * BN;
      if (kiters == 0) {
        // cold group of a weight-gradient GEMM: exact zeros
        const int m = t.m_idx * BM + row_in_tile;
        if (m < p.m) {
          const long long out_row = static_cast<long long>(t.group) * p.m + m;
          if (p.epilogue == HMC_EPI_STORE_F32) {
            float* dst = static_cast<float*>(p.c) + out_row * p.n + col_base;
            for (int c = c_lo; c < c_hi && col_base + c < p.n; c += 4)
              *reinterpret_cast<float4*>(dst + c) = make_float4(0.f, 0.f, 0.f, 0.f);
          } else {
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.c) + out_row * p.n + col_base;
            for (int c = c_lo; c < c_hi && col_base + c < p.n; c += 8)
              *reinterpret_cast<uint4*>(dst + c) = make_uint4(0, 0, 0, 0);
          }
        }
        continue;
      }
      if (!mbar_wait(&acc_full_bar[acc], acc_phase, abort_word, PIPE_BUDGET_NS)) {
        if (lane == 0) report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 3, acc, 0);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
      if (p.mode == HMC_GEMM_RAGGED_K) {
        const bool f32 = p.epilogue == HMC_EPI_STORE_F32;
        const int step = f32 ? 32 : 64;
        const int m0 = t.m_idx * BM + quarter * 32;
#pragma unroll 1
        for (int c = c_lo; c < c_hi; c += step) {
          if (col_base + c >= p.n) break;
          uint32_t v[32];
          uint32_t w[32];
          tmem_ld_32x32(taddr + c, v);
          if (!f32) tmem_ld_32x32(taddr + c + 32, w);
          tmem_ld_wait();
          if (store_pending) {
            if (lane == 0) bulk_wait_read_all();
            __syncwarp();
          }
          uint8_t* row_base = my_stage + lane * 128;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            uint4 o;
            if (f32) {
              o = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            } else {
              const uint32_t* src = q < 4 ? v + 8 * q : w + 8 * (q - 4);
              o.x = pack_bf16x2(__uint_as_float(src[0]), __uint_as_float(src[1]));
              o.y = pack_bf16x2(__uint_as_float(src[2]), __uint_as_float(src[3]));
              o.z = pack_bf16x2(__uint_as_float(src[4]), __uint_as_float(src[5]));
              o.w = pack_bf16x2(__uint_as_float(src[6]), __uint_as_float(src[7]));
            }
            *reinterpret_cast<uint4*>(row_base + ((q ^ (lane & 7)) << 4)) = o;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&tm_c, my_stage, col_base + c, m0, t.group);
            bulk_commit_group();
          }
          store_pending = true;
        }
      } else {
        // Rows are written in the un-padded layout (rows of the tile past the group's end are padding),
        // either into c or - fused combine - into the routed buffers of their source ranks. Each lane
        // finds the destination of its own row; the 32 x 64-column piece is staged in shared memory so
        // that every store instruction writes whole 128-byte pieces of four rows.
        const long long out_row = t.row0 + static_cast<long long>(t.m_idx) * BM + row_in_tile;
        int source = -1;
        const unsigned long long dst_bits = mx_row_destination(p, t, out_row, col_base, source);
        if (store_pending) {  // an earlier weight-gradient tile may still be reading the stage
          if (lane == 0) bulk_wait_read_all();
          __syncwarp();
          store_pending = false;
        }
        {
          const int c = c_lo;  // one 64-column step per warp
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
          const int sub = lane >> 3;
          const int piece = lane & 7;
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const int r = i + sub;
            const unsigned long long base = __shfl_sync(0xffffffffu, dst_bits, r);
            if (base != 0) {
              const uint4 val = *reinterpret_cast<const uint4*>(my_stage + r * 128 + ((piece ^ (r & 7)) << 4));
              st_16(reinterpret_cast<uint8_t*>(base) + c * 2 + piece * 16, val);
            }
          }
          __syncwarp();
        }
        if (p.combine_enabled) {
          // one release-add per destination per warp; the warp barrier above orders the lanes' stores
          const unsigned same = __match_any_sync(0xffffffffu, source);
          if (source >= 0 && lane == __ffs(same) - 1)
            red_release_sys_add(p.combine.peer_ctrl[source] + HMC_CTRL_COMBINE, __popc(same));
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty_bar[acc]);
      if (++acc == ACC_STAGES) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (store_pending && lane == 0) bulk_wait_all();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ----------------------------------------------------------------------------- host side
template <int A_MAJOR, int B_MAJOR>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const Params& p, int grid,
           cudaStream_t stream) {
  static PerDeviceFlag configured{};
  auto kernel = mx_gemm_kernel<A_MAJOR, B_MAJOR>;
  if (int rc = allow_dynamic_smem(kernel, SMEM_BYTES, configured)) return rc;
  kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, tc, p);
  HMC_LAUNCH_OK();
  return 0;
}

}  // namespace
}  // namespace hmc

extern "C" int64_t hmc_mx_gemm_combine_units(int64_t n) {
  // every (32-row, half-tile) piece of every 128-column tile reports its rows once
  return 2 * ((n + 127) / 128);
}

extern "C" int hmc_mx_gemm(const hmc_mx_gemm_args* args, void* stream_ptr) {
  using namespace hmc;
  using namespace hmc::mx;
  HMC_REQUIRE(args != nullptr, HMC_ERR_INVALID, "hmc_mx_gemm: null args");
  const hmc_mx_gemm_args& a = *args;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  ProfileScope profile(HMC_PROFILE_MX_GEMM, stream);
  HMC_REQUIRE(a.mode == HMC_GEMM_RAGGED_M || a.mode == HMC_GEMM_RAGGED_K, HMC_ERR_INVALID,
              "hmc_mx_gemm: unknown mode %d", a.mode);
  HMC_REQUIRE(a.groups > 0 && a.rows >= 0 && a.pad_blocks > 0, HMC_ERR_INVALID,
              "hmc_mx_gemm: groups and pad_blocks must be positive, rows non-negative");
  HMC_REQUIRE(a.pad_blocks >= (a.rows + 127) / 128 && a.pad_blocks * 128 < (1ll << 31), HMC_ERR_INVALID,
              "hmc_mx_gemm: pad_blocks (%lld) cannot hold %lld rows", (long long)a.pad_blocks, (long long)a.rows);
  HMC_REQUIRE(a.a && a.b && (a.c || a.combine || a.epilogue == HMC_EPI_SWIGLU_GRAD_MXQ) && a.a_scale && a.b_scale &&
                  a.group_ends,
              HMC_ERR_INVALID,
              "hmc_mx_gemm: null tensor pointer");
  HMC_REQUIRE(aligned16(a.a) && aligned16(a.b) && aligned16(a.c) && aligned16(a.a_scale) && aligned16(a.b_scale),
              HMC_ERR_INVALID, "hmc_mx_gemm: tensors must be 16-byte aligned");
  HMC_REQUIRE(a.n > 0 && a.n % 128 == 0 && a.n < (1ll << 31), HMC_ERR_LIMIT,
              "hmc_mx_gemm: n (%lld) must be a positive multiple of 128", (long long)a.n);
  if (a.rows == 0 && a.mode == HMC_GEMM_RAGGED_M) return 0;

  Params p{};
  p.mode = a.mode;
  p.epilogue = a.epilogue;
  p.groups = a.groups;
  p.rows = a.rows;
  p.pad_blocks = static_cast<int>(a.pad_blocks);
  p.group_ends = reinterpret_cast<const long long*>(a.group_ends);
  p.a_scale = static_cast<const uint8_t*>(a.a_scale);
  p.b_scale = static_cast<const uint8_t*>(a.b_scale);
  p.c = a.c;
  p.status = a.status;
  p.skip_flag = a.skip_flag;
  p.n = static_cast<int>(a.n);
  p.n_tiles = static_cast<int>(a.n / BN);
  p.n_atoms = p.n_tiles;
  HMC_REQUIRE(a.tile_mode == HMC_TILE_AUTO || a.tile_mode == HMC_TILE_SINGLE || a.tile_mode == HMC_TILE_PAIR, HMC_ERR_INVALID,
              "hmc_mx_gemm: unknown tile_mode %d", a.tile_mode);
  // CTA pairs work on 256 x 256 tiles: twice the flops per operand byte brought into shared memory.
  const bool pair_shape = a.n % 256 == 0 && (a.mode == HMC_GEMM_RAGGED_M || a.m % 256 == 0) && sm_count() >= 2;
  HMC_REQUIRE(a.tile_mode != HMC_TILE_PAIR || pair_shape, HMC_ERR_LIMIT,
              "hmc_mx_gemm: CTA-pair tiles need n (and m for RAGGED_K) to be multiples of 256");
  const bool use_pairs = pair_shape && a.tile_mode != HMC_TILE_SINGLE;
  if (a.combine != nullptr) {
    const hmc_gemm_combine& cb = *a.combine;
    HMC_REQUIRE(a.mode == HMC_GEMM_RAGGED_M, HMC_ERR_INVALID, "hmc_mx_gemm: the fused combine belongs to RAGGED_M GEMMs");
    HMC_REQUIRE(cb.ep >= 1 && cb.ep <= HMC_MAX_EP && cb.local_experts == a.groups, HMC_ERR_INVALID,
                "hmc_mx_gemm: combine needs 1 <= ep <= %d and local_experts == groups", HMC_MAX_EP);
    HMC_REQUIRE(cb.segment_start && cb.combine_target_off && cb.peer_buffers && cb.peer_ctrl && cb.target_rows_limit > 0,
                HMC_ERR_INVALID, "hmc_mx_gemm: null combine table");
    for (int r = 0; r < cb.ep; ++r) {
      HMC_REQUIRE(cb.peer_buffers[r] != nullptr && cb.peer_ctrl[r] != nullptr && aligned16(cb.peer_buffers[r]),
                  HMC_ERR_INVALID, "hmc_mx_gemm: peer %d has no 16-byte aligned routed buffer / control block", r);
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
  const cuuint64_t pad_rows = static_cast<cuuint64_t>(a.pad_blocks) * 128;

  CUtensorMap ta, tb, tc;
  int rc;
  if (a.mode == HMC_GEMM_RAGGED_M) {
    const bool fused = a.epilogue == HMC_EPI_SWIGLU_MXQ || a.epilogue == HMC_EPI_SWIGLU_GRAD_MXQ;
    HMC_REQUIRE(a.epilogue == HMC_EPI_STORE_BF16 || fused, HMC_ERR_INVALID,
                "hmc_mx_gemm: RAGGED_M writes BF16 rows (optionally with a quantised SwiGLU / SwiGLU-grad beside them)");
    if (fused) {
      const bool grad = a.epilogue == HMC_EPI_SWIGLU_GRAD_MXQ;
      HMC_REQUIRE(use_pairs && a.b_major == (grad ? HMC_MAJOR_K : HMC_MAJOR_MN) && a.combine == nullptr, HMC_ERR_INVALID,
                  "hmc_mx_gemm: a quantising epilogue needs CTA-pair tiles (n %% 256 == 0), an %s weight and no fused combine",
                  grad ? "K-major" : "MN-major");
      HMC_REQUIRE(grad ? (a.aux != nullptr && aligned16(a.aux)) : a.c != nullptr, HMC_ERR_INVALID,
                  "hmc_mx_gemm: the SwiGLU epilogue writes U into c; the SwiGLU-grad epilogue reads U from aux");
      HMC_REQUIRE(a.act_row_data && a.act_row_scale && (a.act_col_data == nullptr) == (a.act_col_scale == nullptr) &&
                      aligned16(a.act_row_data) && aligned16(a.act_col_data),
                  HMC_ERR_INVALID,
                  "hmc_mx_gemm: a quantising epilogue needs its 16-byte aligned row outputs (the column pair is optional)");
      p.act_row_data = static_cast<uint8_t*>(a.act_row_data);
      p.act_row_scale = static_cast<uint8_t*>(a.act_row_scale);
      p.act_col_data = static_cast<uint8_t*>(a.act_col_data);
      p.act_col_scale = static_cast<uint8_t*>(a.act_col_scale);
      p.aux = a.aux;
    }
    HMC_REQUIRE(a.k > 0 && a.k % 128 == 0 && a.k < (1ll << 31), HMC_ERR_LIMIT,
                "hmc_mx_gemm: k (%lld) must be a positive multiple of 128", (long long)a.k);
    p.k = static_cast<int>(a.k);
    p.k_blocks = static_cast<int>(a.k / BK);
    {
      cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.k), pad_rows};
      cuuint32_t box[2] = {128, 128};
      if ((rc = make_map(&ta, a.a, 2, dims, box, 1)) != 0) return rc;
    }
    if (a.b_major == HMC_MAJOR_MN) {
      cuuint64_t dims[3] = {static_cast<cuuint64_t>(a.n), static_cast<cuuint64_t>(a.k), static_cast<cuuint64_t>(a.groups)};
      cuuint32_t box[3] = {128, 128, 1};
      if ((rc = make_map(&tb, a.b, 3, dims, box, 1)) != 0) return rc;
    } else {
      cuuint64_t dims[3] = {static_cast<cuuint64_t>(a.k), static_cast<cuuint64_t>(a.n), static_cast<cuuint64_t>(a.groups)};
      cuuint32_t box[3] = {128, 128, 1};
      if ((rc = make_map(&tb, a.b, 3, dims, box, 1)) != 0) return rc;
    }
    tc = ta;
  } else {
    HMC_REQUIRE(a.epilogue == HMC_EPI_STORE_BF16 || a.epilogue == HMC_EPI_STORE_F32, HMC_ERR_INVALID,
                "hmc_mx_gemm: RAGGED_K supports plain stores only");
    HMC_REQUIRE(a.m > 0 && a.m % 128 == 0 && a.m < (1ll << 31), HMC_ERR_LIMIT,
                "hmc_mx_gemm: m (%lld) must be a positive multiple of 128", (long long)a.m);
    p.m = static_cast<int>(a.m);
    p.m_tiles = static_cast<int>(a.m / BM);
    p.m_atoms = p.m_tiles;
    {
      cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.m), pad_rows};
      cuuint32_t box[2] = {128, 128};
      if ((rc = make_map(&ta, a.a, 2, dims, box, 1)) != 0) return rc;
    }
    {
      cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.n), pad_rows};
      cuuint32_t box[2] = {128, 128};
      if ((rc = make_map(&tb, a.b, 2, dims, box, 1)) != 0) return rc;
    }
    {
      const bool f32 = a.epilogue == HMC_EPI_STORE_F32;
      cuuint64_t dims[3] = {static_cast<cuuint64_t>(a.n), static_cast<cuuint64_t>(a.m), static_cast<cuuint64_t>(a.groups)};
      cuuint32_t box[3] = {f32 ? 32u : 64u, 32, 1};
      if ((rc = make_map(&tc, a.c, 3, dims, box, f32 ? 4 : 2)) != 0) return rc;
    }
  }
  int grid = a.max_ctas > 0 ? a.max_ctas : sm_count();
  if (grid > sm_count()) grid = sm_count();
  if (use_pairs) {
    CUtensorMap tsa, tsb;
    const long long a_atoms = a.mode == HMC_GEMM_RAGGED_M ? static_cast<long long>(p.k_blocks) * p.pad_blocks
                                                          : static_cast<long long>(p.pad_blocks) * p.m_atoms;
    const long long b_atoms = a.mode == HMC_GEMM_RAGGED_M ? static_cast<long long>(p.groups) * p.k_blocks * p.n_atoms
                                                          : static_cast<long long>(p.pad_blocks) * p.n_atoms;
    if ((rc = make_atom_map(&tsa, a.a_scale, a_atoms, 1)) != 0) return rc;
    if ((rc = make_atom_map(&tsb, a.b_scale, b_atoms, a.epilogue == HMC_EPI_SWIGLU_MXQ ? 1 : 2)) != 0) return rc;
    p.n_tiles = p.n_atoms / 2;
    p.m_tiles = p.m_atoms / 2;
    const int a_major = a.mode == HMC_GEMM_RAGGED_K ? HMC_MAJOR_MN : HMC_MAJOR_K;
    const int b_major = a.mode == HMC_GEMM_RAGGED_K ? HMC_MAJOR_MN : a.b_major;
    return launch_mx_gemm_pair(ta, tb, tc, tsa, tsb, p, a_major, b_major, grid, stream);
  }
  if (a.mode == HMC_GEMM_RAGGED_K) {
    const long long tiles = static_cast<long long>(p.groups) * p.m_tiles * p.n_tiles;
    if (tiles < grid) grid = static_cast<int>(tiles);
    return launch<HMC_MAJOR_MN, HMC_MAJOR_MN>(ta, tb, tc, p, grid, stream);
  }
  if (a.b_major == HMC_MAJOR_MN) return launch<HMC_MAJOR_K, HMC_MAJOR_MN>(ta, tb, tc, p, grid, stream);
  return launch<HMC_MAJOR_K, HMC_MAJOR_K>(ta, tb, tc, p, grid, stream);
}
