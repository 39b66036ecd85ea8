// CTA-pair variant of the block-scaled FP8 grouped GEMM: two CTAs of a cluster share one 256 x 256 tile
// (tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale, M = 256, N = 256, K = 32 per instruction).
//
// Per 128-element k-block each CTA brings 16 KiB of A (its own 128 rows), 16 KiB of B (its own 128 of the
// tile's 256 columns), the scale atom of its A rows and the two atoms of all 256 B columns into shared
// memory: half the operand bytes per flop of the 128 x 128 one-CTA kernel, whose tensor pipe idles two
// thirds of the time behind the L2 -> shared-memory stream.
//
// The 256 accumulator columns plus the scale columns leave no room for a second accumulator in the 512
// columns of tensor memory. The epilogue therefore drains the whole accumulator into registers first
// (128 values per thread), hands the tensor memory back to the MMA issuer, and only then converts and
// stores, so the next tile's MMAs overlap the stores.
//
// Roles as in the other pair kernels: warp 0 = TMA producer (both CTAs), warp 1 = MMA issuer (leader) and
// TMEM owner, warps 2..9 = epilogue (both CTAs, each on its own 128 accumulator rows).
//
// Two epilogues quantise their own result (template argument FUSED), bit-identical to the stand-alone quantiser
// run on the stored result: 1 = GMM1, where the leader loads gate columns and the second CTA the up columns of
// the same activation columns, U leaves as BF16 and bf16(silu(gate) * up) leaves as E4M3 along both axes; 2 = the
// dA GEMM, which reads the saved U and emits the quantised dU = [dgate | dup] (correct, but slower than the
// separate quantiser launch: the operator keeps it off).
//
// Replaces the reference's MX GMM worker (hyper_multicore/ops/common/mega_moe/adapters/arch35/gmm/
// mxfp8_worker.h:15-159; layouts NN forward, NT for dA / dX, TN for dW: tasks/gmm_mxfp8.py).
#include <cuda.h>

#include "common.cuh"
#include "mx_gemm_shared.cuh"
#include "mx_quant_shared.cuh"
#include "sm100.cuh"

namespace hmc {
namespace mx {
namespace {

using namespace sm100;

constexpr int PAIR_N = 256;
constexpr int PAIR_STAGES = 5;
constexpr int PAIR_DATA_BYTES = 2 * TILE_BYTES;  // this CTA's A rows and B columns of one k-block
constexpr int PAIR_SF_BYTES = 3 * ATOM_BYTES;    // scale atoms: own A rows, then both halves of B
constexpr int PAIR_SMEM_BYTES =
    PAIR_STAGES * PAIR_DATA_BYTES + EPI_WARPS * STORE_STAGE_BYTES + PAIR_STAGES * PAIR_SF_BYTES + 1024 + 256;
// Tensor memory: accumulator in columns [0, 256); four rotating 16-column scale slots behind it
// (A scales in the first 4 columns of a slot, B scales in its last 8).
constexpr uint32_t TMEM_SF_COL = PAIR_N;
constexpr uint32_t SF_SLOT_COLS = 16;
constexpr int SF_SLOTS = 4;
using PairWalker = TileWalkerT<2>;

// Where one warp's quantised values go: row r_in_block of padded block pb, in a [pad_rows, width] tensor pair
// (row-quantised, and optionally column-quantised) with their scale atoms.
struct QuantOut {
  uint8_t* row_data;
  uint8_t* row_scale;
  uint8_t* col_data;   // nullptr: no column-quantised copy
  uint8_t* col_scale;
  int width;
  int pad_blocks;
  int pb;
  int r_in_block;      // this thread's row of the 128-row block: 32 * quarter + lane
};

// Quantises 32 BF16-exact values of this thread's row, columns [col, col + 32) (col a multiple of 32), along the
// row (one scale for the 32 values: thread-local) and down the rows (one scale per column for the 32 rows the
// warp's lanes hold), exactly as mx_quant_kernel does from a tile in memory. The 32 column maxima come from a
// transpose-reduce over the warp (31 shuffles: at every step a lane hands the half of its columns it does not
// keep to the lane `half` away, so lane L ends with the maximum of column L); the 32 exponents then go round
// through 32 bytes of the warp's shared-memory stage.
__device__ __forceinline__ void quantise_chunk(const float (&a)[32], const QuantOut& o, int col, int lane, uint8_t* scratch) {
  const long long pad_row = static_cast<long long>(o.pb) * 128 + o.r_in_block;
  const int cb = col >> 7;           // 128-column block
  const int kk = (col & 127) >> 5;   // 32-column block inside it
  float amax = 0.f;
#pragma unroll
  for (int c = 0; c < 32; ++c) amax = fmaxf(amax, fabsf(a[c]));
  const uint32_t e_row = mxq::block_exponent(amax);
  const float inv_row = mxq::inverse_scale(e_row);
  uint32_t q_row[8];
#pragma unroll
  for (int c = 0; c < 32; c += 4)
    q_row[c >> 2] = mxq::e4m3x2(a[c] * inv_row, a[c + 1] * inv_row) | (mxq::e4m3x2(a[c + 2] * inv_row, a[c + 3] * inv_row) << 16);
  uint8_t* row_dst = o.row_data + pad_row * o.width + col;
  st_16(row_dst, make_uint4(q_row[0], q_row[1], q_row[2], q_row[3]));
  st_16(row_dst + 16, make_uint4(q_row[4], q_row[5], q_row[6], q_row[7]));
  o.row_scale[(static_cast<long long>(cb) * o.pad_blocks + o.pb) * ATOM_BYTES + mxq::atom_offset(o.r_in_block, kk)] =
      static_cast<uint8_t>(e_row);
  if (o.col_data == nullptr) return;

  uint32_t m[32];  // |a| as integers: the order of non-negative floats
#pragma unroll
  for (int c = 0; c < 32; ++c) m[c] = __float_as_uint(fabsf(a[c]));
#pragma unroll
  for (int half = 16; half >= 1; half >>= 1) {
    const bool upper = (lane & half) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const uint32_t send = upper ? m[i] : m[i + half];
      const uint32_t keep = upper ? m[i + half] : m[i];
      m[i] = max(keep, __shfl_xor_sync(0xffffffffu, send, half));
    }
  }
  const uint32_t e_mine = mxq::block_exponent(__uint_as_float(m[0]));  // scale of column `lane`
  __syncwarp();
  scratch[lane] = static_cast<uint8_t>(e_mine);
  __syncwarp();
  const uint4 e_lo = *reinterpret_cast<const uint4*>(scratch);
  const uint4 e_hi = *reinterpret_cast<const uint4*>(scratch + 16);
  const uint32_t e_words[8] = {e_lo.x, e_lo.y, e_lo.z, e_lo.w, e_hi.x, e_hi.y, e_hi.z, e_hi.w};
  uint32_t q_col[8];
#pragma unroll
  for (int c = 0; c < 32; c += 4) {
    const uint32_t e4 = e_words[c >> 2];
    const float i0 = mxq::inverse_scale(e4 & 0xffu), i1 = mxq::inverse_scale((e4 >> 8) & 0xffu);
    const float i2 = mxq::inverse_scale((e4 >> 16) & 0xffu), i3 = mxq::inverse_scale(e4 >> 24);
    q_col[c >> 2] = mxq::e4m3x2(a[c] * i0, a[c + 1] * i1) | (mxq::e4m3x2(a[c + 2] * i2, a[c + 3] * i3) << 16);
  }
  uint8_t* col_dst = o.col_data + pad_row * o.width + col;
  st_16(col_dst, make_uint4(q_col[0], q_col[1], q_col[2], q_col[3]));
  st_16(col_dst + 16, make_uint4(q_col[4], q_col[5], q_col[6], q_col[7]));
  o.col_scale[(static_cast<long long>(o.pb) * (o.width / 128) + cb) * ATOM_BYTES +
              mxq::atom_offset((col & 127) + lane, o.r_in_block >> 5)] = static_cast<uint8_t>(e_mine);
}

template <int A_MAJOR, int B_MAJOR, int FUSED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
mx_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ CUtensorMap tm_c, const __grid_constant__ CUtensorMap tm_sa,
                    const __grid_constant__ CUtensorMap tm_sb, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* store_stage = smem + PAIR_STAGES * PAIR_DATA_BYTES;
  uint8_t* sf_stage = store_stage + EPI_WARPS * STORE_STAGE_BYTES;  // [PAIR_STAGES][3][ATOM_BYTES]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sf_stage + PAIR_STAGES * PAIR_SF_BYTES);
  uint64_t* full_bar = bars;                      // leader only: loads of both CTAs
  uint64_t* empty_bar = bars + PAIR_STAGES;       // one set per CTA
  uint64_t* acc_full_bar = bars + 2 * PAIR_STAGES;      // one per CTA
  uint64_t* acc_empty_bar = bars + 2 * PAIR_STAGES + 1;  // leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * PAIR_STAGES + 2);
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
    mbar_init(acc_full_bar, 1);
    mbar_init(acc_empty_bar, 2 * EPI_WARPS);  // every epilogue warp of both CTAs
    *abort_word = 0;
    mbar_fence_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
    prefetch_tensormap(&tm_sa);
    prefetch_tensormap(&tm_sb);
    if (p.mode == HMC_GEMM_RAGGED_K) prefetch_tensormap(&tm_c);
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
      PairWalker walker(p);
      Tile t;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long idx = pair; ok && walker.get(idx, t); idx += pairs) {
        const int kiters = k_iterations(p, t);
        // RAGGED_M: this CTA's 128-row block of the tile. The second CTA of a group's last, half-empty tile
        // repeats the group's last block; its rows lie past the group's end and are never stored.
        int block = 2 * t.m_idx + static_cast<int>(rank);
        if (block >= t.blocks) block = t.blocks - 1;
        // this CTA's columns of B; with the fused SwiGLU the leader takes 128 gate columns and the second CTA the
        // 128 up columns of the same activation columns, so that a thread's accumulator row holds both
        constexpr bool swiglu = FUSED == 1;
        const int n0 = swiglu ? static_cast<int>(rank) * (p.n / 2) + t.n_idx * 128 : t.n_idx * PAIR_N + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < kiters; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_word, PIPE_BUDGET_NS)) {
            report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 0, stage, kb);
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + stage * PAIR_DATA_BYTES;
          uint8_t* b_dst = a_dst + TILE_BYTES;
          uint8_t* sfa_dst = sf_stage + stage * PAIR_SF_BYTES;
          uint8_t* sfb_dst = sfa_dst + ATOM_BYTES;
          // the leader's barrier counts the bytes of both CTAs
          if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * (PAIR_DATA_BYTES + PAIR_SF_BYTES));
          if (p.mode == HMC_GEMM_RAGGED_M) {
            const int pad_block = t.pad_block0 + block;
            tma_load_2d_pair(a_dst, &tm_a, &full_bar[stage], kb * BK, pad_block * 128);
            if (B_MAJOR == HMC_MAJOR_MN) tma_load_3d_pair(b_dst, &tm_b, &full_bar[stage], n0, kb * BK, t.group);
            else tma_load_3d_pair(b_dst, &tm_b, &full_bar[stage], kb * BK, n0, t.group);
            tma_load_2d_pair(sfa_dst, &tm_sa, &full_bar[stage], 0, kb * p.pad_blocks + pad_block);
            const int sfb_first = (t.group * p.k_blocks + kb) * p.n_atoms;
            if (swiglu) {  // one-atom boxes: the gate and the up columns' scales lie half a row of atoms apart
              tma_load_2d_pair(sfb_dst, &tm_sb, &full_bar[stage], 0, sfb_first + t.n_idx);
              tma_load_2d_pair(sfb_dst + ATOM_BYTES, &tm_sb, &full_bar[stage], 0, sfb_first + p.n_atoms / 2 + t.n_idx);
            } else {
              tma_load_2d_pair(sfb_dst, &tm_sb, &full_bar[stage], 0, sfb_first + 2 * t.n_idx);
            }
          } else {
            const int pad_block = t.pad_block0 + kb;
            const int m0 = t.m_idx * 256 + static_cast<int>(rank) * 128;
            tma_load_2d_pair(a_dst, &tm_a, &full_bar[stage], m0, pad_block * 128);
            tma_load_2d_pair(b_dst, &tm_b, &full_bar[stage], n0, pad_block * 128);
            tma_load_2d_pair(sfa_dst, &tm_sa, &full_bar[stage], 0, pad_block * p.m_atoms + 2 * t.m_idx + static_cast<int>(rank));
            tma_load_2d_pair(sfb_dst, &tm_sb, &full_bar[stage], 0, pad_block * p.n_atoms + 2 * t.n_idx);
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
      uint32_t acc_phase = 0;
      int sf_slot = 0;
      bool ok = true;
      // K-major: a K=32 step is 32 bytes along the 128-byte row. MN-major: 32 k-rows of 128 bytes.
      constexpr uint32_t A_KSTEP = A_MAJOR == HMC_MAJOR_MN ? (32 * 128) >> 4 : 32 >> 4;
      constexpr uint32_t B_KSTEP = B_MAJOR == HMC_MAJOR_MN ? (32 * 128) >> 4 : 32 >> 4;
      for (long long idx = pair; ok && walker.get(idx, t); idx += pairs) {
        const int kiters = k_iterations(p, t);
        if (kiters == 0) continue;  // cold group: the epilogue writes zeros on its own
        if (!mbar_wait(acc_empty_bar, acc_phase ^ 1u, abort_word, PIPE_BUDGET_NS)) {
          if (lane == 0) report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 1, 0, 0);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        for (int kb = 0; kb < kiters; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_word, PIPE_BUDGET_NS)) {
            if (lane == 0) report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 2, stage, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (lane == 0) {
            uint8_t* a_src = smem + stage * PAIR_DATA_BYTES;
            uint8_t* b_src = a_src + TILE_BYTES;
            uint8_t* sf_src = sf_stage + stage * PAIR_SF_BYTES;
            const uint32_t tmem_sfa = tmem_base + TMEM_SF_COL + static_cast<uint32_t>(sf_slot) * SF_SLOT_COLS;
            const uint32_t tmem_sfb = tmem_sfa + 8;
            // scale atoms: un-swizzled, 8-row groups of 16 bytes are 128 bytes apart
            tmem_cp_sf_pair(tmem_sfa, make_smem_desc(smem_u32(sf_src), 0, 128, 0));
            tmem_cp_sf_pair(tmem_sfb, make_smem_desc(smem_u32(sf_src + ATOM_BYTES), 0, 128, 0));
            tmem_cp_sf_pair(tmem_sfb + 4, make_smem_desc(smem_u32(sf_src + 2 * ATOM_BYTES), 0, 128, 0));
            uint64_t da = make_smem_desc(smem_u32(a_src), A_MAJOR == HMC_MAJOR_MN ? TILE_BYTES : 16, 1024, SWIZZLE_128B);
            uint64_t db = make_smem_desc(smem_u32(b_src), B_MAJOR == HMC_MAJOR_MN ? TILE_BYTES : 16, 1024, SWIZZLE_128B);
#pragma unroll
            for (int ks = 0; ks < BK / 32; ++ks) {
              umma_mxf8_pair(tmem_base, da, db, make_idesc_mxf8(256, PAIR_N, A_MAJOR, B_MAJOR, ks), tmem_sfa, tmem_sfb,
                             (kb > 0 || ks > 0) ? 1u : 0u);
              da += A_KSTEP;
              db += B_KSTEP;
            }
            umma_commit_pair(&empty_bar[stage]);  // frees the slot in both CTAs
            if (kb == kiters - 1) umma_commit_pair(acc_full_bar);
          }
          __syncwarp();
          sf_slot = (sf_slot + 1) & (SF_SLOTS - 1);
          if (++stage == PAIR_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        acc_phase ^= 1u;
      }
    }
  } else {
    // ======================================================================== epilogue (both CTAs)
    PairWalker walker(p);
    Tile t;
    uint32_t acc_phase = 0;
    bool ok = true;
    const int quarter = warp & 3;       // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;   // which 128 of the tile's 256 columns this warp handles
    const int row_in_cta = quarter * 32 + lane;
    uint8_t* my_stage = store_stage + (warp - 2) * STORE_STAGE_BYTES;
    const uint32_t leader_acc_empty = map_to_cta(smem_u32(acc_empty_bar), 0);
    bool store_pending = false;
    for (long long idx = pair; ok && walker.get(idx, t); idx += pairs) {
      const int kiters = k_iterations(p, t);
      const int col_base = t.n_idx * PAIR_N + half * 128;
      if (kiters == 0) {
        // cold group of a weight-gradient GEMM: exact zeros, no accumulator involved
        const int m = t.m_idx * 256 + static_cast<int>(rank) * 128 + row_in_cta;
        if (m < p.m) {
          const long long out_row = static_cast<long long>(t.group) * p.m + m;
          if (p.epilogue == HMC_EPI_STORE_F32) {
            float* dst = static_cast<float*>(p.c) + out_row * p.n + col_base;
            for (int c = 0; c < 128; c += 4) *reinterpret_cast<float4*>(dst + c) = make_float4(0.f, 0.f, 0.f, 0.f);
          } else {
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.c) + out_row * p.n + col_base;
            for (int c = 0; c < 128; c += 8) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0, 0, 0, 0);
          }
        }
        continue;
      }
      if (!mbar_wait(acc_full_bar, acc_phase, abort_word, PIPE_BUDGET_NS)) {
        if (lane == 0) report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 3, 0, 0);
        ok = false;
        break;
      }
      acc_phase ^= 1u;
      tc_fence_after_sync();
      // The warp's 32 rows x 128 columns leave tensor memory in one go; the accumulator is then free again.
      // (with the fused SwiGLU: 64 gate columns and the 64 up columns of the same activation columns)
      constexpr bool swiglu = FUSED == 1;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      const uint32_t first = static_cast<uint32_t>(swiglu ? half * 64 : half * 128);
      const uint32_t second = static_cast<uint32_t>(swiglu ? 128 + half * 64 : half * 128 + 64);
      uint32_t v[4][32];
      tmem_ld_32x32(taddr + first, v[0]);
      tmem_ld_32x32(taddr + first + 32, v[1]);
      tmem_ld_32x32(taddr + second, v[2]);
      tmem_ld_32x32(taddr + second + 32, v[3]);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_acc_empty);  // the MMA issuer lives in the leader

      uint8_t* row_base = my_stage + lane * 128;
      if constexpr (FUSED == 1) {
        // U leaves as BF16 rows; bf16(silu(gate) * up) of the BF16-rounded gate and up leaves quantised along the
        // row (32 columns per scale: thread-local) and down the rows (32 rows per scale: this warp's 32 lanes).
        const int block = 2 * t.m_idx + static_cast<int>(rank);
        if (block < t.blocks) {  // the repeated block of a half-empty tile stores nothing
          const int width = p.n / 2;
          const int pb = t.pad_block0 + block;
          const long long out_row = t.row0 + static_cast<long long>(block) * 128 + row_in_cta;
          const long long pad_row = static_cast<long long>(pb) * 128 + row_in_cta;
          const int acol0 = t.n_idx * 128 + half * 64;  // this warp's activation columns
          const unsigned long long dst_bits =
              out_row < t.row1 ? reinterpret_cast<unsigned long long>(static_cast<__nv_bfloat16*>(p.c) + out_row * p.n + acol0) : 0ull;
          const int sub = lane >> 3;
          const int piece = lane & 7;
#pragma unroll
          for (int j = 0; j < 2; ++j) {  // gate columns, then up columns
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              uint32_t* src = v[2 * j + (q >> 2)] + 8 * (q & 3);
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(src[0]), __uint_as_float(src[1]));
              o.y = pack_bf16x2(__uint_as_float(src[2]), __uint_as_float(src[3]));
              o.z = pack_bf16x2(__uint_as_float(src[4]), __uint_as_float(src[5]));
              o.w = pack_bf16x2(__uint_as_float(src[6]), __uint_as_float(src[7]));
              *reinterpret_cast<uint4*>(row_base + ((q ^ (lane & 7)) << 4)) = o;
              // keep the BF16-rounded values: they are what a later reader of U would see
              const uint32_t words[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                const float2 f = unpack_bf16x2(words[w]);
                src[2 * w] = __float_as_uint(f.x);
                src[2 * w + 1] = __float_as_uint(f.y);
              }
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const int r = i + sub;
              const unsigned long long base = __shfl_sync(0xffffffffu, dst_bits, r);
              if (base != 0) {
                const uint4 val = *reinterpret_cast<const uint4*>(my_stage + r * 128 + ((piece ^ (r & 7)) << 4));
                st_16(reinterpret_cast<uint8_t*>(base) + static_cast<long long>(j) * width * 2 + piece * 16, val);
              }
            }
            __syncwarp();
          }
#pragma unroll
          for (int b = 0; b < 2; ++b)
#pragma unroll
            for (int c = 0; c < 32; ++c)
              v[b][c] = __float_as_uint(mxq::swiglu_bf16(__uint_as_float(v[b][c]), __uint_as_float(v[2 + b][c])));
          QuantOut out{p.act_row_data, p.act_row_scale, p.act_col_data, p.act_col_scale, width, p.pad_blocks, pb, row_in_cta};
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            float act[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) act[c] = __uint_as_float(v[b][c]);
            quantise_chunk(act, out, acol0 + 32 * b, lane, my_stage);
          }
        }
      } else if constexpr (FUSED == 2) {
        // acc = dAct. With the saved U = [gate | up] of the same rows: dU = [dgate | dup], rounded to BF16 and
        // quantised along both axes, 32 columns at a time; dAct itself is stored only when the caller wants it.
        const int block = 2 * t.m_idx + static_cast<int>(rank);
        if (block < t.blocks) {
          const int inter = p.n;
          const int pb = t.pad_block0 + block;
          const long long out_row = t.row0 + static_cast<long long>(block) * 128 + row_in_cta;
          const bool row_valid = out_row < t.row1;
          QuantOut out{p.act_row_data, p.act_row_scale, p.act_col_data, p.act_col_scale, 2 * inter, p.pad_blocks, pb, row_in_cta};
          const __nv_bfloat16* u_row = static_cast<const __nv_bfloat16*>(p.aux) + out_row * 2 * inter;
          __nv_bfloat16* da_row = p.c != nullptr ? static_cast<__nv_bfloat16*>(p.c) + out_row * inter : nullptr;
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            const int acol = t.n_idx * PAIR_N + half * 128 + 32 * c4;
            uint4 graw[4], uraw[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              graw[q] = uraw[q] = make_uint4(0, 0, 0, 0);
              if (row_valid) {
                graw[q] = ld_nc_16(u_row + acol + 8 * q);
                uraw[q] = ld_nc_16(u_row + inter + acol + 8 * q);
              }
            }
            float dgate[32], dup[32];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint32_t gw[4] = {graw[q].x, graw[q].y, graw[q].z, graw[q].w};
              const uint32_t uw[4] = {uraw[q].x, uraw[q].y, uraw[q].z, uraw[q].w};
              uint32_t dw[4];
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                const int c = 8 * q + 2 * w;
                dw[w] = pack_bf16x2(__uint_as_float(v[c4][c]), __uint_as_float(v[c4][c + 1]));
                const float2 d = unpack_bf16x2(dw[w]);  // dAct as a reader of the BF16 tensor would see it
                const float2 g = unpack_bf16x2(gw[w]);
                const float2 u = unpack_bf16x2(uw[w]);
                const float s0 = mxq::sigmoid_f(g.x);
                const float s1 = mxq::sigmoid_f(g.y);
                dgate[c] = bf16_round(d.x * u.x * s0 * (1.0f + g.x * (1.0f - s0)));
                dgate[c + 1] = bf16_round(d.y * u.y * s1 * (1.0f + g.y * (1.0f - s1)));
                dup[c] = bf16_round(d.x * (g.x * s0));
                dup[c + 1] = bf16_round(d.y * (g.y * s1));
              }
              if (da_row != nullptr && row_valid) st_16(da_row + acol + 8 * q, make_uint4(dw[0], dw[1], dw[2], dw[3]));
            }
            quantise_chunk(dgate, out, acol, lane, my_stage);
            quantise_chunk(dup, out, inter + acol, lane, my_stage);
          }
        }
      } else if (p.mode == HMC_GEMM_RAGGED_K) {
        const bool f32 = p.epilogue == HMC_EPI_STORE_F32;
        const int m0 = t.m_idx * 256 + static_cast<int>(rank) * 128 + quarter * 32;
        if (f32) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // four boxes of 32 rows x 32 floats
            if (store_pending) {
              if (lane == 0) bulk_wait_read_all();
              __syncwarp();
            }
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<uint4*>(row_base + ((q ^ (lane & 7)) << 4)) =
                  make_uint4(v[j][4 * q], v[j][4 * q + 1], v[j][4 * q + 2], v[j][4 * q + 3]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&tm_c, my_stage, col_base + 32 * j, m0, t.group);
              bulk_commit_group();
            }
            store_pending = true;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 2; ++j) {  // two boxes of 32 rows x 64 bf16
            if (store_pending) {
              if (lane == 0) bulk_wait_read_all();
              __syncwarp();
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const uint32_t* src = v[2 * j + (q >> 2)] + 8 * (q & 3);
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(src[0]), __uint_as_float(src[1]));
              o.y = pack_bf16x2(__uint_as_float(src[2]), __uint_as_float(src[3]));
              o.z = pack_bf16x2(__uint_as_float(src[4]), __uint_as_float(src[5]));
              o.w = pack_bf16x2(__uint_as_float(src[6]), __uint_as_float(src[7]));
              *reinterpret_cast<uint4*>(row_base + ((q ^ (lane & 7)) << 4)) = o;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&tm_c, my_stage, col_base + 64 * j, m0, t.group);
              bulk_commit_group();
            }
            store_pending = true;
          }
        }
      } else {
        // Rows go out in the un-padded layout (rows of the tile past the group's end are padding), into c
        // or - fused combine - into the routed buffers of their source ranks. Each lane finds the
        // destination of its own row; 64-column pieces are staged in shared memory so that every store
        // instruction writes whole 128-byte pieces of four rows.
        const long long out_row =
            t.row0 + (2ll * t.m_idx + static_cast<long long>(rank)) * 128 + row_in_cta;
        int source = -1;
        const unsigned long long dst_bits = mx_row_destination(p, t, out_row, col_base, source);
        if (store_pending) {  // an earlier weight-gradient tile may still be reading the stage
          if (lane == 0) bulk_wait_read_all();
          __syncwarp();
          store_pending = false;
        }
        const int sub = lane >> 3;
        const int piece = lane & 7;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint32_t* src = v[2 * j + (q >> 2)] + 8 * (q & 3);
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(src[0]), __uint_as_float(src[1]));
            o.y = pack_bf16x2(__uint_as_float(src[2]), __uint_as_float(src[3]));
            o.z = pack_bf16x2(__uint_as_float(src[4]), __uint_as_float(src[5]));
            o.w = pack_bf16x2(__uint_as_float(src[6]), __uint_as_float(src[7]));
            *reinterpret_cast<uint4*>(row_base + ((q ^ (lane & 7)) << 4)) = o;
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const int r = i + sub;
            const unsigned long long base = __shfl_sync(0xffffffffu, dst_bits, r);
            if (base != 0) {
              const uint4 val = *reinterpret_cast<const uint4*>(my_stage + r * 128 + ((piece ^ (r & 7)) << 4));
              st_16(reinterpret_cast<uint8_t*>(base) + j * 128 + piece * 16, val);
            }
          }
          __syncwarp();
        }
        if (p.combine_enabled) {
          // One release-add per destination per warp; the warp barrier above orders the lanes' stores. A warp
          // covers 128 columns, which count as two of the 64-column units the receiver waits for.
          const unsigned same = __match_any_sync(0xffffffffu, source);
          if (source >= 0 && lane == __ffs(same) - 1)
            red_release_sys_add(p.combine.peer_ctrl[source] + HMC_CTRL_COMBINE, 2 * __popc(same));
        }
      }
    }
    if (store_pending && lane == 0) bulk_wait_all();  // this thread's stores are in global memory
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

template <int A_MAJOR, int B_MAJOR, int FUSED>
int launch_impl(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tsa,
                const CUtensorMap& tsb, const Params& p, int grid, cudaStream_t stream) {
  static PerDeviceFlag configured{};
  auto kernel = mx_gemm_pair_kernel<A_MAJOR, B_MAJOR, FUSED>;
  if (int rc = allow_dynamic_smem(kernel, PAIR_SMEM_BYTES, configured)) return rc;
  kernel<<<grid, NUM_THREADS, PAIR_SMEM_BYTES, stream>>>(ta, tb, tc, tsa, tsb, p);
  HMC_LAUNCH_OK();
  return 0;
}

}  // namespace

// Called by hmc_mx_gemm when n (and m for RAGGED_K) are multiples of 256. `p.n_tiles` and `p.m_tiles` count
// 256-wide tiles; the scale atoms are still indexed by 128 (`p.n_atoms`, `p.m_atoms`).
int launch_mx_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tsa,
                        const CUtensorMap& tsb, const Params& p, int a_major, int b_major, int grid, cudaStream_t stream) {
  grid &= ~1;  // whole pairs
  if (grid < 2) grid = 2;
  if (p.mode == HMC_GEMM_RAGGED_K) {
    const long long tiles = static_cast<long long>(p.groups) * p.m_tiles * p.n_tiles;
    if (2 * tiles < grid) grid = static_cast<int>(2 * tiles);
    return launch_impl<HMC_MAJOR_MN, HMC_MAJOR_MN, 0>(ta, tb, tc, tsa, tsb, p, grid, stream);
  }
  (void)a_major;
  if (p.epilogue == HMC_EPI_SWIGLU_MXQ) return launch_impl<HMC_MAJOR_K, HMC_MAJOR_MN, 1>(ta, tb, tc, tsa, tsb, p, grid, stream);
  if (p.epilogue == HMC_EPI_SWIGLU_GRAD_MXQ) return launch_impl<HMC_MAJOR_K, HMC_MAJOR_K, 2>(ta, tb, tc, tsa, tsb, p, grid, stream);
  if (b_major == HMC_MAJOR_MN) return launch_impl<HMC_MAJOR_K, HMC_MAJOR_MN, 0>(ta, tb, tc, tsa, tsb, p, grid, stream);
  return launch_impl<HMC_MAJOR_K, HMC_MAJOR_K, 0>(ta, tb, tc, tsa, tsb, p, grid, stream);
}

}  // namespace mx
}  // namespace hmc
