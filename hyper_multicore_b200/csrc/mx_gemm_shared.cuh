// What the two block-scaled FP8 grouped-GEMM kernels share: the launch parameters, the walk over
// (group, row block, column tile) work items, and the host-side tensor-map helpers.
//
// Activation rows live in the padded expert-major layout (every group starts on a 128-row block,
// padding rows are zero), so no operand tile, scale block or scale atom straddles two experts.
// A scale atom is 512 bytes: the UE8M0 scales of 128 rows x 4 blocks of 32 contraction elements.
#pragma once

#include <cuda.h>
#include <stdint.h>

#include "common.cuh"

namespace hmc {
namespace mx {

constexpr int BK = 128;                // contraction elements (= bytes) per k-block
constexpr int TILE_BYTES = 128 * 128;  // one 128 x 128 operand tile of E4M3
constexpr int ATOM_BYTES = 512;
constexpr int EPI_WARPS = 8;
constexpr int NUM_THREADS = 64 + EPI_WARPS * 32;
constexpr int STORE_STAGE_BYTES = 32 * 128;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t SWIZZLE_128B = 2;
constexpr uint64_t PIPE_BUDGET_NS = 4ull * 1000 * 1000 * 1000;

struct Params {
  int mode;
  int epilogue;
  int groups;
  int m;        // RAGGED_K: rows of C per group
  int n;
  int k;        // RAGGED_M: contraction length
  int n_tiles;  // column tiles of the launched kernel (128 or 256 wide)
  int m_tiles;  // RAGGED_K: row tiles of the launched kernel (128 or 256 high)
  int n_atoms;  // n / 128
  int m_atoms;  // RAGGED_K: m / 128
  int k_blocks; // RAGGED_M: k / 128
  int pad_blocks;
  long long rows;
  const long long* group_ends;
  const uint8_t* a_scale;
  const uint8_t* b_scale;
  void* c;
  int* status;
  int combine_enabled;  // RAGGED_M: rows go to `combine` destinations instead of c
  CombineFuse combine;
  // HMC_EPI_SWIGLU_MXQ: quantised bf16(silu(gate) * up), width n / 2, in the layouts of the stand-alone quantiser
  uint8_t* act_row_data;
  uint8_t* act_row_scale;
  uint8_t* act_col_data;
  uint8_t* act_col_scale;
  const int* skip_flag;  // non-zero when the launch runs: no tile is processed (the call was not admitted)
  const void* aux;  // HMC_EPI_SWIGLU_GRAD_MXQ: the saved U [rows, 2n] of the same rows (the outputs above are dU, width 2n)
};

struct Tile {
  int group;
  int m_idx;
  int n_idx;
  long long row0;     // un-padded first row of the group
  long long row1;
  int pad_block0;     // first 128-row block of the group in the padded layout
  int blocks;         // 128-row blocks of the group
};

// Work items in launch order. RAGGED_M: a tile covers BLOCKS_PER_TILE consecutive 128-row blocks of one
// group (the last tile of a group with an odd number of blocks is half empty). RAGGED_K: a tile is
// (row tile, column tile) of one group's [m, n] result. Row tiles vary fastest, so CTAs that run
// side by side read the same weight columns.
template <int BLOCKS_PER_TILE>
struct TileWalkerT {
  const Params& p;
  int group = 0;
  long long base = 0;
  long long row0 = 0;
  long long row1 = 0;
  int pad_block0 = 0;
  int blocks = 0;
  int tiles_in_group = 0;

  __device__ explicit TileWalkerT(const Params& params) : p(params) {
    if (p.skip_flag != nullptr && *p.skip_flag != 0) group = p.groups;  // every role sees an empty problem
    load_group();
  }

  __device__ int row_tiles() const {
    return p.mode == HMC_GEMM_RAGGED_M ? (blocks + BLOCKS_PER_TILE - 1) / BLOCKS_PER_TILE : p.m_tiles;
  }

  __device__ void load_group() {
    if (group >= p.groups) {
      tiles_in_group = 0;
      return;
    }
    row0 = group == 0 ? 0 : p.group_ends[group - 1];
    row1 = p.group_ends[group];
    blocks = static_cast<int>((row1 - row0 + 127) / 128);
    tiles_in_group = row_tiles() * p.n_tiles;
  }

  __device__ bool get(long long idx, Tile& t) {
    while (group < p.groups && idx >= base + tiles_in_group) {
      base += tiles_in_group;
      pad_block0 += blocks;
      ++group;
      load_group();
    }
    if (group >= p.groups) return false;
    const int local = static_cast<int>(idx - base);
    const int mt = row_tiles();
    t.group = group;
    t.m_idx = local % mt;
    t.n_idx = local / mt;
    t.row0 = row0;
    t.row1 = row1;
    t.pad_block0 = pad_block0;
    t.blocks = blocks;
    return true;
  }
};

__device__ __forceinline__ int k_iterations(const Params& p, const Tile& t) {
  return p.mode == HMC_GEMM_RAGGED_M ? p.k_blocks : t.blocks;
}

// Destination of one output row of a RAGGED_M GEMM: the row itself in c, or - fused combine - its place in
// the routed buffer of its source rank. Returns the address of column `col_base` (0 when the row is not
// to be written) and the source rank in `source` (-1 without the fused combine).
__device__ __forceinline__ unsigned long long mx_row_destination(const Params& p, const Tile& t, long long out_row,
                                                                  int col_base, int& source) {
  source = -1;
  if (out_row >= t.row1) return 0;
  if (!p.combine_enabled)
    return reinterpret_cast<unsigned long long>(static_cast<__nv_bfloat16*>(p.c) + out_row * p.n + col_base);
  const CombineFuse& cf = p.combine;
  const long long* seg = cf.segment_start + static_cast<long long>(t.group) * cf.ep;
  int s = 0;
  for (int q = 1; q < cf.ep; ++q)
    if (seg[q] <= out_row) s = q;
  const long long dest = cf.combine_target_off[s * cf.local_experts + t.group] + (out_row - seg[s]);
  if (dest < 0 || dest >= cf.target_rows_limit) {
    report_status(p.status, HMC_STATUS_BAD_INDEX, static_cast<int>(out_row), s, static_cast<int>(dest));
    return 0;
  }
  source = s;
  return reinterpret_cast<unsigned long long>(static_cast<__nv_bfloat16*>(cf.peer_data[s]) + dest * p.n + col_base);
}

// ----------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
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

// elem: 1 = uint8 (E4M3 payload), 2 = bf16, 4 = f32. dims[0] innermost; 128-byte swizzle.
inline int make_map(CUtensorMap* out, const void* base, int rank, const cuuint64_t* dims, const cuuint32_t* box, int elem) {
  EncodeTiledFn fn = encode_fn();
  HMC_REQUIRE(fn != nullptr, HMC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t strides[4];
  cuuint64_t acc = static_cast<cuuint64_t>(elem);
  for (int i = 0; i + 1 < rank; ++i) {
    acc *= dims[i];
    strides[i] = acc;
  }
  cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
  const CUtensorMapDataType type = elem == 1   ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : elem == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(out, type, static_cast<cuuint32_t>(rank), const_cast<void*>(base), dims, strides, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  HMC_REQUIRE(r == CUDA_SUCCESS, HMC_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

// Scale atoms as a 2-D tensor of 32-bit words [atoms][128], un-swizzled; a box is `box_atoms` whole atoms.
inline int make_atom_map(CUtensorMap* out, const void* base, long long atoms, int box_atoms) {
  EncodeTiledFn fn = encode_fn();
  HMC_REQUIRE(fn != nullptr, HMC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {ATOM_BYTES / 4, static_cast<cuuint64_t>(atoms)};
  cuuint64_t strides[1] = {ATOM_BYTES};
  cuuint32_t box[2] = {ATOM_BYTES / 4, static_cast<cuuint32_t>(box_atoms)};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  HMC_REQUIRE(r == CUDA_SUCCESS, HMC_ERR_CUDA, "cuTensorMapEncodeTiled (scale atoms) failed with CUresult %d", (int)r);
  return 0;
}

// Defined in mx_gemm_pair.cu: 256 x 256 tiles on CTA pairs.
int launch_mx_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tsa,
                        const CUtensorMap& tsb, const Params& p, int a_major, int b_major, int grid, cudaStream_t stream);

}  // namespace mx
}  // namespace hmc
