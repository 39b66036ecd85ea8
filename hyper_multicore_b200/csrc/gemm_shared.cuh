// Declarations shared by the grouped BF16 GEMM kernels (one-CTA tiles and CTA-pair tiles).
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "ep_device.cuh"
#include "sm100.cuh"

namespace hmc {
namespace gemm {

using namespace sm100;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int ACC_STAGES = 2;
constexpr int A_TILE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_TILE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int CHUNK_BYTES = 64 * BK * 2;  // one 64-wide MN-major chunk: BK rows of 128 B
constexpr int EPI_WARPS = 8;
constexpr int NUM_THREADS = 64 + EPI_WARPS * 32;
constexpr int STORE_STAGE_BYTES = 32 * 128;  // one 32-row x 128-byte TMA store box per epilogue warp
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_WARPS * STORE_STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t SWIZZLE_128B = 2;

constexpr uint64_t PIPE_BUDGET_NS = 4ull * 1000 * 1000 * 1000;  // default budget of intra-kernel barrier waits

struct Params {
  int mode;      // HMC_GEMM_RAGGED_M / HMC_GEMM_RAGGED_K
  int epilogue;  // HMC_EPI_*
  int groups;
  int m;  // RAGGED_K: rows of C per group. RAGGED_M: unused
  int n;  // logical N of the accumulator (SWIGLU: I, the width of one half)
  int k;  // RAGGED_M: contraction length. RAGGED_K: unused
  int n_tiles;
  int m_tiles;  // RAGGED_K only
  int ldc;      // row stride of C in elements
  int ld_aux;   // row stride of aux in elements
  long long rows;
  const long long* group_ends;
  void* c;
  void* aux;
  const int* ready_counters;  // optional, RAGGED_M: per-group arrival counters (rows landed)
  unsigned long long ready_budget_ns;
  unsigned long long pipe_budget_ns;  // intra-kernel barrier waits; covers the arrival budget when rows are awaited
  int* status;
  int tma_store;           // RAGGED_M plain stores: full tiles leave through shared memory + TMA
  int combine_enabled;     // STORE_BF16 rows go to `combine` destinations instead of c
  CombineFuse combine;
  int swiglu_clamp;        // HMC_CLAMP_*
  float swiglu_limit;
  const float* row_probs;  // optional per-row routing probability (weighting before FC2)
  float* row_dot;          // SWIGLU_GRAD with row_probs: per-row probability gradient (atomic adds)
  int dispatch_enabled;    // extra warps of this kernel send this rank's rows to their owners (RAGGED_M, gated)
  DispatchFuse dispatch;
  const int* skip_flag;    // optional: a non-zero value turns the launch into a no-op
};

__device__ __forceinline__ bool launch_skipped(const Params& p) {
  return p.skip_flag != nullptr && *reinterpret_cast<const volatile int*>(p.skip_flag) != 0;
}

struct Tile {
  int group;
  int m_idx;
  int n_idx;
  long long row0;  // first row of the group in the ragged dimension
  long long row1;  // one past the last row of the group
};

// Walks the static tile order. Tile indices only grow for a given CTA, so the group cursor only
// moves forward and every role (producer, MMA, epilogue) reproduces the same sequence.
template <int TILE_ROWS>
struct TileWalkerT {
  const Params& p;
  int group = 0;
  long long base = 0;  // first linear tile index of `group`
  long long row0 = 0;
  long long row1 = 0;
  int tiles_in_group = 0;

  __device__ explicit TileWalkerT(const Params& params) : p(params) {
    if (p.skip_flag != nullptr && *reinterpret_cast<const volatile int*>(p.skip_flag) != 0) group = p.groups;  // no tiles
    load_group();
  }

  __device__ void load_group() {
    if (group >= p.groups) {
      tiles_in_group = 0;
      return;
    }
    row0 = group == 0 ? 0 : p.group_ends[group - 1];
    row1 = p.group_ends[group];
    if (p.mode == HMC_GEMM_RAGGED_M) {
      long long rows = row1 - row0;
      tiles_in_group = static_cast<int>((rows + TILE_ROWS - 1) / TILE_ROWS) * p.n_tiles;
    } else {
      tiles_in_group = p.m_tiles * p.n_tiles;
    }
  }

  __device__ bool get(long long idx, Tile& t) {
    while (group < p.groups && idx >= base + tiles_in_group) {
      base += tiles_in_group;
      ++group;
      load_group();
    }
    if (group >= p.groups) return false;
    int local = static_cast<int>(idx - base);
    int mt = p.mode == HMC_GEMM_RAGGED_M ? tiles_in_group / p.n_tiles : p.m_tiles;
    t.group = group;
    t.m_idx = local % mt;
    t.n_idx = local / mt;
    t.row0 = row0;
    t.row1 = row1;
    return true;
  }
};

__device__ __forceinline__ int k_iterations(const Params& p, const Tile& t) {
  if (p.mode == HMC_GEMM_RAGGED_M) return (p.k + BK - 1) / BK;
  return static_cast<int>((t.row1 - t.row0 + BK - 1) / BK);
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// SwiGLU with the optional clamp: the gate is clipped from above before or after SiLU, the up
// projection to [-L, L]; a clipped branch passes its gradient while the clipped variable is within
// the bound, equality included.
struct SwigluTerms {
  float act;    // value of the activation
  float dgate;  // d act / d gate
  float dup;    // d act / d up
};

__device__ __forceinline__ SwigluTerms swiglu_terms(float g, float u, int clamp, float limit) {
  const float gx = clamp == HMC_CLAMP_BEFORE_SILU ? fminf(g, limit) : g;
  const float s = 1.0f / (1.0f + __expf(-gx));
  const float silu = gx * s;
  const float dsilu = s * (1.0f + gx * (1.0f - s));
  float gate_factor = silu;
  float uc = u;
  bool gate_pass = true;
  bool up_pass = true;
  if (clamp != HMC_CLAMP_NONE) {
    uc = fminf(fmaxf(u, -limit), limit);
    up_pass = u >= -limit && u <= limit;
    if (clamp == HMC_CLAMP_BEFORE_SILU) {
      gate_pass = g <= limit;
    } else {
      gate_pass = silu <= limit;
      gate_factor = fminf(silu, limit);
    }
  }
  SwigluTerms t;
  t.act = gate_factor * uc;
  t.dgate = gate_pass ? uc * dsilu : 0.0f;
  t.dup = up_pass ? gate_factor : 0.0f;
  return t;
}

// RAGGED_K tail block: rows past the end of the group belong to the next group (or are unwritten).
// Only the 16-row MMA steps that hold valid rows are issued; the invalid rows of the last such step
// are cleared in every 64-wide MN-major chunk of the stage. A 128-byte row stays one 128-byte line
// under the 128-byte swizzle, so whole lines can be cleared without undoing the swizzle.
// Returns the number of 16-row steps to issue; the whole warp calls it.
__device__ __forceinline__ int clear_tail_rows(uint8_t* stage_base, int chunks, int valid, int lane) {
  const int k_steps = (valid + 15) >> 4;
  const int vectors = (k_steps * 16 - valid) * 8;  // 16-byte vectors to clear per chunk
  if (vectors > 0) {
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int chunk = 0; chunk < chunks; ++chunk) {
      uint8_t* base = stage_base + chunk * CHUNK_BYTES + valid * 128;
      for (int i = lane; i < vectors; i += 32) *reinterpret_cast<uint4*>(base + i * 16) = zero;
    }
    fence_proxy_async_smem();
  }
  __syncwarp();
  return k_steps;
}

// Regular [rows, n] output tiles leave through shared memory and TMA stores (clipped at the row and
// column edges by the tensor map): the calling warp writes its 32 accumulator rows x columns
// [c_lo, c_hi) as 32-column boxes at rows m0.. of plane `plane`. FP32 boxes are 32 rows x 128 bytes in
// one 4 KiB stage. BF16 boxes are 32 rows x 64 bytes: the stage holds two of them, so the store of
// one box overlaps the packing of the next. `stores_issued` counts this warp's boxes across tiles.
__device__ __forceinline__ void epilogue_tma_boxes(const Params& p, const CUtensorMap* tm_c, uint32_t taddr,
                                                   uint8_t* my_stage, unsigned& stores_issued, int m0, int plane,
                                                   int col_base, int c_lo, int c_hi, int lane) {
  const bool f32 = p.epilogue == HMC_EPI_STORE_F32;
#pragma unroll 1
  for (int c = c_lo; c < c_hi; c += 32) {
    if (col_base + c >= p.n) break;
    uint32_t v[32];
    tmem_ld_32x32(taddr + c, v);
    tmem_ld_wait();
    uint8_t* box = my_stage;
    if (f32) {
      if (stores_issued > 0) {  // the previous box must have been read out of the stage
        if (lane == 0) bulk_wait_read_all();
        __syncwarp();
      }
      // 16-byte chunk q of row `lane` goes to chunk q ^ (lane & 7): the 128-byte swizzle the
      // tensor map expects, which also spreads a warp's stores over all banks.
      uint8_t* row_base = box + lane * 128;
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<uint4*>(row_base + ((q ^ (lane & 7)) << 4)) =
            make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    } else {
      box = my_stage + (stores_issued & 1) * (STORE_STAGE_BYTES / 2);
      if (stores_issued > 1) {  // the box before the previous one used this half
        if (lane == 0) bulk_wait_read_but_one();
        __syncwarp();
      }
      // 64-byte rows under the 64-byte swizzle: chunk q of row r sits at q ^ ((r >> 1) & 3)
      uint8_t* row_base = box + lane * 64;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 o;
        o.x = pack_bf16x2(__uint_as_float(v[8 * q + 0]), __uint_as_float(v[8 * q + 1]));
        o.y = pack_bf16x2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]));
        o.z = pack_bf16x2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]));
        o.w = pack_bf16x2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]));
        *reinterpret_cast<uint4*>(row_base + ((q ^ ((lane >> 1) & 3)) << 4)) = o;
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_3d(tm_c, box, col_base + c, m0, plane);
      bulk_commit_group();
    }
    ++stores_issued;
  }
}

// Row-major epilogues shared by the one-CTA and the CTA-pair kernels: the calling warp owns TMEM
// lanes [32 * quarter, +32) and the column half `half` of a 128 x 256 accumulator; thread `lane`
// owns output row `out_row` (written only when row_ok).
__device__ __forceinline__ void epilogue_rows(const Params& p, uint32_t taddr, long long out_row, bool row_ok,
                                        int col_base, int half) {
  const int c_lo = half * (BN / 2);
  const int c_hi = c_lo + BN / 2;
  if (p.epilogue == HMC_EPI_STORE_BF16) {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.c) + out_row * p.ldc + col_base;
#pragma unroll 1
    for (int c = c_lo; c < c_hi; c += 32) {
      uint32_t v[32];
      tmem_ld_32x32(taddr + c, v);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          if (col_base + c + j < p.n) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[j + 0]), __uint_as_float(v[j + 1]));
            o.y = pack_bf16x2(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
            o.z = pack_bf16x2(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
            o.w = pack_bf16x2(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
            *reinterpret_cast<uint4*>(dst + c + j) = o;
          }
        }
      }
    }
  } else if (p.epilogue == HMC_EPI_STORE_F32) {
    float* dst = static_cast<float*>(p.c) + out_row * p.ldc + col_base;
#pragma unroll 1
    for (int c = c_lo; c < c_hi; c += 32) {
      uint32_t v[32];
      tmem_ld_32x32(taddr + c, v);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          if (col_base + c + j < p.n) {
            *reinterpret_cast<float4*>(dst + c + j) =
                make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                            __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
          }
        }
      }
    }
  } else if (p.epilogue == HMC_EPI_SWIGLU) {
    // U[row, col] = bf16(gate), U[row, I + col] = bf16(up), Act[row, col] =
    // bf16(silu(gate_bf16) * up_bf16): the rounding points of the reference's golden
    // (tests/common/multicore/fp32_expert_reference.py:22-25).
    __nv_bfloat16* u_dst = static_cast<__nv_bfloat16*>(p.c) + out_row * p.ldc + col_base;
    __nv_bfloat16* a_dst = static_cast<__nv_bfloat16*>(p.aux) + out_row * p.ld_aux + col_base;
    const bool options = p.swiglu_clamp != HMC_CLAMP_NONE || p.row_probs != nullptr;
    // Read past L1: with the dispatch riding in this kernel, a neighbouring row's probability can have been
    // cached (same 128-byte line) before this row's value arrived from its source rank.
    const float prob = (p.row_probs != nullptr && row_ok) ? __ldcg(p.row_probs + out_row) : 1.0f;
#pragma unroll 1
    for (int c = half * (BN / 4); c < (half + 1) * (BN / 4); c += 32) {
      uint32_t g[32], u[32];
      tmem_ld_32x32(taddr + c, g);
      tmem_ld_32x32(taddr + BN / 2 + c, u);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          if (col_base + c + j < p.n) {
            uint32_t go[4], uo[4], ao[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              go[q] = pack_bf16x2(__uint_as_float(g[j + 2 * q]), __uint_as_float(g[j + 2 * q + 1]));
              uo[q] = pack_bf16x2(__uint_as_float(u[j + 2 * q]), __uint_as_float(u[j + 2 * q + 1]));
              const float2 gf = unpack_bf16x2(go[q]);
              const float2 uf = unpack_bf16x2(uo[q]);
              if (!options) {
                ao[q] = pack_bf16x2(silu_f(gf.x) * uf.x, silu_f(gf.y) * uf.y);
              } else {
                float a0 = swiglu_terms(gf.x, uf.x, p.swiglu_clamp, p.swiglu_limit).act;
                float a1 = swiglu_terms(gf.y, uf.y, p.swiglu_clamp, p.swiglu_limit).act;
                if (p.row_probs != nullptr) {
                  // two roundings: the activation first, then its product with the probability
                  a0 = bf16_round(a0) * prob;
                  a1 = bf16_round(a1) * prob;
                }
                ao[q] = pack_bf16x2(a0, a1);
              }
            }
            *reinterpret_cast<uint4*>(u_dst + c + j) = make_uint4(go[0], go[1], go[2], go[3]);
            *reinterpret_cast<uint4*>(u_dst + p.n + c + j) = make_uint4(uo[0], uo[1], uo[2], uo[3]);
            *reinterpret_cast<uint4*>(a_dst + c + j) = make_uint4(ao[0], ao[1], ao[2], ao[3]);
          }
        }
      }
    }
  } else {  // HMC_EPI_SWIGLU_GRAD
    // acc = dAct tile. With saved U = [gate | up] (aux): dU[:, col] = bf16(dA*up*s*(1+g(1-s))),
    // dU[:, I + col] = bf16(dA*silu(g)), dA rounded to BF16 first
    // (tests/common/multicore/fp32_expert_reference.py:29-33).
    const __nv_bfloat16* u_src = static_cast<const __nv_bfloat16*>(p.aux) + out_row * p.ld_aux + col_base;
    __nv_bfloat16* d_dst = static_cast<__nv_bfloat16*>(p.c) + out_row * p.ldc + col_base;
    const bool options = p.swiglu_clamp != HMC_CLAMP_NONE || p.row_probs != nullptr;
    // Read past L1: with the dispatch riding in this kernel, a neighbouring row's probability can have been
    // cached (same 128-byte line) before this row's value arrived from its source rank.
    const float prob = (p.row_probs != nullptr && row_ok) ? __ldcg(p.row_probs + out_row) : 1.0f;
    float dot = 0.0f;
#pragma unroll 1
    for (int c = c_lo; c < c_hi; c += 32) {
      uint32_t v[32];
      tmem_ld_32x32(taddr + c, v);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          if (col_base + c + j < p.n) {
            const uint4 gq = *reinterpret_cast<const uint4*>(u_src + c + j);
            const uint4 uq = *reinterpret_cast<const uint4*>(u_src + p.n + c + j);
            const uint32_t gw[4] = {gq.x, gq.y, gq.z, gq.w};
            const uint32_t uw[4] = {uq.x, uq.y, uq.z, uq.w};
            uint32_t dg[4], du[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 gf = unpack_bf16x2(gw[q]);
              const float2 uf = unpack_bf16x2(uw[q]);
              float da0 = bf16_round(__uint_as_float(v[j + 2 * q]));
              float da1 = bf16_round(__uint_as_float(v[j + 2 * q + 1]));
              if (!options) {
                const float s0 = 1.0f / (1.0f + __expf(-gf.x));
                const float s1 = 1.0f / (1.0f + __expf(-gf.y));
                dg[q] = pack_bf16x2(da0 * uf.x * s0 * (1.0f + gf.x * (1.0f - s0)),
                                    da1 * uf.y * s1 * (1.0f + gf.y * (1.0f - s1)));
                du[q] = pack_bf16x2(da0 * (gf.x * s0), da1 * (gf.y * s1));
              } else {
                const SwigluTerms t0 = swiglu_terms(gf.x, uf.x, p.swiglu_clamp, p.swiglu_limit);
                const SwigluTerms t1 = swiglu_terms(gf.y, uf.y, p.swiglu_clamp, p.swiglu_limit);
                if (p.row_probs != nullptr) {
                  // the accumulator is the gradient of the weighted FC2 input: the probability
                  // gradient uses the unweighted BF16 activation, the activation gradient is
                  // rounded to BF16 after the multiplication
                  dot += bf16_round(t0.act) * da0 + bf16_round(t1.act) * da1;
                  da0 = bf16_round(da0 * prob);
                  da1 = bf16_round(da1 * prob);
                }
                dg[q] = pack_bf16x2(da0 * t0.dgate, da1 * t1.dgate);
                du[q] = pack_bf16x2(da0 * t0.dup, da1 * t1.dup);
              }
            }
            *reinterpret_cast<uint4*>(d_dst + c + j) = make_uint4(dg[0], dg[1], dg[2], dg[3]);
            *reinterpret_cast<uint4*>(d_dst + p.n + c + j) = make_uint4(du[0], du[1], du[2], du[3]);
          }
        }
      }
    }
    if (p.row_dot != nullptr && row_ok) atomicAdd(p.row_dot + out_row, dot);
  }
}

}  // namespace gemm
}  // namespace hmc
