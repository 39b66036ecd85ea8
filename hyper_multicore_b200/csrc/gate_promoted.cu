// Router projection logits[T, E] = float(x[T, H]) . W[E, H]^T on tcgen05 with FP32-level accuracy.
//
// Replaces the FP32 projection of MegaGate (hyper_multicore/modules/mega_gate/function.py:175-178,
// module.py:195-198) for BF16 hidden states. x is exact in BF16; the FP32 weight is split into three
// BF16 parts hi + mid + lo that reproduce it to 24 bits, so every product is exact in FP32 and the
// only error left is the accumulation inside the tensor core, which grows with the length of the
// accumulation chain. The chain is therefore cut every 128 elements of K: two TMEM accumulators
// alternate, and while the tensor core fills one, the epilogue warps add the other into FP32 registers
// (round-to-nearest adds on the CUDA cores). The three parts are stacked along N (64 experts x 3 = 192
// accumulator columns), so one M128 N192 K16 instruction does what three N64 ones did - the kernel was
// bound by the number of MMA instructions, not by their flops or by its loads. The mid and lo parts
// (2^-8 and 2^-16 of the result) are promoted with the hi part and summed in a register set of their own.
//
// One CTA per 128 tokens x 64 experts (x K-slice; the two K-slices of a tile form a cluster and the first adds
// the second's partial sums, a + b, so results repeat bit for bit): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM
// owner, warps 2..5 = promotion + epilogue (one per TMEM lane quarter).
//
// With at most 64 experts an epilogue thread ends up holding the whole logits row of one token, so the ROUTE
// instance of the kernel goes on to score, bias, select and weigh that token (the work of gate_route_kernel) and
// the logits are written once and never read back. Where a tile has two K-slices, each slice finishes 64 of its
// tokens and routes them with two threads per token (route_pair); otherwise one thread routes its token (route_token).
#include <cuda.h>
#include <math.h>

#include "common.cuh"
#include "sm100.cuh"

namespace hmc {
namespace {

using namespace sm100;

constexpr int GM = 128;                      // tokens per CTA
constexpr int GN = 64;                       // experts per CTA
constexpr int GK = 64;                       // K elements per pipeline stage (128-byte rows)
constexpr int G_STAGES = 4;
constexpr int G_PROMOTE = 2;                 // stages per accumulation chain (128 K elements)
constexpr int ACC_COLS = 3 * GN;             // TMEM columns of one accumulator: 64 experts x up to 3 weight parts
constexpr int A_BYTES = GM * GK * 2;         // 16 KiB
constexpr int B_BYTES = GN * GK * 2;         // 8 KiB per weight part
constexpr int G_STAGE_BYTES = A_BYTES + 3 * B_BYTES;
constexpr int G_THREADS = 6 * 32;
constexpr int G_SMEM_BYTES = G_STAGES * G_STAGE_BYTES + 1024 + 256;
constexpr uint32_t G_TMEM_COLS = 512;        // two accumulators of 64 x parts columns: @0 and @192
constexpr uint32_t SWIZZLE_128B = 2;
constexpr uint64_t G_BUDGET_NS = 4ull * 1000 * 1000 * 1000;

// [host-testable begin] From here to the matching end mark the code is plain C++ apart from a handful of intrinsics;
// tests/test_gate_route_host.py compiles it for the CPU with stand-ins for those and checks the Route against the
// reference fixtures without a GPU.
struct GateParams {
  long long tokens;
  int hidden;
  int experts;
  int epad;        // experts rounded up to GN: row pitch between the weight parts
  int parts;       // 3 for FP32 weights, 1 for BF16 weights
  int k_blocks;    // ceil(hidden / GK)
  int k_per_slice; // k-blocks per K-slice (gridDim.z slices)
  float* logits;
  int* status;
  // ROUTE instance only
  const float* text_bias;
  const float* vision_bias;
  const uint8_t* image_mask;
  int use_vision_bias;
  int top_k;
  int scoring;
  float scale;
  float* weights;
  long long* indices;
  float* route_scores;
  float* selected;
  float* denominator;
};

// Route of one token whose logits row v[0, experts) sits in the registers of one thread. Every output equals
// gate_route_kernel's bit for bit: the same elementwise functions, the softmax sum added in that kernel's order
// (lane l of its warp holds experts l and l + 32, then a butterfly over the lanes), selection by the largest
// biased score with NaN as +inf and ties to the lower expert.
__device__ __forceinline__ void route_token(float (&v)[GN], long long token, const GateParams& p) {
  const int experts = p.experts;
  if (p.scoring == HMC_SCORE_SOFTMAX) {
    float m = -INFINITY;
#pragma unroll
    for (int c = 0; c < GN; ++c)
      if (c < experts) m = fmaxf(m, v[c]);
    float part[32];
#pragma unroll
    for (int l = 0; l < 32; ++l) {
      v[l] = l < experts ? expf(v[l] - m) : 0.f;
      v[l + 32] = l + 32 < experts ? expf(v[l + 32] - m) : 0.f;
      part[l] = v[l] + v[l + 32];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int l = 0; l < o; ++l) part[l] = part[l] + part[l + o];
    }
    const float inv = 1.0f / part[0];
#pragma unroll
    for (int c = 0; c < GN; ++c) v[c] *= inv;
  } else if (p.scoring == HMC_SCORE_SIGMOID) {
#pragma unroll
    for (int c = 0; c < GN; ++c) v[c] = 1.0f / (1.0f + expf(-v[c]));
  } else {
#pragma unroll
    for (int c = 0; c < GN; ++c) {
      const float x = v[c];
      v[c] = sqrtf(x > 20.0f ? x : log1pf(expf(x)));  // torch softplus(beta = 1, threshold = 20)
    }
  }

  float* score_out = p.route_scores + token * experts;
  if (experts % 4 == 0) {
#pragma unroll
    for (int c = 0; c < GN; c += 4)
      if (c < experts) *reinterpret_cast<float4*>(score_out + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
  } else {
#pragma unroll
    for (int c = 0; c < GN; ++c)
      if (c < experts) score_out[c] = v[c];
  }

  // Selection keys: the biased scores as integers in float order (NaN as +inf, -0 as +0), so that one value below
  // every float - INT_MIN - can mark an expert that is absent or already taken and a pass costs one compare per expert.
  const float* bias = (p.use_vision_bias && p.image_mask[token]) ? p.vision_bias : p.text_bias;
  constexpr int GONE = static_cast<int>(0x80000000u);
  int key[GN];
#pragma unroll
  for (int c = 0; c < GN; ++c) {
    float b = c < experts ? __fadd_rn(v[c], __ldg(bias + c)) : 0.f;
    b = isnan(b) ? INFINITY : __fadd_rn(b, 0.f);
    const int bits = __float_as_int(b);
    key[c] = c < experts ? (bits ^ ((bits >> 31) & 0x7fffffff)) : GONE;
  }

  float* sel_out = p.selected + token * p.top_k;
  long long* idx_out = p.indices + token * p.top_k;
  float total = 0.f;
  for (int k = 0; k < p.top_k; ++k) {
    // four independent chains over 16 experts each, joined in expert order: the largest key, ties to the lower expert
    int best[4], best_at[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      best[q] = GONE;
      best_at[q] = 0x7fffffff;
#pragma unroll
      for (int c = 16 * q; c < 16 * q + 16; ++c) {
        if (key[c] > best[q]) {
          best[q] = key[c];
          best_at[q] = c;
        }
      }
    }
    int top = best[0], best_idx = best_at[0];
#pragma unroll
    for (int q = 1; q < 4; ++q) {
      if (best[q] > top) {
        top = best[q];
        best_idx = best_at[q];
      }
    }
    if (best_idx == 0x7fffffff) break;  // top_k <= experts: not reached
    float win = 0.f;
#pragma unroll
    for (int c = 0; c < GN; ++c) {
      const bool hit = c == best_idx;
      win = hit ? v[c] : win;
      key[c] = hit ? GONE : key[c];
    }
    total += win;
    sel_out[k] = win;
    idx_out[k] = best_idx;
  }
  const float denom = total + 1.0e-20f;
  p.denominator[token] = denom;
  for (int k = 0; k < p.top_k; ++k) {
    float w = sel_out[k];
    if (p.top_k > 1) w = w / denom;
    p.weights[token * p.top_k + k] = w * p.scale;
  }
}

// The same Route with two threads per token, lanes l and l + 16 of a warp: thread `half` holds experts
// [32 * half, 32 * half + 32) in v[] and the two exchange what the other needs by shuffles, so every phase is half as
// long. Used when the two K-slices of a tile each finish 64 of its tokens. The whole warp runs every step (`valid`
// only guards the stores); results are those of route_token bit for bit.
constexpr int ROUTE_PITCH = GN + 1;             // words per token row staged in shared memory
constexpr int ROUTE_SMEM_OFFSET = GN * GM * 4;  // behind the K-slice exchange area
static_assert(ROUTE_SMEM_OFFSET + (GM / 2) * ROUTE_PITCH * 4 <= G_STAGES * G_STAGE_BYTES, "staged rows fit in the idle ring");

__device__ __forceinline__ void route_pair(float (&v)[32], int half, long long token, bool valid, const GateParams& p) {
  constexpr unsigned FULL = 0xffffffffu;
  constexpr int GONE = static_cast<int>(0x80000000u);
  const int experts = p.experts;
  const int base = 32 * half;
  if (valid) {
    float* dst = p.logits + token * experts + base;
    if (experts % 4 == 0) {
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        if (base + i < experts) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (base + i < experts) dst[i] = v[i];
    }
  }
  if (p.scoring == HMC_SCORE_SOFTMAX) {
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (base + i < experts) m = fmaxf(m, v[i]);
    m = fmaxf(m, __shfl_xor_sync(FULL, m, 16));
    float part[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      v[i] = base + i < experts ? expf(v[i] - m) : 0.f;
      part[i] = v[i] + __shfl_xor_sync(FULL, v[i], 16);  // experts i and i + 32, as a lane of gate_route_kernel adds them
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int l = 0; l < o; ++l) part[l] = part[l] + part[l + o];
    }
    const float inv = 1.0f / part[0];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= inv;
  } else if (p.scoring == HMC_SCORE_SIGMOID) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = 1.0f / (1.0f + expf(-v[i]));
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float x = v[i];
      v[i] = sqrtf(x > 20.0f ? x : log1pf(expf(x)));  // torch softplus(beta = 1, threshold = 20)
    }
  }
  if (valid) {
    float* dst = p.route_scores + token * experts + base;
    if (experts % 4 == 0) {
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        if (base + i < experts) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (base + i < experts) dst[i] = v[i];
    }
  }

  const float* bias = (valid && p.use_vision_bias && p.image_mask[token]) ? p.vision_bias : p.text_bias;
  int key[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float b = base + i < experts ? __fadd_rn(v[i], __ldg(bias + base + i)) : 0.f;
    b = isnan(b) ? INFINITY : __fadd_rn(b, 0.f);
    const int bits = __float_as_int(b);
    key[i] = base + i < experts ? (bits ^ ((bits >> 31) & 0x7fffffff)) : GONE;
  }
  float total = 0.f;
  for (int k = 0; k < p.top_k; ++k) {
    int best = GONE, at = 0x7fffffff, best_hi = GONE, at_hi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (key[i] > best) {
        best = key[i];
        at = base + i;
      }
      if (key[16 + i] > best_hi) {
        best_hi = key[16 + i];
        at_hi = base + 16 + i;
      }
    }
    if (best_hi > best) {
      best = best_hi;
      at = at_hi;
    }
    const int other = __shfl_xor_sync(FULL, best, 16);
    const int other_at = __shfl_xor_sync(FULL, at, 16);
    if (other > best || (other == best && other_at < at)) {
      best = other;
      at = other_at;
    }
    float win = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const bool hit = base + i == at;
      win = hit ? v[i] : win;
      key[i] = hit ? GONE : key[i];
    }
    const float other_win = __shfl_xor_sync(FULL, win, 16);
    if ((at >> 5) != half) win = other_win;
    total += win;
    if (valid && half == 0) {
      p.selected[token * p.top_k + k] = win;
      p.indices[token * p.top_k + k] = at;
    }
  }
  if (valid && half == 0) {
    const float denom = total + 1.0e-20f;
    p.denominator[token] = denom;
    for (int k = 0; k < p.top_k; ++k) {
      float w = p.selected[token * p.top_k + k];
      if (p.top_k > 1) w = w / denom;
      p.weights[token * p.top_k + k] = w * p.scale;
    }
  }
}

// [host-testable end]

// FP32 (or BF16) weight [E, H] -> BF16 parts stacked as rows [part * epad + e] of a [parts * epad, H] matrix
__global__ void gate_split_parts_kernel(const void* __restrict__ w, int w_is_bf16, int experts, int epad, int parts,
                                        long long hidden, __nv_bfloat16* __restrict__ split) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(epad) * hidden) return;
  const int e = static_cast<int>(i / hidden);
  float v = 0.f;
  if (e < experts)
    v = w_is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(w)[i]) : static_cast<const float*>(w)[i];
  const __nv_bfloat16 hi = __float2bfloat16_rn(v);
  split[i] = hi;
  if (parts == 3) {
    const float r1 = v - __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
    split[static_cast<long long>(epad) * hidden + i] = mid;
    split[2ll * epad * hidden + i] = __float2bfloat16_rn(r1 - __bfloat162float(mid));
  }
}

template <bool ROUTE>
__global__ void __launch_bounds__(G_THREADS, 1)
gate_project_promoted_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                             const GateParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + G_STAGES * G_STAGE_BYTES);
  uint64_t* full_bar = bars;                       // [G_STAGES]
  uint64_t* empty_bar = bars + G_STAGES;           // [G_STAGES]
  uint64_t* hi_full_bar = bars + 2 * G_STAGES;     // [2]
  uint64_t* hi_empty_bar = bars + 2 * G_STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * G_STAGES + 4);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * GM;
  const int e0 = blockIdx.y * GN;
  const int kb_begin = blockIdx.z * p.k_per_slice;
  const int kb_end = min(p.k_blocks, kb_begin + p.k_per_slice);
  const int nkb = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < G_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&hi_full_bar[b], 1);
      mbar_init(&hi_empty_bar[b], 4);  // one arrival per promotion warp
    }
    *abort_word = 0;
    mbar_fence_init();
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_w);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, G_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int quarter = warp & 3;
  float sum[GN];  // hi part (then the whole result); lives past the role branches for the cluster exchange
#pragma unroll
  for (int c = 0; c < GN; ++c) sum[c] = 0.f;
  bool ok = true;

  if (warp == 0) {
    // ======================================================================== TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t bytes = A_BYTES + p.parts * B_BYTES;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_word, G_BUDGET_NS)) {
          report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 0, stage, kb);
          break;
        }
        uint8_t* a_dst = smem + stage * G_STAGE_BYTES;
        mbar_arrive_expect_tx(&full_bar[stage], bytes);
        tma_load_2d(a_dst, &tm_x, &full_bar[stage], kb * GK, m0);
        for (int part = 0; part < p.parts; ++part)
          tma_load_2d(a_dst + A_BYTES + part * B_BYTES, &tm_w, &full_bar[stage], kb * GK, part * p.epad + e0);
        if (++stage == G_STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ======================================================================== MMA issuer
    int stage = 0;
    uint32_t phase = 0;
    uint32_t empty_phase[2] = {0, 0};
    // BF16 x BF16 -> FP32, K-major operands, M = 128, N = 64 experts x parts
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (((GN * p.parts) >> 3) << 17) | ((GM >> 4) << 24);
    for (int i = 0; ok && i < nkb; ++i) {
      const int buf = (i / G_PROMOTE) & 1;
      const bool chain_start = i % G_PROMOTE == 0;
      const bool chain_end = i % G_PROMOTE == G_PROMOTE - 1 || i == nkb - 1;
      if (chain_start) {
        if (!mbar_wait(&hi_empty_bar[buf], empty_phase[buf] ^ 1u, abort_word, G_BUDGET_NS)) {
          if (lane == 0) report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 1, buf, i);
          ok = false;
          break;
        }
        tc_fence_after_sync();
      }
      if (!mbar_wait(&full_bar[stage], phase, abort_word, G_BUDGET_NS)) {
        if (lane == 0) report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 2, stage, i);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t a_addr = smem_u32(smem + stage * G_STAGE_BYTES);
        const uint64_t da = make_smem_desc(a_addr, 16, 1024, SWIZZLE_128B);
        // the parts' 64-row tiles lie back to back: one B operand of 64 x parts rows
        const uint64_t db = make_smem_desc(a_addr + A_BYTES, 16, 1024, SWIZZLE_128B);
        const uint32_t tm_acc = tmem_base + static_cast<uint32_t>(buf * ACC_COLS);
#pragma unroll
        for (int ks = 0; ks < GK / 16; ++ks)
          umma_bf16(tm_acc, da + 2 * ks, db + 2 * ks, idesc, (!chain_start || ks > 0) ? 1u : 0u);
        umma_commit(&empty_bar[stage]);
        if (chain_end) umma_commit(&hi_full_bar[buf]);
      }
      __syncwarp();
      if (chain_end) empty_phase[buf] ^= 1u;
      if (++stage == G_STAGES) {
        stage = 0;
        phase ^= 1u;
      }
    }
  } else {
    // ======================================================================== promotion + epilogue
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    float minor[GN];  // mid + lo parts
#pragma unroll
    for (int c = 0; c < GN; ++c) minor[c] = 0.f;
    uint32_t full_phase[2] = {0, 0};
    const int chains = (nkb + G_PROMOTE - 1) / G_PROMOTE;
    for (int it = 0; ok && it < chains; ++it) {
      const int buf = it & 1;
      if (!mbar_wait(&hi_full_bar[buf], full_phase[buf], abort_word, G_BUDGET_NS)) {
        if (lane == 0) report_status(p.status, HMC_STATUS_TIMEOUT_PIPELINE, 3, buf, it);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t acc = tmem_base + lane_base + static_cast<uint32_t>(buf * ACC_COLS);
      uint32_t v[32], w[32];
      tmem_ld_32x32(acc, v);
      tmem_ld_32x32(acc + 32, w);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        sum[c] += __uint_as_float(v[c]);
        sum[32 + c] += __uint_as_float(w[c]);
      }
      if (p.parts == 3) {
#pragma unroll 1
        for (int part = 1; part < 3; ++part) {
          tmem_ld_32x32(acc + static_cast<uint32_t>(part * GN), v);
          tmem_ld_32x32(acc + static_cast<uint32_t>(part * GN + 32), w);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            minor[c] += __uint_as_float(v[c]);
            minor[32 + c] += __uint_as_float(w[c]);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&hi_empty_bar[buf]);  // the tensor core may start the next chain here
      full_phase[buf] ^= 1u;
    }
    if (p.parts == 3) {
#pragma unroll
      for (int c = 0; c < GN; ++c) sum[c] += minor[c];
    }
  }

  // Two K-slices are the two CTAs of a cluster and exchange partial sums through distributed shared memory (the
  // pipeline ring is idle by then); a result is always slice 0's sum + slice 1's.
  const bool sliced = gridDim.z > 1;
  const uint32_t slice = sliced ? cluster_ctarank() : 0u;
  const long long row = static_cast<long long>(m0) + quarter * 32 + lane;
  if (ROUTE && sliced) {
    // Each slice finishes 64 of the tile's tokens - slice 0 rows 0..63, slice 1 rows 64..127 - and routes them with
    // two threads per token.
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // both CTAs' rings are drained
    const int r = quarter * 32 + lane;
    const bool finish_here = (r < GM / 2) == (slice == 0u);
    if (warp >= 2 && !finish_here) {
      const uint32_t peer = map_to_cta(smem_u32(smem), slice ^ 1u);
#pragma unroll
      for (int c = 0; c < GN; ++c)
        st_shared_cluster_f32(peer + static_cast<uint32_t>((c * (GM / 2) + (r & 63)) * 4), sum[c]);
    }
    cluster_sync_all();
    float* rows = reinterpret_cast<float*>(smem + ROUTE_SMEM_OFFSET);
    if (warp >= 2 && finish_here) {
      const float* exchange = reinterpret_cast<const float*>(smem);
      float* mine = rows + (r & 63) * ROUTE_PITCH;
#pragma unroll
      for (int c = 0; c < GN; ++c) mine[c] = sum[c] + exchange[c * (GM / 2) + (r & 63)];
    }
    __syncthreads();
    if (warp >= 2 && nkb > 0) {
      const int half = lane >> 4;
      const int local = quarter * 16 + (lane & 15);
      const long long token = static_cast<long long>(m0) + static_cast<long long>(slice) * (GM / 2) + local;
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = rows[local * ROUTE_PITCH + half * 32 + i];
      route_pair(v, half, token, token < p.tokens, p);
    }
  } else {
    if (sliced) {
      tc_fence_before_sync();
      __syncthreads();
      cluster_sync_all();  // both CTAs' rings are drained
      if (warp >= 2 && slice == 1) {
        const uint32_t peer = map_to_cta(smem_u32(smem), 0);
        const int r = quarter * 32 + lane;
#pragma unroll
        for (int c = 0; c < GN; ++c) st_shared_cluster_f32(peer + static_cast<uint32_t>((c * GM + r) * 4), sum[c]);
      }
      cluster_sync_all();
      if (warp >= 2 && slice == 0) {
        const float* exchange = reinterpret_cast<const float*>(smem);
        const int r = quarter * 32 + lane;
#pragma unroll
        for (int c = 0; c < GN; ++c) sum[c] += exchange[c * GM + r];
      }
    }
    if (warp >= 2 && slice == 0 && ok && row < p.tokens && nkb > 0) {
      float* dst = p.logits + row * p.experts + e0;
      if (p.experts % 4 == 0) {
#pragma unroll
        for (int c = 0; c < GN; c += 4)
          if (e0 + c < p.experts) *reinterpret_cast<float4*>(dst + c) = make_float4(sum[c], sum[c + 1], sum[c + 2], sum[c + 3]);
      } else {
#pragma unroll
        for (int c = 0; c < GN; ++c)
          if (e0 + c < p.experts) dst[c] = sum[c];
      }
      if constexpr (ROUTE) route_token(sum, row, p);  // one column tile: sum[] is the token's whole row
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, G_TMEM_COLS);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn gate_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

int gate_make_map(CUtensorMap* out, const void* base, long long inner, long long outer, int box_inner, int box_outer) {
  EncodeTiledFn fn = gate_encode_fn();
  HMC_REQUIRE(fn != nullptr, HMC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(inner) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  HMC_REQUIRE(r == CUDA_SUCCESS, HMC_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

}  // namespace
}  // namespace hmc

extern "C" int64_t hmc_gate_project_promoted_workspace_bytes(int64_t hidden, int64_t experts) {
  const int64_t epad = (experts + hmc::GN - 1) / hmc::GN * hmc::GN;
  return 3 * epad * hidden * 2;
}

namespace hmc {
namespace {

// Split the weight (unless w == NULL), then one launch of the projection; `route` adds the Route of every token.
int gate_promoted_launch(const char* who, const void* x_bf16, const void* w, int w_is_bf16, int64_t tokens,
                         int64_t hidden, int64_t experts, float* logits, void* workspace, int64_t workspace_bytes,
                         const hmc_gate_route_args* route, int32_t* status, cudaStream_t stream) {
  HMC_REQUIRE(x_bf16 && logits && workspace, HMC_ERR_INVALID, "%s: null tensor pointer", who);
  HMC_REQUIRE(tokens > 0 && experts > 0 && hidden > 0 && hidden % 8 == 0, HMC_ERR_INVALID,
              "%s: extents must be positive and hidden a multiple of 8", who);
  HMC_REQUIRE(tokens < (1ll << 31) && hidden < (1ll << 31) && experts <= 65536, HMC_ERR_LIMIT,
              "%s: extent too large", who);
  HMC_REQUIRE(workspace_bytes >= hmc_gate_project_promoted_workspace_bytes(hidden, experts), HMC_ERR_INVALID,
              "%s: workspace holds %lld bytes, %lld needed", who, (long long)workspace_bytes,
              (long long)hmc_gate_project_promoted_workspace_bytes(hidden, experts));
  HMC_REQUIRE(aligned16(x_bf16) && aligned16(workspace) && aligned16(logits), HMC_ERR_INVALID,
              "%s: 16-byte alignment", who);
  const int epad = static_cast<int>((experts + GN - 1) / GN * GN);
  const int parts = w_is_bf16 ? 1 : 3;
  __nv_bfloat16* split = static_cast<__nv_bfloat16*>(workspace);
  const long long split_elems = static_cast<long long>(epad) * hidden;
  if (w != nullptr) {  // w == NULL: the workspace still holds the parts of an earlier call with the same weight
    gate_split_parts_kernel<<<static_cast<unsigned>((split_elems + 255) / 256), 256, 0, stream>>>(
        w, w_is_bf16, static_cast<int>(experts), epad, parts, hidden, split);
    HMC_LAUNCH_OK();
  }

  CUtensorMap tx, tw;
  int rc;
  if ((rc = gate_make_map(&tx, x_bf16, hidden, tokens, GK, GM)) != 0) return rc;
  if ((rc = gate_make_map(&tw, split, hidden, static_cast<long long>(parts) * epad, GK, GN)) != 0) return rc;

  GateParams p{};
  p.tokens = tokens;
  p.hidden = static_cast<int>(hidden);
  p.experts = static_cast<int>(experts);
  p.epad = epad;
  p.parts = parts;
  p.k_blocks = static_cast<int>((hidden + GK - 1) / GK);
  p.logits = logits;
  p.status = status;
  if (route != nullptr) {
    p.text_bias = route->text_bias;
    p.vision_bias = route->vision_bias;
    p.image_mask = route->image_mask;
    p.use_vision_bias = route->use_vision_bias;
    p.top_k = route->top_k;
    p.scoring = route->scoring;
    p.scale = route->scale;
    p.weights = route->weights;
    p.indices = reinterpret_cast<long long*>(route->indices);
    p.route_scores = route->route_scores;
    p.selected = route->selected;
    p.denominator = route->denominator;
  }
  const unsigned m_tiles = static_cast<unsigned>((tokens + GM - 1) / GM);
  const unsigned n_tiles = static_cast<unsigned>(epad / GN);
  // a second K-slice when one slice per tile would leave most SMs idle
  const int slices = (static_cast<long long>(m_tiles) * n_tiles * 2 <= 2ll * sm_count() && p.k_blocks >= 4 * G_PROMOTE) ? 2 : 1;
  p.k_per_slice = ((p.k_blocks + slices - 1) / slices + G_PROMOTE - 1) / G_PROMOTE * G_PROMOTE;
  static PerDeviceFlag configured{};
  static PerDeviceFlag configured_route{};
  if (route != nullptr) {
    if (int rc2 = allow_dynamic_smem(gate_project_promoted_kernel<true>, G_SMEM_BYTES, configured_route)) return rc2;
  } else {
    if (int rc2 = allow_dynamic_smem(gate_project_promoted_kernel<false>, G_SMEM_BYTES, configured)) return rc2;
  }
  dim3 grid(m_tiles, n_tiles, static_cast<unsigned>(slices));
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = dim3(G_THREADS);
  config.dynamicSmemBytes = G_SMEM_BYTES;
  config.stream = stream;
  cudaLaunchAttribute cluster;
  cluster.id = cudaLaunchAttributeClusterDimension;
  cluster.val.clusterDim.x = 1;
  cluster.val.clusterDim.y = 1;
  cluster.val.clusterDim.z = static_cast<unsigned>(slices);  // the K-slices of a tile exchange through shared memory
  config.attrs = &cluster;
  config.numAttrs = 1;
  if (route != nullptr)
    HMC_CUDA_OK(cudaLaunchKernelEx(&config, gate_project_promoted_kernel<true>, tx, tw, p));
  else
    HMC_CUDA_OK(cudaLaunchKernelEx(&config, gate_project_promoted_kernel<false>, tx, tw, p));
  HMC_LAUNCH_OK();
  return 0;
}

}  // namespace
}  // namespace hmc

extern "C" int hmc_gate_project_promoted(const void* x_bf16, const void* w, int w_is_bf16, int64_t tokens,
                                         int64_t hidden, int64_t experts, float* logits, void* workspace,
                                         int64_t workspace_bytes, int32_t* status, void* stream_ptr) {
  return hmc::gate_promoted_launch("hmc_gate_project_promoted", x_bf16, w, w_is_bf16, tokens, hidden, experts, logits,
                                   workspace, workspace_bytes, nullptr, status, static_cast<cudaStream_t>(stream_ptr));
}

extern "C" int hmc_gate_project_route_supported(int64_t experts, int32_t n_group) {
  return experts >= 1 && experts <= hmc::GN && n_group == 0;
}

extern "C" int hmc_gate_project_route(const void* x_bf16, const void* w, int w_is_bf16, int64_t hidden, float* logits,
                                      void* workspace, int64_t workspace_bytes, const hmc_gate_route_args* route,
                                      int32_t* status, void* stream_ptr) {
  using namespace hmc;
  HMC_REQUIRE(route != nullptr, HMC_ERR_INVALID, "hmc_gate_project_route: null route arguments");
  const hmc_gate_route_args& a = *route;
  HMC_REQUIRE(hmc_gate_project_route_supported(a.experts, a.n_group), HMC_ERR_LIMIT,
              "hmc_gate_project_route: needs at most %d experts and no group limit (experts %d, n_group %d)", GN,
              a.experts, a.n_group);
  // The argument contract of hmc_gate_route; its logits are the ones this call computes.
  HMC_REQUIRE(a.tokens > 0, HMC_ERR_INVALID, "hmc_gate_project_route: tokens must be positive, got %lld",
              (long long)a.tokens);
  HMC_REQUIRE(a.top_k >= 1 && a.top_k <= a.experts, HMC_ERR_INVALID,
              "hmc_gate_project_route: top_k must be in [1, experts], got %d", a.top_k);
  HMC_REQUIRE(isfinite(a.scale), HMC_ERR_INVALID, "hmc_gate_project_route: routed scaling factor must be finite");
  HMC_REQUIRE(a.scoring >= HMC_SCORE_SQRTSOFTPLUS && a.scoring <= HMC_SCORE_SIGMOID, HMC_ERR_INVALID,
              "hmc_gate_project_route: unknown scoring function %d", a.scoring);
  HMC_REQUIRE(a.text_bias && a.weights && a.indices && a.route_scores && a.selected && a.denominator, HMC_ERR_INVALID,
              "hmc_gate_project_route: null tensor pointer");
  HMC_REQUIRE(!a.use_vision_bias || (a.vision_bias && a.image_mask), HMC_ERR_INVALID,
              "hmc_gate_project_route: vision routing needs vision_bias and image_mask");
  HMC_REQUIRE(aligned16(a.route_scores), HMC_ERR_INVALID, "hmc_gate_project_route: route_scores needs 16-byte alignment");
  return gate_promoted_launch("hmc_gate_project_route", x_bf16, w, w_is_bf16, a.tokens, hidden, a.experts, logits,
                              workspace, workspace_bytes, route, status, static_cast<cudaStream_t>(stream_ptr));
}
