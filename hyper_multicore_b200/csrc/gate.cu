// MegaGate: FP32 router projection, top-k Route and RouteGrad as single-pass warp kernels.
//
// Route follows MegaGate._torch_forward (hyper_multicore/modules/mega_gate/module.py:189-227) and
// the native 10-stage Route pipeline (hyper_multicore/ops/hyper_mega_gate/op_kernel/
// route_pipeline.h:73-562) but keeps a token's whole expert row in the registers of one warp, so
// nothing round-trips through global memory between stages. RouteGrad follows the autograd of
// the same expression (hyper_multicore/ops/hyper_mega_gate_grad/op_kernel/route_grad_pipeline.h:
// 138-191 plus the library tail hyper_mega_gate_route_grad_post.cpp:59-140).
#include <math.h>

#include "common.cuh"

namespace hmc {
namespace {

constexpr int WARPS_PER_BLOCK = 8;
constexpr float NEG_INF = -INFINITY;

__device__ __forceinline__ float softplus_ref(float x) {
  // torch softplus(beta=1, threshold=20): x > 20 ? x : log1p(exp(x))
  return x > 20.0f ? x : log1pf(expf(x));
}

// argmax over the warp; ties go to the lower expert index
__device__ __forceinline__ void warp_argmax(float& v, int& idx) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) {
      v = ov;
      idx = oi;
    }
  }
}

template <int NPL>
__global__ void __launch_bounds__(WARPS_PER_BLOCK * 32)
gate_route_kernel(const float* __restrict__ logits, const float* __restrict__ text_bias,
                  const float* __restrict__ vision_bias, const uint8_t* __restrict__ image_mask,
                  int use_vision_bias, long long tokens, int experts, int top_k, float scale,
                  int scoring, float* __restrict__ weights, long long* __restrict__ indices,
                  float* __restrict__ route_scores, float* __restrict__ selected,
                  float* __restrict__ denominator, int n_group, int topk_group) {
  extern __shared__ float group_stage[];  // [WARPS_PER_BLOCK][experts], only with n_group > 0
  const int lane = threadIdx.x & 31;
  const long long token = static_cast<long long>(blockIdx.x) * WARPS_PER_BLOCK + (threadIdx.x >> 5);
  if (token >= tokens) return;

  const float* row = logits + token * experts;
  float score[NPL];
  float biased[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int e = lane + 32 * i;
    score[i] = e < experts ? row[e] : NEG_INF;
  }
  if (scoring == HMC_SCORE_SOFTMAX) {
    float m = NEG_INF;
#pragma unroll
    for (int i = 0; i < NPL; ++i) m = fmaxf(m, score[i]);
    m = warp_max(m);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      score[i] = e < experts ? expf(score[i] - m) : 0.f;
      sum += score[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int i = 0; i < NPL; ++i) score[i] *= inv;
  } else if (scoring == HMC_SCORE_SIGMOID) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) score[i] = 1.0f / (1.0f + expf(-score[i]));
  } else {
#pragma unroll
    for (int i = 0; i < NPL; ++i) score[i] = sqrtf(softplus_ref(score[i]));
  }

  const float* bias = (use_vision_bias && image_mask[token]) ? vision_bias : text_bias;
  float* score_out = route_scores + token * experts;
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int e = lane + 32 * i;
    if (e < experts) {
      score_out[e] = score[i];
      biased[i] = __fadd_rn(score[i], bias[e]);  // never contracted with the softmax scaling: the sum torch rounds
    } else {
      biased[i] = NEG_INF;
    }
  }

  if (n_group > 0) {
    // Group limit: lane g scores group g (sum of its two largest biased scores), the warp picks the
    // topk_group best groups, experts of the other groups leave the selection.
    float* mine = group_stage + (threadIdx.x >> 5) * experts;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      if (e < experts) mine[e] = biased[i];
    }
    __syncwarp();
    const int group_size = experts / n_group;
    float group_score = NEG_INF;
    if (lane < n_group) {
      float first = NEG_INF, second = NEG_INF;
      for (int j = 0; j < group_size; ++j) {
        const float v = mine[lane * group_size + j];
        if (v > first) {
          second = first;
          first = v;
        } else if (v > second) {
          second = v;
        }
      }
      group_score = group_size > 1 ? first + second : first;
    }
    uint32_t chosen = 0;
    for (int k = 0; k < topk_group; ++k) {
      float best = (lane < n_group && !((chosen >> lane) & 1u)) ? group_score : NEG_INF;
      int best_idx = (lane < n_group && !((chosen >> lane) & 1u)) ? lane : 0x7fffffff;
      warp_argmax(best, best_idx);
      if (best_idx < 32) chosen |= 1u << best_idx;
    }
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      if (e < experts && !((chosen >> (e / group_size)) & 1u)) biased[i] = NEG_INF;
    }
  }

  // top-k by repeated warp argmax over the entries not taken yet. NaN orders as +inf (torch.topk
  // treats NaN as the largest value); ties go to the lower expert index.
  float* sel_out = selected + token * top_k;
  long long* idx_out = indices + token * top_k;
  float sum = 0.f;
  uint32_t taken = 0;
  for (int k = 0; k < top_k; ++k) {
    float best = NEG_INF;
    int best_idx = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      if (e < experts && !((taken >> i) & 1u)) {
        const float key = isnan(biased[i]) ? INFINITY : biased[i];
        if (best_idx == 0x7fffffff || key > best) {
          best = key;
          best_idx = e;
        }
      }
    }
    warp_argmax(best, best_idx);
    float win_score = 0.f;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      if (lane + 32 * i == best_idx) {
        win_score = score[i];
        taken |= 1u << i;
      }
    }
    win_score = __shfl_sync(0xffffffffu, win_score, best_idx & 31);
    sum += win_score;  // every lane accumulates the same sequence, in selection order
    if (lane == 0) {
      sel_out[k] = win_score;
      idx_out[k] = best_idx;
    }
  }
  const float denom = sum + 1.0e-20f;
  if (lane == 0) denominator[token] = denom;
  __syncwarp();
  for (int k = lane; k < top_k; k += 32) {
    float w = sel_out[k];
    if (top_k > 1) w = w / denom;
    weights[token * top_k + k] = w * scale;
  }
}

template <int NPL>
__global__ void __launch_bounds__(WARPS_PER_BLOCK * 32)
gate_route_grad_kernel(const float* __restrict__ logits, const float* __restrict__ route_scores,
                       const float* __restrict__ selected, const float* __restrict__ denominator,
                       const long long* __restrict__ indices, const float* __restrict__ grad_weights,
                       long long tokens, int experts, int top_k, float scale, int scoring,
                       float* __restrict__ grad_logits, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const long long token = static_cast<long long>(blockIdx.x) * WARPS_PER_BLOCK + (threadIdx.x >> 5);
  if (token >= tokens) return;

  const float denom = denominator[token];
  const float* sel = selected + token * top_k;
  const float* gw = grad_weights + token * top_k;
  const long long* idx = indices + token * top_k;

  // Gradient of the shared denominator: sum_k -(g_k * scale) * ((sel_k / D) / D), the order in
  // which torch's div backward evaluates it.
  float grad_denom = 0.f;
  if (top_k > 1) {
    for (int k = 0; k < top_k; ++k) grad_denom += -(gw[k] * scale) * ((sel[k] / denom) / denom);
  }
  float grad_score[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) grad_score[i] = 0.f;
  for (int k = 0; k < top_k; ++k) {
    const long long e = idx[k];
    if (e < 0 || e >= experts) {
      if (lane == 0) report_status(status, HMC_STATUS_BAD_INDEX, static_cast<int>(token), k, static_cast<int>(e));
      continue;
    }
    const float g1 = gw[k] * scale;
    const float g = top_k > 1 ? g1 / denom + grad_denom : g1;
#pragma unroll
    for (int i = 0; i < NPL; ++i)
      if (lane + 32 * i == e) grad_score[i] += g;
  }

  const float* x_row = logits + token * experts;
  const float* s_row = route_scores + token * experts;
  float* out = grad_logits + token * experts;
  if (scoring == HMC_SCORE_SOFTMAX) {
    float dot = 0.f;
    float s[NPL];
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      s[i] = e < experts ? s_row[e] : 0.f;
      dot += grad_score[i] * s[i];
    }
    dot = warp_sum(dot);
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      if (e < experts) out[e] = (grad_score[i] - dot) * s[i];
    }
  } else if (scoring == HMC_SCORE_SIGMOID) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      if (e < experts) {
        const float s = s_row[e];
        out[e] = grad_score[i] * (1.0f - s) * s;
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      if (e < experts) {
        // sqrt backward: g / (2 * sqrt(sp)); softplus backward: x > 20 ? g : g * z / (z + 1)
        const float g_sp = grad_score[i] / (2.0f * s_row[e]);
        const float x = x_row[e];
        const float z = expf(x);
        out[e] = x > 20.0f ? g_sp : g_sp * z / (z + 1.0f);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// FP32 projection logits[T, E] = float(x[T, H]) . float(W[E, H])^T on CUDA cores with FP32 FMA.
// 64 x 64 output tile per CTA, 4 x 4 per thread, K staged through shared memory in 32-wide slabs.
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename TX, typename TW>
__global__ void __launch_bounds__(256)
gate_project_kernel(const TX* __restrict__ x, const TW* __restrict__ w, long long tokens, int hidden,
                    int experts, float* __restrict__ logits) {
  constexpr int TM = 64, TN = 64, TK = 32;
  __shared__ float xs[TK][TM + 4];
  __shared__ float ws[TK][TN + 4];
  const long long t0 = static_cast<long long>(blockIdx.x) * TM;
  const int e0 = blockIdx.y * TN;
  const int tx = threadIdx.x & 15;  // expert direction
  const int ty = threadIdx.x >> 4;  // token direction
  float acc[4][4] = {};
  for (int k0 = 0; k0 < hidden; k0 += TK) {
    // 64 rows x 32 k per operand: 256 threads load 8 elements each
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int flat = threadIdx.x + 256 * i;
      const int r = flat >> 5;
      const int kk = flat & 31;
      const long long t = t0 + r;
      const int e = e0 + r;
      const int k = k0 + kk;
      xs[kk][r] = (t < tokens && k < hidden) ? to_f32<TX>(x[t * hidden + k]) : 0.f;
      ws[kk][r] = (e < experts && k < hidden) ? to_f32<TW>(w[static_cast<long long>(e) * hidden + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long t = t0 + ty * 4 + i;
    if (t >= tokens) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = e0 + tx * 4 + j;
      if (e < experts) logits[t * experts + e] = acc[i][j];
    }
  }
}

// FP32 weight [E, H] -> three BF16 parts (hi, mid, lo; hi + mid + lo == w to 24 bits) stacked as
// rows [0, E), [Epad, Epad + E), [2 Epad, 2 Epad + E) of a [3 Epad, H] matrix; other rows zero.
__global__ void gate_split_weight_kernel(const void* __restrict__ w, int w_is_bf16, int experts, int epad, int parts,
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
    const __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
    split[static_cast<long long>(epad) * hidden + i] = mid;
    split[2ll * epad * hidden + i] = lo;
  }
}

// logits[t, e] = sum of the partial products of the weight parts
__global__ void gate_sum_parts_kernel(const float* __restrict__ partial, long long tokens, int experts, int epad,
                                      int parts, float* __restrict__ logits) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= tokens * experts) return;
  const long long t = i / experts;
  const int e = static_cast<int>(i % experts);
  const float* row = partial + t * parts * epad;
  float v = row[e];
  if (parts == 3) v = (v + row[epad + e]) + row[2 * epad + e];
  logits[i] = v;
}

template <int NPL>
void launch_route(const hmc_gate_route_args& a, cudaStream_t stream) {
  const unsigned grid = static_cast<unsigned>((a.tokens + WARPS_PER_BLOCK - 1) / WARPS_PER_BLOCK);
  const size_t smem = a.n_group > 0 ? static_cast<size_t>(WARPS_PER_BLOCK) * a.experts * sizeof(float) : 0;
  gate_route_kernel<NPL><<<grid, WARPS_PER_BLOCK * 32, smem, stream>>>(
      a.logits, a.text_bias, a.vision_bias, a.image_mask, a.use_vision_bias, a.tokens, a.experts, a.top_k,
      a.scale, a.scoring, a.weights, reinterpret_cast<long long*>(a.indices), a.route_scores, a.selected,
      a.denominator, a.n_group, a.topk_group);
}

template <int NPL>
void launch_route_grad(const hmc_gate_route_grad_args& a, cudaStream_t stream) {
  const unsigned grid = static_cast<unsigned>((a.tokens + WARPS_PER_BLOCK - 1) / WARPS_PER_BLOCK);
  gate_route_grad_kernel<NPL><<<grid, WARPS_PER_BLOCK * 32, 0, stream>>>(
      a.logits, a.route_scores, a.selected, a.denominator, reinterpret_cast<const long long*>(a.indices),
      a.grad_weights, a.tokens, a.experts, a.top_k, a.scale, a.scoring, a.grad_logits, a.status);
}

#define HMC_DISPATCH_NPL(experts, CALL)                    \
  do {                                                     \
    const int npl__ = ((experts) + 31) / 32;               \
    if (npl__ <= 1) { CALL(1); }                           \
    else if (npl__ <= 2) { CALL(2); }                      \
    else if (npl__ <= 4) { CALL(4); }                      \
    else if (npl__ <= 8) { CALL(8); }                      \
    else if (npl__ <= 16) { CALL(16); }                    \
    else { CALL(32); }                                     \
  } while (0)

}  // namespace
}  // namespace hmc

extern "C" int hmc_gate_route(const hmc_gate_route_args* args, void* stream_ptr) {
  using namespace hmc;
  HMC_REQUIRE(args != nullptr, HMC_ERR_INVALID, "hmc_gate_route: null args");
  const hmc_gate_route_args& a = *args;
  // Same argument contract as the reference binding (hyper_multicore/torch/csrc/mega_gate.cpp:40-61).
  HMC_REQUIRE(a.tokens > 0, HMC_ERR_INVALID, "hmc_gate_route: tokens must be positive, got %lld", (long long)a.tokens);
  HMC_REQUIRE(a.experts > 0 && a.experts <= 1024, HMC_ERR_LIMIT,
              "hmc_gate_route: experts must be in [1, 1024], got %d", a.experts);
  HMC_REQUIRE(a.top_k >= 1 && a.top_k <= a.experts, HMC_ERR_INVALID,
              "hmc_gate_route: top_k must be in [1, experts], got %d", a.top_k);
  HMC_REQUIRE(isfinite(a.scale), HMC_ERR_INVALID, "hmc_gate_route: routed scaling factor must be finite");
  HMC_REQUIRE(a.scoring >= HMC_SCORE_SQRTSOFTPLUS && a.scoring <= HMC_SCORE_SIGMOID, HMC_ERR_INVALID,
              "hmc_gate_route: unknown scoring function %d", a.scoring);
  HMC_REQUIRE(a.logits && a.text_bias && a.weights && a.indices && a.route_scores && a.selected && a.denominator,
              HMC_ERR_INVALID, "hmc_gate_route: null tensor pointer");
  HMC_REQUIRE(!a.use_vision_bias || (a.vision_bias && a.image_mask), HMC_ERR_INVALID,
              "hmc_gate_route: vision routing needs vision_bias and image_mask");
  if (a.n_group != 0) {
    HMC_REQUIRE(a.n_group >= 1 && a.n_group <= 32 && a.experts % a.n_group == 0, HMC_ERR_INVALID,
                "hmc_gate_route: n_group (%d) must be in [1, 32] and divide experts (%d)", a.n_group, a.experts);
    HMC_REQUIRE(a.topk_group >= 1 && a.topk_group <= a.n_group, HMC_ERR_INVALID,
                "hmc_gate_route: topk_group (%d) must be in [1, n_group]", a.topk_group);
    HMC_REQUIRE(a.top_k <= a.topk_group * (a.experts / a.n_group), HMC_ERR_INVALID,
                "hmc_gate_route: top_k (%d) exceeds the experts of %d groups", a.top_k, a.topk_group);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
#define CALL(N) launch_route<N>(a, stream)
  HMC_DISPATCH_NPL(a.experts, CALL);
#undef CALL
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_gate_route_grad(const hmc_gate_route_grad_args* args, void* stream_ptr) {
  using namespace hmc;
  HMC_REQUIRE(args != nullptr, HMC_ERR_INVALID, "hmc_gate_route_grad: null args");
  const hmc_gate_route_grad_args& a = *args;
  // Contract of hyper_multicore/torch/csrc/mega_gate.cpp:132-176.
  HMC_REQUIRE(a.tokens > 0, HMC_ERR_INVALID, "hmc_gate_route_grad: tokens must be positive");
  HMC_REQUIRE(a.experts > 0 && a.experts <= 1024, HMC_ERR_LIMIT,
              "hmc_gate_route_grad: experts must be in [1, 1024], got %d", a.experts);
  HMC_REQUIRE(a.top_k >= 1 && a.top_k <= a.experts, HMC_ERR_INVALID,
              "hmc_gate_route_grad: top_k must be in [1, experts], got %d", a.top_k);
  HMC_REQUIRE(isfinite(a.scale), HMC_ERR_INVALID, "hmc_gate_route_grad: routed scaling factor must be finite");
  HMC_REQUIRE(a.scoring >= HMC_SCORE_SQRTSOFTPLUS && a.scoring <= HMC_SCORE_SIGMOID, HMC_ERR_INVALID,
              "hmc_gate_route_grad: unknown scoring function %d", a.scoring);
  HMC_REQUIRE(a.logits && a.route_scores && a.selected && a.denominator && a.indices && a.grad_weights &&
                  a.grad_logits,
              HMC_ERR_INVALID, "hmc_gate_route_grad: null tensor pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
#define CALL(N) launch_route_grad<N>(a, stream)
  HMC_DISPATCH_NPL(a.experts, CALL);
#undef CALL
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_gate_project(const void* x, int x_is_bf16, const void* w, int w_is_bf16, int64_t tokens,
                                int64_t hidden, int64_t experts, float* logits, void* stream_ptr) {
  using namespace hmc;
  HMC_REQUIRE(x && w && logits, HMC_ERR_INVALID, "hmc_gate_project: null tensor pointer");
  HMC_REQUIRE(tokens > 0 && hidden > 0 && experts > 0, HMC_ERR_INVALID,
              "hmc_gate_project: extents must be positive");
  HMC_REQUIRE(hidden < (1ll << 31) && experts < 65536 * 64, HMC_ERR_LIMIT, "hmc_gate_project: extent too large");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  dim3 grid(static_cast<unsigned>((tokens + 63) / 64), static_cast<unsigned>((experts + 63) / 64));
  const int h = static_cast<int>(hidden), e = static_cast<int>(experts);
  if (x_is_bf16 && w_is_bf16)
    gate_project_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), tokens, h, e, logits);
  else if (x_is_bf16)
    gate_project_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(w), tokens, h, e, logits);
  else if (w_is_bf16)
    gate_project_kernel<float, __nv_bfloat16><<<grid, 256, 0, stream>>>(
        static_cast<const float*>(x), static_cast<const __nv_bfloat16*>(w), tokens, h, e, logits);
  else
    gate_project_kernel<float, float><<<grid, 256, 0, stream>>>(static_cast<const float*>(x),
                                                                static_cast<const float*>(w), tokens, h, e, logits);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int64_t hmc_gate_project_workspace_bytes(int64_t tokens, int64_t hidden, int64_t experts) {
  const int64_t epad = (experts + 7) / 8 * 8;
  return 3 * epad * hidden * 2 + tokens * 3 * epad * 4 + 512;
}

// Tensor-core projection for BF16 hidden states: the FP32 weight is split into three BF16 parts whose
// sum reproduces it to 24 bits, the products with the (exact) BF16 activations accumulate in FP32 on
// tcgen05, and the three partial results are added. FP32 hidden states use hmc_gate_project.
extern "C" int hmc_gate_project_tc(const void* x_bf16, const void* w, int w_is_bf16, int64_t tokens, int64_t hidden,
                                   int64_t experts, float* logits, void* workspace, int64_t workspace_bytes,
                                   void* stream_ptr) {
  using namespace hmc;
  HMC_REQUIRE(x_bf16 && w && logits && workspace, HMC_ERR_INVALID, "hmc_gate_project_tc: null tensor pointer");
  HMC_REQUIRE(tokens > 0 && experts > 0 && hidden > 0 && hidden % 8 == 0, HMC_ERR_INVALID,
              "hmc_gate_project_tc: extents must be positive and hidden a multiple of 8");
  HMC_REQUIRE(workspace_bytes >= hmc_gate_project_workspace_bytes(tokens, hidden, experts), HMC_ERR_INVALID,
              "hmc_gate_project_tc: workspace holds %lld bytes, %lld needed", (long long)workspace_bytes,
              (long long)hmc_gate_project_workspace_bytes(tokens, hidden, experts));
  HMC_REQUIRE(aligned16(x_bf16) && aligned16(workspace), HMC_ERR_INVALID, "hmc_gate_project_tc: 16-byte alignment");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const int epad = static_cast<int>((experts + 7) / 8 * 8);
  const int parts = w_is_bf16 ? 1 : 3;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  __nv_bfloat16* split = reinterpret_cast<__nv_bfloat16*>(ws);
  float* partial = reinterpret_cast<float*>(ws + 3ll * epad * hidden * 2);
  long long* ends = reinterpret_cast<long long*>(ws + 3ll * epad * hidden * 2 + tokens * 3ll * epad * 4);
  ends = reinterpret_cast<long long*>((reinterpret_cast<uintptr_t>(ends) + 15) & ~static_cast<uintptr_t>(15));
  const long long split_elems = static_cast<long long>(epad) * hidden;
  gate_split_weight_kernel<<<static_cast<unsigned>((split_elems + 255) / 256), 256, 0, stream>>>(
      w, w_is_bf16, static_cast<int>(experts), epad, parts, hidden, split);
  HMC_LAUNCH_OK();
  HMC_CUDA_OK(cudaMemcpyAsync(ends, &tokens, sizeof(long long), cudaMemcpyHostToDevice, stream));
  hmc_grouped_gemm_args g{};
  g.mode = HMC_GEMM_RAGGED_M;
  g.a_major = HMC_MAJOR_K;
  g.b_major = HMC_MAJOR_K;
  g.epilogue = HMC_EPI_STORE_F32;
  g.groups = 1;
  g.tile_mode = HMC_TILE_SINGLE;
  g.rows = tokens;
  g.n = static_cast<int64_t>(parts) * epad;
  g.k = hidden;
  g.a = x_bf16;
  g.b = split;
  g.c = partial;
  g.group_ends = reinterpret_cast<const int64_t*>(ends);
  int rc = hmc_grouped_gemm(&g, stream);
  if (rc != 0) return rc;
  const long long total = tokens * experts;
  gate_sum_parts_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      partial, tokens, static_cast<int>(experts), epad, parts, logits);
  HMC_LAUNCH_OK();
  return 0;
}
