// MegaMHC: four-stream residual mix + mapping prediction (sigmoid / Sinkhorn) + RMSNorm, forward
// and backward, as streaming warp-per-token kernels. The 24-wide projection against phi and its
// two backward contractions are issued to the tcgen05 grouped GEMM by the entry points below.
//
// Math follows the reference's semantic oracle torch_mega_mhc / _predict_mappings / _sinkhorn
// (tests/common/multicore/mega_mhc_golden.py:29-142) and its autograd
// (tests/common/multicore/mega_mhc_grad_golden.py:117-193). Stage order mirrors the native worker
// (hyper_multicore/ops/hyper_mega_mhc/op_kernel/worker_kernel.cpp:92-268): Post, NormCast,
// Projection (un-normalised dot, then scaled by 1/rms), InputMix in BF16, Mapping, RMSNorm.
#include <math.h>

#include "common.cuh"

namespace hmc {
namespace {

constexpr int STREAMS = 4;
constexpr int MIX = 24;       // 4 pre + 4 post + 16 residual-mix logits
constexpr int MIX_PAD = 32;   // padded width of one BF16 split part
constexpr int WARPS = 8;

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                    pack_bf16x2(f[6], f[7]));
}
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// ---------------------------------------------------------------------------------------------
// Forward, stage 1 (one warp per token): residual post-mix, both RMS statistics, BF16 input mix,
// final RMSNorm. The token's mixed row is re-read from the cache line this lane wrote itself.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(WARPS * 32, 2)
mhc_post_kernel(const uint4* __restrict__ prev_out, const uint4* __restrict__ residual,
                const float* __restrict__ prev_pre, const float* __restrict__ prev_post,
                const float* __restrict__ prev_mix, const uint4* __restrict__ norm_weight, long long tokens,
                int hidden, float norm_eps, uint4* __restrict__ new_residual, uint4* __restrict__ mixed_input,
                uint4* __restrict__ block_input, float* __restrict__ inv_rms, float* __restrict__ rms_rstd) {
  const int lane = threadIdx.x & 31;
  const long long t = static_cast<long long>(blockIdx.x) * WARPS + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const int vec = hidden / 8;
  float mix[STREAMS][STREAMS], post[STREAMS], pre[STREAMS];
#pragma unroll
  for (int j = 0; j < STREAMS; ++j) {
    post[j] = prev_post[t * STREAMS + j];
    pre[j] = prev_pre[t * STREAMS + j];
#pragma unroll
    for (int i = 0; i < STREAMS; ++i) mix[j][i] = prev_mix[(t * STREAMS + j) * STREAMS + i];
  }
  const uint4* res_row = residual + t * STREAMS * vec;
  const uint4* out_row = prev_out + t * vec;
  uint4* new_row = new_residual + t * STREAMS * vec;
  uint4* mixed_row = mixed_input + t * vec;
  float sumsq = 0.f, sumsq_mixed = 0.f;
#pragma unroll 2
  for (int v = lane; v < vec; v += 32) {
    float r[STREAMS][8], o[8];
#pragma unroll
    for (int j = 0; j < STREAMS; ++j) unpack8(ld_nc_16(res_row + j * vec + v), r[j]);
    unpack8(ld_nc_16(out_row + v), o);
    float mixed[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < STREAMS; ++i) {
      float n[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float acc = mix[0][i] * r[0][e];
#pragma unroll
        for (int j = 1; j < STREAMS; ++j) acc = fmaf(mix[j][i], r[j][e], acc);
        n[e] = bf16_round(acc + post[i] * o[e]);
        sumsq = fmaf(n[e], n[e], sumsq);
        mixed[e] = fmaf(n[e], pre[i], mixed[e]);
      }
      st_16(new_row + i * vec + v, pack8(n));
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) sumsq_mixed = fmaf(mixed[e], mixed[e], sumsq_mixed);
    st_16(mixed_row + v, pack8(mixed));
  }
  sumsq = warp_sum(sumsq);
  sumsq_mixed = warp_sum(sumsq_mixed);
  const float r4 = rsqrtf(sumsq / static_cast<float>(STREAMS * hidden) + norm_eps);
  const float rstd = rsqrtf(sumsq_mixed / static_cast<float>(hidden) + norm_eps);
  if (lane == 0) {
    inv_rms[t] = r4;
    rms_rstd[t] = rstd;
  }
  uint4* block_row = block_input + t * vec;
  for (int v = lane; v < vec; v += 32) {
    float m[8], w[8], y[8];
    unpack8(ld_16(mixed_row + v), m);
    unpack8(ld_16(norm_weight + v), w);
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = (m[e] * rstd) * w[e];
    st_cs_16(block_row + v, pack8(y));
  }
}

// Sinkhorn forward on a 4x4 matrix held in registers; `sums` (optional) receives the 40 x 4
// normalisers: step 0 = softmax row denominators, odd steps = column sums + eps, even = row sums + eps.
__device__ __forceinline__ void sinkhorn_forward(const float (&logit)[16], float eps, int iters, float (&m)[16],
                                                 float* sums, float* sum_out, float* norm_out, long long t,
                                                 long long tokens) {
  auto emit = [&](int step, const float (&s)[4]) {
    if (sums != nullptr)
      for (int i = 0; i < 4; ++i) sums[step * 4 + i] = s[i];
    if (sum_out != nullptr)
      for (int i = 0; i < 4; ++i) sum_out[(static_cast<long long>(step) * tokens + t) * 4 + i] = s[i];
    if (norm_out != nullptr)
      for (int i = 0; i < 16; ++i) norm_out[(static_cast<long long>(step) * tokens + t) * 16 + i] = m[i];
  };
  float s[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    float mx = fmaxf(fmaxf(logit[r * 4], logit[r * 4 + 1]), fmaxf(logit[r * 4 + 2], logit[r * 4 + 3]));
    float e[4], den = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      e[c] = expf(logit[r * 4 + c] - mx);
      den += e[c];
    }
    s[r] = den;
    const float inv = 1.0f / den;  // one division per normaliser; the four entries take a multiplication each
#pragma unroll
    for (int c = 0; c < 4; ++c) m[r * 4 + c] = e[c] * inv + eps;
  }
  emit(0, s);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    s[c] = m[c] + m[4 + c] + m[8 + c] + m[12 + c] + eps;
    const float inv = 1.0f / s[c];
#pragma unroll
    for (int r = 0; r < 4; ++r) m[r * 4 + c] *= inv;
  }
  emit(1, s);
  for (int it = 1; it < iters; ++it) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      s[r] = m[r * 4] + m[r * 4 + 1] + m[r * 4 + 2] + m[r * 4 + 3] + eps;
      const float inv = 1.0f / s[r];
#pragma unroll
      for (int c = 0; c < 4; ++c) m[r * 4 + c] *= inv;
    }
    emit(2 * it, s);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      s[c] = m[c] + m[4 + c] + m[8 + c] + m[12 + c] + eps;
      const float inv = 1.0f / s[c];
#pragma unroll
      for (int r = 0; r < 4; ++r) m[r * 4 + c] *= inv;
    }
    emit(2 * it + 1, s);
  }
}

// Forward, stage 3 (one thread per token): combine the split projection, scale, map.
__global__ void __launch_bounds__(128)
mhc_mapping_kernel(const float* __restrict__ q_parts, const float* __restrict__ inv_rms,
                   const float* __restrict__ alpha, const float* __restrict__ bias, long long tokens,
                   float hc_eps, int iters, float* __restrict__ next_pre, float* __restrict__ next_post,
                   float* __restrict__ next_mix, float* __restrict__ hc_before_norm, float* __restrict__ sum_out,
                   float* __restrict__ norm_out) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  const float r = inv_rms[t];
  const float a0 = alpha[0], a1 = alpha[1], a2 = alpha[2];
  float l[MIX];
#pragma unroll
  for (int c = 0; c < MIX; ++c) {
    const float q = q_parts[t * 4 * MIX_PAD + c] + q_parts[t * 4 * MIX_PAD + MIX_PAD + c];
    if (hc_before_norm != nullptr) hc_before_norm[t * MIX + c] = q;
    l[c] = q * r;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    next_pre[t * 4 + i] = sigmoid_f(l[i] * a0 + bias[i]) + hc_eps;
    next_post[t * 4 + i] = 2.0f * sigmoid_f(l[4 + i] * a1 + bias[4 + i]);
  }
  float logit[16], m[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) logit[i] = l[8 + i] * a2 + bias[8 + i];
  sinkhorn_forward(logit, hc_eps, iters, m, nullptr, sum_out, norm_out, t, tokens);
#pragma unroll
  for (int i = 0; i < 16; ++i) next_mix[t * 16 + i] = m[i];
}

// phi [24, K] FP32 -> BF16 split rows [128, K] shared by the forward and backward GEMMs:
//   rows 0..23 = hi, 32..55 = lo residual (hi + lo carries 16 mantissa bits), 64..87 = hi again,
//   every other row zero. Forward reads it as B[n, k] (columns 0..63 of the result matter);
//   backward reads it as B[kk, n] against dq laid out as hi | hi | lo | 0.
__global__ void mhc_split_phi_kernel(const float* __restrict__ phi, long long k, __nv_bfloat16* __restrict__ split) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= k) return;
  const __nv_bfloat16 zero = __float2bfloat16_rn(0.f);
  for (int c = 0; c < MIX_PAD; ++c) {
    __nv_bfloat16 hi = zero, lo = zero;
    if (c < MIX) {
      const float v = phi[static_cast<long long>(c) * k + i];
      hi = __float2bfloat16_rn(v);
      lo = __float2bfloat16_rn(v - __bfloat162float(hi));
    }
    split[static_cast<long long>(c) * k + i] = hi;
    split[static_cast<long long>(MIX_PAD + c) * k + i] = lo;
    split[static_cast<long long>(2 * MIX_PAD + c) * k + i] = hi;
    split[static_cast<long long>(3 * MIX_PAD + c) * k + i] = zero;
  }
}

// ---------------------------------------------------------------------------------------------
// Backward, stage 1 (one thread per token): gradients of the mapping head. Recomputes the
// Sinkhorn chain from the cached un-normalised projection, walks it backwards using only the
// normalisers, and emits dq (gradient w.r.t. the un-normalised projection) split into BF16 parts
// for the two tensor-core contractions, the per-token coefficient of the RMS term, and block-level
// partial sums of dalpha / dbias.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
mhc_mapping_grad_kernel(const float* __restrict__ hc_before_norm, const float* __restrict__ inv_rms,
                        const float* __restrict__ alpha, const float* __restrict__ bias,
                        const float* __restrict__ grad_pre, const float* __restrict__ grad_post,
                        const float* __restrict__ grad_mix, long long tokens, int hidden, float hc_eps, int iters,
                        __nv_bfloat16* __restrict__ dq_rows,  // [tokens, 128]: hi | hi | lo | 0
                        __nv_bfloat16* __restrict__ dq_cols,  // [tokens, 64] : hi | lo
                        float* __restrict__ rms_coef, float* __restrict__ grad_alpha, float* __restrict__ grad_bias) {
  __shared__ float red[MIX + 3];
  if (threadIdx.x < MIX + 3) red[threadIdx.x] = 0.f;
  __syncthreads();
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t < tokens) {
    const float r = inv_rms[t];
    const float al[3] = {alpha[0], alpha[1], alpha[2]};
    float q[MIX], l[MIX], da[MIX];
#pragma unroll
    for (int c = 0; c < MIX; ++c) {
      q[c] = hc_before_norm[t * MIX + c];
      l[c] = q[c] * r;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float sp = sigmoid_f(l[i] * al[0] + bias[i]);
      da[i] = grad_pre[t * 4 + i] * sp * (1.0f - sp);
      const float so = sigmoid_f(l[4 + i] * al[1] + bias[4 + i]);
      da[4 + i] = 2.0f * grad_post[t * 4 + i] * so * (1.0f - so);
    }
    float logit[16], m[16], sums[160], g[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) logit[i] = l[8 + i] * al[2] + bias[8 + i];
    sinkhorn_forward(logit, hc_eps, iters, m, sums, nullptr, nullptr, t, tokens);
#pragma unroll
    for (int i = 0; i < 16; ++i) g[i] = grad_mix[t * 16 + i];
    // Each normalisation is out = in / s with s = sum(in) + eps along one axis, so
    // d_in = d_out / s - sum(d_out * out) / s along that axis, and in = out * s.
    for (int step = 2 * iters - 1; step >= 1; --step) {
      const float* s = sums + step * 4;
      if (step & 1) {  // column normalisation
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float dot = 0.f;
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) dot += g[rr * 4 + c] * m[rr * 4 + c];
          const float inv = 1.0f / s[c];
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) {
            g[rr * 4 + c] = (g[rr * 4 + c] - dot) * inv;
            m[rr * 4 + c] *= s[c];
          }
        }
      } else {  // row normalisation
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) {
          float dot = 0.f;
#pragma unroll
          for (int c = 0; c < 4; ++c) dot += g[rr * 4 + c] * m[rr * 4 + c];
          const float inv = 1.0f / s[rr];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            g[rr * 4 + c] = (g[rr * 4 + c] - dot) * inv;
            m[rr * 4 + c] *= s[rr];
          }
        }
      }
    }
    // step 0: m = softmax(logit) + eps
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
      float dot = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) dot += g[rr * 4 + c] * (m[rr * 4 + c] - hc_eps);
#pragma unroll
      for (int c = 0; c < 4; ++c) da[8 + rr * 4 + c] = (m[rr * 4 + c] - hc_eps) * (g[rr * 4 + c] - dot);
    }
    // a_c = l_c * alpha_k + bias_c ; l_c = q_c * r
    float dr = 0.f, dalpha[3] = {0.f, 0.f, 0.f};
    __nv_bfloat16* rows = dq_rows + t * 4 * MIX_PAD;
    __nv_bfloat16* cols = dq_cols + t * 2 * MIX_PAD;
    const __nv_bfloat16 zero = __float2bfloat16_rn(0.f);
#pragma unroll
    for (int c = 0; c < MIX_PAD; ++c) {
      __nv_bfloat16 hi = zero, lo = zero;
      if (c < MIX) {
        const int k = c < 4 ? 0 : (c < 8 ? 1 : 2);
        const float dl = da[c] * al[k];
        dalpha[k] += da[c] * l[c];
        dr += dl * q[c];
        const float dq = dl * r;
        hi = __float2bfloat16_rn(dq);
        lo = __float2bfloat16_rn(dq - __bfloat162float(hi));
        atomicAdd(&red[c], da[c]);
      }
      rows[c] = hi;
      rows[MIX_PAD + c] = hi;
      rows[2 * MIX_PAD + c] = lo;
      rows[3 * MIX_PAD + c] = zero;
      cols[c] = hi;
      cols[MIX_PAD + c] = lo;
    }
    // r = (S + eps)^-1/2 with S = sum(R^2) / (4H): dR += R * (-r^3 * dr / (4H))
    rms_coef[t] = -(r * r * r) * dr / static_cast<float>(STREAMS * hidden);
#pragma unroll
    for (int k = 0; k < 3; ++k) atomicAdd(&red[MIX + k], dalpha[k]);
  }
  __syncthreads();
  if (threadIdx.x < MIX) atomicAdd(&grad_bias[threadIdx.x], red[threadIdx.x]);
  else if (threadIdx.x < MIX + 3) atomicAdd(&grad_alpha[threadIdx.x - MIX], red[threadIdx.x]);
}

// ---------------------------------------------------------------------------------------------
// Backward, stage 2 (one warp per token): everything that streams over the hidden dimension.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(WARPS * 32, 2)
mhc_stream_grad_kernel(const uint4* __restrict__ grad_new_residual, const uint4* __restrict__ grad_block_input,
                       const uint4* __restrict__ new_residual, const uint4* __restrict__ mixed_input,
                       const uint4* __restrict__ residual, const uint4* __restrict__ prev_out,
                       const uint4* __restrict__ proj_grad,  // dq . phi, BF16 [tokens, 4H]
                       const uint4* __restrict__ norm_weight, const float* __restrict__ prev_pre,
                       const float* __restrict__ prev_post, const float* __restrict__ prev_mix,
                       const float* __restrict__ rms_rstd, const float* __restrict__ rms_coef, long long tokens,
                       int hidden, uint4* __restrict__ grad_residual, uint4* __restrict__ grad_prev_out,
                       float* __restrict__ grad_prev_pre, float* __restrict__ grad_prev_post,
                       float* __restrict__ grad_prev_mix) {
  const int vec = hidden / 8;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  for (long long t = static_cast<long long>(blockIdx.x) * WARPS + warp; t < tokens;
       t += static_cast<long long>(gridDim.x) * WARPS) {
    float mix[STREAMS][STREAMS], post[STREAMS], pre[STREAMS];
#pragma unroll
    for (int j = 0; j < STREAMS; ++j) {
      post[j] = prev_post[t * STREAMS + j];
      pre[j] = prev_pre[t * STREAMS + j];
#pragma unroll
      for (int i = 0; i < STREAMS; ++i) mix[j][i] = prev_mix[(t * STREAMS + j) * STREAMS + i];
    }
    const float rstd = rms_rstd[t];
    const float coef = rms_coef[t];
    const uint4* gb_row = grad_block_input + t * vec;
    const uint4* mixed_row = mixed_input + t * vec;
    // pass 1: sum_h (g_block * w) * mixed
    float dot = 0.f;
    for (int v = lane; v < vec; v += 32) {
      float gb[8], w[8], m[8];
      unpack8(ld_16(gb_row + v), gb);
      unpack8(ld_16(norm_weight + v), w);
      unpack8(ld_16(mixed_row + v), m);
#pragma unroll
      for (int e = 0; e < 8; ++e) dot = fmaf(gb[e] * w[e], m[e], dot);
    }
    dot = warp_sum(dot);
    const float back = rstd * rstd * rstd * dot / static_cast<float>(hidden);
    float d_pre[STREAMS] = {0.f, 0.f, 0.f, 0.f}, d_post[STREAMS] = {0.f, 0.f, 0.f, 0.f};
    float d_mix[STREAMS][STREAMS] = {};
    const uint4* new_row = new_residual + t * STREAMS * vec;
    const uint4* gn_row = grad_new_residual + t * STREAMS * vec;
    const uint4* pg_row = proj_grad + t * STREAMS * vec;
    const uint4* res_row = residual + t * STREAMS * vec;
    uint4* gres_row = grad_residual + t * STREAMS * vec;
    for (int v = lane; v < vec; v += 32) {
      float gb[8], w[8], m[8], d_mixed[8];
      unpack8(ld_16(gb_row + v), gb);
      unpack8(ld_16(norm_weight + v), w);
      unpack8(ld_16(mixed_row + v), m);
#pragma unroll
      for (int e = 0; e < 8; ++e) d_mixed[e] = rstd * (gb[e] * w[e]) - m[e] * back;
      float dR[STREAMS][8];
#pragma unroll
      for (int i = 0; i < STREAMS; ++i) {
        float R[8], gn[8], pg[8];
        unpack8(ld_nc_16(new_row + i * vec + v), R);
        unpack8(ld_nc_16(gn_row + i * vec + v), gn);
        unpack8(ld_nc_16(pg_row + i * vec + v), pg);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          dR[i][e] = gn[e] + pre[i] * d_mixed[e] + coef * R[e] + pg[e];
          d_pre[i] = fmaf(d_mixed[e], R[e], d_pre[i]);
        }
      }
      float o[8], d_out[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      unpack8(ld_nc_16(prev_out + t * vec + v), o);
#pragma unroll
      for (int i = 0; i < STREAMS; ++i) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          d_out[e] = fmaf(post[i], dR[i][e], d_out[e]);
          d_post[i] = fmaf(o[e], dR[i][e], d_post[i]);
        }
      }
      st_cs_16(grad_prev_out + t * vec + v, pack8(d_out));
#pragma unroll
      for (int j = 0; j < STREAMS; ++j) {
        float r[8], d_res[8];
        unpack8(ld_nc_16(res_row + j * vec + v), r);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float acc = 0.f;
#pragma unroll
          for (int i = 0; i < STREAMS; ++i) {
            acc = fmaf(mix[j][i], dR[i][e], acc);
            d_mix[j][i] = fmaf(r[e], dR[i][e], d_mix[j][i]);
          }
          d_res[e] = acc;
        }
        st_cs_16(gres_row + j * vec + v, pack8(d_res));
      }
    }
#pragma unroll
    for (int i = 0; i < STREAMS; ++i) {
      d_pre[i] = warp_sum(d_pre[i]);
      d_post[i] = warp_sum(d_post[i]);
#pragma unroll
      for (int j = 0; j < STREAMS; ++j) d_mix[j][i] = warp_sum(d_mix[j][i]);
    }
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < STREAMS; ++i) {
        grad_prev_pre[t * STREAMS + i] = d_pre[i];
        grad_prev_post[t * STREAMS + i] = d_post[i];
#pragma unroll
        for (int j = 0; j < STREAMS; ++j) grad_prev_mix[(t * STREAMS + j) * STREAMS + i] = d_mix[j][i];
      }
    }
  }
}

// d norm_weight[h] = sum_t grad_block_input[t, h] * mixed_input[t, h] * rstd[t]: a column reduction.
// Block = 32 column vectors x 8 token lanes; every thread keeps 8 FP32 partial sums in registers.
__global__ void __launch_bounds__(256)
mhc_norm_weight_grad_kernel(const uint4* __restrict__ grad_block_input, const uint4* __restrict__ mixed_input,
                            const float* __restrict__ rms_rstd, long long tokens, int vec,
                            float* __restrict__ grad_norm_weight) {
  __shared__ float red[8][32][9];
  const int tx = threadIdx.x & 31;
  const int ty = threadIdx.x >> 5;
  const int v = blockIdx.x * 32 + tx;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (v < vec) {
    const long long step = static_cast<long long>(gridDim.y) * 8;
#pragma unroll 4
    for (long long t = static_cast<long long>(blockIdx.y) * 8 + ty; t < tokens; t += step) {
      float gb[8], m[8];
      unpack8(ld_nc_16(grad_block_input + t * vec + v), gb);
      unpack8(ld_nc_16(mixed_input + t * vec + v), m);
      const float r = rms_rstd[t];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = fmaf(gb[e] * m[e], r, acc[e]);
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) red[ty][tx][e] = acc[e];
  __syncthreads();
  // thread (ty, tx) sums column e = ty of vector tx over the 8 token lanes
  if (v < vec) {
    float total = 0.f;
#pragma unroll
    for (int y = 0; y < 8; ++y) total += red[y][tx][ty];
    atomicAdd(grad_norm_weight + static_cast<long long>(v) * 8 + ty, total);
  }
}

// dphi[c, k] = parts[c, k] + parts[32 + c, k]
__global__ void mhc_combine_dphi_kernel(const float* __restrict__ parts, long long k, float* __restrict__ grad_phi) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= k) return;
  for (int c = 0; c < MIX; ++c)
    grad_phi[static_cast<long long>(c) * k + i] =
        parts[static_cast<long long>(c) * k + i] + parts[static_cast<long long>(MIX_PAD + c) * k + i];
}

__global__ void fill_i64_kernel(long long* p, long long v) { *p = v; }

int run_gemm(const hmc_grouped_gemm_args& g, cudaStream_t stream) {
  return hmc_grouped_gemm(&g, stream);
}

}  // namespace
}  // namespace hmc

using namespace hmc;

extern "C" int64_t hmc_mega_mhc_workspace_bytes(int64_t tokens, int64_t hidden) {
  // phi split [128, 4H] bf16 + projection parts [tokens, 128] f32 + one int64 group end
  return 128 * 4 * hidden * 2 + tokens * 128 * 4 + 256;
}

extern "C" int64_t hmc_mega_mhc_grad_workspace_bytes(int64_t tokens, int64_t hidden) {
  const int64_t k = 4 * hidden;
  // phi split [128, 4H] bf16, dq_rows [T,128] bf16, dq_cols [T,64] bf16, proj_grad [T,4H] bf16,
  // dphi parts [64, 4H] f32, rms_coef [T] f32, one int64 group end
  return 128 * k * 2 + tokens * 128 * 2 + tokens * 64 * 2 + tokens * k * 2 + 64 * k * 4 + tokens * 4 + 1024;
}

static int check_mhc_dims(const char* what, int64_t tokens, int64_t hidden, int32_t num_iters) {
  HMC_REQUIRE(tokens > 0 && tokens < (1ll << 31) / 16, HMC_ERR_INVALID, "%s: token count %lld out of range", what,
              (long long)tokens);
  // hidden % 128 == 0 is the reference's rule (hyper_multicore/modules/mega_mhc_common.py:100-118);
  // its upper bounds on hidden are Ascend buffer limits and do not apply here.
  HMC_REQUIRE(hidden > 0 && hidden % 128 == 0, HMC_ERR_INVALID, "%s: hidden size (%lld) must be a multiple of 128",
              what, (long long)hidden);
  HMC_REQUIRE(num_iters >= 1 && num_iters <= 20, HMC_ERR_INVALID, "%s: num_iters must be in [1, 20], got %d", what,
              num_iters);
  return 0;
}

extern "C" int hmc_mega_mhc(const hmc_mega_mhc_args* args, void* stream_ptr) {
  HMC_REQUIRE(args != nullptr, HMC_ERR_INVALID, "hmc_mega_mhc: null args");
  const hmc_mega_mhc_args& a = *args;
  int rc = check_mhc_dims("hmc_mega_mhc", a.tokens, a.hidden, a.num_iters);
  if (rc != 0) return rc;
  HMC_REQUIRE(a.previous_output && a.residual && a.previous_pre_mix && a.previous_post_mix &&
                  a.previous_residual_mix && a.phi && a.alpha && a.bias && a.norm_weight && a.new_residual &&
                  a.next_pre_mix && a.next_post_mix && a.next_residual_mix && a.block_input && a.inv_rms &&
                  a.mixed_input && a.rms_rstd && a.workspace,
              HMC_ERR_INVALID, "hmc_mega_mhc: null tensor pointer");
  HMC_REQUIRE(a.workspace_bytes >= hmc_mega_mhc_workspace_bytes(a.tokens, a.hidden), HMC_ERR_INVALID,
              "hmc_mega_mhc: workspace holds %lld bytes, %lld needed", (long long)a.workspace_bytes,
              (long long)hmc_mega_mhc_workspace_bytes(a.tokens, a.hidden));
  HMC_REQUIRE(aligned16(a.previous_output) && aligned16(a.residual) && aligned16(a.new_residual) &&
                  aligned16(a.block_input) && aligned16(a.mixed_input) && aligned16(a.norm_weight) &&
                  aligned16(a.workspace),
              HMC_ERR_INVALID, "hmc_mega_mhc: activations must be 16-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const int hidden = static_cast<int>(a.hidden);
  const long long k = 4ll * a.hidden;
  uint8_t* ws = static_cast<uint8_t*>(a.workspace);
  __nv_bfloat16* phi_split = reinterpret_cast<__nv_bfloat16*>(ws);
  float* q_parts = reinterpret_cast<float*>(ws + 128 * k * 2);
  long long* ends = reinterpret_cast<long long*>(ws + 128 * k * 2 + a.tokens * 128 * 4);

  mhc_post_kernel<<<static_cast<unsigned>((a.tokens + WARPS - 1) / WARPS), WARPS * 32, 0, stream>>>(
      static_cast<const uint4*>(a.previous_output), static_cast<const uint4*>(a.residual), a.previous_pre_mix,
      a.previous_post_mix, a.previous_residual_mix, static_cast<const uint4*>(a.norm_weight), a.tokens, hidden,
      a.norm_eps, static_cast<uint4*>(a.new_residual), static_cast<uint4*>(a.mixed_input),
      static_cast<uint4*>(a.block_input), a.inv_rms, a.rms_rstd);
  HMC_LAUNCH_OK();
  mhc_split_phi_kernel<<<static_cast<unsigned>((k + 255) / 256), 256, 0, stream>>>(a.phi, k, phi_split);
  HMC_LAUNCH_OK();
  fill_i64_kernel<<<1, 1, 0, stream>>>(ends, a.tokens);
  HMC_LAUNCH_OK();
  hmc_grouped_gemm_args g{};
  g.mode = HMC_GEMM_RAGGED_M;
  g.a_major = HMC_MAJOR_K;
  g.b_major = HMC_MAJOR_K;
  g.epilogue = HMC_EPI_STORE_F32;
  g.groups = 1;
  g.rows = a.tokens;
  g.n = 4 * MIX_PAD;
  g.k = k;
  g.a = a.new_residual;
  g.b = phi_split;
  g.c = q_parts;
  g.group_ends = reinterpret_cast<const int64_t*>(ends);
  g.status = a.status;
  rc = run_gemm(g, stream);
  if (rc != 0) return rc;
  mhc_mapping_kernel<<<static_cast<unsigned>((a.tokens + 31) / 32), 32, 0, stream>>>(
      q_parts, a.inv_rms, a.alpha, a.bias, a.tokens, a.hc_eps, a.num_iters, a.next_pre_mix, a.next_post_mix,
      a.next_residual_mix, a.hc_before_norm, a.need_backward ? a.sum_out : nullptr,
      a.need_backward ? a.norm_out : nullptr);
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_mega_mhc_grad(const hmc_mega_mhc_grad_args* args, void* stream_ptr) {
  HMC_REQUIRE(args != nullptr, HMC_ERR_INVALID, "hmc_mega_mhc_grad: null args");
  const hmc_mega_mhc_grad_args& a = *args;
  int rc = check_mhc_dims("hmc_mega_mhc_grad", a.tokens, a.hidden, a.num_iters);
  if (rc != 0) return rc;
  HMC_REQUIRE(a.grad_new_residual && a.grad_next_pre_mix && a.grad_next_post_mix && a.grad_next_residual_mix &&
                  a.grad_block_input && a.new_residual && a.hc_before_norm && a.inv_rms && a.mixed_input &&
                  a.rms_rstd && a.previous_output && a.residual && a.previous_pre_mix && a.previous_post_mix &&
                  a.previous_residual_mix && a.phi && a.alpha && a.bias && a.norm_weight && a.grad_residual &&
                  a.grad_phi && a.grad_alpha && a.grad_bias && a.grad_previous_output && a.grad_previous_pre_mix &&
                  a.grad_previous_post_mix && a.grad_previous_residual_mix && a.grad_norm_weight && a.workspace,
              HMC_ERR_INVALID, "hmc_mega_mhc_grad: null tensor pointer");
  HMC_REQUIRE(a.workspace_bytes >= hmc_mega_mhc_grad_workspace_bytes(a.tokens, a.hidden), HMC_ERR_INVALID,
              "hmc_mega_mhc_grad: workspace holds %lld bytes, %lld needed", (long long)a.workspace_bytes,
              (long long)hmc_mega_mhc_grad_workspace_bytes(a.tokens, a.hidden));
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const int hidden = static_cast<int>(a.hidden);
  const long long k = 4ll * a.hidden;
  const long long T = a.tokens;
  uint8_t* ws = static_cast<uint8_t*>(a.workspace);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    uint8_t* p = ws + off;
    off += (bytes + 255) & ~static_cast<size_t>(255);
    return p;
  };
  __nv_bfloat16* phi_split = reinterpret_cast<__nv_bfloat16*>(take(128 * k * 2));
  __nv_bfloat16* dq_rows = reinterpret_cast<__nv_bfloat16*>(take(T * 128 * 2));
  __nv_bfloat16* dq_cols = reinterpret_cast<__nv_bfloat16*>(take(T * 64 * 2));
  __nv_bfloat16* proj_grad = reinterpret_cast<__nv_bfloat16*>(take(T * k * 2));
  float* dphi_parts = reinterpret_cast<float*>(take(64 * k * 4));
  float* rms_coef = reinterpret_cast<float*>(take(T * 4));
  long long* ends = reinterpret_cast<long long*>(take(8));
  HMC_REQUIRE(static_cast<int64_t>(off) <= a.workspace_bytes, HMC_ERR_INVALID,
              "hmc_mega_mhc_grad: workspace too small after alignment (%lld needed)", (long long)off);

  HMC_CUDA_OK(cudaMemsetAsync(a.grad_alpha, 0, 3 * sizeof(float), stream));
  HMC_CUDA_OK(cudaMemsetAsync(a.grad_bias, 0, MIX * sizeof(float), stream));
  HMC_CUDA_OK(cudaMemsetAsync(a.grad_norm_weight, 0, a.hidden * sizeof(float), stream));
  mhc_split_phi_kernel<<<static_cast<unsigned>((k + 255) / 256), 256, 0, stream>>>(a.phi, k, phi_split);
  HMC_LAUNCH_OK();
  fill_i64_kernel<<<1, 1, 0, stream>>>(ends, T);
  HMC_LAUNCH_OK();
  mhc_mapping_grad_kernel<<<static_cast<unsigned>((T + 31) / 32), 32, 0, stream>>>(
      a.hc_before_norm, a.inv_rms, a.alpha, a.bias, a.grad_next_pre_mix, a.grad_next_post_mix,
      a.grad_next_residual_mix, T, hidden, a.hc_eps, a.num_iters, dq_rows, dq_cols, rms_coef, a.grad_alpha,
      a.grad_bias);
  HMC_LAUNCH_OK();
  {  // proj_grad[T, 4H] = dq . phi  (contraction over the padded, split 128-wide axis)
    hmc_grouped_gemm_args g{};
    g.mode = HMC_GEMM_RAGGED_M;
    g.a_major = HMC_MAJOR_K;
    g.b_major = HMC_MAJOR_MN;
    g.epilogue = HMC_EPI_STORE_BF16;
    g.groups = 1;
    g.rows = T;
    g.n = k;
    g.k = 128;
    g.tile_mode = HMC_TILE_SINGLE;  // two k-blocks per tile: the store path decides, and 128-row tiles store by TMA
    g.a = dq_rows;
    g.b = phi_split;
    g.c = proj_grad;
    g.group_ends = reinterpret_cast<const int64_t*>(ends);
    g.status = a.status;
    rc = run_gemm(g, stream);
    if (rc != 0) return rc;
  }
  {  // dphi parts[64, 4H] = dq^T . new_residual  (contraction over tokens)
    hmc_grouped_gemm_args g{};
    g.mode = HMC_GEMM_RAGGED_K;
    g.a_major = HMC_MAJOR_MN;
    g.b_major = HMC_MAJOR_MN;
    g.epilogue = HMC_EPI_STORE_F32;
    g.groups = 1;
    g.rows = T;
    g.m = 2 * MIX_PAD;
    g.n = k;
    g.a = dq_cols;
    g.b = a.new_residual;
    g.c = dphi_parts;
    g.group_ends = reinterpret_cast<const int64_t*>(ends);
    g.status = a.status;
    rc = run_gemm(g, stream);
    if (rc != 0) return rc;
  }
  mhc_combine_dphi_kernel<<<static_cast<unsigned>((k + 255) / 256), 256, 0, stream>>>(dphi_parts, k, a.grad_phi);
  HMC_LAUNCH_OK();
  {
    const int vec = hidden / 8;
    dim3 grid_nw(static_cast<unsigned>((vec + 31) / 32), static_cast<unsigned>(T >= 4096 ? 64 : (T + 63) / 64));
    mhc_norm_weight_grad_kernel<<<grid_nw, 256, 0, stream>>>(static_cast<const uint4*>(a.grad_block_input),
                                                             static_cast<const uint4*>(a.mixed_input), a.rms_rstd, T,
                                                             vec, a.grad_norm_weight);
    HMC_LAUNCH_OK();
    int grid = 4 * sm_count();
    const long long need = (T + WARPS - 1) / WARPS;
    if (need < grid) grid = static_cast<int>(need);
    mhc_stream_grad_kernel<<<grid, WARPS * 32, 0, stream>>>(
        static_cast<const uint4*>(a.grad_new_residual), static_cast<const uint4*>(a.grad_block_input),
        static_cast<const uint4*>(a.new_residual), static_cast<const uint4*>(a.mixed_input),
        static_cast<const uint4*>(a.residual), static_cast<const uint4*>(a.previous_output),
        reinterpret_cast<const uint4*>(proj_grad), static_cast<const uint4*>(a.norm_weight), a.previous_pre_mix,
        a.previous_post_mix, a.previous_residual_mix, a.rms_rstd, rms_coef, T, hidden,
        static_cast<uint4*>(a.grad_residual), static_cast<uint4*>(a.grad_previous_output),
        a.grad_previous_pre_mix, a.grad_previous_post_mix, a.grad_previous_residual_mix);
    HMC_LAUNCH_OK();
  }
  return 0;
}
