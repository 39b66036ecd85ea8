// The MXFP8 quantisation rule shared by the stand-alone quantisers and the GEMM epilogues that quantise
// their own results: E4M3 elements with one UE8M0 scale per 32 elements (OCP Microscaling):
//   shared exponent = floor(log2(max |x| of the block)) - 8   (8 = largest E4M3 exponent)
//   element         = round-to-nearest-even(x / 2^exponent), saturating at +-448
// with an all-zero block taking scale 1.
#pragma once

#include <cuda_fp8.h>

#include "common.cuh"

namespace hmc {
namespace mxq {

// biased UE8M0 exponent of a block whose largest magnitude is `amax`
__device__ __forceinline__ uint32_t block_exponent(float amax) {
  if (!(amax > 0.f)) return 127u;
  const int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu) - 8;
  return static_cast<uint32_t>(min(max(e, 0), 254));
}
__device__ __forceinline__ float inverse_scale(uint32_t biased) { return __uint_as_float((254u - biased) << 23); }
// two values -> two E4M3 bytes (first value in the low byte), round to nearest even, saturating
__device__ __forceinline__ uint32_t e4m3x2(float lo, float hi) {
  return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
// SwiGLU on BF16-exact inputs, rounded to BF16: the activation both the quantiser and the fused GEMM epilogue produce
__device__ __forceinline__ float swiglu_bf16(float gate, float up) { return bf16_round(gate * sigmoid_f(gate) * up); }

// byte offset of the scale of (row r of a 128-row block, 32-element block kk of a 128-element block) in a 512-byte atom
__device__ __forceinline__ int atom_offset(int r, int kk) { return (r & 31) * 16 + (r >> 5) * 4 + kk; }

}  // namespace mxq
}  // namespace hmc
