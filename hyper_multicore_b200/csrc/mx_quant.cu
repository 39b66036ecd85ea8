// MXFP8 quantisers: BF16 -> E4M3 with one UE8M0 scale per 32 elements, along the row (for GEMMs
// that contract over the feature axis) and down the rows (for the weight-gradient GEMMs that
// contract over tokens), written in the padded expert-major layout the MX GEMM consumes.
//
// Replaces the reference's dual-axis MX quantiser tasks (hyper_multicore/ops/common/mega_moe/
// adapters/arch35/quantization/dual_axis_mxfp8_worker.h:23-110): plain, fused SwiGLU + quant and
// fused SwiGLUGrad + quant. The reference delegates the arithmetic to a third-party CANN operator
// whose source is not part of that project; the rule used here is the OCP Microscaling one:
//   shared exponent = floor(log2(max |x| of the block)) - 8   (8 = largest E4M3 exponent)
//   element         = round-to-nearest-even(x / 2^exponent), saturating at +-448
// with an all-zero block taking scale 1.
#include "common.cuh"
#include "mx_quant_shared.cuh"

namespace hmc {
namespace {

using namespace mxq;

__device__ __forceinline__ __nv_bfloat162 as_bf162(uint32_t v) { return *reinterpret_cast<const __nv_bfloat162*>(&v); }

constexpr int TILE = 128;
constexpr int LDB = TILE + 8;  // shared-memory row stride in BF16 elements (16-byte rows, conflict-free both ways)
constexpr int THREADS = 256;

struct QuantParams {
  int kind;
  int groups;
  long long rows;
  int pad_blocks;
  int width;  // columns of the quantised result
  const __nv_bfloat16* src;
  const __nv_bfloat16* aux;
  const long long* group_ends;
  uint8_t* row_data;
  uint8_t* row_scale;
  uint8_t* col_data;
  uint8_t* col_scale;
  __nv_bfloat16* dense;
  const int* skip_flag;
};

// Where a tile goes: rows [row0, row0 + valid) of the un-padded source are rows [pad_row0, ...) of the padded
// outputs; the tile covers output columns [out_c0, out_c0 + 128).
struct TilePlace {
  long long row0;
  long long pad_row0;
  int valid;
  int pb;
  int out_c0;
};

// Eight finished (BF16-exact) values of row r, columns out_c0 + c .. + 7: dense copy, shared-memory copy for the
// column pass, and the row-quantised bytes with their scale. The four threads of a 32-column block are
// neighbouring lanes, so the block maximum is two shuffles away.
__device__ __forceinline__ void emit_row_piece(const QuantParams& p, const TilePlace& t, const uint4& packed,
                                               const float (&v)[8], int r, int c, __nv_bfloat16* tile) {
  const int width = p.width;
  if (p.dense != nullptr && r < t.valid) *reinterpret_cast<uint4*>(p.dense + (t.row0 + r) * width + t.out_c0 + c) = packed;
  if (p.col_data != nullptr) *reinterpret_cast<uint4*>(tile + r * LDB + c) = packed;
  if (p.row_data != nullptr) {
    // largest magnitude of the eight values, on the packed BF16 pairs (a maximum is exact in any format)
    const __nv_bfloat162 m01 = __hmax2(__habs2(as_bf162(packed.x)), __habs2(as_bf162(packed.y)));
    const __nv_bfloat162 m23 = __hmax2(__habs2(as_bf162(packed.z)), __habs2(as_bf162(packed.w)));
    const float2 pair = __bfloat1622float2(__hmax2(m01, m23));
    float amax = fmaxf(pair.x, pair.y);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const uint32_t e = block_exponent(amax);
    const float inv = inverse_scale(e);
    uint2 q;
    q.x = e4m3x2(v[0] * inv, v[1] * inv) | (e4m3x2(v[2] * inv, v[3] * inv) << 16);
    q.y = e4m3x2(v[4] * inv, v[5] * inv) | (e4m3x2(v[6] * inv, v[7] * inv) << 16);
    *reinterpret_cast<uint2*>(p.row_data + (t.pad_row0 + r) * width + t.out_c0 + c) = q;
    if ((threadIdx.x & 3) == 0) {
      uint8_t* row_atom = p.row_scale + (static_cast<long long>(t.out_c0 / TILE) * p.pad_blocks + t.pb) * 512;
      row_atom[(r & 31) * 16 + (r >> 5) * 4 + (c >> 5)] = static_cast<uint8_t>(e);
    }
  }
}

// 32-element blocks down each column of one shared-memory tile: one thread per (column pair, 32-row block).
__device__ __forceinline__ void column_pass(const QuantParams& p, const TilePlace& t, const __nv_bfloat16* tile) {
  const int width = p.width;
  uint8_t* atom = p.col_scale + (static_cast<long long>(t.pb) * (width / TILE) + t.out_c0 / TILE) * 512;
  const int cp = threadIdx.x & 63;
  const int jb = threadIdx.x >> 6;
  const uint32_t* src = reinterpret_cast<const uint32_t*>(tile + (32 * jb) * LDB + 2 * cp);
  uint32_t w[32];
  __nv_bfloat162 amax = __floats2bfloat162_rn(0.f, 0.f);  // both columns at once, on the packed pairs
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    w[i] = src[i * (LDB / 2)];
    amax = __hmax2(amax, __habs2(as_bf162(w[i])));
  }
  const float2 amax_f = __bfloat1622float2(amax);
  const uint32_t e0 = block_exponent(amax_f.x), e1 = block_exponent(amax_f.y);
  const float inv0 = inverse_scale(e0), inv1 = inverse_scale(e1);
  uint8_t* dst = p.col_data + (t.pad_row0 + 32 * jb) * width + t.out_c0 + 2 * cp;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float2 f = unpack_bf16x2(w[i]);
    *reinterpret_cast<uint16_t*>(dst + static_cast<long long>(i) * width) =
        static_cast<uint16_t>(e4m3x2(f.x * inv0, f.y * inv1));
  }
  const int c_even = 2 * cp;
  atom[(c_even & 31) * 16 + (c_even >> 5) * 4 + jb] = static_cast<uint8_t>(e0);
  atom[((c_even + 1) & 31) * 16 + ((c_even + 1) >> 5) * 4 + jb] = static_cast<uint8_t>(e1);
}

// One CTA per (128-row padded block, 128-column block of the source). KIND is a compile-time constant so
// that each variant is straight-line code whose global loads are all issued before the first of them is
// used. The SwiGLU-grad variant reads dAct, gate and up once and produces both halves of [dgate | dup].
template <int KIND>
__global__ void __launch_bounds__(THREADS, 3) mx_quant_kernel(const QuantParams p) {
  extern __shared__ __align__(16) __nv_bfloat16 tile[];  // [TILE][LDB] (two of them for SwiGLU-grad), BF16-exact values
  __shared__ long long s_row0;
  __shared__ int s_valid;
  if (p.skip_flag != nullptr && *p.skip_flag != 0) return;  // the call was not admitted (hmc_route_guard)
  const int pb = blockIdx.x;
  const int cb = blockIdx.y;
  // Locate the padded block: groups own ceil(rows / 128) consecutive blocks each. All threads fetch the
  // group ends at once (one memory latency); the first warp then scans the block counts 32 groups at a time.
  __shared__ int s_blocks[HMC_CTRL_MAX_LOCAL_EXPERTS];
  for (int g = threadIdx.x; g < p.groups; g += THREADS) {
    const long long end = p.group_ends[g];
    const long long prev = g > 0 ? p.group_ends[g - 1] : 0;
    s_blocks[g] = static_cast<int>((end - prev + 127) / 128);
  }
  if (threadIdx.x == 0) s_valid = -1;
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int base = 0;
    for (int g0 = 0; g0 < p.groups; g0 += 32) {
      const int g = g0 + lane;
      const int blocks = g < p.groups ? s_blocks[g] : 0;
      int incl = blocks;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int other = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += other;
      }
      const int start = base + incl - blocks;
      const bool hit = pb >= start && pb < start + blocks;
      if (hit) {
        const long long prev = g > 0 ? p.group_ends[g - 1] : 0;
        const long long end = p.group_ends[g];
        s_row0 = prev + static_cast<long long>(pb - start) * 128;
        s_valid = static_cast<int>(min(static_cast<long long>(128), end - s_row0));
      }
      if (__ballot_sync(0xffffffffu, hit) != 0u) break;
      base += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  __syncthreads();
  if (s_valid < 0) return;  // a spare block past the last group: never read by the GEMM
  const int width = p.width;
  const int inter = width / 2;  // SwiGLU-grad: src = dAct[rows, inter], aux = U[rows, width] = [gate | up]
  TilePlace t;
  t.row0 = s_row0;
  t.pad_row0 = static_cast<long long>(pb) * TILE;
  t.valid = s_valid;
  t.pb = pb;
  t.out_c0 = cb * TILE;
  TilePlace t_up = t;  // SwiGLU-grad: the dup half of the same columns
  t_up.out_c0 = inter + cb * TILE;
  __nv_bfloat16* tile_up = tile + TILE * LDB;

  // ---- load (and transform) the tile, 8 BF16 per access: a thread owns columns c .. c+7 of rows rbase,
  // rbase + 16, ...; the loads of PASS rows are in flight together.
  const int rbase = threadIdx.x >> 4;
  const int c = (threadIdx.x & 15) * 8;
  const int c0 = cb * TILE;
  constexpr int PASS = KIND == HMC_MXQ_SWIGLU_GRAD ? 4 : 8;
#pragma unroll 1
  for (int j0 = 0; j0 < TILE / 16; j0 += PASS) {
    uint4 ra[PASS], rb[PASS], rc[PASS];
#pragma unroll
    for (int j = 0; j < PASS; ++j) {
      const int r = rbase + 16 * (j0 + j);
      ra[j] = rb[j] = rc[j] = make_uint4(0, 0, 0, 0);  // padding rows quantise to zeros in every variant
      if (r < t.valid) {
        const long long row = t.row0 + r;
        if (KIND == HMC_MXQ_PLAIN) {
          ra[j] = ld_nc_16(p.src + row * width + c0 + c);
        } else if (KIND == HMC_MXQ_SWIGLU) {
          // src = U[rows, 2 * width] = [gate | up]
          ra[j] = ld_nc_16(p.src + row * 2 * width + c0 + c);
          rb[j] = ld_nc_16(p.src + row * 2 * width + width + c0 + c);
        } else {
          ra[j] = ld_nc_16(p.aux + row * width + c0 + c);
          rb[j] = ld_nc_16(p.aux + row * width + inter + c0 + c);
          rc[j] = ld_nc_16(p.src + row * inter + c0 + c);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < PASS; ++j) {
      const int r = rbase + 16 * (j0 + j);
      const uint32_t aw[4] = {ra[j].x, ra[j].y, ra[j].z, ra[j].w};
      const uint32_t bw[4] = {rb[j].x, rb[j].y, rb[j].z, rb[j].w};
      const uint32_t cw[4] = {rc[j].x, rc[j].y, rc[j].z, rc[j].w};
      float v[8];
      float v_up[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (KIND == HMC_MXQ_PLAIN) {
          const float2 f = unpack_bf16x2(aw[q]);
          v[2 * q] = f.x;
          v[2 * q + 1] = f.y;
        } else if (KIND == HMC_MXQ_SWIGLU) {
          const float2 g = unpack_bf16x2(aw[q]);
          const float2 u = unpack_bf16x2(bw[q]);
          v[2 * q] = swiglu_bf16(g.x, u.x);
          v[2 * q + 1] = swiglu_bf16(g.y, u.y);
        } else {
          const float2 g = unpack_bf16x2(aw[q]);
          const float2 u = unpack_bf16x2(bw[q]);
          const float2 d = unpack_bf16x2(cw[q]);
          const float s0 = sigmoid_f(g.x);
          const float s1 = sigmoid_f(g.y);
          v[2 * q] = bf16_round(d.x * u.x * s0 * (1.0f + g.x * (1.0f - s0)));
          v[2 * q + 1] = bf16_round(d.y * u.y * s1 * (1.0f + g.y * (1.0f - s1)));
          v_up[2 * q] = bf16_round(d.x * (g.x * s0));
          v_up[2 * q + 1] = bf16_round(d.y * (g.y * s1));
        }
      }
      // the same eight values as BF16 pairs (the plain variant's input words are exactly that)
      const uint4 packed = KIND == HMC_MXQ_PLAIN ? ra[j]
                                                 : make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                                              pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
      emit_row_piece(p, t, packed, v, r, c, tile);
      if (KIND == HMC_MXQ_SWIGLU_GRAD)
        emit_row_piece(p, t_up, make_uint4(pack_bf16x2(v_up[0], v_up[1]), pack_bf16x2(v_up[2], v_up[3]),
                                           pack_bf16x2(v_up[4], v_up[5]), pack_bf16x2(v_up[6], v_up[7])),
                       v_up, r, c, tile_up);
    }
  }
  if (p.col_data != nullptr) {
    __syncthreads();
    column_pass(p, t, tile);
    if (KIND == HMC_MXQ_SWIGLU_GRAD) column_pass(p, t_up, tile_up);
  }
}

// Weights [experts, m, n] BF16 -> the reference's physical MX fields. One thread per 32-block.
__global__ void mx_quant_weight_col_kernel(const __nv_bfloat16* __restrict__ w, long long experts, int m, int n,
                                           uint8_t* __restrict__ data, uint8_t* __restrict__ scale) {
  // blocks of 32 along m; scale[e, m/64, n, 2]
  const long long total = experts * (m / 32) * n;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int col = static_cast<int>(i % n);
  const int mb = static_cast<int>((i / n) % (m / 32));
  const long long e = i / (static_cast<long long>(n) * (m / 32));
  const __nv_bfloat16* src = w + (e * m + mb * 32) * n + col;
  float v[32], amax = 0.f;
#pragma unroll
  for (int k = 0; k < 32; ++k) {
    v[k] = __bfloat162float(src[static_cast<long long>(k) * n]);
    amax = fmaxf(amax, fabsf(v[k]));
  }
  const uint32_t ex = block_exponent(amax);
  const float inv = inverse_scale(ex);
  uint8_t* dst = data + (e * m + mb * 32) * n + col;
#pragma unroll
  for (int k = 0; k < 32; ++k) dst[static_cast<long long>(k) * n] = to_e4m3(v[k] * inv);
  scale[((e * (m / 64) + mb / 2) * n + col) * 2 + (mb & 1)] = static_cast<uint8_t>(ex);
}

__global__ void mx_quant_weight_row_kernel(const __nv_bfloat16* __restrict__ w, long long experts, int m, int n,
                                           uint8_t* __restrict__ data, uint8_t* __restrict__ scale) {
  // blocks of 32 along n; scale[e, m, n/64, 2]. One thread per 8 elements (16 bytes in, 8 bytes out, both
  // coalesced); the four threads of a 32-block are neighbouring lanes and share their maximum by shuffles.
  const long long total = experts * m * (n / 8);
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool active = i < total;  // n % 64 == 0: a 32-block never straddles the end, whole warps stay converged
  float v[8];
  float amax = 0.f;
  if (active) {
    const uint4 q = ld_nc_16(w + i * 8);
    const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(words[j]);
      v[2 * j] = f.x;
      v[2 * j + 1] = f.y;
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  if (!active) return;
  const uint32_t ex = block_exponent(amax);
  const float inv = inverse_scale(ex);
  uint2 out;
  out.x = e4m3x2(v[0] * inv, v[1] * inv) | (e4m3x2(v[2] * inv, v[3] * inv) << 16);
  out.y = e4m3x2(v[4] * inv, v[5] * inv) | (e4m3x2(v[6] * inv, v[7] * inv) << 16);
  *reinterpret_cast<uint2*>(data + i * 8) = out;
  if ((i & 3) == 0) {
    const long long block = i >> 2;  // 32-element block index over the whole tensor
    const int nb = static_cast<int>(block % (n / 32));
    const long long row = block / (n / 32);
    scale[(row * (n / 64) + nb / 2) * 2 + (nb & 1)] = static_cast<uint8_t>(ex);
  }
}

// Reference scale tensors -> 512-byte atoms. One thread per output byte.
__global__ void mx_pack_weight_scale_kernel(const uint8_t* __restrict__ scale, int axis, long long experts, int m,
                                            int n, uint8_t* __restrict__ atoms) {
  const long long total = experts * (static_cast<long long>(m) * n / 32);
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int within = static_cast<int>(i & 511);
  const int r32 = within >> 4, r4 = (within >> 2) & 3, kk = within & 3;
  const long long atom = i >> 9;
  if (axis == 0) {
    // atoms [e][m/128][n/128], atom row = n index, kk = 32-block of m inside the 128-block
    const int nb = static_cast<int>(atom % (n / 128));
    const int kb = static_cast<int>((atom / (n / 128)) % (m / 128));
    const long long e = atom / (static_cast<long long>(n / 128) * (m / 128));
    const int col = nb * 128 + r4 * 32 + r32;
    atoms[i] = scale[((e * (m / 64) + kb * 2 + kk / 2) * n + col) * 2 + (kk & 1)];
  } else {
    // atoms [e][n/128][m/128], atom row = m index, kk = 32-block of n inside the 128-block
    const int mb = static_cast<int>(atom % (m / 128));
    const int kb = static_cast<int>((atom / (m / 128)) % (n / 128));
    const long long e = atom / (static_cast<long long>(m / 128) * (n / 128));
    const int row = mb * 128 + r4 * 32 + r32;
    atoms[i] = scale[((e * m + row) * (n / 64) + kb * 2 + kk / 2) * 2 + (kk & 1)];
  }
}

}  // namespace
}  // namespace hmc

using namespace hmc;

extern "C" int hmc_mx_quant(const hmc_mx_quant_args* args, void* stream_ptr) {
  HMC_REQUIRE(args != nullptr, HMC_ERR_INVALID, "hmc_mx_quant: null args");
  const hmc_mx_quant_args& a = *args;
  ProfileScope profile(HMC_PROFILE_MX_QUANT, static_cast<cudaStream_t>(stream_ptr));
  HMC_REQUIRE(a.kind >= HMC_MXQ_PLAIN && a.kind <= HMC_MXQ_SWIGLU_GRAD, HMC_ERR_INVALID, "hmc_mx_quant: unknown kind %d",
              a.kind);
  HMC_REQUIRE(a.groups > 0 && a.rows >= 0 && a.pad_blocks >= (a.rows + 127) / 128 && a.pad_blocks > 0 &&
                  a.pad_blocks <= 65535 * 16,
              HMC_ERR_INVALID, "hmc_mx_quant: bad group / row / pad_blocks arguments");
  HMC_REQUIRE(a.width > 0 && a.width % 128 == 0 && a.width / 128 <= 65535, HMC_ERR_LIMIT,
              "hmc_mx_quant: width (%lld) must be a positive multiple of 128", (long long)a.width);
  HMC_REQUIRE(a.kind != HMC_MXQ_SWIGLU_GRAD || (a.width % 256 == 0 && a.aux != nullptr), HMC_ERR_INVALID,
              "hmc_mx_quant: the SwiGLU-grad kind needs aux = U and a width that is a multiple of 256");
  HMC_REQUIRE(a.src && a.group_ends, HMC_ERR_INVALID, "hmc_mx_quant: null tensor pointer");
  HMC_REQUIRE((a.row_data == nullptr) == (a.row_scale == nullptr) && (a.col_data == nullptr) == (a.col_scale == nullptr),
              HMC_ERR_INVALID, "hmc_mx_quant: data and scale outputs go together");
  HMC_REQUIRE(aligned16(a.src) && (a.aux == nullptr || aligned16(a.aux)) && (a.row_data == nullptr || aligned16(a.row_data)) &&
                  (a.dense == nullptr || aligned16(a.dense)),
              HMC_ERR_INVALID, "hmc_mx_quant: tensors must be 16-byte aligned");
  if (a.rows == 0) return 0;
  QuantParams p{};
  p.kind = a.kind;
  p.groups = a.groups;
  p.rows = a.rows;
  p.pad_blocks = static_cast<int>(a.pad_blocks);
  p.width = static_cast<int>(a.width);
  p.src = static_cast<const __nv_bfloat16*>(a.src);
  p.aux = static_cast<const __nv_bfloat16*>(a.aux);
  p.group_ends = reinterpret_cast<const long long*>(a.group_ends);
  p.row_data = static_cast<uint8_t*>(a.row_data);
  p.row_scale = static_cast<uint8_t*>(a.row_scale);
  p.col_data = static_cast<uint8_t*>(a.col_data);
  p.col_scale = static_cast<uint8_t*>(a.col_scale);
  p.dense = static_cast<__nv_bfloat16*>(a.dense);
  p.skip_flag = a.skip_flag;
  const bool grad = a.kind == HMC_MXQ_SWIGLU_GRAD;  // one CTA produces the dgate and the dup tile of its columns
  const int smem = (grad ? 2 : 1) * TILE * LDB * sizeof(__nv_bfloat16);
  // only blocks that can hold rows are launched: ceil(rows / 128) + groups bounds them
  long long blocks = (a.rows + 127) / 128 + a.groups;
  if (blocks > a.pad_blocks) blocks = a.pad_blocks;
  dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(a.width / (grad ? 256 : 128)));
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (a.kind == HMC_MXQ_PLAIN) {
    static PerDeviceFlag configured{};
    if (int rc = allow_dynamic_smem(mx_quant_kernel<HMC_MXQ_PLAIN>, smem, configured)) return rc;
    mx_quant_kernel<HMC_MXQ_PLAIN><<<grid, THREADS, smem, stream>>>(p);
  } else if (a.kind == HMC_MXQ_SWIGLU) {
    static PerDeviceFlag configured{};
    if (int rc = allow_dynamic_smem(mx_quant_kernel<HMC_MXQ_SWIGLU>, smem, configured)) return rc;
    mx_quant_kernel<HMC_MXQ_SWIGLU><<<grid, THREADS, smem, stream>>>(p);
  } else {
    static PerDeviceFlag configured{};
    if (int rc = allow_dynamic_smem(mx_quant_kernel<HMC_MXQ_SWIGLU_GRAD>, smem, configured)) return rc;
    mx_quant_kernel<HMC_MXQ_SWIGLU_GRAD><<<grid, THREADS, smem, stream>>>(p);
  }
  HMC_LAUNCH_OK();
  return 0;
}

extern "C" int hmc_mx_quant_weight(const void* weight_bf16, int64_t experts, int64_t m, int64_t n, void* col_data,
                                   void* col_scale, void* row_data, void* row_scale, void* stream_ptr) {
  HMC_REQUIRE(weight_bf16 != nullptr && experts > 0, HMC_ERR_INVALID, "hmc_mx_quant_weight: bad arguments");
  // the reference's contract: both matrix extents are multiples of 64 (docs/mega_moe.md:184)
  HMC_REQUIRE(m > 0 && n > 0 && m % 64 == 0 && n % 64 == 0 && m < (1ll << 31) && n < (1ll << 31), HMC_ERR_INVALID,
              "hmc_mx_quant_weight: m (%lld) and n (%lld) must be positive multiples of 64", (long long)m, (long long)n);
  HMC_REQUIRE((col_data == nullptr) == (col_scale == nullptr) && (row_data == nullptr) == (row_scale == nullptr),
              HMC_ERR_INVALID, "hmc_mx_quant_weight: data and scale outputs go together");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(weight_bf16);
  if (col_data != nullptr) {
    const long long total = experts * (m / 32) * n;
    mx_quant_weight_col_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
        w, experts, static_cast<int>(m), static_cast<int>(n), static_cast<uint8_t*>(col_data),
        static_cast<uint8_t*>(col_scale));
    HMC_LAUNCH_OK();
  }
  if (row_data != nullptr) {
    const long long total = experts * m * (n / 8);
    mx_quant_weight_row_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
        w, experts, static_cast<int>(m), static_cast<int>(n), static_cast<uint8_t*>(row_data),
        static_cast<uint8_t*>(row_scale));
    HMC_LAUNCH_OK();
  }
  return 0;
}

extern "C" int hmc_mx_pack_weight_scale(const void* scale, int axis, int64_t experts, int64_t m, int64_t n, void* atoms,
                                        void* stream_ptr) {
  HMC_REQUIRE(scale != nullptr && atoms != nullptr && experts > 0 && (axis == 0 || axis == 1), HMC_ERR_INVALID,
              "hmc_mx_pack_weight_scale: bad arguments");
  HMC_REQUIRE(m > 0 && n > 0 && m % 128 == 0 && n % 128 == 0, HMC_ERR_LIMIT,
              "hmc_mx_pack_weight_scale: m (%lld) and n (%lld) must be multiples of 128 on this backend", (long long)m,
              (long long)n);
  const long long total = experts * (m * n / 32);
  mx_pack_weight_scale_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0,
                                static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const uint8_t*>(scale), axis, experts, static_cast<int>(m), static_cast<int>(n),
      static_cast<uint8_t*>(atoms));
  HMC_LAUNCH_OK();
  return 0;
}
