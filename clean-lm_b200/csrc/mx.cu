// Block-scaled (MXFP8) tensors: layout, quantisation, and RMSNorm with block-scaled outputs.
//
// Format (crates/cleandl/src/mx_tensor.rs:11-20, 339-372): a 2-D tensor whose blocks of 32
// elements along the block dimension share one UE8M0 scale 2^(e - 127); values are FP8 E4M3.
// Rowwise: blocks run along a row, values are a packed [rows, cols] byte matrix.  Colwise: blocks
// run down a column, values are the packed TRANSPOSE [cols, rows].  Scale factors live in the
// 128 x 4 tiled, partition-swizzled layout tcgen05 block-scaled MMAs read
// (crates/cleandl-specialized-kernels/src/utils/block_scale.rs:70-80): the scale of block
// (outer o, block b) is byte  ((o / 128) * ceil(B / 4) + b / 4) * 512 + (o % 32) * 16 +
// ((o % 128) / 32) * 4 + b % 4,  with B blocks per outer index; the buffer is padded to
// 128 outer rows x 4 blocks.
//
// Quantisation follows the reference's norm kernel (block_scale.rs:24-55): the value is rounded
// to bf16, the scale is amax / 448 rounded UP to a power of two, the element is value * 2^-e
// rounded to nearest E4M3 with saturation.  The power of two is found exactly, from the bits of
// amax (the reference divides approximately), which makes the result a pure function of the
// bf16 values.
//
// NormFwd with NormOutput::{Mxfp8Rowwise, Mxfp8RowwiseAndColwise}
// (crates/cleandl/src/execgraph/ops/norm/mod.rs:33-62, kernel
// crates/cleandl-specialized-kernels/src/kernels/norm/forward.rs:509-785): HBM-bound.  One warp
// owns a row; a lane holds 8 consecutive bf16 of every 256-column stripe, so the four lanes of a
// 32-element block reduce their amax with two shuffles.  With the colwise output a CTA owns 32
// consecutive rows (one warp each): the bf16 results of 1024 columns go through shared memory and
// one thread per column quantises the 32 rows of its block and stores one 32-byte sector of the
// transposed output.  NVFP4 (NormOutput::Nvfp4Rowwise): rowwise only, see nvfp4_rows_kernel.
//
// Kernels, from the general to the common case (the host picks in mx_rows_run):
//   mx_rows_kernel            any shape; with the colwise output 1024 columns at a time through
//                             shared memory (rows too long for the kernels below, or a bias)
//   mx_row_cached_kernel      rowwise only, cols <= 8192: the row stays in registers
//   mx_rowcol_tile_kernel     both outputs, 32 whole rows (or 2048-column panels) in shared memory
//   mx_row_full_kernel,       cols % 256 == 0 and no bias: the same two schemes trimmed of every
//   mx_rowcol_full_kernel     operation the arithmetic does not need (these kernels are bound by
//                             the ALU pipe, not by HBM)
//   mx_rowcol_panel_kernel    both outputs by 512- / 1024-column panels, several CTAs per SM; with
//                             the normalisation the panels of a row are a cluster that shares the
//                             row sums through distributed shared memory (rows up to 8192)
//   nvfp4_rows_kernel, nvfp4_row_full_kernel   the NVFP4 rowwise output, general and trimmed
#include "host.h"
#include "ops.h"
#include "ptx.cuh"

#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <mutex>

namespace cdl {
namespace mx {

constexpr int BLOCK = 32;
constexpr int COL_GROUP = 1024;            // columns staged per colwise phase (4 stripes)
constexpr int TILE_LD = COL_GROUP + 8;     // bf16 elements per staged row (16-byte aligned rows)
constexpr size_t COL_SMEM_BYTES = 32 * TILE_LD * 2;

struct Params {
  const __nv_bfloat16* x;
  long long ldx;
  int rows, cols;
  const __nv_bfloat16* gamma;  // nullable
  const __nv_bfloat16* beta;   // nullable
  float eps;
  float* r_inv;  // nullable
  long long r_inv_stride;
  uint8_t* row_values;  // [rows, cols]; nullable
  uint8_t* row_sf;
  uint8_t* col_values;  // [cols, rows]; nullable
  uint8_t* col_sf;
  int panel_cols;  // tile kernel: columns a CTA owns (blockIdx.y selects the panel); cols if one panel
};

__device__ __forceinline__ long long sf_index(int outer, int block, int blocks) {
  return (static_cast<long long>(outer >> 7) * ((blocks + 3) >> 2) + (block >> 2)) * 512 +
         (outer & 31) * 16 + ((outer & 127) >> 5) * 4 + (block & 3);
}

// Biased exponent e of the smallest power of two s = 2^(e - 127) with amax / s <= 448, for a
// non-negative finite amax.  448 = 1.75 * 2^8, so with amax = m * 2^E (1 <= m < 2) the quotient is
// (m / 1.75) * 2^(E - 8): its ceiling power of two is 2^(E - 8) when m <= 1.75 and twice that
// otherwise.  Integer arithmetic on the bits; zero and subnormal amax give the smallest scale.
__device__ __forceinline__ uint32_t scale_exponent(float amax) {
  const uint32_t bits = __float_as_uint(amax);
  const int e = static_cast<int>(bits >> 23) - 8 + ((bits & 0x7FFFFFu) > 0x600000u ? 1 : 0);
  return static_cast<uint32_t>(max(e, 0));
}
// 2^(127 - e), exact (a subnormal for e = 254).
__device__ __forceinline__ float descale_of(uint32_t e) {
  const uint32_t de = 254u - e;
  return __uint_as_float(de != 0 ? de << 23 : 0x00400000u);
}
__device__ __forceinline__ uint32_t fp8x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}
// Two bf16-representable floats -> packed bf16x2 (lo in the low half).
__device__ __forceinline__ uint32_t pack_rounded(float lo, float hi) {
  return __byte_perm(__float_as_uint(lo), __float_as_uint(hi), 0x7632);
}
__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  f[0] = bf16_lo(q.x); f[1] = bf16_hi(q.x); f[2] = bf16_lo(q.y); f[3] = bf16_hi(q.y);
  f[4] = bf16_lo(q.z); f[5] = bf16_hi(q.z); f[6] = bf16_lo(q.w); f[7] = bf16_hi(q.w);
}

// y of 8 consecutive elements: normalisation (NORM) and rounding to bf16.
template <bool NORM>
__device__ __forceinline__ void apply_norm8(const Params& p, const uint4& xq, int c, float r,
                                            float (&f)[8]) {
  unpack8(xq, f);
  if (NORM) {
    float gm[8], bt[8];
    if (p.gamma != nullptr) unpack8(*reinterpret_cast<const uint4*>(p.gamma + c), gm);
    if (p.beta != nullptr) unpack8(*reinterpret_cast<const uint4*>(p.beta + c), bt);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float v = f[j] * r;
      if (p.gamma != nullptr) v *= gm[j];
      if (p.beta != nullptr) v += bt[j];
      f[j] = v;
    }
    // One packed conversion per pair and two unpacking moves: rounding with integer arithmetic
    // costs four ALU operations per element, and the ALU pipe is what bounds these kernels.
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      const uint32_t q = pack_bf16x2(f[j], f[j + 1]);
      f[j] = bf16_lo(q);
      f[j + 1] = bf16_hi(q);
    }
  }
}

// Rowwise quantisation of a lane's 8 elements; the four lanes of a 32-element block are either
// all active or all idle (cols % 32 == 0).  Every lane of the warp must call (shuffles).
__device__ __forceinline__ void quantize_row8(const Params& p, const float (&f)[8], bool active,
                                              long long row, int c, int lane, int row_blocks) {
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  if (active) {
    const uint32_t e = scale_exponent(amax);
    const float ds = descale_of(e);
    uint2 out;
    out.x = fp8x4(f[0] * ds, f[1] * ds, f[2] * ds, f[3] * ds);
    out.y = fp8x4(f[4] * ds, f[5] * ds, f[6] * ds, f[7] * ds);
    *reinterpret_cast<uint2*>(p.row_values + row * p.cols + c) = out;
  }
  // One byte per block: gathering the four scales of an aligned word with shuffles and storing
  // words was measured slower (43 us against 36 us at 16384 x 2048).
  if (active && (lane & 3) == 0)
    p.row_sf[sf_index(static_cast<int>(row), c / BLOCK, row_blocks)] =
        static_cast<uint8_t>(scale_exponent(amax));
}

// NORM: y = x * r * gamma + beta with r = rsqrt(mean x^2 + eps); otherwise y = x.
// COL: the CTA has 32 warps and owns rows [32 * blockIdx.x, +32); otherwise any number of warps,
// each striding over rows.
template <bool NORM, bool COL>
__global__ void __launch_bounds__(COL ? 1024 : 256, 1) mx_rows_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [32][TILE_LD] (COL only)
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps = blockDim.x >> 5;
  const int row_blocks = p.cols / BLOCK;  // blocks per row (rowwise)
  const int col_blocks = p.rows / BLOCK;  // blocks per column (colwise)
  const float inv_cols = 1.0f / static_cast<float>(p.cols);

  const long long row_step = COL ? static_cast<long long>(gridDim.x) * 32
                                 : static_cast<long long>(gridDim.x) * warps;
  for (long long row0 = COL ? static_cast<long long>(blockIdx.x) * 32
                            : static_cast<long long>(blockIdx.x) * warps;
       row0 < p.rows; row0 += row_step) {
    const long long row = row0 + warp;
    const bool row_ok = row < p.rows;
    const __nv_bfloat16* xr = p.x + row * p.ldx;
    float r = 1.0f;
    if (NORM && row_ok) {
      float ss = 0.f;
      for (int c = lane * 8; c < p.cols; c += 256) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(xr + c), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      r = rsqrtf(ss * inv_cols + p.eps);
      if (lane == 0 && p.r_inv != nullptr) p.r_inv[row * p.r_inv_stride] = r;
    }

    for (int g0 = 0; g0 < p.cols; g0 += COL_GROUP) {
      const int g_cols = min(COL_GROUP, p.cols - g0);
      // ---- a warp's row: results of up to four stripes, rowwise output, staging for colwise
      if (row_ok) {
        for (int c0 = g0; c0 < g0 + g_cols; c0 += 256) {  // warp-uniform: the shuffles need all lanes
          const int c = c0 + lane * 8;
          const bool active = c < g0 + g_cols;
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = 0.f;
          if (active) {
            apply_norm8<NORM>(p, *reinterpret_cast<const uint4*>(xr + c), c, r, f);
            if (COL) {
              uint4 q;
              q.x = pack_rounded(f[0], f[1]); q.y = pack_rounded(f[2], f[3]);
              q.z = pack_rounded(f[4], f[5]); q.w = pack_rounded(f[6], f[7]);
              *reinterpret_cast<uint4*>(tile + warp * TILE_LD + (c - g0)) = q;
            }
          }
          if (p.row_values != nullptr) quantize_row8(p, f, active, row, c, lane, row_blocks);
        }
      }
      if (COL) {
        __syncthreads();
        const int c = threadIdx.x;
        if (c < g_cols) {
          // rows % 32 == 0: all 32 staged rows exist
          float v[32];
          float amax = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = __bfloat162float(tile[j * TILE_LD + c]);
            amax = fmaxf(amax, fabsf(v[j]));
          }
          const uint32_t e = scale_exponent(amax);
          const float ds = descale_of(e);
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            w[j] = fp8x4(v[4 * j] * ds, v[4 * j + 1] * ds, v[4 * j + 2] * ds, v[4 * j + 3] * ds);
          st_global_v8(p.col_values + static_cast<long long>(g0 + c) * p.rows + row0, w);
          p.col_sf[sf_index(g0 + c, static_cast<int>(row0 / BLOCK), col_blocks)] = static_cast<uint8_t>(e);
        }
        __syncthreads();
      }
    }
  }
}

// Rowwise output only, rows of up to 256 * NCH columns: the row stays in registers between the
// reduction and the quantisation, so x is read once.
template <bool NORM, int NCH>
__global__ void __launch_bounds__(256, NCH <= 4 ? 4 : NCH <= 8 ? 2 : 1) mx_row_cached_kernel(const Params p) {
  const int lane = threadIdx.x & 31;
  const int row_blocks = p.cols / BLOCK;
  const float inv_cols = 1.0f / static_cast<float>(p.cols);
  const long long warp_global = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const long long warp_stride = static_cast<long long>(gridDim.x) * 8;
  for (long long row = warp_global; row < p.rows; row += warp_stride) {
    const __nv_bfloat16* xr = p.x + row * p.ldx;
    uint4 xv[NCH];
#pragma unroll
    for (int s = 0; s < NCH; ++s) {
      const int c = s * 256 + lane * 8;
      xv[s] = c < p.cols ? ld_nc_v4(xr + c) : make_uint4(0, 0, 0, 0);
    }
    float r = 1.0f;
    if (NORM) {
      float ss = 0.f;
#pragma unroll
      for (int s = 0; s < NCH; ++s) {
        float f[8];
        unpack8(xv[s], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      r = rsqrtf(ss * inv_cols + p.eps);
      if (lane == 0 && p.r_inv != nullptr) p.r_inv[row * p.r_inv_stride] = r;
    }
#pragma unroll
    for (int s = 0; s < NCH; ++s) {
      if (s * 256 < p.cols) {  // warp-uniform
        const int c = s * 256 + lane * 8;
        const bool active = c < p.cols;
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = 0.f;
        if (active) apply_norm8<NORM>(p, xv[s], c, r, f);
        quantize_row8(p, f, active, row, c, lane, row_blocks);
      }
    }
  }
}

// CTAs of 256 threads per SM the trimmed rowwise kernels are compiled for: 3 (80 registers, 24
// warps) measured 0.0253 ms at 16384 x 2048, 2 and 4 (spills at 64 registers) 0.0280 ms.
constexpr int FULL_MIN_CTAS = 3;
// Packed bf16 pairs: |a| and max per half (exact: a maximum picks one of its operands).
__device__ __forceinline__ uint32_t abs_max_bf16x2(uint32_t a, uint32_t b) {
  const __nv_bfloat162 m = __hmax2(__habs2(*reinterpret_cast<const __nv_bfloat162*>(&a)),
                                   __habs2(*reinterpret_cast<const __nv_bfloat162*>(&b)));
  return *reinterpret_cast<const uint32_t*>(&m);
}
__device__ __forceinline__ uint32_t max_bf16x2(uint32_t a, uint32_t b) {
  const __nv_bfloat162 m = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a),
                                   *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&m);
}

// y of a lane's 8 elements as four packed bf16 pairs: x * r (* gamma, f32 from shared memory in
// stage_gamma's layout: gamma2 points at the lane's first float4).
__device__ __forceinline__ void norm_packed8(const uint4& xq, float r, const float4* gamma2,
                                             uint32_t (&q)[4]) {
  float f[8];
  unpack8(xq, f);
  if (gamma2 != nullptr) {
    const float4 g0 = gamma2[0], g1 = gamma2[32];
    f[0] = f[0] * r * g0.x; f[1] = f[1] * r * g0.y; f[2] = f[2] * r * g0.z; f[3] = f[3] * r * g0.w;
    f[4] = f[4] * r * g1.x; f[5] = f[5] * r * g1.y; f[6] = f[6] * r * g1.z; f[7] = f[7] * r * g1.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] *= r;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) q[j] = pack_bf16x2(f[2 * j], f[2 * j + 1]);
}
// Rowwise quantisation of a lane's 8 packed bf16 values, a quarter of a 32-element block (all
// four lanes of a block call): returns the 8 E4M3 bytes, e = the block's scale exponent.
__device__ __forceinline__ uint2 quantize_packed8(const uint32_t (&q)[4], uint32_t& e) {
  uint32_t m = max_bf16x2(abs_max_bf16x2(q[0], q[1]), abs_max_bf16x2(q[2], q[3]));
  m = max_bf16x2(m, __shfl_xor_sync(0xffffffffu, m, 1));
  m = max_bf16x2(m, __shfl_xor_sync(0xffffffffu, m, 2));
  m = max_bf16x2(m, __byte_perm(m, 0, 0x1032));  // both halves: the block's amax
  e = scale_exponent(__uint_as_float(m & 0xFFFF0000u));
  const float ds = descale_of(e);
  uint2 o;
  o.x = fp8x4(bf16_lo(q[0]) * ds, bf16_hi(q[0]) * ds, bf16_lo(q[1]) * ds, bf16_hi(q[1]) * ds);
  o.y = fp8x4(bf16_lo(q[2]) * ds, bf16_hi(q[2]) * ds, bf16_lo(q[3]) * ds, bf16_hi(q[3]) * ds);
  return o;
}
// The scale vector as f32 in shared memory (all threads of the CTA call; ends with a barrier;
// cols % 256 == 0).  Per 256-column stripe 64 float4: the first four values of lane l's eight
// columns at [l], the last four at [32 + l], so that a warp's 128-bit loads touch consecutive
// words (lane-interleaved halves at [2 l], [2 l + 1] would be two-way bank conflicts).
__device__ __forceinline__ void stage_gamma(const __nv_bfloat16* gamma, int cols, float4* s_gamma) {
  for (int c = threadIdx.x * 8; c < cols; c += blockDim.x * 8) {
    float g[8];
    unpack8(*reinterpret_cast<const uint4*>(gamma + c), g);
    const int at = (c >> 8) * 64 + ((c & 255) >> 3);
    s_gamma[at] = make_float4(g[0], g[1], g[2], g[3]);
    s_gamma[at + 32] = make_float4(g[4], g[5], g[6], g[7]);
  }
  __syncthreads();
}

// Rowwise output only, cols == 256 * NCH exactly and no bias (a model's hidden dimension): the
// trimmed form of mx_row_cached_kernel.  What bounds these kernels is the ALU pipe, so this one
// spends as few of its operations per element as the arithmetic allows: the scale vector sits in
// shared memory as f32 (no unpacking per row), the block maximum is taken on the packed bf16
// results (half the operations, and no unpacking before it), no lane is ever idle (no selects),
// and the row's pointers and the row part of the scale index are computed once per row, every
// stripe at a constant offset from them.
template <bool NORM, int NCH>
__global__ void __launch_bounds__(256, NCH <= 8 ? FULL_MIN_CTAS : 1) mx_row_full_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  float4* s_gamma = reinterpret_cast<float4*>(smem_raw);  // [cols] f32 (NORM with a scale vector)
  constexpr int COLS = NCH * 256;
  const int lane = threadIdx.x & 31;
  const bool has_gamma = NORM && p.gamma != nullptr;
  if (has_gamma) stage_gamma(p.gamma, COLS, s_gamma);
  // Block of (stripe s, lane): b = 8 s + lane / 4, so b / 4 = 2 s + lane / 16, b % 4 = lane / 4 % 4.
  const int sf_lane = (lane >> 4) * 512 + ((lane >> 2) & 3);
  const long long warp_global = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const long long warp_stride = static_cast<long long>(gridDim.x) * 8;
  for (long long row = warp_global; row < p.rows; row += warp_stride) {
    const uint4* xr = reinterpret_cast<const uint4*>(p.x + row * p.ldx) + lane;
    uint4 xv[NCH];
#pragma unroll
    for (int s = 0; s < NCH; ++s) xv[s] = ld_nc_v4(xr + s * 32);
    float r = 1.0f;
    if (NORM) {
      float ss = 0.f;
#pragma unroll
      for (int s = 0; s < NCH; ++s) {
        float f[8];
        unpack8(xv[s], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      r = rsqrtf(ss * (1.0f / COLS) + p.eps);
      if (lane == 0 && p.r_inv != nullptr) p.r_inv[row * p.r_inv_stride] = r;
    }
    uint2* out = reinterpret_cast<uint2*>(p.row_values + row * COLS) + lane;
    uint8_t* sf = p.row_sf + (row >> 7) * (NCH * 2 * 512) + (row & 31) * 16 + ((row & 127) >> 5) * 4 +
                  sf_lane;
#pragma unroll
    for (int s = 0; s < NCH; ++s) {
      uint32_t q[4] = {xv[s].x, xv[s].y, xv[s].z, xv[s].w};
      if (NORM) norm_packed8(xv[s], r, has_gamma ? s_gamma + s * 64 + lane : nullptr, q);
      uint32_t e;
      const uint2 o = quantize_packed8(q, e);
      out[s * 32] = o;
      if ((lane & 3) == 0) sf[s * 1024] = static_cast<uint8_t>(e);
    }
  }
}

// Rowwise and colwise outputs, rows short enough for 32 of them to sit in shared memory
// (TILE [32][cols + 8] bf16): a CTA of 32 warps owns 32 rows.  A warp loads its row into the
// tile while it sums the squares, replaces it by the bf16 result (writing the rowwise output on
// the way), and after one barrier every thread quantises whole 32-row blocks of its columns.
// x is read once; the colwise stores are one 32-byte sector per thread.
template <bool NORM>
__global__ void __launch_bounds__(1024, 1) mx_rowcol_tile_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  // Without the normalisation nothing couples the columns of a row, so wide matrices are cut
  // into panels of panel_cols columns (blockIdx.y); with it there is one panel, the whole row.
  const int pc0 = blockIdx.y * p.panel_cols;
  const int pcols = min(p.panel_cols, p.cols - pc0);
  const int ld = p.panel_cols + 8;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int row_blocks = p.cols / BLOCK;
  const int col_blocks = p.rows / BLOCK;
  const float inv_cols = 1.0f / static_cast<float>(p.cols);
  for (long long row0 = static_cast<long long>(blockIdx.x) * 32; row0 < p.rows;
       row0 += static_cast<long long>(gridDim.x) * 32) {
    const long long row = row0 + warp;  // rows % 32 == 0: always a real row
    const __nv_bfloat16* xr = p.x + row * p.ldx + pc0;
    __nv_bfloat16* trow = tile + warp * ld;
    float ss = 0.f;
    for (int c = lane * 8; c < pcols; c += 256) {
      const uint4 q = ld_nc_v4(xr + c);
      *reinterpret_cast<uint4*>(trow + c) = q;
      if (NORM) {
        float f[8];
        unpack8(q, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
      }
    }
    float r = 1.0f;
    if (NORM) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      r = rsqrtf(ss * inv_cols + p.eps);
      if (lane == 0 && p.r_inv != nullptr) p.r_inv[row * p.r_inv_stride] = r;
    }
    for (int c0 = 0; c0 < pcols; c0 += 256) {  // warp-uniform
      const int c = c0 + lane * 8;
      const bool active = c < pcols;
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = 0.f;
      if (active) {
        apply_norm8<NORM>(p, *reinterpret_cast<const uint4*>(trow + c), pc0 + c, r, f);
        if (NORM) {
          uint4 q;
          q.x = pack_rounded(f[0], f[1]); q.y = pack_rounded(f[2], f[3]);
          q.z = pack_rounded(f[4], f[5]); q.w = pack_rounded(f[6], f[7]);
          *reinterpret_cast<uint4*>(trow + c) = q;
        }
      }
      if (p.row_values != nullptr) quantize_row8(p, f, active, row, pc0 + c, lane, row_blocks);
    }
    __syncthreads();
    for (int c = threadIdx.x; c < pcols; c += 1024) {
      float v[32];
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        v[j] = __bfloat162float(tile[j * ld + c]);
        amax = fmaxf(amax, fabsf(v[j]));
      }
      const uint32_t e = scale_exponent(amax);
      const float ds = descale_of(e);
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        w[j] = fp8x4(v[4 * j] * ds, v[4 * j + 1] * ds, v[4 * j + 2] * ds, v[4 * j + 3] * ds);
      st_global_v8(p.col_values + static_cast<long long>(pc0 + c) * p.rows + row0, w);
      p.col_sf[sf_index(pc0 + c, static_cast<int>(row0 / BLOCK), col_blocks)] = static_cast<uint8_t>(e);
    }
    __syncthreads();
  }
}

// Colwise quantisation of columns pc0 + 2 c2 and pc0 + 2 c2 + 1 of a staged tile of 32 rows
// (ld bf16 per row): one 32-bit load brings a pair, the maximum over the rows runs on the pairs,
// and each column leaves as one 32-byte sector of the transposed output.
__device__ __forceinline__ void quantize_column_pair(const Params& p, const __nv_bfloat16* tile, int ld,
                                                     int c2, int pc0, long long row0, int col_blocks) {
  const uint32_t* tp = reinterpret_cast<const uint32_t*>(tile) + c2;
  const int ldw = ld >> 1;
  uint32_t w[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) w[j] = tp[j * ldw];
  uint32_t m = abs_max_bf16x2(w[0], w[1]);
#pragma unroll
  for (int j = 2; j < 32; j += 2) m = max_bf16x2(m, abs_max_bf16x2(w[j], w[j + 1]));
  const uint32_t e_lo = scale_exponent(__uint_as_float(m << 16));
  const uint32_t e_hi = scale_exponent(__uint_as_float(m & 0xFFFF0000u));
  const float ds_lo = descale_of(e_lo), ds_hi = descale_of(e_hi);
  uint32_t o_lo[8], o_hi[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    o_lo[j] = fp8x4(bf16_lo(w[4 * j]) * ds_lo, bf16_lo(w[4 * j + 1]) * ds_lo,
                    bf16_lo(w[4 * j + 2]) * ds_lo, bf16_lo(w[4 * j + 3]) * ds_lo);
    o_hi[j] = fp8x4(bf16_hi(w[4 * j]) * ds_hi, bf16_hi(w[4 * j + 1]) * ds_hi,
                    bf16_hi(w[4 * j + 2]) * ds_hi, bf16_hi(w[4 * j + 3]) * ds_hi);
  }
  const int col = pc0 + 2 * c2;
  uint8_t* dst = p.col_values + static_cast<long long>(col) * p.rows + row0;
  st_global_v8(dst, o_lo);
  st_global_v8(dst + p.rows, o_hi);
  // col is even: the next column's scale sits 16 bytes on (same 128-column tile)
  uint8_t* csf = p.col_sf + sf_index(col, static_cast<int>(row0 / BLOCK), col_blocks);
  csf[0] = static_cast<uint8_t>(e_lo);
  csf[16] = static_cast<uint8_t>(e_hi);
}

// mx_rowcol_tile_kernel for panels whose width is a multiple of 256 and no bias, trimmed like
// mx_row_full_kernel (packed block maxima, f32 scale vector in shared memory behind the tile, no
// idle lanes, index arithmetic hoisted out of the stripes).  The colwise phase takes two columns
// per thread: one 32-bit shared-memory load brings a bf16 pair, the maximum over the 32 rows runs
// on the pairs, and each column still leaves as one 32-byte sector.
template <bool NORM>
__global__ void __launch_bounds__(1024, 1) mx_rowcol_full_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  const int ld = p.panel_cols + 8;
  float4* s_gamma = reinterpret_cast<float4*>(smem_raw + static_cast<size_t>(64) * ld);
  const int pc0 = blockIdx.y * p.panel_cols;
  const int pcols = min(p.panel_cols, p.cols - pc0);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int row_tiles = (p.cols / BLOCK + 3) >> 2;
  const int col_blocks = p.rows / BLOCK;
  const float inv_cols = 1.0f / static_cast<float>(p.cols);
  const bool has_gamma = NORM && p.gamma != nullptr;
  if (has_gamma) stage_gamma(p.gamma, p.cols, s_gamma);  // with NORM the panel is the whole row
  // Block of (stripe at column c0, lane): b = (pc0 + c0) / 32 + lane / 4, the first term a multiple of 8.
  const int sf_lane = (lane >> 4) * 512 + ((lane >> 2) & 3);
  const bool rowwise = p.row_values != nullptr;
  for (long long row0 = static_cast<long long>(blockIdx.x) * 32; row0 < p.rows;
       row0 += static_cast<long long>(gridDim.x) * 32) {
    const long long row = row0 + warp;  // rows % 32 == 0: always a real row
    const __nv_bfloat16* xr = p.x + row * p.ldx + pc0;
    __nv_bfloat16* trow = tile + warp * ld;
    float ss = 0.f;
    for (int c = lane * 8; c < pcols; c += 256) {
      const uint4 q = ld_nc_v4(xr + c);
      *reinterpret_cast<uint4*>(trow + c) = q;
      if (NORM) {
        float f[8];
        unpack8(q, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
      }
    }
    float r = 1.0f;
    if (NORM) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      r = rsqrtf(ss * inv_cols + p.eps);
      if (lane == 0 && p.r_inv != nullptr) p.r_inv[row * p.r_inv_stride] = r;
    }
    if (NORM || rowwise) {
      uint8_t* out = rowwise ? p.row_values + row * p.cols + pc0 + lane * 8 : nullptr;
      uint8_t* sf = rowwise ? p.row_sf + ((row >> 7) * row_tiles + (pc0 >> 7)) * 512 +
                                  (row & 31) * 16 + ((row & 127) >> 5) * 4 + sf_lane
                            : nullptr;
      for (int c0 = 0; c0 < pcols; c0 += 256) {
        const int c = c0 + lane * 8;
        const uint4 xq = *reinterpret_cast<const uint4*>(trow + c);
        uint32_t q[4] = {xq.x, xq.y, xq.z, xq.w};
        if (NORM) {
          norm_packed8(xq, r, has_gamma ? s_gamma + (c0 >> 2) + lane : nullptr, q);
          *reinterpret_cast<uint4*>(trow + c) = make_uint4(q[0], q[1], q[2], q[3]);
        }
        if (rowwise) {  // CTA-uniform: the shuffles see whole warps
          uint32_t e;
          const uint2 o = quantize_packed8(q, e);
          *reinterpret_cast<uint2*>(out + c0) = o;
          if ((lane & 3) == 0) sf[(c0 >> 7) * 512] = static_cast<uint8_t>(e);
        }
      }
    }
    __syncthreads();
    for (int c2 = threadIdx.x; c2 < pcols / 2; c2 += 1024)
      quantize_column_pair(p, tile, ld, c2, pc0, row0, col_blocks);
    __syncthreads();
  }
}

__device__ __forceinline__ void st_shared_cluster_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}

// Rowwise and colwise outputs by panels of W = panel_cols columns (512 or 1024, cols % W == 0,
// no bias): CTA (blockIdx.x, blockIdx.y) owns rows [32 y, +32) x columns [W x, +W) with W / 2
// threads, so that several CTAs share an SM and one's loads run under another's arithmetic (the
// whole-row kernels above hold one CTA per SM and leave half of the issue slots idle), and the
// last wave of CTAs is short.  With NORM the CTAs of a row of panels form a cluster (at most 8):
// each sums the squares of its part of the 32 rows, writes the 32 partial sums into every
// member's shared memory, and after one cluster barrier all of them add the parts in rank order,
// so that every member normalises with the same bits.
template <bool NORM>
__global__ void __launch_bounds__(512, 2) mx_rowcol_panel_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int W = p.panel_cols;
  const int ld = W + 8;
  __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  float4* s_gamma = reinterpret_cast<float4*>(smem_raw + static_cast<size_t>(64) * ld);  // [W] f32
  float* s_ss = reinterpret_cast<float*>(s_gamma + W / 4);                               // [8][32]
  const int pc0 = blockIdx.x * W;
  const long long row0 = static_cast<long long>(blockIdx.y) * 32;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps = blockDim.x >> 5;
  const int row_tiles = (p.cols / BLOCK + 3) >> 2;
  const int col_blocks = p.rows / BLOCK;
  const bool has_gamma = NORM && p.gamma != nullptr;
  const bool rowwise = p.row_values != nullptr;
  const uint32_t rank = NORM ? cluster_ctarank() : 0;
  const uint32_t members = NORM ? gridDim.x : 1;
  if (has_gamma) stage_gamma(p.gamma + pc0, W, s_gamma);
  // A member's shared memory may be written only once that member runs: every CTA of the cluster
  // passes this barrier before the first remote store.
  if (NORM) cluster_sync_all();

  for (int rr = warp; rr < 32; rr += warps) {
    const __nv_bfloat16* xr = p.x + (row0 + rr) * p.ldx + pc0;
    __nv_bfloat16* trow = tile + rr * ld;
    float ss = 0.f;
    for (int c = lane * 8; c < W; c += 256) {
      const uint4 q = ld_nc_v4(xr + c);
      *reinterpret_cast<uint4*>(trow + c) = q;
      if (NORM) {
        float f[8];
        unpack8(q, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
      }
    }
    if (NORM) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane < members)
        st_shared_cluster_f32(mapa_shared(smem_u32(s_ss + rank * 32 + rr), lane), ss);
    }
  }
  if (NORM) cluster_sync_all();  // every member's partial sums have landed; nothing remote after this

  const int sf_lane = (lane >> 4) * 512 + ((lane >> 2) & 3);
  if (NORM || rowwise) {
    for (int rr = warp; rr < 32; rr += warps) {
      const long long row = row0 + rr;
      __nv_bfloat16* trow = tile + rr * ld;
      float r = 1.0f;
      if (NORM) {
        float ss = 0.f;
        for (uint32_t k = 0; k < members; ++k) ss += s_ss[k * 32 + rr];
        r = rsqrtf(ss * (1.0f / static_cast<float>(p.cols)) + p.eps);
        if (rank == 0 && lane == 0 && p.r_inv != nullptr) p.r_inv[row * p.r_inv_stride] = r;
      }
      uint8_t* out = rowwise ? p.row_values + row * p.cols + pc0 + lane * 8 : nullptr;
      uint8_t* sf = rowwise ? p.row_sf + ((row >> 7) * row_tiles + (pc0 >> 7)) * 512 +
                                  (row & 31) * 16 + ((row & 127) >> 5) * 4 + sf_lane
                            : nullptr;
      for (int c0 = 0; c0 < W; c0 += 256) {
        const int c = c0 + lane * 8;
        const uint4 xq = *reinterpret_cast<const uint4*>(trow + c);
        uint32_t q[4] = {xq.x, xq.y, xq.z, xq.w};
        if (NORM) {
          norm_packed8(xq, r, has_gamma ? s_gamma + (c0 >> 2) + lane : nullptr, q);
          *reinterpret_cast<uint4*>(trow + c) = make_uint4(q[0], q[1], q[2], q[3]);
        }
        if (rowwise) {  // CTA-uniform: the shuffles see whole warps
          uint32_t e;
          const uint2 o = quantize_packed8(q, e);
          *reinterpret_cast<uint2*>(out + c0) = o;
          if ((lane & 3) == 0) sf[(c0 >> 7) * 512] = static_cast<uint8_t>(e);
        }
      }
    }
  }
  __syncthreads();
  for (int c2 = threadIdx.x; c2 < W / 2; c2 += blockDim.x)
    quantize_column_pair(p, tile, ld, c2, pc0, row0, col_blocks);
}

// NVFP4 rowwise output (NormOutput::Nvfp4Rowwise, no global scale): blocks of 16 elements, scale
// = amax / 6 rounded to nearest E4M3, elements x * (1 / scale) rounded to nearest E2M1 (ties to
// even, saturating), two per byte; a block whose scale rounds to zero stores zeros
// (crates/cleandl-specialized-kernels/src/utils/block_scale.rs:28-31, 55-66; the reciprocal and
// the product are correctly rounded f32 operations where the reference takes an approximate
// bf16 reciprocal, so that a host restatement reproduces the bits).  A lane's 8 elements are
// half a block: one shuffle.  x is read twice (the second time from cache).
template <bool NORM>
__global__ void __launch_bounds__(256, 2) nvfp4_rows_kernel(const Params p) {
  const int lane = threadIdx.x & 31;
  const int row_blocks = p.cols / 16;
  const float inv_cols = 1.0f / static_cast<float>(p.cols);
  const long long warp_global = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const long long warp_stride = static_cast<long long>(gridDim.x) * 8;
  for (long long row = warp_global; row < p.rows; row += warp_stride) {
    const __nv_bfloat16* xr = p.x + row * p.ldx;
    float r = 1.0f;
    if (NORM) {
      float ss = 0.f;
      for (int c = lane * 8; c < p.cols; c += 256) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(xr + c), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      r = rsqrtf(ss * inv_cols + p.eps);
      if (lane == 0 && p.r_inv != nullptr) p.r_inv[row * p.r_inv_stride] = r;
    }
    for (int c0 = 0; c0 < p.cols; c0 += 256) {  // warp-uniform: the shuffle needs all lanes
      const int c = c0 + lane * 8;
      const bool active = c < p.cols;  // cols % 16 == 0: both lanes of a block agree
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = 0.f;
      if (active) apply_norm8<NORM>(p, *reinterpret_cast<const uint4*>(xr + c), c, r, f);
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      if (active) {
        const __nv_fp8_storage_t sbits =
            __nv_cvt_float_to_fp8(__fdiv_rn(amax, 6.0f), __NV_SATFINITE, __NV_E4M3);
        const float sc = __half2float(__half(__nv_cvt_fp8_to_halfraw(sbits, __NV_E4M3)));
        const float inv = sc != 0.f ? __frcp_rn(sc) : 0.f;  // a zero scale stores zeros
        uint32_t out = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = __fmul_rn(f[2 * j], inv);
          const float b = __fmul_rn(f[2 * j + 1], inv);
          out |= static_cast<uint32_t>(__nv_cvt_float2_to_fp4x2(make_float2(a, b), __NV_E2M1, cudaRoundNearest))
                 << (8 * j);
        }
        *reinterpret_cast<uint32_t*>(p.row_values + (row * p.cols + c) / 2) = out;
        if ((lane & 1) == 0)
          p.row_sf[sf_index(static_cast<int>(row), c / 16, row_blocks)] = sbits;
      }
    }
  }
}

// nvfp4_rows_kernel for cols == 256 * NCH exactly and no bias, trimmed like mx_row_full_kernel:
// the row stays in registers (x is read once), the scale vector sits in shared memory as f32, the
// block maximum is taken on the packed bf16 results, index arithmetic is per row.
template <bool NORM, int NCH>
__global__ void __launch_bounds__(256, NCH <= 8 ? FULL_MIN_CTAS : 1) nvfp4_row_full_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  float4* s_gamma = reinterpret_cast<float4*>(smem_raw);
  constexpr int COLS = NCH * 256;
  const int lane = threadIdx.x & 31;
  const bool has_gamma = NORM && p.gamma != nullptr;
  if (has_gamma) stage_gamma(p.gamma, COLS, s_gamma);
  // Block of (stripe s, lane): b = 16 s + lane / 2, so b / 4 = 4 s + lane / 8, b % 4 = lane / 2 % 4.
  const int sf_lane = (lane >> 3) * 512 + ((lane >> 1) & 3);
  const long long warp_global = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const long long warp_stride = static_cast<long long>(gridDim.x) * 8;
  for (long long row = warp_global; row < p.rows; row += warp_stride) {
    const uint4* xr = reinterpret_cast<const uint4*>(p.x + row * p.ldx) + lane;
    uint4 xv[NCH];
#pragma unroll
    for (int s = 0; s < NCH; ++s) xv[s] = ld_nc_v4(xr + s * 32);
    float r = 1.0f;
    if (NORM) {
      float ss = 0.f;
#pragma unroll
      for (int s = 0; s < NCH; ++s) {
        float f[8];
        unpack8(xv[s], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      r = rsqrtf(ss * (1.0f / COLS) + p.eps);
      if (lane == 0 && p.r_inv != nullptr) p.r_inv[row * p.r_inv_stride] = r;
    }
    uint32_t* out = reinterpret_cast<uint32_t*>(p.row_values + row * (COLS / 2)) + lane;
    uint8_t* sf = p.row_sf + (row >> 7) * (NCH * 4 * 512) + (row & 31) * 16 + ((row & 127) >> 5) * 4 +
                  sf_lane;
#pragma unroll
    for (int s = 0; s < NCH; ++s) {
      uint32_t q[4] = {xv[s].x, xv[s].y, xv[s].z, xv[s].w};
      if (NORM) norm_packed8(xv[s], r, has_gamma ? s_gamma + s * 64 + lane : nullptr, q);
      uint32_t m = max_bf16x2(abs_max_bf16x2(q[0], q[1]), abs_max_bf16x2(q[2], q[3]));
      m = max_bf16x2(m, __shfl_xor_sync(0xffffffffu, m, 1));  // a block of 16 is two lanes
      m = max_bf16x2(m, __byte_perm(m, 0, 0x1032));
      const float amax = __uint_as_float(m & 0xFFFF0000u);
      const __nv_fp8_storage_t sbits =
          __nv_cvt_float_to_fp8(__fdiv_rn(amax, 6.0f), __NV_SATFINITE, __NV_E4M3);
      const float sc = __half2float(__half(__nv_cvt_fp8_to_halfraw(sbits, __NV_E4M3)));
      const float inv = sc != 0.f ? __frcp_rn(sc) : 0.f;  // a zero scale stores zeros
      uint32_t word = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        word |= static_cast<uint32_t>(__nv_cvt_float2_to_fp4x2(
                    make_float2(__fmul_rn(bf16_lo(q[j]), inv), __fmul_rn(bf16_hi(q[j]), inv)), __NV_E2M1,
                    cudaRoundNearest))
                << (8 * j);
      out[s * 32] = word;
      if ((lane & 1) == 0) sf[s * 2048] = sbits;
    }
  }
}

// One thread per block: y[r, c] = value * scale (MXFP8: 32 E4M3 values, UE8M0 scale; NVFP4: 16
// E2M1 values in 8 bytes, E4M3 scale).
__global__ void mx_dequantize_kernel(const uint8_t* __restrict__ values,
                                     const uint8_t* __restrict__ sf, int outer, int inner,
                                     int colwise, int fp4, void* y, int y_f32, long long ldy) {
  const int block = fp4 ? 16 : BLOCK;
  const int blocks = inner / block;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(outer) * blocks) return;
  const int o = static_cast<int>(idx / blocks), b = static_cast<int>(idx % blocks);
  const uint32_t e = sf[sf_index(o, b, blocks)];
  float s;
  if (fp4) s = __half2float(__half(__nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(e), __NV_E4M3)));
  else s = e == 0xFFu ? __int_as_float(0x7FC00000) : __uint_as_float(e != 0 ? e << 23 : 0x00400000u);
  const long long first = static_cast<long long>(o) * inner + b * block;  // element index
  for (int j = 0; j < block; ++j) {
    float v;
    if (fp4) {
      const uint8_t byte = values[(first + j) >> 1];
      const uint32_t nib = (j & 1) ? byte >> 4 : byte & 0xF;
      const float mag = (nib & 7) < 2 ? 0.5f * (nib & 7) : (nib & 7) < 4 ? 0.5f * (nib & 7)
                        : (nib & 7) == 4 ? 2.f : (nib & 7) == 5 ? 3.f : (nib & 7) == 6 ? 4.f : 6.f;
      v = (nib & 8) ? -mag : mag;
    } else {
      v = __half2float(__half(__nv_cvt_fp8_to_halfraw(values[first + j], __NV_E4M3)));
    }
    v *= s;
    const long long r = colwise ? b * block + j : o, c = colwise ? o : b * block + j;
    if (y_f32) static_cast<float*>(y)[r * ldy + c] = v;
    else static_cast<__nv_bfloat16*>(y)[r * ldy + c] = __float2bfloat16_rn(v);
  }
}

}  // namespace mx

int32_t mx_layout(int32_t format, int32_t dim, long long rows, long long cols, size_t* values_bytes,
                  size_t* scale_bytes) {
  if (format != CDL_MXFP8 && format != CDL_NVFP4)
    return fail(CDL_ERR_INVALID, "block-scaled tensors: unknown format %d", format);
  if (dim != CDL_MX_ROWWISE && dim != CDL_MX_COLWISE)
    return fail(CDL_ERR_INVALID, "block-scaled tensors: unknown block dimension %d", dim);
  if (rows < 0 || cols < 0) return fail(CDL_ERR_INVALID, "block-scaled tensors: negative shape");
  const long long outer = dim == CDL_MX_ROWWISE ? rows : cols;
  const long long inner = dim == CDL_MX_ROWWISE ? cols : rows;
  const int block = format == CDL_MXFP8 ? 32 : 16;
  if (inner % block != 0)
    return fail(CDL_ERR_INVALID,
                "block dimension of shape [%lld, %lld] must be a multiple of the %s block size %d",
                rows, cols, format == CDL_MXFP8 ? "MXFP8" : "NVFP4", block);
  if (values_bytes) *values_bytes = static_cast<size_t>(outer) * inner / (format == CDL_MXFP8 ? 1 : 2);
  if (scale_bytes)
    *scale_bytes = static_cast<size_t>((outer + 127) / 128 * 128) * ((inner / block + 3) / 4 * 4);
  return CDL_OK;
}

int32_t mx_check(const char* op, const char* name, const cdl_mx_tensor* t, int32_t dim, long long rows,
                 long long cols) {
  if (t->dim != dim)
    return fail(CDL_ERR_INVALID, "%s: %s must have its blocks along the %s", op, name,
                dim == CDL_MX_ROWWISE ? "rows (rowwise)" : "columns (colwise)");
  if (t->rows != rows || t->cols != cols)
    return fail(CDL_ERR_INVALID, "%s: %s must have shape [%lld, %lld], got [%lld, %lld]", op, name,
                rows, cols, static_cast<long long>(t->rows), static_cast<long long>(t->cols));
  CDL_CHECK(mx_layout(t->format, t->dim, rows, cols, nullptr, nullptr));
  if (rows > 0 && cols > 0) {
    if (!t->values || !t->scale_factors)
      return fail(CDL_ERR_INVALID, "%s: %s has no values or scale factors", op, name);
    if ((reinterpret_cast<uintptr_t>(t->values) & 31) != 0 ||
        (reinterpret_cast<uintptr_t>(t->scale_factors) & 15) != 0)
      return fail(CDL_ERR_UNSUPPORTED,
                  "%s: %s: values must be 32-byte and scale factors 16-byte aligned", op, name);
  }
  return CDL_OK;
}

static int32_t mx_rows_run(const char* op, const cdl_tensor* x, const cdl_tensor* scale,
                           const cdl_tensor* bias, float eps, bool norm, const cdl_mx_tensor* y_row,
                           const cdl_mx_tensor* y_col, const cdl_tensor* r_inv, cudaStream_t stream) {
  using namespace mx;
  if (!x) return fail(CDL_ERR_INVALID, "%s: x is required", op);
  if (!y_row && !y_col) return fail(CDL_ERR_INVALID, "%s: at least one output is required", op);
  if (x->rank != 2) return fail(CDL_ERR_INVALID, "%s: x must be a 2D tensor", op);
  if (x->dtype != CDL_BF16) return fail(CDL_ERR_UNSUPPORTED, "%s: x must be bf16", op);
  const long long rows = x->shape[0], cols = x->shape[1];
  if (cols > 1 && x->stride[1] != 1)
    return fail(CDL_ERR_UNSUPPORTED, "%s: x must have packed rows (contiguous columns)", op);
  if ((reinterpret_cast<uintptr_t>(x->ptr) & 15) != 0 || (rows > 1 && x->stride[0] % 8 != 0))
    return fail(CDL_ERR_UNSUPPORTED, "%s: x must be 16-byte aligned (pointer and row stride)", op);
  if (y_row && y_row->format == CDL_MXFP8 && cols % BLOCK != 0)
    return fail(CDL_ERR_INVALID,
                "%s: the number of columns (%lld) must be a multiple of the MXFP8 block size 32", op,
                cols);
  if (y_row && y_row->format == CDL_NVFP4 && cols % 16 != 0)
    return fail(CDL_ERR_INVALID,
                "%s: the number of columns (%lld) must be a multiple of the NVFP4 block size 16", op,
                cols);
  if (cols % 8 != 0)
    return fail(CDL_ERR_UNSUPPORTED, "%s: the number of columns (%lld) must be a multiple of 8", op,
                cols);
  if (y_row) CDL_CHECK(mx_check(op, "rowwise output", y_row, CDL_MX_ROWWISE, rows, cols));
  if (y_col) CDL_CHECK(mx_check(op, "colwise output", y_col, CDL_MX_COLWISE, rows, cols));
  const bool fp4 = y_row && y_row->format == CDL_NVFP4;
  if (y_col && (fp4 || y_col->format != CDL_MXFP8))
    return fail(CDL_ERR_UNSUPPORTED,
                "%s: a colwise output exists for MXFP8 only (the outputs are MXFP8 rowwise, MXFP8 "
                "rowwise and colwise, or NVFP4 rowwise)", op);
  for (const cdl_tensor* v : {scale, bias}) {
    if (!v) continue;
    if (v->rank != 1 || v->shape[0] != cols || v->dtype != CDL_BF16 || v->stride[0] != 1 ||
        (reinterpret_cast<uintptr_t>(v->ptr) & 15) != 0)
      return fail(CDL_ERR_INVALID, "%s: scale and bias must be contiguous 16-byte aligned bf16 [%lld]",
                  op, cols);
  }
  if (r_inv && (r_inv->rank != 1 || r_inv->shape[0] != rows || r_inv->dtype != CDL_F32))
    return fail(CDL_ERR_INVALID, "%s: r_inv must be f32 [%lld]", op, rows);
  if (rows == 0 || cols == 0) return CDL_OK;
  if (rows > INT32_MAX / 2 || cols > 65536)
    return fail(CDL_ERR_UNSUPPORTED, "%s: shape [%lld, %lld] is too large", op, rows, cols);

  Params p{};
  p.x = static_cast<const __nv_bfloat16*>(x->ptr);
  p.ldx = x->stride[0];
  p.rows = static_cast<int>(rows);
  p.cols = static_cast<int>(cols);
  p.gamma = scale ? static_cast<const __nv_bfloat16*>(scale->ptr) : nullptr;
  p.beta = bias ? static_cast<const __nv_bfloat16*>(bias->ptr) : nullptr;
  p.eps = eps;
  p.r_inv = r_inv ? static_cast<float*>(r_inv->ptr) : nullptr;
  p.r_inv_stride = r_inv ? r_inv->stride[0] : 0;
  if (y_row) {
    p.row_values = static_cast<uint8_t*>(y_row->values);
    p.row_sf = static_cast<uint8_t*>(y_row->scale_factors);
  }
  if (y_col) {
    p.col_values = static_cast<uint8_t*>(y_col->values);
    p.col_sf = static_cast<uint8_t*>(y_col->scale_factors);
  }
  // algorithmic bytes: x read, one byte per element and output, one scale byte per 32
  const double bytes = 2.0 * rows * cols + ((y_row ? 1 : 0) + (y_col ? 1 : 0)) * (rows * cols * (1.0 + 1.0 / 32));
  ProfileScope ps(PROF_NORM_FWD, bytes, stream);
  if (fp4) {
    const long long want = (rows + 7) / 8;
    const unsigned grid = static_cast<unsigned>(want < 16LL * sm_count() ? want : 16LL * sm_count());
    const long long nch = cols / 256;
    const bool full = cols % 256 == 0 && cols <= 4096 && (nch & (nch - 1)) == 0 && !(norm && bias);
    const size_t gamma_bytes = norm && scale ? static_cast<size_t>(cols) * 4 : 0;
#define CDL_FP4_FULL(NCH)                                                                  \
  do {                                                                                     \
    if (norm) nvfp4_row_full_kernel<true, NCH><<<grid, 256, gamma_bytes, stream>>>(p);     \
    else nvfp4_row_full_kernel<false, NCH><<<grid, 256, 0, stream>>>(p);                   \
  } while (0)
    if (full) {
      switch (nch) {
        case 1: CDL_FP4_FULL(1); break;
        case 2: CDL_FP4_FULL(2); break;
        case 4: CDL_FP4_FULL(4); break;
        case 8: CDL_FP4_FULL(8); break;
        default: CDL_FP4_FULL(16); break;
      }
    } else if (norm) nvfp4_rows_kernel<true><<<grid, 256, 0, stream>>>(p);
    else nvfp4_rows_kernel<false><<<grid, 256, 0, stream>>>(p);
#undef CDL_FP4_FULL
  } else if (y_col) {
    int dev = 0;
    CDL_CUDA(cudaGetDevice(&dev));
    const size_t tile_bytes = 32 * static_cast<size_t>(cols + 8) * 2;
    const size_t gamma_bytes = norm && scale ? static_cast<size_t>(cols) * 4 : 0;
    const bool whole_rows = tile_bytes <= 227 * 1024;
    // panels a multiple of 256 columns wide and no bias: the trimmed kernel
    const bool full = cols % 256 == 0 && !(norm && bias) &&
                      (!whole_rows || tile_bytes + gamma_bytes <= 227 * 1024);
    static std::once_flag once[64];
    cudaError_t err = cudaSuccess;
    std::call_once(once[dev & 63], [&] {
      const void* fns[8] = {reinterpret_cast<const void*>(&mx_rows_kernel<true, true>),
                            reinterpret_cast<const void*>(&mx_rows_kernel<false, true>),
                            reinterpret_cast<const void*>(&mx_rowcol_tile_kernel<true>),
                            reinterpret_cast<const void*>(&mx_rowcol_tile_kernel<false>),
                            reinterpret_cast<const void*>(&mx_rowcol_full_kernel<true>),
                            reinterpret_cast<const void*>(&mx_rowcol_full_kernel<false>),
                            reinterpret_cast<const void*>(&mx_rowcol_panel_kernel<true>),
                            reinterpret_cast<const void*>(&mx_rowcol_panel_kernel<false>)};
      for (int i = 0; i < 8 && err == cudaSuccess; ++i)
        err = cudaFuncSetAttribute(fns[i], cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   i < 2 ? static_cast<int>(COL_SMEM_BYTES) : 227 * 1024);
    });
    if (err != cudaSuccess)
      return fail(CDL_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(err));
    const unsigned grid = static_cast<unsigned>(rows / 32);
    // Panels of 1024 (else 512) columns when they tile the row: every plain quantisation, and the
    // normalisation of rows too long for 32 of them to sit in one CTA's shared memory (the panels
    // of a row then form a cluster, which holds at most 8 CTAs; rows that fit measured the same
    // either way and stay with the whole-row kernel).
    const int panel = cols % 1024 == 0 ? 1024 : cols % 512 == 0 ? 512 : 0;
    const bool use_panels = panel != 0 && rows / 32 <= 65535 &&
                            (!norm || (!bias && cols / panel <= 8 && !(whole_rows && full)));
    if (use_panels) {
      p.panel_cols = panel;
      const size_t smem = 64 * static_cast<size_t>(panel + 8) + static_cast<size_t>(panel) * 4 + 8 * 32 * 4;
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(static_cast<unsigned>(cols / panel), grid);
      cfg.blockDim = dim3(static_cast<unsigned>(panel / 2));
      cfg.dynamicSmemBytes = smem;
      cfg.stream = stream;
      cudaLaunchAttribute attr{};
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = norm ? static_cast<unsigned>(cols / panel) : 1;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      if (norm) CDL_CUDA(cudaLaunchKernelEx(&cfg, mx_rowcol_panel_kernel<true>, p));
      else CDL_CUDA(cudaLaunchKernelEx(&cfg, mx_rowcol_panel_kernel<false>, p));
    } else if (whole_rows) {
      p.panel_cols = static_cast<int>(cols);
      if (full && norm) mx_rowcol_full_kernel<true><<<grid, 1024, tile_bytes + gamma_bytes, stream>>>(p);
      else if (full) mx_rowcol_full_kernel<false><<<grid, 1024, tile_bytes, stream>>>(p);
      else if (norm) mx_rowcol_tile_kernel<true><<<grid, 1024, tile_bytes, stream>>>(p);
      else mx_rowcol_tile_kernel<false><<<grid, 1024, tile_bytes, stream>>>(p);
    } else if (!norm) {
      // plain quantisation of wide rows: panels of 2048 columns (a multiple of the 256-column stripe)
      p.panel_cols = 2048;
      const dim3 g2(grid, static_cast<unsigned>((cols + 2047) / 2048));
      if (full) mx_rowcol_full_kernel<false><<<g2, 1024, 32 * (2048 + 8) * 2, stream>>>(p);
      else mx_rowcol_tile_kernel<false><<<g2, 1024, 32 * (2048 + 8) * 2, stream>>>(p);
    } else {
      if (norm) mx_rows_kernel<true, true><<<grid, 1024, COL_SMEM_BYTES, stream>>>(p);
      else mx_rows_kernel<false, true><<<grid, 1024, COL_SMEM_BYTES, stream>>>(p);
    }
  } else {
    const long long want = (rows + 7) / 8;
    const unsigned grid = static_cast<unsigned>(want < 16LL * sm_count() ? want : 16LL * sm_count());
#define CDL_MX_ROW(NCH)                                                                  \
  do {                                                                                   \
    if (norm) mx_row_cached_kernel<true, NCH><<<grid, 256, 0, stream>>>(p);              \
    else mx_row_cached_kernel<false, NCH><<<grid, 256, 0, stream>>>(p);                  \
  } while (0)
    // cols == 256 * NCH exactly, no bias, up to 4096 columns: the trimmed kernel (scale vector
    // as f32 in shared memory, at most 16 KiB)
    const bool full = cols % 256 == 0 && cols <= 4096 && (cols / 256 & (cols / 256 - 1)) == 0 &&
                      !(norm && bias);
    const size_t gamma_bytes = norm && scale ? static_cast<size_t>(cols) * 4 : 0;
#define CDL_MX_FULL(NCH)                                                                 \
  do {                                                                                   \
    if (norm) mx_row_full_kernel<true, NCH><<<grid, 256, gamma_bytes, stream>>>(p);      \
    else mx_row_full_kernel<false, NCH><<<grid, 256, 0, stream>>>(p);                    \
  } while (0)
    if (full) {
      switch (cols / 256) {
        case 1: CDL_MX_FULL(1); break;
        case 2: CDL_MX_FULL(2); break;
        case 4: CDL_MX_FULL(4); break;
        case 8: CDL_MX_FULL(8); break;
        default: CDL_MX_FULL(16); break;
      }
    } else
#undef CDL_MX_FULL
    if (cols <= 256) CDL_MX_ROW(1);
    else if (cols <= 512) CDL_MX_ROW(2);
    else if (cols <= 1024) CDL_MX_ROW(4);
    else if (cols <= 2048) CDL_MX_ROW(8);
    else if (cols <= 4096) CDL_MX_ROW(16);
    else if (cols <= 8192) CDL_MX_ROW(32);
    else if (norm) mx_rows_kernel<true, false><<<grid, 256, 0, stream>>>(p);
    else mx_rows_kernel<false, false><<<grid, 256, 0, stream>>>(p);
#undef CDL_MX_ROW
  }
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

int32_t rmsnorm_fwd_mx_execute(const cdl_tensor* x, const cdl_tensor* scale, const cdl_tensor* bias,
                               float eps, const cdl_mx_tensor* y_row, const cdl_mx_tensor* y_col,
                               const cdl_tensor* r_inv, cudaStream_t stream) {
  if (!y_row)
    return fail(CDL_ERR_INVALID, "norm_fwd (mxfp8): the rowwise output is required "
                                 "(the outputs are rowwise, or rowwise and colwise)");
  return mx_rows_run("norm_fwd (mxfp8)", x, scale, bias, eps, true, y_row, y_col, r_inv, stream);
}

int32_t mx_quantize_execute(const cdl_tensor* x, const cdl_mx_tensor* y_row,
                            const cdl_mx_tensor* y_col, cudaStream_t stream) {
  return mx_rows_run("mx_quantize", x, nullptr, nullptr, 0.f, false, y_row, y_col, nullptr, stream);
}

int32_t mx_dequantize_execute(const cdl_mx_tensor* x, const cdl_tensor* y, cudaStream_t stream) {
  const char* op = "mx_dequantize";
  if (!x || !y) return fail(CDL_ERR_INVALID, "%s: x and y are required", op);
  CDL_CHECK(mx_check(op, "x", x, x->dim, x->rows, x->cols));
  if (y->rank != 2 || y->shape[0] != x->rows || y->shape[1] != x->cols ||
      (y->dtype != CDL_BF16 && y->dtype != CDL_F32) || (x->cols > 1 && y->stride[1] != 1))
    return fail(CDL_ERR_INVALID, "%s: y must be a bf16 or f32 [%lld, %lld] tensor with packed rows", op,
                static_cast<long long>(x->rows), static_cast<long long>(x->cols));
  if (x->rows == 0 || x->cols == 0) return CDL_OK;
  const bool colwise = x->dim == CDL_MX_COLWISE;
  const long long outer = colwise ? x->cols : x->rows, inner = colwise ? x->rows : x->cols;
  if (outer > INT32_MAX / 2 || inner > INT32_MAX / 2)
    return fail(CDL_ERR_UNSUPPORTED, "%s: shape too large", op);
  const bool fp4 = x->format == CDL_NVFP4;
  const long long n = outer * (inner / (fp4 ? 16 : mx::BLOCK));
  mx::mx_dequantize_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
      static_cast<const uint8_t*>(x->values), static_cast<const uint8_t*>(x->scale_factors),
      static_cast<int>(outer), static_cast<int>(inner), colwise ? 1 : 0, fp4 ? 1 : 0, y->ptr,
      y->dtype == CDL_F32 ? 1 : 0, y->stride[0]);
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

}  // namespace cdl

extern "C" {

int32_t cdl_b200_mx_layout(int32_t format, int32_t dim, int64_t rows, int64_t cols,
                           size_t* values_bytes, size_t* scale_bytes) {
  return cdl::mx_layout(format, dim, rows, cols, values_bytes, scale_bytes);
}

int32_t cdl_b200_mx_quantize(const cdl_tensor* x, const cdl_mx_tensor* y_rowwise,
                             const cdl_mx_tensor* y_colwise, cdl_stream stream) {
  return cdl::mx_quantize_execute(x, y_rowwise, y_colwise, static_cast<cudaStream_t>(stream));
}

int32_t cdl_b200_mx_dequantize(const cdl_mx_tensor* x, const cdl_tensor* y, cdl_stream stream) {
  return cdl::mx_dequantize_execute(x, y, static_cast<cudaStream_t>(stream));
}

int32_t cdl_b200_rmsnorm_fwd_mx(const cdl_tensor* x, const cdl_tensor* scale, const cdl_tensor* bias,
                                float eps, const cdl_mx_tensor* y_rowwise,
                                const cdl_mx_tensor* y_colwise, const cdl_tensor* r_inv,
                                cdl_stream stream) {
  return cdl::rmsnorm_fwd_mx_execute(x, scale, bias, eps, y_rowwise, y_colwise, r_inv,
                                     static_cast<cudaStream_t>(stream));
}

}  // extern "C"
