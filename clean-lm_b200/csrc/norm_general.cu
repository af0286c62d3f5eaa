// General NormFwd for what the vectorised kernels of rmsnorm.cu do not take: f32 inputs or
// outputs, f32 scale / bias, a column count that is not a multiple of 8 or exceeds 8192, strided or
// unaligned rows.  In the reference these shapes run on its Tile IR fallback (NormFwd with
// NormOutput::Plain, crates/cleandl/src/execgraph/ops/norm/mod.rs:223-261; the case list of
// fallback_configurations, crates/cleandl/tests/norm.rs:414-470: every combination of f32 / bf16
// x, output, scale and bias for both norm types, and rows of 20000 columns).
//
//   RmsNorm:   y = x * rsqrt(mean x^2 + eps) * scale + bias
//   LayerNorm: y = (x - mean x) * rsqrt(mean (x - mean x)^2 + eps) * scale + bias
// in f32, one warp per row, scalar accesses, the row read two or three times (from cache after the
// first).  The completeness path: correct for any layout, no claim on speed.
#include "host.h"
#include "ops.h"
#include "ptx.cuh"

namespace cdl {
namespace norm_general {

struct Vec {
  const void* ptr;  // nullable
  long long stride;
  int f32;
};
struct Params {
  const void* x;
  long long x_row, x_col;
  int x_f32;
  void* y;
  long long y_row, y_col;
  int y_f32;
  Vec scale, bias;
  float* mean;  // nullable
  long long mean_stride;
  float* r_inv;  // nullable
  long long r_inv_stride;
  int rows, cols;
  float eps;
  int layer;
};

__device__ __forceinline__ float load(const void* p, long long i, int f32) {
  return f32 ? static_cast<const float*>(p)[i]
             : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(256) norm_general_kernel(const Params p) {
  const int lane = threadIdx.x & 31;
  const long long warp = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * 8;
  const float inv_cols = 1.0f / static_cast<float>(p.cols);
  for (long long row = warp; row < p.rows; row += stride) {
    const long long xb = row * p.x_row;
    float mean = 0.f;
    if (p.layer) {
      float s = 0.f;
      for (int c = lane; c < p.cols; c += 32) s += load(p.x, xb + c * p.x_col, p.x_f32);
      mean = warp_sum(s) * inv_cols;
    }
    float ss = 0.f;
    for (int c = lane; c < p.cols; c += 32) {
      const float d = load(p.x, xb + c * p.x_col, p.x_f32) - mean;
      ss = fmaf(d, d, ss);
    }
    const float r = rsqrtf(warp_sum(ss) * inv_cols + p.eps);
    if (lane == 0) {
      if (p.mean != nullptr) p.mean[row * p.mean_stride] = mean;
      if (p.r_inv != nullptr) p.r_inv[row * p.r_inv_stride] = r;
    }
    const long long yb = row * p.y_row;
    for (int c = lane; c < p.cols; c += 32) {
      float v = (load(p.x, xb + c * p.x_col, p.x_f32) - mean) * r;
      if (p.scale.ptr != nullptr) v *= load(p.scale.ptr, c * p.scale.stride, p.scale.f32);
      if (p.bias.ptr != nullptr) v += load(p.bias.ptr, c * p.bias.stride, p.bias.f32);
      const long long yi = yb + c * p.y_col;
      if (p.y_f32) static_cast<float*>(p.y)[yi] = v;
      else static_cast<__nv_bfloat16*>(p.y)[yi] = __float2bfloat16_rn(v);
    }
  }
}

static bool float_type(int32_t dt) { return dt == CDL_BF16 || dt == CDL_F32; }

}  // namespace norm_general

// layer = 0: RmsNorm (mean must be null), 1: LayerNorm.  Validates everything itself.
int32_t norm_general_execute(int layer, const cdl_tensor* x, const cdl_tensor* scale,
                             const cdl_tensor* bias, float eps, const cdl_tensor* y,
                             const cdl_tensor* mean, const cdl_tensor* r_inv, cudaStream_t stream) {
  using namespace norm_general;
  const char* op = layer ? "norm_fwd (layer norm)" : "norm_fwd";
  if (!x || !y) return fail(CDL_ERR_INVALID, "%s: x and y are required", op);
  if (x->rank != 2) return fail(CDL_ERR_INVALID, "%s: x must be a 2D tensor", op);
  const long long rows = x->shape[0], cols = x->shape[1];
  if (y->rank != 2 || y->shape[0] != rows || y->shape[1] != cols)
    return fail(CDL_ERR_INVALID, "%s: y must be a 2D tensor of shape [%lld, %lld]", op, rows, cols);
  if (!float_type(x->dtype) || !float_type(y->dtype))
    return fail(CDL_ERR_UNSUPPORTED, "%s: x and y must be f32 or bf16", op);
  for (const cdl_tensor* v : {scale, bias}) {
    if (!v) continue;
    if (v->rank != 1 || v->shape[0] != cols)
      return fail(CDL_ERR_INVALID, "%s: %s must have shape [%lld]", op, v == scale ? "scale" : "bias",
                  cols);
    if (!float_type(v->dtype))
      return fail(CDL_ERR_UNSUPPORTED, "%s: %s must be f32 or bf16", op, v == scale ? "scale" : "bias");
  }
  for (const cdl_tensor* v : {mean, r_inv}) {
    if (!v) continue;
    if (v->rank != 1 || v->shape[0] != rows || v->dtype != CDL_F32)
      return fail(CDL_ERR_INVALID, "%s: %s must be f32 [%lld]", op, v == mean ? "mean" : "r_inv", rows);
  }
  if (rows == 0 || cols == 0) return CDL_OK;
  if (rows > INT32_MAX || cols > INT32_MAX)
    return fail(CDL_ERR_UNSUPPORTED, "%s: shape [%lld, %lld] is too large", op, rows, cols);
  Params p{};
  p.x = x->ptr; p.x_row = x->stride[0]; p.x_col = x->stride[1]; p.x_f32 = x->dtype == CDL_F32;
  p.y = y->ptr; p.y_row = y->stride[0]; p.y_col = y->stride[1]; p.y_f32 = y->dtype == CDL_F32;
  if (scale) p.scale = Vec{scale->ptr, scale->stride[0], scale->dtype == CDL_F32};
  if (bias) p.bias = Vec{bias->ptr, bias->stride[0], bias->dtype == CDL_F32};
  if (mean) { p.mean = static_cast<float*>(mean->ptr); p.mean_stride = mean->stride[0]; }
  if (r_inv) { p.r_inv = static_cast<float*>(r_inv->ptr); p.r_inv_stride = r_inv->stride[0]; }
  p.rows = static_cast<int>(rows);
  p.cols = static_cast<int>(cols);
  p.eps = eps;
  p.layer = layer;
  const double elem = (p.x_f32 ? 4.0 : 2.0) + (p.y_f32 ? 4.0 : 2.0);
  ProfileScope ps(PROF_NORM_FWD, elem * rows * cols, stream);
  const long long want = (rows + 7) / 8;
  const unsigned grid = static_cast<unsigned>(want < 16LL * sm_count() ? want : 16LL * sm_count());
  norm_general_kernel<<<grid, 256, 0, stream>>>(p);
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

}  // namespace cdl
