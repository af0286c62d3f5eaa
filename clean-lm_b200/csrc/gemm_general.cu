// General matmul for the operands the tensor-memory kernels of gemm.cu cannot take: pointers or
// leading dimensions that are not 16-byte aligned (TMA cannot describe them; the reference hands
// them to cuBLASLt, tests `unaligned_operands`, crates/cleandl/tests/matmul.rs:604-630) and f32
// inputs (`f32_tf32_matmul`, tests/matmul.rs:243-265: the reference computes those with TF32
// tensor cores, 10 mantissa bits; here the products are full f32, which its tolerance contains).
//
// D = alpha * A . B + beta * C with arbitrary element strides for A and B, f32 accumulation on
// the CUDA cores.  This is the completeness path, not a fast one: a 64 x 64 tile per CTA of 256
// threads, 4 x 4 outputs per thread, K in steps of 16 through shared memory with scalar loads.
#include "host.h"
#include "ops.h"
#include "ptx.cuh"

namespace cdl {
namespace gemm_general {

struct Params {
  const void* a;
  const void* b;
  const void* c;  // nullable
  void* d;
  long long a_batch, a_row, a_col;  // element strides of A [batch, M, K]
  long long b_batch, b_row, b_col;  // B [batch, K, N]
  long long c_batch, c_row;         // C [batch, M, N], last dimension contiguous
  long long d_batch, d_row;
  int M, N, K;
  int c_f32, d_f32;
  float alpha, beta;
};

constexpr int TILE = 64;
constexpr int KSTEP = 16;

__device__ __forceinline__ float load_as_f32(const float* p) { return *p; }
__device__ __forceinline__ float load_as_f32(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__global__ void __launch_bounds__(256) gemm_general_kernel(const Params p) {
  __shared__ float s_a[KSTEP][TILE + 1];  // [k][m]
  __shared__ float s_b[KSTEP][TILE + 1];  // [k][n]
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // outputs rows ty * 4 .., columns tx * 4 ..
  const int m0 = blockIdx.y * TILE, n0 = blockIdx.x * TILE;
  const long long batch = blockIdx.z;
  const T* a = static_cast<const T*>(p.a) + batch * p.a_batch;
  const T* b = static_cast<const T*>(p.b) + batch * p.b_batch;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < p.K; k0 += KSTEP) {
    // 64 x 16 elements of each operand, four per thread; a warp walks the operand's rows (A) or
    // columns (B), whichever index the tile's 64 runs over, so that contiguous operands coalesce
    // in at least one of their two layouts.
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      const int kk = e >> 6, mn = e & 63;
      const int k = k0 + kk;
      const int m = m0 + mn, n = n0 + mn;
      s_a[kk][mn] = (k < p.K && m < p.M) ? load_as_f32(a + m * p.a_row + k * p.a_col) : 0.f;
      s_b[kk][mn] = (k < p.K && n < p.N) ? load_as_f32(b + k * p.b_row + n * p.b_col) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < KSTEP; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        av[i] = s_a[kk][ty * 4 + i];
        bv[i] = s_b[kk][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      float v = p.alpha * acc[i][j];
      if (p.c != nullptr) {
        const long long ci = batch * p.c_batch + m * p.c_row + n;
        v += p.beta * (p.c_f32 ? static_cast<const float*>(p.c)[ci]
                               : __bfloat162float(static_cast<const __nv_bfloat16*>(p.c)[ci]));
      }
      const long long di = batch * p.d_batch + m * p.d_row + n;
      if (p.d_f32) static_cast<float*>(p.d)[di] = v;
      else static_cast<__nv_bfloat16*>(p.d)[di] = __float2bfloat16_rn(v);
    }
  }
}

}  // namespace gemm_general

// Operands as validated by matmul_execute_epi (ranks, shapes, dtypes of one kind, contiguous last
// dimension of C and D); nothing here depends on alignment.
int32_t matmul_general_execute(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* c,
                               const cdl_tensor* d, float alpha, float beta, cudaStream_t stream) {
  using namespace gemm_general;
  const int r = a->rank;
  const long long batch = r == 3 ? a->shape[0] : 1;
  Params p{};
  p.a = a->ptr;
  p.b = b->ptr;
  p.d = d->ptr;
  p.M = static_cast<int>(a->shape[r - 2]);
  p.K = static_cast<int>(a->shape[r - 1]);
  p.N = static_cast<int>(b->shape[r - 1]);
  p.a_batch = r == 3 ? a->stride[0] : 0;
  p.a_row = a->stride[r - 2];
  p.a_col = a->stride[r - 1];
  p.b_batch = r == 3 ? b->stride[0] : 0;
  p.b_row = b->stride[r - 2];
  p.b_col = b->stride[r - 1];
  p.d_batch = r == 3 ? d->stride[0] : 0;
  p.d_row = d->stride[r - 2];
  p.d_f32 = d->dtype == CDL_F32 ? 1 : 0;
  if (c != nullptr && beta != 0.0f) {
    p.c = c->ptr;
    p.c_batch = r == 3 ? c->stride[0] : 0;
    p.c_row = c->stride[r - 2];
    p.c_f32 = c->dtype == CDL_F32 ? 1 : 0;
  }
  p.alpha = alpha;
  p.beta = beta;
  const dim3 grid(static_cast<unsigned>((p.N + TILE - 1) / TILE),
                  static_cast<unsigned>((p.M + TILE - 1) / TILE), static_cast<unsigned>(batch));
  if (grid.y > 65535)
    return fail(CDL_ERR_UNSUPPORTED, "matmul (general path): more than %d rows", 65535 * TILE);
  ProfileScope ps(PROF_GEMM, 2.0 * batch * p.M * p.N * p.K, stream);
  if (a->dtype == CDL_F32) gemm_general_kernel<float><<<grid, 256, 0, stream>>>(p);
  else gemm_general_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

}  // namespace cdl
