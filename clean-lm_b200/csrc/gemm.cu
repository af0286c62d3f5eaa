// BF16 GEMM  D = alpha * A . B + beta * C  on the 5th-generation tensor cores (tcgen05).
//
// Operator semantics follow Matmul / MatmulExecutor of the reference
// (crates/cleandl/src/execgraph/ops/matmul.rs:61-68, 1092-1183), which hands the problem to
// cuBLASLt; the kernel itself is written for sm_100a from scratch.  (The reference's own, disabled,
// tcgen05 kernel is crates/cleandl/rust-kernels/src/sky_matmul/tcgen05_bf16.rs.)
//
// Kernel structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: loads a 128 x 64 A tile and a 256 x 64 B tile per stage into
//               128-byte-swizzled shared memory (4-stage ring, 48 KiB per stage).
//   warp 1      MMA issuer: one elected thread issues 4 tcgen05.mma (M128 N256 K16) per stage into
//               one of two 256-column f32 accumulators in TMEM; tcgen05.commit releases the stage
//               and, after the last K block, publishes the accumulator.
//   warps 2-5   epilogue: tcgen05.ld the accumulator (one row per thread, 32 columns at a time),
//               apply alpha / beta*C, convert and store straight to global memory.  The second
//               accumulator lets the epilogue of tile i overlap the main loop of tile i+1.
// Both operands may be K-major (K contiguous) or MN-major (M or N contiguous); that covers
// forward (A row-major, B row-major), dgrad (B transposed view) and wgrad (A transposed view)
// without copies.  M/N/K tails rely on TMA zero fill for loads and on predicated stores.
#include "host.h"
#include "ptx.cuh"

#include <mutex>

namespace cdl {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int RASTER_W = 8;  // N tiles per raster panel
constexpr size_t SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 256;

struct Params {
  int M, N, K, batch;
  int num_m_tiles, num_n_tiles, num_tiles, k_blocks;
  int a_mn, b_mn;      // 1 = operand is MN-major (M or N contiguous)
  int out_f32, c_mode; // c_mode: 0 none, 1 bf16, 2 f32
  void* d;
  const void* c;
  long long ldd, ldc, d_batch, c_batch;  // in elements
  int d_vec, c_vec;                      // 1 = rows are 16-byte aligned, vector access allowed
  float alpha, beta;
  int* status;
};

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_word;
};

__device__ __forceinline__ void tile_coords(const Params& p, int tile, int& b, int& m, int& n) {
  const int per_batch = p.num_m_tiles * p.num_n_tiles;
  b = tile / per_batch;
  int r = tile - b * per_batch;
  const int panel_tiles = RASTER_W * p.num_m_tiles;
  const int panel = r / panel_tiles;
  const int first_n = panel * RASTER_W;
  const int width = min(RASTER_W, p.num_n_tiles - first_n);
  r -= panel * panel_tiles;
  m = r / width;
  n = first_n + (r - m * width);
}

__global__ void __launch_bounds__(THREADS, 1)
    gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a,
                     const __grid_constant__ CUtensorMap tmap_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(smem + STAGES * STAGE_BYTES);
  volatile int* abort_word = &bars->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->acc_full[i], 1);
      mbar_init(&bars->acc_empty[i], 4);
    }
    bars->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
        int b, tm, tn;
        tile_coords(p, tile, b, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_word, 101)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_arrive_expect_tx(&bars->full[s], STAGE_BYTES);
          const int k0 = kb * BK;
          if (p.a_mn) {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_3d(sa + i * 8192, &tmap_a, &bars->full[s], m0 + i * 64, k0, b);
          } else {
            tma_load_3d(sa, &tmap_a, &bars->full[s], k0, m0, b);
          }
          if (p.b_mn) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_3d(sb + i * 8192, &tmap_b, &bars->full[s], n0 + i * 64, k0, b);
          } else {
            tma_load_3d(sb, &tmap_b, &bars->full[s], k0, n0, b);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, p.a_mn, p.b_mn);
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
      const uint32_t a_kstep = p.a_mn ? 2048u : 32u, b_kstep = p.b_mn ? 2048u : 32u;
      uint32_t it = 0;
      int t = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++t) {
        const int acc = t & 1;
        const uint32_t acc_ph = (t >> 1) & 1;
        if (!mbar_wait(&bars->acc_empty[acc], acc_ph ^ 1, abort_word, 201)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars->full[s], ph, abort_word, 202)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = smem_desc_sw128(sa + k * a_kstep, a_lbo, 1024);
            const uint64_t db = smem_desc_sw128(sb + k * b_kstep, b_lbo, 1024);
            umma_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&bars->empty[s]);
        }
        if (ok) umma_commit(&bars->acc_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    int t = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++t) {
      int b, tm, tn;
      tile_coords(p, tile, b, tm, tn);
      const int acc = t & 1;
      const uint32_t acc_ph = (t >> 1) & 1;
      if (!mbar_wait(&bars->acc_full[acc], acc_ph, abort_word, 301)) break;
      tc_fence_after();
      const int row = tm * BM + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        const int col0 = tn * BN + ch * 32;
        if (col0 >= p.N) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld32(t_row + ch * 32, r);
        tmem_wait_ld();
        if (row_ok) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = p.alpha * __uint_as_float(r[j]);
          if (p.c_mode == 1) {
            const __nv_bfloat16* cp = static_cast<const __nv_bfloat16*>(p.c) +
                                      b * p.c_batch + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (p.c_vec && col0 + g * 8 + 8 <= p.N) {
                const uint4 q = *reinterpret_cast<const uint4*>(cp + g * 8);
                const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  v[g * 8 + 2 * j] += p.beta * bf16_lo(w[j]);
                  v[g * 8 + 2 * j + 1] += p.beta * bf16_hi(w[j]);
                }
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (col0 + g * 8 + j < p.N)
                    v[g * 8 + j] += p.beta * __bfloat162float(cp[g * 8 + j]);
              }
            }
          } else if (p.c_mode == 2) {
            const float* cp = static_cast<const float*>(p.c) + b * p.c_batch +
                              static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              if (p.c_vec && col0 + g * 4 + 4 <= p.N) {
                const float4 q = *reinterpret_cast<const float4*>(cp + g * 4);
                v[g * 4 + 0] += p.beta * q.x;
                v[g * 4 + 1] += p.beta * q.y;
                v[g * 4 + 2] += p.beta * q.z;
                v[g * 4 + 3] += p.beta * q.w;
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  if (col0 + g * 4 + j < p.N) v[g * 4 + j] += p.beta * cp[g * 4 + j];
              }
            }
          }
          if (p.out_f32) {
            float* dp = static_cast<float*>(p.d) + b * p.d_batch +
                        static_cast<long long>(row) * p.ldd + col0;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              if (p.d_vec && col0 + g * 4 + 4 <= p.N) {
                *reinterpret_cast<float4*>(dp + g * 4) =
                    make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  if (col0 + g * 4 + j < p.N) dp[g * 4 + j] = v[g * 4 + j];
              }
            }
          } else {
            __nv_bfloat16* dp = static_cast<__nv_bfloat16*>(p.d) + b * p.d_batch +
                                static_cast<long long>(row) * p.ldd + col0;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (p.d_vec && col0 + g * 8 + 8 <= p.N) {
                uint4 q;
                q.x = pack_bf16x2(v[g * 8 + 0], v[g * 8 + 1]);
                q.y = pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]);
                q.z = pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]);
                q.w = pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]);
                *reinterpret_cast<uint4*>(dp + g * 8) = q;
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (col0 + g * 8 + j < p.N) dp[g * 8 + j] = __float2bfloat16_rn(v[g * 8 + j]);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
    }
  }

  // ------------------------------------------------------------ tear-down
  __syncwarp();
  if (*abort_word != 0) {
    // Give loads that may still be in flight time to land before shared memory is released.
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_word != 0) atomicExch(p.status, *abort_word);
}

// Splits a [rows, cols] (or batched) bf16 view into major-ness and leading dimension.
struct OperandLayout {
  int mn_major;     // 1 when the non-contraction dimension is the contiguous one
  long long ld;     // stride of the other dimension, elements
  long long batch;  // batch stride, elements
};

static int32_t analyze_operand(const char* name, const cdl_tensor* t, bool contraction_is_last,
                               OperandLayout* out) {
  const int r = t->rank;
  const long long rows = t->shape[r - 2], cols = t->shape[r - 1];
  const long long s_row = t->stride[r - 2], s_col = t->stride[r - 1];
  const bool aligned_base = (reinterpret_cast<uintptr_t>(t->ptr) & 15) == 0;
  out->batch = r == 3 ? t->stride[0] : 0;
  const bool batch_ok = r != 3 || t->shape[0] <= 1 || (out->batch % 8 == 0 && out->batch > 0);
  // A dimension of extent 1 has no meaningful stride, so either reading may apply; take the
  // first one whose leading dimension TMA can describe.
  const bool last_contig = s_col == 1 || cols == 1;
  const bool first_contig = s_row == 1 || rows == 1;
  if (!last_contig && !first_contig)
    return fail(CDL_ERR_INVALID,
                "matmul operand %s must have a contiguous dimension (strides [%lld, %lld])", name,
                s_row, s_col);
  auto round8 = [](long long v) { return (v + 7) / 8 * 8; };
  const long long ld_last = rows == 1 ? round8(cols) : s_row;   // rows are ld_last apart
  const long long ld_first = cols == 1 ? round8(rows) : s_col;  // columns are ld_first apart
  const bool last_ok = last_contig && ld_last % 8 == 0 && ld_last >= cols;
  const bool first_ok = first_contig && ld_first % 8 == 0 && ld_first >= rows;
  if (!aligned_base || !batch_ok || (!last_ok && !first_ok))
    return fail(CDL_ERR_UNSUPPORTED,
                "matmul operand %s: TMA needs a 16-byte aligned base, leading dimension and batch "
                "stride (ptr %p, strides [%lld, %lld] elements, batch stride %lld)",
                name, t->ptr, s_row, s_col, out->batch);
  const bool use_last = last_ok;
  out->ld = use_last ? ld_last : ld_first;
  // contraction_is_last: the operand is A [M, K]; otherwise it is B [K, N].
  const bool k_contig = contraction_is_last ? use_last : !use_last;
  out->mn_major = k_contig ? 0 : 1;
  return CDL_OK;
}

}  // namespace gemm

int32_t matmul_execute(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* c,
                       const cdl_tensor* d, float alpha, float beta, cudaStream_t stream) {
  using namespace gemm;
  if (!a || !b || !d) return fail(CDL_ERR_INVALID, "matmul: a, b and d are required");
  if (a->rank != b->rank || (a->rank != 2 && a->rank != 3) || d->rank != a->rank)
    return fail(CDL_ERR_INVALID,
                "matmul operands must all have rank 2 or all rank 3 (got rank %d, %d, %d)",
                a->rank, b->rank, d->rank);
  if (a->dtype != CDL_BF16 || b->dtype != CDL_BF16)
    return fail(a->dtype == CDL_F32 && b->dtype == CDL_F32 ? CDL_ERR_UNSUPPORTED : CDL_ERR_INVALID,
                "matmul inputs must be f32 or bf16 and of one type; this library implements bf16 "
                "(got %s x %s)",
                dtype_name(a->dtype), dtype_name(b->dtype));
  if (d->dtype != CDL_BF16 && d->dtype != CDL_F32)
    return fail(CDL_ERR_INVALID, "matmul output must be f32 or bf16");
  const int r = a->rank;
  const long long batch = r == 3 ? a->shape[0] : 1;
  const long long M = a->shape[r - 2], K = a->shape[r - 1], N = b->shape[r - 1];
  if (b->shape[r - 2] != K)
    return fail(CDL_ERR_INVALID, "matmul contraction dimensions differ: a is [.., %lld, %lld], b is [.., %lld, %lld]",
                M, K, (long long)b->shape[r - 2], N);
  if (r == 3 && (b->shape[0] != batch || d->shape[0] != batch))
    return fail(CDL_ERR_INVALID, "matmul batch dimensions differ");
  if (d->shape[r - 2] != M || d->shape[r - 1] != N)
    return fail(CDL_ERR_INVALID, "matmul output shape must be [%lld, %lld]", M, N);
  if (d->stride[r - 1] != 1 && N > 1)
    return fail(CDL_ERR_INVALID, "matmul output must be row-major with a contiguous last dimension");
  const bool use_c = c != nullptr && beta != 0.0f;
  if (use_c) {
    if (c->rank != r || c->shape[r - 2] != M || c->shape[r - 1] != N ||
        (r == 3 && c->shape[0] != batch))
      return fail(CDL_ERR_INVALID, "matmul c must have the output's shape");
    if (c->dtype != CDL_BF16 && c->dtype != CDL_F32)
      return fail(CDL_ERR_INVALID, "matmul c must be f32 or bf16");
    if (c->stride[r - 1] != 1 && N > 1)
      return fail(CDL_ERR_INVALID, "matmul c must have a contiguous last dimension");
  }
  if (batch == 0 || M == 0 || N == 0) return CDL_OK;  // empty output: nothing to do
  if (K == 0) return fail(CDL_ERR_INVALID, "matmul: K is zero");
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX || batch > 65535)
    return fail(CDL_ERR_UNSUPPORTED, "matmul dimension too large");

  OperandLayout la, lb;
  CDL_CHECK(analyze_operand("a", a, true, &la));
  CDL_CHECK(analyze_operand("b", b, false, &lb));

  CUtensorMap tm_a, tm_b;
  {
    // Innermost-first dims: K-major operand = [K, M|N, batch]; MN-major = [M|N, K, batch].
    const uint64_t bs_a = static_cast<uint64_t>(batch > 1 ? la.batch : la.ld * (la.mn_major ? K : M)) * 2;
    const uint64_t bs_b = static_cast<uint64_t>(batch > 1 ? lb.batch : lb.ld * (lb.mn_major ? K : N)) * 2;
    uint64_t da[3], sa[3], db[3], sb[3];
    uint32_t ba[3], bb[3];
    if (la.mn_major) {
      da[0] = M; da[1] = K; ba[0] = 64; ba[1] = 64;
    } else {
      da[0] = K; da[1] = M; ba[0] = 64; ba[1] = BM;
    }
    da[2] = batch; ba[2] = 1; sa[0] = 0; sa[1] = la.ld * 2; sa[2] = bs_a;
    if (lb.mn_major) {
      db[0] = N; db[1] = K; bb[0] = 64; bb[1] = 64;
    } else {
      db[0] = K; db[1] = N; bb[0] = 64; bb[1] = BN;
    }
    db[2] = batch; bb[2] = 1; sb[0] = 0; sb[1] = lb.ld * 2; sb[2] = bs_b;
    CDL_CHECK(encode_tmap(&tm_a, a->ptr, CDL_BF16, 3, da, sa, ba, true));
    CDL_CHECK(encode_tmap(&tm_b, b->ptr, CDL_BF16, 3, db, sb, bb, true));
  }

  Params p;
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.batch = static_cast<int>(batch);
  p.num_m_tiles = static_cast<int>((M + BM - 1) / BM);
  p.num_n_tiles = static_cast<int>((N + BN - 1) / BN);
  const long long tiles = batch * p.num_m_tiles * p.num_n_tiles;
  if (tiles > INT32_MAX) return fail(CDL_ERR_UNSUPPORTED, "matmul: too many tiles");
  p.num_tiles = static_cast<int>(tiles);
  p.k_blocks = static_cast<int>((K + BK - 1) / BK);
  p.a_mn = la.mn_major;
  p.b_mn = lb.mn_major;
  p.out_f32 = d->dtype == CDL_F32;
  p.c_mode = !use_c ? 0 : (c->dtype == CDL_BF16 ? 1 : 2);
  p.d = d->ptr;
  p.c = use_c ? c->ptr : nullptr;
  p.ldd = M > 1 ? d->stride[r - 2] : N;
  p.ldc = use_c ? (M > 1 ? c->stride[r - 2] : N) : 0;
  p.d_batch = r == 3 ? d->stride[0] : 0;
  p.c_batch = use_c && r == 3 ? c->stride[0] : 0;
  auto vec_ok = [](const void* ptr, long long ld, long long bstride, size_t es) {
    return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && (ld * es) % 16 == 0 &&
           (bstride * es) % 16 == 0;
  };
  p.d_vec = vec_ok(p.d, p.ldd, p.d_batch, dtype_size(d->dtype));
  p.c_vec = use_c ? vec_ok(p.c, p.ldc, p.c_batch, dtype_size(c->dtype)) : 0;
  p.alpha = alpha;
  p.beta = use_c ? beta : 0.0f;
  p.status = device_status_ptr();
  if (!p.status) return fail(CDL_ERR_CUDA, "cannot resolve the device status word");

  static std::once_flag attr_once[64];
  int dev = 0;
  CDL_CUDA(cudaGetDevice(&dev));
  cudaError_t attr_err = cudaSuccess;
  std::call_once(attr_once[dev & 63], [&] {
    attr_err = cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(SMEM_BYTES));
  });
  if (attr_err != cudaSuccess)
    return fail(CDL_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(attr_err));

  const int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  ProfileScope ps(PROF_GEMM, 2.0 * static_cast<double>(batch) * M * N * K, stream);
  gemm_bf16_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(tm_a, tm_b, p);
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

}  // namespace cdl

extern "C" {

int32_t cdl_b200_matmul(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* c,
                        const cdl_tensor* d, float alpha, float beta, void* scratch,
                        size_t scratch_bytes, cdl_stream stream) {
  (void)scratch;
  (void)scratch_bytes;
  return cdl::matmul_execute(a, b, c, d, alpha, beta, static_cast<cudaStream_t>(stream));
}

int32_t cdl_b200_matmul_scratch_bytes(const cdl_tensor* a, const cdl_tensor* b,
                                      const cdl_tensor* d, size_t* bytes_out) {
  (void)a;
  (void)b;
  (void)d;
  if (bytes_out) *bytes_out = 0;
  return CDL_OK;
}

}  // extern "C"
