// BF16 GEMM  D = alpha * A . B + beta * C  on the 5th-generation tensor cores (tcgen05).
//
// Operator semantics follow Matmul / MatmulExecutor of the reference
// (crates/cleandl/src/execgraph/ops/matmul.rs:61-68, 1092-1183), which hands the problem to
// cuBLASLt; the kernel itself is written for sm_100a from scratch.  (The reference's own, disabled,
// tcgen05 kernel is crates/cleandl/rust-kernels/src/sky_matmul/tcgen05_bf16.rs.)
//
// Kernel structure (one persistent CTA per SM, 320 threads):
//   warp 0      TMA producer: loads a 128 x 64 A tile and a 256 x 64 B tile per stage into
//               128-byte-swizzled shared memory (4-stage ring, 48 KiB per stage).
//   warp 1      MMA issuer: one elected thread issues 4 tcgen05.mma (M128 N256 K16) per stage into
//               one of two 256-column f32 accumulators in TMEM; tcgen05.commit releases the stage
//               and, after the last K block, publishes the accumulator.
//   warps 2-9   epilogue: tcgen05.ld the accumulator (one row per thread, 32 columns at a time),
//               apply alpha / beta*C, convert and store straight to global memory.  The second
//               accumulator lets the epilogue of tile i overlap the main loop of tile i+1.
// Both operands may be K-major (K contiguous) or MN-major (M or N contiguous); that covers
// forward (A row-major, B row-major), dgrad (B transposed view) and wgrad (A transposed view)
// without copies.  M/N/K tails rely on TMA zero fill for loads and on predicated stores.
#include "host.h"
#include "ops.h"
#include "ptx.cuh"

#include <stdlib.h>
#include <string.h>

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
constexpr int THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue (two per TMEM lane quadrant)
constexpr int EPI_WARPS = 8;
constexpr int TMEM_COLS = 512;
constexpr int RASTER_W = 8;  // N tiles per raster panel (upper bound; see Params::raster_w)
// L2 budget for A plus one raster panel of B (see the raster_w computation on the host).
#ifndef CDL_GEMM_RASTER_BUDGET_MB
#define CDL_GEMM_RASTER_BUDGET_MB 96
#endif
constexpr size_t SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 256;

struct Params {
  int M, N, K, batch;
  int num_m_tiles, num_n_tiles, num_tiles, k_blocks;
  int raster_w;        // N tiles per raster panel, 1 .. RASTER_W
  int a_mn, b_mn;      // 1 = operand is MN-major (M or N contiguous)
  int out_f32, c_mode; // c_mode: 0 none, 1 bf16, 2 f32
  void* d;
  const void* c;
  long long ldd, ldc, d_batch, c_batch;  // in elements
  int d_vec, c_vec;                      // 1 = rows are 16-byte aligned, vector access allowed
  float alpha, beta;
  int split_k;     // K slices per tile (pair kernel, accumulate-in-place form only); 1 = none
  int atomic_out;  // 1 = add alpha * partial into D with red.global.add (D already holds C)
  // Fused SwiGLU epilogues (bf16 [M, N] operands, 16-byte aligned rows):
  //   1: D = G (the product),           out2 = SiLU(G) * aux0           (aux0 = up projection)
  //   2: D = SiLU(aux0) * R,            out2 = R * aux1 * dSiLU(aux0)   (R = product, aux0 = gate, aux1 = up)
  int wide;  // 1 = D, C and the fused operands all have 32-byte aligned rows: 256-bit accesses
  int epi_mode;
  const __nv_bfloat16* aux0;
  const __nv_bfloat16* aux1;
  __nv_bfloat16* out2;
  long long ld_aux0, ld_aux1, ld_out2;
  // Epilogue mode 3, rotate-half RoPE on the heads (128 columns each) below rope_cols:
  //   d[r, h 128 + i]      = x[i] cos(pos, i) - x[i + 64] sin(pos, i)
  //   d[r, h 128 + i + 64] = x[i + 64] cos(pos, i) + x[i] sin(pos, i)        (i < 64)
  // with x the product's row, pos = r % rope_seqlen, or r - cu_seqlens[b] for the sequence b that
  // holds row r of a ragged batch; the table is f32 [positions, 128] = cos | sin.
  const float* rope_table;
  const int* rope_cu;  // cu_seqlens of a ragged batch (device), or nullptr
  int rope_seqlen, rope_cols, rope_nseq;
  // Pair kernel: counter of the work units handed out beyond every cluster's first one (zero
  // between launches; one counter per device and stream).
  unsigned int* sched_counter;
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
  const int panel_tiles = p.raster_w * p.num_m_tiles;
  const int panel = r / panel_tiles;
  const int first_n = panel * p.raster_w;
  const int width = min(p.raster_w, p.num_n_tiles - first_n);
  r -= panel * panel_tiles;
  m = r / width;
  n = first_n + (r - m * width);
}

// sigmoid(x) = 0.5 + 0.5 tanh(x / 2): one MUFU operation per element (tanh.approx, relative error
// about 2^-11, below the bf16 rounding of the outputs).  The reference's fused epilogues use
// rcp.approx(1 + ex2.approx(-x log2 e)) (crates/cleandl/rust-kernels/src/sky_matmul/
// tcgen05_bf16.rs:851-854), two MUFU operations; at 16 per clock per SM the 65536 elements of a
// 256 x 256 tile then cost half the time of the tile's main loop, and the epilogue warps, not the
// tensor pipe, set the pace of the fused GEMMs.
__device__ __forceinline__ float fast_sigmoid(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(0.5f, t, 0.5f);
}

// 32 consecutive columns of one output row, all operands 32-byte aligned: C read, fused
// SwiGLU or plain conversion, 256-bit stores.
__device__ __forceinline__ void store_chunk_wide(const Params& p, float (&v)[32], int b, int row,
                                                 int col0) {
  const long long r64 = row;
  if (p.c_mode == 1) {
    const __nv_bfloat16* cp = static_cast<const __nv_bfloat16*>(p.c) + b * p.c_batch + r64 * p.ldc + col0;
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      uint32_t w[8];
      ld_global_v8(cp + g * 16, w);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[g * 16 + 2 * j] += p.beta * bf16_lo(w[j]);
        v[g * 16 + 2 * j + 1] += p.beta * bf16_hi(w[j]);
      }
    }
  } else if (p.c_mode == 2) {
    const float* cp = static_cast<const float*>(p.c) + b * p.c_batch + r64 * p.ldc + col0;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint32_t w[8];
      ld_global_v8(cp + g * 8, w);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[g * 8 + j] += p.beta * __uint_as_float(w[j]);
    }
  }
  if (p.epi_mode != 0) {
    __nv_bfloat16* dp = static_cast<__nv_bfloat16*>(p.d) + r64 * p.ldd + col0;
    __nv_bfloat16* op = p.out2 + r64 * p.ld_out2 + col0;
    const __nv_bfloat16* a0 = p.aux0 + r64 * p.ld_aux0 + col0;
    const __nv_bfloat16* a1 = p.aux1 + r64 * p.ld_aux1 + col0;  // only dereferenced in mode 2
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      uint32_t w0[8], w1[8], q1[8], q2[8];
      ld_global_v8(a0 + g * 16, w0);
      if (p.epi_mode == 2) ld_global_v8(a1 + g * 16, w1);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float o1[2], o2[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float rr = v[g * 16 + 2 * j + e];
          const float x0 = e ? bf16_hi(w0[j]) : bf16_lo(w0[j]);
          if (p.epi_mode == 1) {
            o1[e] = rr;
            o2[e] = rr * fast_sigmoid(rr) * x0;
          } else {
            const float x1 = e ? bf16_hi(w1[j]) : bf16_lo(w1[j]);
            const float sg = fast_sigmoid(x0);
            o1[e] = x0 * sg * rr;
            o2[e] = rr * x1 * (sg + x0 * sg * (1.0f - sg));
          }
        }
        q1[j] = pack_bf16x2(o1[0], o1[1]);
        q2[j] = pack_bf16x2(o2[0], o2[1]);
      }
      st_global_v8(dp + g * 16, q1);
      st_global_v8(op + g * 16, q2);
    }
  } else if (p.out_f32) {
    float* dp = static_cast<float*>(p.d) + b * p.d_batch + r64 * p.ldd + col0;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] = __float_as_uint(v[g * 8 + j]);
      st_global_v8(dp + g * 8, w);
    }
  } else {
    __nv_bfloat16* dp = static_cast<__nv_bfloat16*>(p.d) + b * p.d_batch + r64 * p.ldd + col0;
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] = pack_bf16x2(v[g * 16 + 2 * j], v[g * 16 + 2 * j + 1]);
      st_global_v8(dp + g * 16, w);
    }
  }
}

// Epilogue of one accumulator for the calling warp: thread `lane` owns output row `row`
// (TMEM lane = its lane inside the warp's quadrant); t_row addresses column 0 of the accumulator
// at the warp's first lane.  Applies alpha / beta * C, converts and stores 128 columns (the warp's half of the tile).
__device__ __forceinline__ void store_tile_rows(const Params& p, uint32_t t_row, int b, int row,
                                                int col_base) {
  const bool row_ok = row < p.M;
#pragma unroll 1
  for (int ch = 0; ch < BN / 64; ++ch) {
    const int col0 = col_base + ch * 32;
    if (col0 >= p.N) break;  // warp-uniform
    uint32_t r[32];
    tmem_ld32(t_row + ch * 32, r);
    tmem_wait_ld();
    if (row_ok) {
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = p.alpha * __uint_as_float(r[j]);
      if (p.wide && !p.atomic_out && col0 + 32 <= p.N) {
        // Fast path: every row involved is 32-byte aligned, so each thread moves whole 32-byte
        // sectors with 256-bit accesses (a thread owns a row, so narrower accesses would touch
        // every sector twice).
        store_chunk_wide(p, v, b, row, col0);
        continue;
      }
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
      if (p.epi_mode != 0) {
        // sigmoid via ex2 / rcp approximations, as in the reference's fused epilogues
        // (crates/cleandl/rust-kernels/src/sky_matmul/tcgen05_bf16.rs:851-877).
        __nv_bfloat16* dp = static_cast<__nv_bfloat16*>(p.d) + static_cast<long long>(row) * p.ldd + col0;
        __nv_bfloat16* op = p.out2 + static_cast<long long>(row) * p.ld_out2 + col0;
        const __nv_bfloat16* a0 = p.aux0 + static_cast<long long>(row) * p.ld_aux0 + col0;
        const __nv_bfloat16* a1 = p.epi_mode == 2 ? p.aux1 + static_cast<long long>(row) * p.ld_aux1 + col0 : nullptr;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          if (col0 + g * 8 + 8 <= p.N) {  // N % 8 == 0 is checked on the host
            const uint4 q0 = *reinterpret_cast<const uint4*>(a0 + g * 8);
            const uint32_t w0[4] = {q0.x, q0.y, q0.z, q0.w};
            uint32_t w1[4] = {0, 0, 0, 0};
            if (p.epi_mode == 2) {
              const uint4 q1 = *reinterpret_cast<const uint4*>(a1 + g * 8);
              w1[0] = q1.x; w1[1] = q1.y; w1[2] = q1.z; w1[3] = q1.w;
            }
            float o1[8], o2[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float r = v[g * 8 + j];
              const float x0 = (j & 1) ? bf16_hi(w0[j >> 1]) : bf16_lo(w0[j >> 1]);
              if (p.epi_mode == 1) {
                const float sg = fast_sigmoid(r);
                o1[j] = r;
                o2[j] = r * sg * x0;
              } else {
                const float x1 = (j & 1) ? bf16_hi(w1[j >> 1]) : bf16_lo(w1[j >> 1]);
                const float sg = fast_sigmoid(x0);
                o1[j] = x0 * sg * r;
                o2[j] = r * x1 * (sg + x0 * sg * (1.0f - sg));
              }
            }
            uint4 qa, qb;
            qa.x = pack_bf16x2(o1[0], o1[1]); qa.y = pack_bf16x2(o1[2], o1[3]);
            qa.z = pack_bf16x2(o1[4], o1[5]); qa.w = pack_bf16x2(o1[6], o1[7]);
            qb.x = pack_bf16x2(o2[0], o2[1]); qb.y = pack_bf16x2(o2[2], o2[3]);
            qb.z = pack_bf16x2(o2[4], o2[5]); qb.w = pack_bf16x2(o2[6], o2[7]);
            *reinterpret_cast<uint4*>(dp + g * 8) = qa;
            *reinterpret_cast<uint4*>(op + g * 8) = qb;
          }
        }
      } else if (p.atomic_out) {
        // K-sliced accumulation: D (f32, already holding C) += alpha * partial.  Several slices
        // of a tile add concurrently, so the order of the f32 additions is not fixed.
        float* dp = static_cast<float*>(p.d) + b * p.d_batch +
                    static_cast<long long>(row) * p.ldd + col0;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          if (p.d_vec && col0 + g * 4 + 4 <= p.N) {
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dp + g * 4),
                         "f"(v[g * 4]), "f"(v[g * 4 + 1]), "f"(v[g * 4 + 2]), "f"(v[g * 4 + 3])
                         : "memory");
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (col0 + g * 4 + j < p.N) atomicAdd(dp + g * 4 + j, v[g * 4 + j]);
          }
        }
      } else if (p.out_f32) {
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
}

// Epilogue of mode 3 for the calling warp: its 128 columns are one head.  The rotation pairs column
// i with column i + 64, so the 32-column chunks are drained in pairs (0, 2) and (1, 3); heads at or
// beyond rope_cols (the value heads of a fused qkv projection) are stored unrotated.
__device__ __forceinline__ void store_tile_rows_rope(const Params& p, uint32_t t_row, int row,
                                                     int col_base) {
  if (col_base >= p.N) return;  // warp-uniform
  const bool row_ok = row < p.M;
  const bool rotate = col_base < p.rope_cols;  // warp-uniform
  int pos = 0;
  if (row_ok && rotate) {
    if (p.rope_cu != nullptr) {
      // ragged batch: the position restarts at every sequence; rows after the last sequence keep
      // position 0 (they are padding)
      int lo_i = 0, hi_i = p.rope_nseq;  // largest b with cu[b] <= row
      while (hi_i - lo_i > 1) {
        const int mid = (lo_i + hi_i) >> 1;
        if (p.rope_cu[mid] <= row) lo_i = mid;
        else hi_i = mid;
      }
      pos = row < p.rope_cu[p.rope_nseq] ? min(row - p.rope_cu[lo_i], p.rope_seqlen - 1) : 0;
    } else {
      pos = row % p.rope_seqlen;
    }
  }
  const float* cs = p.rope_table + static_cast<long long>(pos) * 128;
  __nv_bfloat16* dp = static_cast<__nv_bfloat16*>(p.d) + static_cast<long long>(row) * p.ldd + col_base;
#pragma unroll 1
  for (int pr = 0; pr < 2; ++pr) {
    uint32_t lo[32], hi[32];
    tmem_ld32(t_row + pr * 32, lo);
    tmem_ld32(t_row + (pr + 2) * 32, hi);
    tmem_wait_ld();
    if (!row_ok) continue;
    uint32_t olo[16], ohi[16];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float c[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
      if (rotate) {
        const float4 cv = __ldg(reinterpret_cast<const float4*>(cs + pr * 32 + g * 4));
        const float4 sv = __ldg(reinterpret_cast<const float4*>(cs + 64 + pr * 32 + g * 4));
        c[0] = cv.x; c[1] = cv.y; c[2] = cv.z; c[3] = cv.w;
        sn[0] = sv.x; sn[1] = sv.y; sn[2] = sv.z; sn[3] = sv.w;
      }
      float rl[4], rh[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float l = p.alpha * __uint_as_float(lo[g * 4 + e]), h = p.alpha * __uint_as_float(hi[g * 4 + e]);
        rl[e] = l * c[e] - h * sn[e];
        rh[e] = h * c[e] + l * sn[e];
      }
      olo[g * 2] = pack_bf16x2(rl[0], rl[1]);
      olo[g * 2 + 1] = pack_bf16x2(rl[2], rl[3]);
      ohi[g * 2] = pack_bf16x2(rh[0], rh[1]);
      ohi[g * 2 + 1] = pack_bf16x2(rh[2], rh[3]);
    }
    if (p.wide) {  // whole 32-byte sectors per access, as in store_chunk_wide
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const uint32_t wl[8] = {olo[g * 8], olo[g * 8 + 1], olo[g * 8 + 2], olo[g * 8 + 3],
                                olo[g * 8 + 4], olo[g * 8 + 5], olo[g * 8 + 6], olo[g * 8 + 7]};
        const uint32_t wh[8] = {ohi[g * 8], ohi[g * 8 + 1], ohi[g * 8 + 2], ohi[g * 8 + 3],
                                ohi[g * 8 + 4], ohi[g * 8 + 5], ohi[g * 8 + 6], ohi[g * 8 + 7]};
        st_global_v8(dp + pr * 32 + g * 16, wl);
        st_global_v8(dp + (pr + 2) * 32 + g * 16, wh);
      }
    } else {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        *reinterpret_cast<uint4*>(dp + pr * 32 + g * 8) =
            make_uint4(olo[g * 4], olo[g * 4 + 1], olo[g * 4 + 2], olo[g * 4 + 3]);
        *reinterpret_cast<uint4*>(dp + (pr + 2) * 32 + g * 8) =
            make_uint4(ohi[g * 4], ohi[g * 4 + 1], ohi[g * 4 + 2], ohi[g * 4 + 3]);
      }
    }
  }
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
      mbar_init(&bars->acc_empty[i], EPI_WARPS);
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
  // Everything above overlaps the tail of the previous kernel of the stream; operands are read
  // (and outputs written) only from here on.
  grid_dep_wait();
  grid_dep_launch();

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
    // ------------------------------------------------------------ epilogue (warps 2..9)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;  // which 128 of the tile's 256 columns
    int t = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++t) {
      int b, tm, tn;
      tile_coords(p, tile, b, tm, tn);
      const int acc = t & 1;
      const uint32_t acc_ph = (t >> 1) & 1;
      if (!mbar_wait(&bars->acc_full[acc], acc_ph, abort_word, 301)) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN + half * (BN / 2);
      if (p.epi_mode == 3) store_tile_rows_rope(p, t_row, tm * BM + quad * 32 + lane, tn * BN + half * (BN / 2));
      else store_tile_rows(p, t_row, b, tm * BM + quad * 32 + lane, tn * BN + half * (BN / 2));
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

// ------------------------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs computes a 256 x 256 tile with tcgen05.mma.cta_group::2.
// Each CTA loads its own 128 rows of A and its own 128-column half of B (32 KiB per stage, so the
// ring is 6 deep), which halves the B traffic per SM; the pair's leader (cluster rank 0) issues
// every MMA for both CTAs and each CTA drains its own 128 accumulator rows from its own TMEM.
// Cross-CTA signalling: the peer's TMA loads complete on the leader's `full` barrier
// (cta_group::2 form of the load, barrier given as a cluster address); the leader releases
// stages and publishes accumulators with one tcgen05.commit per CTA (local and peer address); the
// peer's epilogue warps arrive on the leader's `acc_empty` barrier with a remote mbarrier.arrive.
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_STAGE_BYTES = 2 * A_BYTES;  // A 128 x 64 and half of B 128 x 64
constexpr int PAIR_M = 2 * BM;
constexpr size_t PAIR_SMEM_BYTES = 1024 + PAIR_STAGES * PAIR_STAGE_BYTES + 256;

// Work units are handed out at run time: a cluster's first unit is its index, every further one
// comes from a global counter, so a cluster that finds its SMs late (another kernel, e.g. a
// collective, holds them) takes less work instead of holding its fixed share back to the end.
// The leader's producer thread draws the unit for step t and publishes it in slot t % SCHED_SLOTS
// of both CTAs' rings: locally with a store and an arrival on sched_full, in the peer with one
// st.async that carries the value and completes the peer's sched_full (armed by the peer's
// producer thread with expect-tx).  No role can be SCHED_SLOTS units ahead of another (6 stages of
// operands and 2 accumulators bound the distance), so slots are reused without a release barrier.
constexpr int SCHED_SLOTS = 16;
constexpr uint32_t SCHED_DONE = 0xffffffffu;
struct PairBarriers {
  uint64_t full[PAIR_STAGES];
  uint64_t empty[PAIR_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t sched_full[SCHED_SLOTS];
  uint32_t unit_ring[SCHED_SLOTS];
  uint32_t tmem_base;
  int abort_word;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
    gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                          const __grid_constant__ CUtensorMap tmap_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  PairBarriers* bars = reinterpret_cast<PairBarriers*>(smem + PAIR_STAGES * PAIR_STAGE_BYTES);
  volatile int* abort_word = &bars->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  // Work unit = (tile, K slice); slices exist only in the accumulate-in-place form.
  const int num_units = p.num_tiles * p.split_k;
  // Unit numbering with K slices: tiles are taken in chunks of one wave (as many tiles as the
  // grid has clusters); within a chunk all tiles of K slice 0 come first, then all of slice 1, ...
  // The clusters that run at the same time then work on neighbouring tiles of ONE slice and share
  // its A and B panels through L2, and the chunk's slices follow each other while the chunk's
  // part of D (19 MB at 74 tiles) is still in L2.  Weight gradient 2048 x 5632 x 16384 (251 MB of
  // operands, 46 MB of f32 output read and written): numbered tile by tile (a wave = three slices
  // of ~25 tiles, which share nothing) 693 MB read + 42 MB written; slice by slice over all tiles
  // 525 + 75 MB (every slice pass brings all of D back).
  auto unit_range = [&](int unit, int& tile, int& kb0, int& kb1) {
    int slice;
    if (p.split_k == 1) {
      tile = unit;
      slice = 0;
    } else {
      const int per_chunk = num_clusters * p.split_k;
      const int chunk = unit / per_chunk;
      const int r = unit - chunk * per_chunk;
      const int first = chunk * num_clusters;
      const int in_chunk = p.num_tiles - first < num_clusters ? p.num_tiles - first : num_clusters;
      slice = r / in_chunk;
      tile = first + (r - slice * in_chunk);
    }
    kb0 = static_cast<int>(static_cast<long long>(slice) * p.k_blocks / p.split_k);
    kb1 = static_cast<int>(static_cast<long long>(slice + 1) * p.k_blocks / p.split_k);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->acc_full[i], 1);
      mbar_init(&bars->acc_empty[i], 2 * EPI_WARPS);  // epilogue warps of both CTAs (leader's copy is used)
    }
    for (int i = 0; i < SCHED_SLOTS; ++i) mbar_init(&bars->sched_full[i], 1);
    bars->abort_word = 0;
    fence_mbar_init();
    // the peer's slots wait for the leader's 4-byte st.async
    if (rank != 0)
      for (int i = 0; i < SCHED_SLOTS; ++i) mbar_arrive_expect_tx(&bars->sched_full[i], 4);
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  grid_dep_wait();  // set-up above overlaps the previous kernel's tail; global memory from here on
  grid_dep_launch();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      // The leader's producer also hands out the units (see PairBarriers).  Every cluster with a
      // valid first unit draws from the counter after each unit it takes, until a draw runs past
      // the last unit; the launch's last draw puts the counter back to zero.
      const int fetchers = num_clusters < num_units ? num_clusters : num_units;
      const unsigned total_draws = static_cast<unsigned>((num_units > num_clusters ? num_units - num_clusters : 0) + fetchers);
      uint32_t unit_u = cluster_id < num_units ? static_cast<uint32_t>(cluster_id) : SCHED_DONE;
      unsigned drawn = 0;  // the draw for the next step, under way while this step's tiles load
      for (int t = 0; ok; ++t) {
        const int slot = t % SCHED_SLOTS;
        if (rank == 0) {
          if (t > 0) {
            if (p.sched_counter != nullptr) {
              unit_u = static_cast<unsigned>(num_clusters) + drawn < static_cast<unsigned>(num_units)
                           ? static_cast<uint32_t>(num_clusters) + drawn
                           : SCHED_DONE;
              if (drawn + 1 == total_draws) atomicExch(p.sched_counter, 0u);
            } else {  // fixed round-robin assignment
              const long long u = static_cast<long long>(cluster_id) + static_cast<long long>(t) * num_clusters;
              unit_u = u < num_units ? static_cast<uint32_t>(u) : SCHED_DONE;
            }
          }
          bars->unit_ring[slot] = unit_u;
          mbar_arrive(&bars->sched_full[slot]);
          st_async_u32(mapa_shared(smem_u32(&bars->unit_ring[slot]), 1), unit_u,
                       mapa_shared(smem_u32(&bars->sched_full[slot]), 1));
          if (unit_u != SCHED_DONE && p.sched_counter != nullptr) drawn = atomicAdd(p.sched_counter, 1u);
        } else {
          if (!mbar_wait(&bars->sched_full[slot], (t / SCHED_SLOTS) & 1, abort_word, 112)) break;
          unit_u = bars->unit_ring[slot];
          mbar_arrive_expect_tx(&bars->sched_full[slot], 4);  // armed again for step t + SCHED_SLOTS
        }
        if (unit_u == SCHED_DONE) break;
        const int unit = static_cast<int>(unit_u);
        int tile, kb0, kb1, b, tm, tn;
        unit_range(unit, tile, kb0, kb1);
        tile_coords(p, tile, b, tm, tn);
        const int m0 = tm * PAIR_M + static_cast<int>(rank) * BM;
        const int n0 = tn * BN + static_cast<int>(rank) * (BN / 2);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % PAIR_STAGES;
          const uint32_t ph = (it / PAIR_STAGES) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_word, 111)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * PAIR_STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          // Bytes of both CTAs land on the leader's barrier.
          if (rank == 0) mbar_arrive_expect_tx(&bars->full[s], 2 * PAIR_STAGE_BYTES);
          const uint32_t full_leader = mapa_shared(smem_u32(&bars->full[s]), 0);
          const int k0 = kb * BK;
          if (p.a_mn) {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_3d_pair(sa + i * 8192, &tmap_a, full_leader, m0 + i * 64, k0, b);
          } else {
            tma_load_3d_pair(sa, &tmap_a, full_leader, k0, m0, b);
          }
          if (p.b_mn) {
#pragma unroll
            for (int i = 0; i < BN / 128; ++i)
              tma_load_3d_pair(sb + i * 8192, &tmap_b, full_leader, n0 + i * 64, k0, b);
          } else {
            tma_load_3d_pair(sb, &tmap_b, full_leader, k0, n0, b);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0 && elect_one()) {
      const uint32_t idesc = make_idesc_bf16(PAIR_M, BN, p.a_mn, p.b_mn);
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
      const uint32_t a_kstep = p.a_mn ? 2048u : 32u, b_kstep = p.b_mn ? 2048u : 32u;
      uint32_t it = 0;
      int t = 0;
      bool ok = true;
      for (; ok; ++t) {
        const int slot = t % SCHED_SLOTS;
        if (!mbar_wait(&bars->sched_full[slot], (t / SCHED_SLOTS) & 1, abort_word, 213)) break;
        const uint32_t unit_u = bars->unit_ring[slot];
        if (unit_u == SCHED_DONE) break;
        const int unit = static_cast<int>(unit_u);
        int tile, kb0, kb1;
        unit_range(unit, tile, kb0, kb1);
        const int acc = t & 1;
        const uint32_t acc_ph = (t >> 1) & 1;
        if (!mbar_wait(&bars->acc_empty[acc], acc_ph ^ 1, abort_word, 211)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % PAIR_STAGES;
          const uint32_t ph = (it / PAIR_STAGES) & 1;
          if (!mbar_wait(&bars->full[s], ph, abort_word, 212)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * PAIR_STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = smem_desc_sw128(sa + k * a_kstep, a_lbo, 1024);
            const uint64_t db = smem_desc_sw128(sb + k * b_kstep, b_lbo, 1024);
            umma_ss_pair(d_tmem, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          const uint32_t e = smem_u32(&bars->empty[s]);
          umma_commit_pair(e);                  // own producer
          umma_commit_pair(mapa_shared(e, 1));  // the peer's producer
        }
        if (ok) {
          const uint32_t f = smem_u32(&bars->acc_full[acc]);
          umma_commit_pair(f);
          umma_commit_pair(mapa_shared(f, 1));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    int t = 0;
    for (;; ++t) {
      const int slot = t % SCHED_SLOTS;
      if (!mbar_wait(&bars->sched_full[slot], (t / SCHED_SLOTS) & 1, abort_word, 312)) break;
      const uint32_t unit_u = bars->unit_ring[slot];
      if (unit_u == SCHED_DONE) break;
      const int unit = static_cast<int>(unit_u);
      int tile, kb0, kb1, b, tm, tn;
      unit_range(unit, tile, kb0, kb1);
      tile_coords(p, tile, b, tm, tn);
      const int acc = t & 1;
      const uint32_t acc_ph = (t >> 1) & 1;
      if (!mbar_wait(&bars->acc_full[acc], acc_ph, abort_word, 311)) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN + half * (BN / 2);
      const int row = tm * PAIR_M + static_cast<int>(rank) * BM + quad * 32 + lane;
      if (p.epi_mode == 3) store_tile_rows_rope(p, t_row, row, tn * BN + half * (BN / 2));
      else store_tile_rows(p, t_row, b, row, tn * BN + half * (BN / 2));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&bars->acc_empty[acc]), 0));
    }
  }

  // ------------------------------------------------------------ tear-down
  __syncwarp();
  if (*abort_word != 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer may still signal into this CTA's shared memory until here
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
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

static int32_t check_epi_operand(const char* name, const cdl_tensor* t, long long M, long long N) {
  if (!t || t->rank != 2 || t->shape[0] != M || t->shape[1] != N || t->dtype != CDL_BF16 ||
      t->stride[1] != 1 || t->stride[0] % 8 != 0 || (reinterpret_cast<uintptr_t>(t->ptr) & 15) != 0)
    return fail(CDL_ERR_INVALID,
                "matmul (fused SwiGLU): %s must be bf16 [%lld, %lld] with 16-byte aligned rows", name, M, N);
  return CDL_OK;
}

int32_t matmul_execute(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* c,
                       const cdl_tensor* d, float alpha, float beta, cudaStream_t stream,
                       const cdl_matmul_options* opts) {
  return matmul_execute_epi(a, b, c, d, alpha, beta, 0, nullptr, nullptr, nullptr, stream, opts, nullptr);
}

int32_t matmul_execute_epi(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* c,
                           const cdl_tensor* d, float alpha, float beta, int epi_mode,
                           const cdl_tensor* aux0, const cdl_tensor* aux1, const cdl_tensor* out2,
                           cudaStream_t stream, const cdl_matmul_options* opts, const RopeEpilogue* rope) {
  using namespace gemm;
  const int variant = opts ? opts->variant : CDL_GEMM_AUTO;
  if (variant < CDL_GEMM_AUTO || variant > CDL_GEMM_CTA_PAIR)
    return fail(CDL_ERR_INVALID, "matmul: unknown kernel variant %d", variant);
  if (!a || !b || !d) return fail(CDL_ERR_INVALID, "matmul: a, b and d are required");
  if (a->rank != b->rank || (a->rank != 2 && a->rank != 3) || d->rank != a->rank)
    return fail(CDL_ERR_INVALID,
                "matmul operands must all have rank 2 or all rank 3 (got rank %d, %d, %d)",
                a->rank, b->rank, d->rank);
  const bool f32_inputs = a->dtype == CDL_F32 && b->dtype == CDL_F32;
  if (!f32_inputs && (a->dtype != CDL_BF16 || b->dtype != CDL_BF16))
    return fail(CDL_ERR_INVALID, "matmul inputs must be f32 or bf16 and of one type (got %s x %s)",
                dtype_name(a->dtype), dtype_name(b->dtype));
  if (f32_inputs && epi_mode != 0)
    return fail(CDL_ERR_UNSUPPORTED, "matmul (fused SwiGLU): inputs must be bf16");
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

  // f32 inputs, and bf16 operands TMA cannot describe (unaligned pointer or leading dimension):
  // the general CUDA-core kernel (gemm_general.cu).  Operands without any contiguous dimension
  // stay rejected, as in the reference.
  if (f32_inputs) return matmul_general_execute(a, b, c, d, alpha, beta, stream);
  OperandLayout la, lb;
  for (int which = 0; which < 2; ++which) {
    const int32_t rc = which == 0 ? analyze_operand("a", a, true, &la) : analyze_operand("b", b, false, &lb);
    if (rc == CDL_ERR_UNSUPPORTED && epi_mode == 0)
      return matmul_general_execute(a, b, c, d, alpha, beta, stream);
    CDL_CHECK(rc);
  }

  // Kernel choice: CTA pairs (256 x 256 tiles) whenever the problem has more than one 128-row
  // slab, unless the caller's options name a variant.
  const bool use_pair = variant == CDL_GEMM_AUTO ? M > BM : variant == CDL_GEMM_CTA_PAIR;
  const int tile_m = use_pair ? PAIR_M : BM;
  const uint32_t b_box_rows = use_pair ? BN / 2 : BN;

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
      db[0] = K; db[1] = N; bb[0] = 64; bb[1] = b_box_rows;
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
  p.num_m_tiles = static_cast<int>((M + tile_m - 1) / tile_m);
  p.num_n_tiles = static_cast<int>((N + BN - 1) / BN);
  const long long tiles = batch * p.num_m_tiles * p.num_n_tiles;
  if (tiles > INT32_MAX) return fail(CDL_ERR_UNSUPPORTED, "matmul: too many tiles");
  p.num_tiles = static_cast<int>(tiles);
  p.k_blocks = static_cast<int>((K + BK - 1) / BK);
  {
    // Raster panels: all M tiles of `raster_w` N tiles run together, so the panel's B columns
    // (raster_w * 256 * K elements) and, when it fits next to them, all of A are served from L2
    // while the panel lasts.  With a long K (the weight-gradient shapes: K = tokens) eight B
    // column panels plus A exceed the L2's 126 MB and both get evicted and re-read from HBM, so
    // the panel is narrowed until A and the panel's B fit a budget of 96 MB.
    const double a_bytes = 2.0 * static_cast<double>(M) * K;
    const double b_panel = 2.0 * BN * static_cast<double>(K);
    const double budget = static_cast<double>(CDL_GEMM_RASTER_BUDGET_MB) * 1024 * 1024;
    int w = RASTER_W;
    if (a_bytes <= 0.75 * budget)
      while (w > 2 && a_bytes + w * b_panel > budget) --w;
    p.raster_w = w;
  }
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
  p.split_k = 1;
  p.sched_counter = nullptr;
  p.atomic_out = 0;
  p.epi_mode = 0;
  p.aux0 = p.aux1 = nullptr;
  p.out2 = nullptr;
  p.ld_aux0 = p.ld_aux1 = p.ld_out2 = 0;
  p.rope_table = nullptr;
  p.rope_cu = nullptr;
  p.rope_seqlen = p.rope_cols = p.rope_nseq = 0;
  if (epi_mode == 3) {
    if (!rope || !rope->table || rope->seqlen <= 0 || rope->rot_cols < 0 || rope->rot_cols % 128 != 0 ||
        rope->rot_cols > N || (rope->cu_seqlens != nullptr && rope->num_seqs <= 0))
      return fail(CDL_ERR_INVALID, "matmul (RoPE epilogue): table, seqlen > 0 and rot_cols (a multiple of 128, "
                  "at most N) are required");
    if (r != 2 || use_c || d->dtype != CDL_BF16 || N % 128 != 0 || !p.d_vec ||
        (reinterpret_cast<uintptr_t>(rope->table) & 15) != 0)
      return fail(CDL_ERR_INVALID, "matmul (RoPE epilogue): rank 2, no C operand, bf16 output with 16-byte "
                  "aligned rows, N %% 128 == 0 and a 16-byte aligned table are required");
    p.epi_mode = 3;
    p.rope_table = rope->table;
    p.rope_cu = rope->cu_seqlens;
    p.rope_seqlen = rope->seqlen;
    p.rope_cols = rope->rot_cols;
    p.rope_nseq = rope->num_seqs;
  } else if (epi_mode != 0) {
    if (r != 2 || use_c || d->dtype != CDL_BF16 || N % 8 != 0 || !p.d_vec)
      return fail(CDL_ERR_INVALID,
                  "matmul (fused SwiGLU): rank 2, no C operand, bf16 output with 16-byte aligned rows "
                  "and N %% 8 == 0 are required");
    CDL_CHECK(check_epi_operand("aux0", aux0, M, N));
    CDL_CHECK(check_epi_operand("out2", out2, M, N));
    if (epi_mode == 2) CDL_CHECK(check_epi_operand("aux1", aux1, M, N));
    p.epi_mode = epi_mode;
    p.aux0 = static_cast<const __nv_bfloat16*>(aux0->ptr);
    p.ld_aux0 = aux0->stride[0];
    p.out2 = static_cast<__nv_bfloat16*>(out2->ptr);
    p.ld_out2 = out2->stride[0];
    if (epi_mode == 2) {
      p.aux1 = static_cast<const __nv_bfloat16*>(aux1->ptr);
      p.ld_aux1 = aux1->stride[0];
    }
  }
  {
    auto al32 = [](const void* ptr, long long ld, long long bstride, size_t es) {
      return (reinterpret_cast<uintptr_t>(ptr) & 31) == 0 && (ld * es) % 32 == 0 &&
             (bstride * es) % 32 == 0;
    };
    bool w = al32(p.d, p.ldd, p.d_batch, dtype_size(d->dtype));
    if (use_c) w = w && al32(p.c, p.ldc, p.c_batch, dtype_size(c->dtype));
    if (p.epi_mode == 1 || p.epi_mode == 2) {
      w = w && al32(p.aux0, p.ld_aux0, 0, 2) && al32(p.out2, p.ld_out2, 0, 2);
      if (p.epi_mode == 2) w = w && al32(p.aux1, p.ld_aux1, 0, 2);
    }
    p.wide = w ? 1 : 0;
  }
  p.status = device_status_ptr();
  if (!p.status) return fail(CDL_ERR_CUDA, "cannot resolve the device status word");

  static std::once_flag attr_once[64];
  static int max_clusters[64] = {};
  int dev = 0;
  CDL_CUDA(cudaGetDevice(&dev));
  cudaError_t attr_err = cudaSuccess;
  std::call_once(attr_once[dev & 63], [&] {
    attr_err = cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(SMEM_BYTES));
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(gemm_bf16_pair_kernel,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(PAIR_SMEM_BYTES));
    // How many CTA pairs the device can hold at once (GPCs with an odd SM count lose one SM).
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(sm_count() & ~1));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
    if (attr_err == cudaSuccess &&
        cudaOccupancyMaxActiveClusters(&n, gemm_bf16_pair_kernel, &cfg) == cudaSuccess && n > 0)
      max_clusters[dev & 63] = n;
    else
      max_clusters[dev & 63] = sm_count() / 2;
    (void)cudaGetLastError();
  });
  if (attr_err != cudaSuccess)
    return fail(CDL_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(attr_err));

  // K slicing for the accumulate-in-place form (D = C, f32, beta = 1: the weight-gradient GEMM,
  // whose output is small and whose K is long).  Slices add into D with atomics, which removes
  // the tile-count quantisation (e.g. 192 tiles on 74 CTA pairs = 2.6 waves) at the price of an
  // unordered f32 sum; the caller's `deterministic` option turns it off.
  if (use_pair && use_c && p.out_f32 && c->dtype == CDL_F32 && c->ptr == d->ptr && beta == 1.0f &&
      p.ldc == p.ldd && p.c_batch == p.d_batch) {
    if (!(opts && opts->deterministic != 0)) {
      const int nc = max_clusters[dev & 63];
      int best_s = 1;
      double best_cost = 1e30;
      for (int sp = 1; sp <= 8 && sp * 8 <= p.k_blocks; ++sp) {
        const long long units = static_cast<long long>(p.num_tiles) * sp;
        const long long waves = (units + nc - 1) / nc;
        // time ~ waves * (K slice + a fixed per-unit cost worth ~6 K blocks of epilogue / ramp)
        const double cost = static_cast<double>(waves) * (static_cast<double>(p.k_blocks) / sp + 6.0);
        if (cost < best_cost * 0.97) {
          best_cost = cost;
          best_s = sp;
        }
      }
      if (best_s > 1) {
        p.split_k = best_s;
        p.atomic_out = 1;
        p.c_mode = 0;  // D already holds C; the slices only add
        // Only one K slice of the operands is live at a time (units are numbered slice by slice
        // within a chunk of tiles): the raster panel may be as wide as that slice allows.
        const double a_slice = 2.0 * static_cast<double>(M) * K / best_s;
        const double b_panel_slice = 2.0 * BN * static_cast<double>(K) / best_s;
        const double budget = static_cast<double>(CDL_GEMM_RASTER_BUDGET_MB) * 1024 * 1024;
        int w = RASTER_W;
        if (a_slice <= 0.75 * budget)
          while (w > 2 && a_slice + w * b_panel_slice > budget) --w;
        p.raster_w = w;
      }
    }
  }

  ProfileScope ps(PROF_GEMM, 2.0 * static_cast<double>(batch) * M * N * K, stream);
  if (use_pair) {
    const long long units = static_cast<long long>(p.num_tiles) * p.split_k;
    const int clusters = units < max_clusters[dev & 63] ? static_cast<int>(units) : max_clusters[dev & 63];
    p.sched_counter = units > clusters ? sched_counter_for(0, dev, stream) : nullptr;
    CDL_CUDA(launch_pdl(gemm_bf16_pair_kernel, dim3(2 * clusters), dim3(THREADS), PAIR_SMEM_BYTES, stream,
                        tm_a, tm_b, p));
  } else {
    const int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
    CDL_CUDA(launch_pdl(gemm_bf16_kernel, dim3(grid), dim3(THREADS), SMEM_BYTES, stream, tm_a, tm_b, p));
  }
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

int32_t cdl_b200_matmul_opt(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* c,
                            const cdl_tensor* d, float alpha, float beta,
                            const cdl_matmul_options* options, void* scratch, size_t scratch_bytes,
                            cdl_stream stream) {
  (void)scratch;
  (void)scratch_bytes;
  return cdl::matmul_execute(a, b, c, d, alpha, beta, static_cast<cudaStream_t>(stream), options);
}

int32_t cdl_b200_matmul_candidates(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* d,
                                   cdl_matmul_options* out, int32_t capacity, int32_t* count) {
  using namespace cdl;
  if (!a || !b || !d || !count || (capacity > 0 && !out))
    return fail(CDL_ERR_INVALID, "matmul_candidates: a, b, d, count (and out) are required");
  cdl_matmul_options list[4];
  int n = 0;
  const bool tensor_core = a->dtype == CDL_BF16 && b->dtype == CDL_BF16 && a->rank >= 2 &&
                           a->rank == b->rank && [&] {
                             gemm::OperandLayout la, lb;
                             const bool ok = gemm::analyze_operand("a", a, true, &la) == CDL_OK &&
                                             gemm::analyze_operand("b", b, false, &lb) == CDL_OK;
                             last_error().clear();
                             return ok;
                           }();
  if (!tensor_core) {
    list[n++] = {CDL_GEMM_AUTO, 0};
  } else {
    const long long M = a->shape[a->rank - 2];
    const bool accumulates = d->dtype == CDL_F32;  // the weight-gradient form may slice K
    const int first = M > gemm::BM ? CDL_GEMM_CTA_PAIR : CDL_GEMM_ONE_CTA;
    const int second = first == CDL_GEMM_CTA_PAIR ? CDL_GEMM_ONE_CTA : CDL_GEMM_CTA_PAIR;
    list[n++] = {first, 0};
    if (accumulates && first == CDL_GEMM_CTA_PAIR) list[n++] = {first, 1};
    list[n++] = {second, 0};
    if (accumulates && second == CDL_GEMM_CTA_PAIR) list[n++] = {second, 1};
  }
  *count = n;
  for (int i = 0; i < n && i < capacity; ++i) out[i] = list[i];
  return CDL_OK;
}

int32_t cdl_b200_matmul_swiglu_gate(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* up,
                                    const cdl_tensor* gate_out, const cdl_tensor* act_out,
                                    cdl_stream stream) {
  return cdl::matmul_execute_epi(a, b, nullptr, gate_out, 1.0f, 0.0f, 1, up, nullptr, act_out,
                                 static_cast<cudaStream_t>(stream), nullptr, nullptr);
}

int32_t cdl_b200_matmul_rope(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* cos_sin,
                             int32_t rot_heads, int32_t seqlen, const cdl_tensor* cu_seqlens,
                             const cdl_tensor* d, cdl_stream stream) {
  using namespace cdl;
  const char* op = "matmul (RoPE epilogue)";
  if (!cos_sin || cos_sin->rank != 2 || cos_sin->dtype != CDL_F32 || cos_sin->shape[1] != 128 ||
      cos_sin->stride[1] != 1 || cos_sin->stride[0] != 128 || seqlen <= 0 || cos_sin->shape[0] < seqlen)
    return fail(CDL_ERR_INVALID, "%s: cos_sin must be packed f32 [>= seqlen, 128] (head_dim 128)", op);
  if (rot_heads < 0) return fail(CDL_ERR_INVALID, "%s: rot_heads must not be negative", op);
  if (cu_seqlens && (cu_seqlens->rank != 1 || cu_seqlens->dtype != CDL_I32 || cu_seqlens->stride[0] != 1 ||
                     cu_seqlens->shape[0] < 2))
    return fail(CDL_ERR_INVALID, "%s: cu_seqlens must be a packed i32 vector of num_seqs + 1 entries", op);
  RopeEpilogue rope{static_cast<const float*>(cos_sin->ptr), seqlen, rot_heads * 128,
                    cu_seqlens ? static_cast<const int*>(cu_seqlens->ptr) : nullptr,
                    cu_seqlens ? static_cast<int>(cu_seqlens->shape[0] - 1) : 0};
  return matmul_execute_epi(a, b, nullptr, d, 1.0f, 0.0f, 3, nullptr, nullptr, nullptr,
                            static_cast<cudaStream_t>(stream), nullptr, &rope);
}

int32_t cdl_b200_matmul_swiglu_dgrad(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* gate,
                                     const cdl_tensor* up, const cdl_tensor* d_up_out,
                                     const cdl_tensor* d_gate_out, cdl_stream stream) {
  return cdl::matmul_execute_epi(a, b, nullptr, d_up_out, 1.0f, 0.0f, 2, gate, up, d_gate_out,
                                 static_cast<cudaStream_t>(stream), nullptr, nullptr);
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
