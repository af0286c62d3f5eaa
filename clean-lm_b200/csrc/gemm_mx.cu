// Matmul with block-scaled (MXFP8 or NVFP4) operands: D = alpha * dequant(A) . dequant(B), f32
// accumulate; plain bf16 / f32 output or an MXFP8 block-scaled one.
//
// The reference forwards this case to cuBLASLt block scaling
// (crates/cleandl/src/execgraph/ops/matmul.rs:808-838, InputKind::Mx; tests
// crates/cleandl/tests/matmul.rs:1041-1060); its own block-scaled tcgen05 kernel generator is
// crates/cleandl-specialized-kernels/src/kernels/matmul/tcgen05.rs.  A is rowwise [M, K], B is
// colwise [K, N]: both value matrices are K-contiguous bytes, both scale tensors are in the
// 128 x 4 tiled layout, which is what the hardware reads.
//
// Two kernels share the design below: a one-CTA kernel (128 x 256 tiles) and, further down, the
// CTA-pair kernel (256 x 256 tiles) that is used whenever M > 128.  The text describes MXFP8;
// Cfg<> lists what changes for NVFP4.
//
// Kernel: persistent, one CTA per SM, 128 x 256 output tiles, K in steps of 128 bytes (one
// 128-byte swizzled row per operand row, four K = 32 instructions).  Per stage the producer warp
// brings A (16 KiB) and B (32 KiB) with TMA and the three 512-byte scale tiles (one of A's 128
// rows, two of B's 256) with bulk copies; the MMA thread copies the scale tiles into tensor
// memory (tcgen05.cp, ordered with its MMAs) and issues
// tcgen05.mma.kind::mxf8f6f4.block_scale, selecting the K block's scale byte in the instruction
// descriptor.
//
// Tensor memory holds 512 columns: two 256-column accumulators do not fit beside the 12 scale
// columns, so the accumulators OVERLAP by 16 columns (columns [0,256) and [240,496), scales at
// [496,508)).  The epilogue of a tile drains the 16 shared columns first and signals; the first
// MMA of the next tile waits for that signal only, so the rest of the epilogue still overlaps
// the next tile's main loop.
#include "host.h"
#include "ops.h"
#include "ptx.cuh"

#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <stdlib.h>
#include <string.h>

#include <mutex>

namespace cdl {
namespace gemm_mx {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;  // elements == bytes
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK;
constexpr int B_BYTES = BN * BK;
constexpr int SF_TILE = 512;  // scales of 128 rows x 4 blocks
constexpr int SF_OFF = A_BYTES + B_BYTES;
constexpr int THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue
constexpr int EPI_WARPS = 8;
constexpr int TMEM_COLS = 512;
constexpr int RASTER_W = 8;

// What differs between the two formats.  A stage is always 128 bytes of K per operand row and four
// instructions.  MXFP8: 128 elements, one scale byte per row and instruction, so one 512-byte
// scale tile per 128 rows and stage, the instruction picks its byte.  NVFP4: 256 elements, four
// scale bytes per row and instruction, so four scale tiles per 128 rows and stage and 48 scale
// columns in tensor memory; the accumulators then overlap by 48 columns.
template <int FP4>
struct Cfg {
  static constexpr int SFT = FP4 ? 4 : 1;        // scale tiles per 128 operand rows per stage
  static constexpr int K_STAGE = FP4 ? 256 : 128;  // elements of K per stage
  static constexpr int K_MMA = FP4 ? 64 : 32;      // elements of K per instruction
  static constexpr int STAGE_BYTES = (FP4 ? 54 : 50) * 1024;  // A, B, 3 * SFT scale tiles; 1024-aligned
  static constexpr int OVERLAP = FP4 ? 48 : 16;    // columns the two accumulators share
  static constexpr int OVL_CHUNKS = FP4 ? 2 : 1;   // 32-column chunks that cover them
  static constexpr int ACC1_COL = 256 - OVERLAP;   // accumulator 0 at column 0, accumulator 1 here
  static constexpr int SFA_COL = 512 - 12 * SFT;
  static constexpr int SFB_COL = SFA_COL + 4 * SFT;
  static constexpr size_t SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 256;
  static_assert(SF_OFF + 3 * SFT * SF_TILE <= STAGE_BYTES, "stage layout");
  static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KiB of shared memory a CTA can opt in to");
  static_assert(ACC1_COL + 256 <= SFA_COL && ACC1_COL % 16 == 0, "tensor memory layout");
};

struct Params {
  int M, N, K;
  int num_m_tiles, num_n_tiles, num_tiles, k_tiles;
  const uint8_t* sfa;  // scale tiles of A: [ceil(M/128)][sf_k_tiles][512]
  const uint8_t* sfb;  // scale tiles of B: [ceil(N/128)][sf_k_tiles][512]
  int sf_k_tiles;      // ceil(blocks along K / 4)
  void* d;
  long long ldd;
  int out_f32, wide;
  // C operand (plain outputs only): c_mode 0 none, 1 bf16, 2 f32; v = alpha * acc + beta * C
  int c_mode;
  const void* c;
  long long ldc;
  float beta;
  // Block-scaled output, rowwise: out_mx 1 = MXFP8, 2 = NVFP4 values and scale tiles.
  int out_mx;
  uint8_t* out_values;
  uint8_t* out_sf;
  float alpha;
  int* status;
};

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t overlap_free;
  uint32_t tmem_base;
  int abort_word;
};

__device__ __forceinline__ void tile_coords(const Params& p, int tile, int& m, int& n) {
  const int panel_tiles = RASTER_W * p.num_m_tiles;
  const int panel = tile / panel_tiles;
  const int first_n = panel * RASTER_W;
  const int width = min(RASTER_W, p.num_n_tiles - first_n);
  const int r = tile - panel * panel_tiles;
  m = r / width;
  n = first_n + (r - m * width);
}

// 32 consecutive columns of one output row.
__device__ __forceinline__ void store32(const Params& p, const uint32_t (&r)[32], int row, int col0) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = p.alpha * __uint_as_float(r[j]);
  const bool full = col0 + 32 <= p.N;
  if (p.c_mode == 1) {
    const __nv_bfloat16* cp = static_cast<const __nv_bfloat16*>(p.c) + static_cast<long long>(row) * p.ldc + col0;
    if (p.wide && full) {
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
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) v[j] += p.beta * __bfloat162float(cp[j]);
    }
  } else if (p.c_mode == 2) {
    const float* cp = static_cast<const float*>(p.c) + static_cast<long long>(row) * p.ldc + col0;
    if (p.wide && full) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint32_t w[8];
        ld_global_v8(cp + g * 8, w);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[g * 8 + j] += p.beta * __uint_as_float(w[j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) v[j] += p.beta * cp[j];
    }
  }
  if (p.out_f32) {
    float* dp = static_cast<float*>(p.d) + static_cast<long long>(row) * p.ldd + col0;
    if (p.wide && full) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) w[j] = __float_as_uint(v[g * 8 + j]);
        st_global_v8(dp + g * 8, w);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) dp[j] = v[j];
    }
  } else {
    __nv_bfloat16* dp = static_cast<__nv_bfloat16*>(p.d) + static_cast<long long>(row) * p.ldd + col0;
    if (p.wide && full) {
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) w[j] = pack_bf16x2(v[g * 16 + 2 * j], v[g * 16 + 2 * j + 1]);
        st_global_v8(dp + g * 16, w);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) dp[j] = __float2bfloat16_rn(v[j]);
    }
  }
}

__device__ __forceinline__ long long sf_index(int outer, int block, int blocks) {
  return (static_cast<long long>(outer >> 7) * ((blocks + 3) >> 2) + (block >> 2)) * 512 +
         (outer & 31) * 16 + ((outer & 127) >> 5) * 4 + (block & 3);
}
// Scale exponent and descale factor of a block with maximum magnitude amax (the quantiser of
// mx.cu: amax / 448 rounded up to a power of two).
__device__ __forceinline__ uint32_t scale_exponent(float amax) {
  const uint32_t bits = __float_as_uint(amax);
  const int e = static_cast<int>(bits >> 23) - 8 + ((bits & 0x7FFFFFu) > 0x600000u ? 1 : 0);
  return static_cast<uint32_t>(min(max(e, 0), 254));
}
__device__ __forceinline__ float descale_of(uint32_t e) {
  const uint32_t de = 254u - e;
  return __uint_as_float(de != 0 ? de << 23 : 0x00400000u);
}
__device__ __forceinline__ uint32_t fp8x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// The NVFP4 form of the block-scaled store: the 32 columns are two blocks of 16; scale = amax / 6
// rounded to nearest E4M3, elements x * (1 / scale) rounded to nearest E2M1 (the quantiser of mx.cu).
__device__ __forceinline__ void store32_nvfp4(const Params& p, const uint32_t (&r)[32], int row, int col0) {
  if (row >= p.M) return;
  uint32_t out[4];
  uint32_t sf2 = 0;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float v[16];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      v[j] = p.alpha * __uint_as_float(r[h * 16 + j]);
      amax = fmaxf(amax, fabsf(v[j]));
    }
    const __nv_fp8_storage_t sbits = __nv_cvt_float_to_fp8(__fdiv_rn(amax, 6.0f), __NV_SATFINITE, __NV_E4M3);
    const float sc = __half2float(__half(__nv_cvt_fp8_to_halfraw(sbits, __NV_E4M3)));
    const float inv = sc != 0.f ? __frcp_rn(sc) : 0.f;  // a zero scale stores zeros
    sf2 |= static_cast<uint32_t>(sbits) << (8 * h);
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      uint32_t word = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = __fmul_rn(v[w * 8 + 2 * j], inv);
        const float b = __fmul_rn(v[w * 8 + 2 * j + 1], inv);
        word |= static_cast<uint32_t>(__nv_cvt_float2_to_fp4x2(make_float2(a, b), __NV_E2M1, cudaRoundNearest))
                << (8 * j);
      }
      out[h * 2 + w] = word;
    }
  }
  // N % 32 == 0: 16 bytes of values, 16-byte aligned; the two scales are neighbours in a tile
  *reinterpret_cast<uint4*>(p.out_values + (static_cast<long long>(row) * p.N + col0) / 2) =
      make_uint4(out[0], out[1], out[2], out[3]);
  *reinterpret_cast<uint16_t*>(p.out_sf + sf_index(row, col0 >> 4, p.N >> 4)) = static_cast<uint16_t>(sf2);
}

// Block-scaled (rowwise MXFP8) store of 32 consecutive columns of one output row: they are one
// block of the row.  A colwise output never reaches the kernel: the host runs it as the rowwise
// output of the transposed product (matmul_mx_out_execute).
__device__ __forceinline__ void store32_mx(const Params& p, const uint32_t (&r)[32], int row, int col0) {
  if (row >= p.M) return;
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    v[j] = p.alpha * __uint_as_float(r[j]);
    amax = fmaxf(amax, fabsf(v[j]));
  }
  const uint32_t e = scale_exponent(amax);
  const float ds = descale_of(e);
  uint32_t w[8];
#pragma unroll
  for (int j = 0; j < 8; ++j)
    w[j] = fp8x4(v[4 * j] * ds, v[4 * j + 1] * ds, v[4 * j + 2] * ds, v[4 * j + 3] * ds);
  st_global_v8(p.out_values + static_cast<long long>(row) * p.N + col0, w);  // N % 32 == 0
  p.out_sf[sf_index(row, col0 >> 5, p.N >> 5)] = static_cast<uint8_t>(e);
}

template <int FP4>
__global__ void __launch_bounds__(THREADS, 1)
    gemm_mx_kernel(const __grid_constant__ CUtensorMap tmap_a,
                   const __grid_constant__ CUtensorMap tmap_b, const Params p) {
  using C = Cfg<FP4>;
  constexpr int STAGE_BYTES = C::STAGE_BYTES;
  constexpr int SFT = C::SFT;
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
    mbar_init(&bars->overlap_free, 4);
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
    // ------------------------------------------------------------ producer
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(p, tile, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        // The second scale tile of B exists only if the tensor has rows beyond n0 + 128.
        const bool sfb2 = n0 + 128 < p.N;
        const uint8_t* sfa_row = p.sfa + static_cast<long long>(tm) * p.sf_k_tiles * SF_TILE;
        const uint8_t* sfb_row = p.sfb + static_cast<long long>(2 * tn) * p.sf_k_tiles * SF_TILE;
        for (int kt = 0; kt < p.k_tiles; ++kt, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_word, 401)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          uint8_t* ssf = sa + SF_OFF;
          // scale tiles of this stage that exist (the K tail may hold fewer than SFT)
          const uint32_t sf_bytes = static_cast<uint32_t>(min(SFT, p.sf_k_tiles - kt * SFT)) * SF_TILE;
          mbar_arrive_expect_tx(&bars->full[s], A_BYTES + B_BYTES + (sfb2 ? 3 : 2) * sf_bytes);
          const int k0 = kt * BK;  // byte coordinate along K
          tma_load_3d(sa, &tmap_a, &bars->full[s], k0, m0, 0);
          tma_load_3d(sb, &tmap_b, &bars->full[s], k0, n0, 0);
          const long long sf_off = static_cast<long long>(kt) * SFT * SF_TILE;
          bulk_load_1d(ssf, sfa_row + sf_off, sf_bytes, &bars->full[s]);
          bulk_load_1d(ssf + SFT * SF_TILE, sfb_row + sf_off, sf_bytes, &bars->full[s]);
          if (sfb2)
            bulk_load_1d(ssf + 2 * SFT * SF_TILE,
                         sfb_row + static_cast<long long>(p.sf_k_tiles) * SF_TILE + sf_off, sf_bytes,
                         &bars->full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      uint32_t it = 0;
      int t = 0;
      bool ok = true;
      const uint32_t sfa_t = tmem_base + C::SFA_COL, sfb_t = tmem_base + C::SFB_COL;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++t) {
        const int acc = t & 1;
        const uint32_t acc_ph = (t >> 1) & 1;
        if (!mbar_wait(&bars->acc_empty[acc], acc_ph ^ 1, abort_word, 402)) break;
        // the columns this accumulator shares with the previous tile's have been drained
        if (t > 0 && !mbar_wait(&bars->overlap_free, (t - 1) & 1, abort_word, 403)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * C::ACC1_COL;
        for (int kt = 0; kt < p.k_tiles; ++kt, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars->full[s], ph, abort_word, 404)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          const uint32_t ssf = sa + SF_OFF;
          // K % K_MMA == 0; the tail stage issues only the instructions (and copies only the
          // scale tiles) that exist
          const int kblocks = min(4, (p.K - kt * C::K_STAGE) / C::K_MMA);
          const int sf_tiles = FP4 ? kblocks : 1;
#pragma unroll
          for (int j = 0; j < SFT; ++j) {
            if (j < sf_tiles) {
              // tile j of A; tile j of B's two 128-row chunks, side by side for instruction j
              tmem_cp_32x128b_warpx4(sfa_t + 4 * j, smem_desc_rows16(ssf + j * SF_TILE));
              tmem_cp_32x128b_warpx4(sfb_t + 8 * j, smem_desc_rows16(ssf + (SFT + j) * SF_TILE));
              tmem_cp_32x128b_warpx4(sfb_t + 8 * j + 4,
                                     smem_desc_rows16(ssf + (2 * SFT + j) * SF_TILE));
            }
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (k < kblocks) {
              const uint64_t da = smem_desc_sw128(sa + k * 32, 16, 1024);
              const uint64_t db = smem_desc_sw128(sb + k * 32, 16, 1024);
              if (FP4)
                umma_nvf4_ss(d_tmem, da, db, make_idesc_nvf4(BM, BN), sfa_t + 4 * k, sfb_t + 8 * k,
                             (kt | k) != 0 ? 1u : 0u);
              else
                umma_mxf8_ss(d_tmem, da, db, make_idesc_mxf8(BM, BN, k, k), sfa_t, sfb_t,
                             (kt | k) != 0 ? 1u : 0u);
            }
          }
          umma_commit(&bars->empty[s]);
        }
        if (ok) umma_commit(&bars->acc_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    const int quad = warp & 3;         // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;  // which 128 of the tile's 256 columns
    int t = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++t) {
      int tm, tn;
      tile_coords(p, tile, tm, tn);
      const int acc = t & 1;
      const uint32_t acc_ph = (t >> 1) & 1;
      if (!mbar_wait(&bars->acc_full[acc], acc_ph, abort_word, 405)) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * C::ACC1_COL + half * 128;
      const int row = tm * BM + quad * 32 + lane;
      const int col_base = tn * BN + half * 128;
      // The columns shared with the other accumulator are the last of accumulator 0 (the end of
      // its second half) and the first of accumulator 1 (the start of its first half): the half
      // that owns them reads those chunks first (accumulator 0: from the last chunk backwards)
      // and frees the columns.
      const bool owner = half == (acc == 0 ? 1 : 0);
      const bool backwards = owner && acc == 0;
      auto emit = [&](const uint32_t (&r)[32], int ch) {
        const int col0 = col_base + ch * 32;
        if (p.out_mx == 0) {
          if (row < p.M && col0 < p.N) store32(p, r, row, col0);
        } else if (col0 < p.N) {
          if (p.out_mx == 2) store32_nvfp4(p, r, row, col0);
          else store32_mx(p, r, row, col0);
        }
      };
      int i = 0;
      if (owner) {
        // every shared chunk is in registers before the first store: the next tile's first MMA
        // waits for this arrival, and a chunk's global stores would sit on that path
        uint32_t r0[32], r1[32];
        const int ch0 = backwards ? 3 : 0, ch1 = backwards ? 2 : 1;
        tmem_ld32(t_row + ch0 * 32, r0);
        if (C::OVL_CHUNKS == 2) tmem_ld32(t_row + ch1 * 32, r1);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->overlap_free);
        emit(r0, ch0);
        if (C::OVL_CHUNKS == 2) emit(r1, ch1);
        i = C::OVL_CHUNKS;
      }
#pragma unroll 1
      for (; i < 4; ++i) {
        const int ch = backwards ? 3 - i : i;
        uint32_t r[32];
        tmem_ld32(t_row + ch * 32, r);
        tmem_wait_ld();
        emit(r, ch);
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

// ------------------------------------------------------------------------------------------
// CTA-pair variant (cluster of two, tcgen05.mma.cta_group::2, 256 x 256 tiles).  The one-CTA
// kernel above is bound by the L2 -> SM operand traffic (48 KiB per stage per SM, measured
// 12.6 TB/s in aggregate); a pair splits B between its CTAs, so a stage is A (16 KiB) + half of B
// (16 KiB) per SM.  Each CTA also brings the scale tiles it needs into its own shared memory: A's
// for its own 128 rows and B's for all 256 columns (every CTA's tensor core multiplies its rows
// with the whole B).  They come through a tensor map over the scale buffer ([tiles * 2][256]
// bytes, a tile = two rows) because the cta_group::2 form of the load can credit the LEADER's
// barrier; tcgen05.cp.cta_group::2 then moves them into both CTAs' tensor memory, each from its
// own shared memory.  The rest is the protocol of the bf16 pair kernel: the leader issues every
// MMA and commits to both CTAs' barriers, the peer's epilogue warps arrive remotely.
template <int FP4>
struct PairCfg {
  static constexpr int SFT = Cfg<FP4>::SFT;
  static constexpr int HALF_B_BYTES = B_BYTES / 2;
  static constexpr int SF_OFF = A_BYTES + HALF_B_BYTES;
  static constexpr int SF_BYTES = 3 * SFT * SF_TILE;
  static constexpr int STAGE_BYTES = SF_OFF + (FP4 ? 6 : 2) * 1024;  // 34 / 38 KiB, 1024-aligned
  static constexpr int STAGES = FP4 ? 5 : 6;
  static constexpr int TX_BYTES = A_BYTES + HALF_B_BYTES + SF_BYTES;  // per CTA and stage
  static constexpr size_t SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 256;
  static_assert(SF_OFF + SF_BYTES <= STAGE_BYTES, "stage layout");
  static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KiB of shared memory a CTA can opt in to");
};

struct PairBarriers {
  uint64_t full[6];
  uint64_t empty[6];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t overlap_free;
  uint32_t tmem_base;
  int abort_word;
};

template <int FP4>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
    gemm_mx_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                        const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_sfa,
                        const __grid_constant__ CUtensorMap tmap_sfb, const Params p) {
  using C = Cfg<FP4>;
  using PC = PairCfg<FP4>;
  constexpr int STAGE_BYTES = PC::STAGE_BYTES;
  constexpr int NSTAGES = PC::STAGES;
  constexpr int SFT = C::SFT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  PairBarriers* bars = reinterpret_cast<PairBarriers*>(smem + NSTAGES * STAGE_BYTES);
  volatile int* abort_word = &bars->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->acc_full[i], 1);
      mbar_init(&bars->acc_empty[i], 2 * EPI_WARPS);  // both CTAs' epilogue warps; the leader's copy is used
    }
    mbar_init(&bars->overlap_free, 8);  // the four owning warps of each CTA
    bars->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_sfa);
    tma_prefetch_desc(&tmap_sfb);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < p.num_tiles && ok; tile += num_clusters) {
        int tm, tn;
        tile_coords(p, tile, tm, tn);
        const int m0 = tm * 2 * BM + static_cast<int>(rank) * BM;
        const int n0 = tn * BN + static_cast<int>(rank) * (BN / 2);
        // first scale-tile rows (a tile is two 256-byte rows of the scale tensor map)
        const int sfa_row = 2 * (tm * 2 + static_cast<int>(rank)) * p.sf_k_tiles;
        const int sfb_row = 2 * (tn * 2) * p.sf_k_tiles;
        for (int kt = 0; kt < p.k_tiles; ++kt, ++it) {
          const int s = it % NSTAGES;
          const uint32_t ph = (it / NSTAGES) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_word, 411)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          uint8_t* ssf = sa + PC::SF_OFF;
          // Bytes of both CTAs land on the leader's barrier.  Every load moves its whole box
          // (rows beyond a tensor are filled with zeros), so the count is a constant.
          if (rank == 0) mbar_arrive_expect_tx(&bars->full[s], 2 * PC::TX_BYTES);
          const uint32_t full_leader = mapa_shared(smem_u32(&bars->full[s]), 0);
          const int k0 = kt * BK;  // byte coordinate along K
          tma_load_3d_pair(sa, &tmap_a, full_leader, k0, m0, 0);
          tma_load_3d_pair(sb, &tmap_b, full_leader, k0, n0, 0);
          const int sf_k = 2 * kt * SFT;
          tma_load_3d_pair(ssf, &tmap_sfa, full_leader, 0, sfa_row + sf_k, 0);
          tma_load_3d_pair(ssf + SFT * SF_TILE, &tmap_sfb, full_leader, 0, sfb_row + sf_k, 0);
          tma_load_3d_pair(ssf + 2 * SFT * SF_TILE, &tmap_sfb, full_leader, 0,
                           sfb_row + 2 * p.sf_k_tiles + sf_k, 0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0 && elect_one()) {
      uint32_t it = 0;
      int t = 0;
      bool ok = true;
      const uint32_t sfa_t = tmem_base + C::SFA_COL, sfb_t = tmem_base + C::SFB_COL;
      for (int tile = cluster_id; tile < p.num_tiles && ok; tile += num_clusters, ++t) {
        const int acc = t & 1;
        const uint32_t acc_ph = (t >> 1) & 1;
        if (!mbar_wait(&bars->acc_empty[acc], acc_ph ^ 1, abort_word, 412)) break;
        if (t > 0 && !mbar_wait(&bars->overlap_free, (t - 1) & 1, abort_word, 413)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * C::ACC1_COL;
        for (int kt = 0; kt < p.k_tiles; ++kt, ++it) {
          const int s = it % NSTAGES;
          const uint32_t ph = (it / NSTAGES) & 1;
          if (!mbar_wait(&bars->full[s], ph, abort_word, 414)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          const uint32_t ssf = sa + PC::SF_OFF;
          const int kblocks = min(4, (p.K - kt * C::K_STAGE) / C::K_MMA);
          const int sf_tiles = FP4 ? kblocks : 1;
#pragma unroll
          for (int j = 0; j < SFT; ++j) {
            if (j < sf_tiles) {
              tmem_cp_32x128b_warpx4_pair(sfa_t + 4 * j, smem_desc_rows16(ssf + j * SF_TILE));
              tmem_cp_32x128b_warpx4_pair(sfb_t + 8 * j, smem_desc_rows16(ssf + (SFT + j) * SF_TILE));
              tmem_cp_32x128b_warpx4_pair(sfb_t + 8 * j + 4,
                                          smem_desc_rows16(ssf + (2 * SFT + j) * SF_TILE));
            }
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (k < kblocks) {
              const uint64_t da = smem_desc_sw128(sa + k * 32, 16, 1024);
              const uint64_t db = smem_desc_sw128(sb + k * 32, 16, 1024);
              if (FP4)
                umma_nvf4_ss_pair(d_tmem, da, db, make_idesc_nvf4(2 * BM, BN), sfa_t + 4 * k,
                                  sfb_t + 8 * k, (kt | k) != 0 ? 1u : 0u);
              else
                umma_mxf8_ss_pair(d_tmem, da, db, make_idesc_mxf8(2 * BM, BN, k, k), sfa_t, sfb_t,
                                  (kt | k) != 0 ? 1u : 0u);
            }
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
    const uint32_t ovl_leader = mapa_shared(smem_u32(&bars->overlap_free), 0);
    int t = 0;
    for (int tile = cluster_id; tile < p.num_tiles; tile += num_clusters, ++t) {
      int tm, tn;
      tile_coords(p, tile, tm, tn);
      const int acc = t & 1;
      const uint32_t acc_ph = (t >> 1) & 1;
      if (!mbar_wait(&bars->acc_full[acc], acc_ph, abort_word, 415)) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * C::ACC1_COL + half * 128;
      const int row = tm * 2 * BM + static_cast<int>(rank) * BM + quad * 32 + lane;
      const int col_base = tn * BN + half * 128;
      const bool owner = half == (acc == 0 ? 1 : 0);
      const bool backwards = owner && acc == 0;
      auto emit = [&](const uint32_t (&r)[32], int ch) {
        const int col0 = col_base + ch * 32;
        if (p.out_mx == 0) {
          if (row < p.M && col0 < p.N) store32(p, r, row, col0);
        } else if (col0 < p.N) {
          if (p.out_mx == 2) store32_nvfp4(p, r, row, col0);
          else store32_mx(p, r, row, col0);
        }
      };
      int i = 0;
      if (owner) {
        uint32_t r0[32], r1[32];
        const int ch0 = backwards ? 3 : 0, ch1 = backwards ? 2 : 1;
        tmem_ld32(t_row + ch0 * 32, r0);
        if (C::OVL_CHUNKS == 2) tmem_ld32(t_row + ch1 * 32, r1);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(ovl_leader);
        emit(r0, ch0);
        if (C::OVL_CHUNKS == 2) emit(r1, ch1);
        i = C::OVL_CHUNKS;
      }
#pragma unroll 1
      for (; i < 4; ++i) {
        const int ch = backwards ? 3 - i : i;
        uint32_t r[32];
        tmem_ld32(t_row + ch * 32, r);
        tmem_wait_ld();
        emit(r, ch);
      }
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

}  // namespace gemm_mx

static int32_t matmul_mx_run(const char* op, const cdl_mx_tensor* a, const cdl_mx_tensor* b,
                             const cdl_tensor* c, const cdl_tensor* d, const cdl_mx_tensor* d_mx,
                             float alpha, float beta, cudaStream_t stream,
                             const cdl_matmul_options* opts = nullptr) {
  using namespace gemm_mx;
  if (!a || !b || (!d && !d_mx)) return fail(CDL_ERR_INVALID, "%s: a, b and d are required", op);
  const int variant = opts ? opts->variant : CDL_GEMM_AUTO;
  if (variant < CDL_GEMM_AUTO || variant > CDL_GEMM_CTA_PAIR)
    return fail(CDL_ERR_INVALID, "%s: unknown kernel variant %d", op, variant);
  if ((a->format != CDL_MXFP8 && a->format != CDL_NVFP4) || b->format != a->format)
    return fail(CDL_ERR_UNSUPPORTED,
                "%s: both operands must be MXFP8, or both NVFP4 (mixed block-scaled formats are not "
                "accepted, as in the reference)", op);
  if (a->dim != CDL_MX_ROWWISE)
    return fail(CDL_ERR_INVALID,
                "%s: block-scaled A must have its blocks along the contraction dimension (rowwise)", op);
  if (b->dim != CDL_MX_COLWISE)
    return fail(CDL_ERR_INVALID,
                "%s: block-scaled B must have its blocks along the contraction dimension (colwise)", op);
  const long long M = a->rows, K = a->cols, N = b->cols;
  if (b->rows != K)
    return fail(CDL_ERR_INVALID, "%s: contraction dimensions differ: A is [%lld, %lld], B is [%lld, %lld]",
                op, M, K, static_cast<long long>(b->rows), N);
  CDL_CHECK(mx_check(op, "a", a, CDL_MX_ROWWISE, M, K));
  CDL_CHECK(mx_check(op, "b", b, CDL_MX_COLWISE, K, N));
  const bool fp4 = a->format == CDL_NVFP4;
  if (fp4 && K % 64 != 0)
    return fail(CDL_ERR_UNSUPPORTED, "%s: NVFP4 operands need K to be a multiple of 64 (got %lld)", op, K);
  if (d_mx) {
    if (d_mx->dim != CDL_MX_ROWWISE)  // (a colwise output arrives here transposed)
      return fail(CDL_ERR_INVALID, "%s: unknown block dimension of the output", op);
    if (d_mx->format != CDL_MXFP8 && d_mx->format != CDL_NVFP4)
      return fail(CDL_ERR_INVALID, "%s: unknown format of the block-scaled output", op);
    CDL_CHECK(mx_check(op, "d", d_mx, d_mx->dim, M, N));
    if (N % 32 != 0)
      return fail(CDL_ERR_UNSUPPORTED,
                  "%s: the block dimension of a block-scaled output must be a multiple of 32 (got %lld)",
                  op, N);
  } else {
    if (d->rank != 2 || d->shape[0] != M || d->shape[1] != N)
      return fail(CDL_ERR_INVALID, "%s: d must have shape [%lld, %lld]", op, M, N);
    if (d->dtype != CDL_BF16 && d->dtype != CDL_F32)
      return fail(CDL_ERR_UNSUPPORTED, "%s: the output must be f32 or bf16", op);
    if (N > 1 && d->stride[1] != 1)
      return fail(CDL_ERR_UNSUPPORTED, "%s: d must have contiguous rows", op);
    if ((reinterpret_cast<uintptr_t>(d->ptr) & (dtype_size(d->dtype) - 1)) != 0)
      return fail(CDL_ERR_INVALID, "%s: d is not aligned to its element size", op);
    if (c) {
      if (c->rank != 2 || c->shape[0] != M || c->shape[1] != N)
        return fail(CDL_ERR_INVALID, "%s: c must have shape [%lld, %lld]", op, M, N);
      if (c->dtype != CDL_BF16 && c->dtype != CDL_F32)
        return fail(CDL_ERR_UNSUPPORTED, "%s: c must be f32 or bf16", op);
      if (N > 1 && c->stride[1] != 1)
        return fail(CDL_ERR_UNSUPPORTED, "%s: c must have contiguous rows", op);
      if ((reinterpret_cast<uintptr_t>(c->ptr) & (dtype_size(c->dtype) - 1)) != 0)
        return fail(CDL_ERR_INVALID, "%s: c is not aligned to its element size", op);
    }
  }
  if (M == 0 || N == 0) return CDL_OK;
  if (K == 0) return fail(CDL_ERR_INVALID, "%s: K is zero", op);
  if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30))
    return fail(CDL_ERR_UNSUPPORTED, "%s: dimension too large", op);

  static std::once_flag attr_once[64];
  int dev = 0;
  CDL_CUDA(cudaGetDevice(&dev));
  cudaError_t attr_err = cudaSuccess;
  std::call_once(attr_once[dev & 63], [&] {
    attr_err = cudaFuncSetAttribute(gemm_mx_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(Cfg<0>::SMEM_BYTES));
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(gemm_mx_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(Cfg<1>::SMEM_BYTES));
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(gemm_mx_pair_kernel<0>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(PairCfg<0>::SMEM_BYTES));
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(gemm_mx_pair_kernel<1>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(PairCfg<1>::SMEM_BYTES));
  });
  if (attr_err != cudaSuccess)
    return fail(CDL_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(attr_err));

  Params p{};
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.num_m_tiles = static_cast<int>((M + BM - 1) / BM);
  p.num_n_tiles = static_cast<int>((N + BN - 1) / BN);
  p.num_tiles = p.num_m_tiles * p.num_n_tiles;
  const long long k_stage = fp4 ? Cfg<1>::K_STAGE : Cfg<0>::K_STAGE;
  const long long k_bytes = fp4 ? K / 2 : K;  // bytes of a row of values
  p.k_tiles = static_cast<int>((K + k_stage - 1) / k_stage);
  p.sf_k_tiles = static_cast<int>((K / (fp4 ? 16 : 32) + 3) / 4);
  p.sfa = static_cast<const uint8_t*>(a->scale_factors);
  p.sfb = static_cast<const uint8_t*>(b->scale_factors);
  if (d_mx) {
    p.out_mx = d_mx->format == CDL_NVFP4 ? 2 : 1;
    p.out_values = static_cast<uint8_t*>(d_mx->values);
    p.out_sf = static_cast<uint8_t*>(d_mx->scale_factors);
  } else {
    p.d = d->ptr;
    p.ldd = d->stride[0];
    p.out_f32 = d->dtype == CDL_F32;
    p.wide = (reinterpret_cast<uintptr_t>(d->ptr) & 31) == 0 &&
             (M == 1 || (d->stride[0] * dtype_size(d->dtype)) % 32 == 0);
    if (c && beta != 0.f) {
      p.c_mode = c->dtype == CDL_BF16 ? 1 : 2;
      p.c = c->ptr;
      p.ldc = c->stride[0];
      p.beta = beta;
      p.wide = p.wide && (reinterpret_cast<uintptr_t>(c->ptr) & 31) == 0 &&
               (M == 1 || (c->stride[0] * dtype_size(c->dtype)) % 32 == 0);
    }
  }
  p.alpha = alpha;
  p.status = device_status_ptr();
  if (!p.status) return fail(CDL_ERR_CUDA, "cannot resolve the device status word");

  CUtensorMap ta, tb;
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(k_bytes), static_cast<uint64_t>(M), 1};
    const uint64_t strides[3] = {1, static_cast<uint64_t>(k_bytes), static_cast<uint64_t>(k_bytes) * M};
    const uint32_t box[3] = {BK, BM, 1};
    CDL_CHECK(encode_tmap(&ta, a->values, TMAP_U8, 3, dims, strides, box, true));
  }
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(k_bytes), static_cast<uint64_t>(N), 1};
    const uint64_t strides[3] = {1, static_cast<uint64_t>(k_bytes), static_cast<uint64_t>(k_bytes) * N};
    const uint32_t box[3] = {BK, BN, 1};
    CDL_CHECK(encode_tmap(&tb, b->values, TMAP_U8, 3, dims, strides, box, true));
  }
  ProfileScope ps(PROF_GEMM, 2.0 * M * N * K, stream);
  if (variant == CDL_GEMM_AUTO ? M > BM : variant == CDL_GEMM_CTA_PAIR) {
    // CTA pairs over 256 x 256 tiles
    p.num_m_tiles = static_cast<int>((M + 2 * BM - 1) / (2 * BM));
    p.num_tiles = p.num_m_tiles * p.num_n_tiles;
    CUtensorMap tbh, tsa, tsb;
    {
      const uint64_t dims[3] = {static_cast<uint64_t>(k_bytes), static_cast<uint64_t>(N), 1};
      const uint64_t strides[3] = {1, static_cast<uint64_t>(k_bytes), static_cast<uint64_t>(k_bytes) * N};
      const uint32_t box[3] = {BK, BN / 2, 1};
      CDL_CHECK(encode_tmap(&tbh, b->values, TMAP_U8, 3, dims, strides, box, true));
    }
    const uint32_t sft = fp4 ? 4 : 1;
    auto sf_map = [&](CUtensorMap* out, const void* base, long long outer) -> int32_t {
      // the scale buffer as rows of 256 bytes: tile i = rows 2i, 2i + 1
      const uint64_t tiles = static_cast<uint64_t>((outer + 127) / 128) * p.sf_k_tiles;
      const uint64_t dims[3] = {256, 2 * tiles, 1};
      const uint64_t strides[3] = {1, 256, 512 * tiles};
      const uint32_t box[3] = {256, 2 * sft, 1};
      return encode_tmap(out, base, TMAP_U8, 3, dims, strides, box, false);
    };
    CDL_CHECK(sf_map(&tsa, a->scale_factors, M));
    CDL_CHECK(sf_map(&tsb, b->scale_factors, N));
    int grid = 2 * p.num_tiles < sm_count() ? 2 * p.num_tiles : sm_count();
    grid &= ~1;
    if (fp4)
      gemm_mx_pair_kernel<1><<<grid, THREADS, PairCfg<1>::SMEM_BYTES, stream>>>(ta, tbh, tsa, tsb, p);
    else
      gemm_mx_pair_kernel<0><<<grid, THREADS, PairCfg<0>::SMEM_BYTES, stream>>>(ta, tbh, tsa, tsb, p);
  } else {
    const int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
    if (fp4) gemm_mx_kernel<1><<<grid, THREADS, Cfg<1>::SMEM_BYTES, stream>>>(ta, tb, p);
    else gemm_mx_kernel<0><<<grid, THREADS, Cfg<0>::SMEM_BYTES, stream>>>(ta, tb, p);
  }
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

int32_t matmul_mx_execute(const cdl_mx_tensor* a, const cdl_mx_tensor* b, const cdl_tensor* c,
                          const cdl_tensor* d, float alpha, float beta, cudaStream_t stream,
                          const cdl_matmul_options* opts) {
  return matmul_mx_run("matmul (block-scaled operands)", a, b, c, d, nullptr, alpha, beta, stream,
                       opts);
}

int32_t matmul_mx_out_execute(const cdl_mx_tensor* a, const cdl_mx_tensor* b, const cdl_mx_tensor* d,
                              float alpha, cudaStream_t stream) {
  const char* op = "matmul (block-scaled operands and output)";
  if (!d) return fail(CDL_ERR_INVALID, "%s: d is required", op);
  if (a && b && d->dim == CDL_MX_COLWISE && a->dim == CDL_MX_ROWWISE && b->dim == CDL_MX_COLWISE) {
    // A colwise D is a rowwise D^T = B^T . A^T, and the buffers already are what that product
    // needs: B's values are the rowwise [N, K] matrix, A's values are the colwise [K, M] one, D's
    // values are the packed [N, M] transpose with blocks along M.  So the colwise output runs as
    // the rowwise epilogue (a thread's 32 columns are one block) of the swapped problem.
    cdl_mx_tensor at = *b, bt = *a, dt = *d;
    at.dim = CDL_MX_ROWWISE; at.rows = b->cols; at.cols = b->rows;
    bt.dim = CDL_MX_COLWISE; bt.rows = a->cols; bt.cols = a->rows;
    dt.dim = CDL_MX_ROWWISE; dt.rows = d->cols; dt.cols = d->rows;
    if (d->rows != a->rows || d->cols != b->cols)
      return fail(CDL_ERR_INVALID, "%s: d must have shape [%lld, %lld]", op,
                  static_cast<long long>(a->rows), static_cast<long long>(b->cols));
    return matmul_mx_run(op, &at, &bt, nullptr, nullptr, &dt, alpha, 0.f, stream);
  }
  return matmul_mx_run(op, a, b, nullptr, nullptr, d, alpha, 0.f, stream);
}

}  // namespace cdl

extern "C" {

int32_t cdl_b200_matmul_mx(const cdl_mx_tensor* a, const cdl_mx_tensor* b, const cdl_tensor* c,
                           const cdl_tensor* d, float alpha, float beta, cdl_stream stream) {
  return cdl::matmul_mx_execute(a, b, c, d, alpha, beta, static_cast<cudaStream_t>(stream));
}

int32_t cdl_b200_matmul_mx_opt(const cdl_mx_tensor* a, const cdl_mx_tensor* b, const cdl_tensor* c,
                               const cdl_tensor* d, float alpha, float beta,
                               const cdl_matmul_options* options, cdl_stream stream) {
  return cdl::matmul_mx_execute(a, b, c, d, alpha, beta, static_cast<cudaStream_t>(stream), options);
}

int32_t cdl_b200_matmul_mx_out(const cdl_mx_tensor* a, const cdl_mx_tensor* b, const cdl_mx_tensor* d,
                               float alpha, cdl_stream stream) {
  return cdl::matmul_mx_out_execute(a, b, d, alpha, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
