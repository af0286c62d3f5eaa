// RMSNorm forward and backward: HBM-bound streaming kernels.
//
// Forward follows NormFwd / SpecializedExecutor of the reference
// (crates/cleandl/src/execgraph/ops/norm/mod.rs:72-85, ops/norm/specialized.rs:116-200; kernel
// crates/cleandl-specialized-kernels/src/kernels/norm/forward.rs:569-657):
//     r_i = rsqrt(mean_j x_ij^2 + eps);   y_ij = bf16((f32(x_ij) * r_i) * scale_j + bias_j)
// Backward has no implementation in the reference tree, only call sites
// (crates/sky-1/src/training/model/decoder.rs:599-607, 684-692); the math is the derivative of
// the forward above.
//
// Design: one warp owns one row at a time.  A lane holds 8 consecutive bf16 (one 128-bit
// access) of every 256-column stripe, so a warp's access is a fully coalesced 512 B; the whole
// row stays in registers between the reduction and the scaling pass, which makes both kernels
// single-pass over HBM.  Row reductions are five shuffle steps; no shared memory or block
// barrier is on the critical path.
#include "host.h"
#include "ops.h"
#include "ptx.cuh"

#include <stdlib.h>
#include <string.h>

#include <mutex>

namespace cdl {
namespace norm {

constexpr int FWD_THREADS = 256;
constexpr int BWD_THREADS = 128;
constexpr int BWD_BLOCKS_PER_SM = 3;
constexpr int MAX_PARTIALS = 1024;  // upper bound on backward grid size (scratch sizing)

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  f[0] = bf16_lo(q.x); f[1] = bf16_hi(q.x); f[2] = bf16_lo(q.y); f[3] = bf16_hi(q.y);
  f[4] = bf16_lo(q.z); f[5] = bf16_hi(q.z); f[6] = bf16_lo(q.w); f[7] = bf16_hi(q.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 q;
  q.x = pack_bf16x2(f[0], f[1]); q.y = pack_bf16x2(f[2], f[3]);
  q.z = pack_bf16x2(f[4], f[5]); q.w = pack_bf16x2(f[6], f[7]);
  return q;
}

// Adds (or, for the first warp, stores) a warp's per-lane dscale sums into the CTA's row in shared
// memory: 128-bit accesses, so a lane's 8 consecutive floats cost two conflict-free transactions.
template <int NCH>
__device__ __forceinline__ void fold_dscale(float* s_part, const float (&acc)[NCH * 8], int cols, int lane,
                                            bool first) {
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int col = c * 256 + lane * 8;
    if (col < cols) {
      float4* dst = reinterpret_cast<float4*>(s_part + col);
      float4 lo = make_float4(acc[c * 8 + 0], acc[c * 8 + 1], acc[c * 8 + 2], acc[c * 8 + 3]);
      float4 hi = make_float4(acc[c * 8 + 4], acc[c * 8 + 5], acc[c * 8 + 6], acc[c * 8 + 7]);
      if (!first) {
        const float4 a = dst[0], b = dst[1];
        lo.x += a.x; lo.y += a.y; lo.z += a.z; lo.w += a.w;
        hi.x += b.x; hi.y += b.y; hi.z += b.z; hi.w += b.w;
      }
      dst[0] = lo;
      dst[1] = hi;
    }
  }
}

// NCH = number of 256-column stripes a row spans (cols <= 256 * NCH).
template <int NCH>
__global__ void __launch_bounds__(FWD_THREADS, NCH <= 8 ? 4 : 1)
    rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                       const __nv_bfloat16* __restrict__ scale,
                       const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y,
                       long long ldy, float* __restrict__ r_inv, long long r_inv_stride, int rows,
                       int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = FWD_THREADS / 32;
  const long long warp_global = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
  const long long warp_stride = static_cast<long long>(gridDim.x) * warps_per_block;
  const float inv_cols = 1.0f / static_cast<float>(cols);
  grid_dep_wait();
  grid_dep_launch();

  for (long long row = warp_global; row < rows; row += warp_stride) {
    const __nv_bfloat16* xr = x + row * ldx;
    uint4 v[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = c * 256 + lane * 8;
      v[c] = col < cols ? ld_nc_v4(xr + col) : make_uint4(0, 0, 0, 0);
    }
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      float f[8];
      unpack8(v[c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss * inv_cols + eps);
    if (r_inv != nullptr && lane == 0) r_inv[row * r_inv_stride] = r;
    __nv_bfloat16* yr = y + row * ldy;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = c * 256 + lane * 8;
      if (col < cols) {
        float f[8];
        unpack8(v[c], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] *= r;
        if (scale != nullptr) {
          float s[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(scale + col)), s);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] *= s[j];
        }
        if (bias != nullptr) {
          float b[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(bias + col)), b);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] += b[j];
        }
        st_cs_v4(yr + col, pack8(f));
      }
    }
  }
}

// LayerNorm forward (NormType::LayerNorm of the reference, crates/cleandl/src/execgraph/ops/norm/
// mod.rs:23-30; reference tests/norm.rs:97-130): mean_i = mean_j x_ij, r_i = rsqrt(mean_j
// (x_ij - mean_i)^2 + eps), y_ij = bf16((x_ij - mean_i) * r_i * scale_j + bias_j); optional mean
// and r_inv outputs.  Same shape as the RMSNorm forward: a warp per row, the row in registers, the
// variance taken around the mean in a second pass over the registers (no E[x^2] - mean^2).
template <int NCH>
__global__ void __launch_bounds__(FWD_THREADS, NCH <= 4 ? 4 : NCH <= 8 ? 3 : 1)
    layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                         const __nv_bfloat16* __restrict__ scale,
                         const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y,
                         long long ldy, float* __restrict__ mean_out, long long mean_stride,
                         float* __restrict__ r_inv, long long r_inv_stride, int rows, int cols,
                         float eps) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = FWD_THREADS / 32;
  const long long warp_global = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
  const long long warp_stride = static_cast<long long>(gridDim.x) * warps_per_block;
  const float inv_cols = 1.0f / static_cast<float>(cols);
  grid_dep_wait();
  grid_dep_launch();
  for (long long row = warp_global; row < rows; row += warp_stride) {
    const __nv_bfloat16* xr = x + row * ldx;
    uint4 v[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = c * 256 + lane * 8;
      v[c] = col < cols ? ld_nc_v4(xr + col) : make_uint4(0, 0, 0, 0);
    }
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      float f[8];
      unpack8(v[c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += f[j];
    }
    const float mean = warp_sum(sum) * inv_cols;
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      if (c * 256 + lane * 8 < cols) {
        float f[8];
        unpack8(v[c], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j] - mean, f[j] - mean, ss);
      }
    }
    const float r = rsqrtf(warp_sum(ss) * inv_cols + eps);
    if (lane == 0) {
      if (mean_out != nullptr) mean_out[row * mean_stride] = mean;
      if (r_inv != nullptr) r_inv[row * r_inv_stride] = r;
    }
    __nv_bfloat16* yr = y + row * ldy;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = c * 256 + lane * 8;
      if (col < cols) {
        float f[8];
        unpack8(v[c], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = (f[j] - mean) * r;
        if (scale != nullptr) {
          float sc[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(scale + col)), sc);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] *= sc[j];
        }
        if (bias != nullptr) {
          float b[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(bias + col)), b);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] += b[j];
        }
        st_cs_v4(yr + col, pack8(f));
      }
    }
  }
}

// Pipelined forward: one persistent CTA per SM; warp 8 streams whole rows into a shared-memory
// ring with 1-D bulk copies (up to 128 KiB in flight per SM, independent of how fast the rows
// are consumed), warps 0-7 each take every 8th row of the CTA's slice out of the ring, reduce
// it with shuffles and store y straight from registers.
constexpr int PIPE_CONSUMERS = 8;
constexpr int PIPE_THREADS = (PIPE_CONSUMERS + 1) * 32;
constexpr int PIPE_RING_BYTES = 128 * 1024;

template <int NCH>
__global__ void __launch_bounds__(PIPE_THREADS, 1)
    rmsnorm_fwd_pipe_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                            const __nv_bfloat16* __restrict__ scale,
                            const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y,
                            long long ldy, float* __restrict__ r_inv, long long r_inv_stride,
                            int rows, int cols, float eps, int stages, int* status) {
  extern __shared__ __align__(128) uint8_t ring[];
  const int row_bytes = cols * 2;
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(stages) * row_bytes);
  uint64_t* empty = full + stages;
  volatile int* abort_word = reinterpret_cast<volatile int*>(empty + stages);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // contiguous slice of rows for this CTA
  const int per = (rows + gridDim.x - 1) / gridDim.x;
  const int row_begin = min(rows, static_cast<int>(blockIdx.x) * per);
  const int row_end = min(rows, row_begin + per);
  const int n = row_end - row_begin;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    *abort_word = 0;
    fence_mbar_init();
  }
  __syncthreads();
  grid_dep_wait();
  grid_dep_launch();
  if (warp == PIPE_CONSUMERS) {
    if (lane == 0) {
      for (int i = 0; i < n; ++i) {
        const int s = i % stages;
        const uint32_t ph = ((i / stages) & 1) ^ 1;
        if (!mbar_wait(&empty[s], ph, abort_word, 701)) break;
        mbar_arrive_expect_tx(&full[s], row_bytes);
        bulk_load_1d(ring + static_cast<size_t>(s) * row_bytes, x + (row_begin + i) * ldx, row_bytes,
                     &full[s]);
      }
    }
  } else {
    const float inv_cols = 1.0f / static_cast<float>(cols);
    // the scale for this lane's columns stays in registers for the whole slice
    uint4 sc[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = c * 256 + lane * 8;
      sc[c] = (scale != nullptr && col < cols) ? __ldg(reinterpret_cast<const uint4*>(scale + col))
                                               : make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
    }
    for (int i = warp; i < n; i += PIPE_CONSUMERS) {
      const int s = i % stages;
      const uint32_t ph = (i / stages) & 1;
      // (see the backward's consumer: the previous use of the stage must have been released
      // before a parity wait on `full` is unambiguous)
      if (i >= stages && !mbar_wait(&empty[s], ph ^ 1, abort_word, 703)) break;
      if (!mbar_wait(&full[s], ph, abort_word, 702)) break;
      const uint8_t* src = ring + static_cast<size_t>(s) * row_bytes;
      uint4 v[NCH];
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col = c * 256 + lane * 8;
        v[c] = col < cols ? *reinterpret_cast<const uint4*>(src + col * 2) : make_uint4(0, 0, 0, 0);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);  // the row is in registers: the slot can be refilled
      float ss = 0.f;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        float f[8];
        unpack8(v[c], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
      }
      ss = warp_sum(ss);
      const float r = rsqrtf(ss * inv_cols + eps);
      const long long row = row_begin + i;
      if (r_inv != nullptr && lane == 0) r_inv[row * r_inv_stride] = r;
      __nv_bfloat16* yr = y + row * ldy;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col = c * 256 + lane * 8;
        if (col < cols) {
          float f[8], sf[8];
          unpack8(v[c], f);
          unpack8(sc[c], sf);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = (f[j] * r) * sf[j];
          if (bias != nullptr) {
            float bf[8];
            unpack8(__ldg(reinterpret_cast<const uint4*>(bias + col)), bf);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] += bf[j];
          }
          st_cs_v4(yr + col, pack8(f));
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && *abort_word != 0) atomicExch(status, *abort_word);
}

// Backward.  Every warp walks rows (grid-stride), keeps per-lane partial sums of
// dscale for its columns in registers when DSCALE is set, and at the end the block folds its
// warps' partials through shared memory into one row of `partials` [gridDim.x, cols].
template <int NCH, bool DSCALE>
__global__ void __launch_bounds__(BWD_THREADS, BWD_BLOCKS_PER_SM)
    rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                       const __nv_bfloat16* __restrict__ dy, long long lddy,
                       const __nv_bfloat16* __restrict__ res, long long ldres,
                       const __nv_bfloat16* __restrict__ scale, const float* __restrict__ r_inv,
                       long long r_inv_stride, __nv_bfloat16* __restrict__ dx, long long lddx,
                       float* __restrict__ partials, int rows, int cols) {
  extern __shared__ float s_part[];  // [cols] when DSCALE
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps_per_block = BWD_THREADS / 32;
  const long long warp_global = static_cast<long long>(blockIdx.x) * warps_per_block + warp;
  const long long warp_stride = static_cast<long long>(gridDim.x) * warps_per_block;
  const float inv_cols = 1.0f / static_cast<float>(cols);

  float acc[DSCALE ? NCH * 8 : 1];
#pragma unroll
  for (int i = 0; i < (DSCALE ? NCH * 8 : 1); ++i) acc[i] = 0.f;
  grid_dep_wait();
  grid_dep_launch();

  for (long long row = warp_global; row < rows; row += warp_stride) {
    const __nv_bfloat16* xr = x + row * ldx;
    const __nv_bfloat16* dyr = dy + row * lddy;
    uint4 vx[NCH], vd[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = c * 256 + lane * 8;
      const bool in = col < cols;
      vx[c] = in ? ld_nc_v4(xr + col) : make_uint4(0, 0, 0, 0);
      vd[c] = in ? ld_nc_v4(dyr + col) : make_uint4(0, 0, 0, 0);
    }
    const float r = r_inv[row * r_inv_stride];
    // g = dy * scale (kept in vd's place as f32 is too large: recompute in the second pass).
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = c * 256 + lane * 8;
      if (col < cols) {
        float fx[8], fd[8], fs[8];
        unpack8(vx[c], fx);
        unpack8(vd[c], fd);
        unpack8(__ldg(reinterpret_cast<const uint4*>(scale + col)), fs);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dot = fmaf(fd[j] * fs[j], fx[j], dot);
          if (DSCALE) acc[c * 8 + j] = fmaf(fd[j] * fx[j], r, acc[c * 8 + j]);
        }
      }
    }
    dot = warp_sum(dot);
    const float k = r * r * (dot * inv_cols);  // dx = r * (g - x * k)
    __nv_bfloat16* dxr = dx + row * lddx;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = c * 256 + lane * 8;
      if (col < cols) {
        float fx[8], fd[8], fs[8], o[8];
        unpack8(vx[c], fx);
        unpack8(vd[c], fd);
        unpack8(__ldg(reinterpret_cast<const uint4*>(scale + col)), fs);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r * (fd[j] * fs[j] - fx[j] * k);
        if (res != nullptr) {
          float fr[8];
          unpack8(ld_nc_v4(res + row * ldres + col), fr);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += fr[j];
        }
        st_cs_v4(dxr + col, pack8(o));
      }
    }
  }

  if constexpr (DSCALE) {
    // Fold the block's warps one after another (fixed order: deterministic).
    for (int w = 0; w < warps_per_block; ++w) {
      if (warp == w) fold_dscale<NCH>(s_part, acc, cols, lane, w == 0);
      __syncthreads();
    }
    float* out = partials + static_cast<long long>(blockIdx.x) * cols;
    for (int i = threadIdx.x; i < cols; i += BWD_THREADS) out[i] = s_part[i];
  }
}

// Pipelined backward (cols <= 2048): like the pipelined forward, warp 8 streams the x, dy (and
// residual) rows of the CTA's slice into a shared-memory ring with bulk copies; warps 0-7 take
// every 8th row, keep their partial dscale sums in registers, and the CTA writes one partial
// row at the end (folded through the ring's memory once the pipeline has drained).
// The backward's ring is fed by two producer warps (one lane each): the lane that issues a row's
// copies spends ~800 clk per row on the barrier wait, the expect-tx arrival and three bulk copies
// (measured: the kernel's time per row followed that lane, not the memory system), more than the
// ~550 clk a row may take at the measured copy bandwidth.  Producer p takes the rows i with
// i % 2 == p; with an even number of stages it also owns the stages s with s % 2 == p.
constexpr int BWD_PIPE_PRODUCERS = 2;
constexpr int BWD_PIPE_THREADS = (PIPE_CONSUMERS + BWD_PIPE_PRODUCERS) * 32;

template <int NCH>
__global__ void __launch_bounds__(BWD_PIPE_THREADS, 1)
    rmsnorm_bwd_pipe_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                            const __nv_bfloat16* __restrict__ dy, long long lddy,
                            const __nv_bfloat16* __restrict__ res, long long ldres,
                            const __nv_bfloat16* __restrict__ scale, const float* __restrict__ r_inv,
                            long long r_inv_stride, __nv_bfloat16* __restrict__ dx, long long lddx,
                            float* __restrict__ partials, int rows, int cols, int stages, int* status) {
  extern __shared__ __align__(128) uint8_t ring[];
  const int row_bytes = cols * 2;
  const int ntens = res != nullptr ? 3 : 2;
  const int stage_bytes = ntens * row_bytes;
  uint8_t* s_scale = ring + static_cast<size_t>(stages) * stage_bytes;  // bf16 [cols]
  uint64_t* full = reinterpret_cast<uint64_t*>(s_scale + row_bytes);
  uint64_t* empty = full + stages;
  volatile int* abort_word = reinterpret_cast<volatile int*>(empty + stages);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = (rows + gridDim.x - 1) / gridDim.x;
  const int row_begin = min(rows, static_cast<int>(blockIdx.x) * per);
  const int row_end = min(rows, row_begin + per);
  const int n = row_end - row_begin;
  const int producer = (warp >= PIPE_CONSUMERS && lane == 0) ? warp - PIPE_CONSUMERS : -1;
  auto load_row = [&](int i, int s) {
    uint8_t* dst = ring + static_cast<size_t>(s) * stage_bytes;
    const long long row = row_begin + i;
    mbar_arrive_expect_tx(&full[s], stage_bytes);
    bulk_load_1d(dst, x + row * ldx, row_bytes, &full[s]);
    bulk_load_1d(dst + row_bytes, dy + row * lddy, row_bytes, &full[s]);
    if (ntens == 3) bulk_load_1d(dst + 2 * row_bytes, res + row * ldres, row_bytes, &full[s]);
  };
  // Each producer lane sets up the barriers of its own stages and fills them once before the CTA
  // synchronises: the first rows are on their way while the other warps fetch the scale.
  if (threadIdx.x == 0) *abort_word = 0;
  if (producer >= 0) {
    for (int s = producer; s < stages; s += BWD_PIPE_PRODUCERS) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    fence_mbar_init();
  }
  grid_dep_wait();
  grid_dep_launch();
  const int first_round = min(n, stages);
  if (producer >= 0)
    for (int i = producer; i < first_round; i += BWD_PIPE_PRODUCERS) load_row(i, i);
  for (int i = threadIdx.x * 8; i < cols; i += BWD_PIPE_THREADS * 8)
    *reinterpret_cast<uint4*>(s_scale + i * 2) = __ldg(reinterpret_cast<const uint4*>(scale + i));
  __syncthreads();

  float acc[NCH * 8];
#pragma unroll
  for (int i = 0; i < NCH * 8; ++i) acc[i] = 0.f;

  if (warp >= PIPE_CONSUMERS) {
    if (producer >= 0) {
      // stage and phase advance without divisions: the stage steps by 2 and wraps (stages is even)
      int s = producer;
      uint32_t ph = 0;  // phase of `empty` that frees the stage for its second use
      for (int i = first_round + ((first_round ^ producer) & 1); i < n; i += BWD_PIPE_PRODUCERS) {
        // first_round == stages here (n > stages), so row i goes to stage i % stages
        if (!mbar_wait(&empty[s], ph, abort_word, 711)) break;
        load_row(i, s);
        s += BWD_PIPE_PRODUCERS;
        if (s >= stages) {
          s -= stages;
          ph ^= 1;
        }
      }
    }
  } else {
    const float inv_cols = 1.0f / static_cast<float>(cols);
    for (int i = warp; i < n; i += PIPE_CONSUMERS) {
      const int s = i % stages;
      const uint32_t ph = (i / stages) & 1;
      const long long row = row_begin + i;
      const float r = r_inv[row * r_inv_stride];  // on its way while the row's tiles land
      // The consumer warps run independently, so this warp can reach the stage's next use before
      // another warp has taken the previous one (or before that one's copies have landed): a
      // parity wait on `full` would then pass on the phase before last.  The stage's previous
      // use has been released (`empty`) only after its data arrived and was read, and that
      // release cannot be two phases behind (this warp's previous row was loaded after it).
      if (i >= stages && !mbar_wait(&empty[s], ph ^ 1, abort_word, 713)) break;
      if (!mbar_wait(&full[s], ph, abort_word, 712)) break;
      const uint8_t* src = ring + static_cast<size_t>(s) * stage_bytes;
      uint4 vx[NCH], vd[NCH];
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col = c * 256 + lane * 8;
        const bool in = col < cols;
        vx[c] = in ? *reinterpret_cast<const uint4*>(src + col * 2) : make_uint4(0, 0, 0, 0);
        vd[c] = in ? *reinterpret_cast<const uint4*>(src + row_bytes + col * 2) : make_uint4(0, 0, 0, 0);
      }
      float dot = 0.f;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col = c * 256 + lane * 8;
        if (col < cols) {
          float fx[8], fd[8], fs[8];
          unpack8(vx[c], fx);
          unpack8(vd[c], fd);
          unpack8(*reinterpret_cast<const uint4*>(s_scale + col * 2), fs);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            dot = fmaf(fd[j] * fs[j], fx[j], dot);
            acc[c * 8 + j] = fmaf(fd[j] * fx[j], r, acc[c * 8 + j]);
          }
        }
      }
      dot = warp_sum(dot);
      const float k = r * r * (dot * inv_cols);  // dx = r * (g - x * k)
      __nv_bfloat16* dxr = dx + row * lddx;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col = c * 256 + lane * 8;
        if (col < cols) {
          float fx[8], fd[8], fs[8], o[8];
          unpack8(vx[c], fx);
          unpack8(vd[c], fd);
          unpack8(*reinterpret_cast<const uint4*>(s_scale + col * 2), fs);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = r * (fd[j] * fs[j] - fx[j] * k);
          if (ntens == 3) {
            float fr[8];
            unpack8(*reinterpret_cast<const uint4*>(src + 2 * row_bytes + col * 2), fr);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] += fr[j];
          }
          st_cs_v4(dxr + col, pack8(o));
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
  }
  // Fold the 8 consumer warps' partial sums in warp order through the (now idle) ring.
  __syncthreads();
  float* s_part = reinterpret_cast<float*>(ring);
  for (int w = 0; w < PIPE_CONSUMERS; ++w) {
    if (warp == w) fold_dscale<NCH>(s_part, acc, cols, lane, w == 0);
    __syncthreads();
  }
  float* out = partials + static_cast<long long>(blockIdx.x) * cols;
  for (int i = threadIdx.x; i < cols; i += BWD_PIPE_THREADS) out[i] = s_part[i];
  if (threadIdx.x == 0 && *abort_word != 0) atomicExch(status, *abort_word);
}

// dscale partials for rows too wide for register accumulators: block (bx, by) sums rows
// by, by + gridDim.y, ... for 128 columns.
__global__ void __launch_bounds__(128)
    dscale_cols_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                       const __nv_bfloat16* __restrict__ dy, long long lddy,
                       const float* __restrict__ r_inv, long long r_inv_stride,
                       float* __restrict__ partials, int rows, int cols) {
  const int col = blockIdx.x * 128 + threadIdx.x;
  grid_dep_wait();
  grid_dep_launch();
  if (col >= cols) return;
  float acc = 0.f;
  for (long long row = blockIdx.y; row < rows; row += gridDim.y)
    acc = fmaf(__bfloat162float(dy[row * lddy + col]) * __bfloat162float(x[row * ldx + col]),
               r_inv[row * r_inv_stride], acc);
  partials[static_cast<long long>(blockIdx.y) * cols + col] = acc;
}

// dscale[j] += sum_b partials[b][j], summed in a fixed order.  The partial rows were written a
// moment ago (L2 hits), so the kernel is bound by load round trips, not bandwidth: a CTA owns 16
// columns and spreads the rows over 32 groups of threads, each thread keeps four loads in flight,
// and the 32 group sums are folded through shared memory in group order.  (With 8 groups and two
// loads in flight the 444 partial rows of a [16384, 2048] backward took ~8 us of a 48 us call.)
constexpr int FIN_COLS = 16, FIN_GROUPS = 32;
__global__ void __launch_bounds__(FIN_COLS * FIN_GROUPS)
    dscale_finalize_kernel(const float* __restrict__ partials, int num_partials, int cols,
                           float* __restrict__ dscale, long long dscale_stride) {
  __shared__ float s_sum[FIN_GROUPS][FIN_COLS];
  const int cx = threadIdx.x % FIN_COLS, rg = threadIdx.x / FIN_COLS;
  const int col = blockIdx.x * FIN_COLS + cx;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  grid_dep_wait();
  grid_dep_launch();
  if (col < cols) {
    const float* p = partials + col;
    int b = rg;
    for (; b + 3 * FIN_GROUPS < num_partials; b += 4 * FIN_GROUPS) {
      s0 += p[static_cast<long long>(b) * cols];
      s1 += p[static_cast<long long>(b + FIN_GROUPS) * cols];
      s2 += p[static_cast<long long>(b + 2 * FIN_GROUPS) * cols];
      s3 += p[static_cast<long long>(b + 3 * FIN_GROUPS) * cols];
    }
    for (; b < num_partials; b += FIN_GROUPS) s0 += p[static_cast<long long>(b) * cols];
  }
  s_sum[rg][cx] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (rg == 0 && col < cols) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < FIN_GROUPS; ++w) t += s_sum[w][cx];
    dscale[col * dscale_stride] += t;
  }
}

static int32_t check_rows(const char* op, const char* name, const cdl_tensor* t, long long rows,
                          long long cols) {
  if (t->rank != 2 || t->shape[0] != rows || t->shape[1] != cols)
    return fail(CDL_ERR_INVALID, "%s: %s must be a 2D tensor of shape [%lld, %lld]", op, name, rows,
                cols);
  if (t->dtype != CDL_BF16) return fail(CDL_ERR_UNSUPPORTED, "%s: %s must be bf16", op, name);
  if (cols > 1 && t->stride[1] != 1)
    return fail(CDL_ERR_UNSUPPORTED, "%s: %s must have packed rows (contiguous columns)", op, name);
  if ((reinterpret_cast<uintptr_t>(t->ptr) & 15) != 0 || (rows > 1 && t->stride[0] % 8 != 0))
    return fail(CDL_ERR_UNSUPPORTED, "%s: %s must be 16-byte aligned (pointer and row stride)", op,
                name);
  return CDL_OK;
}

static int32_t check_vec(const char* op, const char* name, const cdl_tensor* t, long long n,
                         int32_t dtype, bool need_contig) {
  if (t->rank != 1 || t->shape[0] != n)
    return fail(CDL_ERR_INVALID, "%s: %s must have shape [%lld]", op, name, n);
  if (t->dtype != dtype)
    return fail(CDL_ERR_UNSUPPORTED, "%s: %s must be %s", op, name, dtype_name(dtype));
  if (need_contig && (t->stride[0] != 1 || (reinterpret_cast<uintptr_t>(t->ptr) & 15) != 0))
    return fail(CDL_ERR_UNSUPPORTED, "%s: %s must be contiguous and 16-byte aligned", op, name);
  return CDL_OK;
}

// Whether the vectorised kernels take these operands; everything else goes to the general kernel
// (norm_general.cu), which also reports the invalid ones.
static bool fast_rows(const cdl_tensor* t, long long rows, long long cols) {
  return t->rank == 2 && t->shape[0] == rows && t->shape[1] == cols && t->dtype == CDL_BF16 &&
         (cols <= 1 || t->stride[1] == 1) && (reinterpret_cast<uintptr_t>(t->ptr) & 15) == 0 &&
         (rows <= 1 || t->stride[0] % 8 == 0);
}
static bool fast_vec(const cdl_tensor* t, long long n) {
  return t->rank == 1 && t->shape[0] == n && t->dtype == CDL_BF16 && t->stride[0] == 1 &&
         (reinterpret_cast<uintptr_t>(t->ptr) & 15) == 0;
}
static bool fast_norm_operands(const cdl_tensor* x, const cdl_tensor* scale, const cdl_tensor* bias,
                               const cdl_tensor* y) {
  if (x->rank != 2) return false;
  const long long rows = x->shape[0], cols = x->shape[1];
  return cols % 8 == 0 && cols <= 8192 && fast_rows(x, rows, cols) && fast_rows(y, rows, cols) &&
         (!scale || fast_vec(scale, cols)) && (!bias || fast_vec(bias, cols));
}

template <int NCH>
static void launch_fwd(const cdl_tensor* x, const cdl_tensor* scale, const cdl_tensor* bias,
                       float eps, const cdl_tensor* y, const cdl_tensor* r_inv, int rows, int cols,
                       int variant, cudaStream_t stream) {
  int* status = device_status_ptr();
  if constexpr (NCH <= 8) {
  // The pipelined forward measured slower than the warp-per-row one, so only an explicit request
  // selects it.
  if (status != nullptr && rows >= 2 * sm_count() && variant == CDL_NORM_PIPELINED) {
    const int row_bytes = cols * 2;
    int stages = PIPE_RING_BYTES / row_bytes;
    if (stages > 64) stages = 64;
    const size_t smem = static_cast<size_t>(stages) * row_bytes + 2 * stages * sizeof(uint64_t) + 16;
    static std::once_flag once[64];
    int dev = 0;
    cudaGetDevice(&dev);
    std::call_once(once[dev & 63], [&] {
      cudaFuncSetAttribute(rmsnorm_fwd_pipe_kernel<NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           PIPE_RING_BYTES + 2 * 64 * static_cast<int>(sizeof(uint64_t)) + 16);
    });
    launch_pdl(rmsnorm_fwd_pipe_kernel<NCH>, dim3(sm_count()), dim3(PIPE_THREADS), smem, stream,
        static_cast<const __nv_bfloat16*>(x->ptr), x->stride[0],
        scale ? static_cast<const __nv_bfloat16*>(scale->ptr) : nullptr,
        bias ? static_cast<const __nv_bfloat16*>(bias->ptr) : nullptr,
        static_cast<__nv_bfloat16*>(y->ptr), y->stride[0],
        r_inv ? static_cast<float*>(r_inv->ptr) : nullptr, r_inv ? r_inv->stride[0] : 0, rows, cols,
        eps, stages, status);
    return;
  }
  }
  const int warps = FWD_THREADS / 32;
  const long long want = (static_cast<long long>(rows) + warps - 1) / warps;
  const int grid = static_cast<int>(want < 1 ? 1 : (want > (1 << 24) ? (1 << 24) : want));
  launch_pdl(rmsnorm_fwd_kernel<NCH>, dim3(grid), dim3(FWD_THREADS), 0, stream,
      static_cast<const __nv_bfloat16*>(x->ptr), x->stride[0],
      scale ? static_cast<const __nv_bfloat16*>(scale->ptr) : nullptr,
      bias ? static_cast<const __nv_bfloat16*>(bias->ptr) : nullptr,
      static_cast<__nv_bfloat16*>(y->ptr), y->stride[0],
      r_inv ? static_cast<float*>(r_inv->ptr) : nullptr, r_inv ? r_inv->stride[0] : 0, rows, cols,
      eps);
}

template <int NCH, bool DSCALE>
static void launch_bwd(const cdl_tensor* x, const cdl_tensor* dy, const cdl_tensor* res,
                       const cdl_tensor* scale, const cdl_tensor* r_inv, const cdl_tensor* dx,
                       float* partials, int grid, int rows, int cols, cudaStream_t stream) {
  const size_t smem = DSCALE ? static_cast<size_t>(cols) * sizeof(float) : 0;
  launch_pdl(rmsnorm_bwd_kernel<NCH, DSCALE>, dim3(grid), dim3(BWD_THREADS), smem, stream,
      static_cast<const __nv_bfloat16*>(x->ptr), x->stride[0],
      static_cast<const __nv_bfloat16*>(dy->ptr), dy->stride[0],
      res ? static_cast<const __nv_bfloat16*>(res->ptr) : nullptr, res ? res->stride[0] : 0,
      static_cast<const __nv_bfloat16*>(scale->ptr), static_cast<const float*>(r_inv->ptr),
      r_inv->stride[0], static_cast<__nv_bfloat16*>(dx->ptr), dx->stride[0], partials, rows, cols);
}

template <int NCH>
static void launch_bwd_pipe(const cdl_tensor* x, const cdl_tensor* dy, const cdl_tensor* res,
                            const cdl_tensor* scale, const cdl_tensor* r_inv, const cdl_tensor* dx,
                            float* partials, int rows, int cols, int* status, cudaStream_t stream) {
  const int row_bytes = cols * 2;
  const int stage_bytes = (res ? 3 : 2) * row_bytes;
  int stages = (160 * 1024) / stage_bytes;
  if (stages > 64) stages = 64;
  stages &= ~1;  // even: each of the two producer lanes owns every other stage
  const size_t smem = static_cast<size_t>(stages) * stage_bytes + row_bytes + 2 * stages * sizeof(uint64_t) + 16;
  static std::once_flag once[64];
  int dev = 0;
  cudaGetDevice(&dev);
  std::call_once(once[dev & 63], [&] {
    cudaFuncSetAttribute(rmsnorm_bwd_pipe_kernel<NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         160 * 1024 + 4096 + 2 * 64 * static_cast<int>(sizeof(uint64_t)) + 16);
  });
  launch_pdl(rmsnorm_bwd_pipe_kernel<NCH>, dim3(sm_count()), dim3(BWD_PIPE_THREADS), smem, stream,
      static_cast<const __nv_bfloat16*>(x->ptr), x->stride[0],
      static_cast<const __nv_bfloat16*>(dy->ptr), dy->stride[0],
      res ? static_cast<const __nv_bfloat16*>(res->ptr) : nullptr, res ? res->stride[0] : 0,
      static_cast<const __nv_bfloat16*>(scale->ptr), static_cast<const float*>(r_inv->ptr),
      r_inv->stride[0], static_cast<__nv_bfloat16*>(dx->ptr), dx->stride[0], partials, rows, cols,
      stages, status);
}

}  // namespace norm

int32_t rmsnorm_fwd_execute(const cdl_tensor* x, const cdl_tensor* scale, const cdl_tensor* bias,
                            float eps, const cdl_tensor* y, const cdl_tensor* r_inv,
                            cudaStream_t stream, const cdl_norm_options* opts) {
  using namespace norm;
  const char* op = "norm_fwd";
  if (!x || !y) return fail(CDL_ERR_INVALID, "%s: x and y are required", op);
  const int variant = opts ? opts->variant : CDL_NORM_AUTO;
  if (variant < CDL_NORM_AUTO || variant > CDL_NORM_PIPELINED)
    return fail(CDL_ERR_INVALID, "%s: unknown kernel variant %d", op, variant);
  if (!fast_norm_operands(x, scale, bias, y))
    return norm_general_execute(0, x, scale, bias, eps, y, nullptr, r_inv, stream);
  const long long rows = x->shape[0], cols = x->shape[1];
  if (r_inv) CDL_CHECK(check_vec(op, "r_inv", r_inv, rows, CDL_F32, false));
  if (rows == 0 || cols == 0) return CDL_OK;
  if (rows > INT32_MAX) return fail(CDL_ERR_UNSUPPORTED, "%s: too many rows", op);
  const int r = static_cast<int>(rows), c = static_cast<int>(cols);
  ProfileScope ps(PROF_NORM_FWD, 4.0 * rows * cols + 2.0 * cols + (r_inv ? 4.0 * rows : 0.0), stream);
  if (c <= 256) launch_fwd<1>(x, scale, bias, eps, y, r_inv, r, c, variant, stream);
  else if (c <= 512) launch_fwd<2>(x, scale, bias, eps, y, r_inv, r, c, variant, stream);
  else if (c <= 1024) launch_fwd<4>(x, scale, bias, eps, y, r_inv, r, c, variant, stream);
  else if (c <= 2048) launch_fwd<8>(x, scale, bias, eps, y, r_inv, r, c, variant, stream);
  else if (c <= 4096) launch_fwd<16>(x, scale, bias, eps, y, r_inv, r, c, variant, stream);
  else launch_fwd<32>(x, scale, bias, eps, y, r_inv, r, c, variant, stream);
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

template <int NCH>
static void launch_layernorm(const cdl_tensor* x, const cdl_tensor* scale, const cdl_tensor* bias,
                             float eps, const cdl_tensor* y, const cdl_tensor* mean,
                             const cdl_tensor* r_inv, int rows, int cols, cudaStream_t stream) {
  using namespace norm;
  const int warps = FWD_THREADS / 32;
  const long long want = (static_cast<long long>(rows) + warps - 1) / warps;
  const int grid = static_cast<int>(want > (1 << 24) ? (1 << 24) : want);
  launch_pdl(layernorm_fwd_kernel<NCH>, dim3(grid), dim3(FWD_THREADS), 0, stream,
      static_cast<const __nv_bfloat16*>(x->ptr), x->stride[0],
      scale ? static_cast<const __nv_bfloat16*>(scale->ptr) : nullptr,
      bias ? static_cast<const __nv_bfloat16*>(bias->ptr) : nullptr,
      static_cast<__nv_bfloat16*>(y->ptr), y->stride[0],
      mean ? static_cast<float*>(mean->ptr) : nullptr, mean ? mean->stride[0] : 0,
      r_inv ? static_cast<float*>(r_inv->ptr) : nullptr, r_inv ? r_inv->stride[0] : 0, rows, cols, eps);
}

int32_t layernorm_fwd_execute(const cdl_tensor* x, const cdl_tensor* scale, const cdl_tensor* bias,
                              float eps, const cdl_tensor* y, const cdl_tensor* mean,
                              const cdl_tensor* r_inv, cudaStream_t stream) {
  using namespace norm;
  const char* op = "norm_fwd (layer norm)";
  if (!x || !y) return fail(CDL_ERR_INVALID, "%s: x and y are required", op);
  if (!fast_norm_operands(x, scale, bias, y))
    return norm_general_execute(1, x, scale, bias, eps, y, mean, r_inv, stream);
  const long long rows = x->shape[0], cols = x->shape[1];
  if (mean) CDL_CHECK(check_vec(op, "mean", mean, rows, CDL_F32, false));
  if (r_inv) CDL_CHECK(check_vec(op, "r_inv", r_inv, rows, CDL_F32, false));
  if (rows == 0 || cols == 0) return CDL_OK;
  if (rows > INT32_MAX) return fail(CDL_ERR_UNSUPPORTED, "%s: too many rows", op);
  const int r = static_cast<int>(rows), c = static_cast<int>(cols);
  ProfileScope ps(PROF_NORM_FWD, 4.0 * rows * cols + 2.0 * cols + 8.0 * rows, stream);
  if (c <= 256) launch_layernorm<1>(x, scale, bias, eps, y, mean, r_inv, r, c, stream);
  else if (c <= 512) launch_layernorm<2>(x, scale, bias, eps, y, mean, r_inv, r, c, stream);
  else if (c <= 1024) launch_layernorm<4>(x, scale, bias, eps, y, mean, r_inv, r, c, stream);
  else if (c <= 2048) launch_layernorm<8>(x, scale, bias, eps, y, mean, r_inv, r, c, stream);
  else if (c <= 4096) launch_layernorm<16>(x, scale, bias, eps, y, mean, r_inv, r, c, stream);
  else launch_layernorm<32>(x, scale, bias, eps, y, mean, r_inv, r, c, stream);
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

size_t rmsnorm_bwd_scratch_bytes(long long rows, long long cols) {
  (void)rows;
  return static_cast<size_t>(norm::MAX_PARTIALS) * static_cast<size_t>(cols) * sizeof(float);
}

int32_t rmsnorm_bwd_execute(const cdl_tensor* x, const cdl_tensor* dy, const cdl_tensor* res,
                            const cdl_tensor* scale, const cdl_tensor* r_inv, const cdl_tensor* dx,
                            const cdl_tensor* dscale, void* scratch, size_t scratch_bytes,
                            cudaStream_t stream, const cdl_norm_options* opts) {
  using namespace norm;
  const char* op = "norm_bwd";
  const int variant = opts ? opts->variant : CDL_NORM_AUTO;
  if (variant < CDL_NORM_AUTO || variant > CDL_NORM_PIPELINED)
    return fail(CDL_ERR_INVALID, "%s: unknown kernel variant %d", op, variant);
  if (!x || !dy || !scale || !r_inv || !dx || !dscale)
    return fail(CDL_ERR_INVALID, "%s: x, dy, scale, r_inv, dx and dscale are required", op);
  if (x->rank != 2) return fail(CDL_ERR_INVALID, "%s: x must be a 2D tensor", op);
  const long long rows = x->shape[0], cols = x->shape[1];
  if (cols % 8 != 0 || cols > 8192)
    return fail(CDL_ERR_UNSUPPORTED,
                "%s: cols must be a multiple of 8 and at most 8192 (got %lld)", op, cols);
  CDL_CHECK(check_rows(op, "x", x, rows, cols));
  CDL_CHECK(check_rows(op, "dy", dy, rows, cols));
  CDL_CHECK(check_rows(op, "dx", dx, rows, cols));
  if (res) CDL_CHECK(check_rows(op, "residual_dy", res, rows, cols));
  CDL_CHECK(check_vec(op, "scale", scale, cols, CDL_BF16, true));
  CDL_CHECK(check_vec(op, "r_inv", r_inv, rows, CDL_F32, false));
  CDL_CHECK(check_vec(op, "dscale", dscale, cols, CDL_F32, false));
  if (cols == 0 || rows == 0) return CDL_OK;
  if (rows > INT32_MAX) return fail(CDL_ERR_UNSUPPORTED, "%s: too many rows", op);
  if (scratch == nullptr || scratch_bytes < rmsnorm_bwd_scratch_bytes(rows, cols) ||
      (reinterpret_cast<uintptr_t>(scratch) & 15) != 0)
    return fail(CDL_ERR_INVALID, "%s: scratch must be 16-byte aligned and hold %zu bytes (got %zu)",
                op, rmsnorm_bwd_scratch_bytes(rows, cols), scratch_bytes);
  const int r = static_cast<int>(rows), c = static_cast<int>(cols);
  float* partials = static_cast<float*>(scratch);
  const int warps = BWD_THREADS / 32;
  int grid = sm_count() * BWD_BLOCKS_PER_SM;
  if (grid > MAX_PARTIALS) grid = MAX_PARTIALS;
  const int need = (r + warps - 1) / warps;
  if (grid > need) grid = need;
  int num_partials = grid;
  // Measured back to back at [16384, 2048] with two producer lanes feeding the ring: the pipelined
  // kernel takes 44.5 us without and 52.5 us with a residual gradient, the warp-per-row kernel
  // 45 us and 81 us (the third row does not fit its registers next to the dscale accumulators);
  // at 65536 rows 139 / 171 us against 147 us for the warp-per-row form without residual.
  const bool pipe = c <= 2048 && r >= 2 * sm_count() &&
                    (variant == CDL_NORM_AUTO || variant == CDL_NORM_PIPELINED);
  ProfileScope ps(PROF_NORM_BWD, (res ? 8.0 : 6.0) * rows * cols + 6.0 * cols + 4.0 * rows, stream);
  if (pipe) {
    num_partials = sm_count();
    int* status = device_status_ptr();
    if (!status) return fail(CDL_ERR_CUDA, "cannot resolve the device status word");
    if (c <= 256) launch_bwd_pipe<1>(x, dy, res, scale, r_inv, dx, partials, r, c, status, stream);
    else if (c <= 512) launch_bwd_pipe<2>(x, dy, res, scale, r_inv, dx, partials, r, c, status, stream);
    else if (c <= 1024) launch_bwd_pipe<4>(x, dy, res, scale, r_inv, dx, partials, r, c, status, stream);
    else launch_bwd_pipe<8>(x, dy, res, scale, r_inv, dx, partials, r, c, status, stream);
  } else if (c <= 256) launch_bwd<1, true>(x, dy, res, scale, r_inv, dx, partials, grid, r, c, stream);
  else if (c <= 512) launch_bwd<2, true>(x, dy, res, scale, r_inv, dx, partials, grid, r, c, stream);
  else if (c <= 1024) launch_bwd<4, true>(x, dy, res, scale, r_inv, dx, partials, grid, r, c, stream);
  else if (c <= 2048) launch_bwd<8, true>(x, dy, res, scale, r_inv, dx, partials, grid, r, c, stream);
  else {
    if (c <= 4096) launch_bwd<16, false>(x, dy, res, scale, r_inv, dx, nullptr, grid, r, c, stream);
    else launch_bwd<32, false>(x, dy, res, scale, r_inv, dx, nullptr, grid, r, c, stream);
    num_partials = r < 256 ? r : 256;
    dim3 g((c + 127) / 128, num_partials);
    launch_pdl(dscale_cols_kernel, g, dim3(128), 0, stream,
        static_cast<const __nv_bfloat16*>(x->ptr), x->stride[0],
        static_cast<const __nv_bfloat16*>(dy->ptr), dy->stride[0],
        static_cast<const float*>(r_inv->ptr), r_inv->stride[0], partials, r, c);
  }
  CDL_CUDA(cudaGetLastError());
  launch_pdl(dscale_finalize_kernel, dim3((c + FIN_COLS - 1) / FIN_COLS), dim3(FIN_COLS * FIN_GROUPS), 0, stream,
             static_cast<const float*>(partials), num_partials, c, static_cast<float*>(dscale->ptr),
             static_cast<long long>(dscale->stride[0]));
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}


// ---------------------------------------------------------------- allocation-free backward
// Scratch for cdl_b200_rmsnorm_bwd_static: one fixed array in the module's global memory, so a
// caller that is not allowed to allocate (or to be handed) device scratch can still run the
// backward.  8 MiB = 1024 partial rows x 2048 columns of f32; held by every device that loads
// the library until the process exits.
namespace norm {
constexpr long long STATIC_MAX_COLS = 2048;
constexpr size_t STATIC_SCRATCH_FLOATS = static_cast<size_t>(MAX_PARTIALS) * STATIC_MAX_COLS;
static __device__ __align__(256) float g_static_partials[STATIC_SCRATCH_FLOATS];
}  // namespace norm

int32_t rmsnorm_bwd_static_execute(const cdl_tensor* x, const cdl_tensor* dy, const cdl_tensor* res,
                                   const cdl_tensor* scale, const cdl_tensor* r_inv,
                                   const cdl_tensor* dx, const cdl_tensor* dscale,
                                   cudaStream_t stream) {
  const char* op = "norm_bwd_static";
  if (!x || x->rank != 2) return fail(CDL_ERR_INVALID, "%s: x must be a 2D tensor", op);
  if (x->shape[1] > norm::STATIC_MAX_COLS)
    return fail(CDL_ERR_UNSUPPORTED,
                "%s: cols = %lld exceeds the built-in scratch (at most %lld columns); use "
                "cdl_b200_rmsnorm_bwd with caller-provided scratch instead",
                op, (long long)x->shape[1], norm::STATIC_MAX_COLS);
  // In host code the array's name is only a handle; the kernels need its device address, which
  // differs per device.  Resolve it once per device, with that device current.
  static float* addr[64] = {};
  static std::mutex mu;
  int dev = 0;
  CDL_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(CDL_ERR_UNSUPPORTED, "%s: device index %d out of range", op, dev);
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
      void* p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, norm::g_static_partials);
      if (e != cudaSuccess || p == nullptr)
        return fail(CDL_ERR_CUDA, "%s: cudaGetSymbolAddress failed: %s", op, cudaGetErrorString(e));
      addr[dev] = static_cast<float*>(p);
    }
    scratch = addr[dev];
  }
  const size_t bytes = norm::STATIC_SCRATCH_FLOATS * sizeof(float);
  if (rmsnorm_bwd_scratch_bytes(x->shape[0], x->shape[1]) > bytes)
    return fail(CDL_ERR_UNSUPPORTED, "%s: problem needs more than the built-in %zu bytes of scratch",
                op, bytes);
  // Every partial row that is read is written first by the same call, so the array needs no
  // clearing between calls.
  return rmsnorm_bwd_execute(x, dy, res, scale, r_inv, dx, dscale, scratch, bytes, stream);
}

}  // namespace cdl

extern "C" {

int32_t cdl_b200_rmsnorm_fwd(const cdl_tensor* x, const cdl_tensor* scale, const cdl_tensor* bias,
                             float eps, const cdl_tensor* y, const cdl_tensor* r_inv,
                             cdl_stream stream) {
  return cdl::rmsnorm_fwd_execute(x, scale, bias, eps, y, r_inv,
                                  static_cast<cudaStream_t>(stream));
}

int32_t cdl_b200_rmsnorm_fwd_opt(const cdl_tensor* x, const cdl_tensor* scale,
                                 const cdl_tensor* bias, float eps, const cdl_tensor* y,
                                 const cdl_tensor* r_inv, const cdl_norm_options* options,
                                 cdl_stream stream) {
  return cdl::rmsnorm_fwd_execute(x, scale, bias, eps, y, r_inv, static_cast<cudaStream_t>(stream),
                                  options);
}

int32_t cdl_b200_layernorm_fwd(const cdl_tensor* x, const cdl_tensor* scale, const cdl_tensor* bias,
                               float eps, const cdl_tensor* y, const cdl_tensor* mean,
                               const cdl_tensor* r_inv, cdl_stream stream) {
  return cdl::layernorm_fwd_execute(x, scale, bias, eps, y, mean, r_inv,
                                    static_cast<cudaStream_t>(stream));
}

int32_t cdl_b200_rmsnorm_bwd(const cdl_tensor* x, const cdl_tensor* dy,
                             const cdl_tensor* residual_dy, const cdl_tensor* scale,
                             const cdl_tensor* r_inv, const cdl_tensor* dx,
                             const cdl_tensor* dscale, void* scratch, size_t scratch_bytes,
                             cdl_stream stream) {
  return cdl::rmsnorm_bwd_execute(x, dy, residual_dy, scale, r_inv, dx, dscale, scratch,
                                  scratch_bytes, static_cast<cudaStream_t>(stream));
}

int32_t cdl_b200_rmsnorm_bwd_opt(const cdl_tensor* x, const cdl_tensor* dy,
                                 const cdl_tensor* residual_dy, const cdl_tensor* scale,
                                 const cdl_tensor* r_inv, const cdl_tensor* dx,
                                 const cdl_tensor* dscale, const cdl_norm_options* options,
                                 void* scratch, size_t scratch_bytes, cdl_stream stream) {
  return cdl::rmsnorm_bwd_execute(x, dy, residual_dy, scale, r_inv, dx, dscale, scratch,
                                  scratch_bytes, static_cast<cudaStream_t>(stream), options);
}

int32_t cdl_b200_rmsnorm_bwd_static(const cdl_tensor* x, const cdl_tensor* dy,
                                    const cdl_tensor* residual_dy, const cdl_tensor* scale,
                                    const cdl_tensor* r_inv, const cdl_tensor* dx,
                                    const cdl_tensor* dscale, cdl_stream stream) {
  return cdl::rmsnorm_bwd_static_execute(x, dy, residual_dy, scale, r_inv, dx, dscale,
                                         static_cast<cudaStream_t>(stream));
}

int32_t cdl_b200_rmsnorm_bwd_scratch_bytes(int64_t rows, int64_t cols, size_t* bytes_out) {
  if (rows < 0 || cols < 0) return cdl::fail(CDL_ERR_INVALID, "norm_bwd: negative shape");
  if (bytes_out) *bytes_out = cdl::rmsnorm_bwd_scratch_bytes(rows, cols);
  return CDL_OK;
}

}  // extern "C"
