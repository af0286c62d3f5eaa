// Flash attention backward on tcgen05 tensor cores: dQ, dK, dV from Q, K, V, O, dO and LSE.
//
// Operator semantics follow AttentionBwd of the reference (crates/cleandl/src/execgraph/ops/
// attention/mod.rs:366-374, 852-935; operand order q, k, v, out, d_out, lse :899-905), whose
// arithmetic lives in flash-attention-rs; the math is the one of the reference's f64 test oracle
// (crates/cleandl/tests/attention.rs:444-462):
//   delta_i = sum_d dO_id O_id;  P = exp(S - LSE);  dV = P^T dO;  dP = dO V^T;
//   dS = P o (dP - delta) * scale;  dQ = dS K;  dK = dS^T Q.
//
// Three kernels, none of which uses atomics (the result is bit-reproducible):
//   1. preprocess: delta and LSE * log2(e) per query row into scratch (rows padded to 128).
//   2. dK/dV: one CTA per (128-key block, kv head, batch) walks the query blocks that see it.
//      Everything is computed TRANSPOSED so that a thread owns one key row:
//        S^T  = K Q^T   (SS) -> TMEM [0,128)     P^T (bf16) overwrites it in place
//        dP^T = V dO^T  (SS) -> TMEM [128,256)
//        dV  += P^T dO  (A = P^T from TMEM)      -> TMEM [256,384)
//        dK  += dS^T Q  (A = dS^T from TMEM, written over dP^T) -> TMEM [384,512)
//   3. dQ: one CTA per (128-query block, head, batch) walks the key blocks it sees and recomputes
//      S and dP (two extra products per block pair) so that dQ accumulates in TMEM instead of
//      being reduced through global memory from the dK/dV kernel -- measured on B200, the L2
//      reduction traffic of that single-kernel form (64 KiB per block pair) took longer than the
//      two recomputed products:
//        S  = Q K^T   (SS) -> TMEM S[j & 1]      dS (bf16) overwrites it in place
//        dP = dO V^T  (SS) -> TMEM [256,384)
//        dQ += dS K   (A = dS from TMEM)          -> TMEM [384,512)
// Kernels 2 and 3 exist in two forms: one short-lived CTA per block, and (the default when there
// are more blocks than SMs) one CTA per SM that walks many blocks handed out at run time, so
// that launch, allocation, first loads and first products of a block run under the previous
// block's last products and stores.  Both forms execute the same arithmetic in the same order.
// Scratch: LSE2 and delta, f32 [B, H, Sq_pad] each.
#include "host.h"
#include "ptx.cuh"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

namespace cdl {

int32_t attn_check_operand(const char* op, const char* name, const cdl_tensor* t, long long B,
                           long long S, long long H, long long D);
int32_t attn_encode_tmap(CUtensorMap* out, const cdl_tensor* t);
int32_t attn_encode_tmap_rows(CUtensorMap* out, const cdl_tensor* t, uint32_t box_rows);
int32_t attn_packed_view(const char* op, const char* name, const cdl_tensor* t, long long total,
                         long long heads, cdl_tensor* view);
int32_t attn_check_cu_seqlens(const char* op, const char* name, const cdl_tensor* t, long long batch);

namespace attn_bwd {

constexpr int D = 128;
constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int TILE_BYTES = 128 * 128 * 2;
constexpr int PANEL_BYTES = TILE_BYTES / 2;
constexpr int THREADS = 384;  // warps 0-3 control (TMA, MMA, 2 idle), warps 4-11 compute
constexpr int TMEM_COLS = 512;
// dK/dV kernel: K, V, Q x 2 stages, dO x 2 stages, row statistics, barriers
constexpr int KV_COL_S = 0, KV_COL_DP = 128, KV_COL_DV = 256, KV_COL_DK = 384;
constexpr size_t KV_SMEM_BYTES = 6 * TILE_BYTES + 2 * 2 * 128 * sizeof(float) + 256;
// dQ kernel: Q, dO, K x 3 stages (S of block j+1 is issued a block ahead and dQ of block j reads
// its K last, so two stages would expose the TMA latency every block), V x 2 stages, barriers
constexpr int Q_COL_S = 0, Q_COL_DP = 256, Q_COL_DQ = 384;  // S is double-buffered: [0,128) [128,256)
constexpr int QK_STAGES = 3;
constexpr size_t Q_SMEM_BYTES = (4 + QK_STAGES) * TILE_BYTES + 256;
static_assert(KV_SMEM_BYTES <= 232448 && Q_SMEM_BYTES <= 232448,
              "exceeds the 227 KiB of shared memory a CTA can opt in to");

// Registers per thread of the dK/dV kernel's roles (control warps / compute warps; 168 at launch,
// LOW + 2 HIGH = 3 x 168): with 56 the issuing lane spills.
constexpr int KV_LOW_REGS = 72, KV_HIGH_REGS = 216;

// Bytes of Q, dO, K, V a chunk of the CTA order may span (see cta_coords).  Measured at B 8 / 2,
// S 2048, B 1 S 8192 and B 4 S 4096 against the old order (all blocks of one head, then the next
// head): 16 MB 0.555 / 0.145 / 0.789 / 0.880 ms against 0.561 / 0.166 / 0.825 / 0.897; 8 MB 0.561 /
// 0.162 / 0.837 / 0.900; 48 MB 0.575 / 0.154 / 0.81-0.84 (too many CTAs of one length in step).
#ifndef CDL_ATTN_BWD_CHUNK_MB
#define CDL_ATTN_BWD_CHUNK_MB 16
#endif
// Items per SM the last chunk of that order should hold (see tail_pairs_of).
#ifndef CDL_ATTN_BWD_TAIL_X
#define CDL_ATTN_BWD_TAIL_X 2
#endif

// 1: the dK/dV and dQ kernels run as one CTA per SM over many key / query blocks when there are
// more blocks than SMs; 0: always one CTA per block.
#ifndef CDL_ATTN_BWD_PERSISTENT
#define CDL_ATTN_BWD_PERSISTENT 1
#endif

// Status code (device status word) of a packed sequence longer than max_seqlen_q / max_seqlen_k.
constexpr int STATUS_SEQ_EXCEEDS_BOUND = 921;

struct Params {
  int B, H, Hkv, Sq, Sk, Sq_pad;
  int causal;
  float scale, scale_log2;
  const float* lse2;   // [B, H, Sq_pad]  LSE * log2(e), +inf for rows that contribute nothing
  const float* delta;  // [B, H, Sq_pad]
  __nv_bfloat16* dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  long long dq_sb, dq_ss, dq_sh, dk_sb, dk_ss, dk_sh, dv_sb, dv_ss, dv_sh;
  // Packed layout: sequence b is rows cu_q[b] .. cu_q[b + 1] of q / o / dO / dQ and
  // cu_k[b] .. cu_k[b + 1] of k / v / dK / dV; Sq / Sk are then the bounds the grids were sized
  // with (Sq_pad pads that bound).  nullptr: dense layout.
  const int* cu_q;
  const int* cu_k;
  // Rotary embedding folded into the dQ / dK stores: f32 [rope_rows, 128] = cos(64) | sin(64) per
  // position (the position of a row is its index in its sequence), or nullptr.  q and k are then
  // the rotated tensors the forward consumed and dQ / dK come out as gradients of the tensors
  // before the rotation.
  const float* rope;
  int rope_rows;
  // CTA order (see cta_coords): number of blocks along the sequence, heads x batch, heads per chunk
  // and (head, batch) pairs of the last chunk
  int kv_blocks, kv_heads_total, kv_chunk, kv_tail;  // dK/dV kernel
  int q_blocks, q_heads_total, q_chunk, q_tail;      // dQ kernel
  int variant;  // cdl_attn_variant of the call (read on the host only)
  int* status;
};

struct KvBarriers {
  uint64_t kv_full;
  uint64_t q_full[2], q_empty[2], do_full[2], do_empty[2];
  uint64_t s_full, dp_full, p_ready, ds_ready, dv_done, dk_done;
  uint32_t tmem_base;
  int abort_word;
};

struct QBarriers {
  uint64_t qdo_full;
  uint64_t k_full[QK_STAGES], k_empty[QK_STAGES], v_full[2], v_empty[2];
  uint64_t s_full[2], dp_full, ds_ready, dq_done;
  uint32_t tmem_base;
  int abort_word;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Packed f32x2 arithmetic: one issue slot for two lanes of work.
__device__ __forceinline__ uint64_t pk2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void upk2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t sub_x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul_x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// Of every 16 exponentials, this many go to the polynomial: it balances the MUFU pipe against the
// FMA pipe for the instruction mix of the P phases (one FMA per element plus six per polynomial).
#ifndef CDL_POLY_OF_16
#define CDL_POLY_OF_16 6
#endif
constexpr int POLY_OF_16 = CDL_POLY_OF_16;
// Two polynomial exponentials at once with packed f32x2 arithmetic (one issue slot for two lanes
// of work; the scheme of exp2_poly in ptx.cuh).
__device__ __forceinline__ void exp2_poly_pair(float x0, float x1, float& r0, float& r1) {
  auto pack2 = [](float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
  };
  auto unpack2 = [](uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); };
  auto fma2 = [](uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
  };
  auto add2 = [](uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
  };
  auto sub2 = [](uint64_t a, uint64_t b) {
    uint64_t d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
  };
  const uint64_t xc = pack2(fmaxf(x0, -126.0f), fmaxf(x1, -126.0f));
  const uint64_t magic = pack2(12582912.0f, 12582912.0f);
  const uint64_t t = add2(xc, magic);
  const uint64_t f = sub2(xc, sub2(t, magic));
  uint64_t r = fma2(f, pack2(0.0551716685f, 0.0551716685f), pack2(0.2426111251f, 0.2426111251f));
  r = fma2(r, f, pack2(0.6932609677f, 0.6932609677f));
  r = fma2(r, f, pack2(0.9999280572f, 0.9999280572f));
  float t0, t1, p0, p1;
  unpack2(t, t0, t1);
  unpack2(r, p0, p1);
  r0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
  r1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}

// Columns C and C + 1 (C even): the first POLY_OF_16 (even) of every 16 take the polynomial.
template <int C>
__device__ __forceinline__ void exp2_row_step(const float (&x)[64], float (&y)[64]) {
  if constexpr (C < 64) {
#ifndef CDL_ATTN_BWD_SCALAR_POLY
    if constexpr ((C & 15) < POLY_OF_16) {
      exp2_poly_pair(x[C], x[C + 1], y[C], y[C + 1]);
    } else {
      y[C] = ex2(x[C]);
      y[C + 1] = ex2(x[C + 1]);
    }
#else
    y[C] = (C & 15) < POLY_OF_16 ? exp2_poly(x[C]) : ex2(x[C]);
    y[C + 1] = ((C + 1) & 15) < POLY_OF_16 ? exp2_poly(x[C + 1]) : ex2(x[C + 1]);
#endif
    exp2_row_step<C + 2>(x, y);
  }
}
static_assert(POLY_OF_16 % 2 == 0, "the polynomial takes column pairs");

__device__ __forceinline__ void exp2_row64(const float (&x)[64], float (&y)[64]) {
  exp2_row_step<0>(x, y);
}

__device__ __forceinline__ void compute_bar_sync() {
  asm volatile("bar.sync 1, 256;" ::: "memory");
}

// Inverse rotary rotation of the staged dQ / dK rows, in place of the transposed-rotation kernel
// that would otherwise re-read the tensor.  Thread (wg, r) has staged columns [64 wg, 64 wg + 64) of
// row r as bf16 in two 128-byte-swizzled panels of [128 rows][64 columns]; the rotation pairs column
// i with column i + 64, i.e. 16-byte chunk c of a row in the first panel with chunk c of that row
// in the second.  The rotation itself is dealt out anew: the 128 x 8 (row, chunk) units go to the
// 256 compute threads in order, unit i * 256 + ct to thread ct, so that eight neighbouring threads
// read one row's cosines and sines side by side (the table rows of a tile are contiguous) and one
// row of each panel without bank conflicts; a thread's 16 table loads are issued together by
// rope_units_load, early enough to land under the last product, and a thread overwrites exactly
// what it has read, so no barrier separates reading from writing.  With x the staged
// (bf16-rounded) values, out_lo = x_lo cos + x_hi sin and out_hi = x_hi cos - x_lo sin, in f32 as
// the stand-alone kernel computes them from the stored bf16 tensor.  The caller synchronises the
// compute threads between staging and apply.  (Two earlier forms kept a thread on its own row:
// all 128 table values of the row loaded chunk by chunk behind the barrier, then half of them
// loaded ahead.  A warp's load then touches 32 table rows, 32 cache lines per instruction, and
// the rotation cost 0.2 ms, then 0.1 ms per backward call at B 8, S 2048 -- more than the
// stand-alone rotation kernels it replaced.)
struct RopeUnits {
  float4 t[16];  // per unit: cos[0..4), cos[4..8), sin[0..4), sin[4..8) of its chunk
};
__device__ __forceinline__ void rope_units_load(const float* table, int pos0, int rope_rows, int ct, RopeUnits& ru) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int id = i * 256 + ct;
    const int row = id >> 3, c = id & 7;
    const float* cs = table + static_cast<long long>(min(pos0 + row, rope_rows - 1)) * 128;
    ru.t[i * 4 + 0] = __ldg(reinterpret_cast<const float4*>(cs + c * 8));
    ru.t[i * 4 + 1] = __ldg(reinterpret_cast<const float4*>(cs + c * 8 + 4));
    ru.t[i * 4 + 2] = __ldg(reinterpret_cast<const float4*>(cs + 64 + c * 8));
    ru.t[i * 4 + 3] = __ldg(reinterpret_cast<const float4*>(cs + 64 + c * 8 + 4));
  }
}
// to_stage: the rotated chunks go back to the staging tile (a TMA store follows); otherwise to
// global memory: `dst_tile` is column 0 of the tile's first row, rows at `row_stride` elements,
// the first `rows_ok` of them inside the sequence.
__device__ __forceinline__ void rope_inverse_apply(uint8_t* stage, int ct, const RopeUnits& ru, bool to_stage,
                                                   __nv_bfloat16* dst_tile, long long row_stride, int rows_ok) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int id = i * 256 + ct;
    const int row = id >> 3, c = id & 7;
    uint8_t* lo_row = stage + row * 128;
    uint8_t* hi_row = stage + PANEL_BYTES + row * 128;
    const int off = (c ^ (row & 7)) << 4;
    const uint4 a = *reinterpret_cast<const uint4*>(lo_row + off);
    const uint4 b = *reinterpret_cast<const uint4*>(hi_row + off);
    const float4 c0 = ru.t[i * 4 + 0], c1 = ru.t[i * 4 + 1], s0 = ru.t[i * 4 + 2], s1 = ru.t[i * 4 + 3];
    const float cv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
    uint32_t lw[4], hw[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float x0 = __uint_as_float(aw[e] << 16), x1 = __uint_as_float(aw[e] & 0xffff0000u);
      const float y0 = __uint_as_float(bw[e] << 16), y1 = __uint_as_float(bw[e] & 0xffff0000u);
      lw[e] = pack_bf16x2(x0 * cv[2 * e] + y0 * sv[2 * e], x1 * cv[2 * e + 1] + y1 * sv[2 * e + 1]);
      hw[e] = pack_bf16x2(y0 * cv[2 * e] - x0 * sv[2 * e], y1 * cv[2 * e + 1] - x1 * sv[2 * e + 1]);
    }
    const uint4 ol = make_uint4(lw[0], lw[1], lw[2], lw[3]), oh = make_uint4(hw[0], hw[1], hw[2], hw[3]);
    if (to_stage) {
      *reinterpret_cast<uint4*>(lo_row + off) = ol;
      *reinterpret_cast<uint4*>(hi_row + off) = oh;
    } else if (row < rows_ok) {
      *reinterpret_cast<uint4*>(dst_tile + row * row_stride + c * 8) = ol;
      *reinterpret_cast<uint4*>(dst_tile + row * row_stride + 64 + c * 8) = oh;
    }
  }
}

// The issuing thread builds a descriptor with one 32-bit add: the low word (start address and
// leading byte offset) is computed once per tile, the K step adds a compile-time constant, the high
// word is constant.  Between two products it executes as little as possible: whatever it does
// there is time the tensor pipe may idle.
constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version 1, SW128
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo_bytes) {
  return ((addr & 0x3FFFFu) >> 4) | ((lbo_bytes >> 4) << 16);
}
__device__ __forceinline__ uint64_t desc_at(uint32_t lo, uint32_t byte_off) {
  return (static_cast<uint64_t>(DESC_HI) << 32) | (lo + (byte_off >> 4));
}
// Byte offset of K step k (16 elements): K-major tile (two 16 KiB panels of 64 elements) and
// MN-major tile (16 rows of 128 bytes per step).
__device__ __forceinline__ constexpr uint32_t koff_k(int k) { return (k >> 2) * PANEL_BYTES + (k & 3) * 32; }
__device__ __forceinline__ constexpr uint32_t koff_mn(int k) { return k * 2048; }
// TMEM column of K step k of a bf16 A operand stored as two 32-column halves at +0 and +64.
__device__ __forceinline__ constexpr uint32_t acol(int k) { return (k >> 2) * 64 + (k & 3) * 8; }

// ---------------------------------------------------------------- preprocess
// delta = sum_d dO * O and lse2 = lse * log2(e) per query row.  A block takes PRE_ROWS rows x 16
// heads of one sequence: half a warp (16 lanes x 8 bf16 = one 256-byte row of O and of dO) per
// head walks the rows, so the block's half-warps read the heads of a row side by side (4 KiB
// contiguous in the usual [batch, row, head, 128] layout) with eight rows' loads in flight per
// thread; the results turn through shared memory so that the [batch, head, padded row] statistics
// are written PRE_ROWS rows at a time.  (One half-warp per row with the rows of a head side by
// side, 256-byte pieces 4 KiB apart: 40 us for the 134 MB of B 8, S 2048, H 16; this form ~29.
// 8 rows per block against 16: the same there, 3 % better at B 2 where 16 leave 256 blocks.)
#ifndef CDL_PRE_ROWS
#define CDL_PRE_ROWS 8
#endif
constexpr int PRE_ROWS = CDL_PRE_ROWS, PRE_HEADS = 16;
__global__ void __launch_bounds__(256)
    attn_bwd_preprocess_kernel(const __nv_bfloat16* __restrict__ o, long long o_sb, long long o_ss,
                               long long o_sh, const __nv_bfloat16* __restrict__ d_o,
                               long long do_sb, long long do_ss, long long do_sh,
                               const float* __restrict__ lse, long long lse_sb, long long lse_sh,
                               long long lse_ss, float* __restrict__ lse2,
                               float* __restrict__ delta, int B, int H, int Sq, int Sq_pad,
                               const int* __restrict__ cu_q) {
  grid_dep_wait();
  grid_dep_launch();
  __shared__ float s_delta[PRE_HEADS][PRE_ROWS + 1];
  const int head_tiles = (H + PRE_HEADS - 1) / PRE_HEADS;
  const int row_tiles = Sq_pad / PRE_ROWS;
  long long blk = blockIdx.x;
  const int h0 = static_cast<int>(blk % head_tiles) * PRE_HEADS;
  blk /= head_tiles;
  const int row0 = static_cast<int>(blk % row_tiles) * PRE_ROWS;
  const int b = static_cast<int>(blk / row_tiles);
  if (b >= B) return;
  // packed layout: the rows of sequence b start at cu_q[b] of a single batch
  long long gbase = 0, gb = b;
  int len = Sq;
  if (cu_q != nullptr) {
    const int base = cu_q[b];
    len = min(cu_q[b + 1] - base, Sq);  // a sequence longer than the bound is cut there
    gbase = base;
    gb = 0;
  }
  const int hw = threadIdx.x >> 4, sub = threadIdx.x & 15;
  {
    const int h = h0 + hw;
    const __nv_bfloat16* po = o + gb * o_sb + (gbase + row0) * o_ss + h * o_sh + sub * 8;
    const __nv_bfloat16* pd = d_o + gb * do_sb + (gbase + row0) * do_ss + h * do_sh + sub * 8;
#pragma unroll
    for (int half = 0; half < PRE_ROWS / 8; ++half) {
      uint4 vo[8], vd[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rl = half * 8 + i;
        const bool in = h < H && row0 + rl < len;
        vo[i] = in ? ld_nc_v4(po + rl * o_ss) : make_uint4(0u, 0u, 0u, 0u);
        vd[i] = in ? ld_nc_v4(pd + rl * do_ss) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float dl = bf16_lo(vo[i].x) * bf16_lo(vd[i].x) + bf16_hi(vo[i].x) * bf16_hi(vd[i].x) +
                   bf16_lo(vo[i].y) * bf16_lo(vd[i].y) + bf16_hi(vo[i].y) * bf16_hi(vd[i].y) +
                   bf16_lo(vo[i].z) * bf16_lo(vd[i].z) + bf16_hi(vo[i].z) * bf16_hi(vd[i].z) +
                   bf16_lo(vo[i].w) * bf16_lo(vd[i].w) + bf16_hi(vo[i].w) * bf16_hi(vd[i].w);
#pragma unroll
        for (int s = 8; s > 0; s >>= 1) dl += __shfl_xor_sync(0xffffffffu, dl, s);
        if (sub == 0) s_delta[hw][half * 8 + i] = dl;
      }
    }
  }
  __syncthreads();
  {
    const int hl = threadIdx.x / PRE_ROWS, rl = threadIdx.x % PRE_ROWS;
    const int h = h0 + hl, row = row0 + rl;
    if (hl < PRE_HEADS && h < H) {
      float l2 = INFINITY;
      if (row < len) {
        const float l = lse[gb * lse_sb + h * lse_sh + (gbase + row) * lse_ss];
        l2 = l == -INFINITY ? INFINITY : l * 1.4426950408889634f;
      }
      const long long item = (static_cast<long long>(b) * H + h) * Sq_pad + row;
      lse2[item] = l2;
      delta[item] = s_delta[hl][rl];
    }
  }
}


// ---------------------------------------------------------------- dK / dV kernel
// Order of the one-shot CTAs.  A CTA's length is the number of blocks its own block sees, which
// under the causal mask runs from all of them down to one, and the hardware places CTAs in index
// order as SMs free up: the grid is one-dimensional and counts, within a chunk of `chunk` (head,
// batch) pairs, the longest block of every pair first, then the second longest, ...; so the
// launch ends on its shortest CTAs instead of on a full-length one, and a chunk's Q, dO, K, V
// (sized to stay in L2) are re-read from L2 by the CTAs that follow.  `rank` is the block's place in
// the order longest-first, `hb` the (head, batch) pair.
__device__ __forceinline__ void cta_coords(int linear, int blocks, int heads_total, int chunk, int tail,
                                           int& rank, int& hb) {
  // The last `tail` pairs form one chunk (see tail_pairs_of): the launch should end on many short
  // items, not on the long ones of a small last chunk.
  const int body = heads_total - tail;
  int first, in_chunk, r;
  if (linear >= body * blocks) {
    first = body;
    in_chunk = tail;
    r = linear - body * blocks;
  } else {
    const int per_chunk = chunk * blocks;
    const int c = linear / per_chunk;
    r = linear - c * per_chunk;
    first = c * chunk;
    in_chunk = chunk;
  }
  rank = r / in_chunk;
  hb = first + (r - rank * in_chunk);
}

// ROPE: the inverse rotary rotation runs in the store epilogue (p.rope is set).  A template
// parameter, not a branch on p.rope: with the branch the compiler kept the rotation's registers
// alive through the main loop of both paths (108 against 28 bytes of spills in the persistent
// dK/dV kernel, 0.494 against 0.459 ms per call WITHOUT the rotation at B 8, S 2048).
template <bool ROPE>
__global__ void __launch_bounds__(THREADS, 1)
    attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmap_q,
                         const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v,
                         const __grid_constant__ CUtensorMap tmap_do,
                         const __grid_constant__ CUtensorMap tmap_dk,
                         const __grid_constant__ CUtensorMap tmap_dv, const Params p_in) {
  // Per-sequence view: in the packed layout a sequence has its own lengths and its rows start at
  // q_base / k_base of a single batch (bt = 0).  Rows a tile loads beyond its sequence belong to
  // the next one: keys beyond Sk are masked, queries beyond Sq carry lse2 = +inf (P = 0), and
  // neither is stored.
  Params p = p_in;
  int cta_rank, cta_hb;
  cta_coords(static_cast<int>(blockIdx.x), p_in.kv_blocks, p_in.kv_heads_total, p_in.kv_chunk, p_in.kv_tail, cta_rank, cta_hb);
  const int cta_b = cta_hb / p_in.Hkv;
  int q_base = 0, k_base = 0, bt = cta_b;
  if (p_in.cu_q != nullptr) {
    grid_dep_wait();  // the sequence offsets may come from the previous kernel of the stream
    q_base = p_in.cu_q[cta_b];
    p.Sq = p_in.cu_q[cta_b + 1] - q_base;
    k_base = p_in.cu_k[cta_b];
    p.Sk = p_in.cu_k[cta_b + 1] - k_base;
    bt = 0;
    // The grids and the statistics scratch are sized with the caller's bounds: a longer sequence
    // is cut at the bound (nothing beyond the scratch is touched) and reported.
    if (p.Sq > p_in.Sq || p.Sk > p_in.Sk) {
      if (threadIdx.x == 0) atomicExch(p.status, STATUS_SEQ_EXCEEDS_BOUND);
      p.Sq = min(p.Sq, p_in.Sq);
      p.Sk = min(p.Sk, p_in.Sk);
    }
  }
  // Shared memory is used to the last kilobytes, so there is no room for manual alignment slack:
  // the 1024-byte alignment the swizzled tiles need is requested from the compiler and verified.
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(p.status, 901);
    return;
  }
  uint8_t* s_k = smem;
  uint8_t* s_v = smem + TILE_BYTES;
  uint8_t* s_q = smem + 2 * TILE_BYTES;   // 2 stages
  uint8_t* s_do = smem + 4 * TILE_BYTES;  // 2 stages
  float* s_lse = reinterpret_cast<float*>(smem + 6 * TILE_BYTES);  // [2][128]
  float* s_delta = s_lse + 2 * 128;                                // [2][128]
  KvBarriers* bars = reinterpret_cast<KvBarriers*>(s_delta + 2 * 128);
  volatile int* abort_word = &bars->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_blk = cta_rank;  // key block 0 is seen by every query block: the longest CTA
  const int kvh = cta_hb % p_in.Hkv;
  const int b = cta_b;
  const int key0 = n_blk * BKV;
  const int group = p.H / p.Hkv;
  const int shift = p.Sk - p.Sq;  // query i sees keys <= i + shift
  const int num_q_blocks = (p.Sq + BQ - 1) / BQ;
  const int m_start = p.causal ? max(0, key0 - shift) / BQ : 0;
  const int m_count = max(0, num_q_blocks - m_start);
  // iteration it -> head kvh * group + it / m_count, query block m_start + it % m_count
  const int iters = key0 < p.Sk ? m_count * group : 0;  // (a key block beyond a packed sequence)

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->q_full[i], 1);
      mbar_init(&bars->q_empty[i], 1);
      mbar_init(&bars->do_full[i], 1);
      mbar_init(&bars->do_empty[i], 1);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->dp_full, 1);
    // One arrival per compute warp: the arrivals of all 256 threads on one barrier word are
    // serialised (measured in the forward kernel: ~500 clk for 128 of them).
    mbar_init(&bars->p_ready, 8);
    mbar_init(&bars->ds_ready, 8);
    mbar_init(&bars->dv_done, 1);
    mbar_init(&bars->dk_done, 1);
    bars->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_do);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  grid_dep_wait();  // the set-up above overlaps the previous kernel's tail; global memory from here on
  grid_dep_launch();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    setmaxnreg_dec<KV_LOW_REGS>();
    if (elect_one() && iters > 0) {
      mbar_arrive_expect_tx(&bars->kv_full, 2 * TILE_BYTES);
#pragma unroll
      for (int dh = 0; dh < 2; ++dh) {
        tma_load_4d(s_k + dh * PANEL_BYTES, &tmap_k, &bars->kv_full, dh * 64, k_base + key0, kvh, bt);
        tma_load_4d(s_v + dh * PANEL_BYTES, &tmap_v, &bars->kv_full, dh * 64, k_base + key0, kvh, bt);
      }
      for (int it = 0; it < iters; ++it) {
        const int h = kvh * group + it / m_count;
        const int q0 = (m_start + it % m_count) * BQ;
        const int s = it & 1;
        const uint32_t ph = ((it >> 1) & 1) ^ 1;
        if (!mbar_wait(&bars->q_empty[s], ph, abort_word, 121)) break;
        mbar_arrive_expect_tx(&bars->q_full[s], TILE_BYTES);
#pragma unroll
        for (int dh = 0; dh < 2; ++dh)
          tma_load_4d(s_q + s * TILE_BYTES + dh * PANEL_BYTES, &tmap_q, &bars->q_full[s], dh * 64,
                      q_base + q0, h, bt);
        if (!mbar_wait(&bars->do_empty[s], ph, abort_word, 122)) break;
        mbar_arrive_expect_tx(&bars->do_full[s], TILE_BYTES);
#pragma unroll
        for (int dh = 0; dh < 2; ++dh)
          tma_load_4d(s_do + s * TILE_BYTES + dh * PANEL_BYTES, &tmap_do, &bars->do_full[s],
                      dh * 64, q_base + q0, h, bt);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // Issue order: dV(it), S^T(it+1), dK(it), dP^T(it+1): the products of the next query block
    // that do not depend on this block's dS^T are issued before the one that does, so the
    // compute warps always find their next input ready.
    setmaxnreg_dec<KV_LOW_REGS>();
    if (elect_one() && iters > 0) {
      const uint32_t idesc_kk = make_idesc_bf16(128, 128, 0, 0);  // both operands K-major
      const uint32_t idesc_kmn = make_idesc_bf16(128, 128, 0, 1); // A K-major / TMEM, B MN-major
      const uint32_t k_lo = desc_lo(smem_u32(s_k), 16), v_lo = desc_lo(smem_u32(s_v), 16);
      const uint32_t q_lo = desc_lo(smem_u32(s_q), 16), do_lo = desc_lo(smem_u32(s_do), 16);
      const uint32_t q_mn_lo = desc_lo(smem_u32(s_q), PANEL_BYTES), do_mn_lo = desc_lo(smem_u32(s_do), PANEL_BYTES);
      const uint32_t d_s = tmem_base + KV_COL_S, d_dp = tmem_base + KV_COL_DP;
      const uint32_t d_dv = tmem_base + KV_COL_DV, d_dk = tmem_base + KV_COL_DK;
      auto issue_s = [&](uint32_t stage) {  // S^T = K Q^T
        const uint32_t qa = q_lo + stage * (TILE_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(d_s, desc_at(k_lo, koff_k(k)), desc_at(qa, koff_k(k)), idesc_kk, k != 0);
        umma_commit(&bars->s_full);
      };
      auto issue_dp = [&](uint32_t stage) {  // dP^T = V dO^T
        const uint32_t da = do_lo + stage * (TILE_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(d_dp, desc_at(v_lo, koff_k(k)), desc_at(da, koff_k(k)), idesc_kk, k != 0);
        umma_commit(&bars->dp_full);
      };
      bool ok = mbar_wait(&bars->kv_full, 0, abort_word, 221) &&
                mbar_wait(&bars->q_full[0], 0, abort_word, 222);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        ok = mbar_wait(&bars->do_full[0], 0, abort_word, 223);
      }
      if (ok) {
        tc_fence_after();
        issue_dp(0);
      }
      for (int it = 0; it < iters && ok; ++it) {
        const uint32_t s = it & 1;
        const uint32_t ph = it & 1;
        const bool has_next = it + 1 < iters;
        if (has_next) {  // Q and dO of the next block: loaded an iteration ago as a rule
          const uint32_t ph_next = ((it + 1) >> 1) & 1;
          ok = mbar_wait(&bars->q_full[s ^ 1], ph_next, abort_word, 227) &&
               mbar_wait(&bars->do_full[s ^ 1], ph_next, abort_word, 228);
          if (!ok) break;
        }
        const uint32_t acc = it > 0 ? 1u : 0u;
        const uint32_t qf = q_mn_lo + s * (TILE_BYTES >> 4), df = do_mn_lo + s * (TILE_BYTES >> 4);
        // dV += P^T dO  (A = P^T from TMEM)
        ok = mbar_wait(&bars->p_ready, ph, abort_word, 225);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ts(d_dv, d_s + acol(k), desc_at(df, koff_mn(k)), idesc_kmn, k != 0 ? 1u : acc);
        umma_commit(&bars->do_empty[s]);  // dP^T(it) and dV(it) were the readers of this dO stage
        if (!has_next) umma_commit(&bars->dv_done);  // dV is final: its rows leave while dK finishes
        // S^T of the next query block; it overwrites P^T, which dV (issued above) reads first.
        if (has_next) issue_s(s ^ 1);
        // dK += dS^T Q  (A = dS^T from TMEM, written over dP^T)
        ok = mbar_wait(&bars->ds_ready, ph, abort_word, 226);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ts(d_dk, d_dp + acol(k), desc_at(qf, koff_mn(k)), idesc_kmn, k != 0 ? 1u : acc);
        umma_commit(&bars->q_empty[s]);
        // dP^T of the next block overwrites dS^T, which dK (issued above) reads first.
        if (has_next) issue_dp(s ^ 1);
      }
      if (ok) umma_commit(&bars->dk_done);
    }
  } else if (warp < 4) {
    setmaxnreg_dec<KV_LOW_REGS>();
  } else {
    // ------------------------------------------------------------ compute warps (4..11)
    // Per iteration: dS^T(it) from dP^T(it) and the P^T kept in registers, then P^T(it+1), which
    // overlaps the dK product of this block.
    setmaxnreg_inc<KV_HIGH_REGS>();
    const int ct = threadIdx.x - 128;  // 0..255
    const int wg = (warp - 4) >> 2;    // column (query) half this thread works on
    const int quad = warp & 3;
    const int r = quad * 32 + lane;    // key row inside the block == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int key = key0 + r;
    bool ok = true;

    auto it_head = [&](int it) { return kvh * group + it / m_count; };
    auto it_q0 = [&](int it) { return (m_start + it % m_count) * BQ; };
    // Row statistics of iteration `it`: threads 0..127 fetch LSE2, 128..255 fetch delta.
    auto fetch_stat = [&](int it) -> float {
      const long long base = (static_cast<long long>(b) * p.H + it_head(it)) * p.Sq_pad + it_q0(it);
      return ct < 128 ? p.lse2[base + ct] : p.delta[base + ct - 128];
    };
    auto store_stat = [&](int stage, float v) {
      if (ct < 128) s_lse[stage * 128 + ct] = -v;  // negated: it is the addend of a packed FMA
      else s_delta[stage * 128 + ct - 128] = v;
    };
    float pr[64];

    // P^T(it) = exp2(S^T * scale_log2 - lse2) -> registers (f32) and TMEM (bf16)
    auto p_phase = [&](int it) -> bool {
      const int q0 = it_q0(it);
      const float4* lse_s = reinterpret_cast<const float4*>(s_lse + (it & 1) * 128 + wg * 64);
      const bool need_mask = (p.causal && key0 + BKV - 1 > q0 + shift) || key0 + BKV > p.Sk;
      if (!mbar_wait(&bars->s_full, it & 1, abort_word, 321)) return false;
      tc_fence_after();
      {
        uint32_t sr[2][32];
        tmem_ld32(tmem_base + lane_addr + KV_COL_S + wg * 64, sr[0]);
        tmem_ld32(tmem_base + lane_addr + KV_COL_S + wg * 64 + 32, sr[1]);
        tmem_wait_ld();
        float x[64];
        const uint64_t scale2 = pk2(p.scale_log2, p.scale_log2);
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4) {
          const float4 l4 = lse_s[c4];  // the statistics are stored negated (store_stat)
          const int c = c4 * 4;
          upk2(fma_x2(pk2(__uint_as_float(sr[c >> 5][c & 31]), __uint_as_float(sr[c >> 5][(c & 31) + 1])), scale2,
                      pk2(l4.x, l4.y)),
               x[c], x[c + 1]);
          upk2(fma_x2(pk2(__uint_as_float(sr[c >> 5][(c & 31) + 2]), __uint_as_float(sr[c >> 5][(c & 31) + 3])), scale2,
                      pk2(l4.z, l4.w)),
               x[c + 2], x[c + 3]);
        }
        exp2_row64(x, pr);
        if (need_mask) {  // warp-uniform; only blocks on the diagonal or at the end of the keys
#pragma unroll
          for (int c = 0; c < 64; ++c) {
            const int qrow = q0 + wg * 64 + c;
            if (key >= p.Sk || (p.causal && key > qrow + shift)) pr[c] = 0.f;
          }
        }
      }
      {
        // P^T (bf16 pairs) of this thread's 64 queries goes over the first 32 of the 64 S^T columns
        // it has just read (queries 0-63 in columns [0,32), queries 64-127 in columns [64,96)), so
        // the two column halves need no barrier between their loads and stores.
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) pk[c] = pack_bf16x2(pr[2 * c], pr[2 * c + 1]);
        tmem_st32(tmem_base + lane_addr + KV_COL_S + wg * 64, pk);
        tmem_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_ready);
      return true;
    };

    float stat_next = 0.f;
    if (iters > 0) store_stat(0, fetch_stat(0));
    if (iters > 1) stat_next = fetch_stat(1);
    compute_bar_sync();
    if (iters > 0) ok = p_phase(0);
    if (iters > 1) store_stat(1, stat_next);
    compute_bar_sync();

    for (int it = 0; it < iters && ok; ++it) {
      const uint32_t ph = it & 1;
      if (it + 2 < iters) stat_next = fetch_stat(it + 2);  // lands while this iteration computes

      // ---- dS^T / scale = P^T o (dP^T - delta)  -> TMEM (bf16) over the dP^T columns
      if (!mbar_wait(&bars->dp_full, ph, abort_word, 322)) { ok = false; break; }
      tc_fence_after();
      {
        const float4* delta_s = reinterpret_cast<const float4*>(s_delta + (it & 1) * 128 + wg * 64);
        uint32_t dr[2][32];
        tmem_ld32(tmem_base + lane_addr + KV_COL_DP + wg * 64, dr[0]);
        tmem_ld32(tmem_base + lane_addr + KV_COL_DP + wg * 64 + 32, dr[1]);
        tmem_wait_ld();
        uint32_t pk[32];
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const float4 d0 = delta_s[ch * 2], d1 = delta_s[ch * 2 + 1];
          const float dl[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
          float d[8];
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            const int c = ch * 8 + j;
            // (scale: dK epilogue)
            upk2(mul_x2(pk2(pr[c], pr[c + 1]),
                        sub_x2(pk2(__uint_as_float(dr[c >> 5][c & 31]), __uint_as_float(dr[c >> 5][(c & 31) + 1])),
                               pk2(dl[j], dl[j + 1]))),
                 d[j], d[j + 1]);
          }
          pk[ch * 4 + 0] = pack_bf16x2(d[0], d[1]);
          pk[ch * 4 + 1] = pack_bf16x2(d[2], d[3]);
          pk[ch * 4 + 2] = pack_bf16x2(d[4], d[5]);
          pk[ch * 4 + 3] = pack_bf16x2(d[6], d[7]);
        }
        // dS^T (bf16 pairs) goes over the first 32 of the 64 dP^T columns this thread has read,
        // like P^T over S^T: the dK product reads its A operand from tensor memory (a TS MMA
        // issues every ~82 clk, an SS one every ~112 clk), and no shared-memory tile, proxy fence
        // or barrier between the two column halves is needed.
        tmem_st32(tmem_base + lane_addr + KV_COL_DP + wg * 64, pk);
        tmem_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->ds_ready);

      // ---- P^T of the next query block (overlaps the dK product of this one)
      if (it + 1 < iters && !p_phase(it + 1)) { ok = false; break; }

      // Statistics of iteration it + 2 replace those of iteration it (all reads of them are
      // behind the barrier inside p_phase above or, for the last iterations, behind this one).
      compute_bar_sync();
      if (it + 2 < iters) store_stat(it & 1, stat_next);
      compute_bar_sync();
    }

    // ---- epilogue: dV and dK rows of this key block
    RopeUnits rope_units;  // the table values of the inverse rotation: on their way while dV is staged
    if (ROPE) rope_units_load(p.rope, key0, p.rope_rows, ct, rope_units);
    if (ok && iters > 0) {
      ok = mbar_wait(&bars->dv_done, 0, abort_word, 325);
      tc_fence_after();
    }
    if (ok) {
      // The tiles go out through shared memory and one TMA store per 64-column panel: a thread
      // owns a row, so direct stores would touch 32 rows per instruction.  The staging tiles are
      // operand stages whose readers have completed; the panel layout is the loads' 128-byte swizzle.  A store
      // clips rows beyond the tensor, not rows of the next packed sequence: a partial block of a
      // packed sequence stores its rows directly.
      const bool staged = p.cu_k == nullptr || key0 + BKV <= p.Sk;
      const bool row_ok = key < p.Sk;
      __nv_bfloat16* dv_row = p.dv + bt * p.dv_sb + static_cast<long long>(k_base + key) * p.dv_ss + kvh * p.dv_sh + wg * 64;
      __nv_bfloat16* dk_row = p.dk + bt * p.dk_sb + static_cast<long long>(k_base + key) * p.dk_ss + kvh * p.dk_sh + wg * 64;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = which == 0 ? dv_row : dk_row;
        // dV is staged in a dO stage (dV's own products were their last readers) while the last
        // dK product may still read Q; dK, once that product is done, in a Q stage.
        if (which == 1 && iters > 0) {
          if (!mbar_wait(&bars->dk_done, 0, abort_word, 324)) break;
          tc_fence_after();
        }
        uint8_t* stage = which == 0 ? s_do : s_q;
        uint8_t* stage_row = stage + wg * PANEL_BYTES + r * 128;
        const uint32_t col = (which == 0 ? KV_COL_DV : KV_COL_DK) + wg * 64;
        const bool rotate = which == 1 && ROPE;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t a[32];
          if (iters > 0) {
            tmem_ld32(tmem_base + lane_addr + col + half * 32, a);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) a[i] = 0u;
          }
          const float sc = which == 0 ? 1.0f : p.scale;  // dS^T was accumulated without the scale
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 q;
            q.x = pack_bf16x2(__uint_as_float(a[g * 8 + 0]) * sc, __uint_as_float(a[g * 8 + 1]) * sc);
            q.y = pack_bf16x2(__uint_as_float(a[g * 8 + 2]) * sc, __uint_as_float(a[g * 8 + 3]) * sc);
            q.z = pack_bf16x2(__uint_as_float(a[g * 8 + 4]) * sc, __uint_as_float(a[g * 8 + 5]) * sc);
            q.w = pack_bf16x2(__uint_as_float(a[g * 8 + 6]) * sc, __uint_as_float(a[g * 8 + 7]) * sc);
            if (staged || rotate)
              *reinterpret_cast<uint4*>(stage_row + (((half * 4 + g) ^ (r & 7)) << 4)) = q;
            else if (row_ok)
              *reinterpret_cast<uint4*>(dst + half * 32 + g * 8) = q;
          }
        }
        if (rotate) {
          // dK of the keys before the rotary rotation: the staged rows are rotated back in place
          compute_bar_sync();
          rope_inverse_apply(stage, ct, rope_units, staged, dst - wg * 64 - r * p.dk_ss, p.dk_ss, p.Sk - key0);
        }
        if (staged) {
          fence_proxy_async_smem();
          compute_bar_sync();
          if (ct == 0) {
            const CUtensorMap* tm = which == 0 ? &tmap_dv : &tmap_dk;
            tma_store_4d(tm, stage, 0, k_base + key0, kvh, bt);
            tma_store_4d(tm, stage + PANEL_BYTES, 64, k_base + key0, kvh, bt);
            tma_store_commit();
          }
        }
      }
      if (staged && ct == 0) tma_store_wait_read<0>();  // shared memory is read before the CTA ends
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
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_word != 0) atomicExch(p.status, *abort_word);
}

// ---------------------------------------------------------------- dK / dV kernel, persistent form
// The same tile program as attn_bwd_dkdv_kernel, run by one CTA per SM over many (key block, kv
// head, batch) items, so that what a one-shot CTA pays per item -- its launch, the tensor-memory
// allocation, the first operand loads and the first two products before any compute warp has
// work -- happens under the previous item's last query block and store epilogue:
//   * items are numbered in the order of cta_coords (longest first inside an L2-sized chunk) and
//     drawn from a counter by the producer lane, which publishes them through a small ring in
//     shared memory (-1: no further item);
//   * all barrier phases count query blocks (or items) across items;
//   * K is free for the next item's load once the item's last S^T has run, V once its last dP^T
//     has (k_free / v_free, committed by the issuing lane one query block before the item ends),
//     and the next item's first Q / dO go to the stage the last query block does not use;
//   * the issuing lane starts S^T and dP^T of the next item's first query block right behind the
//     last dK product; dV and dK leave tensor memory (staged in the dO / Q stage of the item's
//     last query block, which the storing thread releases when the TMA stores have read it)
//     before the compute warps write the next item's first P^T, and the products that overwrite
//     the accumulators wait for that P^T / dS^T -- so the accumulators need no barrier of
//     their own.
constexpr int KVP_SLOTS = 4;
struct KvpBarriers {
  uint64_t kv_full, k_free, v_free;
  uint64_t q_full[2], q_empty[2], do_full[2], do_empty[2];
  uint64_t s_full, dp_full, p_ready, ds_ready, dv_done, dk_done;
  uint64_t item_full[KVP_SLOTS], item_read[KVP_SLOTS];
  int item_ring[KVP_SLOTS];
  uint32_t tmem_base;
  int abort_word;
};
constexpr size_t KVP_SMEM_BYTES = 6 * TILE_BYTES + 2 * 2 * 128 * sizeof(float) + sizeof(KvpBarriers);
static_assert(KVP_SMEM_BYTES <= 232448, "exceeds the 227 KiB of shared memory a CTA can opt in to");

// One item: key block `key0` of kv head `kvh` of sequence `b`, walked over `iters` query blocks
// (query block m_start + it % m_count of head kvh * group + it / m_count).
struct KvItem {
  int b, kvh, bt, key0, q_base, k_base, Sq, Sk, shift, m_start, m_count, iters;
  bool exceeds;  // a packed sequence longer than the bound the launch was sized with
};
__device__ __forceinline__ KvItem kv_item_of(const Params& p, int idx) {
  KvItem v;
  int rank, hb;
  cta_coords(idx, p.kv_blocks, p.kv_heads_total, p.kv_chunk, p.kv_tail, rank, hb);
  v.b = hb / p.Hkv;
  v.kvh = hb - v.b * p.Hkv;
  v.bt = v.b;
  v.q_base = 0;
  v.k_base = 0;
  v.Sq = p.Sq;
  v.Sk = p.Sk;
  v.exceeds = false;
  if (p.cu_q != nullptr) {
    v.q_base = p.cu_q[v.b];
    v.Sq = p.cu_q[v.b + 1] - v.q_base;
    v.k_base = p.cu_k[v.b];
    v.Sk = p.cu_k[v.b + 1] - v.k_base;
    v.bt = 0;
    if (v.Sq > p.Sq || v.Sk > p.Sk) {
      v.exceeds = true;
      v.Sq = min(v.Sq, p.Sq);
      v.Sk = min(v.Sk, p.Sk);
    }
  }
  v.key0 = rank * BKV;
  v.shift = v.Sk - v.Sq;
  const int num_q_blocks = (v.Sq + BQ - 1) / BQ;
  v.m_start = p.causal ? max(0, v.key0 - v.shift) / BQ : 0;
  v.m_count = max(0, num_q_blocks - v.m_start);
  v.iters = v.key0 < v.Sk ? v.m_count * (p.H / p.Hkv) : 0;
  return v;
}
// Items of a CTA when no counter is available: a boustrophedon deal of the longest-first order.
__device__ __forceinline__ int kvp_fixed_item(int k, int cid, int nc, int total) {
  if (static_cast<long long>(k) * nc >= total) return -1;
  const int idx = k * nc + ((k & 1) ? nc - 1 - cid : cid);
  return idx < total ? idx : -1;
}

template <bool ROPE>  // see attn_bwd_dkdv_kernel
__global__ void __launch_bounds__(THREADS, 1)
    attn_bwd_dkdv_persistent_kernel(const __grid_constant__ CUtensorMap tmap_q,
                                    const __grid_constant__ CUtensorMap tmap_k,
                                    const __grid_constant__ CUtensorMap tmap_v,
                                    const __grid_constant__ CUtensorMap tmap_do,
                                    const __grid_constant__ CUtensorMap tmap_dk,
                                    const __grid_constant__ CUtensorMap tmap_dv, const Params p,
                                    unsigned int* item_counter) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(p.status, 901);
    return;
  }
  uint8_t* s_k = smem;
  uint8_t* s_v = smem + TILE_BYTES;
  uint8_t* s_q = smem + 2 * TILE_BYTES;   // 2 stages
  uint8_t* s_do = smem + 4 * TILE_BYTES;  // 2 stages
  float* s_lse = reinterpret_cast<float*>(smem + 6 * TILE_BYTES);  // [2][128]
  float* s_delta = s_lse + 2 * 128;                                // [2][128]
  KvpBarriers* bars = reinterpret_cast<KvpBarriers*>(s_delta + 2 * 128);
  volatile int* abort_word = &bars->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int group = p.H / p.Hkv;
  const int total = p.kv_blocks * p.kv_heads_total;
  const int nc = static_cast<int>(gridDim.x), cid = static_cast<int>(blockIdx.x);

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    mbar_init(&bars->k_free, 1);
    mbar_init(&bars->v_free, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->q_full[i], 1);
      mbar_init(&bars->q_empty[i], 1);
      mbar_init(&bars->do_full[i], 1);
      mbar_init(&bars->do_empty[i], 1);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->p_ready, 8);  // one arrival per compute warp
    mbar_init(&bars->ds_ready, 8);
    mbar_init(&bars->dv_done, 1);
    mbar_init(&bars->dk_done, 1);
    for (int i = 0; i < KVP_SLOTS; ++i) {
      mbar_init(&bars->item_full[i], 1);
      mbar_init(&bars->item_read[i], 9);  // the issuing lane and the eight compute warps
    }
    bars->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_do);
    tma_prefetch_desc(&tmap_dk);
    tma_prefetch_desc(&tmap_dv);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  grid_dep_wait();  // the set-up above overlaps the previous kernel's tail; global memory from here on
  grid_dep_launch();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (and item hand-out)
    setmaxnreg_dec<KV_LOW_REGS>();
    if (elect_one()) {
      // Every item is drawn, a CTA's first one too: a CTA that finds its SM late (another kernel
      // holds it, e.g. a collective of a data-parallel step) then finds nothing left instead of
      // running one of the longest items after everybody else has finished.  A CTA draws until a
      // draw runs past the last item; the launch's last draw puts the counter back to zero.
      const unsigned total_draws = static_cast<unsigned>(total) + static_cast<unsigned>(nc);
      int idx = -1;
      unsigned drawn = item_counter != nullptr ? atomicAdd(item_counter, 1u) : 0u;
      uint32_t g = 0, kvn = 0;  // query blocks / non-empty items so far
      bool ok = true;
      for (int k = 0; ok; ++k) {
        if (item_counter != nullptr) {
          idx = drawn < static_cast<unsigned>(total) ? static_cast<int>(drawn) : -1;
          if (drawn + 1 == total_draws) atomicExch(item_counter, 0u);
        } else {
          idx = kvp_fixed_item(k, cid, nc, total);
        }
        if (k >= KVP_SLOTS &&
            !mbar_wait(&bars->item_read[k % KVP_SLOTS], ((k / KVP_SLOTS) - 1) & 1, abort_word, 124)) {
          ok = false;
          break;
        }
        bars->item_ring[k % KVP_SLOTS] = idx;
        mbar_arrive(&bars->item_full[k % KVP_SLOTS]);
        if (idx < 0) break;
        const KvItem v = kv_item_of(p, idx);
        if (v.exceeds) atomicExch(p.status, STATUS_SEQ_EXCEEDS_BOUND);
        if (v.iters > 0) {
          ok = mbar_wait(&bars->k_free, (kvn & 1) ^ 1, abort_word, 125) &&
               mbar_wait(&bars->v_free, (kvn & 1) ^ 1, abort_word, 126);
          if (!ok) break;
          ++kvn;
          mbar_arrive_expect_tx(&bars->kv_full, 2 * TILE_BYTES);
#pragma unroll
          for (int dh = 0; dh < 2; ++dh) {
            tma_load_4d(s_k + dh * PANEL_BYTES, &tmap_k, &bars->kv_full, dh * 64, v.k_base + v.key0, v.kvh, v.bt);
            tma_load_4d(s_v + dh * PANEL_BYTES, &tmap_v, &bars->kv_full, dh * 64, v.k_base + v.key0, v.kvh, v.bt);
          }
          int h = v.kvh * group, m = v.m_start;
          for (int it = 0; it < v.iters; ++it, ++g) {
            const int q0 = m * BQ;
            const int s = g & 1;
            const uint32_t ph = ((g >> 1) & 1) ^ 1;
            if (!mbar_wait(&bars->q_empty[s], ph, abort_word, 121)) { ok = false; break; }
            mbar_arrive_expect_tx(&bars->q_full[s], TILE_BYTES);
#pragma unroll
            for (int dh = 0; dh < 2; ++dh)
              tma_load_4d(s_q + s * TILE_BYTES + dh * PANEL_BYTES, &tmap_q, &bars->q_full[s], dh * 64,
                          v.q_base + q0, h, v.bt);
            if (!mbar_wait(&bars->do_empty[s], ph, abort_word, 122)) { ok = false; break; }
            mbar_arrive_expect_tx(&bars->do_full[s], TILE_BYTES);
#pragma unroll
            for (int dh = 0; dh < 2; ++dh)
              tma_load_4d(s_do + s * TILE_BYTES + dh * PANEL_BYTES, &tmap_do, &bars->do_full[s],
                          dh * 64, v.q_base + q0, h, v.bt);
            if (++m == v.m_start + v.m_count) {
              m = v.m_start;
              ++h;
            }
          }
        }
        // The next item is drawn when this item's last loads are on their way.
        if (ok && item_counter != nullptr) drawn = atomicAdd(item_counter, 1u);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // Issue order inside an item: dV(it), S^T(it+1), dK(it), dP^T(it+1); behind the last dK of an
    // item come S^T(0) and dP^T(0) of the next one.
    setmaxnreg_dec<KV_LOW_REGS>();
    if (elect_one()) {
      const uint32_t idesc_kk = make_idesc_bf16(128, 128, 0, 0);  // both operands K-major
      const uint32_t idesc_kmn = make_idesc_bf16(128, 128, 0, 1); // A K-major / TMEM, B MN-major
      const uint32_t k_lo = desc_lo(smem_u32(s_k), 16), v_lo = desc_lo(smem_u32(s_v), 16);
      const uint32_t q_lo = desc_lo(smem_u32(s_q), 16), do_lo = desc_lo(smem_u32(s_do), 16);
      const uint32_t q_mn_lo = desc_lo(smem_u32(s_q), PANEL_BYTES), do_mn_lo = desc_lo(smem_u32(s_do), PANEL_BYTES);
      const uint32_t d_s = tmem_base + KV_COL_S, d_dp = tmem_base + KV_COL_DP;
      const uint32_t d_dv = tmem_base + KV_COL_DV, d_dk = tmem_base + KV_COL_DK;
      auto issue_s = [&](uint32_t stage) {  // S^T = K Q^T
        const uint32_t qa = q_lo + stage * (TILE_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(d_s, desc_at(k_lo, koff_k(k)), desc_at(qa, koff_k(k)), idesc_kk, k != 0);
        umma_commit(&bars->s_full);
      };
      auto issue_dp = [&](uint32_t stage) {  // dP^T = V dO^T
        const uint32_t da = do_lo + stage * (TILE_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(d_dp, desc_at(v_lo, koff_k(k)), desc_at(da, koff_k(k)), idesc_kk, k != 0);
        umma_commit(&bars->dp_full);
      };
      uint32_t g = 0, kvn = 0;
      bool ok = true;
      for (int k = 0; ok; ++k) {
        if (!mbar_wait(&bars->item_full[k % KVP_SLOTS], (k / KVP_SLOTS) & 1, abort_word, 224)) break;
        const int idx = bars->item_ring[k % KVP_SLOTS];
        mbar_arrive(&bars->item_read[k % KVP_SLOTS]);
        if (idx < 0) break;
        const int iters = kv_item_of(p, idx).iters;
        if (iters == 0) continue;
        {
          const uint32_t s0 = g & 1, par0 = (g >> 1) & 1;
          ok = mbar_wait(&bars->kv_full, kvn & 1, abort_word, 221) &&
               mbar_wait(&bars->q_full[s0], par0, abort_word, 222);
          if (!ok) break;
          tc_fence_after();
          issue_s(s0);
          if (iters == 1) umma_commit(&bars->k_free);
          ok = mbar_wait(&bars->do_full[s0], par0, abort_word, 223);
          if (!ok) break;
          tc_fence_after();
          issue_dp(s0);
          if (iters == 1) umma_commit(&bars->v_free);
        }
        for (int it = 0; it < iters; ++it, ++g) {
          const uint32_t s = g & 1;
          const uint32_t ph = g & 1;
          const bool has_next = it + 1 < iters;
          if (has_next) {  // Q and dO of the next block: loaded an iteration ago as a rule
            const uint32_t ph_next = ((g + 1) >> 1) & 1;
            ok = mbar_wait(&bars->q_full[s ^ 1], ph_next, abort_word, 227) &&
                 mbar_wait(&bars->do_full[s ^ 1], ph_next, abort_word, 228);
            if (!ok) break;
          }
          const uint32_t acc = it > 0 ? 1u : 0u;
          const uint32_t qf = q_mn_lo + s * (TILE_BYTES >> 4), df = do_mn_lo + s * (TILE_BYTES >> 4);
          // dV += P^T dO  (A = P^T from TMEM).  The first one of an item overwrites the previous
          // item's dV, which the compute warps have read before they wrote this P^T.
          ok = mbar_wait(&bars->p_ready, ph, abort_word, 225);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ts(d_dv, d_s + acol(kk), desc_at(df, koff_mn(kk)), idesc_kmn, kk != 0 ? 1u : acc);
          // dP^T(it) and dV(it) were the readers of this dO stage; after the item's last query
          // block the stage carries dV out and the storing thread releases it.
          if (has_next) {
            umma_commit(&bars->do_empty[s]);
            issue_s(s ^ 1);  // overwrites P^T, which dV (issued above) reads first
            if (it + 2 == iters) umma_commit(&bars->k_free);
          } else {
            umma_commit(&bars->dv_done);
          }
          // dK += dS^T Q  (A = dS^T from TMEM, written over dP^T)
          ok = mbar_wait(&bars->ds_ready, ph, abort_word, 226);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ts(d_dk, d_dp + acol(kk), desc_at(qf, koff_mn(kk)), idesc_kmn, kk != 0 ? 1u : acc);
          if (has_next) {
            umma_commit(&bars->q_empty[s]);
            issue_dp(s ^ 1);  // overwrites dS^T, which dK (issued above) reads first
            if (it + 2 == iters) umma_commit(&bars->v_free);
          } else {
            umma_commit(&bars->dk_done);
          }
        }
        ++kvn;
      }
    }
  } else if (warp < 4) {
    setmaxnreg_dec<KV_LOW_REGS>();
  } else {
    // ------------------------------------------------------------ compute warps (4..11)
    setmaxnreg_inc<KV_HIGH_REGS>();
    const int ct = threadIdx.x - 128;  // 0..255
    const int wg = (warp - 4) >> 2;    // column (query) half this thread works on
    const int quad = warp & 3;
    const int r = quad * 32 + lane;    // key row inside the block == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    bool ok = true;

    // Row statistics of query block `it` of an item: threads 0..127 fetch LSE2, 128..255 delta.
    auto fetch_stat = [&](const KvItem& v, int it) -> float {
      const int hh = it / v.m_count;
      const long long base = (static_cast<long long>(v.b) * p.H + v.kvh * group + hh) * p.Sq_pad +
                             (v.m_start + it - hh * v.m_count) * BQ;
      return ct < 128 ? p.lse2[base + ct] : p.delta[base + ct - 128];
    };
    auto store_stat = [&](uint32_t stage, float x) {
      if (ct < 128) s_lse[stage * 128 + ct] = -x;  // negated: it is the addend of a packed FMA
      else s_delta[stage * 128 + ct - 128] = x;
    };
    auto read_item = [&](int k) -> int {
      if (!mbar_wait(&bars->item_full[k % KVP_SLOTS], (k / KVP_SLOTS) & 1, abort_word, 326)) return -2;
      const int idx = bars->item_ring[k % KVP_SLOTS];
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->item_read[k % KVP_SLOTS]);
      return idx;
    };
    float pr[64];
    uint32_t g = 0, kvn = 0;

    // P^T = exp2(S^T * scale_log2 - lse2) of running query block gi -> registers (f32) and TMEM (bf16)
    auto p_phase = [&](const KvItem& v, int it, uint32_t gi) -> bool {
      const int q0 = (v.m_start + it % v.m_count) * BQ;
      const int key = v.key0 + r;
      const float4* lse_s = reinterpret_cast<const float4*>(s_lse + (gi & 1) * 128 + wg * 64);
      const bool need_mask = (p.causal && v.key0 + BKV - 1 > q0 + v.shift) || v.key0 + BKV > v.Sk;
      if (!mbar_wait(&bars->s_full, gi & 1, abort_word, 321)) return false;
      tc_fence_after();
      {
        uint32_t sr[2][32];
        tmem_ld32(tmem_base + lane_addr + KV_COL_S + wg * 64, sr[0]);
        tmem_ld32(tmem_base + lane_addr + KV_COL_S + wg * 64 + 32, sr[1]);
        tmem_wait_ld();
        float x[64];
        const uint64_t scale2 = pk2(p.scale_log2, p.scale_log2);
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4) {
          const float4 l4 = lse_s[c4];  // the statistics are stored negated (store_stat)
          const int c = c4 * 4;
          upk2(fma_x2(pk2(__uint_as_float(sr[c >> 5][c & 31]), __uint_as_float(sr[c >> 5][(c & 31) + 1])), scale2,
                      pk2(l4.x, l4.y)),
               x[c], x[c + 1]);
          upk2(fma_x2(pk2(__uint_as_float(sr[c >> 5][(c & 31) + 2]), __uint_as_float(sr[c >> 5][(c & 31) + 3])), scale2,
                      pk2(l4.z, l4.w)),
               x[c + 2], x[c + 3]);
        }
        exp2_row64(x, pr);
        if (need_mask) {  // warp-uniform; only blocks on the diagonal or at the end of the keys
#pragma unroll
          for (int c = 0; c < 64; ++c) {
            const int qrow = q0 + wg * 64 + c;
            if (key >= v.Sk || (p.causal && key > qrow + v.shift)) pr[c] = 0.f;
          }
        }
      }
      {
        // P^T (bf16 pairs) goes over the first 32 of the 64 S^T columns this thread has read
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) pk[c] = pack_bf16x2(pr[2 * c], pr[2 * c + 1]);
        tmem_st32(tmem_base + lane_addr + KV_COL_S + wg * 64, pk);
        tmem_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_ready);
      return true;
    };

    int idx = read_item(0);
    KvItem v;
    float st0 = 0.f, st1 = 0.f;  // statistics of the item's first two query blocks
    if (idx >= 0) {
      v = kv_item_of(p, idx);
      if (v.iters > 0) st0 = fetch_stat(v, 0);
      if (v.iters > 1) st1 = fetch_stat(v, 1);
    }
    for (int k = 0; idx >= 0 && ok; ++k) {
      const int iters = v.iters;
      const int key = v.key0 + r;
      if (iters > 0) {
        store_stat(g & 1, st0);
        if (iters > 1) store_stat((g + 1) & 1, st1);
        compute_bar_sync();
        ok = p_phase(v, 0, g);
        float stat_next = 0.f;
        for (int it = 0; it < iters && ok; ++it) {
          const uint32_t gi = g + it;
          const uint32_t ph = gi & 1;
          if (it + 2 < iters) stat_next = fetch_stat(v, it + 2);  // lands while this iteration computes

          // ---- dS^T / scale = P^T o (dP^T - delta)  -> TMEM (bf16) over the dP^T columns
          if (!mbar_wait(&bars->dp_full, ph, abort_word, 322)) { ok = false; break; }
          tc_fence_after();
          {
            const float4* delta_s = reinterpret_cast<const float4*>(s_delta + (gi & 1) * 128 + wg * 64);
            uint32_t dr[2][32];
            tmem_ld32(tmem_base + lane_addr + KV_COL_DP + wg * 64, dr[0]);
            tmem_ld32(tmem_base + lane_addr + KV_COL_DP + wg * 64 + 32, dr[1]);
            tmem_wait_ld();
            uint32_t pk[32];
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
              const float4 d0 = delta_s[ch * 2], d1 = delta_s[ch * 2 + 1];
              const float dl[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
              float d[8];
#pragma unroll
              for (int j = 0; j < 8; j += 2) {
                const int c = ch * 8 + j;
                upk2(mul_x2(pk2(pr[c], pr[c + 1]),
                            sub_x2(pk2(__uint_as_float(dr[c >> 5][c & 31]), __uint_as_float(dr[c >> 5][(c & 31) + 1])),
                                   pk2(dl[j], dl[j + 1]))),
                     d[j], d[j + 1]);
              }
              pk[ch * 4 + 0] = pack_bf16x2(d[0], d[1]);
              pk[ch * 4 + 1] = pack_bf16x2(d[2], d[3]);
              pk[ch * 4 + 2] = pack_bf16x2(d[4], d[5]);
              pk[ch * 4 + 3] = pack_bf16x2(d[6], d[7]);
            }
            tmem_st32(tmem_base + lane_addr + KV_COL_DP + wg * 64, pk);
            tmem_wait_st();
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->ds_ready);

          // ---- P^T of the next query block (overlaps the dK product of this one)
          if (it + 1 < iters && !p_phase(v, it + 1, gi + 1)) { ok = false; break; }

          // Statistics of query block it + 2 replace those of query block it.
          compute_bar_sync();
          if (it + 2 < iters) store_stat(gi & 1, stat_next);
          compute_bar_sync();
        }
        if (!ok) break;
      }

      // The next item and the statistics of its first query blocks: fetched before the stores so
      // that they have landed when the epilogue is through.
      const int idx_next = read_item(k + 1);
      KvItem vn = v;
      if (idx_next >= 0) {
        vn = kv_item_of(p, idx_next);
        if (vn.iters > 0) st0 = fetch_stat(vn, 0);
        if (vn.iters > 1) st1 = fetch_stat(vn, 1);
      }

      __nv_bfloat16* dv_row = p.dv + v.bt * p.dv_sb + static_cast<long long>(v.k_base + key) * p.dv_ss + v.kvh * p.dv_sh + wg * 64;
      __nv_bfloat16* dk_row = p.dk + v.bt * p.dk_sb + static_cast<long long>(v.k_base + key) * p.dk_ss + v.kvh * p.dk_sh + wg * 64;
      if (iters == 0) {
        // Keys no query sees (a sequence without queries): their gradients are zero.
        if (key < v.Sk) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            *reinterpret_cast<uint4*>(dv_row + c * 8) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(dk_row + c * 8) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      } else {
        // ---- epilogue: dV and dK rows of this key block leave through the dO / Q stage of the
        // item's last query block (the loads' 128-byte swizzle) and one TMA store per 64-column
        // panel.  A store clips rows beyond the tensor, not rows of the next packed sequence: a
        // partial block of a packed sequence stores its rows directly.
        const uint32_t s_last = (g + iters - 1) & 1;
        const bool staged = p.cu_k == nullptr || v.key0 + BKV <= v.Sk;
        const bool row_ok = key < v.Sk;
        RopeUnits rope_units;  // the table values of the inverse rotation: on their way while dV is staged
        if (ROPE) rope_units_load(p.rope, v.key0, p.rope_rows, ct, rope_units);
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          __nv_bfloat16* dst = which == 0 ? dv_row : dk_row;
          // dV is complete one product before dK and is staged while that product runs.
          if (!mbar_wait(which == 0 ? &bars->dv_done : &bars->dk_done, kvn & 1, abort_word, 324 + which)) {
            ok = false;
            break;
          }
          tc_fence_after();
          uint8_t* stage = (which == 0 ? s_do : s_q) + s_last * TILE_BYTES;
          uint8_t* stage_row = stage + wg * PANEL_BYTES + r * 128;
          const uint32_t col = (which == 0 ? KV_COL_DV : KV_COL_DK) + wg * 64;
          const bool rotate = which == 1 && ROPE;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t a[32];
            tmem_ld32(tmem_base + lane_addr + col + half * 32, a);
            tmem_wait_ld();
            const float sc = which == 0 ? 1.0f : p.scale;  // dS^T was accumulated without the scale
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
              uint4 q;
              q.x = pack_bf16x2(__uint_as_float(a[gq * 8 + 0]) * sc, __uint_as_float(a[gq * 8 + 1]) * sc);
              q.y = pack_bf16x2(__uint_as_float(a[gq * 8 + 2]) * sc, __uint_as_float(a[gq * 8 + 3]) * sc);
              q.z = pack_bf16x2(__uint_as_float(a[gq * 8 + 4]) * sc, __uint_as_float(a[gq * 8 + 5]) * sc);
              q.w = pack_bf16x2(__uint_as_float(a[gq * 8 + 6]) * sc, __uint_as_float(a[gq * 8 + 7]) * sc);
              if (staged || rotate)
                *reinterpret_cast<uint4*>(stage_row + (((half * 4 + gq) ^ (r & 7)) << 4)) = q;
              else if (row_ok)
                *reinterpret_cast<uint4*>(dst + half * 32 + gq * 8) = q;
            }
          }
          if (rotate) {
            // dK of the keys before the rotary rotation: the staged rows are rotated back in place
            compute_bar_sync();
            rope_inverse_apply(stage, ct, rope_units, staged, dst - wg * 64 - r * p.dk_ss, p.dk_ss, v.Sk - v.key0);
          }
          if (staged) fence_proxy_async_smem();
          compute_bar_sync();  // every thread is through with the stage (and with the accumulator)
          if (staged && ct == 0) {
            const CUtensorMap* tm = which == 0 ? &tmap_dv : &tmap_dk;
            tma_store_4d(tm, stage, 0, v.k_base + v.key0, v.kvh, v.bt);
            tma_store_4d(tm, stage + PANEL_BYTES, 64, v.k_base + v.key0, v.kvh, v.bt);
            tma_store_commit();
          }
        }
        if (!ok) break;
        // The two stages go back to the producer when the stores have read them.
        if (ct == 0) {
          if (staged) tma_store_wait_read<1>();
          mbar_arrive(&bars->do_empty[s_last]);
          if (staged) tma_store_wait_read<0>();
          mbar_arrive(&bars->q_empty[s_last]);
        }
        // The accumulators are read: the next item's first dV / dK products, which overwrite
        // them, are ordered after this through that item's first p_ready / ds_ready arrivals.
        tc_fence_before();
        g += iters;
        ++kvn;
      }
      v = vn;
      idx = idx_next;
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
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_word != 0) atomicExch(p.status, *abort_word);
}

// ---------------------------------------------------------------- dQ kernel
// Number of 128-key blocks the query rows [q0, q0 + 128) see.
__device__ __forceinline__ int dq_kv_blocks(const Params& p, int q0) {
  if (q0 >= p.Sq) return 0;
  int max_key = p.Sk - 1;
  if (p.causal) max_key = min(max_key, min(q0 + BQ - 1, p.Sq - 1) + p.Sk - p.Sq);
  return max_key < 0 ? 0 : max_key / BKV + 1;
}

template <bool ROPE>  // see attn_bwd_dkdv_kernel
__global__ void __launch_bounds__(THREADS, 1)
    attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q,
                       const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v,
                       const __grid_constant__ CUtensorMap tmap_do,
                       const __grid_constant__ CUtensorMap tmap_dq, const Params p_in) {
  extern __shared__ __align__(1024) uint8_t smem[];
  Params p = p_in;  // per-sequence view, as in the dK/dV kernel
  int cta_rank, cta_hb;
  cta_coords(static_cast<int>(blockIdx.x), p_in.q_blocks, p_in.q_heads_total, p_in.q_chunk, p_in.q_tail, cta_rank, cta_hb);
  const int cta_b = cta_hb / p_in.H;
  int q_base = 0, k_base = 0, bt = cta_b;
  if (p_in.cu_q != nullptr) {
    grid_dep_wait();  // the sequence offsets may come from the previous kernel of the stream
    q_base = p_in.cu_q[cta_b];
    p.Sq = p_in.cu_q[cta_b + 1] - q_base;
    k_base = p_in.cu_k[cta_b];
    p.Sk = p_in.cu_k[cta_b + 1] - k_base;
    bt = 0;
    if (p.Sq > p_in.Sq || p.Sk > p_in.Sk) {
      if (threadIdx.x == 0) atomicExch(p.status, STATUS_SEQ_EXCEEDS_BOUND);
      p.Sq = min(p.Sq, p_in.Sq);
      p.Sk = min(p.Sk, p_in.Sk);
    }
  }
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(p.status, 902);
    return;
  }
  uint8_t* s_q = smem;
  uint8_t* s_do = smem + TILE_BYTES;
  uint8_t* s_k = smem + 2 * TILE_BYTES;                 // QK_STAGES stages
  uint8_t* s_v = s_k + QK_STAGES * TILE_BYTES;          // 2 stages
  QBarriers* bars = reinterpret_cast<QBarriers*>(s_v + 2 * TILE_BYTES);
  volatile int* abort_word = &bars->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q_block = p_in.q_blocks - 1 - cta_rank;  // the last query block sees the most keys
  const int h = cta_hb % p_in.H;
  const int b = cta_b;
  const int kvh = h / (p.H / p.Hkv);
  const int q0 = q_block * BQ;
  const int n_kv = dq_kv_blocks(p, q0);

  if (threadIdx.x == 0) {
    mbar_init(&bars->qdo_full, 1);
    for (int i = 0; i < QK_STAGES; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->v_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
    }
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->ds_ready, 8);  // one arrival per compute warp
    mbar_init(&bars->dq_done, 1);
    bars->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_do);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  grid_dep_wait();  // the set-up above overlaps the previous kernel's tail; global memory from here on
  grid_dep_launch();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    setmaxnreg_dec<56>();
    if (elect_one() && n_kv > 0) {
      mbar_arrive_expect_tx(&bars->qdo_full, 2 * TILE_BYTES);
#pragma unroll
      for (int dh = 0; dh < 2; ++dh) {
        tma_load_4d(s_q + dh * PANEL_BYTES, &tmap_q, &bars->qdo_full, dh * 64, q_base + q0, h, bt);
        tma_load_4d(s_do + dh * PANEL_BYTES, &tmap_do, &bars->qdo_full, dh * 64, q_base + q0, h, bt);
      }
      for (int j = 0; j < n_kv; ++j) {
        const int sk = j % QK_STAGES;
        if (!mbar_wait(&bars->k_empty[sk], ((j / QK_STAGES) & 1) ^ 1, abort_word, 131)) break;
        mbar_arrive_expect_tx(&bars->k_full[sk], TILE_BYTES);
#pragma unroll
        for (int dh = 0; dh < 2; ++dh)
          tma_load_4d(s_k + sk * TILE_BYTES + dh * PANEL_BYTES, &tmap_k, &bars->k_full[sk], dh * 64,
                      k_base + j * BKV, kvh, bt);
        const int s = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(&bars->v_empty[s], ph, abort_word, 132)) break;
        mbar_arrive_expect_tx(&bars->v_full[s], TILE_BYTES);
#pragma unroll
        for (int dh = 0; dh < 2; ++dh)
          tma_load_4d(s_v + s * TILE_BYTES + dh * PANEL_BYTES, &tmap_v, &bars->v_full[s], dh * 64,
                      k_base + j * BKV, kvh, bt);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // Issue order: S(j+1) [other S buffer], then after dS(j) has arrived dP(j+1) and dQ(j).
    setmaxnreg_dec<56>();
    if (elect_one() && n_kv > 0) {
      const uint32_t idesc_kk = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_kmn = make_idesc_bf16(128, 128, 0, 1);
      const uint32_t q_lo = desc_lo(smem_u32(s_q), 16), do_lo = desc_lo(smem_u32(s_do), 16);
      const uint32_t k_lo = desc_lo(smem_u32(s_k), 16), v_lo = desc_lo(smem_u32(s_v), 16);
      const uint32_t k_mn_lo = desc_lo(smem_u32(s_k), PANEL_BYTES);
      const uint32_t d_s = tmem_base + Q_COL_S, d_dp = tmem_base + Q_COL_DP, d_dq = tmem_base + Q_COL_DQ;
      auto issue_s = [&](uint32_t buf, uint32_t stage) {  // S = Q K_j^T
        const uint32_t ka = k_lo + stage * (TILE_BYTES >> 4);
        const uint32_t d = d_s + buf * 128;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(d, desc_at(q_lo, koff_k(k)), desc_at(ka, koff_k(k)), idesc_kk, k != 0);
        umma_commit(&bars->s_full[buf]);
      };
      auto issue_dp = [&](uint32_t stage) {  // dP = dO V_j^T
        const uint32_t va = v_lo + stage * (TILE_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(d_dp, desc_at(do_lo, koff_k(k)), desc_at(va, koff_k(k)), idesc_kk, k != 0);
        umma_commit(&bars->dp_full);
        umma_commit(&bars->v_empty[stage]);
      };
      bool ok = mbar_wait(&bars->qdo_full, 0, abort_word, 231) &&
                mbar_wait(&bars->k_full[0], 0, abort_word, 232);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        ok = mbar_wait(&bars->v_full[0], 0, abort_word, 233);
      }
      if (ok) {
        tc_fence_after();
        issue_dp(0);
      }
      uint32_t sk = 0;  // K stage of block j
      for (int j = 0; j < n_kv && ok; ++j) {
        const uint32_t s = j & 1;  // S buffer and V stage
        const uint32_t sk1 = sk + 1 == QK_STAGES ? 0 : sk + 1;
        const bool has_next = j + 1 < n_kv;
        if (has_next) {
          // K and V of the next block (loaded a block ago as a rule).  S buffer s ^ 1 held
          // dS(j-1), whose reader dQ(j-1) was issued before this point.
          ok = mbar_wait(&bars->k_full[sk1], ((j + 1) / QK_STAGES) & 1, abort_word, 234) &&
               mbar_wait(&bars->v_full[s ^ 1], ((j + 1) >> 1) & 1, abort_word, 236);
          if (!ok) break;
          tc_fence_after();
          issue_s(s ^ 1, sk1);
        }
        ok = mbar_wait(&bars->ds_ready, j & 1, abort_word, 235);
        if (!ok) break;
        tc_fence_after();
        if (has_next) issue_dp(s ^ 1);
        // dQ += dS K_j : A = dS (bf16 pairs in columns [0,32) and [64,96) of the S buffer),
        // B = K_j MN-major
        const uint32_t kf = k_mn_lo + sk * (TILE_BYTES >> 4);
        const uint32_t a_ds = d_s + s * 128;
        const uint32_t acc = j > 0 ? 1u : 0u;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ts(d_dq, a_ds + acol(k), desc_at(kf, koff_mn(k)), idesc_kmn, k != 0 ? 1u : acc);
        umma_commit(&bars->k_empty[sk]);
        sk = sk1;
      }
      if (ok) umma_commit(&bars->dq_done);
    }
  } else if (warp < 4) {
    setmaxnreg_dec<56>();
  } else {
    // ------------------------------------------------------------ compute warps (4..11)
    setmaxnreg_inc<224>();
    const int wg = (warp - 4) >> 2;  // key-column half this thread works on
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // query row inside the block == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int row = q0 + r;
    const int shift = p.Sk - p.Sq;
    const long long stat_idx = (static_cast<long long>(b) * p.H + h) * p.Sq_pad + row;
    const float lse2 = p.lse2[stat_idx];   // +inf for rows that contribute nothing (and padding)
    const float delta = p.delta[stat_idx];
    const int key_limit = p.causal ? min(p.Sk - 1, row + shift) : p.Sk - 1;
    const int warp_limit = p.causal ? min(p.Sk - 1, q0 + quad * 32 + shift) : p.Sk - 1;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int s = j & 1;
      const int key0 = j * BKV + wg * 64;
      const bool need_mask = key0 + 63 > warp_limit;  // warp-uniform
      if (!mbar_wait(&bars->s_full[s], (j >> 1) & 1, abort_word, 331)) { ok = false; break; }
      tc_fence_after();
      float pr[64];
      {
        uint32_t sr[2][32];
        tmem_ld32(tmem_base + lane_addr + Q_COL_S + s * 128 + wg * 64, sr[0]);
        tmem_ld32(tmem_base + lane_addr + Q_COL_S + s * 128 + wg * 64 + 32, sr[1]);
        tmem_wait_ld();
        float x[64];
        const uint64_t scale2 = pk2(p.scale_log2, p.scale_log2), neg_lse2 = pk2(-lse2, -lse2);
#pragma unroll
        for (int c = 0; c < 64; c += 2)
          upk2(fma_x2(pk2(__uint_as_float(sr[c >> 5][c & 31]), __uint_as_float(sr[c >> 5][(c & 31) + 1])), scale2, neg_lse2),
               x[c], x[c + 1]);
        exp2_row64(x, pr);
        if (need_mask) {  // warp-uniform
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (key0 + c > key_limit) pr[c] = 0.f;
        }
      }
      if (!mbar_wait(&bars->dp_full, j & 1, abort_word, 332)) { ok = false; break; }
      tc_fence_after();
      uint32_t pk[32];
      {
        uint32_t dr[2][32];
        tmem_ld32(tmem_base + lane_addr + Q_COL_DP + wg * 64, dr[0]);
        tmem_ld32(tmem_base + lane_addr + Q_COL_DP + wg * 64 + 32, dr[1]);
        tmem_wait_ld();
        const uint64_t delta2 = pk2(delta, delta);
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          // without the softmax scale: it is applied once, when dQ leaves tensor memory
          float d0, d1;
          upk2(mul_x2(pk2(pr[2 * c], pr[2 * c + 1]),
                      sub_x2(pk2(__uint_as_float(dr[(2 * c) >> 5][(2 * c) & 31]),
                                 __uint_as_float(dr[(2 * c) >> 5][((2 * c) & 31) + 1])),
                             delta2)),
               d0, d1);
          pk[c] = pack_bf16x2(d0, d1);
        }
      }
      // dS (bf16 pairs) of this thread's 64 keys goes over the first 32 of the 64 S columns it has
      // read (keys 0-63 in columns [0,32), keys 64-127 in columns [64,96) of the buffer): no barrier
      // between the two column halves is needed.
      tmem_st32(tmem_base + lane_addr + Q_COL_S + s * 128 + wg * 64, pk);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->ds_ready);
    }

    // ---- epilogue: this thread's 64 columns of its dQ row
    RopeUnits rope_units;  // the table values of the inverse rotation: on their way under the last product
    if (ROPE) rope_units_load(p.rope, q0, p.rope_rows, threadIdx.x - 128, rope_units);
    if (ok && n_kv > 0) {
      ok = mbar_wait(&bars->dq_done, 0, abort_word, 333);
      tc_fence_after();
    }
    if (ok && q0 < p.Sq) {
      // Through shared memory and TMA stores, as in the dK/dV kernel; the first K stage is free.
      const bool staged = p.cu_q == nullptr || q0 + BQ <= p.Sq;
      __nv_bfloat16* dst = p.dq + bt * p.dq_sb + static_cast<long long>(q_base + row) * p.dq_ss + h * p.dq_sh + wg * 64;
      uint8_t* stage_row = s_k + wg * PANEL_BYTES + r * 128;
      const bool rotate = ROPE;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t a[32];
        if (n_kv > 0) {
          tmem_ld32(tmem_base + lane_addr + Q_COL_DQ + wg * 64 + half * 32, a);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) a[i] = 0u;
        }
        const float sc = p.scale;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 q;
          q.x = pack_bf16x2(__uint_as_float(a[g * 8 + 0]) * sc, __uint_as_float(a[g * 8 + 1]) * sc);
          q.y = pack_bf16x2(__uint_as_float(a[g * 8 + 2]) * sc, __uint_as_float(a[g * 8 + 3]) * sc);
          q.z = pack_bf16x2(__uint_as_float(a[g * 8 + 4]) * sc, __uint_as_float(a[g * 8 + 5]) * sc);
          q.w = pack_bf16x2(__uint_as_float(a[g * 8 + 6]) * sc, __uint_as_float(a[g * 8 + 7]) * sc);
          if (staged || rotate)
            *reinterpret_cast<uint4*>(stage_row + (((half * 4 + g) ^ (r & 7)) << 4)) = q;
          else if (row < p.Sq)
            *reinterpret_cast<uint4*>(dst + half * 32 + g * 8) = q;
        }
      }
      if (rotate) {
        // dQ of the queries before the rotary rotation (see rope_inverse_apply)
        compute_bar_sync();
        rope_inverse_apply(s_k, threadIdx.x - 128, rope_units, staged, dst - wg * 64 - r * p.dq_ss, p.dq_ss, p.Sq - q0);
      }
      if (staged) {
        fence_proxy_async_smem();
        compute_bar_sync();
        if (threadIdx.x == 128) {
          tma_store_4d(&tmap_dq, s_k, 0, q_base + q0, h, bt);
          tma_store_4d(&tmap_dq, s_k + PANEL_BYTES, 64, q_base + q0, h, bt);
          tma_store_commit();
          tma_store_wait_read<0>();
        }
      }
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
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_word != 0) atomicExch(p.status, *abort_word);
}

// ---------------------------------------------------------------- dQ kernel, persistent form
// attn_bwd_dq_kernel's tile program run by one CTA per SM over many (query block, head, batch)
// items, handed out like the items of the persistent dK/dV kernel.  All barrier phases count key
// blocks (or items) across items; the K / V stages keep cycling.  Q is free for the next item's
// load once the item's last S has run, dO once its last dP has (q_free / do_free, committed one
// key block before the item ends); S and dP of the next item's first key block are issued right
// behind the item's last dQ product; dQ leaves through the K stage of the item's last key block,
// which the storing thread gives back to the producer when the TMA stores have read it.  The next
// item's first dQ product, which overwrites the accumulator, waits for that item's first dS, which
// the compute warps write after they have read the accumulator.
struct QpBarriers {
  uint64_t qdo_full, q_free, do_free;
  uint64_t k_full[QK_STAGES], k_empty[QK_STAGES], v_full[2], v_empty[2];
  uint64_t s_full[2], dp_full, ds_ready, dq_done;
  uint64_t item_full[KVP_SLOTS], item_read[KVP_SLOTS];
  int item_ring[KVP_SLOTS];
  uint32_t tmem_base;
  int abort_word;
};
constexpr size_t QP_SMEM_BYTES = (4 + QK_STAGES) * TILE_BYTES + sizeof(QpBarriers);
static_assert(QP_SMEM_BYTES <= 232448, "exceeds the 227 KiB of shared memory a CTA can opt in to");

// One item: query rows [q0, q0 + 128) of head h of sequence b, walked over n_kv key blocks.
struct QItem {
  int b, h, kvh, bt, q0, q_base, k_base, Sq, Sk, n_kv;
  bool exceeds;
};
__device__ __forceinline__ QItem q_item_of(const Params& p, int idx) {
  QItem v;
  int rank, hb;
  cta_coords(idx, p.q_blocks, p.q_heads_total, p.q_chunk, p.q_tail, rank, hb);
  v.b = hb / p.H;
  v.h = hb - v.b * p.H;
  v.kvh = v.h / (p.H / p.Hkv);
  v.bt = v.b;
  v.q_base = 0;
  v.k_base = 0;
  v.Sq = p.Sq;
  v.Sk = p.Sk;
  v.exceeds = false;
  if (p.cu_q != nullptr) {
    v.q_base = p.cu_q[v.b];
    v.Sq = p.cu_q[v.b + 1] - v.q_base;
    v.k_base = p.cu_k[v.b];
    v.Sk = p.cu_k[v.b + 1] - v.k_base;
    v.bt = 0;
    if (v.Sq > p.Sq || v.Sk > p.Sk) {
      v.exceeds = true;
      v.Sq = min(v.Sq, p.Sq);
      v.Sk = min(v.Sk, p.Sk);
    }
  }
  v.q0 = (p.q_blocks - 1 - rank) * BQ;  // the last query block sees the most keys
  v.n_kv = 0;
  if (v.q0 < v.Sq) {
    int max_key = v.Sk - 1;
    if (p.causal) max_key = min(max_key, min(v.q0 + BQ - 1, v.Sq - 1) + v.Sk - v.Sq);
    v.n_kv = max_key < 0 ? 0 : max_key / BKV + 1;
  }
  return v;
}

template <bool ROPE>  // see attn_bwd_dkdv_kernel
__global__ void __launch_bounds__(THREADS, 1)
    attn_bwd_dq_persistent_kernel(const __grid_constant__ CUtensorMap tmap_q,
                                  const __grid_constant__ CUtensorMap tmap_k,
                                  const __grid_constant__ CUtensorMap tmap_v,
                                  const __grid_constant__ CUtensorMap tmap_do,
                                  const __grid_constant__ CUtensorMap tmap_dq, const Params p,
                                  unsigned int* item_counter) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(p.status, 902);
    return;
  }
  uint8_t* s_q = smem;
  uint8_t* s_do = smem + TILE_BYTES;
  uint8_t* s_k = smem + 2 * TILE_BYTES;                 // QK_STAGES stages
  uint8_t* s_v = s_k + QK_STAGES * TILE_BYTES;          // 2 stages
  QpBarriers* bars = reinterpret_cast<QpBarriers*>(s_v + 2 * TILE_BYTES);
  volatile int* abort_word = &bars->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total = p.q_blocks * p.q_heads_total;
  const int nc = static_cast<int>(gridDim.x), cid = static_cast<int>(blockIdx.x);

  if (threadIdx.x == 0) {
    mbar_init(&bars->qdo_full, 1);
    mbar_init(&bars->q_free, 1);
    mbar_init(&bars->do_free, 1);
    for (int i = 0; i < QK_STAGES; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->v_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
    }
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->ds_ready, 8);  // one arrival per compute warp
    mbar_init(&bars->dq_done, 1);
    for (int i = 0; i < KVP_SLOTS; ++i) {
      mbar_init(&bars->item_full[i], 1);
      mbar_init(&bars->item_read[i], 9);  // the issuing lane and the eight compute warps
    }
    bars->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_do);
    tma_prefetch_desc(&tmap_dq);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  grid_dep_wait();  // the set-up above overlaps the previous kernel's tail; global memory from here on
  grid_dep_launch();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (and item hand-out)
    setmaxnreg_dec<KV_LOW_REGS>();
    if (elect_one()) {
      // every item is drawn, the first one too (see the dK/dV kernel)
      const unsigned total_draws = static_cast<unsigned>(total) + static_cast<unsigned>(nc);
      int idx = -1;
      unsigned drawn = item_counter != nullptr ? atomicAdd(item_counter, 1u) : 0u;
      uint32_t g = 0, qn = 0;        // key blocks / non-empty items so far
      uint32_t sk = 0, kpar = 0;     // K stage of key block g and the parity of its use
      bool ok = true;
      for (int k = 0; ok; ++k) {
        if (item_counter != nullptr) {
          idx = drawn < static_cast<unsigned>(total) ? static_cast<int>(drawn) : -1;
          if (drawn + 1 == total_draws) atomicExch(item_counter, 0u);
        } else {
          idx = kvp_fixed_item(k, cid, nc, total);
        }
        if (k >= KVP_SLOTS &&
            !mbar_wait(&bars->item_read[k % KVP_SLOTS], ((k / KVP_SLOTS) - 1) & 1, abort_word, 134)) {
          ok = false;
          break;
        }
        bars->item_ring[k % KVP_SLOTS] = idx;
        mbar_arrive(&bars->item_full[k % KVP_SLOTS]);
        if (idx < 0) break;
        const QItem v = q_item_of(p, idx);
        if (v.exceeds) atomicExch(p.status, STATUS_SEQ_EXCEEDS_BOUND);
        if (v.n_kv > 0) {
          ok = mbar_wait(&bars->q_free, (qn & 1) ^ 1, abort_word, 135) &&
               mbar_wait(&bars->do_free, (qn & 1) ^ 1, abort_word, 136);
          if (!ok) break;
          ++qn;
          mbar_arrive_expect_tx(&bars->qdo_full, 2 * TILE_BYTES);
#pragma unroll
          for (int dh = 0; dh < 2; ++dh) {
            tma_load_4d(s_q + dh * PANEL_BYTES, &tmap_q, &bars->qdo_full, dh * 64, v.q_base + v.q0, v.h, v.bt);
            tma_load_4d(s_do + dh * PANEL_BYTES, &tmap_do, &bars->qdo_full, dh * 64, v.q_base + v.q0, v.h, v.bt);
          }
          for (int j = 0; j < v.n_kv; ++j, ++g) {
            if (!mbar_wait(&bars->k_empty[sk], kpar ^ 1, abort_word, 131)) { ok = false; break; }
            mbar_arrive_expect_tx(&bars->k_full[sk], TILE_BYTES);
#pragma unroll
            for (int dh = 0; dh < 2; ++dh)
              tma_load_4d(s_k + sk * TILE_BYTES + dh * PANEL_BYTES, &tmap_k, &bars->k_full[sk], dh * 64,
                          v.k_base + j * BKV, v.kvh, v.bt);
            const uint32_t s = g & 1;
            if (!mbar_wait(&bars->v_empty[s], ((g >> 1) & 1) ^ 1, abort_word, 132)) { ok = false; break; }
            mbar_arrive_expect_tx(&bars->v_full[s], TILE_BYTES);
#pragma unroll
            for (int dh = 0; dh < 2; ++dh)
              tma_load_4d(s_v + s * TILE_BYTES + dh * PANEL_BYTES, &tmap_v, &bars->v_full[s], dh * 64,
                          v.k_base + j * BKV, v.kvh, v.bt);
            if (++sk == QK_STAGES) {
              sk = 0;
              kpar ^= 1;
            }
          }
        }
        // The next item is drawn when this item's last loads are on their way.
        if (ok && item_counter != nullptr) drawn = atomicAdd(item_counter, 1u);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // Issue order inside an item: S(j+1) [other S buffer], then after dS(j) has arrived dP(j+1)
    // and dQ(j); behind the last dQ of an item come S(0) and dP(0) of the next one.
    setmaxnreg_dec<KV_LOW_REGS>();
    if (elect_one()) {
      const uint32_t idesc_kk = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_kmn = make_idesc_bf16(128, 128, 0, 1);
      const uint32_t q_lo = desc_lo(smem_u32(s_q), 16), do_lo = desc_lo(smem_u32(s_do), 16);
      const uint32_t k_lo = desc_lo(smem_u32(s_k), 16), v_lo = desc_lo(smem_u32(s_v), 16);
      const uint32_t k_mn_lo = desc_lo(smem_u32(s_k), PANEL_BYTES);
      const uint32_t d_s = tmem_base + Q_COL_S, d_dp = tmem_base + Q_COL_DP, d_dq = tmem_base + Q_COL_DQ;
      auto issue_s = [&](uint32_t buf, uint32_t stage) {  // S = Q K_j^T
        const uint32_t ka = k_lo + stage * (TILE_BYTES >> 4);
        const uint32_t d = d_s + buf * 128;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(d, desc_at(q_lo, koff_k(k)), desc_at(ka, koff_k(k)), idesc_kk, k != 0);
        umma_commit(&bars->s_full[buf]);
      };
      auto issue_dp = [&](uint32_t stage) {  // dP = dO V_j^T
        const uint32_t va = v_lo + stage * (TILE_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(d_dp, desc_at(do_lo, koff_k(k)), desc_at(va, koff_k(k)), idesc_kk, k != 0);
        umma_commit(&bars->dp_full);
        umma_commit(&bars->v_empty[stage]);
      };
      uint32_t g = 0, qn = 0, sk = 0, kpar = 0;
      bool ok = true;
      for (int k = 0; ok; ++k) {
        if (!mbar_wait(&bars->item_full[k % KVP_SLOTS], (k / KVP_SLOTS) & 1, abort_word, 237)) break;
        const int idx = bars->item_ring[k % KVP_SLOTS];
        mbar_arrive(&bars->item_read[k % KVP_SLOTS]);
        if (idx < 0) break;
        const int n_kv = q_item_of(p, idx).n_kv;
        if (n_kv == 0) continue;
        ok = mbar_wait(&bars->qdo_full, qn & 1, abort_word, 231) &&
             mbar_wait(&bars->k_full[sk], kpar, abort_word, 232);
        if (!ok) break;
        tc_fence_after();
        issue_s(g & 1, sk);
        if (n_kv == 1) umma_commit(&bars->q_free);
        ok = mbar_wait(&bars->v_full[g & 1], (g >> 1) & 1, abort_word, 233);
        if (!ok) break;
        tc_fence_after();
        issue_dp(g & 1);
        if (n_kv == 1) umma_commit(&bars->do_free);
        for (int j = 0; j < n_kv; ++j, ++g) {
          const uint32_t s = g & 1;  // S buffer and V stage
          const uint32_t sk1 = sk + 1 == QK_STAGES ? 0 : sk + 1;
          const uint32_t kpar1 = sk1 == 0 ? kpar ^ 1 : kpar;
          const bool has_next = j + 1 < n_kv;
          if (has_next) {
            // K and V of the next block (loaded a block ago as a rule).  S buffer s ^ 1 held
            // dS of the block before, whose reader dQ was issued before this point.
            ok = mbar_wait(&bars->k_full[sk1], kpar1, abort_word, 234) &&
                 mbar_wait(&bars->v_full[s ^ 1], ((g + 1) >> 1) & 1, abort_word, 236);
            if (!ok) break;
            tc_fence_after();
            issue_s(s ^ 1, sk1);
            if (j + 2 == n_kv) umma_commit(&bars->q_free);
          }
          ok = mbar_wait(&bars->ds_ready, g & 1, abort_word, 235);
          if (!ok) break;
          tc_fence_after();
          if (has_next) {
            issue_dp(s ^ 1);
            if (j + 2 == n_kv) umma_commit(&bars->do_free);
          }
          // dQ += dS K_j : A = dS (bf16 pairs in columns [0,32) and [64,96) of the S buffer),
          // B = K_j MN-major.  The first one of an item overwrites the previous item's dQ, which
          // the compute warps have read before they wrote this dS.
          const uint32_t kf = k_mn_lo + sk * (TILE_BYTES >> 4);
          const uint32_t a_ds = d_s + s * 128;
          const uint32_t acc = j > 0 ? 1u : 0u;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ts(d_dq, a_ds + acol(kk), desc_at(kf, koff_mn(kk)), idesc_kmn, kk != 0 ? 1u : acc);
          // After the item's last key block its K stage carries dQ out; the storing thread
          // releases it.
          if (has_next) umma_commit(&bars->k_empty[sk]);
          else umma_commit(&bars->dq_done);
          sk = sk1;
          kpar = kpar1;
        }
        ++qn;
      }
    }
  } else if (warp < 4) {
    setmaxnreg_dec<KV_LOW_REGS>();
  } else {
    // ------------------------------------------------------------ compute warps (4..11)
    setmaxnreg_inc<KV_HIGH_REGS>();
    const int ct = threadIdx.x - 128;
    const int wg = (warp - 4) >> 2;  // key-column half this thread works on
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // query row inside the block == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    bool ok = true;
    auto read_item = [&](int k) -> int {
      if (!mbar_wait(&bars->item_full[k % KVP_SLOTS], (k / KVP_SLOTS) & 1, abort_word, 336)) return -2;
      const int idx = bars->item_ring[k % KVP_SLOTS];
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->item_read[k % KVP_SLOTS]);
      return idx;
    };
    auto stat_index = [&](const QItem& v) {
      return (static_cast<long long>(v.b) * p.H + v.h) * p.Sq_pad + v.q0 + r;
    };
    uint32_t g = 0, qn = 0;
    int idx = read_item(0);
    QItem v;
    float lse2 = 0.f, delta = 0.f;  // +inf / 0 for rows that contribute nothing (and padding)
    if (idx >= 0) {
      v = q_item_of(p, idx);
      if (v.n_kv > 0) {
        lse2 = p.lse2[stat_index(v)];
        delta = p.delta[stat_index(v)];
      }
    }
    for (int k = 0; idx >= 0 && ok; ++k) {
      const int n_kv = v.n_kv;
      const int row = v.q0 + r;
      const int shift = v.Sk - v.Sq;
      const int key_limit = p.causal ? min(v.Sk - 1, row + shift) : v.Sk - 1;
      const int warp_limit = p.causal ? min(v.Sk - 1, v.q0 + quad * 32 + shift) : v.Sk - 1;
      for (int j = 0; j < n_kv; ++j) {
        const uint32_t gi = g + j;
        const uint32_t s = gi & 1;
        const int key0 = j * BKV + wg * 64;
        const bool need_mask = key0 + 63 > warp_limit;  // warp-uniform
        if (!mbar_wait(&bars->s_full[s], (gi >> 1) & 1, abort_word, 331)) { ok = false; break; }
        tc_fence_after();
        float pr[64];
        {
          uint32_t sr[2][32];
          tmem_ld32(tmem_base + lane_addr + Q_COL_S + s * 128 + wg * 64, sr[0]);
          tmem_ld32(tmem_base + lane_addr + Q_COL_S + s * 128 + wg * 64 + 32, sr[1]);
          tmem_wait_ld();
          float x[64];
          const uint64_t scale2 = pk2(p.scale_log2, p.scale_log2), neg_lse2 = pk2(-lse2, -lse2);
#pragma unroll
          for (int c = 0; c < 64; c += 2)
            upk2(fma_x2(pk2(__uint_as_float(sr[c >> 5][c & 31]), __uint_as_float(sr[c >> 5][(c & 31) + 1])), scale2, neg_lse2),
                 x[c], x[c + 1]);
          exp2_row64(x, pr);
          if (need_mask) {  // warp-uniform
#pragma unroll
            for (int c = 0; c < 64; ++c)
              if (key0 + c > key_limit) pr[c] = 0.f;
          }
        }
        if (!mbar_wait(&bars->dp_full, gi & 1, abort_word, 332)) { ok = false; break; }
        tc_fence_after();
        uint32_t pk[32];
        {
          uint32_t dr[2][32];
          tmem_ld32(tmem_base + lane_addr + Q_COL_DP + wg * 64, dr[0]);
          tmem_ld32(tmem_base + lane_addr + Q_COL_DP + wg * 64 + 32, dr[1]);
          tmem_wait_ld();
          const uint64_t delta2 = pk2(delta, delta);
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            // without the softmax scale: it is applied once, when dQ leaves tensor memory
            float d0, d1;
            upk2(mul_x2(pk2(pr[2 * c], pr[2 * c + 1]),
                        sub_x2(pk2(__uint_as_float(dr[(2 * c) >> 5][(2 * c) & 31]),
                                   __uint_as_float(dr[(2 * c) >> 5][((2 * c) & 31) + 1])),
                               delta2)),
                 d0, d1);
            pk[c] = pack_bf16x2(d0, d1);
          }
        }
        // dS (bf16 pairs) of this thread's 64 keys goes over the first 32 of the 64 S columns it has read
        tmem_st32(tmem_base + lane_addr + Q_COL_S + s * 128 + wg * 64, pk);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->ds_ready);
      }
      if (!ok) break;

      // The next item and its row statistics: fetched before the stores so that they have landed
      // when the epilogue is through.
      const int idx_next = read_item(k + 1);
      QItem vn = v;
      float lse2_next = 0.f, delta_next = 0.f;
      if (idx_next >= 0) {
        vn = q_item_of(p, idx_next);
        if (vn.n_kv > 0) {
          lse2_next = p.lse2[stat_index(vn)];
          delta_next = p.delta[stat_index(vn)];
        }
      }

      __nv_bfloat16* dst = p.dq + v.bt * p.dq_sb + static_cast<long long>(v.q_base + row) * p.dq_ss + v.h * p.dq_sh + wg * 64;
      if (n_kv == 0) {
        // Query rows without any visible key: their gradient is zero.
        if (row < v.Sq) {
#pragma unroll
          for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
      } else {
        // ---- epilogue: this thread's 64 columns of its dQ row, through the K stage of the item's
        // last key block and TMA stores (a partial block of a packed sequence stores directly)
        RopeUnits rope_units;  // the table values of the inverse rotation: on their way under the last product
        if (ROPE) rope_units_load(p.rope, v.q0, p.rope_rows, ct, rope_units);
        if (!mbar_wait(&bars->dq_done, qn & 1, abort_word, 333)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sk_last = (g + n_kv - 1) % QK_STAGES;
        uint8_t* stage = s_k + sk_last * TILE_BYTES;
        const bool staged = p.cu_q == nullptr || v.q0 + BQ <= v.Sq;
        uint8_t* stage_row = stage + wg * PANEL_BYTES + r * 128;
        const bool rotate = ROPE;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t a[32];
          tmem_ld32(tmem_base + lane_addr + Q_COL_DQ + wg * 64 + half * 32, a);
          tmem_wait_ld();
          const float sc = p.scale;
#pragma unroll
          for (int gq = 0; gq < 4; ++gq) {
            uint4 q;
            q.x = pack_bf16x2(__uint_as_float(a[gq * 8 + 0]) * sc, __uint_as_float(a[gq * 8 + 1]) * sc);
            q.y = pack_bf16x2(__uint_as_float(a[gq * 8 + 2]) * sc, __uint_as_float(a[gq * 8 + 3]) * sc);
            q.z = pack_bf16x2(__uint_as_float(a[gq * 8 + 4]) * sc, __uint_as_float(a[gq * 8 + 5]) * sc);
            q.w = pack_bf16x2(__uint_as_float(a[gq * 8 + 6]) * sc, __uint_as_float(a[gq * 8 + 7]) * sc);
            if (staged || rotate)
              *reinterpret_cast<uint4*>(stage_row + (((half * 4 + gq) ^ (r & 7)) << 4)) = q;
            else if (row < v.Sq)
              *reinterpret_cast<uint4*>(dst + half * 32 + gq * 8) = q;
          }
        }
        if (rotate) {
          // dQ of the queries before the rotary rotation (see rope_inverse_apply)
          compute_bar_sync();
          rope_inverse_apply(stage, ct, rope_units, staged, dst - wg * 64 - r * p.dq_ss, p.dq_ss, v.Sq - v.q0);
        }
        if (staged) fence_proxy_async_smem();
        compute_bar_sync();  // every thread is through with the stage (and with the accumulator)
        if (ct == 0) {
          if (staged) {
            tma_store_4d(&tmap_dq, stage, 0, v.q_base + v.q0, v.h, v.bt);
            tma_store_4d(&tmap_dq, stage + PANEL_BYTES, 64, v.q_base + v.q0, v.h, v.bt);
            tma_store_commit();
            tma_store_wait_read<0>();
          }
          mbar_arrive(&bars->k_empty[sk_last]);  // the stage goes back to the producer
        }
        tc_fence_before();
        g += n_kv;
        ++qn;
      }
      v = vn;
      idx = idx_next;
      lse2 = lse2_next;
      delta = delta_next;
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
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_word != 0) atomicExch(p.status, *abort_word);
}

static long long pad128(long long v) { return (v + 127) / 128 * 128; }

}  // namespace attn_bwd

size_t attn_bwd_scratch_bytes(long long B, long long Sq, long long H) {
  return 2 * static_cast<size_t>(B) * H * attn_bwd::pad128(Sq) * sizeof(float);
}

// Launches preprocess, dK/dV and dQ for a filled-in Params (p.Sq / p.Sk: the lengths the grids
// are sized with; q .. d_o: [B, S, H, D] views; lse strides as (batch, head, row)).
static int32_t bwd_run(const attn_bwd::Params& p_const, const cdl_tensor* q, const cdl_tensor* k,
                       const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* d_o,
                       const float* lse, long long lse_sb, long long lse_sh, long long lse_ss,
                       const cdl_tensor* dq, const cdl_tensor* dk, const cdl_tensor* dv,
                       double work, cudaStream_t stream) {
  attn_bwd::Params p = p_const;  // the CTA-order fields are filled in below
  using namespace attn_bwd;
  static std::once_flag attr_once[64];
  int dev = 0;
  CDL_CUDA(cudaGetDevice(&dev));
  cudaError_t attr_err = cudaSuccess;
  std::call_once(attr_once[dev & 63], [&] {
    auto opt_in = [&](const void* fn, size_t bytes) {
      if (attr_err == cudaSuccess)
        attr_err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    };
    opt_in(reinterpret_cast<const void*>(attn_bwd_dkdv_kernel<false>), KV_SMEM_BYTES);
    opt_in(reinterpret_cast<const void*>(attn_bwd_dkdv_kernel<true>), KV_SMEM_BYTES);
    opt_in(reinterpret_cast<const void*>(attn_bwd_dkdv_persistent_kernel<false>), KVP_SMEM_BYTES);
    opt_in(reinterpret_cast<const void*>(attn_bwd_dkdv_persistent_kernel<true>), KVP_SMEM_BYTES);
    opt_in(reinterpret_cast<const void*>(attn_bwd_dq_kernel<false>), Q_SMEM_BYTES);
    opt_in(reinterpret_cast<const void*>(attn_bwd_dq_kernel<true>), Q_SMEM_BYTES);
    opt_in(reinterpret_cast<const void*>(attn_bwd_dq_persistent_kernel<false>), QP_SMEM_BYTES);
    opt_in(reinterpret_cast<const void*>(attn_bwd_dq_persistent_kernel<true>), QP_SMEM_BYTES);
  });
  if (attr_err != cudaSuccess)
    return fail(CDL_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(attr_err));

  const long long B = p.B, H = p.H, Hkv = p.Hkv, Sq = p.Sq, Sk = p.Sk;
  const bool rope = p.rope != nullptr;
  const bool have_q = q->shape[1] > 0 && Sq > 0, have_k = k->shape[1] > 0 && Sk > 0;
  ProfileScope ps(PROF_ATTN_BWD, work, stream);
  if (have_q) {
    const long long blocks_ll = B * (p.Sq_pad / PRE_ROWS) * ((H + PRE_HEADS - 1) / PRE_HEADS);
    if (blocks_ll > 0x7fffffffll) return fail(CDL_ERR_UNSUPPORTED, "attention_bwd: too many rows for one launch");
    const unsigned blocks = static_cast<unsigned>(blocks_ll);
    CDL_CUDA(launch_pdl(attn_bwd_preprocess_kernel, dim3(blocks), dim3(256), 0, stream,
        static_cast<const __nv_bfloat16*>(o->ptr), o->stride[0], o->stride[1], o->stride[2],
        static_cast<const __nv_bfloat16*>(d_o->ptr), d_o->stride[0], d_o->stride[1], d_o->stride[2],
        lse, lse_sb, lse_sh, lse_ss, const_cast<float*>(p.lse2), const_cast<float*>(p.delta), p.B,
        p.H, p.Sq, p.Sq_pad, p.cu_q));
    CDL_CUDA(cudaGetLastError());
  }
  CUtensorMap tq, tk, tv, tdo, tdq, tdk, tdv;
  if (have_q) {
    CDL_CHECK(attn_encode_tmap(&tq, q));
    CDL_CHECK(attn_encode_tmap(&tdo, d_o));
    CDL_CHECK(attn_encode_tmap(&tdq, dq));
  } else {
    memset(&tq, 0, sizeof tq);
    tdo = tq;
    tdq = tq;
  }
  if (have_k) {
    CDL_CHECK(attn_encode_tmap(&tk, k));
    CDL_CHECK(attn_encode_tmap(&tv, v));
    CDL_CHECK(attn_encode_tmap(&tdk, dk));
    CDL_CHECK(attn_encode_tmap(&tdv, dv));
  } else {
    memset(&tk, 0, sizeof tk);
    tv = tk;
    tdk = tk;
    tdv = tk;
  }
  // (head, batch) pairs per chunk of the CTA order: their Q, dO, K and V should stay in L2
  auto chunk_of = [&](long long heads_total) {
    const double per_head = 4.0 * 2.0 * D * static_cast<double>(Sq > Sk ? Sq : Sk);
    long long c = static_cast<long long>(static_cast<double>(CDL_ATTN_BWD_CHUNK_MB) * 1024 * 1024 / per_head);
    if (c < 1) c = 1;
    return static_cast<int>(c < heads_total ? c : heads_total);
  };
  // Pairs of the last chunk: what the chunks before it leave over, grown chunk by chunk until it
  // holds CDL_ATTN_BWD_TAIL_X items per SM (or everything).  Items are taken longest first inside
  // a chunk, so a last chunk of fewer items than CTAs ends on its longest item with most SMs idle
  // (measured at B 8, S 2048: 128 items in the last chunk, the CTAs busy 94 % of the kernel).
  auto tail_pairs_of = [&](long long heads_total, int chunk, long long blocks) {
    long long tail = heads_total % chunk == 0 ? chunk : heads_total % chunk;
    while (tail < heads_total && tail * blocks < static_cast<long long>(CDL_ATTN_BWD_TAIL_X) * sm_count()) tail += chunk;
    return static_cast<int>(tail < heads_total ? tail : heads_total);
  };
  p.kv_blocks = static_cast<int>((Sk + BKV - 1) / BKV);
  p.kv_heads_total = static_cast<int>(Hkv * B);
  p.kv_chunk = chunk_of(Hkv * B);
  p.kv_tail = tail_pairs_of(Hkv * B, p.kv_chunk, p.kv_blocks);
  p.q_blocks = static_cast<int>((Sq + BQ - 1) / BQ);
  p.q_heads_total = static_cast<int>(H * B);
  p.q_chunk = chunk_of(H * B);
  p.q_tail = tail_pairs_of(H * B, p.q_chunk, p.q_blocks);
  if (have_k) {
    const long long items = static_cast<long long>(p.kv_blocks) * p.kv_heads_total;
    // More items than SMs: one CTA per SM takes them one after the other (items handed out at
    // run time from a counter of this stream; without one, a fixed deal).
    const bool persistent = p.variant == CDL_ATTN_PERSISTENT ||
                            (p.variant == CDL_ATTN_AUTO && CDL_ATTN_BWD_PERSISTENT && items > sm_count());
    if (persistent && items < (1ll << 30)) {
      const long long ctas = items < sm_count() ? items : sm_count();
      unsigned int* counter = items > ctas ? sched_counter_for(2, dev, stream) : nullptr;
      CDL_CUDA(launch_pdl(rope ? attn_bwd_dkdv_persistent_kernel<true> : attn_bwd_dkdv_persistent_kernel<false>,
                          dim3(static_cast<unsigned>(ctas)), dim3(THREADS),
                          KVP_SMEM_BYTES, stream, tq, tk, tv, tdo, tdk, tdv, p, counter));
    } else {
      dim3 grid(static_cast<unsigned>(items));
      CDL_CUDA(launch_pdl(rope ? attn_bwd_dkdv_kernel<true> : attn_bwd_dkdv_kernel<false>, grid, dim3(THREADS), KV_SMEM_BYTES,
                          stream, tq, tk, tv, tdo, tdk, tdv, p));
    }
    CDL_CUDA(cudaGetLastError());
  }
  if (have_q) {
    const long long items = static_cast<long long>(p.q_blocks) * p.q_heads_total;
    const bool persistent = p.variant == CDL_ATTN_PERSISTENT ||
                            (p.variant == CDL_ATTN_AUTO && CDL_ATTN_BWD_PERSISTENT && items > sm_count());
    if (persistent && items < (1ll << 30)) {
      const long long ctas = items < sm_count() ? items : sm_count();
      unsigned int* counter = items > ctas ? sched_counter_for(3, dev, stream) : nullptr;
      CDL_CUDA(launch_pdl(rope ? attn_bwd_dq_persistent_kernel<true> : attn_bwd_dq_persistent_kernel<false>,
                          dim3(static_cast<unsigned>(ctas)), dim3(THREADS),
                          QP_SMEM_BYTES, stream, tq, tk, tv, tdo, tdq, p, counter));
    } else {
      dim3 grid(static_cast<unsigned>(items));
      CDL_CUDA(launch_pdl(rope ? attn_bwd_dq_kernel<true> : attn_bwd_dq_kernel<false>, grid, dim3(THREADS), Q_SMEM_BYTES, stream,
                          tq, tk, tv, tdo, tdq, p));
    }
    CDL_CUDA(cudaGetLastError());
  }
  return CDL_OK;
}

// The rotary table of the fused inverse rotation: f32 [rows, 128] contiguous, one row per position.
static int32_t check_rope_table(const char* op, const cdl_tensor* t, long long min_rows, attn_bwd::Params* p) {
  p->rope = nullptr;
  p->rope_rows = 0;
  if (t == nullptr) return CDL_OK;
  if (t->rank != 2 || t->dtype != CDL_F32 || t->shape[1] != 128 || t->stride[1] != 1 || t->stride[0] != 128 ||
      t->ptr == nullptr || (reinterpret_cast<uintptr_t>(t->ptr) & 15) != 0)
    return fail(CDL_ERR_INVALID, "%s: the rotary table must be contiguous f32 [positions, 128], 16-byte aligned", op);
  if (t->shape[0] < min_rows)
    return fail(CDL_ERR_INVALID, "%s: the rotary table has %lld positions, the longest sequence %lld", op,
                static_cast<long long>(t->shape[0]), min_rows);
  p->rope = static_cast<const float*>(t->ptr);
  p->rope_rows = static_cast<int>(t->shape[0]);
  return CDL_OK;
}

int32_t attn_bwd_execute(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                         const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* d_o,
                         const cdl_tensor* lse, const cdl_tensor* dq, const cdl_tensor* dk,
                         const cdl_tensor* dv, void* scratch, size_t scratch_bytes,
                         cudaStream_t stream, const cdl_tensor* rope_table) {
  using namespace attn_bwd;
  const char* op = "attention_bwd";
  if (!desc || !q || !k || !v || !o || !d_o || !lse || !dq || !dk || !dv)
    return fail(CDL_ERR_INVALID, "%s: every operand is required", op);
  if (q->rank != 4 || k->rank != 4)
    return fail(CDL_ERR_INVALID, "%s: q and k must be [batch, seqlen, heads, head_dim]", op);
  const long long B = q->shape[0], Sq = q->shape[1], H = q->shape[2], Dh = q->shape[3];
  const long long Sk = k->shape[1], Hkv = k->shape[2];
  if (desc->variant < CDL_ATTN_AUTO || desc->variant > CDL_ATTN_PERSISTENT)
    return fail(CDL_ERR_INVALID, "%s: unknown kernel variant %d", op, desc->variant);
  if (Dh != D)
    return fail(CDL_ERR_UNSUPPORTED, "%s: head dimension %lld is not implemented (only 128)", op, Dh);
  if (Hkv <= 0 || H % Hkv != 0)
    return fail(CDL_ERR_INVALID, "%s: query heads (%lld) must be a multiple of kv heads (%lld)", op,
                H, Hkv);
  CDL_CHECK(attn_check_operand(op, "q", q, B, Sq, H, D));
  CDL_CHECK(attn_check_operand(op, "k", k, B, Sk, Hkv, D));
  CDL_CHECK(attn_check_operand(op, "v", v, B, Sk, Hkv, D));
  CDL_CHECK(attn_check_operand(op, "out", o, B, Sq, H, D));
  CDL_CHECK(attn_check_operand(op, "d_out", d_o, B, Sq, H, D));
  CDL_CHECK(attn_check_operand(op, "dq", dq, B, Sq, H, D));
  CDL_CHECK(attn_check_operand(op, "dk", dk, B, Sk, Hkv, D));
  CDL_CHECK(attn_check_operand(op, "dv", dv, B, Sk, Hkv, D));
  if (lse->rank != 3 || lse->shape[0] != B || lse->shape[1] != H || lse->shape[2] != Sq ||
      lse->dtype != CDL_F32)
    return fail(CDL_ERR_INVALID, "%s: lse must be f32 [batch, heads, seqlen_q]", op);
  if (B == 0 || H == 0 || (Sq == 0 && Sk == 0)) return CDL_OK;
  if (B > 65535 || H > 65535 || Sq > (1 << 30) || Sk > (1 << 30))
    return fail(CDL_ERR_UNSUPPORTED, "%s: dimension too large", op);
  const size_t need = attn_bwd_scratch_bytes(B, Sq, H);
  if (need > 0 && (scratch == nullptr || scratch_bytes < need ||
                   (reinterpret_cast<uintptr_t>(scratch) & 15) != 0))
    return fail(CDL_ERR_INVALID, "%s: scratch must be 16-byte aligned and hold %zu bytes (got %zu)",
                op, need, scratch_bytes);

  const long long Sq_pad = pad128(Sq);
  float* lse2 = static_cast<float*>(scratch);
  float* delta = lse2 + B * H * Sq_pad;

  Params p;
  p.B = static_cast<int>(B);
  p.H = static_cast<int>(H);
  p.Hkv = static_cast<int>(Hkv);
  p.Sq = static_cast<int>(Sq);
  p.Sk = static_cast<int>(Sk);
  p.Sq_pad = static_cast<int>(Sq_pad);
  p.causal = desc->causal != 0;
  p.variant = desc->variant;
  p.scale = desc->softmax_scale > 0.f ? desc->softmax_scale : 1.0f / sqrtf(static_cast<float>(D));
  p.scale_log2 = p.scale * 1.4426950408889634f;
  p.lse2 = lse2;
  p.delta = delta;
  p.dq = static_cast<__nv_bfloat16*>(dq->ptr);
  p.dk = static_cast<__nv_bfloat16*>(dk->ptr);
  p.dv = static_cast<__nv_bfloat16*>(dv->ptr);
  p.dq_sb = dq->stride[0]; p.dq_ss = dq->stride[1]; p.dq_sh = dq->stride[2];
  p.dk_sb = dk->stride[0]; p.dk_ss = dk->stride[1]; p.dk_sh = dk->stride[2];
  p.dv_sb = dv->stride[0]; p.dv_ss = dv->stride[1]; p.dv_sh = dv->stride[2];
  p.status = device_status_ptr();
  if (!p.status) return fail(CDL_ERR_CUDA, "cannot resolve the device status word");

  p.cu_q = nullptr;
  p.cu_k = nullptr;
  CDL_CHECK(check_rope_table(op, rope_table, Sq > Sk ? Sq : Sk, &p));
  // 14 B H Sq Sk D with the recomputed S and dP of the dQ kernel; reported as the conventional
  // 10 B H Sq Sk D (2.5 x forward), halved for the causal mask.
  return bwd_run(p, q, k, v, o, d_o, static_cast<const float*>(lse->ptr), lse->stride[0],
                 lse->stride[1], lse->stride[2], dq, dk, dv, 10.0 * B * H * Sq * Sk * D * (p.causal ? 0.5 : 1.0),
                 stream);
}

size_t attn_bwd_packed_scratch_bytes(long long batch, long long max_seqlen_q, long long H) {
  return attn_bwd_scratch_bytes(batch, max_seqlen_q, H);
}

int32_t attn_bwd_packed_execute(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                                const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* d_o,
                                const cdl_tensor* lse, const cdl_tensor* cu_q, const cdl_tensor* cu_k,
                                long long max_q, long long max_k, const cdl_tensor* dq,
                                const cdl_tensor* dk, const cdl_tensor* dv, void* scratch,
                                size_t scratch_bytes, cudaStream_t stream,
                                const cdl_tensor* rope_table) {
  using namespace attn_bwd;
  const char* op = "attention_bwd (packed)";
  if (!desc || !q || !k || !v || !o || !d_o || !lse || !dq || !dk || !dv || !cu_q || !cu_k)
    return fail(CDL_ERR_INVALID, "%s: every operand is required", op);
  if (q->rank != 3 || k->rank != 3)
    return fail(CDL_ERR_INVALID, "%s: q and k must be [total, heads, head_dim]", op);
  const long long Tq = q->shape[0], H = q->shape[1], Dh = q->shape[2];
  const long long Tk = k->shape[0], Hkv = k->shape[1];
  const long long B = cu_q->rank == 1 ? cu_q->shape[0] - 1 : -1;
  if (desc->variant < CDL_ATTN_AUTO || desc->variant > CDL_ATTN_PERSISTENT)
    return fail(CDL_ERR_INVALID, "%s: unknown kernel variant %d", op, desc->variant);
  if (Dh != D)
    return fail(CDL_ERR_UNSUPPORTED, "%s: head dimension %lld is not implemented (only 128)", op, Dh);
  if (Hkv <= 0 || H % Hkv != 0)
    return fail(CDL_ERR_INVALID, "%s: query heads (%lld) must be a multiple of kv heads (%lld)", op,
                H, Hkv);
  if (B < 0) return fail(CDL_ERR_INVALID, "%s: cu_seqlens_q must hold batch + 1 entries", op);
  CDL_CHECK(attn_check_cu_seqlens(op, "cu_seqlens_q", cu_q, B));
  CDL_CHECK(attn_check_cu_seqlens(op, "cu_seqlens_k", cu_k, B));
  cdl_tensor q4, k4, v4, o4, do4, dq4, dk4, dv4;
  CDL_CHECK(attn_packed_view(op, "q", q, Tq, H, &q4));
  CDL_CHECK(attn_packed_view(op, "k", k, Tk, Hkv, &k4));
  CDL_CHECK(attn_packed_view(op, "v", v, Tk, Hkv, &v4));
  CDL_CHECK(attn_packed_view(op, "out", o, Tq, H, &o4));
  CDL_CHECK(attn_packed_view(op, "d_out", d_o, Tq, H, &do4));
  CDL_CHECK(attn_packed_view(op, "dq", dq, Tq, H, &dq4));
  CDL_CHECK(attn_packed_view(op, "dk", dk, Tk, Hkv, &dk4));
  CDL_CHECK(attn_packed_view(op, "dv", dv, Tk, Hkv, &dv4));
  if (lse->rank != 2 || lse->shape[0] != H || lse->shape[1] != Tq || lse->dtype != CDL_F32)
    return fail(CDL_ERR_INVALID, "%s: lse must be f32 [heads, total_q]", op);
  if (max_q <= 0 || max_q > Tq) max_q = Tq;
  if (max_k <= 0 || max_k > Tk) max_k = Tk;
  if (B == 0 || H == 0 || (Tq == 0 && Tk == 0)) return CDL_OK;
  if (B > 65535 || H > 65535 || Tq > (1 << 30) || Tk > (1 << 30))
    return fail(CDL_ERR_UNSUPPORTED, "%s: dimension too large", op);
  const size_t need = attn_bwd_packed_scratch_bytes(B, max_q, H);
  if (need > 0 && (scratch == nullptr || scratch_bytes < need ||
                   (reinterpret_cast<uintptr_t>(scratch) & 15) != 0))
    return fail(CDL_ERR_INVALID, "%s: scratch must be 16-byte aligned and hold %zu bytes (got %zu)",
                op, need, scratch_bytes);
  const long long Sq_pad = pad128(max_q);
  Params p;
  p.B = static_cast<int>(B);
  p.H = static_cast<int>(H);
  p.Hkv = static_cast<int>(Hkv);
  p.Sq = static_cast<int>(max_q);
  p.Sk = static_cast<int>(max_k);
  p.Sq_pad = static_cast<int>(Sq_pad);
  p.causal = desc->causal != 0;
  p.variant = desc->variant;
  p.scale = desc->softmax_scale > 0.f ? desc->softmax_scale : 1.0f / sqrtf(static_cast<float>(D));
  p.scale_log2 = p.scale * 1.4426950408889634f;
  p.lse2 = static_cast<float*>(scratch);
  p.delta = p.lse2 + B * H * Sq_pad;
  p.dq = static_cast<__nv_bfloat16*>(dq->ptr);
  p.dk = static_cast<__nv_bfloat16*>(dk->ptr);
  p.dv = static_cast<__nv_bfloat16*>(dv->ptr);
  p.dq_sb = 0; p.dq_ss = dq->stride[0]; p.dq_sh = dq->stride[1];
  p.dk_sb = 0; p.dk_ss = dk->stride[0]; p.dk_sh = dk->stride[1];
  p.dv_sb = 0; p.dv_ss = dv->stride[0]; p.dv_sh = dv->stride[1];
  p.cu_q = static_cast<const int*>(cu_q->ptr);
  p.cu_k = static_cast<const int*>(cu_k->ptr);
  CDL_CHECK(check_rope_table(op, rope_table, max_q > max_k ? max_q : max_k, &p));
  p.status = device_status_ptr();
  if (!p.status) return fail(CDL_ERR_CUDA, "cannot resolve the device status word");
  const double mean_q = static_cast<double>(Tq) / B, mean_k = static_cast<double>(Tk) / B;
  return bwd_run(p, &q4, &k4, &v4, &o4, &do4, static_cast<const float*>(lse->ptr), 0, lse->stride[0],
                 lse->stride[1], &dq4, &dk4, &dv4, 10.0 * B * H * mean_q * mean_k * D * (p.causal ? 0.5 : 1.0), stream);
}

}  // namespace cdl

extern "C" {

int32_t cdl_b200_attn_bwd_packed(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                                 const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* d_out,
                                 const cdl_tensor* lse, const cdl_tensor* cu_seqlens_q,
                                 const cdl_tensor* cu_seqlens_k, int64_t max_seqlen_q,
                                 int64_t max_seqlen_k, const cdl_tensor* dq, const cdl_tensor* dk,
                                 const cdl_tensor* dv, void* scratch, size_t scratch_bytes,
                                 cdl_stream stream) {
  return cdl::attn_bwd_packed_execute(desc, q, k, v, o, d_out, lse, cu_seqlens_q, cu_seqlens_k,
                                      max_seqlen_q, max_seqlen_k, dq, dk, dv, scratch, scratch_bytes,
                                      static_cast<cudaStream_t>(stream), nullptr);
}

int32_t cdl_b200_attn_bwd_packed_scratch_bytes(int64_t batch, int64_t max_seqlen_q, int64_t heads,
                                               size_t* bytes_out) {
  if (batch < 0 || max_seqlen_q < 0 || heads < 0)
    return cdl::fail(CDL_ERR_INVALID, "attention_bwd (packed): negative dimension");
  if (bytes_out) *bytes_out = cdl::attn_bwd_packed_scratch_bytes(batch, max_seqlen_q, heads);
  return CDL_OK;
}

int32_t cdl_b200_attn_bwd(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                          const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* d_out,
                          const cdl_tensor* lse, const cdl_tensor* dq, const cdl_tensor* dk,
                          const cdl_tensor* dv, void* scratch, size_t scratch_bytes,
                          cdl_stream stream) {
  return cdl::attn_bwd_execute(desc, q, k, v, o, d_out, lse, dq, dk, dv, scratch, scratch_bytes,
                               static_cast<cudaStream_t>(stream), nullptr);
}

int32_t cdl_b200_attn_bwd_rope(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                               const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* d_out,
                               const cdl_tensor* lse, const cdl_tensor* cos_sin, const cdl_tensor* dq,
                               const cdl_tensor* dk, const cdl_tensor* dv, void* scratch,
                               size_t scratch_bytes, cdl_stream stream) {
  if (!cos_sin) return cdl::fail(CDL_ERR_INVALID, "attention_bwd: the rotary table is required");
  return cdl::attn_bwd_execute(desc, q, k, v, o, d_out, lse, dq, dk, dv, scratch, scratch_bytes,
                               static_cast<cudaStream_t>(stream), cos_sin);
}

int32_t cdl_b200_attn_bwd_packed_rope(const cdl_attn_desc* desc, const cdl_tensor* q,
                                      const cdl_tensor* k, const cdl_tensor* v, const cdl_tensor* o,
                                      const cdl_tensor* d_out, const cdl_tensor* lse,
                                      const cdl_tensor* cu_seqlens_q, const cdl_tensor* cu_seqlens_k,
                                      int64_t max_seqlen_q, int64_t max_seqlen_k,
                                      const cdl_tensor* cos_sin, const cdl_tensor* dq,
                                      const cdl_tensor* dk, const cdl_tensor* dv, void* scratch,
                                      size_t scratch_bytes, cdl_stream stream) {
  if (!cos_sin) return cdl::fail(CDL_ERR_INVALID, "attention_bwd (packed): the rotary table is required");
  return cdl::attn_bwd_packed_execute(desc, q, k, v, o, d_out, lse, cu_seqlens_q, cu_seqlens_k,
                                      max_seqlen_q, max_seqlen_k, dq, dk, dv, scratch, scratch_bytes,
                                      static_cast<cudaStream_t>(stream), cos_sin);
}

int32_t cdl_b200_attn_bwd_scratch_bytes(const cdl_tensor* q, const cdl_tensor* k,
                                        size_t* bytes_out) {
  (void)k;
  if (!q || q->rank != 4)
    return cdl::fail(CDL_ERR_INVALID, "attention_bwd: q must be [batch, seqlen, heads, head_dim]");
  if (bytes_out) *bytes_out = cdl::attn_bwd_scratch_bytes(q->shape[0], q->shape[1], q->shape[2]);
  return CDL_OK;
}

}  // extern "C"
