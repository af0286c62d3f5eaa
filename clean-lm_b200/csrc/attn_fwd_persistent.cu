// Flash attention forward, persistent form: one CTA per SM walks work items of 256 query rows
// (two 128-row tiles) of one (batch, head), longest first.
//
// Operator semantics as in attn_fwd.cu (AttentionFwd of the reference, crates/cleandl/src/execgraph/
// ops/attention/mod.rs:353-363, 807-850; exec.rs:358-416).  The tile program is the one of
// attn_fwd.cu (S = Q K^T into tensor memory, one softmax thread per row, P written back over S as
// bf16, O += P V with A = P from tensor memory, the two tiles alternating on the tensor core);
// what differs:
//
//   * Persistent CTAs.  Work items are ordered by the number of key blocks they see and handed
//     out at run time, longest first (a counter per stream; see fixed_item_of), so barrier
//     set-up, the tensor-memory allocation and the first loads are paid once per SM instead of
//     once per 256 rows, and the next item's Q, K and V arrive while the current item's last
//     blocks are computed.
//   * One issuing warp per tile, each a stream across items.  A tile whose item is finished has
//     its next item's first S = Q K^T issued at once, so the softmax warps find it when their
//     output is stored, while the other tile still works on its last blocks (under causal
//     masking the upper tile of an item always has one block less).  With one issuing warp that
//     walked item by item the tensor pipe drained and refilled at every item: ~7000 clk per item
//     against ~3700 per key block.
//   * Exponentials on two pipes.  The 2 x 16384 exponentials of a step take 2048 clk of the MUFU
//     pipe alone (16 per clk per SM), about as long as the step's four products.  A fixed share of
//     every row's exponentials is evaluated on the FMA pipe with packed f32x2 arithmetic
//     (exp2_poly2); scaling, row sums and the bf16 conversion are packed, the row maximum uses
//     three-input max.
//   * Lazy rescale.  O and the row sum are rescaled only when a row's maximum has grown by more
//     than 2^8 since the value the exponentials are taken against (rare after a tile's first
//     blocks), so the wait for the previous P V and the pass over O leave the common path.
//     (Taking the exponentials speculatively against the old maximum, with the block's maximum
//     computed alongside, was measured too: 7 % slower at B=8 S=2048, the re-take after a grown
//     maximum costs more than the separate pass over the scores it saves.)
//   * The MMA warps stay converged (one elected lane polls, issues and commits) and every wait
//     sleeps in mbarrier.try_wait with a time hint instead of spinning next to the softmax warps
//     of its scheduler partition.
//
// A CTA-pair version (tcgen05.mma.cta_group::2, M = 256 over two SMs, which issues at the full
// 64 clk per K step where the one-CTA forms take ~112 / ~82) was built and measured first: correct,
// but each key block then carries two cross-CTA hand-overs on its dependent chain (S ready ->
// peer's softmax, peer's P ready -> leader's MMA warp), together 1100-1600 clk against the ~530
// the faster products save, so the step took 4450-5000 clk and the one-CTA form is used.
//
// TMEM: S0/P0 [0,128) S1/P1 [128,256) O0 [256,384) O1 [384,512).
#include "host.h"
#include "ops.h"
#include "ptx.cuh"

#include <math.h>
#include <string.h>

#include <mutex>

namespace cdl {
namespace attn_fwd_ps {

constexpr int D = 128;
constexpr int BQ = 128;                    // rows per tile
constexpr int BKV = 128;                   // keys per block
constexpr int ROWS_PER_ITEM = 2 * BQ;      // two tiles
constexpr int TILE_BYTES = 128 * 128 * 2;  // a 128 x 128 bf16 tile as two [128 rows][64 d] panels
constexpr int PANEL_BYTES = TILE_BYTES / 2;
constexpr int KV_STAGES = 2;
constexpr int ITEM_SLOTS = 16;
constexpr int THREADS = 384;  // warp 0 TMA, warps 1-2 MMA (one per tile), warp 3 idle, warps 4-11 softmax
constexpr int TMEM_COLS = 512;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units
constexpr size_t SMEM_BYTES = 1024 + 2 * TILE_BYTES + 2 * KV_STAGES * TILE_BYTES + TILE_BYTES + 512;  // Q, K/V stages, O staging, barriers
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KiB of shared memory a CTA can opt in to");

// Which of the 16 column pairs of every 32-column chunk take the polynomial instead of MUFU.
#ifndef CDL_ATTN_POLY_MASK
#define CDL_ATTN_POLY_MASK 0x4924u
#endif
constexpr uint32_t POLY_MASK = CDL_ATTN_POLY_MASK;
// Registers per thread after the roles split: the loader / issuer warp group gives up what the
// two softmax warp groups take (LOW_REGS + 2 HIGH_REGS = 3 x 168, the launch allocation).
#ifndef CDL_ATTN_LOW_REGS
#define CDL_ATTN_LOW_REGS 88
#endif
constexpr int LOW_REGS = CDL_ATTN_LOW_REGS;
constexpr int HIGH_REGS = (3 * 168 - LOW_REGS) / 2;
static_assert(LOW_REGS % 8 == 0 && HIGH_REGS % 8 == 0, "setmaxnreg takes multiples of 8");

// Timeline probe (builds with -DCDL_ATTN_PROBE only): CTA 0 stamps clock64 at the hand-over
// points of its first 64 key blocks; cdl_attn_probe_read copies the stamps out.  Slots: 0-5 MMA
// lane (P ready seen / P V issued / next Q K^T issued, per tile), 8-13 and 16-21 first softmax
// thread of tile 0 / 1 (S seen, S in registers, max done, MMA lane past the P barrier, P stored,
// arrived), 6-7 MMA lane begins to wait for P, 24-31 MMA lane around tile 0's products (before
// P V, after its 8 issues, after its commit, before the wait for K, before Q K^T, after its 8
// issues, after its commit, end of the step).
#ifdef CDL_ATTN_PROBE
__device__ long long g_probe_items[16 * 16];  // [item of CTA 0][slot]
#define CDL_PROBE_ITEM(k, slot)                                                            \
  do {                                                                                     \
    if (blockIdx.x == 0 && (k) < 16) g_probe_items[(k) * 16 + (slot)] = clock64();         \
  } while (0)
__device__ long long g_probe[64 * 32];
#define CDL_PROBE(it, slot)                                                            \
  do {                                                                                 \
    if (blockIdx.x == 0 && (it) < 64u) g_probe[(it) * 32 + (slot)] = clock64();        \
  } while (0)
#else
#define CDL_PROBE(it, slot) \
  do {                      \
  } while (0)
#define CDL_PROBE_ITEM(k, slot) \
  do {                          \
  } while (0)
#endif

struct Params {
  int B, H, Hkv, Sq, Sk;
  int causal;
  float scale_log2;  // softmax_scale * log2(e)
  __nv_bfloat16* o;
  long long o_sb, o_ss, o_sh;  // element strides of O [B, Sq, H, D]
  float* lse;                  // [B, H, Sq] or nullptr
  long long lse_sb, lse_sh, lse_ss;
  const int* cu_q;  // packed layout (see attn_fwd.cu); nullptr: dense
  const int* cu_k;
  int num_q_blocks;  // ceil(Sq / 256)
  int total_items;   // num_q_blocks * H * B
  int o_tma;  // 1: finished tiles leave through the staging tile and TMA stores
  unsigned int* item_counter;  // items handed out beyond every CTA's first one (zero between launches), or nullptr
  int* status;
};

struct Barriers {
  uint64_t q_full[2], q_empty[2];
  uint64_t k_full[KV_STAGES], k_empty[KV_STAGES], v_full[KV_STAGES], v_empty[KV_STAGES];
  uint64_t s_full[2], p_ready[2], o_done[2];
  uint64_t item_full[ITEM_SLOTS], item_read[ITEM_SLOTS];
  uint64_t stage_free;     // the O staging tile: one release per use, users take tickets
  uint32_t stage_ticket;
  int item_ring[ITEM_SLOTS];
  uint32_t tmem_base;
  int abort_word;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- packed f32x2 arithmetic (one issue slot for two lanes of work)
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint32_t cvt_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// 2^x for two arguments <= 0 on the FMA / integer pipes (the scheme of exp2_poly in ptx.cuh):
// n = round(x) read from the low mantissa bits of x + 1.5 * 2^23, a degree-3 polynomial for
// 2^(x - n) on [-0.5, 0.5], n added to the exponent field.  Relative error 1.4e-4; arguments
// below -126 (including -inf) give 2^-126.
__device__ __forceinline__ void exp2_poly2(uint64_t x, float& r0, float& r1) {
  float x0, x1;
  unpack2(x, x0, x1);
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

// Number of 128-key blocks tile rows [r0, r0 + 128) need; 0 when the tile has no valid row.
__device__ __forceinline__ int kv_blocks_for_tile(int Sq, int Sk, int causal, int r0) {
  if (r0 >= Sq) return 0;
  int max_key = Sk - 1;
  if (causal) {
    const int r_last = min(r0 + BQ - 1, Sq - 1);
    max_key = min(max_key, r_last + Sk - Sq);
  }
  return max_key < 0 ? 0 : max_key / BKV + 1;
}

// Work items are ordered longest first (last query block first).  Every item is drawn from a
// counter at run time by the producer lane, which publishes the k-th item of the CTA in slot
// k % ITEM_SLOTS of a ring in shared memory (-1: no further item).  The MMA lane (once per tile) and the softmax warps read the slot after its
// barrier and report that on item_read; the producer refills a slot only when all ten readers
// have (items without key blocks pass through no other barrier, so nothing else would bound how
// far the producer runs ahead).  Handing items out at run
// time is the longest-first schedule itself, and a CTA that finds its SM late (another kernel
// holds it, e.g. a collective of a data-parallel step) takes fewer items, or none, instead of
// keeping a fixed share back to the end.  Without a counter (fixed assignment): a boustrophedon deal.
__device__ __forceinline__ int fixed_item_of(int k, int cid, int nc, int total) {
  if (static_cast<long long>(k) * nc >= total) return -1;
  const int idx = k * nc + ((k & 1) ? nc - 1 - cid : cid);
  return idx < total ? idx : -1;
}

// Per-sequence view of an item: head, lengths, row bases and block counts of the two tiles.
struct View {
  int h, b, Sq, Sk, q_base, k_base, bt, m0, n0, n1, n_max;  // n0 / n1: key blocks of the two tiles
};
__device__ __forceinline__ View view_of(const Params& p, int idx) {
  View v;
  const int bh = p.H * p.B;
  const int qb = p.num_q_blocks - 1 - idx / bh;
  const int r = idx % bh;
  v.h = r % p.H;
  v.b = r / p.H;
  v.Sq = p.Sq;
  v.Sk = p.Sk;
  v.q_base = 0;
  v.k_base = 0;
  v.bt = v.b;
  if (p.cu_q != nullptr) {
    // Packed layout: every sequence has its own lengths and its rows start at q_base / k_base of a
    // single "batch" (bt = 0).  Rows a tile loads beyond its sequence belong to the next one (or
    // are zero beyond the tensor): their scores are masked like keys beyond Sk, their outputs are
    // not stored.
    v.q_base = p.cu_q[v.b];
    v.Sq = min(p.cu_q[v.b + 1] - v.q_base, p.Sq);
    v.k_base = p.cu_k[v.b];
    v.Sk = p.cu_k[v.b + 1] - v.k_base;
    v.bt = 0;
  }
  v.m0 = qb * ROWS_PER_ITEM;
  v.n0 = kv_blocks_for_tile(v.Sq, v.Sk, p.causal, v.m0);
  v.n1 = kv_blocks_for_tile(v.Sq, v.Sk, p.causal, v.m0 + BQ);
  v.n_max = max(v.n0, v.n1);
  return v;
}

__global__ void __launch_bounds__(THREADS, 1)
    attn_fwd_persistent_kernel(const __grid_constant__ CUtensorMap tmap_q,
                               const __grid_constant__ CUtensorMap tmap_k,
                               const __grid_constant__ CUtensorMap tmap_v,
                               const __grid_constant__ CUtensorMap tmap_o, const Params p_in) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* s_q = smem;                               // 2 tiles
  uint8_t* s_k = smem + 2 * TILE_BYTES;              // KV_STAGES tiles
  uint8_t* s_v = s_k + KV_STAGES * TILE_BYTES;       // KV_STAGES tiles
  uint8_t* s_o = s_v + KV_STAGES * TILE_BYTES;       // 1 tile: staging of a finished O tile
  Barriers* bars = reinterpret_cast<Barriers*>(s_o + TILE_BYTES);
  volatile int* abort_word = &bars->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cid = blockIdx.x;
  const int nc = gridDim.x;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->q_full[i], 1);
      mbar_init(&bars->q_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->p_ready[i], 4);  // one arrival per softmax warp of the tile
      mbar_init(&bars->o_done[i], 1);
    }
    for (int i = 0; i < ITEM_SLOTS; ++i) {
      mbar_init(&bars->item_full[i], 1);
      mbar_init(&bars->item_read[i], 10);  // the eight softmax warps and the MMA lane's two tile cursors
    }
    for (int i = 0; i < KV_STAGES; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->v_empty[i], 1);
    }
    mbar_init(&bars->stage_free, 1);
    bars->stage_ticket = 0;
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
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  grid_dep_wait();  // the set-up above overlaps the previous kernel's tail; global memory from here on
  grid_dep_launch();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    setmaxnreg_dec<LOW_REGS>();
    if (elect_one()) {
      uint32_t kv_cnt = 0, q_cnt[2] = {0, 0};
      bool ok = true;
      // Every item is drawn, a CTA's first one too: a CTA that finds its SM late then finds
      // nothing left instead of running one of the longest items after everybody else has
      // finished.  A CTA draws until a draw runs past the last item; the launch's last draw puts
      // the counter back to zero.
      const int total = p_in.total_items;
      const unsigned total_draws = static_cast<unsigned>(total) + static_cast<unsigned>(nc);
      int idx = -1;
      unsigned drawn = p_in.item_counter != nullptr ? atomicAdd(p_in.item_counter, 1u) : 0u;  // the draw for the next item
      for (int k = 0; ok; ++k) {
        if (p_in.item_counter != nullptr) {
          idx = drawn < static_cast<unsigned>(total) ? static_cast<int>(drawn) : -1;
          if (drawn + 1 == total_draws) atomicExch(p_in.item_counter, 0u);
        } else {
          idx = fixed_item_of(k, cid, nc, total);
        }
        if (k >= ITEM_SLOTS &&
            !mbar_wait(&bars->item_read[k % ITEM_SLOTS], ((k / ITEM_SLOTS) - 1) & 1, abort_word, 124)) {
          ok = false;
          break;
        }
        bars->item_ring[k % ITEM_SLOTS] = idx;
        mbar_arrive(&bars->item_full[k % ITEM_SLOTS]);
        if (idx < 0) break;
        const View v = view_of(p_in, idx);
        const int kvh = v.h / (p_in.H / p_in.Hkv);
        // Q_t of the previous item is free once its last Q K^T has run.  Tile 0 finishes an item
        // first, so its Q and the first K go ahead of tile 1's Q.
        auto load_q = [&](int t) {
          if ((t == 0 ? v.n0 : v.n1) == 0 || !ok) return;
          ok = mbar_wait(&bars->q_empty[t], (q_cnt[t] & 1) ^ 1, abort_word, 121);
          if (!ok) return;
          ++q_cnt[t];
          mbar_arrive_expect_tx(&bars->q_full[t], TILE_BYTES);
#pragma unroll
          for (int dh = 0; dh < 2; ++dh)
            tma_load_4d(s_q + t * TILE_BYTES + dh * PANEL_BYTES, &tmap_q, &bars->q_full[t], dh * 64,
                        v.q_base + v.m0 + t * BQ, v.h, v.bt);
        };
        load_q(0);
        if (v.n_max == 0) load_q(1);
        for (int j = 0; j < v.n_max && ok; ++j, ++kv_cnt) {
          const int s = kv_cnt % KV_STAGES;
          const uint32_t ph = (kv_cnt / KV_STAGES) & 1;
          ok = mbar_wait(&bars->k_empty[s], ph ^ 1, abort_word, 122);
          if (!ok) break;
          mbar_arrive_expect_tx(&bars->k_full[s], TILE_BYTES);
#pragma unroll
          for (int dh = 0; dh < 2; ++dh)
            tma_load_4d(s_k + s * TILE_BYTES + dh * PANEL_BYTES, &tmap_k, &bars->k_full[s], dh * 64,
                        v.k_base + j * BKV, kvh, v.bt);
          if (j == 0) load_q(1);
          if (!ok) break;
          ok = mbar_wait(&bars->v_empty[s], ph ^ 1, abort_word, 123);
          if (!ok) break;
          mbar_arrive_expect_tx(&bars->v_full[s], TILE_BYTES);
#pragma unroll
          for (int dh = 0; dh < 2; ++dh)
            tma_load_4d(s_v + s * TILE_BYTES + dh * PANEL_BYTES, &tmap_v, &bars->v_full[s], dh * 64,
                        v.k_base + j * BKV, kvh, v.bt);
        }
        // The next item is drawn only now, when this item's last loads are on their way (two key
        // blocks before its products end): items differ in length, and an item reserved earlier
        // would be held back by a CTA that is busy while others run dry.
        if (ok && p_in.item_counter != nullptr) drawn = atomicAdd(p_in.item_counter, 1u);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The ring slots (key blocks of the CTA's items, in order) are the steps of one loop.  In step
    // r each tile that uses slot r gets O += P V for it and then S = Q K^T for the tile's next
    // block, also when that block is the first of the next item: a tile whose item is finished
    // (under causal masking the upper tile has one block less) has its next S under way while the
    // other tile works on its last block and the softmax warps store the finished output.  The
    // fixed order P V (0), Q K^T (0), P V (1), Q K^T (1) keeps the two tiles in opposite phase:
    // one tile's softmax runs while the other's products do.
    // The issuing lane shares its scheduler partition with two softmax warps that always have
    // an instruction ready, so its scalar code runs at a few clocks per dependent instruction and
    // sits on the critical path between "P ready" and the products: one lane runs the loop alone
    // (no warp-wide broadcasts), the per-tile state lives in scalars (indexed arrays would go to
    // local memory), and a K or V slot one tile has waited for is not waited for again by the other.
    setmaxnreg_dec<LOW_REGS>();
    if (elect_one()) {
      const uint32_t idesc_qk = make_idesc_bf16(BQ, BKV, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(BQ, D, 0, 1);
      // A descriptor costs one 32-bit add: low word per operand, constant high word (SBO 1024,
      // version 1, 128-byte swizzle).
      constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
      auto lo_of = [](uint32_t addr, uint32_t lbo) { return ((addr & 0x3FFFFu) >> 4) | ((lbo >> 4) << 16); };
      auto desc = [&](uint32_t lo, uint32_t off) {
        return (static_cast<uint64_t>(DESC_HI) << 32) | (lo + (off >> 4));
      };
      const uint32_t q_lo = lo_of(smem_u32(s_q), 16), k_lo = lo_of(smem_u32(s_k), 16);
      const uint32_t v_lo = lo_of(smem_u32(s_v), PANEL_BYTES);
      // S_t = Q_t K_j^T: 8 products of K = 16 over the two 64-wide d panels.
      auto issue_qk = [&](const int t, uint32_t stage, int r) {
        const uint32_t qa = q_lo + t * (TILE_BYTES >> 4), ka = k_lo + stage * (TILE_BYTES >> 4);
        const uint32_t d = tmem_base + t * 128;
        if (t == 0 && r >= 0) CDL_PROBE(r, 28);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * PANEL_BYTES + (k & 3) * 32;
          umma_ss(d, desc(qa, off), desc(ka, off), idesc_qk, k != 0);
        }
        if (t == 0 && r >= 0) CDL_PROBE(r, 29);
        umma_commit(&bars->s_full[t]);
        if (t == 0 && r >= 0) CDL_PROBE(r, 30);
      };
      // O_t (+)= P_t V_j: A = P (bf16 pairs in TMEM), B = V, MN-major.
      auto issue_pv = [&](const int t, uint32_t stage, bool accumulate, int r) {
        const uint32_t va = v_lo + stage * (TILE_BYTES >> 4);
        const uint32_t d = tmem_base + 256 + t * 128, a = tmem_base + t * 128;
        const uint32_t acc = accumulate ? 1u : 0u;
        if (t == 0) CDL_PROBE(r, 24);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k)
          umma_ts(d, a + k * 8, desc(va, k * 2048), idesc_pv, k != 0 ? 1u : acc);
        if (t == 0) CDL_PROBE(r, 25);
        umma_commit(&bars->o_done[t]);
        if (t == 0) CDL_PROBE(r, 26);
      };
      // Per tile: the block its next Q K^T is for (item ordinal k, block j of n, ring slot; n == 0
      // once the tile has no further block) and the block whose S has been issued and whose P V
      // is due (pend, pend_slot, acc: not the first block of its item).
      struct Tile {
        int k, j, n;
        uint32_t slot, next_base, pend_slot, q_cnt, p_cnt;
        bool pend, acc;
        bool open;  // the tile's next item has not been published yet (n == 0, slot >= next_base)
      };
      Tile T0{-1, 0, 0, 0u, 0u, 0u, 0u, 0u, false, false, true};
      Tile T1 = T0;
      // Moves a tile's cursor to the first block of the next item the tile takes part in.  The
      // items come from the producer's ring; one that is not published yet is waited for only
      // when step r needs the answer, i.e. when the tile's next block could be at slot r + 1 or
      // earlier.  (By then the producer can have published it: all it waits for before that is
      // the release of slots that steps before r have released.  Waiting earlier could stall the
      // other tile's products, which the producer may need in order to get there.)
      auto next_item = [&](Tile& T, const int t, const int r) {
        while (true) {
          const int k = T.k + 1;
          uint64_t* bar = &bars->item_full[k % ITEM_SLOTS];
          const uint32_t par = (k / ITEM_SLOTS) & 1;
          if (!mbar_test(bar, par)) {
            if (static_cast<int>(T.next_base) > r + 1) {
              T.open = true;
              T.n = 0;
              T.slot = T.next_base;
              return;
            }
            if (!mbar_wait(bar, par, abort_word, 225)) {  // the abort word ends every other wait too
              T.open = false;
              T.n = 0;
              T.slot = T.next_base;
              return;
            }
          }
          T.k = k;
          const int idx = bars->item_ring[k % ITEM_SLOTS];
          mbar_arrive(&bars->item_read[k % ITEM_SLOTS]);
          if (idx < 0) {
            T.open = false;
            T.n = 0;
            T.slot = T.next_base;
            return;
          }
          const View v = view_of(p_in, idx);
          const uint32_t base = T.next_base;
          T.next_base = base + v.n_max;
          const int n_t = t == 0 ? v.n0 : v.n1;
          if (n_t > 0) {
            T.open = false;
            T.j = 0;
            T.n = n_t;
            T.slot = base;
            return;
          }
        }
      };
      next_item(T0, 0, -1);
      next_item(T1, 1, -1);
      // Ring slots this lane has seen filled, per stage (slot + 1 of the latest one).
      uint32_t k_seen0 = 0, k_seen1 = 0, v_seen0 = 0, v_seen1 = 0;
      // One tile's part of step r: P V for slot r if the tile has it, then S = Q K^T of the tile's
      // next block.  A block two slots ahead (the tile skipped a slot that only the other tile
      // uses) is started only if its operands are there already, so that this step's other
      // products do not wait for it; otherwise it is started in the next step.
      auto turn = [&](Tile& T, const int t, const int r) -> bool {
        if (T.open && !T.pend) next_item(T, t, r);
        if (T.pend && static_cast<int>(T.pend_slot) == r) {
          const uint32_t st = static_cast<uint32_t>(r) % KV_STAGES;
          if (t == 0) CDL_PROBE(r, 6); else CDL_PROBE(r, 7);
          if (!mbar_wait(&bars->p_ready[t], T.p_cnt & 1, abort_word, 223)) return false;
          ++T.p_cnt;
          if (t == 0) CDL_PROBE(r, 11); else CDL_PROBE(r, 19);
          if ((st ? v_seen1 : v_seen0) <= static_cast<uint32_t>(r)) {
            if (!mbar_wait(&bars->v_full[st], (static_cast<uint32_t>(r) / KV_STAGES) & 1, abort_word, 224))
              return false;
            if (st) v_seen1 = r + 1; else v_seen0 = r + 1;
          }
          CDL_PROBE(r, 3 * t);
          tc_fence_after();
          issue_pv(t, st, T.acc, r);
          T.pend = false;
          CDL_PROBE(r, 3 * t + 1);
          if (T.open) next_item(T, t, r);
        }
        if (!T.pend && T.n > 0 && static_cast<int>(T.slot) <= r + 2) {
          const uint32_t s = T.slot;
          const uint32_t sst = s % KV_STAGES, sph = (s / KV_STAGES) & 1;
          const bool first = T.j == 0;
          const bool k_known = (sst ? k_seen1 : k_seen0) > s;
          bool go = true;
          if (static_cast<int>(s) == r + 2)
            go = (k_known || mbar_test(&bars->k_full[sst], sph)) &&
                 (!first || mbar_test(&bars->q_full[t], T.q_cnt & 1));
          if (go) {
            if (first) {
              if (!mbar_wait(&bars->q_full[t], T.q_cnt & 1, abort_word, 221)) return false;
              ++T.q_cnt;
            }
            if (t == 0 && r >= 0) CDL_PROBE(r, 27);
            if (!k_known) {
              if (!mbar_wait(&bars->k_full[sst], sph, abort_word, 222)) return false;
              if (sst) k_seen1 = s + 1; else k_seen0 = s + 1;
            }
            tc_fence_after();
            issue_qk(t, sst, r);
            if (r >= 0) CDL_PROBE(r, 3 * t + 2);
            T.pend = true;
            T.pend_slot = s;
            T.acc = !first;
            if (T.j + 1 == T.n) {
              umma_commit(&bars->q_empty[t]);  // the last reader of Q_t
              next_item(T, t, r);
            } else {
              ++T.j;
              ++T.slot;
            }
          }
        }
        return true;
      };
      // r = -1 is the prologue (the first Q K^T of each tile); the loop ends when both tiles have
      // neither a block to start nor a P V due.
      for (int r = -1; T0.pend || T1.pend || T0.n > 0 || T1.n > 0 || T0.open || T1.open; ++r) {
        if (!turn(T0, 0, r) || !turn(T1, 1, r)) break;
        // Every P V that reads V of slot r and every Q K^T that reads K of slot r + 1 has been
        // issued (a Q K^T is issued one or two steps before its slot's step).
        if (r >= 0) umma_commit(&bars->v_empty[static_cast<uint32_t>(r) % KV_STAGES]);
        umma_commit(&bars->k_empty[static_cast<uint32_t>(r + 1) % KV_STAGES]);
        if (r >= 0) CDL_PROBE(r, 31);
      }
    }
    __syncwarp();
  } else if (warp < 4) {
    setmaxnreg_dec<LOW_REGS>();
  } else {
    // ------------------------------------------------------------ softmax + epilogue
    setmaxnreg_inc<HIGH_REGS>();
    const int t = (warp - 4) >> 2;  // query tile of this warp group
    const int quad = warp & 3;      // TMEM lane quadrant
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem_base + lane_addr + t * 128;
    const uint32_t t_o = tmem_base + lane_addr + 256 + t * 128;
    const uint64_t scale2 = pack2(p_in.scale_log2, p_in.scale_log2);
    const bool probe_thread = quad == 0 && lane == 0;
    uint32_t s_cnt = 0, o_cnt = 0;  // phases of s_full[t] / o_done[t] this thread has passed
    bool ok = true;

    for (int k = 0; ok; ++k) {
      if (!mbar_wait(&bars->item_full[k % ITEM_SLOTS], (k / ITEM_SLOTS) & 1, abort_word, 324)) break;
      const int idx = bars->item_ring[k % ITEM_SLOTS];
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->item_read[k % ITEM_SLOTS]);
      if (idx < 0) break;
      const View v = view_of(p_in, idx);
      const int n_t = t == 0 ? v.n0 : v.n1;
      const int tile_row0 = v.m0 + t * BQ;
      const int row = tile_row0 + row_in_tile;
      const bool row_ok = row < v.Sq;
      // Last key this row may see.
      const int key_limit = p_in.causal ? min(v.Sk - 1, row + v.Sk - v.Sq) : v.Sk - 1;
      const int warp_first_row = tile_row0 + quad * 32;

      float m_used = -INFINITY;  // max the exponentials are taken against (scaled, log2 domain)
      float l = 0.f;
      if (probe_thread) CDL_PROBE_ITEM(k, 4 + 4 * t);  // softmax: item begins (+1: last P handed over, +2: O final seen, +3: epilogue done)
      for (int j = 0; j < n_t; ++j) {
        if (!mbar_wait(&bars->s_full[t], s_cnt & 1, abort_word, 321)) {
          ok = false;
          break;
        }
        ++s_cnt;
        if (probe_thread) CDL_PROBE(s_cnt - 1, 8 + 8 * t);
        tc_fence_after();
        uint32_t sr[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(t_s + c * 32, sr[c]);
        tmem_wait_ld();
        if (probe_thread) CDL_PROBE(s_cnt - 1, 9 + 8 * t);
        const int key0 = j * BKV;
        // Warp-uniform: does any row of this warp see a masked key in this block?
        const int warp_limit = p_in.causal ? warp_first_row + v.Sk - v.Sq : v.Sk - 1;
        const bool need_mask = key0 + BKV - 1 > min(warp_limit, v.Sk - 1);
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (key0 + c * 32 + i > key_limit) sr[c][i] = 0xff800000u;  // -inf
        }
        // Row max over the raw scores (four chains of three-input max), scaled afterwards: scale > 0.
        auto row_max = [&]() -> float {
          float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              mxa[0] = max3(mxa[0], __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
              mxa[1] = max3(mxa[1], __uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3]));
              mxa[2] = max3(mxa[2], __uint_as_float(sr[c][i + 4]), __uint_as_float(sr[c][i + 5]));
              mxa[3] = max3(mxa[3], __uint_as_float(sr[c][i + 6]), __uint_as_float(sr[c][i + 7]));
            }
          return fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3])) * p_in.scale_log2;
        };
        // P = 2^(S * scale - m_eff) for the whole row: stored to TMEM chunk by chunk, the row sum
        // returned.
        auto exp_store = [&](float m_eff) -> float {
          const uint64_t neg_m2 = pack2(-m_eff, -m_eff);
          uint64_t sum2[2] = {0ull, 0ull};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float r0 = __uint_as_float(sr[c][2 * i]), r1 = __uint_as_float(sr[c][2 * i + 1]);
              const uint64_t x = fma2(pack2(r0, r1), scale2, neg_m2);
              float p0, p1;
              if ((POLY_MASK >> i) & 1u) {
                exp2_poly2(x, p0, p1);
              } else {
                float x0, x1;
                unpack2(x, x0, x1);
                p0 = ex2(x0);
                p1 = ex2(x1);
              }
              sum2[i & 1] = add2(sum2[i & 1], pack2(p0, p1));
              pk[i] = cvt_bf16x2(p0, p1);
            }
            tmem_st16(t_s + c * 16, pk);
          }
          float s0, s1, s2, s3;
          unpack2(sum2[0], s0, s1);
          unpack2(sum2[1], s2, s3);
          return (s0 + s1) + (s2 + s3);
        };
        // Moves the reference maximum of the rows that grew to `mx` and rescales O and l for them
        // (lazy rescale: only when a maximum grew by more than the threshold).
        auto rescale = [&](float mx, bool grow) -> bool {
          if (j > 0) {
            // o_done has completed o_cnt + j phases once P V of block j - 1 is done
            if (!mbar_wait(&bars->o_done[t], (o_cnt + j - 1) & 1, abort_word, 322)) return false;
            tc_fence_after();
            const float f = grow ? (m_used == -INFINITY ? 0.f : ex2(m_used - mx)) : 1.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t orow[32];
              tmem_ld32(t_o + c * 32, orow);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * f);
              tmem_st32(t_o + c * 32, orow);
            }
            l *= f;
          }
          if (grow) m_used = mx;
          return true;
        };
        const float mx = row_max();
        const bool grow = mx > m_used + RESCALE_THRESHOLD || (m_used == -INFINITY && mx > -INFINITY);
        if (__any_sync(0xffffffffu, grow) && !rescale(mx, grow)) {
          ok = false;
          break;
        }
        if (probe_thread) CDL_PROBE(s_cnt - 1, 10 + 8 * t);
        const float sum = exp_store(m_used == -INFINITY ? 0.f : m_used);
        l += sum;
        tmem_wait_st();
        if (probe_thread) CDL_PROBE(s_cnt - 1, 12 + 8 * t);
        tc_fence_before();
        // One arrival per warp: 128 arrivals on one barrier word are serialised (measured: about
        // 500 clk between the last thread's arrive and the waiter's wake-up, against ~100 for four).
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_ready[t]);
        if (probe_thread) CDL_PROBE(s_cnt - 1, 13 + 8 * t);
      }
      if (!ok) break;
      if (probe_thread) CDL_PROBE_ITEM(k, 5 + 4 * t);

      if (n_t > 0) {
        if (!mbar_wait(&bars->o_done[t], (o_cnt + n_t - 1) & 1, abort_word, 323)) {
          ok = false;
          break;
        }
        o_cnt += n_t;
        tc_fence_after();
      }
      if (probe_thread) CDL_PROBE_ITEM(k, 6 + 4 * t);
      // A row that saw no key at all: the polynomial's 2^-126 floor must not pass for a sum.
      if (m_used == -INFINITY) l = 0.f;
      if (tile_row0 < v.Sq) {
        const float inv_l = l > 0.f ? 1.f / l : 0.f;
        // A whole tile leaves through a staging tile in shared memory (the loads' 128-byte swizzle,
        // two [128 rows][64 columns] panels) and two TMA stores: a thread owns a row, so its own
        // stores touch 32 rows per instruction and cost the softmax warps ~2 300 clk per tile and
        // item.  The staging tile is shared by the two tiles of the CTA (tickets; a use is
        // released when the store has read it).  A store clips rows beyond the tensor, not rows of
        // the next packed sequence: a partial tile of a packed sequence stores its rows directly.
        const bool staged = p_in.o_tma != 0 && (p_in.cu_q == nullptr || tile_row0 + BQ <= v.Sq);
        const bool tile_leader = quad == 0 && lane == 0;
        auto tile_bar = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(2 + t) : "memory"); };
        if (staged) {
          if (tile_leader) {
            const uint32_t ticket = atomicAdd(&bars->stage_ticket, 1u);
            if (!mbar_wait(&bars->stage_free, (ticket & 1u) ^ 1u, abort_word, 326)) ok = false;
          }
          tile_bar();
        }
        __nv_bfloat16* orow_ptr =
            p_in.o + v.bt * p_in.o_sb + static_cast<long long>(v.q_base + row) * p_in.o_ss + v.h * p_in.o_sh;
        // every row of the tensor starts on a 32-byte boundary (warp-uniform)
        const bool wide_rows = ((reinterpret_cast<uintptr_t>(p_in.o) | static_cast<uintptr_t>(p_in.o_sb * 2) |
                                 static_cast<uintptr_t>(p_in.o_ss * 2) | static_cast<uintptr_t>(p_in.o_sh * 2)) & 31) == 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t orow[32];
          if (n_t > 0) {
            tmem_ld32(t_o + c * 32, orow);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) orow[i] = 0u;
          }
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            w[i] = cvt_bf16x2(__uint_as_float(orow[2 * i]) * inv_l, __uint_as_float(orow[2 * i + 1]) * inv_l);
          if (staged) {
            uint8_t* panel_row = s_o + (c >> 1) * PANEL_BYTES + row_in_tile * 128;
#pragma unroll
            for (int g = 0; g < 4; ++g)
              *reinterpret_cast<uint4*>(panel_row + ((((c & 1) * 4 + g) ^ (row_in_tile & 7)) << 4)) =
                  make_uint4(w[g * 4 + 0], w[g * 4 + 1], w[g * 4 + 2], w[g * 4 + 3]);
          } else if (row_ok) {
            // 256-bit stores (whole 32-byte sectors) where the rows allow them
            if (wide_rows) {
#pragma unroll
              for (int g = 0; g < 2; ++g) {
                const uint32_t v8[8] = {w[g * 8 + 0], w[g * 8 + 1], w[g * 8 + 2], w[g * 8 + 3],
                                        w[g * 8 + 4], w[g * 8 + 5], w[g * 8 + 6], w[g * 8 + 7]};
                st_global_v8(orow_ptr + c * 32 + g * 16, v8);
              }
            } else {
#pragma unroll
              for (int g = 0; g < 4; ++g)
                *reinterpret_cast<uint4*>(orow_ptr + c * 32 + g * 8) =
                    make_uint4(w[g * 4 + 0], w[g * 4 + 1], w[g * 4 + 2], w[g * 4 + 3]);
            }
          }
        }
        if (staged) {
          fence_proxy_async_smem();
          tile_bar();
          if (tile_leader) {
            tma_store_4d(&tmap_o, s_o, 0, v.q_base + tile_row0, v.h, v.bt);
            tma_store_4d(&tmap_o, s_o + PANEL_BYTES, 64, v.q_base + tile_row0, v.h, v.bt);
            tma_store_commit();
            tma_store_wait_read<0>();
            mbar_arrive(&bars->stage_free);
          }
        }
        if (row_ok && p_in.lse != nullptr) {
          const float lse = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
          p_in.lse[v.bt * p_in.lse_sb + v.h * p_in.lse_sh +
                   static_cast<long long>(v.q_base + row) * p_in.lse_ss] = lse;
        }
      }
      // The O columns are read: the next item's first P V (which overwrites them) is ordered after
      // this through the p_ready arrival of that item's first block.
      tc_fence_before();
      if (probe_thread) CDL_PROBE_ITEM(k, 7 + 4 * t);
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
  if (threadIdx.x == 0 && *abort_word != 0) atomicExch(p_in.status, *abort_word);
}

}  // namespace attn_fwd_ps

int32_t attn_encode_tmap_rows(CUtensorMap* out, const cdl_tensor* t, uint32_t box_rows);

// Launches the persistent kernel for operands the caller has validated (q, k, v are
// [B, S, heads, 128] views; the packed layout passes single-batch views and the cu_seqlens
// pointers).
int32_t attn_fwd_persistent_launch(const cdl_tensor* q, const cdl_tensor* k, const cdl_tensor* v,
                                   long long B, long long H, long long Hkv, long long Sq, long long Sk,
                                   bool causal, float scale_log2, __nv_bfloat16* o, long long o_sb,
                                   long long o_ss, long long o_sh, float* lse, long long lse_sb,
                                   long long lse_sh, long long lse_ss, const int* cu_q,
                                   const int* cu_k, bool any_keys, cudaStream_t stream) {
  using namespace attn_fwd_ps;
  Params p;
  p.B = static_cast<int>(B);
  p.H = static_cast<int>(H);
  p.Hkv = static_cast<int>(Hkv);
  p.Sq = static_cast<int>(Sq);
  p.Sk = static_cast<int>(Sk);
  p.causal = causal ? 1 : 0;
  p.scale_log2 = scale_log2;
  p.o = o;
  p.o_sb = o_sb;
  p.o_ss = o_ss;
  p.o_sh = o_sh;
  p.lse = lse;
  p.lse_sb = lse_sb;
  p.lse_sh = lse_sh;
  p.lse_ss = lse_ss;
  p.cu_q = cu_q;
  p.cu_k = cu_k;
  p.num_q_blocks = static_cast<int>((Sq + ROWS_PER_ITEM - 1) / ROWS_PER_ITEM);
  const long long items = static_cast<long long>(p.num_q_blocks) * H * B;
  if (items > INT32_MAX) return fail(CDL_ERR_UNSUPPORTED, "attention_fwd: too many work items");
  p.total_items = static_cast<int>(items);
  p.item_counter = nullptr;
  p.status = device_status_ptr();
  if (!p.status) return fail(CDL_ERR_CUDA, "cannot resolve the device status word");

  // O as a tensor of q's shape for the TMA stores of finished tiles; rows that TMA cannot
  // describe (strides off the 16-byte grid) are stored by the threads directly.
  CUtensorMap to;
  {
    cdl_tensor ot = *q;
    ot.ptr = o;
    ot.stride[0] = o_sb;
    ot.stride[1] = o_ss;
    ot.stride[2] = o_sh;
    ot.stride[3] = 1;
    const bool describable = (reinterpret_cast<uintptr_t>(o) & 15) == 0 && o_ss % 8 == 0 && o_sh % 8 == 0 &&
                             (q->shape[0] <= 1 || o_sb % 8 == 0);
    p.o_tma = 0;
    if (describable && attn_encode_tmap_rows(&to, &ot, 128) == CDL_OK) p.o_tma = 1;
    if (!p.o_tma) memset(&to, 0, sizeof to);
  }
  CUtensorMap tq, tk, tv;
  if (any_keys) {
    CDL_CHECK(attn_encode_tmap_rows(&tq, q, 128));
    CDL_CHECK(attn_encode_tmap_rows(&tk, k, 128));
    CDL_CHECK(attn_encode_tmap_rows(&tv, v, 128));
  } else {
    // No keys at all: the kernel never touches the maps (every tile has zero blocks).
    memset(&tq, 0, sizeof tq);
    tk = tq;
    tv = tq;
  }

  static std::once_flag attr_once[64];
  int dev = 0;
  CDL_CUDA(cudaGetDevice(&dev));
  cudaError_t attr_err = cudaSuccess;
  std::call_once(attr_once[dev & 63], [&] {
    attr_err = cudaFuncSetAttribute(attn_fwd_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(SMEM_BYTES));
  });
  if (attr_err != cudaSuccess)
    return fail(CDL_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(attr_err));
  const int grid = items < sm_count() ? static_cast<int>(items) : sm_count();
  if (items > grid) p.item_counter = sched_counter_for(1, dev, stream);
  CDL_CUDA(launch_pdl(attn_fwd_persistent_kernel, dim3(grid), dim3(THREADS), SMEM_BYTES, stream, tq, tk, tv, to, p));
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

}  // namespace cdl

#ifdef CDL_ATTN_PROBE
extern "C" int32_t cdl_attn_probe_items_read(long long* out) {
  return cudaMemcpyFromSymbol(out, cdl::attn_fwd_ps::g_probe_items, sizeof(cdl::attn_fwd_ps::g_probe_items)) ==
                 cudaSuccess
             ? 0
             : -3;
}
extern "C" int32_t cdl_attn_probe_read(long long* out) {
  return cudaMemcpyFromSymbol(out, cdl::attn_fwd_ps::g_probe, sizeof(cdl::attn_fwd_ps::g_probe)) == cudaSuccess
             ? 0
             : -3;
}
#endif
