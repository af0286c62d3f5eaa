// Causal / dense flash attention forward on tcgen05 tensor cores with TMEM accumulators.
//
// Operator semantics follow AttentionFwd of the reference (crates/cleandl/src/execgraph/ops/
// attention/mod.rs:353-363, 807-850; exec.rs:358-416), which forwards to flash-attention-rs:
//   S = scale * Q K^T, bottom-right aligned causal mask, P = softmax(S), O = P V,
//   LSE = max + ln(sum exp) (natural log, f32, [B, H, Sq]); rows without a visible key give
//   O = 0 and LSE = -inf (attention/mod.rs:104-105).
//
// One CTA computes 256 query rows (two 128-row tiles) of one (batch, head); 384 threads (warps 2, 3
// idle: they only exist so that register re-allocation works on whole warp groups):
//   warp 0       TMA producer: Q once, then K and V blocks of 128 keys through two 2-stage rings.
//   warp 1       MMA issuer: S_t = Q_t K^T (SS form) into TMEM, O_t += P_t V (A = P from TMEM).
//   warps 4-7    softmax for tile 0, warps 8-11 for tile 1: one thread per query row.  A thread
//                reads its S row from TMEM, keeps the running max / sum in registers, writes
//                P (bf16) back into the TMEM columns S occupied, and only rescales the O
//                accumulator in TMEM when the running max grew by more than 2^8.
// The two tiles alternate on the tensor core (P0 V, Q0 K', P1 V, Q1 K'), so one tile's
// softmax overlaps the other tile's MMAs.  TMEM: S0/P0 [0,128) S1/P1 [128,256) O0 [256,384)
// O1 [384,512).
#include "host.h"
#include "ops.h"
#include "ptx.cuh"

#include <math.h>
#include <string.h>

#include <mutex>

namespace cdl {
namespace attn_fwd {

constexpr int D = 128;        // head dimension
constexpr int BQ = 128;       // query rows per tile
constexpr int BKV = 128;      // keys per block
constexpr int TILE_BYTES = 128 * 128 * 2;  // 32 KiB: a 128 x 128 bf16 tile as two 64-wide panels
constexpr int PANEL_BYTES = TILE_BYTES / 2;
constexpr int THREADS = 384;  // warp group 0: TMA, MMA, 2 idle; groups 1, 2: softmax
constexpr int TMEM_COLS = 512;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units
constexpr size_t SMEM_BYTES = 1024 + 6 * TILE_BYTES + 256;

struct Params {
  int B, H, Hkv, Sq, Sk;
  int causal;
  float scale_log2;  // softmax_scale * log2(e)
  __nv_bfloat16* o;
  long long o_sb, o_ss, o_sh;  // element strides of O [B, Sq, H, D]
  float* lse;                  // [B, H, Sq] or nullptr
  long long lse_sb, lse_sh, lse_ss;
  // Packed layout (q [total_q, H, D], k / v [total_k, Hkv, D]): sequence b is rows
  // cu_q[b] .. cu_q[b + 1] of q and cu_k[b] .. cu_k[b + 1] of k and v; Sq / Sk above are then the
  // bounds the grid was sized with.  nullptr: dense layout.
  const int* cu_q;
  const int* cu_k;
  int* status;
};

struct Barriers {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[2], p_ready[2], o_done[2];
  uint32_t tmem_base;
  int abort_word;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Number of 128-key blocks tile rows [r0, r0 + 128) need; 0 when the tile has no valid row.
__device__ __forceinline__ int kv_blocks_for_tile(const Params& p, int r0) {
  if (r0 >= p.Sq) return 0;
  int max_key = p.Sk - 1;
  if (p.causal) {
    const int r_last = min(r0 + BQ - 1, p.Sq - 1);
    max_key = min(max_key, r_last + p.Sk - p.Sq);
  }
  return max_key < 0 ? 0 : max_key / BKV + 1;
}

__global__ void __launch_bounds__(THREADS, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q,
                    const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const Params p_in) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* s_q = smem;                   // 2 tiles
  uint8_t* s_k = smem + 2 * TILE_BYTES;  // 2 stages
  uint8_t* s_v = smem + 4 * TILE_BYTES;  // 2 stages
  Barriers* bars = reinterpret_cast<Barriers*>(smem + 6 * TILE_BYTES);
  volatile int* abort_word = &bars->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Heaviest query blocks (most visible keys) are scheduled first.
  const int q_block = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  // Per-sequence view of the problem: in the packed layout every sequence has its own lengths
  // and its rows start at q_base / k_base of a single "batch" (bt = 0).  Rows a tile loads beyond
  // its sequence belong to the next one (or are zero beyond the tensor): their scores are masked
  // like keys beyond Sk, their outputs are not stored.
  Params p = p_in;
  int q_base = 0, k_base = 0, bt = b;
  if (p_in.cu_q != nullptr) {
    grid_dep_wait();  // the sequence offsets may come from the previous kernel of the stream
    q_base = p_in.cu_q[b];
    p.Sq = p_in.cu_q[b + 1] - q_base;
    k_base = p_in.cu_k[b];
    p.Sk = p_in.cu_k[b + 1] - k_base;
    bt = 0;
  }
  const int kvh = h / (p.H / p.Hkv);
  const int m0 = q_block * 2 * BQ;
  const int n0 = kv_blocks_for_tile(p, m0);
  const int n1 = kv_blocks_for_tile(p, m0 + BQ);
  const int n_max = max(n0, n1);

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->v_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->p_ready[i], 128);
      mbar_init(&bars->o_done[i], 1);
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
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  grid_dep_wait();  // the set-up above overlaps the previous kernel's tail; global memory from here on
  grid_dep_launch();
  // The control warps need few registers; hand theirs to the softmax warp groups, which hold a
  // whole 128-column row of scores per thread.

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    setmaxnreg_dec<56>();
    if (elect_one() && n_max > 0) {
      mbar_arrive_expect_tx(&bars->q_full, 2 * TILE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int dh = 0; dh < 2; ++dh)
          tma_load_4d(s_q + t * TILE_BYTES + dh * PANEL_BYTES, &tmap_q, &bars->q_full, dh * 64,
                      q_base + m0 + t * BQ, h, bt);
      for (int j = 0; j < n_max; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&bars->k_empty[s], ph ^ 1, abort_word, 111)) break;
        mbar_arrive_expect_tx(&bars->k_full[s], TILE_BYTES);
#pragma unroll
        for (int dh = 0; dh < 2; ++dh)
          tma_load_4d(s_k + s * TILE_BYTES + dh * PANEL_BYTES, &tmap_k, &bars->k_full[s], dh * 64,
                      k_base + j * BKV, kvh, bt);
        if (!mbar_wait(&bars->v_empty[s], ph ^ 1, abort_word, 112)) break;
        mbar_arrive_expect_tx(&bars->v_full[s], TILE_BYTES);
#pragma unroll
        for (int dh = 0; dh < 2; ++dh)
          tma_load_4d(s_v + s * TILE_BYTES + dh * PANEL_BYTES, &tmap_v, &bars->v_full[s], dh * 64,
                      k_base + j * BKV, kvh, bt);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    setmaxnreg_dec<56>();
    if (elect_one() && n_max > 0) {
      const uint32_t idesc_qk = make_idesc_bf16(BQ, BKV, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(BQ, D, 0, 1);
      // A descriptor costs the issuing thread one 32-bit add: the low word (start address and
      // leading byte offset) is computed once per operand, a K step adds a constant, the high
      // word (SBO 1024, version 1, 128-byte swizzle) is constant.
      constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
      auto lo_of = [](uint32_t addr, uint32_t lbo) { return ((addr & 0x3FFFFu) >> 4) | ((lbo >> 4) << 16); };
      auto desc = [&](uint32_t lo, uint32_t off) {
        return (static_cast<uint64_t>(DESC_HI) << 32) | (lo + (off >> 4));
      };
      const uint32_t q_lo = lo_of(smem_u32(s_q), 16), k_lo = lo_of(smem_u32(s_k), 16);
      const uint32_t v_lo = lo_of(smem_u32(s_v), PANEL_BYTES);
      const int n_t[2] = {n0, n1};
      // S_t = Q_t K_j^T : 8 MMAs of K = 16 over the two 64-wide d panels.
      auto issue_qk = [&](int t, int stage) {
        const uint32_t qa = q_lo + t * (TILE_BYTES >> 4), ka = k_lo + stage * (TILE_BYTES >> 4);
        const uint32_t d = tmem_base + t * 128;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * PANEL_BYTES + (k & 3) * 32;
          umma_ss(d, desc(qa, off), desc(ka, off), idesc_qk, k != 0);
        }
      };
      // O_t (+)= P_t V_j : A = P (bf16 pairs in TMEM columns), B = V as an MN-major tile.
      auto issue_pv = [&](int t, int stage, bool accumulate) {
        const uint32_t va = v_lo + stage * (TILE_BYTES >> 4);
        const uint32_t d = tmem_base + 256 + t * 128, a = tmem_base + t * 128;
        const uint32_t acc = accumulate ? 1u : 0u;
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k)
          umma_ts(d, a + k * 8, desc(va, k * 2048), idesc_pv, k != 0 ? 1u : acc);
      };
      bool ok = mbar_wait(&bars->q_full, 0, abort_word, 211);
      ok = ok && mbar_wait(&bars->k_full[0], 0, abort_word, 212);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (n_t[t] > 0) {
            issue_qk(t, 0);
            umma_commit(&bars->s_full[t]);
          }
        umma_commit(&bars->k_empty[0]);
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int s = j & 1, sn = (j + 1) & 1;
        const uint32_t ph = (j >> 1) & 1, phn = ((j + 1) >> 1) & 1;
        for (int t = 0; t < 2 && ok; ++t) {
          if (j < n_t[t]) {
            ok = mbar_wait(&bars->p_ready[t], j & 1, abort_word, 213) &&
                 mbar_wait(&bars->v_full[s], ph, abort_word, 214);
            if (!ok) break;
            tc_fence_after();
            issue_pv(t, s, j > 0);
            umma_commit(&bars->o_done[t]);
          }
          if (j + 1 < n_t[t]) {
            ok = mbar_wait(&bars->k_full[sn], phn, abort_word, 215);
            if (!ok) break;
            tc_fence_after();
            issue_qk(t, sn);
            umma_commit(&bars->s_full[t]);
          }
        }
        if (!ok) break;
        umma_commit(&bars->v_empty[s]);
        if (j + 1 < n_max) umma_commit(&bars->k_empty[sn]);
      }
    }
  } else if (warp < 4) {
    setmaxnreg_dec<56>();
  } else {
    // ------------------------------------------------------------ softmax + epilogue
    setmaxnreg_inc<224>();
    const int t = (warp - 4) >> 2;  // query tile of this warp group
    const int quad = warp & 3;      // TMEM lane quadrant
    const int row_in_tile = quad * 32 + lane;
    const int row = m0 + t * BQ + row_in_tile;
    const int n_t = t == 0 ? n0 : n1;
    const bool row_ok = row < p.Sq;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem_base + lane_addr + t * 128;
    const uint32_t t_o = tmem_base + lane_addr + 256 + t * 128;
    // Last key this row may see.
    const int key_limit = p.causal ? min(p.Sk - 1, row + p.Sk - p.Sq) : p.Sk - 1;

    float m_used = -INFINITY;  // max the exponentials are taken against (scaled, log2 domain)
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_t; ++j) {
      if (!mbar_wait(&bars->s_full[t], j & 1, abort_word, 311)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t sr[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(t_s + c * 32, sr[c]);
      tmem_wait_ld();
      const int key0 = j * BKV;
      // Warp-uniform: does any row of this warp see a masked key in this block?
      const int warp_first_row = m0 + t * BQ + quad * 32;
      const int warp_limit = p.causal ? warp_first_row + p.Sk - p.Sq : p.Sk - 1;
      const bool need_mask = key0 + BKV - 1 > min(warp_limit, p.Sk - 1);
      // Row max over the raw scores (four independent chains), scaled afterwards: scale > 0.
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (key0 + c * 32 + i > key_limit) sr[c][i] = 0xff800000u;  // -inf
      }
      float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          mxa[0] = fmaxf(mxa[0], __uint_as_float(sr[c][i]));
          mxa[1] = fmaxf(mxa[1], __uint_as_float(sr[c][i + 1]));
          mxa[2] = fmaxf(mxa[2], __uint_as_float(sr[c][i + 2]));
          mxa[3] = fmaxf(mxa[3], __uint_as_float(sr[c][i + 3]));
        }
      const float mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3])) * p.scale_log2;
      // Lazy rescale: move the reference max only when it grew by more than the threshold.
      const bool grow = mx > m_used + RESCALE_THRESHOLD || (m_used == -INFINITY && mx > -INFINITY);
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        if (!mbar_wait(&bars->o_done[t], (j - 1) & 1, abort_word, 312)) {
          ok = false;
          break;
        }
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
      const float m_eff = m_used == -INFINITY ? 0.f : m_used;
      float suma[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          // (All exponentials on the MUFU pipe: moving a share of them to a polynomial on the FMA
          // pipe, which pays in the backward kernels, measured slower here -- this kernel waits
          // on the tensor pipe, not on MUFU.)
          const float p0 = ex2(fmaf(__uint_as_float(sr[c][2 * i]), p.scale_log2, -m_eff));
          const float p1 = ex2(fmaf(__uint_as_float(sr[c][2 * i + 1]), p.scale_log2, -m_eff));
          suma[(i & 1) * 2] += p0;
          suma[(i & 1) * 2 + 1] += p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
        tmem_st16(t_s + c * 16, pk);
      }
      const float sum = (suma[0] + suma[1]) + (suma[2] + suma[3]);
      l += sum;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&bars->p_ready[t]);
    }

    if (ok && n_t > 0) {
      ok = mbar_wait(&bars->o_done[t], (n_t - 1) & 1, abort_word, 313);
      tc_fence_after();
    }
    if (ok && m0 + t * BQ < p.Sq) {
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow_ptr = p.o + bt * p.o_sb + static_cast<long long>(q_base + row) * p.o_ss + h * p.o_sh;
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
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 q;
            q.x = pack_bf16x2(__uint_as_float(orow[g * 8 + 0]) * inv_l, __uint_as_float(orow[g * 8 + 1]) * inv_l);
            q.y = pack_bf16x2(__uint_as_float(orow[g * 8 + 2]) * inv_l, __uint_as_float(orow[g * 8 + 3]) * inv_l);
            q.z = pack_bf16x2(__uint_as_float(orow[g * 8 + 4]) * inv_l, __uint_as_float(orow[g * 8 + 5]) * inv_l);
            q.w = pack_bf16x2(__uint_as_float(orow[g * 8 + 6]) * inv_l, __uint_as_float(orow[g * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow_ptr + c * 32 + g * 8) = q;
          }
        }
      }
      if (row_ok && p.lse != nullptr) {
        const float lse = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
        p.lse[bt * p.lse_sb + h * p.lse_sh + static_cast<long long>(q_base + row) * p.lse_ss] = lse;
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

}  // namespace attn_fwd

// Validates a dense [B, S, H, D] bf16 operand and encodes its tensor map with 64 x 128 boxes.
int32_t attn_check_operand(const char* op, const char* name, const cdl_tensor* t, long long B,
                           long long S, long long H, long long D) {
  if (!t) return fail(CDL_ERR_INVALID, "%s: %s is required", op, name);
  if (t->rank != 4 || t->shape[0] != B || t->shape[1] != S || t->shape[2] != H || t->shape[3] != D)
    return fail(CDL_ERR_INVALID, "%s: %s must have shape [%lld, %lld, %lld, %lld]", op, name, B, S,
                H, D);
  if (t->dtype != CDL_BF16)
    return fail(CDL_ERR_UNSUPPORTED, "%s: %s must be bf16 (f16 and fp8 are not implemented)", op,
                name);
  if (t->stride[3] != 1)
    return fail(CDL_ERR_INVALID, "%s: the head dimension of %s must be contiguous", op, name);
  if ((reinterpret_cast<uintptr_t>(t->ptr) & 15) != 0 || t->stride[0] % 8 != 0 ||
      t->stride[1] % 8 != 0 || t->stride[2] % 8 != 0)
    return fail(CDL_ERR_INVALID, "%s: %s needs a 16-byte aligned pointer and strides", op, name);
  return CDL_OK;
}

int32_t attn_encode_tmap_rows(CUtensorMap* out, const cdl_tensor* t, uint32_t box_rows);

int32_t attn_encode_tmap(CUtensorMap* out, const cdl_tensor* t) {
  return attn_encode_tmap_rows(out, t, 128);
}

// Same view with a box of `box_rows` sequence positions x 64 head-dimension elements.
int32_t attn_encode_tmap_rows(CUtensorMap* out, const cdl_tensor* t, uint32_t box_rows) {
  // innermost-first: D, S, H, B
  const uint64_t dims[4] = {static_cast<uint64_t>(t->shape[3]), static_cast<uint64_t>(t->shape[1]),
                            static_cast<uint64_t>(t->shape[2]), static_cast<uint64_t>(t->shape[0])};
  auto st = [&](int i, long long fallback) {
    return static_cast<uint64_t>((t->shape[i] > 1 ? t->stride[i] : fallback)) * 2;
  };
  const long long row = t->shape[3];
  const uint64_t strides[4] = {0, st(1, row), st(2, row), st(0, row)};
  const uint32_t box[4] = {64, box_rows, 1, 1};
  return encode_tmap(out, t->ptr, CDL_BF16, 4, dims, strides, box, true);
}

static int32_t fwd_set_attributes() {
  static std::once_flag attr_once[64];
  int dev = 0;
  CDL_CUDA(cudaGetDevice(&dev));
  cudaError_t attr_err = cudaSuccess;
  std::call_once(attr_once[dev & 63], [&] {
    attr_err = cudaFuncSetAttribute(attn_fwd::attn_fwd_kernel,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(attn_fwd::SMEM_BYTES));
  });
  if (attr_err != cudaSuccess)
    return fail(CDL_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(attr_err));
  return CDL_OK;
}

int32_t attn_fwd_execute(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                         const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* lse,
                         cudaStream_t stream) {
  using namespace attn_fwd;
  const char* op = "attention_fwd";
  if (!desc || !q || !k || !v || !o) return fail(CDL_ERR_INVALID, "%s: desc, q, k, v, o are required", op);
  if (q->rank != 4 || k->rank != 4)
    return fail(CDL_ERR_INVALID, "%s: q and k must be [batch, seqlen, heads, head_dim]", op);
  const long long B = q->shape[0], Sq = q->shape[1], H = q->shape[2], Dh = q->shape[3];
  const long long Sk = k->shape[1], Hkv = k->shape[2];
  if (Dh != D)
    return fail(CDL_ERR_UNSUPPORTED, "%s: head dimension %lld is not implemented (only 128 of the "
                "reference's {64, 96, 128, 256})", op, Dh);
  if (Hkv <= 0 || H % Hkv != 0)
    return fail(CDL_ERR_INVALID, "%s: query heads (%lld) must be a multiple of kv heads (%lld)", op,
                H, Hkv);
  CDL_CHECK(attn_check_operand(op, "q", q, B, Sq, H, D));
  CDL_CHECK(attn_check_operand(op, "k", k, B, Sk, Hkv, D));
  CDL_CHECK(attn_check_operand(op, "v", v, B, Sk, Hkv, D));
  CDL_CHECK(attn_check_operand(op, "out", o, B, Sq, H, D));
  if (lse) {
    if (lse->rank != 3 || lse->shape[0] != B || lse->shape[1] != H || lse->shape[2] != Sq ||
        lse->dtype != CDL_F32)
      return fail(CDL_ERR_INVALID, "%s: lse must be f32 [batch, heads, seqlen_q]", op);
  }
  if (B == 0 || Sq == 0 || H == 0) return CDL_OK;
  if (B > 65535 || H > 65535 || Sq > (1 << 30) || Sk > (1 << 30))
    return fail(CDL_ERR_UNSUPPORTED, "%s: dimension too large", op);

  Params p;
  p.B = static_cast<int>(B);
  p.H = static_cast<int>(H);
  p.Hkv = static_cast<int>(Hkv);
  p.Sq = static_cast<int>(Sq);
  p.Sk = static_cast<int>(Sk);
  p.causal = desc->causal != 0;
  const float scale = desc->softmax_scale > 0.f ? desc->softmax_scale : 1.0f / sqrtf(static_cast<float>(D));
  p.scale_log2 = scale * 1.4426950408889634f;
  p.o = static_cast<__nv_bfloat16*>(o->ptr);
  p.o_sb = o->stride[0];
  p.o_ss = o->stride[1];
  p.o_sh = o->stride[2];
  p.lse = lse ? static_cast<float*>(lse->ptr) : nullptr;
  p.lse_sb = lse ? lse->stride[0] : 0;
  p.lse_sh = lse ? lse->stride[1] : 0;
  p.lse_ss = lse ? lse->stride[2] : 0;
  p.cu_q = nullptr;
  p.cu_k = nullptr;
  p.status = device_status_ptr();
  if (!p.status) return fail(CDL_ERR_CUDA, "cannot resolve the device status word");

  const int variant = desc->variant;
  if (variant < CDL_ATTN_AUTO || variant > CDL_ATTN_PERSISTENT)
    return fail(CDL_ERR_INVALID, "%s: unknown kernel variant %d", op, variant);
  if (variant != CDL_ATTN_ONE_SHOT) {
    ProfileScope ps(PROF_ATTN_FWD, 4.0 * B * H * Sq * Sk * D * (p.causal ? 0.5 : 1.0), stream);
    return attn_fwd_persistent_launch(q, k, v, B, H, Hkv, Sq, Sk, p.causal != 0, p.scale_log2, p.o, p.o_sb,
                                p.o_ss, p.o_sh, p.lse, p.lse_sb, p.lse_sh, p.lse_ss, nullptr, nullptr,
                                Sk > 0, stream);
  }

  CUtensorMap tq, tk, tv;
  if (Sk > 0) {
    CDL_CHECK(attn_encode_tmap(&tq, q));
    CDL_CHECK(attn_encode_tmap(&tk, k));
    CDL_CHECK(attn_encode_tmap(&tv, v));
  } else {
    // No keys at all: the kernel never touches the maps (every tile has zero blocks).
    memset(&tq, 0, sizeof tq);
    tk = tq;
    tv = tq;
  }

  CDL_CHECK(fwd_set_attributes());
  dim3 grid(static_cast<unsigned>((Sq + 2 * BQ - 1) / (2 * BQ)), static_cast<unsigned>(H),
            static_cast<unsigned>(B));
  // FLOP by the flash-attention convention: 4 B H Sq Sk D, halved for the causal mask.
  ProfileScope ps(PROF_ATTN_FWD, 4.0 * B * H * Sq * Sk * D * (p.causal ? 0.5 : 1.0), stream);
  CDL_CUDA(launch_pdl(attn_fwd_kernel, grid, dim3(THREADS), SMEM_BYTES, stream, tq, tk, tv, p));
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}


// Checks a packed [total, heads, 128] bf16 operand and returns its [1, total, heads, 128] view.
int32_t attn_packed_view(const char* op, const char* name, const cdl_tensor* t, long long total,
                         long long heads, cdl_tensor* view) {
  if (!t) return fail(CDL_ERR_INVALID, "%s: %s is required", op, name);
  if (t->rank != 3 || t->shape[0] != total || t->shape[1] != heads || t->shape[2] != attn_fwd::D)
    return fail(CDL_ERR_INVALID, "%s: %s must have shape [%lld, %lld, %d]", op, name, total, heads,
                attn_fwd::D);
  view->ptr = t->ptr;
  view->dtype = t->dtype;
  view->rank = 4;
  view->shape[0] = 1;
  view->shape[1] = total;
  view->shape[2] = heads;
  view->shape[3] = attn_fwd::D;
  view->stride[0] = 0;
  view->stride[1] = t->stride[0];
  view->stride[2] = t->stride[1];
  view->stride[3] = t->stride[2];
  return attn_check_operand(op, name, view, 1, total, heads, attn_fwd::D);
}

// Checks an i32 [batch + 1] device vector of cumulative sequence lengths.
int32_t attn_check_cu_seqlens(const char* op, const char* name, const cdl_tensor* t, long long batch) {
  if (!t || t->rank != 1 || t->dtype != CDL_I32 || t->shape[0] != batch + 1 || t->stride[0] != 1 ||
      (reinterpret_cast<uintptr_t>(t->ptr) & 3) != 0)
    return fail(CDL_ERR_INVALID, "%s: %s must be a contiguous i32 vector of batch + 1 = %lld entries",
                op, name, batch + 1);
  return CDL_OK;
}

int32_t attn_fwd_packed_execute(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                                const cdl_tensor* v, const cdl_tensor* cu_q, const cdl_tensor* cu_k,
                                long long max_q, long long max_k, const cdl_tensor* o,
                                const cdl_tensor* lse, cudaStream_t stream) {
  using namespace attn_fwd;
  const char* op = "attention_fwd (packed)";
  if (!desc || !q || !k || !v || !o || !cu_q || !cu_k)
    return fail(CDL_ERR_INVALID, "%s: desc, q, k, v, cu_seqlens_q, cu_seqlens_k, o are required", op);
  if (q->rank != 3 || k->rank != 3)
    return fail(CDL_ERR_INVALID, "%s: q and k must be [total, heads, head_dim]", op);
  const long long Tq = q->shape[0], H = q->shape[1], Dh = q->shape[2];
  const long long Tk = k->shape[0], Hkv = k->shape[1];
  const long long B = cu_q->rank == 1 ? cu_q->shape[0] - 1 : -1;
  if (Dh != D)
    return fail(CDL_ERR_UNSUPPORTED, "%s: head dimension %lld is not implemented (only 128)", op, Dh);
  if (Hkv <= 0 || H % Hkv != 0)
    return fail(CDL_ERR_INVALID, "%s: query heads (%lld) must be a multiple of kv heads (%lld)", op,
                H, Hkv);
  if (B < 0) return fail(CDL_ERR_INVALID, "%s: cu_seqlens_q must hold batch + 1 entries", op);
  CDL_CHECK(attn_check_cu_seqlens(op, "cu_seqlens_q", cu_q, B));
  CDL_CHECK(attn_check_cu_seqlens(op, "cu_seqlens_k", cu_k, B));
  cdl_tensor q4, k4, v4, o4;
  CDL_CHECK(attn_packed_view(op, "q", q, Tq, H, &q4));
  CDL_CHECK(attn_packed_view(op, "k", k, Tk, Hkv, &k4));
  CDL_CHECK(attn_packed_view(op, "v", v, Tk, Hkv, &v4));
  CDL_CHECK(attn_packed_view(op, "out", o, Tq, H, &o4));
  if (lse) {
    if (lse->rank != 2 || lse->shape[0] != H || lse->shape[1] != Tq || lse->dtype != CDL_F32)
      return fail(CDL_ERR_INVALID, "%s: lse must be f32 [heads, total_q]", op);
  }
  if (max_q <= 0 || max_q > Tq) max_q = Tq;  // the bound only sizes the grid
  if (max_k <= 0 || max_k > Tk) max_k = Tk;
  if (B == 0 || Tq == 0 || H == 0) return CDL_OK;
  if (B > 65535 || H > 65535 || Tq > (1 << 30) || Tk > (1 << 30))
    return fail(CDL_ERR_UNSUPPORTED, "%s: dimension too large", op);

  Params p;
  p.B = static_cast<int>(B);
  p.H = static_cast<int>(H);
  p.Hkv = static_cast<int>(Hkv);
  p.Sq = static_cast<int>(max_q);
  p.Sk = static_cast<int>(max_k);
  p.causal = desc->causal != 0;
  const float scale = desc->softmax_scale > 0.f ? desc->softmax_scale : 1.0f / sqrtf(static_cast<float>(D));
  p.scale_log2 = scale * 1.4426950408889634f;
  p.o = static_cast<__nv_bfloat16*>(o->ptr);
  p.o_sb = 0;
  p.o_ss = o->stride[0];
  p.o_sh = o->stride[1];
  p.lse = lse ? static_cast<float*>(lse->ptr) : nullptr;
  p.lse_sb = 0;
  p.lse_sh = lse ? lse->stride[0] : 0;
  p.lse_ss = lse ? lse->stride[1] : 0;
  p.cu_q = static_cast<const int*>(cu_q->ptr);
  p.cu_k = static_cast<const int*>(cu_k->ptr);
  p.status = device_status_ptr();
  if (!p.status) return fail(CDL_ERR_CUDA, "cannot resolve the device status word");

  const int variant = desc->variant;
  if (variant < CDL_ATTN_AUTO || variant > CDL_ATTN_PERSISTENT)
    return fail(CDL_ERR_INVALID, "%s: unknown kernel variant %d", op, variant);
  if (variant != CDL_ATTN_ONE_SHOT) {
    const double mq = static_cast<double>(Tq) / B, mk = static_cast<double>(Tk) / B;
    ProfileScope ps(PROF_ATTN_FWD, 4.0 * B * H * mq * mk * D * (p.causal ? 0.5 : 1.0), stream);
    return attn_fwd_persistent_launch(&q4, &k4, &v4, B, H, Hkv, max_q, max_k, p.causal != 0, p.scale_log2, p.o,
                                0, p.o_ss, p.o_sh, p.lse, 0, p.lse_sh, p.lse_ss, p.cu_q, p.cu_k, Tk > 0,
                                stream);
  }

  CUtensorMap tq, tk, tv;
  if (Tk > 0) {
    CDL_CHECK(attn_encode_tmap(&tq, &q4));
    CDL_CHECK(attn_encode_tmap(&tk, &k4));
    CDL_CHECK(attn_encode_tmap(&tv, &v4));
  } else {
    memset(&tq, 0, sizeof tq);
    tk = tq;
    tv = tq;
  }
  CDL_CHECK(fwd_set_attributes());
  dim3 grid(static_cast<unsigned>((max_q + 2 * BQ - 1) / (2 * BQ)), static_cast<unsigned>(H),
            static_cast<unsigned>(B));
  // The sequence lengths live on the device: the work figure uses the packed totals as if every
  // sequence had the mean length.
  const double mean_q = static_cast<double>(Tq) / B, mean_k = static_cast<double>(Tk) / B;
  ProfileScope ps(PROF_ATTN_FWD, 4.0 * B * H * mean_q * mean_k * D * (p.causal ? 0.5 : 1.0), stream);
  CDL_CUDA(launch_pdl(attn_fwd_kernel, grid, dim3(THREADS), SMEM_BYTES, stream, tq, tk, tv, p));
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

}  // namespace cdl

extern "C" {

int32_t cdl_b200_attn_fwd_packed(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                                 const cdl_tensor* v, const cdl_tensor* cu_seqlens_q,
                                 const cdl_tensor* cu_seqlens_k, int64_t max_seqlen_q,
                                 int64_t max_seqlen_k, const cdl_tensor* o, const cdl_tensor* lse,
                                 cdl_stream stream) {
  return cdl::attn_fwd_packed_execute(desc, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                                      max_seqlen_k, o, lse, static_cast<cudaStream_t>(stream));
}

int32_t cdl_b200_attn_fwd(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                          const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* lse,
                          cdl_stream stream) {
  return cdl::attn_fwd_execute(desc, q, k, v, o, lse, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
