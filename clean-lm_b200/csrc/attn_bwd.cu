// Flash attention backward on tcgen05 tensor cores: dQ, dK, dV from Q, K, V, O, dO and LSE.
//
// Operator semantics follow AttentionBwd of the reference (crates/cleandl/src/execgraph/ops/
// attention/mod.rs:366-374, 852-935; operand order q, k, v, out, d_out, lse :899-905), whose
// arithmetic lives in flash-attention-rs; the math is the one of the reference's f64 test oracle
// (crates/cleandl/tests/attention.rs:444-462):
//   delta_i = sum_d dO_id O_id;  P = exp(S - LSE);  dV = P^T dO;  dP = dO V^T;
//   dS = P o (dP - delta) * scale;  dQ = dS K;  dK = dS^T Q.
//
// Three kernels:
//   1. preprocess: delta and LSE * log2(e) per query row into scratch (rows padded to 128).
//   2. main: one CTA per (128-key block, kv head, batch) walks the query blocks that see it.
//      Everything is computed TRANSPOSED so that a thread owns one key row:
//        S^T  = K Q^T          (SS)  -> TMEM [0,128)     P^T (bf16) overwrites it in place
//        dP^T = V dO^T         (SS)  -> TMEM [128,256)
//        dV  += P^T dO         (A = P^T from TMEM)        -> TMEM [256,384)
//        dK  += dS^T Q         (A = dS^T from shared)     -> TMEM [384,512)
//        dQ   = dS K           (SS)  -> TMEM [128,256), added to an f32 dQ accumulator in global
//                                      memory by TMA reduce operations issued by a dedicated
//                                      warp group (staged through shared memory).
//      dS^T is written once to shared memory in the 128-byte-swizzled layout that serves both as
//      the K-major A operand of the dK product and as the MN-major A operand of the dQ product.
//   3. postprocess: dQ accumulator f32 -> bf16.
// Scratch: dQ accumulator [B, Sq, H, D] f32, then LSE2 and delta [B, H, Sq_pad] f32.
#include "host.h"
#include "ptx.cuh"

#include <math.h>
#include <string.h>

#include <mutex>

namespace cdl {

int32_t attn_check_operand(const char* op, const char* name, const cdl_tensor* t, long long B,
                           long long S, long long H, long long D);
int32_t attn_encode_tmap(CUtensorMap* out, const cdl_tensor* t);

namespace attn_bwd {

constexpr int D = 128;
constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int TILE_BYTES = 128 * 128 * 2;
constexpr int PANEL_BYTES = TILE_BYTES / 2;
constexpr int THREADS = 512;  // warps 0-3 control (TMA, MMA, 2 idle), 4-11 compute, 12-15 dQ reduce
constexpr int DQ_CHUNK_BYTES = 128 * 32 * 4;  // 128 query rows x 32 head-dim columns of f32
constexpr int TMEM_COLS = 512;
constexpr int COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DK = 384;
// K, V, Q x 2 stages, dO, dS^T, 2 dQ staging chunks
constexpr size_t SMEM_BYTES =
    6 * TILE_BYTES + 2 * DQ_CHUNK_BYTES + 2 * 2 * 128 * sizeof(float) + 256;
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KiB of shared memory a CTA can opt in to");

struct Params {
  int B, H, Hkv, Sq, Sk, Sq_pad;
  int causal;
  float scale, scale_log2;
  const float* lse2;   // [B, H, Sq_pad]  LSE * log2(e), +inf for rows that contribute nothing
  const float* delta;  // [B, H, Sq_pad]
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  long long dk_sb, dk_ss, dk_sh, dv_sb, dv_ss, dv_sh;
  int* status;
};

struct Barriers {
  uint64_t kv_full;
  uint64_t q_full[2], q_empty[2];
  uint64_t do_full, do_empty;
  uint64_t s_full, dp_full, p_ready, ds_ready, dq_full, dq_read;
  uint32_t tmem_base;
  int abort_word;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void compute_bar_sync() {
  asm volatile("bar.sync 1, 256;" ::: "memory");
}
__device__ __forceinline__ void reduce_bar_sync() {
  asm volatile("bar.sync 2, 128;" ::: "memory");
}

// ---------------------------------------------------------------- preprocess
// Half a warp per (b, h, padded row): 16 lanes x 8 bf16 = one 256-byte row of O and of dO.
// delta = sum_d dO * O, lse2 = lse * log2(e).
__global__ void __launch_bounds__(256)
    attn_bwd_preprocess_kernel(const __nv_bfloat16* __restrict__ o, long long o_sb, long long o_ss,
                               long long o_sh, const __nv_bfloat16* __restrict__ d_o,
                               long long do_sb, long long do_ss, long long do_sh,
                               const float* __restrict__ lse, long long lse_sb, long long lse_sh,
                               long long lse_ss, float* __restrict__ lse2,
                               float* __restrict__ delta, int B, int H, int Sq, int Sq_pad) {
  const long long item = (static_cast<long long>(blockIdx.x) * 256 + threadIdx.x) >> 4;
  const int sub = threadIdx.x & 15;
  const long long total = static_cast<long long>(B) * H * Sq_pad;
  const bool live = item < total;
  const long long it = live ? item : 0;
  const int row = static_cast<int>(it % Sq_pad);
  const int h = static_cast<int>((it / Sq_pad) % H);
  const int b = static_cast<int>(it / (static_cast<long long>(Sq_pad) * H));
  float dl = 0.f, l2 = INFINITY;
  const bool in = live && row < Sq;
  if (in) {
    const uint4 vo = ld_nc_v4(o + b * o_sb + row * o_ss + h * o_sh + sub * 8);
    const uint4 vd = ld_nc_v4(d_o + b * do_sb + row * do_ss + h * do_sh + sub * 8);
    dl = bf16_lo(vo.x) * bf16_lo(vd.x) + bf16_hi(vo.x) * bf16_hi(vd.x) +
         bf16_lo(vo.y) * bf16_lo(vd.y) + bf16_hi(vo.y) * bf16_hi(vd.y) +
         bf16_lo(vo.z) * bf16_lo(vd.z) + bf16_hi(vo.z) * bf16_hi(vd.z) +
         bf16_lo(vo.w) * bf16_lo(vd.w) + bf16_hi(vo.w) * bf16_hi(vd.w);
  }
#pragma unroll
  for (int s = 8; s > 0; s >>= 1) dl += __shfl_xor_sync(0xffffffffu, dl, s);
  if (in && sub == 0) {
    const float l = lse[b * lse_sb + h * lse_sh + row * lse_ss];
    l2 = l == -INFINITY ? INFINITY : l * 1.4426950408889634f;
  }
  if (live && sub == 0) {
    lse2[item] = l2;
    delta[item] = dl;
  }
}

// ---------------------------------------------------------------- postprocess
__global__ void __launch_bounds__(256)
    attn_bwd_convert_dq_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq,
                               long long dq_sb, long long dq_ss, long long dq_sh, int B, int Sq,
                               int H) {
  // one thread per 8 consecutive d
  const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  const long long total = static_cast<long long>(B) * Sq * H * (D / 8);
  if (idx >= total) return;
  const int d8 = static_cast<int>(idx % (D / 8));
  const int h = static_cast<int>((idx / (D / 8)) % H);
  const int s = static_cast<int>((idx / (D / 8) / H) % Sq);
  const int b = static_cast<int>(idx / (D / 8) / H / Sq);
  const float4 a0 = *reinterpret_cast<const float4*>(acc + idx * 8);
  const float4 a1 = *reinterpret_cast<const float4*>(acc + idx * 8 + 4);
  uint4 q;
  q.x = pack_bf16x2(a0.x, a0.y);
  q.y = pack_bf16x2(a0.z, a0.w);
  q.z = pack_bf16x2(a1.x, a1.y);
  q.w = pack_bf16x2(a1.z, a1.w);
  *reinterpret_cast<uint4*>(dq + b * dq_sb + s * dq_ss + h * dq_sh + d8 * 8) = q;
}

// ---------------------------------------------------------------- main kernel
__global__ void __launch_bounds__(THREADS, 1)
    attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q,
                    const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v,
                    const __grid_constant__ CUtensorMap tmap_do,
                    const __grid_constant__ CUtensorMap tmap_dq, const Params p) {
  // 227 KiB are used to the last kilobyte, so there is no room for manual alignment slack: the
  // 1024-byte alignment the swizzled tiles need is requested from the compiler and verified.
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(p.status, 901);
    return;
  }
  uint8_t* s_k = smem;
  uint8_t* s_v = smem + TILE_BYTES;
  uint8_t* s_q = smem + 2 * TILE_BYTES;  // 2 stages
  uint8_t* s_do = smem + 4 * TILE_BYTES;
  uint8_t* s_ds = smem + 5 * TILE_BYTES;
  uint8_t* s_dq = smem + 6 * TILE_BYTES;  // 2 staging chunks for the dQ reduction
  float* s_lse = reinterpret_cast<float*>(smem + 6 * TILE_BYTES + 2 * DQ_CHUNK_BYTES);  // [2][128]
  float* s_delta = s_lse + 2 * 128;                                // [2][128]
  Barriers* bars = reinterpret_cast<Barriers*>(s_delta + 2 * 128);
  volatile int* abort_word = &bars->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_blk = blockIdx.x;
  const int kvh = blockIdx.y;
  const int b = blockIdx.z;
  const int key0 = n_blk * BKV;
  const int group = p.H / p.Hkv;
  const int shift = p.Sk - p.Sq;  // query i sees keys <= i + shift
  const int num_q_blocks = (p.Sq + BQ - 1) / BQ;
  const int m_start = p.causal ? max(0, key0 - shift) / BQ : 0;
  const int m_count = max(0, num_q_blocks - m_start);
  const int iters = m_count * group;  // iteration it -> head kvh*group + it / m_count, block m_start + it % m_count

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->q_full[i], 1);
      mbar_init(&bars->q_empty[i], 1);
    }
    mbar_init(&bars->do_full, 1);
    mbar_init(&bars->do_empty, 1);
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->p_ready, 256);
    mbar_init(&bars->ds_ready, 256);
    mbar_init(&bars->dq_full, 1);
    mbar_init(&bars->dq_read, 128);
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    setmaxnreg_dec<40>();
    if (elect_one() && iters > 0) {
      mbar_arrive_expect_tx(&bars->kv_full, 2 * TILE_BYTES);
#pragma unroll
      for (int dh = 0; dh < 2; ++dh) {
        tma_load_4d(s_k + dh * PANEL_BYTES, &tmap_k, &bars->kv_full, dh * 64, key0, kvh, b);
        tma_load_4d(s_v + dh * PANEL_BYTES, &tmap_v, &bars->kv_full, dh * 64, key0, kvh, b);
      }
      for (int it = 0; it < iters; ++it) {
        const int h = kvh * group + it / m_count;
        const int q0 = (m_start + it % m_count) * BQ;
        const int s = it & 1;
        if (!mbar_wait(&bars->q_empty[s], ((it >> 1) & 1) ^ 1, abort_word, 121)) break;
        mbar_arrive_expect_tx(&bars->q_full[s], TILE_BYTES);
#pragma unroll
        for (int dh = 0; dh < 2; ++dh)
          tma_load_4d(s_q + s * TILE_BYTES + dh * PANEL_BYTES, &tmap_q, &bars->q_full[s], dh * 64,
                      q0, h, b);
        if (!mbar_wait(&bars->do_empty, (it & 1) ^ 1, abort_word, 122)) break;
        mbar_arrive_expect_tx(&bars->do_full, TILE_BYTES);
#pragma unroll
        for (int dh = 0; dh < 2; ++dh)
          tma_load_4d(s_do + dh * PANEL_BYTES, &tmap_do, &bars->do_full, dh * 64, q0, h, b);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // Issue order per iteration: dP^T(it), dV(it), S^T(it+1), dK(it), dQ(it).  S^T of the next
    // query block is issued before this block's dK / dQ so the compute warps can turn it into
    // P^T while those two products run.
    setmaxnreg_dec<40>();
    if (elect_one() && iters > 0) {
      const uint32_t idesc_kk = make_idesc_bf16(128, 128, 0, 0);  // both operands K-major
      const uint32_t idesc_kmn = make_idesc_bf16(128, 128, 0, 1); // A K-major / TMEM, B MN-major
      const uint32_t idesc_mnmn = make_idesc_bf16(128, 128, 1, 1);
      const uint32_t k_addr = smem_u32(s_k), v_addr = smem_u32(s_v), q_addr = smem_u32(s_q);
      const uint32_t do_addr = smem_u32(s_do), ds_addr = smem_u32(s_ds);
      auto koff = [](int k) { return static_cast<uint32_t>((k >> 2) * PANEL_BYTES + (k & 3) * 32); };
      auto issue_s = [&](int it) {  // S^T = K Q^T
        const uint32_t qa = q_addr + (it & 1) * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(tmem_base + COL_S, smem_desc_sw128(k_addr + koff(k), 16, 1024),
                  smem_desc_sw128(qa + koff(k), 16, 1024), idesc_kk, k != 0);
        umma_commit(&bars->s_full);
      };
      bool ok = mbar_wait(&bars->kv_full, 0, abort_word, 221) &&
                mbar_wait(&bars->q_full[0], 0, abort_word, 222);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int it = 0; it < iters && ok; ++it) {
        const int s = it & 1;
        const uint32_t ph = it & 1;
        const uint32_t qa = q_addr + s * TILE_BYTES;
        // dP^T = V dO^T  (its TMEM columns held dQ of the previous iteration)
        ok = mbar_wait(&bars->do_full, ph, abort_word, 223);
        if (ok && it > 0) ok = mbar_wait(&bars->dq_read, (it - 1) & 1, abort_word, 224);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(tmem_base + COL_DP, smem_desc_sw128(v_addr + koff(k), 16, 1024),
                  smem_desc_sw128(do_addr + koff(k), 16, 1024), idesc_kk, k != 0);
        umma_commit(&bars->dp_full);
        // dV += P^T dO
        ok = mbar_wait(&bars->p_ready, ph, abort_word, 225);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ts(tmem_base + COL_DV, tmem_base + COL_S + k * 8,
                  smem_desc_sw128(do_addr + k * 2048, PANEL_BYTES, 1024), idesc_kmn,
                  (it > 0 || k != 0) ? 1u : 0u);
        // dO is free once dP^T and dV have read it: this commit covers both.
        umma_commit(&bars->do_empty);
        // S^T of the next query block; it overwrites P^T, which dV (issued above) reads first.
        if (it + 1 < iters) {
          ok = mbar_wait(&bars->q_full[s ^ 1], ((it + 1) >> 1) & 1, abort_word, 227);
          if (!ok) break;
          tc_fence_after();
          issue_s(it + 1);
        }
        // dK += dS^T Q ;  dQ = dS K   (dS^T tile: K-major A for dK, MN-major A for dQ)
        ok = mbar_wait(&bars->ds_ready, ph, abort_word, 226);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(tmem_base + COL_DK, smem_desc_sw128(ds_addr + koff(k), 16, 1024),
                  smem_desc_sw128(qa + k * 2048, PANEL_BYTES, 1024), idesc_kmn,
                  (it > 0 || k != 0) ? 1u : 0u);
        umma_commit(&bars->q_empty[s]);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(tmem_base + COL_DP, smem_desc_sw128(ds_addr + k * 2048, PANEL_BYTES, 1024),
                  smem_desc_sw128(k_addr + k * 2048, PANEL_BYTES, 1024), idesc_mnmn, k != 0);
        umma_commit(&bars->dq_full);
      }
    }
  } else if (warp < 4) {
    setmaxnreg_dec<40>();
  } else if (warp >= 12) {
    // ------------------------------------------------------------ dQ reduction warps (12..15)
    // One thread per query row.  The dQ tile is moved TMEM -> registers -> swizzled shared
    // memory in four 32-column chunks (two staging buffers) and added to the f32 accumulator in
    // global memory by TMA reduce operations, so no atomic instruction goes through the LSU.
    setmaxnreg_dec<72>();
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const bool leader = threadIdx.x == 12 * 32;
    bool ok = true;
    for (int it = 0; it < iters && ok; ++it) {
      const int h = kvh * group + it / m_count;
      const int q0 = (m_start + it % m_count) * BQ;
      if (!mbar_wait(&bars->dq_full, it & 1, abort_word, 421)) { ok = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint8_t* stage = s_dq + (c & 1) * DQ_CHUNK_BYTES;
        // The reduce issued from this staging buffer two chunks ago must have read it.
        if (leader) tma_store_wait_read<1>();
        reduce_bar_sync();
        uint32_t v[32];
        tmem_ld32(tmem_base + lane_addr + COL_DP + c * 32, v);
        tmem_wait_ld();
        if (c == 3) {
          tc_fence_before();
          mbar_arrive(&bars->dq_read);  // the tile is out of TMEM: dP^T of the next block may land
        }
        uint8_t* row_ptr = stage + r * 128;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch)
          *reinterpret_cast<uint4*>(row_ptr + ((ch ^ (r & 7)) << 4)) =
              make_uint4(v[ch * 4], v[ch * 4 + 1], v[ch * 4 + 2], v[ch * 4 + 3]);
        fence_proxy_async_smem();
        reduce_bar_sync();
        if (leader) {
          tma_reduce_add_4d(&tmap_dq, stage, c * 32, h, q0, b);
          tma_store_commit();
        }
      }
    }
    if (leader) tma_store_wait<0>();
  } else {
    // ------------------------------------------------------------ compute warps (4..11)
    // Software pipeline per iteration: dS(it), then P(it+1), which runs while the tensor core
    // computes dK(it) and dQ(it).
    setmaxnreg_inc<200>();
    const int ct = threadIdx.x - 128;  // 0..255
    const int wg = (warp - 4) >> 2;    // column half this thread works on
    const int quad = warp & 3;
    const int r = quad * 32 + lane;    // row inside the block == TMEM lane
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
      if (ct < 128) s_lse[stage * 128 + ct] = v;
      else s_delta[stage * 128 + ct - 128] = v;
    };
    float pr[64];

    // P^T(it) = exp2(S^T * scale_log2 - lse2) -> registers and (bf16) TMEM
    auto p_phase = [&](int it) -> bool {
      const int q0 = it_q0(it);
      const float4* lse_s = reinterpret_cast<const float4*>(s_lse + (it & 1) * 128 + wg * 64);
      const bool need_mask = (p.causal && key0 + BKV - 1 > q0 + shift) || key0 + BKV > p.Sk;
      if (!mbar_wait(&bars->s_full, it & 1, abort_word, 321)) return false;
      tc_fence_after();
      {
        uint32_t sr[2][32];
        tmem_ld32(tmem_base + lane_addr + COL_S + wg * 64, sr[0]);
        tmem_ld32(tmem_base + lane_addr + COL_S + wg * 64 + 32, sr[1]);
        tmem_wait_ld();
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4) {
          const float4 l4 = lse_s[c4];
          const float l[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = c4 * 4 + j;
            float v = ex2(fmaf(__uint_as_float(sr[c >> 5][c & 31]), p.scale_log2, -l[j]));
            if (need_mask) {
              const int qrow = q0 + wg * 64 + c;
              if (key >= p.Sk || (p.causal && key > qrow + shift)) v = 0.f;
            }
            pr[c] = v;
          }
        }
      }
      compute_bar_sync();  // both halves have read S^T before P^T overwrites its columns
      {
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) pk[c] = pack_bf16x2(pr[2 * c], pr[2 * c + 1]);
        tmem_st32(tmem_base + lane_addr + COL_S + wg * 32, pk);
        tmem_wait_st();
      }
      tc_fence_before();
      mbar_arrive(&bars->p_ready);
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

      // ---- dS^T = P^T o (dP^T - delta) * scale  -> shared memory (128-byte swizzle)
      if (!mbar_wait(&bars->dp_full, ph, abort_word, 322)) { ok = false; break; }
      tc_fence_after();
      {
        const float4* delta_s = reinterpret_cast<const float4*>(s_delta + (it & 1) * 128 + wg * 64);
        uint32_t dr[2][32];
        tmem_ld32(tmem_base + lane_addr + COL_DP + wg * 64, dr[0]);
        tmem_ld32(tmem_base + lane_addr + COL_DP + wg * 64 + 32, dr[1]);
        tmem_wait_ld();
        uint8_t* row_ptr = s_ds + wg * PANEL_BYTES + r * 128;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const float4 d0 = delta_s[ch * 2], d1 = delta_s[ch * 2 + 1];
          const float dl[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
          float d[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int c = ch * 8 + j;
            d[j] = pr[c] * (__uint_as_float(dr[c >> 5][c & 31]) - dl[j]) * p.scale;
          }
          uint4 q;
          q.x = pack_bf16x2(d[0], d[1]);
          q.y = pack_bf16x2(d[2], d[3]);
          q.z = pack_bf16x2(d[4], d[5]);
          q.w = pack_bf16x2(d[6], d[7]);
          *reinterpret_cast<uint4*>(row_ptr + ((ch ^ (r & 7)) << 4)) = q;
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&bars->ds_ready);

      // ---- P^T of the next query block (overlaps the dK / dQ products of this one)
      if (it + 1 < iters && !p_phase(it + 1)) { ok = false; break; }

      // Statistics of iteration it + 2 replace those of iteration it (all reads of them are
      // behind the barrier inside p_phase above or, for the last iterations, behind this one).
      compute_bar_sync();
      if (it + 2 < iters) store_stat(it & 1, stat_next);
      compute_bar_sync();
    }

    // ---- epilogue: dV and dK rows of this key block (every product has finished once the last
    // dQ commit has arrived)
    if (ok && iters > 0) {
      ok = mbar_wait(&bars->dq_full, (iters - 1) & 1, abort_word, 324);
      tc_fence_after();
    }
    if (ok) {
      const bool row_ok = key < p.Sk;
      __nv_bfloat16* dv_row = p.dv + b * p.dv_sb + static_cast<long long>(key) * p.dv_ss + kvh * p.dv_sh + wg * 64;
      __nv_bfloat16* dk_row = p.dk + b * p.dk_sb + static_cast<long long>(key) * p.dk_ss + kvh * p.dk_sh + wg * 64;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = which == 0 ? dv_row : dk_row;
        const uint32_t col = (which == 0 ? COL_DV : COL_DK) + wg * 64;
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
          if (row_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 q;
              q.x = pack_bf16x2(__uint_as_float(a[g * 8 + 0]), __uint_as_float(a[g * 8 + 1]));
              q.y = pack_bf16x2(__uint_as_float(a[g * 8 + 2]), __uint_as_float(a[g * 8 + 3]));
              q.z = pack_bf16x2(__uint_as_float(a[g * 8 + 4]), __uint_as_float(a[g * 8 + 5]));
              q.w = pack_bf16x2(__uint_as_float(a[g * 8 + 6]), __uint_as_float(a[g * 8 + 7]));
              *reinterpret_cast<uint4*>(dst + half * 32 + g * 8) = q;
            }
          }
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

static long long pad128(long long v) { return (v + 127) / 128 * 128; }

}  // namespace attn_bwd

size_t attn_bwd_scratch_bytes(long long B, long long Sq, long long H) {
  using namespace attn_bwd;
  return static_cast<size_t>(B) * Sq * H * D * sizeof(float) +
         2 * static_cast<size_t>(B) * H * pad128(Sq) * sizeof(float);
}

int32_t attn_bwd_execute(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                         const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* d_o,
                         const cdl_tensor* lse, const cdl_tensor* dq, const cdl_tensor* dk,
                         const cdl_tensor* dv, void* scratch, size_t scratch_bytes,
                         cudaStream_t stream) {
  using namespace attn_bwd;
  const char* op = "attention_bwd";
  if (!desc || !q || !k || !v || !o || !d_o || !lse || !dq || !dk || !dv)
    return fail(CDL_ERR_INVALID, "%s: every operand is required", op);
  if (q->rank != 4 || k->rank != 4)
    return fail(CDL_ERR_INVALID, "%s: q and k must be [batch, seqlen, heads, head_dim]", op);
  const long long B = q->shape[0], Sq = q->shape[1], H = q->shape[2], Dh = q->shape[3];
  const long long Sk = k->shape[1], Hkv = k->shape[2];
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
  if (B > 65535 || Hkv > 65535 || Sq > (1 << 30) || Sk > (1 << 30))
    return fail(CDL_ERR_UNSUPPORTED, "%s: dimension too large", op);
  const size_t need = attn_bwd_scratch_bytes(B, Sq, H);
  if (need > 0 && (scratch == nullptr || scratch_bytes < need ||
                   (reinterpret_cast<uintptr_t>(scratch) & 15) != 0))
    return fail(CDL_ERR_INVALID, "%s: scratch must be 16-byte aligned and hold %zu bytes (got %zu)",
                op, need, scratch_bytes);

  const long long Sq_pad = pad128(Sq);
  float* dq_acc = static_cast<float*>(scratch);
  float* lse2 = dq_acc + B * Sq * H * D;
  float* delta = lse2 + B * H * Sq_pad;

  Params p;
  p.B = static_cast<int>(B);
  p.H = static_cast<int>(H);
  p.Hkv = static_cast<int>(Hkv);
  p.Sq = static_cast<int>(Sq);
  p.Sk = static_cast<int>(Sk);
  p.Sq_pad = static_cast<int>(Sq_pad);
  p.causal = desc->causal != 0;
  p.scale = desc->softmax_scale > 0.f ? desc->softmax_scale : 1.0f / sqrtf(static_cast<float>(D));
  p.scale_log2 = p.scale * 1.4426950408889634f;
  p.lse2 = lse2;
  p.delta = delta;
  p.dk = static_cast<__nv_bfloat16*>(dk->ptr);
  p.dv = static_cast<__nv_bfloat16*>(dv->ptr);
  p.dk_sb = dk->stride[0]; p.dk_ss = dk->stride[1]; p.dk_sh = dk->stride[2];
  p.dv_sb = dv->stride[0]; p.dv_ss = dv->stride[1]; p.dv_sh = dv->stride[2];
  p.status = device_status_ptr();
  if (!p.status) return fail(CDL_ERR_CUDA, "cannot resolve the device status word");

  ProfileScope ps(PROF_ATTN_BWD, 10.0 * B * H * Sq * Sk * D * (p.causal ? 0.5 : 1.0), stream);
  if (Sq > 0) {
    CDL_CUDA(cudaMemsetAsync(dq_acc, 0, static_cast<size_t>(B) * Sq * H * D * sizeof(float), stream));
    const long long items = B * H * Sq_pad;
    const unsigned blocks = static_cast<unsigned>((items * 16 + 255) / 256);
    attn_bwd_preprocess_kernel<<<blocks, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(o->ptr), o->stride[0], o->stride[1], o->stride[2],
        static_cast<const __nv_bfloat16*>(d_o->ptr), d_o->stride[0], d_o->stride[1], d_o->stride[2],
        static_cast<const float*>(lse->ptr), lse->stride[0], lse->stride[1], lse->stride[2], lse2,
        delta, p.B, p.H, p.Sq, p.Sq_pad);
    CDL_CUDA(cudaGetLastError());
  }

  if (Sk > 0) {
    CUtensorMap tq, tk, tv, tdo;
    if (Sq > 0) {
      CDL_CHECK(attn_encode_tmap(&tq, q));
      CDL_CHECK(attn_encode_tmap(&tdo, d_o));
    } else {
      memset(&tq, 0, sizeof tq);
      tdo = tq;
    }
    CDL_CHECK(attn_encode_tmap(&tk, k));
    CDL_CHECK(attn_encode_tmap(&tv, v));
    CUtensorMap tdq;
    if (Sq > 0) {
      // f32 accumulator [B, Sq, H, D] seen innermost-first as (D, H, Sq, B); one reduce moves a
      // 32-column x 128-row chunk of one head.
      const uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(H),
                                static_cast<uint64_t>(Sq), static_cast<uint64_t>(B)};
      const uint64_t strides[4] = {0, static_cast<uint64_t>(D) * 4, static_cast<uint64_t>(H) * D * 4,
                                   static_cast<uint64_t>(Sq) * H * D * 4};
      const uint32_t box[4] = {32, 1, 128, 1};
      CDL_CHECK(encode_tmap(&tdq, dq_acc, CDL_F32, 4, dims, strides, box, true));
    } else {
      memset(&tdq, 0, sizeof tdq);
    }

    static std::once_flag attr_once[64];
    int dev = 0;
    CDL_CUDA(cudaGetDevice(&dev));
    cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once[dev & 63], [&] {
      attr_err = cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(SMEM_BYTES));
    });
    if (attr_err != cudaSuccess)
      return fail(CDL_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(attr_err));

    dim3 grid(static_cast<unsigned>((Sk + BKV - 1) / BKV), static_cast<unsigned>(Hkv),
              static_cast<unsigned>(B));
    attn_bwd_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(tq, tk, tv, tdo, tdq, p);
    CDL_CUDA(cudaGetLastError());
  }

  if (Sq > 0) {
    const long long total = B * Sq * H * (D / 8);
    attn_bwd_convert_dq_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
        dq_acc, static_cast<__nv_bfloat16*>(dq->ptr), dq->stride[0], dq->stride[1], dq->stride[2],
        p.B, p.Sq, p.H);
    CDL_CUDA(cudaGetLastError());
  }
  return CDL_OK;
}

}  // namespace cdl

extern "C" {

int32_t cdl_b200_attn_bwd(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                          const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* d_out,
                          const cdl_tensor* lse, const cdl_tensor* dq, const cdl_tensor* dk,
                          const cdl_tensor* dv, void* scratch, size_t scratch_bytes,
                          cdl_stream stream) {
  return cdl::attn_bwd_execute(desc, q, k, v, o, d_out, lse, dq, dk, dv, scratch, scratch_bytes,
                               static_cast<cudaStream_t>(stream));
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
