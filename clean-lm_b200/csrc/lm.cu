// Loss and optimizer-step kernels of the sky-1 LM training step (all HBM-bound).
//
// The reference's kernels for these lived in its legacy `cleandl::operators::{loss, adamw,
// embedding}` module, which is not in its tree; the call sites are
//   cross-entropy producing the logits' gradient in the forward pass
//       crates/sky-1/src/training/model/mod.rs:262-271
//   embedding scatter-add                 crates/sky-1/src/training/model/mod.rs:351-356
//   gradient sum of squares + AdamW with global-norm clipping, f32 master -> bf16 replica, then
//   zero-filled gradients                 crates/sky-1/src/training/model/decoder.rs:716-752,
//                                         crates/sky-1/src/training/model/mod.rs:361-420
// The math is the textbook one (softmax cross-entropy, decoupled weight decay).
#include "host.h"
#include "ptx.cuh"

#include <math.h>

namespace cdl {
namespace lm {

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

constexpr int XENT_THREADS = 512;

// One CTA per token row.  Pass 1 streams the row from HBM and keeps an online (max, sum);
// pass 2 re-reads it (the row was just read, so it comes from L2) and overwrites it with
//   d_logits = (softmax - onehot(target)) * grad_scale.
// loss[row] = lse - logit[target]; rows with target < 0 are ignored (loss 0, gradient 0).
__global__ void __launch_bounds__(XENT_THREADS)
    xent_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, long long ld,
                        const int* __restrict__ targets, float* __restrict__ loss, int vocab,
                        float grad_scale) {
  __shared__ float s_m[XENT_THREADS / 32], s_s[XENT_THREADS / 32];
  __shared__ float s_lse;
  const long long row = blockIdx.x;
  __nv_bfloat16* x = logits + row * ld;
  const int target = targets[row];
  const int groups = vocab / 8;
  float m = -INFINITY, s = 0.f;
  for (int g = threadIdx.x; g < groups; g += XENT_THREADS) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(x + g * 8), f);
    float gm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) gm = fmaxf(gm, f[j]);
    const float nm = fmaxf(m, gm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  // combine (m, s) pairs: warp, then CTA
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
  }
  if ((threadIdx.x & 31) == 0) {
    s_m[threadIdx.x >> 5] = m;
    s_s[threadIdx.x >> 5] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float mm = s_m[0], ss = s_s[0];
    for (int w = 1; w < XENT_THREADS / 32; ++w) {
      const float nm = fmaxf(mm, s_m[w]);
      ss = (mm == -INFINITY ? 0.f : ss * __expf(mm - nm)) +
           (s_m[w] == -INFINITY ? 0.f : s_s[w] * __expf(s_m[w] - nm));
      mm = nm;
    }
    const float lse = mm + logf(ss);
    s_lse = lse;
    loss[row] = target >= 0 && target < vocab ? lse - __bfloat162float(x[target]) : 0.f;
  }
  __syncthreads();
  const float lse = s_lse;
  const float scale = target >= 0 && target < vocab ? grad_scale : 0.f;
  for (int g = threadIdx.x; g < groups; g += XENT_THREADS) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(x + g * 8), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p = __expf(f[j] - lse);
      f[j] = (p - (g * 8 + j == target ? 1.f : 0.f)) * scale;
    }
    *reinterpret_cast<uint4*>(x + g * 8) = pack8(f);
  }
}

// d_table[tokens[t], :] += d_x[t, :]  (f32 accumulate; order of the atomic adds is not fixed)
__global__ void __launch_bounds__(256)
    embedding_bwd_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ dx,
                         float* __restrict__ d_table, long long n_tokens, int hidden8, int vocab) {
  const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (idx >= n_tokens * hidden8) return;
  const long long t = idx / hidden8;
  const int g = static_cast<int>(idx - t * hidden8);
  const int tok = tokens[t];
  if (tok < 0 || tok >= vocab) return;
  float f[8];
  unpack8(ld_nc_v4(dx + idx * 8), f);
  float* dst = d_table + (static_cast<long long>(tok) * hidden8 + g) * 8;
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(f[0]), "f"(f[1]),
               "f"(f[2]), "f"(f[3])
               : "memory");
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4), "f"(f[4]), "f"(f[5]),
               "f"(f[6]), "f"(f[7])
               : "memory");
}

constexpr int RED_THREADS = 256;
constexpr int RED_BLOCKS = 1024;

__device__ __forceinline__ float block_sum(float v, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
  if (threadIdx.x < 32) {
    r = threadIdx.x < RED_THREADS / 32 ? smem[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  }
  return r;  // valid in thread 0
}

// partials[b] = sum of x^2 (square = 1) or of x (square = 0) over a fixed slice: deterministic.
__global__ void __launch_bounds__(RED_THREADS)
    reduce_partial_kernel(const float* __restrict__ x, long long n, float* __restrict__ partials,
                          int square) {
  __shared__ float smem[RED_THREADS / 32];
  float acc = 0.f;
  const long long n4 = n / 4;
  for (long long i = static_cast<long long>(blockIdx.x) * RED_THREADS + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * RED_THREADS) {
    const float4 v = *reinterpret_cast<const float4*>(x + i * 4);
    acc += square ? (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w) : (v.x + v.y) + (v.z + v.w);
  }
  if (blockIdx.x == 0 && threadIdx.x < n - n4 * 4) {
    const float v = x[n4 * 4 + threadIdx.x];
    acc += square ? v * v : v;
  }
  const float r = block_sum(acc, smem);
  if (threadIdx.x == 0) partials[blockIdx.x] = r;
}
// out[0] = (accumulate ? out[0] : 0) + scale * sum(partials)
__global__ void __launch_bounds__(RED_THREADS)
    reduce_final_kernel(const float* __restrict__ partials, int count, float* __restrict__ out,
                        float scale, int accumulate) {
  __shared__ float smem[RED_THREADS / 32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < count; i += RED_THREADS) acc += partials[i];
  const float r = block_sum(acc, smem);
  if (threadIdx.x == 0) out[0] = (accumulate ? out[0] : 0.f) + scale * r;
}

struct AdamParams {
  float lr, beta1, beta2, eps, weight_decay;
  float bias1, bias2;   // 1 - beta^step
  float grad_scale;     // applied to the raw gradient (e.g. 1 / accumulation steps)
  float max_norm;       // <= 0 disables clipping
};

// AdamW over a flat range.  grad_sumsq (device scalar, may be null) is the sum of squares of the
// UNSCALED gradients of the whole model; the clip factor is min(1, max_norm / (norm + 1e-6)).
// Writes the f32 master weight, its bf16 replica, the moments, and zeroes the gradient.
__global__ void __launch_bounds__(256)
    adamw_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ replica,
                 float* __restrict__ grad, float* __restrict__ m, float* __restrict__ v, long long n,
                 const float* __restrict__ grad_sumsq, const AdamParams p) {
  float gs = p.grad_scale;
  if (grad_sumsq != nullptr && p.max_norm > 0.f) {
    const float norm = sqrtf(grad_sumsq[0]) * p.grad_scale;
    gs *= fminf(1.0f, p.max_norm / (norm + 1e-6f));
  }
  const long long i4 = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  const long long base = i4 * 4;
  if (base >= n) return;
  if (base + 4 <= n) {
    float4 w = *reinterpret_cast<float4*>(master + base);
    float4 g = *reinterpret_cast<float4*>(grad + base);
    float4 mm = *reinterpret_cast<float4*>(m + base);
    float4 vv = *reinterpret_cast<float4*>(v + base);
    float* wp = &w.x; float* gp = &g.x; float* mp = &mm.x; float* vp = &vv.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = gp[j] * gs;
      mp[j] = p.beta1 * mp[j] + (1.f - p.beta1) * gj;
      vp[j] = p.beta2 * vp[j] + (1.f - p.beta2) * gj * gj;
      const float mh = mp[j] / p.bias1, vh = vp[j] / p.bias2;
      wp[j] = wp[j] - p.lr * (mh / (sqrtf(vh) + p.eps) + p.weight_decay * wp[j]);
    }
    *reinterpret_cast<float4*>(master + base) = w;
    *reinterpret_cast<float4*>(m + base) = mm;
    *reinterpret_cast<float4*>(v + base) = vv;
    *reinterpret_cast<float4*>(grad + base) = make_float4(0.f, 0.f, 0.f, 0.f);
    uint2 r;
    r.x = pack_bf16x2(w.x, w.y);
    r.y = pack_bf16x2(w.z, w.w);
    *reinterpret_cast<uint2*>(replica + base) = r;
  } else {
    for (long long i = base; i < n; ++i) {
      const float gj = grad[i] * gs;
      const float mj = p.beta1 * m[i] + (1.f - p.beta1) * gj;
      const float vj = p.beta2 * v[i] + (1.f - p.beta2) * gj * gj;
      const float wj = master[i] - p.lr * ((mj / p.bias1) / (sqrtf(vj / p.bias2) + p.eps) +
                                           p.weight_decay * master[i]);
      m[i] = mj; v[i] = vj; master[i] = wj; grad[i] = 0.f;
      replica[i] = __float2bfloat16_rn(wj);
    }
  }
}

}  // namespace lm

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int32_t xent_execute(const cdl_tensor* logits, const cdl_tensor* targets, const cdl_tensor* loss,
                     float grad_scale, cudaStream_t stream) {
  const char* op = "cross_entropy";
  if (!logits || !targets || !loss) return fail(CDL_ERR_INVALID, "%s: logits, targets, loss are required", op);
  if (logits->rank != 2 || logits->dtype != CDL_BF16 || logits->stride[1] != 1 ||
      logits->stride[0] % 8 != 0 || !aligned16(logits->ptr))
    return fail(CDL_ERR_INVALID, "%s: logits must be bf16 [tokens, vocab] with 16-byte aligned rows", op);
  const long long T = logits->shape[0], V = logits->shape[1];
  if (V % 8 != 0 || V <= 0 || V > INT32_MAX)
    return fail(CDL_ERR_UNSUPPORTED, "%s: vocab must be a positive multiple of 8", op);
  if (targets->rank != 1 || targets->dtype != CDL_I32 || targets->shape[0] != T || targets->stride[0] != 1)
    return fail(CDL_ERR_INVALID, "%s: targets must be packed i32 [tokens]", op);
  if (loss->rank != 1 || loss->dtype != CDL_F32 || loss->shape[0] != T || loss->stride[0] != 1)
    return fail(CDL_ERR_INVALID, "%s: loss must be packed f32 [tokens]", op);
  if (T == 0) return CDL_OK;
  if (T > INT32_MAX) return fail(CDL_ERR_UNSUPPORTED, "%s: too many tokens", op);
  ProfileScope ps(PROF_ELEMENTWISE, 4.0 * T * V, stream);
  lm::xent_fwd_bwd_kernel<<<static_cast<unsigned>(T), lm::XENT_THREADS, 0, stream>>>(
      static_cast<__nv_bfloat16*>(logits->ptr), logits->stride[0], static_cast<const int*>(targets->ptr),
      static_cast<float*>(loss->ptr), static_cast<int>(V), grad_scale);
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

int32_t embedding_bwd_execute(const cdl_tensor* tokens, const cdl_tensor* dx, const cdl_tensor* d_table,
                              cudaStream_t stream) {
  const char* op = "embedding_bwd";
  if (!tokens || !dx || !d_table) return fail(CDL_ERR_INVALID, "%s: tokens, dx, d_table are required", op);
  if (tokens->rank != 1 || tokens->dtype != CDL_I32 || tokens->stride[0] != 1)
    return fail(CDL_ERR_INVALID, "%s: tokens must be a packed i32 vector", op);
  const long long n = tokens->shape[0];
  if (d_table->rank != 2 || d_table->dtype != CDL_F32 || d_table->stride[1] != 1 ||
      d_table->stride[0] != d_table->shape[1] || d_table->shape[1] % 8 != 0 || !aligned16(d_table->ptr))
    return fail(CDL_ERR_INVALID, "%s: d_table must be packed f32 [vocab, hidden], hidden %% 8 == 0", op);
  const long long hidden = d_table->shape[1];
  if (dx->rank != 2 || dx->dtype != CDL_BF16 || dx->shape[0] != n || dx->shape[1] != hidden ||
      dx->stride[1] != 1 || dx->stride[0] != hidden || !aligned16(dx->ptr))
    return fail(CDL_ERR_INVALID, "%s: dx must be packed bf16 [tokens, hidden]", op);
  if (n == 0 || hidden == 0) return CDL_OK;
  const long long total = n * (hidden / 8);
  ProfileScope ps(PROF_ELEMENTWISE, 10.0 * n * hidden, stream);
  lm::embedding_bwd_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      static_cast<const int*>(tokens->ptr), static_cast<const __nv_bfloat16*>(dx->ptr),
      static_cast<float*>(d_table->ptr), n, static_cast<int>(hidden / 8),
      static_cast<int>(d_table->shape[0]));
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

int32_t reduce_execute(const float* x, long long n, float* out, float scale, int square, int accumulate,
                       float* scratch, size_t scratch_bytes, cudaStream_t stream) {
  const char* op = "reduce";
  if (!x || !out || n < 0) return fail(CDL_ERR_INVALID, "%s: x, out are required", op);
  if (!aligned16(x)) return fail(CDL_ERR_INVALID, "%s: x must be 16-byte aligned", op);
  if (!scratch || scratch_bytes < lm::RED_BLOCKS * sizeof(float))
    return fail(CDL_ERR_INVALID, "%s: scratch must hold %zu bytes", op, lm::RED_BLOCKS * sizeof(float));
  long long want = (n / 4 + lm::RED_THREADS - 1) / lm::RED_THREADS;
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > lm::RED_BLOCKS ? lm::RED_BLOCKS : want));
  ProfileScope ps(PROF_ELEMENTWISE, 4.0 * n, stream);
  lm::reduce_partial_kernel<<<blocks, lm::RED_THREADS, 0, stream>>>(x, n, scratch, square);
  CDL_CUDA(cudaGetLastError());
  lm::reduce_final_kernel<<<1, lm::RED_THREADS, 0, stream>>>(scratch, blocks, out, scale, accumulate);
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

}  // namespace cdl

extern "C" {

int32_t cdl_b200_cross_entropy(const cdl_tensor* logits, const cdl_tensor* targets,
                               const cdl_tensor* loss, float grad_scale, cdl_stream stream) {
  return cdl::xent_execute(logits, targets, loss, grad_scale, static_cast<cudaStream_t>(stream));
}

int32_t cdl_b200_embedding_bwd(const cdl_tensor* tokens, const cdl_tensor* dx,
                               const cdl_tensor* d_table, cdl_stream stream) {
  return cdl::embedding_bwd_execute(tokens, dx, d_table, static_cast<cudaStream_t>(stream));
}

int32_t cdl_b200_sum(const float* x, int64_t n, float* out, float scale, int32_t square,
                     int32_t accumulate, void* scratch, size_t scratch_bytes, cdl_stream stream) {
  return cdl::reduce_execute(x, n, out, scale, square, accumulate, static_cast<float*>(scratch),
                             scratch_bytes, static_cast<cudaStream_t>(stream));
}

int32_t cdl_b200_adamw(float* master, void* replica_bf16, float* grad, float* m, float* v, int64_t n,
                       const float* grad_sumsq, const cdl_adamw_params* hp, cdl_stream stream) {
  if (!master || !replica_bf16 || !grad || !m || !v || !hp)
    return cdl::fail(CDL_ERR_INVALID, "adamw: every buffer and the hyper-parameters are required");
  if (n < 0 || hp->step < 1) return cdl::fail(CDL_ERR_INVALID, "adamw: n >= 0 and step >= 1 are required");
  if ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(grad) |
       reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15 ||
      reinterpret_cast<uintptr_t>(replica_bf16) & 7)
    return cdl::fail(CDL_ERR_INVALID, "adamw: f32 buffers must be 16-byte aligned, the replica 8-byte");
  if (n == 0) return CDL_OK;
  cdl::lm::AdamParams p;
  p.lr = hp->lr; p.beta1 = hp->beta1; p.beta2 = hp->beta2; p.eps = hp->eps;
  p.weight_decay = hp->weight_decay;
  p.bias1 = 1.0f - powf(hp->beta1, static_cast<float>(hp->step));
  p.bias2 = 1.0f - powf(hp->beta2, static_cast<float>(hp->step));
  p.grad_scale = hp->grad_scale;
  p.max_norm = hp->max_grad_norm;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cdl::ProfileScope ps(cdl::PROF_ELEMENTWISE, 34.0 * n, st);
  const long long blocks = ((n + 3) / 4 + 255) / 256;
  cdl::lm::adamw_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(
      master, static_cast<__nv_bfloat16*>(replica_bf16), grad, m, v, n, grad_sumsq, p);
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

}  // extern "C"
