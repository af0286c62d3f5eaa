// Bandwidth-bound glue of the sky-1 block: rotary position embedding and the SwiGLU
// activation, forward and backward.  The reference's implementations of these lived in its
// legacy `cleandl::operators::{rope, swiglu_ffn}` module, which is not in the tree; only the call
// sites remain (crates/sky-1/src/training/model/decoder.rs:363-378, 487-496, 645-655), plus the
// SiLU formulas of its fused GEMM epilogues (crates/cleandl/rust-kernels/src/sky_matmul/
// tcgen05_bf16.rs:851-877).  All kernels use 128-bit accesses, one 8-element group per thread.
#include "host.h"
#include "ptx.cuh"

namespace cdl {
namespace elem {

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

// Rotate-half RoPE, in place, on the first `rot_heads` heads of x viewed [tokens, heads, D]:
//   x'[i]       = x[i] cos - x[i + D/2] sin * sign
//   x'[i + D/2] = x[i + D/2] cos + x[i] sin * sign        (sign = -1 gives the backward pass)
// cos_sin is f32 [seqlen, D] = cos[0..D/2) | sin[0..D/2) per position; position = token % seqlen.
__global__ void __launch_bounds__(256)
    rope_kernel(__nv_bfloat16* __restrict__ x, long long token_stride, long long head_stride,
                const float* __restrict__ cos_sin, long long tokens, int seqlen, int rot_heads,
                int half_dim, float sign, const int* __restrict__ cu_seqlens, int num_seqs) {
  grid_dep_wait();
  grid_dep_launch();
  const int groups = half_dim / 8;  // 8-element groups per half
  const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  const long long total = tokens * rot_heads * groups;
  if (idx >= total) return;
  const int g = static_cast<int>(idx % groups);
  const int head = static_cast<int>((idx / groups) % rot_heads);
  const long long token = idx / groups / rot_heads;
  int pos;
  if (cu_seqlens != nullptr) {
    // ragged batch: the position restarts at every sequence; `seqlen` is the table's row count
    if (token >= cu_seqlens[num_seqs]) return;  // padding rows after the last sequence
    int lo_i = 0, hi_i = num_seqs;              // largest b with cu_seqlens[b] <= token
    while (hi_i - lo_i > 1) {
      const int mid = (lo_i + hi_i) >> 1;
      if (cu_seqlens[mid] <= token) lo_i = mid;
      else hi_i = mid;
    }
    pos = min(static_cast<int>(token - cu_seqlens[lo_i]), seqlen - 1);
  } else {
    pos = static_cast<int>(token % seqlen);
  }
  __nv_bfloat16* p = x + token * token_stride + head * head_stride + g * 8;
  const uint4 lo_q = *reinterpret_cast<const uint4*>(p);
  const uint4 hi_q = *reinterpret_cast<const uint4*>(p + half_dim);
  float lo[8], hi[8], olo[8], ohi[8];
  unpack8(lo_q, lo);
  unpack8(hi_q, hi);
  const float* cs = cos_sin + static_cast<long long>(pos) * 2 * half_dim + g * 8;
  const float4 c0 = *reinterpret_cast<const float4*>(cs);
  const float4 c1 = *reinterpret_cast<const float4*>(cs + 4);
  const float4 s0 = *reinterpret_cast<const float4*>(cs + half_dim);
  const float4 s1 = *reinterpret_cast<const float4*>(cs + half_dim + 4);
  const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float sn = s[j] * sign;
    olo[j] = lo[j] * c[j] - hi[j] * sn;
    ohi[j] = hi[j] * c[j] + lo[j] * sn;
  }
  *reinterpret_cast<uint4*>(p) = pack8(olo);
  *reinterpret_cast<uint4*>(p + half_dim) = pack8(ohi);
}

__device__ __forceinline__ float sigmoidf_fast(float x) {
  return __frcp_rn(1.0f + __expf(-x));
}

// act = SiLU(gate) * up
__global__ void __launch_bounds__(256)
    swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                      __nv_bfloat16* __restrict__ act, long long n8) {
  const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (idx >= n8) return;
  float g[8], u[8], a[8];
  unpack8(ld_nc_v4(gate + idx * 8), g);
  unpack8(ld_nc_v4(up + idx * 8), u);
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = g[j] * sigmoidf_fast(g[j]) * u[j];
  *reinterpret_cast<uint4*>(act + idx * 8) = pack8(a);
}

// d_up = d_act * SiLU(gate);  d_gate = d_act * up * (s + gate * s * (1 - s)),  s = sigmoid(gate)
__global__ void __launch_bounds__(256)
    swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ d_act, const __nv_bfloat16* __restrict__ gate,
                      const __nv_bfloat16* __restrict__ up, __nv_bfloat16* __restrict__ d_gate,
                      __nv_bfloat16* __restrict__ d_up, long long n8) {
  const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (idx >= n8) return;
  float da[8], g[8], u[8], dg[8], du[8];
  unpack8(ld_nc_v4(d_act + idx * 8), da);
  unpack8(ld_nc_v4(gate + idx * 8), g);
  unpack8(ld_nc_v4(up + idx * 8), u);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float s = sigmoidf_fast(g[j]);
    du[j] = da[j] * g[j] * s;
    dg[j] = da[j] * u[j] * (s + g[j] * s * (1.0f - s));
  }
  *reinterpret_cast<uint4*>(d_gate + idx * 8) = pack8(dg);
  *reinterpret_cast<uint4*>(d_up + idx * 8) = pack8(du);
}

// out[t, :] = table[tokens[t], :]; one thread per 8 elements.
__global__ void __launch_bounds__(256)
    embedding_fwd_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ table,
                         __nv_bfloat16* __restrict__ out, long long n_tokens, int hidden8, int vocab) {
  const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (idx >= n_tokens * hidden8) return;
  const long long t = idx / hidden8;
  const int g = static_cast<int>(idx - t * hidden8);
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(table + static_cast<long long>(tok) * hidden8 * 8) + g);
  *reinterpret_cast<uint4*>(out + idx * 8) = v;
}

}  // namespace elem

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int32_t rope_ragged_execute(const cdl_tensor* x, const cdl_tensor* cos_sin, int32_t rot_heads,
                            int32_t seqlen, const cdl_tensor* cu_seqlens, int32_t backward,
                            cudaStream_t stream);

int32_t rope_execute(const cdl_tensor* x, const cdl_tensor* cos_sin, int32_t rot_heads,
                     int32_t seqlen, int32_t backward, cudaStream_t stream) {
  return rope_ragged_execute(x, cos_sin, rot_heads, seqlen, nullptr, backward, stream);
}

// cu_seqlens (nullable): i32 [num_seqs + 1]; with it, token t of sequence b has position
// t - cu_seqlens[b] and `seqlen` is only the number of table rows that may be used.
int32_t rope_ragged_execute(const cdl_tensor* x, const cdl_tensor* cos_sin, int32_t rot_heads,
                            int32_t seqlen, const cdl_tensor* cu_seqlens, int32_t backward,
                            cudaStream_t stream) {
  const char* op = "rope";
  if (cu_seqlens && (cu_seqlens->rank != 1 || cu_seqlens->dtype != CDL_I32 || cu_seqlens->shape[0] < 1 ||
                     cu_seqlens->stride[0] != 1))
    return fail(CDL_ERR_INVALID, "%s: cu_seqlens must be a contiguous i32 vector of batch + 1 entries", op);
  if (!x || !cos_sin) return fail(CDL_ERR_INVALID, "%s: x and cos_sin are required", op);
  if (x->rank != 3 || x->dtype != CDL_BF16)
    return fail(CDL_ERR_INVALID, "%s: x must be bf16 [tokens, heads, head_dim]", op);
  const long long tokens = x->shape[0], heads = x->shape[1], d = x->shape[2];
  if (d % 16 != 0 || x->stride[2] != 1 || x->stride[0] % 8 != 0 || x->stride[1] % 8 != 0 ||
      !aligned16(x->ptr))
    return fail(CDL_ERR_INVALID, "%s: head_dim must be a multiple of 16, contiguous, 16-byte aligned", op);
  if (rot_heads < 0 || rot_heads > heads)
    return fail(CDL_ERR_INVALID, "%s: rot_heads %d exceeds heads %lld", op, rot_heads, heads);
  if (seqlen <= 0 || cos_sin->rank != 2 || cos_sin->dtype != CDL_F32 || cos_sin->shape[0] < seqlen ||
      cos_sin->shape[1] != d || cos_sin->stride[1] != 1 || cos_sin->stride[0] != d ||
      !aligned16(cos_sin->ptr))
    return fail(CDL_ERR_INVALID, "%s: cos_sin must be packed f32 [>= seqlen, head_dim]", op);
  const long long total = tokens * rot_heads * (d / 16);
  if (total == 0) return CDL_OK;
  ProfileScope ps(PROF_ELEMENTWISE, static_cast<double>(total) * 64, stream);
  CDL_CUDA(launch_pdl(elem::rope_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, stream,
      static_cast<__nv_bfloat16*>(x->ptr), x->stride[0], x->stride[1],
      static_cast<const float*>(cos_sin->ptr), tokens, seqlen, rot_heads, static_cast<int>(d / 2),
      backward ? -1.0f : 1.0f, cu_seqlens ? static_cast<const int*>(cu_seqlens->ptr) : nullptr,
      cu_seqlens ? static_cast<int>(cu_seqlens->shape[0] - 1) : 0));
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

static int32_t check_flat(const char* op, const char* name, const cdl_tensor* t, long long n) {
  if (!t) return fail(CDL_ERR_INVALID, "%s: %s is required", op, name);
  long long cnt = 1;
  for (int i = 0; i < t->rank; ++i) cnt *= t->shape[i];
  long long expect = 1;
  bool packed = true;
  for (int i = t->rank - 1; i >= 0; --i) {
    if (t->shape[i] != 1 && t->stride[i] != expect) packed = false;
    expect *= t->shape[i];
  }
  if (cnt != n || t->dtype != CDL_BF16 || !packed || !aligned16(t->ptr))
    return fail(CDL_ERR_INVALID, "%s: %s must be a packed, 16-byte aligned bf16 tensor of %lld elements",
                op, name, n);
  return CDL_OK;
}

int32_t swiglu_fwd_execute(const cdl_tensor* gate, const cdl_tensor* up, const cdl_tensor* act,
                           cudaStream_t stream) {
  const char* op = "swiglu_fwd";
  if (!gate) return fail(CDL_ERR_INVALID, "%s: gate is required", op);
  long long n = 1;
  for (int i = 0; i < gate->rank; ++i) n *= gate->shape[i];
  CDL_CHECK(check_flat(op, "gate", gate, n));
  CDL_CHECK(check_flat(op, "up", up, n));
  CDL_CHECK(check_flat(op, "act", act, n));
  if (n % 8 != 0) return fail(CDL_ERR_INVALID, "%s: element count must be a multiple of 8", op);
  if (n == 0) return CDL_OK;
  ProfileScope ps(PROF_ELEMENTWISE, static_cast<double>(n) * 6, stream);
  elem::swiglu_fwd_kernel<<<static_cast<unsigned>((n / 8 + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gate->ptr), static_cast<const __nv_bfloat16*>(up->ptr),
      static_cast<__nv_bfloat16*>(act->ptr), n / 8);
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

int32_t swiglu_bwd_execute(const cdl_tensor* d_act, const cdl_tensor* gate, const cdl_tensor* up,
                           const cdl_tensor* d_gate, const cdl_tensor* d_up, cudaStream_t stream) {
  const char* op = "swiglu_bwd";
  if (!gate) return fail(CDL_ERR_INVALID, "%s: gate is required", op);
  long long n = 1;
  for (int i = 0; i < gate->rank; ++i) n *= gate->shape[i];
  CDL_CHECK(check_flat(op, "d_act", d_act, n));
  CDL_CHECK(check_flat(op, "gate", gate, n));
  CDL_CHECK(check_flat(op, "up", up, n));
  CDL_CHECK(check_flat(op, "d_gate", d_gate, n));
  CDL_CHECK(check_flat(op, "d_up", d_up, n));
  if (n % 8 != 0) return fail(CDL_ERR_INVALID, "%s: element count must be a multiple of 8", op);
  if (n == 0) return CDL_OK;
  ProfileScope ps(PROF_ELEMENTWISE, static_cast<double>(n) * 10, stream);
  elem::swiglu_bwd_kernel<<<static_cast<unsigned>((n / 8 + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(d_act->ptr), static_cast<const __nv_bfloat16*>(gate->ptr),
      static_cast<const __nv_bfloat16*>(up->ptr), static_cast<__nv_bfloat16*>(d_gate->ptr),
      static_cast<__nv_bfloat16*>(d_up->ptr), n / 8);
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

int32_t embedding_fwd_execute(const cdl_tensor* tokens, const cdl_tensor* table,
                              const cdl_tensor* out, cudaStream_t stream) {
  const char* op = "embedding_fwd";
  if (!tokens || !table || !out) return fail(CDL_ERR_INVALID, "%s: tokens, table, out are required", op);
  if (tokens->rank != 1 || tokens->dtype != CDL_I32 || tokens->stride[0] != 1)
    return fail(CDL_ERR_INVALID, "%s: tokens must be a packed i32 vector", op);
  if (table->rank != 2 || table->dtype != CDL_BF16 || table->stride[1] != 1 ||
      table->stride[0] != table->shape[1] || table->shape[1] % 8 != 0 || !aligned16(table->ptr))
    return fail(CDL_ERR_INVALID, "%s: table must be packed bf16 [vocab, hidden], hidden %% 8 == 0", op);
  const long long n = tokens->shape[0], hidden = table->shape[1];
  if (out->rank != 2 || out->dtype != CDL_BF16 || out->shape[0] != n || out->shape[1] != hidden ||
      out->stride[1] != 1 || out->stride[0] != hidden || !aligned16(out->ptr))
    return fail(CDL_ERR_INVALID, "%s: out must be packed bf16 [tokens, hidden]", op);
  if (n == 0 || hidden == 0) return CDL_OK;
  if (table->shape[0] <= 0) return fail(CDL_ERR_INVALID, "%s: empty vocabulary", op);
  const long long total = n * (hidden / 8);
  ProfileScope ps(PROF_ELEMENTWISE, static_cast<double>(n) * hidden * 4, stream);
  elem::embedding_fwd_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      static_cast<const int*>(tokens->ptr), static_cast<const __nv_bfloat16*>(table->ptr),
      static_cast<__nv_bfloat16*>(out->ptr), n, static_cast<int>(hidden / 8),
      static_cast<int>(table->shape[0]));
  CDL_CUDA(cudaGetLastError());
  return CDL_OK;
}

}  // namespace cdl

extern "C" {

int32_t cdl_b200_embedding_fwd(const cdl_tensor* tokens, const cdl_tensor* table,
                               const cdl_tensor* out, cdl_stream stream) {
  return cdl::embedding_fwd_execute(tokens, table, out, static_cast<cudaStream_t>(stream));
}

int32_t cdl_b200_rope(const cdl_tensor* x, const cdl_tensor* cos_sin, int32_t rot_heads,
                      int32_t seqlen, int32_t backward, cdl_stream stream) {
  return cdl::rope_execute(x, cos_sin, rot_heads, seqlen, backward, static_cast<cudaStream_t>(stream));
}
int32_t cdl_b200_rope_ragged(const cdl_tensor* x, const cdl_tensor* cos_sin, int32_t rot_heads,
                             const cdl_tensor* cu_seqlens, int32_t backward, cdl_stream stream) {
  if (!cu_seqlens || !cos_sin || cos_sin->rank != 2)
    return cdl::fail(CDL_ERR_INVALID, "rope: cu_seqlens and a [positions, head_dim] table are required");
  return cdl::rope_ragged_execute(x, cos_sin, rot_heads, static_cast<int32_t>(cos_sin->shape[0]),
                                  cu_seqlens, backward, static_cast<cudaStream_t>(stream));
}
int32_t cdl_b200_swiglu_fwd(const cdl_tensor* gate, const cdl_tensor* up, const cdl_tensor* act,
                            cdl_stream stream) {
  return cdl::swiglu_fwd_execute(gate, up, act, static_cast<cudaStream_t>(stream));
}
int32_t cdl_b200_swiglu_bwd(const cdl_tensor* d_act, const cdl_tensor* gate, const cdl_tensor* up,
                            const cdl_tensor* d_gate, const cdl_tensor* d_up, cdl_stream stream) {
  return cdl::swiglu_bwd_execute(d_act, gate, up, d_gate, d_up, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
