// Internal C++ entry points of the operators (one per exec-graph node of the reference); the
// extern "C" functions and the sky-1 block are thin layers over these.
#pragma once
#include <cuda_bf16.h>

#include "host.h"

namespace cdl {

int32_t matmul_execute(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* c,
                       const cdl_tensor* d, float alpha, float beta, cudaStream_t stream,
                       const cdl_matmul_options* opts = nullptr);
// gemm_general.cu: any strides, bf16 or f32 inputs, CUDA cores (operands already validated).
int32_t matmul_general_execute(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* c,
                               const cdl_tensor* d, float alpha, float beta, cudaStream_t stream);
// Arguments of the RoPE epilogue (epi_mode 3): rotate-half RoPE on the heads (128 columns each)
// below rot_cols of the product; position = row % seqlen, or the row's offset inside its sequence
// of a ragged batch (cu_seqlens: num_seqs + 1 device entries).
struct RopeEpilogue {
  const float* table;  // f32 [positions, 128] = cos | sin
  int seqlen;          // dense: sequence length; ragged: rows of the table
  int rot_cols;
  const int* cu_seqlens;
  int num_seqs;
};
// epi_mode 1: d = product, out2 = SiLU(product) * aux0.  epi_mode 2: d = SiLU(aux0) * product,
// out2 = product * aux1 * dSiLU(aux0).  epi_mode 3: d = RoPE(product), see RopeEpilogue.
int32_t matmul_execute_epi(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* c,
                           const cdl_tensor* d, float alpha, float beta, int epi_mode,
                           const cdl_tensor* aux0, const cdl_tensor* aux1, const cdl_tensor* out2,
                           cudaStream_t stream, const cdl_matmul_options* opts = nullptr,
                           const RopeEpilogue* rope = nullptr);
// norm_general.cu: any float types, strides and column counts (layer = 0 RmsNorm, 1 LayerNorm).
int32_t norm_general_execute(int layer, const cdl_tensor* x, const cdl_tensor* scale,
                             const cdl_tensor* bias, float eps, const cdl_tensor* y,
                             const cdl_tensor* mean, const cdl_tensor* r_inv, cudaStream_t stream);
int32_t rmsnorm_fwd_execute(const cdl_tensor* x, const cdl_tensor* scale, const cdl_tensor* bias,
                            float eps, const cdl_tensor* y, const cdl_tensor* r_inv,
                            cudaStream_t stream, const cdl_norm_options* opts = nullptr);
int32_t layernorm_fwd_execute(const cdl_tensor* x, const cdl_tensor* scale, const cdl_tensor* bias,
                              float eps, const cdl_tensor* y, const cdl_tensor* mean,
                              const cdl_tensor* r_inv, cudaStream_t stream);
size_t rmsnorm_bwd_scratch_bytes(long long rows, long long cols);
int32_t rmsnorm_bwd_execute(const cdl_tensor* x, const cdl_tensor* dy, const cdl_tensor* res,
                            const cdl_tensor* scale, const cdl_tensor* r_inv, const cdl_tensor* dx,
                            const cdl_tensor* dscale, void* scratch, size_t scratch_bytes,
                            cudaStream_t stream, const cdl_norm_options* opts = nullptr);
int32_t attn_fwd_execute(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                         const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* lse,
                         cudaStream_t stream);
// attn_fwd_persistent.cu: the persistent forward for validated operands ([B, S, heads, 128] views).
int32_t attn_fwd_persistent_launch(const cdl_tensor* q, const cdl_tensor* k, const cdl_tensor* v,
                             long long B, long long H, long long Hkv, long long Sq, long long Sk,
                             bool causal, float scale_log2, __nv_bfloat16* o, long long o_sb,
                             long long o_ss, long long o_sh, float* lse, long long lse_sb,
                             long long lse_sh, long long lse_ss, const int* cu_q, const int* cu_k,
                             bool any_keys, cudaStream_t stream);
size_t attn_bwd_scratch_bytes(long long B, long long Sq, long long H);
int32_t attn_bwd_execute(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                         const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* d_o,
                         const cdl_tensor* lse, const cdl_tensor* dq, const cdl_tensor* dk,
                         const cdl_tensor* dv, void* scratch, size_t scratch_bytes,
                         cudaStream_t stream, const cdl_tensor* rope_table = nullptr);
int32_t attn_fwd_packed_execute(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                                const cdl_tensor* v, const cdl_tensor* cu_q, const cdl_tensor* cu_k,
                                long long max_q, long long max_k, const cdl_tensor* o,
                                const cdl_tensor* lse, cudaStream_t stream);
size_t attn_bwd_packed_scratch_bytes(long long batch, long long max_seqlen_q, long long H);
int32_t attn_bwd_packed_execute(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                                const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* d_o,
                                const cdl_tensor* lse, const cdl_tensor* cu_q, const cdl_tensor* cu_k,
                                long long max_q, long long max_k, const cdl_tensor* dq,
                                const cdl_tensor* dk, const cdl_tensor* dv, void* scratch,
                                size_t scratch_bytes, cudaStream_t stream,
                                const cdl_tensor* rope_table = nullptr);
int32_t rope_execute(const cdl_tensor* x, const cdl_tensor* cos_sin, int32_t rot_heads,
                     int32_t seqlen, int32_t backward, cudaStream_t stream);
int32_t rope_ragged_execute(const cdl_tensor* x, const cdl_tensor* cos_sin, int32_t rot_heads,
                            int32_t seqlen, const cdl_tensor* cu_seqlens, int32_t backward,
                            cudaStream_t stream);
int32_t swiglu_fwd_execute(const cdl_tensor* gate, const cdl_tensor* up, const cdl_tensor* act,
                           cudaStream_t stream);
int32_t swiglu_bwd_execute(const cdl_tensor* d_act, const cdl_tensor* gate, const cdl_tensor* up,
                           const cdl_tensor* d_gate, const cdl_tensor* d_up, cudaStream_t stream);

// Block-scaled (MXFP8) tensors.
int32_t mx_layout(int32_t format, int32_t dim, long long rows, long long cols, size_t* values_bytes,
                  size_t* scale_bytes);
int32_t mx_check(const char* op, const char* name, const cdl_mx_tensor* t, int32_t dim, long long rows,
                 long long cols);
int32_t mx_quantize_execute(const cdl_tensor* x, const cdl_mx_tensor* y_row,
                            const cdl_mx_tensor* y_col, cudaStream_t stream);
int32_t mx_dequantize_execute(const cdl_mx_tensor* x, const cdl_tensor* y, cudaStream_t stream);
int32_t rmsnorm_fwd_mx_execute(const cdl_tensor* x, const cdl_tensor* scale, const cdl_tensor* bias,
                               float eps, const cdl_mx_tensor* y_row, const cdl_mx_tensor* y_col,
                               const cdl_tensor* r_inv, cudaStream_t stream);
int32_t matmul_mx_execute(const cdl_mx_tensor* a, const cdl_mx_tensor* b, const cdl_tensor* c,
                          const cdl_tensor* d, float alpha, float beta, cudaStream_t stream,
                          const cdl_matmul_options* opts = nullptr);
int32_t matmul_mx_out_execute(const cdl_mx_tensor* a, const cdl_mx_tensor* b, const cdl_mx_tensor* d,
                              float alpha, cudaStream_t stream);

// Packed row-major views.
inline cdl_tensor view2(const void* p, int32_t dt, long long r, long long c) {
  cdl_tensor t{};
  t.ptr = const_cast<void*>(p);
  t.dtype = dt;
  t.rank = 2;
  t.shape[0] = r; t.shape[1] = c;
  t.stride[0] = c; t.stride[1] = 1;
  return t;
}
inline cdl_tensor view1(const void* p, int32_t dt, long long n) {
  cdl_tensor t{};
  t.ptr = const_cast<void*>(p);
  t.dtype = dt;
  t.rank = 1;
  t.shape[0] = n;
  t.stride[0] = 1;
  return t;
}
inline cdl_tensor transposed(const cdl_tensor& t) {
  cdl_tensor o = t;
  o.shape[0] = t.shape[1]; o.shape[1] = t.shape[0];
  o.stride[0] = t.stride[1]; o.stride[1] = t.stride[0];
  return o;
}

}  // namespace cdl
