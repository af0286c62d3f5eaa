/* cleandl_b200 — C ABI of the B200 (sm_100a) kernels behind clean-lm's exec-graph operators.
 *
 * Each entry point is what an `Executor::execute` of crates/cleandl would call for that
 * operator (crates/cleandl/src/execgraph/op.rs:130-142).  The conventions follow that trait:
 *   - nothing here allocates or frees device memory, and nothing synchronises the device or the
 *     stream (the two `*_status` helpers are the only exception and say so);
 *   - all work is enqueued on the caller's stream;
 *   - outputs and scratch have undefined contents on entry and are fully written;
 *   - every function returns 0 on success and a negative cdl_status otherwise, with a message
 *     available from cdl_b200_last_error() (thread-local); none throws or aborts;
 *   - empty shapes are a silent success (ops/matmul.rs:1095-1097, ops/norm/specialized.rs:133-135);
 *   - the library is re-entrant: execute may be called from any thread for any stream.
 * Only sm_100 devices are accepted; there is no CPU path and no other GPU architecture.
 */
#ifndef CLEANDL_B200_H
#define CLEANDL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  CDL_OK = 0,
  CDL_ERR_INVALID = -1,     /* operand validation failed (shape, type, layout, alignment) */
  CDL_ERR_UNSUPPORTED = -2, /* valid for the reference operator, not implemented here */
  CDL_ERR_CUDA = -3,        /* a CUDA runtime / driver call failed */
  CDL_ERR_DEVICE = -4       /* a kernel recorded an error (bounded wait ran out) */
} cdl_status;

typedef enum { CDL_BF16 = 0, CDL_F32 = 1, CDL_I32 = 2 } cdl_dtype;

/* A strided view of device memory.  Strides are in ELEMENTS, like TensorView's layout
 * (crates/cleandl/src/tensor.rs:20-856).  rank <= 4. */
typedef struct {
  void* ptr;
  int32_t dtype; /* cdl_dtype */
  int32_t rank;
  int64_t shape[4];
  int64_t stride[4];
} cdl_tensor;

/* CUDA stream handle (cudaStream_t / CUstream) passed as an opaque pointer. */
typedef void* cdl_stream;

/* ---- library state ------------------------------------------------------------------- */

/* Message of the last failing call on this thread ("" if none). */
const char* cdl_b200_last_error(void);

/* 0 if `device` has compute capability 10.x, CDL_ERR_UNSUPPORTED otherwise.  Mirrors the exact
 * architecture gate of kernel-build-util (crates/kernel-build-util/src/lib.rs:96-107). */
int32_t cdl_b200_device_ok(int32_t device);

/* Reads and clears the current device's kernel status word: 0 = no kernel gave up on a wait.
 * SYNCHRONISES the device.  Test / debugging aid, not part of the hot path. */
int32_t cdl_b200_device_status(int32_t* status_out);

/* Opt-in per-launch timing, the counterpart of the CUDA-event timing inside the reference's tuner
 * (crates/cleandl/src/execgraph/tune.rs:219-255).  After _start, every kernel launch of the
 * operators below is bracketed by two CUDA events on its stream (events are created inside _start,
 * never on the hot path).  _stop SYNCHRONISES the device and returns one record per launch in
 * launch order: kind 1 = GEMM, 2 / 3 = RMSNorm fwd / bwd, 4 / 5 = attention fwd / bwd,
 * 6 = elementwise; work = algorithmic FLOP (kinds 1, 4, 5) or bytes (others). */
typedef struct {
  int32_t kind;
  float ms;
  double work;
} cdl_profile_record;
int32_t cdl_b200_profile_start(int32_t max_records);
int32_t cdl_b200_profile_stop(cdl_profile_record* out, int32_t capacity, int32_t* count);

/* ---- Per-call kernel choices -------------------------------------------------------------
 * The reference's executors hand the engine's tuner a list of candidate implementations with the
 * heuristic default first (crates/cleandl/src/execgraph/op.rs:301-318; the matmul's list is built
 * in crates/cleandl/src/execgraph/ops/matmul.rs:667-729), and the tuner times each one per graph
 * node.  The `*_opt` entry points below take that choice as an argument (NULL = the library's own
 * heuristic, i.e. what the plain entry points do), and the `*_candidates` calls enumerate the
 * valid choices for a problem, default first.  Nothing in the library reads an environment
 * variable. */
typedef enum {
  CDL_GEMM_AUTO = 0,    /* heuristic: CTA pairs whenever M > 128 */
  CDL_GEMM_ONE_CTA = 1, /* 128 x 256 tiles, one CTA per tile */
  CDL_GEMM_CTA_PAIR = 2 /* 256 x 256 tiles, tcgen05.mma.cta_group::2 over a cluster of two CTAs */
} cdl_gemm_variant;
typedef struct {
  int32_t variant;       /* cdl_gemm_variant */
  int32_t deterministic; /* != 0: fixed f32 summation order.  The accumulate-in-place form
                          * (D = C in f32, beta = 1: the weight-gradient GEMM) otherwise cuts K into
                          * slices that add into D with red.global.add, so its low-order bits can
                          * differ from run to run. */
} cdl_matmul_options;
typedef enum {
  CDL_NORM_AUTO = 0,         /* heuristic (measured per form, see cdl_b200_rmsnorm_bwd) */
  CDL_NORM_WARP_PER_ROW = 1, /* rows streamed straight from global memory into registers */
  CDL_NORM_PIPELINED = 2     /* persistent CTAs, rows staged through a shared-memory ring of bulk
                              * copies; cols <= 2048 and rows >= 2 per SM, else the other form */
} cdl_norm_variant;
typedef struct {
  int32_t variant; /* cdl_norm_variant */
} cdl_norm_options;

/* ---- Matmul: D = alpha * A . B + beta * C ----------------------------------------------
 * Replaces MatmulExecutor::execute (crates/cleandl/src/execgraph/ops/matmul.rs:1092-1183),
 * which forwards to cuBLASLt.  A is [M,K] or [batch,M,K]; B is [K,N] or [batch,K,N]; C
 * (nullable; needs beta != 0 to matter) and D are [M,N] / [batch,M,N].  A and B are views with
 * one contiguous dimension (a transposed view is free, matmul.rs:128-157), both bf16 or both
 * f32; D and C are bf16 or f32; accumulation is f32.  forward = (A row-major, B row-major),
 * dgrad = (A row-major, B transposed view), wgrad = (A transposed view, B row-major, D = C f32,
 * beta 1).  bf16 operands whose base address and non-unit strides are 16-byte aligned take the
 * tensor-core kernels; other layouts (tests/matmul.rs:604-630) and f32 inputs
 * (tests/matmul.rs:243-265; full f32 products, where cuBLASLt uses TF32) take a general
 * CUDA-core kernel that is correct but slow.  K == 0 is an error ("K is zero", matmul.rs tests
 * :825-843).  D may alias C. */
int32_t cdl_b200_matmul(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* c,
                        const cdl_tensor* d, float alpha, float beta, void* scratch,
                        size_t scratch_bytes, cdl_stream stream);
/* The same product with the kernel choice made by the caller (NULL options = cdl_b200_matmul).
 * By default the weight-gradient form (D = C in f32, beta = 1, M > 128) is NOT bit-reproducible
 * from run to run (K slices meet in D through f32 atomics; every result is within the f32
 * summation bound of every other); options->deterministic != 0 gives a fixed order at the cost
 * of idle SMs on small outputs.  All other forms are always bit-reproducible. */
int32_t cdl_b200_matmul_opt(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* c,
                            const cdl_tensor* d, float alpha, float beta,
                            const cdl_matmul_options* options, void* scratch, size_t scratch_bytes,
                            cdl_stream stream);
/* Writes the valid choices for this problem to out[0 .. *count), the heuristic default first (the
 * order Executor candidates have, op.rs:301-318); at most `capacity` entries, *count = how many
 * exist.  Problems that take the general CUDA-core kernel have the single candidate AUTO. */
int32_t cdl_b200_matmul_candidates(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* d,
                                   cdl_matmul_options* out, int32_t capacity, int32_t* count);
/* GEMM with the SwiGLU activation fused into its epilogue, the counterparts of the reference's
 * sky_matmul_swiglu_gate_train_fwd and sky_matmul_swiglu_down_train_dgrad kernels
 * (crates/cleandl/rust-kernels/src/sky_matmul/tcgen05_bf16.rs:879-942, 944-1031, entry points
 * :1201-1223).  All [M, N] operands are bf16 with 16-byte aligned rows, N % 8 == 0.
 *   gate:  G = A . B;  gate_out = G;  act_out = SiLU(G) * up
 *   dgrad: R = A . B;  d_up_out = SiLU(gate) * R;  d_gate_out = R * up * dSiLU(gate)
 * with dSiLU(g) = s + g s (1 - s), s = sigmoid(g). */
int32_t cdl_b200_matmul_swiglu_gate(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* up,
                                    const cdl_tensor* gate_out, const cdl_tensor* act_out,
                                    cdl_stream stream);
int32_t cdl_b200_matmul_swiglu_dgrad(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* gate,
                                     const cdl_tensor* up, const cdl_tensor* d_up_out,
                                     const cdl_tensor* d_gate_out, cdl_stream stream);
/* D = RoPE(A . B): the product (bf16 [M, N], N % 128 == 0, 16-byte aligned rows) with rotate-half
 * RoPE applied in the epilogue to heads [0, rot_heads) of 128 columns of every row -- the fused
 * QKV projection of the sky-1 block followed by its RoPE on the q and k heads
 * (crates/sky-1/src/training/model/decoder.rs:350-378) in one kernel, without the extra pass over
 * the qkv tensor.  cos_sin, seqlen, cu_seqlens (nullable: ragged batch) as for cdl_b200_rope /
 * cdl_b200_rope_ragged; the row index is the token index. */
int32_t cdl_b200_matmul_rope(const cdl_tensor* a, const cdl_tensor* b, const cdl_tensor* cos_sin,
                             int32_t rot_heads, int32_t seqlen, const cdl_tensor* cu_seqlens,
                             const cdl_tensor* d, cdl_stream stream);
/* Scratch the call above needs for these operands (Executor::scratch_bytes, op.rs:132-135). */
int32_t cdl_b200_matmul_scratch_bytes(const cdl_tensor* a, const cdl_tensor* b,
                                      const cdl_tensor* d, size_t* bytes_out);

/* ---- RMSNorm forward -------------------------------------------------------------------
 * Replaces SpecializedExecutor::execute (crates/cleandl/src/execgraph/ops/norm/specialized.rs:
 * 116-200) and the kernel it launches (crates/cleandl-specialized-kernels/src/kernels/norm/
 * forward.rs:509-785):  r_i = rsqrt(mean_j x_ij^2 + eps);  y_ij = bf16(x_ij * r_i * scale_j + bias_j).
 * x, y: [rows, cols]; scale, bias: [cols], nullable; r_inv: f32 [rows], nullable (the op's
 * save_stats).  bf16 operands with packed, 16-byte aligned rows, cols % 8 == 0 and cols <= 8192
 * (the domain of the reference's specialized kernel, specialized.rs:24-73) take the vectorised
 * kernels; everything else the reference's fallback accepts (f32 or bf16 x, y, scale and bias in
 * any combination, any column count and strides; crates/cleandl/tests/norm.rs:414-470) takes a
 * general kernel: y = (f32 or bf16)(x * r_i * scale_j + bias_j) computed in f32. */
int32_t cdl_b200_rmsnorm_fwd(const cdl_tensor* x, const cdl_tensor* scale, const cdl_tensor* bias,
                             float eps, const cdl_tensor* y, const cdl_tensor* r_inv,
                             cdl_stream stream);
/* The same with the kernel form chosen by the caller (NULL options = the call above). */
int32_t cdl_b200_rmsnorm_fwd_opt(const cdl_tensor* x, const cdl_tensor* scale,
                                 const cdl_tensor* bias, float eps, const cdl_tensor* y,
                                 const cdl_tensor* r_inv, const cdl_norm_options* options,
                                 cdl_stream stream);

/* LayerNorm forward: NormFwd with NormType::LayerNorm (ops/norm/mod.rs:23-30; tests
 * crates/cleandl/tests/norm.rs:97-130): y = bf16((x - mean) * r_inv * scale + bias) with
 * mean = mean_j x, r_inv = rsqrt(mean_j (x - mean)^2 + eps).  Operands as for the RMSNorm forward;
 * mean and r_inv (f32 [rows], nullable) are the saved statistics. */
int32_t cdl_b200_layernorm_fwd(const cdl_tensor* x, const cdl_tensor* scale, const cdl_tensor* bias,
                               float eps, const cdl_tensor* y, const cdl_tensor* mean,
                               const cdl_tensor* r_inv, cdl_stream stream);

/* ---- RMSNorm backward ------------------------------------------------------------------
 * The reference tree holds only the call sites (crates/sky-1/src/training/model/decoder.rs:
 * 599-607, 684-692): dx = rmsnorm_backward(x, dy, residual_dy, scale, r_inv; dscale +=).
 *   g_ij = dy_ij * scale_j;  c_i = mean_j(g_ij * x_ij);
 *   dx_ij = r_i * g_ij - r_i^3 * x_ij * c_i (+ residual_dy_ij);   dscale_j += sum_i dy_ij x_ij r_i.
 * x, dy, residual_dy (nullable), dx: bf16 [rows, cols]; scale bf16 [cols]; r_inv f32 [rows];
 * dscale f32 [cols], ACCUMULATED in place.  Scratch: see *_scratch_bytes. */
int32_t cdl_b200_rmsnorm_bwd(const cdl_tensor* x, const cdl_tensor* dy,
                             const cdl_tensor* residual_dy, const cdl_tensor* scale,
                             const cdl_tensor* r_inv, const cdl_tensor* dx,
                             const cdl_tensor* dscale, void* scratch, size_t scratch_bytes,
                             cdl_stream stream);
int32_t cdl_b200_rmsnorm_bwd_scratch_bytes(int64_t rows, int64_t cols, size_t* bytes_out);
/* The same with the kernel form chosen by the caller (NULL options = the heuristic: pipelined when
 * a residual gradient is fused in, warp-per-row otherwise).  Both forms sum dscale in a fixed
 * order and are bit-reproducible. */
int32_t cdl_b200_rmsnorm_bwd_opt(const cdl_tensor* x, const cdl_tensor* dy,
                                 const cdl_tensor* residual_dy, const cdl_tensor* scale,
                                 const cdl_tensor* r_inv, const cdl_tensor* dx,
                                 const cdl_tensor* dscale, const cdl_norm_options* options,
                                 void* scratch, size_t scratch_bytes, cdl_stream stream);

/* RMSNorm backward for callers that cannot supply scratch.  (No counterpart in the reference: its
 * engine always hands an executor a scratch slice.)  Some hosts of this library may not allocate
 * device memory at the point where they need the backward — code running inside a memory-pool
 * callback, a real-time loop with a fixed memory budget, a plugin whose host owns every
 * allocation — and have no scratch slice to lend either.  This variant takes the same operands as
 * cdl_b200_rmsnorm_bwd minus the scratch and uses an 8 MiB array that lives inside the library's
 * device image instead (every GPU that loads the library holds those 8 MiB until exit).  Limits
 * and rules:
 *   - cols <= 2048 (what the built-in array can hold); larger problems return
 *     CDL_ERR_UNSUPPORTED and should use cdl_b200_rmsnorm_bwd;
 *   - it calls no cudaMalloc / cudaFree or any other allocating routine;
 *   - the first call on each device looks up the array's device address (once, under a lock), and
 *     the first call per device and per column class (<= 256, 512, 1024, 2048 columns) also sets
 *     the kernel's shared-memory attribute; make those first calls before starting any stream
 *     capture;
 *   - all calls on a device share the one array: calls that may overlap on the GPU (different
 *     streams) race on it and must be serialised by the caller.  Nothing needs clearing between
 *     calls, each call overwrites what it later reads. */
int32_t cdl_b200_rmsnorm_bwd_static(const cdl_tensor* x, const cdl_tensor* dy,
                                    const cdl_tensor* residual_dy, const cdl_tensor* scale,
                                    const cdl_tensor* r_inv, const cdl_tensor* dx,
                                    const cdl_tensor* dscale, cdl_stream stream);

/* ---- Block-scaled (MX) tensors ------------------------------------------------------------
 * The reference's MxTensor (crates/cleandl/src/mx_tensor.rs:11-30, layout MxLayout::new
 * :339-372): a 2-D tensor quantised in blocks of 32 elements that share one UE8M0 scale; values
 * are FP8 E4M3 (MXFP8).  dim says along which logical dimension the blocks run:
 *   rowwise  values = packed bytes [rows, cols], blocks along a row    (cols % 32 == 0)
 *   colwise  values = packed bytes [cols, rows] (the transpose), blocks down a column (rows % 32 == 0)
 * scale_factors is the 128 x 4 tiled, partition-swizzled byte layout block-scaled tensor-core
 * instructions read: with outer = the non-block dimension and B = blocks per outer index, the
 * scale of block (o, b) is byte ((o / 128) * ceil(B / 4) + b / 4) * 512 + (o % 32) * 16 +
 * ((o % 128) / 32) * 4 + b % 4 of a buffer of round_up(outer, 128) * round_up(B, 4) bytes
 * (crates/cleandl/tests/common/mod.rs:124-129).  values must be 32-byte and scale_factors 16-byte
 * aligned.
 * NVFP4 (MxFormat::Nvfp4, without a global scale factor): blocks of 16 FP4 E2M1 elements, two per
 * byte along the block dimension (the even element in the low nibble), with one E4M3 scale;
 * same scale layout with B = blocks of 16.  Implemented: rowwise quantisation / RMSNorm output,
 * dequantisation, matmul operands. */
typedef enum { CDL_MXFP8 = 0, CDL_NVFP4 = 1 } cdl_mx_format;
typedef enum { CDL_MX_ROWWISE = 0, CDL_MX_COLWISE = 1 } cdl_mx_dim;
typedef struct {
  void* values;
  void* scale_factors;
  int32_t format; /* cdl_mx_format */
  int32_t dim;    /* cdl_mx_dim */
  int64_t rows, cols; /* logical shape */
} cdl_mx_tensor;

/* Bytes of the two buffers of a block-scaled tensor (MxLayout::new, mx_tensor.rs:339-372). */
int32_t cdl_b200_mx_layout(int32_t format, int32_t dim, int64_t rows, int64_t cols,
                           size_t* values_bytes, size_t* scale_bytes);

/* Quantises bf16 x [rows, cols] (packed rows, 16-byte aligned) into a rowwise and / or a colwise
 * block-scaled tensor (either may be NULL, not both): per block, scale = amax / 448 rounded up
 * to a power of two, element = x / scale rounded to nearest E4M3, saturating
 * (crates/cleandl-specialized-kernels/src/utils/block_scale.rs:24-55; the host quantiser of
 * crates/cleandl/tests/matmul.rs:885-952 gives the same bits).  Scale bytes of the padding are
 * not written.  NVFP4 (y_rowwise only): scale = amax / 6 rounded to nearest E4M3, element =
 * x * (1 / scale), reciprocal and product correctly rounded in f32, rounded to nearest E2M1, ties
 * to even, saturating; zeros when the scale rounds to zero (block_scale.rs:28-31, 55-66). */
int32_t cdl_b200_mx_quantize(const cdl_tensor* x, const cdl_mx_tensor* y_rowwise,
                             const cdl_mx_tensor* y_colwise, cdl_stream stream);

/* y (bf16 or f32 [rows, cols], packed rows) = values * scale.  A test and debugging aid. */
int32_t cdl_b200_mx_dequantize(const cdl_mx_tensor* x, const cdl_tensor* y, cdl_stream stream);

/* RMSNorm forward with block-scaled outputs: NormFwd with NormOutput::Mxfp8Rowwise (y_colwise
 * NULL) or ::Mxfp8RowwiseAndColwise (crates/cleandl/src/execgraph/ops/norm/mod.rs:33-62; kernel
 * crates/cleandl-specialized-kernels/src/kernels/norm/forward.rs:509-785).  Operands as for
 * cdl_b200_rmsnorm_fwd; the result is rounded to bf16 and then quantised as by
 * cdl_b200_mx_quantize.  The colwise output needs rows % 32 == 0 (norm/mod.rs validation).
 * An NVFP4 y_rowwise (and no y_colwise) gives NormOutput::Nvfp4Rowwise. */
int32_t cdl_b200_rmsnorm_fwd_mx(const cdl_tensor* x, const cdl_tensor* scale, const cdl_tensor* bias,
                                float eps, const cdl_mx_tensor* y_rowwise,
                                const cdl_mx_tensor* y_colwise, const cdl_tensor* r_inv,
                                cdl_stream stream);

/* D = alpha * A . B + beta * C with block-scaled operands: Matmul with InputKind::Mx(Mxfp8)
 * (crates/cleandl/src/execgraph/ops/matmul.rs:808-838, forwarded to cuBLASLt block scaling by the
 * reference; tests crates/cleandl/tests/matmul.rs:1041-1060).  A is rowwise [M, K], B is colwise
 * [K, N] (both K-contiguous), D and C (nullable; needs beta != 0 to matter; may be D itself) are
 * bf16 or f32 [M, N] with contiguous rows; accumulation is f32.
 * K % 32 == 0.  Both operands NVFP4 (InputKind::Mx(Nvfp4), tests :1063-1080) works the same way
 * with K % 64 == 0; mixed formats are rejected like in the reference (:569-571). */
int32_t cdl_b200_matmul_mx(const cdl_mx_tensor* a, const cdl_mx_tensor* b, const cdl_tensor* c,
                           const cdl_tensor* d, float alpha, float beta, cdl_stream stream);
/* The same with the kernel variant chosen by the caller (NULL options = the call above; the
 * block-scaled kernels are always bit-reproducible, `deterministic` is ignored). */
int32_t cdl_b200_matmul_mx_opt(const cdl_mx_tensor* a, const cdl_mx_tensor* b, const cdl_tensor* c,
                               const cdl_tensor* d, float alpha, float beta,
                               const cdl_matmul_options* options, cdl_stream stream);

/* The same product with a block-scaled output: MatmulOutput::BlockScaled { Mxfp8, dim }
 * (crates/cleandl/src/execgraph/ops/matmul.rs:826-834; test crates/cleandl/tests/matmul.rs:
 * 1083-1115).  d is an MXFP8 or NVFP4 tensor of logical shape [M, N], rowwise (N % 32 == 0) or
 * colwise (M % 32 == 0); the f32 accumulator times alpha is quantised block by block in the
 * epilogue as by cdl_b200_mx_quantize (without the intermediate rounding to bf16).  Operands
 * and output may have different formats. */
int32_t cdl_b200_matmul_mx_out(const cdl_mx_tensor* a, const cdl_mx_tensor* b, const cdl_mx_tensor* d,
                               float alpha, cdl_stream stream);

/* ---- Flash attention -------------------------------------------------------------------
 * Replaces AttentionExecutor::execute (crates/cleandl/src/execgraph/ops/attention/exec.rs:
 * 358-416), which forwards to flash-attention-rs.  Dense layout only: q [B,Sq,H,D], k and v
 * [B,Sk,Hkv,D] bf16, last dimension contiguous, other strides 16-byte aligned (views into a
 * fused QKV buffer are fine); o like q; lse f32 [B,H,Sq] (natural log; -inf for rows with no
 * visible key).  The causal mask is aligned to the bottom right: query i sees keys
 * j <= i + Sk - Sq (attention/mod.rs:24-31).  D = 128, H % Hkv == 0. */
typedef enum {
  CDL_ATTN_AUTO = 0,      /* the library's choice (the persistent kernel) */
  CDL_ATTN_ONE_SHOT = 1,  /* forward: one short-lived CTA per 256 query rows; backward: one
                           * short-lived CTA per 128-key block (dK, dV) */
  CDL_ATTN_PERSISTENT = 2 /* forward: one CTA per SM walks the 256-row work items, longest first;
                           * part of the exponentials on the FMA pipe; backward: one CTA per SM
                           * walks the key blocks (dK, dV), longest first.  The automatic choice
                           * of the backward is this form when there are more key blocks than SMs. */
} cdl_attn_variant;
typedef struct {
  float softmax_scale; /* <= 0 selects 1/sqrt(D) (exec.rs:198-200) */
  int32_t causal;      /* 0 = AttentionMask::None, 1 = AttentionMask::Causal */
  int32_t variant;     /* cdl_attn_variant: a tuner's per-node choice (see "Per-call kernel
                        * choices").  0 = default. */
} cdl_attn_desc;

int32_t cdl_b200_attn_fwd(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                          const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* lse,
                          cdl_stream stream);
/* Operand order of the reference backward: q, k, v, out, d_out, lse (attention/mod.rs:899-905);
 * outputs dq, dk, dv in the input dtype (:915-919). */
int32_t cdl_b200_attn_bwd(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                          const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* d_out,
                          const cdl_tensor* lse, const cdl_tensor* dq, const cdl_tensor* dk,
                          const cdl_tensor* dv, void* scratch, size_t scratch_bytes,
                          cdl_stream stream);
int32_t cdl_b200_attn_bwd_scratch_bytes(const cdl_tensor* q, const cdl_tensor* k,
                                        size_t* bytes_out);

/* Packed ("varlen") layout of the reference's QueryLayout::Packed / KvLayout::Packed
 * (attention/mod.rs:55-79): q, out, d_out, dq are [total_q, heads, 128] and k, v, dk, dv are
 * [total_k, kv_heads, 128]; sequence b is rows cu_seqlens_q[b] .. cu_seqlens_q[b + 1] of the former
 * and cu_seqlens_k[b] .. cu_seqlens_k[b + 1] of the latter (i32 [batch + 1] in device memory); the
 * mask is aligned bottom-right per sequence; lse is f32 [heads, total_q] (mod.rs:674-677).
 * max_seqlen_q / max_seqlen_k bound every sequence's length and only size the grids (<= 0: the
 * packed total, as `None` does in the reference).  Rows outside every sequence (padding at the
 * end) are neither read into a result nor written; they must hold finite values, because a key
 * row that a tile loads beyond its sequence is multiplied by a zero probability, not skipped. */
int32_t cdl_b200_attn_fwd_packed(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                                 const cdl_tensor* v, const cdl_tensor* cu_seqlens_q,
                                 const cdl_tensor* cu_seqlens_k, int64_t max_seqlen_q,
                                 int64_t max_seqlen_k, const cdl_tensor* o, const cdl_tensor* lse,
                                 cdl_stream stream);
int32_t cdl_b200_attn_bwd_packed(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                                 const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* d_out,
                                 const cdl_tensor* lse, const cdl_tensor* cu_seqlens_q,
                                 const cdl_tensor* cu_seqlens_k, int64_t max_seqlen_q,
                                 int64_t max_seqlen_k, const cdl_tensor* dq, const cdl_tensor* dk,
                                 const cdl_tensor* dv, void* scratch, size_t scratch_bytes,
                                 cdl_stream stream);
int32_t cdl_b200_attn_bwd_packed_scratch_bytes(int64_t batch, int64_t max_seqlen_q, int64_t heads,
                                               size_t* bytes_out);

/* The backward with the rotary embedding's transpose folded into the dQ and dK stores.  q and k are
 * the rotated tensors the forward consumed (as cdl_b200_matmul_rope or cdl_b200_rope produce
 * them); dq and dk come out as the gradients of q and k BEFORE the rotation, so the separate
 * backward call of cdl_b200_rope (one more read and write of both tensors) goes away.  cos_sin is
 * the table of cdl_b200_rope: f32 [positions, 128] = cos(64) | sin(64), at least as many positions
 * as the longest sequence; a row's position is its index in its sequence.  Every head of q and k
 * is rotated, as at the reference's call sites (crates/sky-1/src/training/model/decoder.rs:
 * 363-378 forward, :645-655 backward).
 * The values are those of the two-call form up to one bf16 rounding of f32 arithmetic on the same
 * bf16-rounded dQ / dK.  No counterpart in the reference, whose backward graph holds a separate
 * RoPE node. */
int32_t cdl_b200_attn_bwd_rope(const cdl_attn_desc* desc, const cdl_tensor* q, const cdl_tensor* k,
                               const cdl_tensor* v, const cdl_tensor* o, const cdl_tensor* d_out,
                               const cdl_tensor* lse, const cdl_tensor* cos_sin, const cdl_tensor* dq,
                               const cdl_tensor* dk, const cdl_tensor* dv, void* scratch,
                               size_t scratch_bytes, cdl_stream stream);
int32_t cdl_b200_attn_bwd_packed_rope(const cdl_attn_desc* desc, const cdl_tensor* q,
                                      const cdl_tensor* k, const cdl_tensor* v, const cdl_tensor* o,
                                      const cdl_tensor* d_out, const cdl_tensor* lse,
                                      const cdl_tensor* cu_seqlens_q, const cdl_tensor* cu_seqlens_k,
                                      int64_t max_seqlen_q, int64_t max_seqlen_k,
                                      const cdl_tensor* cos_sin, const cdl_tensor* dq,
                                      const cdl_tensor* dk, const cdl_tensor* dv, void* scratch,
                                      size_t scratch_bytes, cdl_stream stream);

/* ---- Elementwise glue of the sky-1 block -----------------------------------------------
 * The reference's kernels for these lived in its legacy `cleandl::operators` module, which is
 * absent from its tree; the call sites are crates/sky-1/src/training/model/decoder.rs:363-378
 * and :645-655 (RoPE forward / backward on the q and k heads of the fused qkv tensor) and
 * :487-496, :548-558 (SwiGLU).  The SiLU / dSiLU formulas are those of the reference's fused
 * GEMM epilogues (crates/cleandl/rust-kernels/src/sky_matmul/tcgen05_bf16.rs:851-877). */

/* Rotate-half RoPE in place on heads [0, rot_heads) of x bf16 [tokens, heads, head_dim];
 * cos_sin f32 [>= seqlen, head_dim] holds cos | sin per position; position = token % seqlen;
 * backward != 0 applies the inverse rotation (the gradient). */
int32_t cdl_b200_rope(const cdl_tensor* x, const cdl_tensor* cos_sin, int32_t rot_heads,
                      int32_t seqlen, int32_t backward, cdl_stream stream);
/* RoPE over a ragged batch: token t of sequence b (rows cu_seqlens[b] .. cu_seqlens[b + 1]) has
 * position t - cu_seqlens[b]; the table has one row per position; rows after the last sequence are
 * left untouched. */
int32_t cdl_b200_rope_ragged(const cdl_tensor* x, const cdl_tensor* cos_sin, int32_t rot_heads,
                             const cdl_tensor* cu_seqlens, int32_t backward, cdl_stream stream);
/* act = SiLU(gate) * up, packed bf16 tensors of equal size. */
int32_t cdl_b200_swiglu_fwd(const cdl_tensor* gate, const cdl_tensor* up, const cdl_tensor* act,
                            cdl_stream stream);
/* d_up = d_act * SiLU(gate);  d_gate = d_act * up * dSiLU(gate).  d_up may alias d_act. */
int32_t cdl_b200_swiglu_bwd(const cdl_tensor* d_act, const cdl_tensor* gate, const cdl_tensor* up,
                            const cdl_tensor* d_gate, const cdl_tensor* d_up, cdl_stream stream);

/* out[t, :] = table[tokens[t], :]; tokens i32 [T], table bf16 [vocab, hidden], out bf16 [T, hidden].
 * Call site: crates/sky-1/src/training/model/mod.rs:221-226 (embedding lookup). */
int32_t cdl_b200_embedding_fwd(const cdl_tensor* tokens, const cdl_tensor* table,
                               const cdl_tensor* out, cdl_stream stream);

/* ---- Loss and optimizer step of the LM ---------------------------------------------------
 * Call sites in the reference (the kernels themselves are not in its tree):
 * crates/sky-1/src/training/model/mod.rs:262-271 (cross-entropy that leaves the logits' gradient
 * in place of the logits), :351-356 (embedding scatter-add), :361-420 and decoder.rs:716-752
 * (gradient sum of squares, AdamW with global-norm clipping writing the f32 master weight and its
 * bf16 replica, then zero-filled gradients; no weight decay on norm gains, decoder.rs:724-731). */

/* loss[t] = logsumexp(logits[t, :]) - logits[t, targets[t]];  logits[t, :] is OVERWRITTEN with
 * (softmax - onehot) * grad_scale.  targets[t] < 0 marks an ignored row (loss 0, gradient 0).
 * logits bf16 [T, vocab], vocab % 8 == 0; targets i32 [T]; loss f32 [T]. */
int32_t cdl_b200_cross_entropy(const cdl_tensor* logits, const cdl_tensor* targets,
                               const cdl_tensor* loss, float grad_scale, cdl_stream stream);
/* d_table[tokens[t], :] += dx[t, :];  d_table f32 [vocab, hidden], dx bf16 [T, hidden]. */
int32_t cdl_b200_embedding_bwd(const cdl_tensor* tokens, const cdl_tensor* dx,
                               const cdl_tensor* d_table, cdl_stream stream);
/* out[0] = (accumulate ? out[0] : 0) + scale * sum_i (square ? x_i^2 : x_i), summed in a fixed
 * order (deterministic).  scratch: 4096 bytes. */
int32_t cdl_b200_sum(const float* x, int64_t n, float* out, float scale, int32_t square,
                     int32_t accumulate, void* scratch, size_t scratch_bytes, cdl_stream stream);
typedef struct {
  float lr, beta1, beta2, eps, weight_decay;
  int32_t step;        /* 1-based, for the bias correction */
  float grad_scale;    /* multiplies the raw gradient (e.g. 1 / data-parallel ranks) */
  float max_grad_norm; /* <= 0: no clipping; else clip by sqrt(*grad_sumsq) * grad_scale */
} cdl_adamw_params;
/* AdamW over n contiguous elements: updates master (f32), replica (bf16), m, v, zeroes grad.
 * grad_sumsq: device scalar with the sum of squares of ALL raw gradients of the model (nullable). */
int32_t cdl_b200_adamw(float* master, void* replica_bf16, float* grad, float* m, float* v, int64_t n,
                       const float* grad_sumsq, const cdl_adamw_params* hp, cdl_stream stream);

/* ---- sky-1 decoder block ---------------------------------------------------------------
 * One call per direction for the dataflow of DecoderExecutor::train_forward / train_backward
 * (crates/sky-1/src/training/model/decoder.rs:332-520, 523-695): pre-RMSNorm, fused QKV
 * projection, RoPE, causal attention, output projection with fused residual, pre-RMSNorm,
 * SwiGLU FFN with fused residual.  All tensors are packed row-major device buffers; tokens
 * T = batch * seqlen.  Weights are bf16 stored [in, out] (decoder.rs:166-173); gradients are
 * f32 and ACCUMULATED (parameter.rs:69-74).  head_dim must be 128. */
typedef enum {
  CDL_SKY1_DETERMINISTIC = 1 /* weight-gradient GEMMs with a fixed summation order
                              * (cdl_matmul_options.deterministic for every product of the block) */
} cdl_sky1_flags;
typedef struct {
  int32_t batch, seqlen, hidden, heads, kv_heads, head_dim, ffn;
  float eps;
  int32_t flags; /* bit set of cdl_sky1_flags; 0 = defaults */
} cdl_sky1_config;
typedef struct { /* bf16 */
  const void* norm1; /* [hidden] */
  const void* wqkv;  /* [hidden, (heads + 2 kv_heads) head_dim] */
  const void* wo;    /* [heads head_dim, hidden] */
  const void* norm2; /* [hidden] */
  const void* wup;   /* [hidden, ffn] */
  const void* wgate; /* [hidden, ffn] */
  const void* wdown; /* [ffn, hidden] */
} cdl_sky1_weights;
typedef struct { /* f32, same shapes as the weights */
  float *norm1, *wqkv, *wo, *norm2, *wup, *wgate, *wdown;
} cdl_sky1_grads;
typedef struct { /* activations the forward saves for the backward (decoder.rs:506-519) */
  void* qkv;  /* bf16 [T, (heads + 2 kv_heads) head_dim], after RoPE */
  void* attn; /* bf16 [T, heads head_dim] */
  float* lse; /* f32 [batch, heads, seqlen] */
  void* o;    /* bf16 [T, hidden]: attention output projection + residual */
  void* up;   /* bf16 [T, ffn] */
  void* gate; /* bf16 [T, ffn] */
  void* act;  /* bf16 [T, ffn] */
} cdl_sky1_saved;

/* Ragged batch (the layout sky-1 trains with: `decoder_ragged_seqlen.cu_seqlen()`,
 * crates/sky-1/src/training/model/decoder.rs:372-378, 440-455): the T = batch * seqlen token rows
 * of the block's buffers hold num_seqs sequences, sequence b in rows cu_seqlens[b] ..
 * cu_seqlens[b + 1] (i32 [num_seqs + 1], device memory); RoPE positions restart at every
 * sequence, attention is causal within a sequence, the saved lse is f32 [heads, T], the RoPE table
 * has max_seqlen rows.  Rows after the last sequence are padding: x there must be finite and dy
 * must be zero (their attention output and their d_qkv are zeroed by the library), so that they add
 * nothing to the weight gradients. */
typedef struct {
  const int32_t* cu_seqlens;
  int32_t num_seqs;
  int32_t max_seqlen; /* bound on every sequence's length */
} cdl_sky1_ragged;

int32_t cdl_b200_sky1_block_workspace_bytes_ragged(const cdl_sky1_config* cfg,
                                                   const cdl_sky1_ragged* ragged, size_t* fwd_bytes,
                                                   size_t* bwd_bytes);
int32_t cdl_b200_sky1_block_fwd_ragged(const cdl_sky1_config* cfg, const cdl_sky1_weights* weights,
                                       const void* x, const float* rope_cos_sin,
                                       const cdl_sky1_ragged* ragged, const cdl_sky1_saved* saved,
                                       void* out, void* workspace, size_t workspace_bytes,
                                       cdl_stream stream);
int32_t cdl_b200_sky1_block_bwd_ragged(const cdl_sky1_config* cfg, const cdl_sky1_weights* weights,
                                       const void* x, const float* rope_cos_sin,
                                       const cdl_sky1_ragged* ragged, const cdl_sky1_saved* saved,
                                       const void* dy, const cdl_sky1_grads* grads, void* dx,
                                       void* workspace, size_t workspace_bytes, int32_t phase,
                                       cdl_stream stream);

int32_t cdl_b200_sky1_block_workspace_bytes(const cdl_sky1_config* cfg, size_t* fwd_bytes,
                                            size_t* bwd_bytes);
/* x, out: bf16 [T, hidden]; rope_cos_sin: f32 [seqlen, head_dim]; workspace 256-byte aligned. */
int32_t cdl_b200_sky1_block_fwd(const cdl_sky1_config* cfg, const cdl_sky1_weights* weights,
                                const void* x, const float* rope_cos_sin,
                                const cdl_sky1_saved* saved, void* out, void* workspace,
                                size_t workspace_bytes, cdl_stream stream);
/* dy: gradient of out; dx: gradient of x (both bf16 [T, hidden]).  `phase` lets a data-parallel
 * caller start reducing the FFN gradients while the attention half still runs: 0 = whole
 * backward; 1 = FFN half only (after it, grads wdown / wup / wgate / norm2 are final and the
 * workspace holds the intermediate gradient); 2 = attention half (must follow phase 1 with the
 * same workspace, untouched in between). */
int32_t cdl_b200_sky1_block_bwd(const cdl_sky1_config* cfg, const cdl_sky1_weights* weights,
                                const void* x, const float* rope_cos_sin,
                                const cdl_sky1_saved* saved, const void* dy,
                                const cdl_sky1_grads* grads, void* dx, void* workspace,
                                size_t workspace_bytes, int32_t phase, cdl_stream stream);

/* The whole backward with one CUDA event per group of weight gradients, for a data-parallel
 * caller that reduces gradients while the backward still runs (finer than the two phases above and
 * without returning to the host in between).  Each handle is a cudaEvent_t or NULL; the library
 * records it on `stream` right after the last kernel that writes the group is enqueued, in this
 * order: wdown; wup; wgate and norm2; wo; wqkv and norm1 (the last one also marks the end of the
 * backward).  The caller lets its communication stream wait for an event and starts that group's
 * all-reduce.  `ragged` may be NULL (dense batch).  No counterpart in the reference, whose
 * data-parallel reduction runs after the backward graph (crates/sky-1/src/training). */
typedef struct {
  void *wdown, *wup, *wgate_norm2, *wo, *wqkv_norm1;
} cdl_sky1_grad_events;
int32_t cdl_b200_sky1_block_bwd_events(const cdl_sky1_config* cfg, const cdl_sky1_weights* weights,
                                       const void* x, const float* rope_cos_sin,
                                       const cdl_sky1_ragged* ragged, const cdl_sky1_saved* saved,
                                       const void* dy, const cdl_sky1_grads* grads, void* dx,
                                       void* workspace, size_t workspace_bytes,
                                       const cdl_sky1_grad_events* events, cdl_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* CLEANDL_B200_H */
