//! Raw bindings of `include/cleandl_b200.h` (libcleandl_b200.so).  SOURCE ONLY: this tree has no
//! Rust toolchain, so nothing here was compiled; it is the binding a maintainer of
//! `crates/cleandl` would add, kept next to the header so that a signature change shows up here.
//!
//! Every function returns 0 on success and a negative `cdl_status` otherwise; the message of the
//! last failure on the calling thread is `cdl_b200_last_error()`.  Nothing allocates, nothing
//! synchronises, all work goes to the stream passed in (`Executor::execute`'s contract,
//! crates/cleandl/src/execgraph/op.rs:130-142).
#![allow(non_camel_case_types)]

use std::ffi::{c_char, c_void};

pub const CDL_BF16: i32 = 0;
pub const CDL_F32: i32 = 1;
pub const CDL_I32: i32 = 2;

/// `cdl_tensor`: a strided view of device memory, strides in elements, rank <= 4.
#[repr(C)]
#[derive(Copy, Clone, Debug)]
pub struct CdlTensor {
    pub ptr: *mut c_void,
    pub dtype: i32,
    pub rank: i32,
    pub shape: [i64; 4],
    pub stride: [i64; 4],
}

/// `cdl_attn_desc`.
#[repr(C)]
#[derive(Copy, Clone, Debug)]
pub struct CdlAttnDesc {
    pub softmax_scale: f32, // <= 0: 1 / sqrt(head_dim)
    pub causal: i32,        // 0 = AttentionMask::None, 1 = AttentionMask::Causal
    pub variant: i32,       // cdl_attn_variant: 0 auto, 1 one short-lived CTA per block, 2 one CTA per SM (forward and backward)
}

/// `cdl_matmul_options`: what a tuner candidate of the matmul executor carries.
#[repr(C)]
#[derive(Copy, Clone, Debug, PartialEq, Eq, serde::Serialize, serde::Deserialize)]
pub struct CdlMatmulOptions {
    pub variant: i32,       // cdl_gemm_variant: 0 auto, 1 one CTA, 2 CTA pair
    pub deterministic: i32, // != 0: fixed f32 summation order for the weight-gradient form
}

/// `cdl_norm_options`.
#[repr(C)]
#[derive(Copy, Clone, Debug, PartialEq, Eq, serde::Serialize, serde::Deserialize)]
pub struct CdlNormOptions {
    pub variant: i32, // cdl_norm_variant: 0 auto, 1 warp per row, 2 pipelined
}

/// `cdl_mx_tensor`: MxFormat::Mxfp8 = 0, Nvfp4 = 1; MxDim::Rowwise = 0, Colwise = 1.
#[repr(C)]
#[derive(Copy, Clone, Debug)]
pub struct CdlMxTensor {
    pub values: *mut c_void,
    pub scale_factors: *mut c_void,
    pub format: i32,
    pub dim: i32,
    pub rows: i64,
    pub cols: i64,
}

#[link(name = "cleandl_b200")]
extern "C" {
    pub fn cdl_b200_last_error() -> *const c_char;
    pub fn cdl_b200_device_ok(device: i32) -> i32;
    pub fn cdl_b200_device_status(status_out: *mut i32) -> i32;

    // ---- matmul (replaces MatmulExecutor::execute, ops/matmul.rs:1092-1183)
    pub fn cdl_b200_matmul(
        a: *const CdlTensor, b: *const CdlTensor, c: *const CdlTensor, d: *const CdlTensor,
        alpha: f32, beta: f32, scratch: *mut c_void, scratch_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_matmul_opt(
        a: *const CdlTensor, b: *const CdlTensor, c: *const CdlTensor, d: *const CdlTensor,
        alpha: f32, beta: f32, options: *const CdlMatmulOptions, scratch: *mut c_void,
        scratch_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_matmul_candidates(
        a: *const CdlTensor, b: *const CdlTensor, d: *const CdlTensor,
        out: *mut CdlMatmulOptions, capacity: i32, count: *mut i32,
    ) -> i32;
    pub fn cdl_b200_matmul_scratch_bytes(
        a: *const CdlTensor, b: *const CdlTensor, d: *const CdlTensor, bytes_out: *mut usize,
    ) -> i32;
    pub fn cdl_b200_matmul_rope(
        a: *const CdlTensor, b: *const CdlTensor, cos_sin: *const CdlTensor, rot_heads: i32,
        seqlen: i32, cu_seqlens: *const CdlTensor, d: *const CdlTensor, stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_matmul_swiglu_gate(
        a: *const CdlTensor, b: *const CdlTensor, up: *const CdlTensor,
        gate_out: *const CdlTensor, act_out: *const CdlTensor, stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_matmul_swiglu_dgrad(
        a: *const CdlTensor, b: *const CdlTensor, gate: *const CdlTensor, up: *const CdlTensor,
        d_up_out: *const CdlTensor, d_gate_out: *const CdlTensor, stream: *mut c_void,
    ) -> i32;

    // ---- norms (replace SpecializedExecutor::execute, ops/norm/specialized.rs:116-200)
    pub fn cdl_b200_rmsnorm_fwd(
        x: *const CdlTensor, scale: *const CdlTensor, bias: *const CdlTensor, eps: f32,
        y: *const CdlTensor, r_inv: *const CdlTensor, stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_rmsnorm_fwd_opt(
        x: *const CdlTensor, scale: *const CdlTensor, bias: *const CdlTensor, eps: f32,
        y: *const CdlTensor, r_inv: *const CdlTensor, options: *const CdlNormOptions,
        stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_layernorm_fwd(
        x: *const CdlTensor, scale: *const CdlTensor, bias: *const CdlTensor, eps: f32,
        y: *const CdlTensor, mean: *const CdlTensor, r_inv: *const CdlTensor, stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_rmsnorm_bwd(
        x: *const CdlTensor, dy: *const CdlTensor, residual_dy: *const CdlTensor,
        scale: *const CdlTensor, r_inv: *const CdlTensor, dx: *const CdlTensor,
        dscale: *const CdlTensor, scratch: *mut c_void, scratch_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_rmsnorm_bwd_opt(
        x: *const CdlTensor, dy: *const CdlTensor, residual_dy: *const CdlTensor,
        scale: *const CdlTensor, r_inv: *const CdlTensor, dx: *const CdlTensor,
        dscale: *const CdlTensor, options: *const CdlNormOptions, scratch: *mut c_void,
        scratch_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_rmsnorm_bwd_static(
        x: *const CdlTensor, dy: *const CdlTensor, residual_dy: *const CdlTensor,
        scale: *const CdlTensor, r_inv: *const CdlTensor, dx: *const CdlTensor,
        dscale: *const CdlTensor, stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_rmsnorm_bwd_scratch_bytes(rows: i64, cols: i64, bytes_out: *mut usize) -> i32;

    // ---- attention (replaces AttentionExecutor::execute, ops/attention/exec.rs:358-416)
    pub fn cdl_b200_attn_fwd(
        desc: *const CdlAttnDesc, q: *const CdlTensor, k: *const CdlTensor, v: *const CdlTensor,
        o: *const CdlTensor, lse: *const CdlTensor, stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_attn_bwd(
        desc: *const CdlAttnDesc, q: *const CdlTensor, k: *const CdlTensor, v: *const CdlTensor,
        o: *const CdlTensor, d_out: *const CdlTensor, lse: *const CdlTensor, dq: *const CdlTensor,
        dk: *const CdlTensor, dv: *const CdlTensor, scratch: *mut c_void, scratch_bytes: usize,
        stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_attn_bwd_scratch_bytes(
        q: *const CdlTensor, k: *const CdlTensor, bytes_out: *mut usize,
    ) -> i32;
    pub fn cdl_b200_attn_fwd_packed(
        desc: *const CdlAttnDesc, q: *const CdlTensor, k: *const CdlTensor, v: *const CdlTensor,
        cu_seqlens_q: *const CdlTensor, cu_seqlens_k: *const CdlTensor, max_seqlen_q: i64,
        max_seqlen_k: i64, o: *const CdlTensor, lse: *const CdlTensor, stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_attn_bwd_packed(
        desc: *const CdlAttnDesc, q: *const CdlTensor, k: *const CdlTensor, v: *const CdlTensor,
        o: *const CdlTensor, d_out: *const CdlTensor, lse: *const CdlTensor,
        cu_seqlens_q: *const CdlTensor, cu_seqlens_k: *const CdlTensor, max_seqlen_q: i64,
        max_seqlen_k: i64, dq: *const CdlTensor, dk: *const CdlTensor, dv: *const CdlTensor,
        scratch: *mut c_void, scratch_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_attn_bwd_packed_scratch_bytes(
        batch: i64, max_seqlen_q: i64, heads: i64, bytes_out: *mut usize,
    ) -> i32;
    // The backward with the inverse rotary rotation of dQ / dK in its store epilogues (q and k are
    // the rotated tensors): for a graph pass that fuses the RoPE node behind AttentionBwd.
    pub fn cdl_b200_attn_bwd_rope(
        desc: *const CdlAttnDesc, q: *const CdlTensor, k: *const CdlTensor, v: *const CdlTensor,
        o: *const CdlTensor, d_out: *const CdlTensor, lse: *const CdlTensor,
        cos_sin: *const CdlTensor, dq: *const CdlTensor, dk: *const CdlTensor,
        dv: *const CdlTensor, scratch: *mut c_void, scratch_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_attn_bwd_packed_rope(
        desc: *const CdlAttnDesc, q: *const CdlTensor, k: *const CdlTensor, v: *const CdlTensor,
        o: *const CdlTensor, d_out: *const CdlTensor, lse: *const CdlTensor,
        cu_seqlens_q: *const CdlTensor, cu_seqlens_k: *const CdlTensor, max_seqlen_q: i64,
        max_seqlen_k: i64, cos_sin: *const CdlTensor, dq: *const CdlTensor, dk: *const CdlTensor,
        dv: *const CdlTensor, scratch: *mut c_void, scratch_bytes: usize, stream: *mut c_void,
    ) -> i32;

    // ---- block-scaled tensors (MxTensor, crates/cleandl/src/mx_tensor.rs:11-30)
    pub fn cdl_b200_mx_layout(
        format: i32, dim: i32, rows: i64, cols: i64, values_bytes: *mut usize,
        scale_bytes: *mut usize,
    ) -> i32;
    pub fn cdl_b200_mx_quantize(
        x: *const CdlTensor, y_rowwise: *const CdlMxTensor, y_colwise: *const CdlMxTensor,
        stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_mx_dequantize(x: *const CdlMxTensor, y: *const CdlTensor, stream: *mut c_void) -> i32;
    pub fn cdl_b200_rmsnorm_fwd_mx(
        x: *const CdlTensor, scale: *const CdlTensor, bias: *const CdlTensor, eps: f32,
        y_rowwise: *const CdlMxTensor, y_colwise: *const CdlMxTensor, r_inv: *const CdlTensor,
        stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_matmul_mx(
        a: *const CdlMxTensor, b: *const CdlMxTensor, c: *const CdlTensor, d: *const CdlTensor,
        alpha: f32, beta: f32, stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_matmul_mx_opt(
        a: *const CdlMxTensor, b: *const CdlMxTensor, c: *const CdlTensor, d: *const CdlTensor,
        alpha: f32, beta: f32, options: *const CdlMatmulOptions, stream: *mut c_void,
    ) -> i32;
    pub fn cdl_b200_matmul_mx_out(
        a: *const CdlMxTensor, b: *const CdlMxTensor, d: *const CdlMxTensor, alpha: f32,
        stream: *mut c_void,
    ) -> i32;
}
