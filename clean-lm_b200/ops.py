"""Operator front ends mirroring the reference's graph nodes, executing eagerly on torch tensors.

Names, options and error behaviour follow the reference's DSL entry points:
  `SymTensor::matmul`         crates/cleandl/src/execgraph/ops/matmul.rs:90-108   -> matmul
  `SymTensor::norm_fwd`       crates/cleandl/src/execgraph/ops/norm/mod.rs:126-160 -> norm_fwd
  `SymTensor::attention_fwd`  crates/cleandl/src/execgraph/ops/attention/mod.rs:276-350
  `SymTensor::attention_bwd`  (same file)                                          -> attention_*
`norm_bwd` follows the legacy call site crates/sky-1/src/training/model/decoder.rs:599-607.

This layer plays the engine's part (plan.rs:397-451): it allocates outputs and scratch with torch,
then calls the C ABI on the current CUDA stream.  All arithmetic happens in the CUDA library.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import CdlAttnDesc, check, lib, ref, tensor_arg


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise _lib.CdlError(-1, "operands must live in device memory (there is no CPU path)")


# --------------------------------------------------------------------------- matmul
@dataclass
class MatmulOpts:
    """`MatmulOpts` of the reference (ops/matmul.rs:71-88)."""

    out: torch.dtype = torch.bfloat16
    c: Optional[torch.Tensor] = None  # needs a nonzero beta to have an effect
    alpha: float = 1.0
    beta: float = 0.0
    # Kernel choice, the argument an engine's tuner would vary per graph node (cdl_matmul_options):
    variant: int = _lib.GEMM_AUTO
    deterministic: bool = False  # fixed f32 summation order for the accumulate-in-place form


def matmul(a: torch.Tensor, b: torch.Tensor, opts: MatmulOpts | None = None,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """D = alpha * A . B + beta * C.  `a`/`b` may be transposed views (`.mT`); `out` may be
    given to write in place (e.g. out = c for accumulating wgrads)."""
    opts = opts or MatmulOpts()
    _require_cuda(a, b, opts.c, out)
    if a.dim() != b.dim() or a.dim() not in (2, 3):
        raise _lib.CdlError(-1, f"matmul operands must both have rank 2 or rank 3 "
                                f"(got rank {a.dim()} and {b.dim()})")
    if a.shape[-1] != b.shape[-2]:
        raise _lib.CdlError(-1, f"matmul contraction dimensions differ: {tuple(a.shape)} x "
                                f"{tuple(b.shape)}")
    if out is None:
        out = torch.empty(*a.shape[:-1], b.shape[-1], dtype=opts.out, device=a.device)
    ta, tb, tc, td = tensor_arg(a), tensor_arg(b), tensor_arg(opts.c), tensor_arg(out)
    if opts.variant == _lib.GEMM_AUTO and not opts.deterministic:
        check(lib.cdl_b200_matmul(ref(ta), ref(tb), ref(tc), ref(td), opts.alpha, opts.beta, None, 0,
                                  _stream()))
    else:
        mo = _lib.CdlMatmulOptions(int(opts.variant), 1 if opts.deterministic else 0)
        check(lib.cdl_b200_matmul_opt(ref(ta), ref(tb), ref(tc), ref(td), opts.alpha, opts.beta,
                                      ctypes.byref(mo), None, 0, _stream()))
    return out


def matmul_candidates(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> list:
    """[(variant, deterministic), ...] valid for this problem, the heuristic default first
    (what an Executor would hand the tuner, op.rs:301-318)."""
    buf = (_lib.CdlMatmulOptions * 8)()
    n = ctypes.c_int32(0)
    ta, tb, td = tensor_arg(a), tensor_arg(b), tensor_arg(out)
    check(lib.cdl_b200_matmul_candidates(ref(ta), ref(tb), ref(td), buf, 8, ctypes.byref(n)))
    return [(buf[i].variant, bool(buf[i].deterministic)) for i in range(n.value)]


# --------------------------------------------------------------------------- norm
@dataclass
class NormFwdOpts:
    """`NormFwdOpts` of the reference (ops/norm/mod.rs:87-111); `out` is the element type of
    `NormOutput::Plain` (bf16 or f32; the block-scaled outputs are in `mx.norm_fwd_mx`).
    `norm_type`: "rms" (`NormType::RmsNorm`) or "layer" (`LayerNorm`)."""

    scale: Optional[torch.Tensor] = None
    bias: Optional[torch.Tensor] = None
    eps: float = 1e-6
    save_stats: bool = False
    norm_type: str = "rms"
    out: torch.dtype = torch.bfloat16
    variant: int = _lib.NORM_AUTO  # cdl_norm_options.variant (RMSNorm only)


@dataclass
class NormFwdOutputs:
    y: torch.Tensor
    r_inv: Optional[torch.Tensor]  # per-row reciprocal RMS / standard deviation (f32), with save_stats
    mean: Optional[torch.Tensor] = None  # per-row mean (f32): layer norm with save_stats


def norm_fwd(x: torch.Tensor, opts: NormFwdOpts | None = None) -> NormFwdOutputs:
    opts = opts or NormFwdOpts()
    _require_cuda(x, opts.scale, opts.bias)
    if x.dim() != 2:
        raise _lib.CdlError(-1, "norm_fwd: x must be a 2D tensor")
    y = torch.empty(x.shape, dtype=opts.out, device=x.device)
    r_inv = torch.empty(x.shape[0], dtype=torch.float32, device=x.device) if opts.save_stats else None
    tx, ts, tb, ty, tr = (tensor_arg(t) for t in (x, opts.scale, opts.bias, y, r_inv))
    if opts.norm_type == "layer":
        mean = torch.empty(x.shape[0], dtype=torch.float32, device=x.device) if opts.save_stats else None
        tm = tensor_arg(mean)
        check(lib.cdl_b200_layernorm_fwd(ref(tx), ref(ts), ref(tb), opts.eps, ref(ty), ref(tm), ref(tr),
                                         _stream()))
        return NormFwdOutputs(y, r_inv, mean)
    if opts.norm_type != "rms":
        raise _lib.CdlError(-1, f"norm_fwd: unknown norm type '{opts.norm_type}'")
    if opts.variant != _lib.NORM_AUTO:
        no = _lib.CdlNormOptions(int(opts.variant))
        check(lib.cdl_b200_rmsnorm_fwd_opt(ref(tx), ref(ts), ref(tb), opts.eps, ref(ty), ref(tr),
                                           ctypes.byref(no), _stream()))
        return NormFwdOutputs(y, r_inv)
    check(lib.cdl_b200_rmsnorm_fwd(ref(tx), ref(ts), ref(tb), opts.eps, ref(ty), ref(tr), _stream()))
    return NormFwdOutputs(y, r_inv)


def norm_bwd_scratch_bytes(rows: int, cols: int) -> int:
    n = ctypes.c_size_t(0)
    check(lib.cdl_b200_rmsnorm_bwd_scratch_bytes(rows, cols, ctypes.byref(n)))
    return n.value


def norm_bwd(x, dy, scale, r_inv, dscale, residual_dy=None, scratch=None, dx=None,
             variant: int = _lib.NORM_AUTO) -> torch.Tensor:
    """dx of RMSNorm; `dscale` (f32 [cols]) is accumulated in place.  `variant` selects the
    kernel form (cdl_norm_options.variant)."""
    _require_cuda(x, dy, scale, r_inv, dscale, residual_dy)
    if x.dim() != 2:
        raise _lib.CdlError(-1, "norm_bwd: x must be a 2D tensor")
    if dx is None:
        dx = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    need = norm_bwd_scratch_bytes(x.shape[0], x.shape[1])
    if scratch is None:
        scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=x.device)
    args = [tensor_arg(t) for t in (x, dy, residual_dy, scale, r_inv, dx, dscale)]
    if variant != _lib.NORM_AUTO:
        no = _lib.CdlNormOptions(int(variant))
        check(lib.cdl_b200_rmsnorm_bwd_opt(*(ref(a) for a in args), ctypes.byref(no),
                                           ctypes.c_void_p(scratch.data_ptr()),
                                           scratch.numel() * scratch.element_size(), _stream()))
        return dx
    check(lib.cdl_b200_rmsnorm_bwd(*(ref(a) for a in args), ctypes.c_void_p(scratch.data_ptr()),
                                   scratch.numel() * scratch.element_size(), _stream()))
    return dx


# --------------------------------------------------------------------------- attention
@dataclass
class AttentionOpts:
    """The subset of `AttentionOpts` (ops/attention/mod.rs:94-112) this library implements:
    dense or packed layouts, mask None or Causal, no softcap.

    Packed layout (`QueryLayout::Packed` / `KvLayout::Packed`, mod.rs:55-79): q is
    [total_q, heads, head_dim], k and v are [total_k, kv_heads, head_dim], sequence b is rows
    cu_seqlens[b] .. cu_seqlens[b + 1]; both cu_seqlens (i32 [batch + 1], on the device) must be
    given together.  max_seqlen bounds every sequence's length; None is the packed total."""

    softmax_scale: Optional[float] = None  # None is 1 / sqrt(head_dim)
    causal: bool = True
    cu_seqlens_q: Optional[torch.Tensor] = None
    cu_seqlens_k: Optional[torch.Tensor] = None
    max_seqlen_q: Optional[int] = None
    max_seqlen_k: Optional[int] = None
    variant: int = _lib.ATTN_AUTO  # cdl_attn_desc.variant: the forward kernel (a tuner's choice)

    @property
    def packed(self) -> bool:
        if (self.cu_seqlens_q is None) != (self.cu_seqlens_k is None):
            raise _lib.CdlError(-1, "attention: cu_seqlens_q and cu_seqlens_k must be given together")
        return self.cu_seqlens_q is not None


@dataclass
class AttentionFwdOutputs:
    out: torch.Tensor
    lse: Optional[torch.Tensor]  # f32 [batch, heads, seqlen_q] (packed: [heads, total_q]), natural log


def _attn_desc(opts: AttentionOpts) -> CdlAttnDesc:
    d = CdlAttnDesc()
    d.softmax_scale = float(opts.softmax_scale) if opts.softmax_scale is not None else 0.0
    d.causal = 1 if opts.causal else 0
    d.variant = int(opts.variant)
    return d


def attention_fwd(q, k, v, opts: AttentionOpts | None = None, lse: bool = True,
                  out=None) -> AttentionFwdOutputs:
    """`out` (dense layout only) receives the result in place of a new tensor."""
    opts = opts or AttentionOpts()
    _require_cuda(q, k, v)
    if opts.packed:
        if q.dim() != 3:
            raise _lib.CdlError(-1, "attention: packed q must be [total_q, heads, head_dim]")
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        lse_t = (torch.empty(q.shape[1], q.shape[0], dtype=torch.float32, device=q.device)
                 if lse else None)
        desc = _attn_desc(opts)
        a = [tensor_arg(t) for t in (q, k, v, opts.cu_seqlens_q, opts.cu_seqlens_k)]
        b = [tensor_arg(t) for t in (out, lse_t)]
        check(lib.cdl_b200_attn_fwd_packed(ctypes.byref(desc), *(ref(x) for x in a),
                                           int(opts.max_seqlen_q or 0), int(opts.max_seqlen_k or 0),
                                           *(ref(x) for x in b), _stream()))
        return AttentionFwdOutputs(out, lse_t)
    if q.dim() != 4:
        raise _lib.CdlError(-1, "attention: q must be [batch, seqlen, heads, head_dim]")
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    lse_t = (torch.empty(q.shape[0], q.shape[2], q.shape[1], dtype=torch.float32, device=q.device)
             if lse else None)
    desc = _attn_desc(opts)
    args = [tensor_arg(t) for t in (q, k, v, out, lse_t)]
    check(lib.cdl_b200_attn_fwd(ctypes.byref(desc), *(ref(a) for a in args), _stream()))
    return AttentionFwdOutputs(out, lse_t)


def attention_bwd_scratch_bytes(q, k) -> int:
    n = ctypes.c_size_t(0)
    tq, tk = tensor_arg(q), tensor_arg(k)
    check(lib.cdl_b200_attn_bwd_scratch_bytes(ref(tq), ref(tk), ctypes.byref(n)))
    return n.value


def attention_bwd(q, k, v, out, d_out, lse, opts: AttentionOpts | None = None, scratch=None,
                  dq=None, dk=None, dv=None, rope_table=None):
    """Returns (dq, dk, dv) in the input dtype (ops/attention/mod.rs:915-919).

    With ``rope_table`` (f32 [positions, 128] = cos | sin) q and k are taken as rotated by the
    rotary embedding and dq, dk are the gradients of the tensors before the rotation: the
    transposed rotation runs in the kernels' store epilogues instead of as a call of its own."""
    opts = opts or AttentionOpts()
    _require_cuda(q, k, v, out, d_out, lse)
    if rope_table is not None:
        _require_cuda(rope_table)
    dq = torch.empty(q.shape, dtype=q.dtype, device=q.device) if dq is None else dq
    dk = torch.empty(k.shape, dtype=k.dtype, device=k.device) if dk is None else dk
    dv = torch.empty(v.shape, dtype=v.dtype, device=v.device) if dv is None else dv
    if opts.packed:
        if q.dim() != 3:
            raise _lib.CdlError(-1, "attention: packed q must be [total_q, heads, head_dim]")
        batch = opts.cu_seqlens_q.shape[0] - 1
        max_q = int(opts.max_seqlen_q or 0)
        n = ctypes.c_size_t(0)
        check(lib.cdl_b200_attn_bwd_packed_scratch_bytes(
            batch, max_q if 0 < max_q <= q.shape[0] else q.shape[0], q.shape[1], ctypes.byref(n)))
        if scratch is None:
            scratch = torch.empty(max(n.value, 16), dtype=torch.uint8, device=q.device)
        desc = _attn_desc(opts)
        a = [tensor_arg(t) for t in (q, k, v, out, d_out, lse, opts.cu_seqlens_q, opts.cu_seqlens_k)]
        b = [tensor_arg(t) for t in (dq, dk, dv)]
        if rope_table is not None:
            b.insert(0, tensor_arg(rope_table))
        fn = lib.cdl_b200_attn_bwd_packed if rope_table is None else lib.cdl_b200_attn_bwd_packed_rope
        check(fn(ctypes.byref(desc), *(ref(x) for x in a), max_q, int(opts.max_seqlen_k or 0),
                 *(ref(x) for x in b), ctypes.c_void_p(scratch.data_ptr()),
                 scratch.numel() * scratch.element_size(), _stream()))
        return dq, dk, dv
    need = attention_bwd_scratch_bytes(q, k)
    if scratch is None:
        scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
    desc = _attn_desc(opts)
    tensors = (q, k, v, out, d_out, lse) + (() if rope_table is None else (rope_table,)) + (dq, dk, dv)
    args = [tensor_arg(t) for t in tensors]
    fn = lib.cdl_b200_attn_bwd if rope_table is None else lib.cdl_b200_attn_bwd_rope
    check(fn(ctypes.byref(desc), *(ref(a) for a in args), ctypes.c_void_p(scratch.data_ptr()),
             scratch.numel() * scratch.element_size(), _stream()))
    return dq, dk, dv
