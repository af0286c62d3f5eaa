"""Block-scaled (MXFP8) tensors and the operators that produce and consume them.

Mirrors the reference's `MxTensor` (crates/cleandl/src/mx_tensor.rs:11-137), `NormFwd` with
`NormOutput::Mxfp8Rowwise` / `Mxfp8RowwiseAndColwise` (crates/cleandl/src/execgraph/ops/norm/
mod.rs:33-62) and `Matmul` with block-scaled inputs (ops/matmul.rs:808-838).  torch owns the
device memory; all arithmetic happens in the CUDA library.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import CdlMxTensor, check, lib, ref, tensor_arg

MXFP8, NVFP4 = _lib.CDL_MXFP8, _lib.CDL_NVFP4
ROWWISE, COLWISE = _lib.CDL_MX_ROWWISE, _lib.CDL_MX_COLWISE
BLOCK = 32  # MXFP8; NVFP4 blocks hold 16 elements


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def layout_bytes(rows: int, cols: int, dim: int, fmt: int = MXFP8):
    """(values bytes, scale-factor bytes) of a block-scaled [rows, cols] tensor (`MxLayout::new`)."""
    v, s = ctypes.c_size_t(0), ctypes.c_size_t(0)
    check(lib.cdl_b200_mx_layout(fmt, dim, rows, cols, ctypes.byref(v), ctypes.byref(s)))
    return v.value, s.value


@dataclass
class MxTensor:
    """values: uint8 [rows, cols] (rowwise) or [cols, rows] (colwise), for NVFP4 with two elements
    per byte along the last dimension; scale_factors: uint8, the 128 x 4 tiled layout, flat."""

    values: torch.Tensor
    scale_factors: torch.Tensor
    dim: int
    rows: int
    cols: int
    format: int = MXFP8

    @staticmethod
    def empty(rows: int, cols: int, dim: int, device="cuda", zero_scales: bool = False,
              fmt: int = MXFP8) -> "MxTensor":
        vb, sb = layout_bytes(rows, cols, dim, fmt)
        outer, inner = (rows, cols) if dim == ROWWISE else (cols, rows)
        values = torch.empty(outer, inner // (2 if fmt == NVFP4 else 1), dtype=torch.uint8, device=device)
        assert values.numel() == vb
        make = torch.zeros if zero_scales else torch.empty
        return MxTensor(values, make(sb, dtype=torch.uint8, device=device), dim, rows, cols, fmt)

    def transposed(self) -> "MxTensor":
        """The same buffers seen as the transposed logical matrix: a rowwise [r, c] tensor is a
        colwise [c, r] tensor (`into_transposed`, crates/cleandl/tests/matmul.rs:939-943)."""
        return MxTensor(self.values, self.scale_factors, COLWISE if self.dim == ROWWISE else ROWWISE,
                        self.cols, self.rows, self.format)

    def arg(self) -> CdlMxTensor:
        return CdlMxTensor(self.values.data_ptr(), self.scale_factors.data_ptr(), self.format, self.dim,
                           self.rows, self.cols)


def _mx_arg(t: Optional[MxTensor]):
    return None if t is None else t.arg()


def quantize(x: torch.Tensor, rowwise: bool = True, colwise: bool = False, fmt: int = MXFP8,
             out=None):
    """bf16 [rows, cols] -> (rowwise MxTensor or None, colwise MxTensor or None).  NVFP4 has the
    rowwise form only; a colwise NVFP4 operand is `quantize(x.T.contiguous(), fmt=NVFP4)[0].transposed()`.
    `out` = (rowwise, colwise) of an earlier call reuses those buffers."""
    if not x.is_cuda:
        raise _lib.CdlError(-1, "operands must live in device memory (there is no CPU path)")
    rows, cols = x.shape
    if out is not None:
        yr, yc = out
    else:
        yr = MxTensor.empty(rows, cols, ROWWISE, x.device, zero_scales=True, fmt=fmt) if rowwise else None
        yc = MxTensor.empty(rows, cols, COLWISE, x.device, zero_scales=True, fmt=fmt) if colwise else None
    tx, ar, ac = tensor_arg(x), _mx_arg(yr), _mx_arg(yc)
    check(lib.cdl_b200_mx_quantize(ref(tx), ref(ar), ref(ac), _stream()))
    return yr, yc


def dequantize(t: MxTensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    y = torch.empty(t.rows, t.cols, dtype=dtype, device=t.values.device)
    a, ty = t.arg(), tensor_arg(y)
    check(lib.cdl_b200_mx_dequantize(ref(a), ref(ty), _stream()))
    return y


@dataclass
class NormMxOutputs:
    y: MxTensor
    y_col: Optional[MxTensor]
    r_inv: Optional[torch.Tensor]


def norm_fwd_mx(x: torch.Tensor, scale: Optional[torch.Tensor] = None,
                bias: Optional[torch.Tensor] = None, eps: float = 1e-6, colwise: bool = False,
                save_stats: bool = False, out: Optional[NormMxOutputs] = None,
                fmt: int = MXFP8) -> NormMxOutputs:
    """RMSNorm forward with `NormOutput::Mxfp8Rowwise` (or `...RowwiseAndColwise`) outputs, or with
    `NormOutput::Nvfp4Rowwise` (`fmt=NVFP4`).
    `out` reuses the buffers of an earlier call (the engine's pre-allocated outputs)."""
    if not x.is_cuda:
        raise _lib.CdlError(-1, "operands must live in device memory (there is no CPU path)")
    if x.dim() != 2:
        raise _lib.CdlError(-1, f"norm input must be a 2D tensor, got rank {x.dim()}")
    rows, cols = x.shape
    if out is not None:
        yr, yc, r_inv = out.y, out.y_col, out.r_inv
    else:
        yr = MxTensor.empty(rows, cols, ROWWISE, x.device, zero_scales=True, fmt=fmt)
        yc = MxTensor.empty(rows, cols, COLWISE, x.device, zero_scales=True, fmt=fmt) if colwise else None
        r_inv = torch.empty(rows, dtype=torch.float32, device=x.device) if save_stats else None
    tx, ts, tb, tr = tensor_arg(x), tensor_arg(scale), tensor_arg(bias), tensor_arg(r_inv)
    ar, ac = _mx_arg(yr), _mx_arg(yc)
    check(lib.cdl_b200_rmsnorm_fwd_mx(ref(tx), ref(ts), ref(tb), eps, ref(ar), ref(ac), ref(tr),
                                      _stream()))
    return NormMxOutputs(yr, yc, r_inv)


def matmul_mx(a: MxTensor, b: MxTensor, out_dtype: torch.dtype = torch.bfloat16, alpha: float = 1.0,
              out: Optional[torch.Tensor] = None, c: Optional[torch.Tensor] = None,
              beta: float = 0.0, variant: int = 0) -> torch.Tensor:
    """D = alpha * A . B + beta * C for a rowwise A [M, K] and a colwise B [K, N]; `c` may be `out`
    (accumulation in place).  `variant`: cdl_gemm_variant (0 = the library's heuristic)."""
    if out is None:
        out = torch.empty(a.rows, b.cols, dtype=out_dtype, device=a.values.device)
    aa, ab, tc, td = a.arg(), b.arg(), tensor_arg(c), tensor_arg(out)
    if variant != 0:
        import ctypes

        from ._lib import CdlMatmulOptions
        mo = CdlMatmulOptions(int(variant), 0)
        check(lib.cdl_b200_matmul_mx_opt(ref(aa), ref(ab), ref(tc), ref(td), alpha, beta,
                                         ctypes.byref(mo), _stream()))
        return out
    check(lib.cdl_b200_matmul_mx(ref(aa), ref(ab), ref(tc), ref(td), alpha, beta, _stream()))
    return out


def matmul_mx_out(a: MxTensor, b: MxTensor, dim: int = ROWWISE, alpha: float = 1.0,
                  out: Optional[MxTensor] = None, fmt: int = MXFP8) -> MxTensor:
    """The same product with `MatmulOutput::BlockScaled { format, dim }`: a block-scaled [M, N] result."""
    if out is None:
        out = MxTensor.empty(a.rows, b.cols, dim, a.values.device, zero_scales=True, fmt=fmt)
    aa, ab, ad = a.arg(), b.arg(), out.arg()
    check(lib.cdl_b200_matmul_mx_out(ref(aa), ref(ab), ref(ad), alpha, _stream()))
    return out
