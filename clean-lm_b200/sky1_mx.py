"""sky-1 decoder block with MXFP8 matrix products: the bf16 block's dataflow
(crates/sky-1/src/training/model/decoder.rs:332-695) with every GEMM operand block-scaled.

The reference has no such block (its decoder is bf16); this module composes the reference's own
block-scaled operators the way its kernels are laid out to be used -- RMSNorm writes MXFP8 rowwise
and colwise outputs (`NormOutput::Mxfp8RowwiseAndColwise`), matmuls take block-scaled inputs
(`InputKind::Mx`) -- so that the row is measured end to end.  Everything between the products stays
bf16 (RoPE, attention, SwiGLU, norm backward), residual adds ride in the products' epilogues
(`c`, `beta`), weight gradients accumulate in f32 in place.

Which quantisation a product needs (blocks run along its contraction dimension):
  forward   Y[T,N]  = X[T,K] . W[K,N]         X rowwise,            W colwise
  dgrad     dX[T,K] = dY[T,N] . W^T[N,K]      dY rowwise,           W^T colwise = W rowwise, transposed view
  wgrad     dW[K,N] = X^T[K,T] . dY[T,N]      X^T rowwise = X colwise, transposed view;  dY colwise
Weights are quantised both ways once per optimizer step (`requantize_weights`), activations and
gradients once where they are produced.  Experimental: numerics are those of MXFP8, not of the
bf16 block; tests hold it to the bf16 block within the format's error.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib, mx, ops
from ._lib import check, lib, ref, tensor_arg
from .sky1 import Sky1Config, rope_table

WEIGHTS = ("wqkv", "wo", "wup", "wgate", "wdown")


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class Sky1BlockMX:
    def __init__(self, cfg: Sky1Config, params: dict, device="cuda"):
        self.cfg = cfg
        self.device = device
        self.params = {n: params[n].to(device=device, dtype=torch.bfloat16).contiguous() for n in params}
        self.grads = {n: torch.zeros(s, dtype=torch.float32, device=device)
                      for n, s in cfg.param_shapes().items()}
        self.table = rope_table(cfg.seqlen, cfg.head_dim, cfg.rope_base, device)
        t, h, f, q = cfg.tokens, cfg.hidden, cfg.ffn, cfg.qkv_dim
        hd = cfg.heads * cfg.head_dim
        bf = dict(dtype=torch.bfloat16, device=device)
        self.buf = {
            "qkv": torch.empty(t, q, **bf), "attn": torch.empty(t, hd, **bf), "o": torch.empty(t, h, **bf),
            "up": torch.empty(t, f, **bf), "gate": torch.empty(t, f, **bf), "act": torch.empty(t, f, **bf),
            "d_act": torch.empty(t, f, **bf), "d_gate": torch.empty(t, f, **bf), "dh": torch.empty(t, h, **bf),
            "d_o": torch.empty(t, h, **bf), "d_attn": torch.empty(t, hd, **bf), "d_qkv": torch.empty(t, q, **bf),
        }
        self.r_inv = {1: torch.empty(t, dtype=torch.float32, device=device),
                      2: torch.empty(t, dtype=torch.float32, device=device)}

        def pair(rows, cols):  # rowwise and colwise MXFP8 buffers of a [rows, cols] tensor
            return (mx.MxTensor.empty(rows, cols, mx.ROWWISE, device, zero_scales=True),
                    mx.MxTensor.empty(rows, cols, mx.COLWISE, device, zero_scales=True))

        self.q = {"h1": pair(t, h), "attn": pair(t, hd), "h2": pair(t, h), "act": pair(t, f),
                  "dy": pair(t, h), "d_up": pair(t, f), "d_gate": pair(t, f), "d_o": pair(t, h),
                  "d_qkv": pair(t, q)}
        self.wq = {n: pair(*self.params[n].shape) for n in WEIGHTS}
        self.requantize_weights()
        self.norm_scratch = torch.empty(ops.norm_bwd_scratch_bytes(t, h), dtype=torch.uint8, device=device)
        qv = self.buf["qkv"].view(cfg.batch, cfg.seqlen, cfg.heads + 2 * cfg.kv_heads, cfg.head_dim)
        self._q, self._k, self._v = (qv[:, :, :cfg.heads], qv[:, :, cfg.heads:cfg.heads + cfg.kv_heads],
                                     qv[:, :, cfg.heads + cfg.kv_heads:])
        self.attn_scratch = torch.empty(ops.attention_bwd_scratch_bytes(self._q, self._k), dtype=torch.uint8,
                                        device=device)
        self.lse = None
        self._x = None

    # ------------------------------------------------------------------ helpers
    def requantize_weights(self):
        """MXFP8 copies of the bf16 weights, both ways; call after every optimizer step."""
        for n in WEIGHTS:
            mx.quantize(self.params[n], rowwise=True, colwise=True, out=self.wq[n])

    def _rope(self, x2d, backward: int):
        cfg = self.cfg
        x3 = x2d.view(cfg.tokens, cfg.heads + 2 * cfg.kv_heads, cfg.head_dim)
        tx, tt = tensor_arg(x3), tensor_arg(self.table)
        check(lib.cdl_b200_rope(ref(tx), ref(tt), cfg.heads + cfg.kv_heads, cfg.seqlen, backward, _stream()))

    def _quant(self, name, x):
        mx.quantize(x, rowwise=True, colwise=True, out=self.q[name])
        return self.q[name]

    @staticmethod
    def _fwd(x_row, w_pair, out, c=None):       # Y = X . W (+ C)
        return mx.matmul_mx(x_row, w_pair[1], out=out, c=c, beta=1.0 if c is not None else 0.0)

    @staticmethod
    def _dgrad(dy_row, w_pair, out, c=None):    # dX = dY . W^T (+ C)
        return mx.matmul_mx(dy_row, w_pair[0].transposed(), out=out, c=c, beta=1.0 if c is not None else 0.0)

    @staticmethod
    def _wgrad(x_col, dy_col, grad):            # dW += X^T . dY
        return mx.matmul_mx(x_col.transposed(), dy_col, out=grad, c=grad, beta=1.0)

    # ------------------------------------------------------------------ forward / backward
    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        cfg, b, p = self.cfg, self.buf, self.params
        out = torch.empty_like(x) if out is None else out
        self._x = x
        n1 = mx.norm_fwd_mx(x, p["norm1"], eps=cfg.eps, colwise=True, save_stats=True,
                            out=mx.NormMxOutputs(*self.q["h1"], self.r_inv[1]))
        self._fwd(n1.y, self.wq["wqkv"], b["qkv"])
        self._rope(b["qkv"], 0)
        att = ops.attention_fwd(self._q, self._k, self._v, ops.AttentionOpts(causal=True),
                                out=b["attn"].view(cfg.batch, cfg.seqlen, cfg.heads, cfg.head_dim))
        self.lse = att.lse
        qa = self._quant("attn", b["attn"])
        self._fwd(qa[0], self.wq["wo"], b["o"], c=x)                       # o = attn Wo + x
        n2 = mx.norm_fwd_mx(b["o"], p["norm2"], eps=cfg.eps, colwise=True, save_stats=True,
                            out=mx.NormMxOutputs(*self.q["h2"], self.r_inv[2]))
        self._fwd(n2.y, self.wq["wup"], b["up"])
        self._fwd(n2.y, self.wq["wgate"], b["gate"])
        tg, tu, ta = tensor_arg(b["gate"]), tensor_arg(b["up"]), tensor_arg(b["act"])
        check(lib.cdl_b200_swiglu_fwd(ref(tg), ref(tu), ref(ta), _stream()))
        qact = self._quant("act", b["act"])
        self._fwd(qact[0], self.wq["wdown"], out, c=b["o"])                # out = act Wdown + o
        return out

    def backward(self, dy: torch.Tensor, dx: torch.Tensor | None = None) -> torch.Tensor:
        cfg, b, p, g = self.cfg, self.buf, self.params, self.grads
        dx = torch.empty_like(dy) if dx is None else dx
        qdy = self._quant("dy", dy)
        self._wgrad(self.q["act"][1], qdy[1], g["wdown"])
        self._dgrad(qdy[0], self.wq["wdown"], b["d_act"])
        targs = [tensor_arg(t) for t in (b["d_act"], b["gate"], b["up"], b["d_gate"], b["d_act"])]
        check(lib.cdl_b200_swiglu_bwd(*(ref(a) for a in targs), _stream()))   # d_up over d_act
        qdu, qdg = self._quant("d_up", b["d_act"]), self._quant("d_gate", b["d_gate"])
        self._wgrad(self.q["h2"][1], qdu[1], g["wup"])
        self._wgrad(self.q["h2"][1], qdg[1], g["wgate"])
        self._dgrad(qdu[0], self.wq["wup"], b["dh"])
        self._dgrad(qdg[0], self.wq["wgate"], b["dh"], c=b["dh"])
        ops.norm_bwd(b["o"], b["dh"], p["norm2"], self.r_inv[2], g["norm2"], residual_dy=dy,
                     scratch=self.norm_scratch, dx=b["d_o"])
        qdo = self._quant("d_o", b["d_o"])
        self._wgrad(self.q["attn"][1], qdo[1], g["wo"])
        self._dgrad(qdo[0], self.wq["wo"], b["d_attn"])
        dqv = b["d_qkv"].view(cfg.batch, cfg.seqlen, cfg.heads + 2 * cfg.kv_heads, cfg.head_dim)
        h, kv = cfg.heads, cfg.kv_heads
        ops.attention_bwd(self._q, self._k, self._v, b["attn"].view(cfg.batch, cfg.seqlen, h, cfg.head_dim),
                          b["d_attn"].view(cfg.batch, cfg.seqlen, h, cfg.head_dim), self.lse,
                          ops.AttentionOpts(causal=True), scratch=self.attn_scratch,
                          dq=dqv[:, :, :h], dk=dqv[:, :, h:h + kv], dv=dqv[:, :, h + kv:])
        self._rope(b["d_qkv"], 1)
        qdq = self._quant("d_qkv", b["d_qkv"])
        self._wgrad(self.q["h1"][1], qdq[1], g["wqkv"])
        self._dgrad(qdq[0], self.wq["wqkv"], b["dh"])
        ops.norm_bwd(self._x, b["dh"], p["norm1"], self.r_inv[1], g["norm1"], residual_dy=b["d_o"],
                     scratch=self.norm_scratch, dx=dx)
        return dx

    def zero_grads(self):
        for v in self.grads.values():
            v.zero_()
