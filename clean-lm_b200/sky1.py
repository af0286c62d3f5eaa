"""sky-1 decoder block on the C ABI (host side of `cdl_b200_sky1_block_fwd/_bwd`).

Mirrors the reference's DecoderExecutor (crates/sky-1/src/training/model/decoder.rs:332-752):
parameters are bf16 replicas stored [in, out] with f32 gradients (parameter.rs:11-17), the forward
saves qkv / attn / lse / o / up / gate / act, and the backward accumulates weight gradients.
torch only owns the memory; every kernel is in libcleandl_b200.so.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import check, lib

PARAM_NAMES = _lib._BLOCK_PARAMS


@dataclass
class Sky1Config:
    batch: int = 8
    seqlen: int = 2048
    hidden: int = 2048
    heads: int = 16
    kv_heads: int = 16
    head_dim: int = 128
    ffn: int = 5632
    eps: float = 1e-6
    rope_base: float = 10000.0

    @property
    def tokens(self) -> int:
        return self.batch * self.seqlen

    @property
    def qkv_dim(self) -> int:
        return (self.heads + 2 * self.kv_heads) * self.head_dim

    def param_shapes(self) -> dict:
        hd = self.heads * self.head_dim
        return {"norm1": (self.hidden,), "wqkv": (self.hidden, self.qkv_dim), "wo": (hd, self.hidden),
                "norm2": (self.hidden,), "wup": (self.hidden, self.ffn),
                "wgate": (self.hidden, self.ffn), "wdown": (self.ffn, self.hidden)}

    def param_count(self) -> int:
        return sum(math.prod(s) for s in self.param_shapes().values())

    def c_struct(self) -> _lib.CdlSky1Config:
        return _lib.CdlSky1Config(self.batch, self.seqlen, self.hidden, self.heads, self.kv_heads,
                                  self.head_dim, self.ffn, self.eps)

    def flops_fwd_bwd(self) -> float:
        """Algorithmic FLOP of one block forward + backward: 3 x the five GEMMs' 2MNK plus causal
        attention forward (4 B H S^2 D / 2) and backward (2.5 x forward)."""
        t, hd = self.tokens, self.heads * self.head_dim
        gemm = 2.0 * t * (self.hidden * self.qkv_dim + hd * self.hidden + 3 * self.hidden * self.ffn)
        attn = 4.0 * self.batch * self.heads * self.seqlen ** 2 * self.head_dim / 2
        return 3 * gemm + 3.5 * attn


def rope_table(seqlen: int, head_dim: int, base: float = 10000.0, device="cuda") -> torch.Tensor:
    """f32 [seqlen, head_dim] = cos | sin of pos * base^(-2i/D) (rotate-half convention)."""
    half = head_dim // 2
    inv_freq = base ** (-torch.arange(half, dtype=torch.float64) * 2.0 / head_dim)
    ang = torch.arange(seqlen, dtype=torch.float64)[:, None] * inv_freq[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=1).to(torch.float32).to(device)


def init_params(cfg: Sky1Config, seed: int, std: float = 0.02) -> dict:
    """bf16 weights ~ N(0, std) and norm gains = 1, generated on the CPU from `seed`."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in cfg.param_shapes().items():
        if name.startswith("norm"):
            out[name] = torch.ones(shape, dtype=torch.bfloat16)
        else:
            out[name] = (torch.randn(shape, generator=gen) * std).to(torch.bfloat16)
    return out


class Sky1Block:
    """One decoder block: device weights, f32 gradient buffers, saved activations."""

    def __init__(self, cfg: Sky1Config, params: dict, device="cuda", grads: dict | None = None,
                 workspace: torch.Tensor | None = None, table: torch.Tensor | None = None):
        self.cfg = cfg
        self.device = device
        self.params = {n: params[n].to(device=device, dtype=torch.bfloat16).contiguous()
                       for n in PARAM_NAMES}
        for n, shape in cfg.param_shapes().items():
            if tuple(self.params[n].shape) != tuple(shape):
                raise _lib.CdlError(-1, f"parameter {n} must have shape {shape}")
        # Gradients may be views into a caller-owned flat bucket (see the data-parallel step).
        self.grads = grads if grads is not None else {
            n: torch.zeros(s, dtype=torch.float32, device=device) for n, s in cfg.param_shapes().items()}
        t = cfg.tokens
        bf = dict(dtype=torch.bfloat16, device=device)
        self.saved = {
            "qkv": torch.empty(t, cfg.qkv_dim, **bf),
            "attn": torch.empty(t, cfg.heads * cfg.head_dim, **bf),
            "lse": torch.empty(cfg.batch, cfg.heads, cfg.seqlen, dtype=torch.float32, device=device),
            "o": torch.empty(t, cfg.hidden, **bf),
            "up": torch.empty(t, cfg.ffn, **bf),
            "gate": torch.empty(t, cfg.ffn, **bf),
            "act": torch.empty(t, cfg.ffn, **bf),
        }
        self.table = table if table is not None else rope_table(cfg.seqlen, cfg.head_dim,
                                                                 cfg.rope_base, device)
        self._cfg_c = cfg.c_struct()
        fwd, bwd = ctypes.c_size_t(0), ctypes.c_size_t(0)
        check(lib.cdl_b200_sky1_block_workspace_bytes(ctypes.byref(self._cfg_c), ctypes.byref(fwd),
                                                      ctypes.byref(bwd)))
        self.workspace_bytes = max(fwd.value, bwd.value)
        self.workspace = workspace if workspace is not None else torch.empty(
            self.workspace_bytes, dtype=torch.uint8, device=device)
        if self.workspace.numel() < self.workspace_bytes:
            raise _lib.CdlError(-1, f"workspace must hold {self.workspace_bytes} bytes")
        self._w_c = _lib.CdlSky1Weights(*(self.params[n].data_ptr() for n in PARAM_NAMES))
        self._g_c = _lib.CdlSky1Grads(*(self.grads[n].data_ptr() for n in PARAM_NAMES))
        self._s_c = _lib.CdlSky1Saved(*(self.saved[n].data_ptr()
                                        for n in ("qkv", "attn", "lse", "o", "up", "gate", "act")))
        self._x = None

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """x: bf16 [tokens, hidden] (or [batch, seqlen, hidden]); keeps a reference for backward."""
        cfg = self.cfg
        if x.dtype != torch.bfloat16 or x.numel() != cfg.tokens * cfg.hidden or not x.is_contiguous():
            raise _lib.CdlError(-1, "x must be a contiguous bf16 tensor of [tokens, hidden]")
        out = torch.empty_like(x) if out is None else out
        check(lib.cdl_b200_sky1_block_fwd(
            ctypes.byref(self._cfg_c), ctypes.byref(self._w_c), x.data_ptr(), self.table.data_ptr(),
            ctypes.byref(self._s_c), out.data_ptr(), self.workspace.data_ptr(),
            self.workspace.numel(), self._stream()))
        self._x = x
        return out

    def backward(self, dy: torch.Tensor, dx: torch.Tensor | None = None, phase: int = 0) -> torch.Tensor:
        """dy: gradient of the forward's output. Accumulates into self.grads; returns dx.
        phase 1 / 2 run the FFN half / the attention half (see cdl_b200_sky1_block_bwd)."""
        if self._x is None:
            raise _lib.CdlError(-1, "backward called before forward")
        if dy.dtype != torch.bfloat16 or dy.numel() != self._x.numel() or not dy.is_contiguous():
            raise _lib.CdlError(-1, "dy must be a contiguous bf16 tensor shaped like x")
        dx = torch.empty_like(dy) if dx is None else dx
        check(lib.cdl_b200_sky1_block_bwd(
            ctypes.byref(self._cfg_c), ctypes.byref(self._w_c), self._x.data_ptr(),
            self.table.data_ptr(), ctypes.byref(self._s_c), dy.data_ptr(), ctypes.byref(self._g_c),
            dx.data_ptr(), self.workspace.data_ptr(), self.workspace.numel(), phase, self._stream()))
        return dx

    def zero_grads(self):
        for g in self.grads.values():
            g.zero_()
