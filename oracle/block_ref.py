"""TEST INFRASTRUCTURE — float64 restatement of the sky-1 decoder block (forward + autograd).

Follows the dataflow of the reference's DecoderExecutor (crates/sky-1/src/training/model/
decoder.rs: train_forward :332-520, train_backward :523-695).  PARITY UNPINNED: that code is dead
in the reference (it calls an operator module that is not in the tree), its RoPE / RMSNorm-backward /
SwiGLU kernels have no source and no tests, so this file follows the textbook math (rotate-half
RoPE with base 10000, SiLU gate) and the call-site order only.  Used by tests, the smoke check and
the bench's CPU legs; never by the product.
"""
from __future__ import annotations

import math

import torch


def rope_table(seqlen: int, head_dim: int, base: float = 10000.0) -> torch.Tensor:
    """f32 [seqlen, head_dim]: cos(pos * base^(-2i/D)) for i < D/2, then sin of the same angles."""
    half = head_dim // 2
    inv_freq = base ** (-torch.arange(half, dtype=torch.float64) * 2.0 / head_dim)
    ang = torch.arange(seqlen, dtype=torch.float64)[:, None] * inv_freq[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=1).to(torch.float32)


def rope(x: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x [B, S, heads, D]; rotate-half convention."""
    half = x.shape[-1] // 2
    cos = table[: x.shape[1], :half].to(x.dtype)[None, :, None, :]
    sin = table[: x.shape[1], half:].to(x.dtype)[None, :, None, :]
    lo, hi = x[..., :half], x[..., half:]
    return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], dim=-1)


def rmsnorm(x, gamma, eps):
    r = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * r * gamma


def attention(q, k, v, causal=True):
    """q [B, S, H, D], k/v [B, S, Hkv, D]; bottom-right aligned causal mask."""
    b, sq, h, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    k = k.repeat_interleave(h // hk, dim=2)
    v = v.repeat_interleave(h // hk, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, k) / math.sqrt(d)
    if causal:
        i = torch.arange(sq, device=q.device)[:, None]
        j = torch.arange(sk, device=q.device)[None, :]
        s = s.masked_fill(j > i + sk - sq, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhqk,bkhd->bqhd", p, v)


def block_forward(x, w, cfg, table, dtype=torch.float64):
    """x [B, S, hidden]; w: dict of tensors named like cdl_sky1_weights. Returns out [B, S, hidden]."""
    B, S, _ = x.shape
    H, Hkv, D = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    x = x.to(dtype)
    W = {k: v.to(dtype) for k, v in w.items()}
    h1 = rmsnorm(x, W["norm1"], cfg["eps"])
    qkv = (h1 @ W["wqkv"]).view(B, S, H + 2 * Hkv, D)
    q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]
    q, k = rope(q, table.to(dtype)), rope(k, table.to(dtype))
    attn = attention(q, k, v).reshape(B, S, H * D)
    o = attn @ W["wo"] + x
    h2 = rmsnorm(o, W["norm2"], cfg["eps"])
    up, gate = h2 @ W["wup"], h2 @ W["wgate"]
    act = torch.nn.functional.silu(gate) * up
    return act @ W["wdown"] + o


def block_forward_backward(x, w, dy, cfg, table, dtype=torch.float64):
    """Returns (out, dx, grads dict) computed with autograd in `dtype`."""
    xr = x.to(dtype).detach().requires_grad_(True)
    wr = {k: v.to(dtype).detach().requires_grad_(True) for k, v in w.items()}
    out = block_forward(xr, wr, cfg, table, dtype)
    out.backward(dy.to(dtype))
    return out.detach(), xr.grad, {k: v.grad for k, v in wr.items()}
