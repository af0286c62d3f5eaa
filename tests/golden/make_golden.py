"""Generates tests/golden/*.npz: seeded inputs and float64 results of the hot-path operators,
computed with torch (autograd for the gradients) — an implementation independent of the C oracle
in oracle/cpu_ref.c, which the CPU tests compare against these files.

The reference project ships no golden vectors of its own (its tests draw inputs from Rust RNG
streams at run time and compare with in-test f64 references), and it cannot be built in this
environment, so these fixtures pin the oracle to a second implementation rather than to reference
outputs.  Run from the repository root:  python tests/golden/make_golden.py
"""
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent


def bf16(t):
    return t.to(torch.bfloat16).to(torch.float64)


def main():
    gen = torch.Generator().manual_seed(20240)
    # matmul with alpha / beta / C  (shape of the reference's odd-sized case 129 x 264 x 72)
    a, b, c = bf16(torch.rand(129, 264, generator=gen) * 2 - 1), bf16(torch.rand(264, 72, generator=gen) * 2 - 1), \
        bf16(torch.rand(129, 72, generator=gen) * 2 - 1)
    np.savez_compressed(OUT / "matmul.npz", a=a.float().numpy(), b=b.float().numpy(), c=c.float().numpy(),
                        alpha=np.float32(0.5), beta=np.float32(-2.0),
                        out=(0.5 * a @ b - 2.0 * c).float().numpy())
    # rmsnorm forward / backward
    rows, cols, eps = 37, 136, 1e-6
    x = bf16(torch.randn(rows, cols, generator=gen) * 2 + 0.5).requires_grad_(True)
    scale = bf16(torch.rand(cols, generator=gen) + 0.5).requires_grad_(True)
    bias = bf16(torch.randn(cols, generator=gen))
    dy = bf16(torch.randn(rows, cols, generator=gen))
    r = torch.rsqrt((x * x).mean(1, keepdim=True) + eps)
    y = x * r * scale
    y.backward(dy)
    np.savez_compressed(OUT / "rmsnorm.npz", x=x.detach().float().numpy(), scale=scale.detach().float().numpy(),
                        bias=bias.float().numpy(), dy=dy.float().numpy(), eps=np.float32(eps),
                        y=(y.detach() + bias).float().numpy(), r_inv=r.detach().squeeze(1).float().numpy(),
                        dx=x.grad.float().numpy(), dscale=scale.grad.numpy())
    # attention forward / backward, GQA, sq < sk, bottom-right aligned causal mask
    B, sq, sk, hq, hk, d = 1, 40, 72, 2, 1, 128
    q = bf16(torch.randn(B, sq, hq, d, generator=gen)).requires_grad_(True)
    k = bf16(torch.randn(B, sk, hk, d, generator=gen)).requires_grad_(True)
    v = bf16(torch.randn(B, sk, hk, d, generator=gen)).requires_grad_(True)
    do = bf16(torch.randn(B, sq, hq, d, generator=gen))
    kk, vv = k.repeat_interleave(hq // hk, 2), v.repeat_interleave(hq // hk, 2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, kk) / d ** 0.5
    i, j = torch.arange(sq)[:, None], torch.arange(sk)[None, :]
    s = s.masked_fill(j > i + sk - sq, float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vv)
    o.backward(do)
    np.savez_compressed(OUT / "attention.npz", q=q.detach().float().numpy(), k=k.detach().float().numpy(),
                        v=v.detach().float().numpy(), d_out=do.float().numpy(), out=o.detach().float().numpy(),
                        lse=lse.detach().float().numpy(), dq=q.grad.float().numpy(), dk=k.grad.float().numpy(),
                        dv=v.grad.float().numpy())


if __name__ == "__main__":
    main()
