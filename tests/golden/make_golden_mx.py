"""Generates tests/golden/mx.npz: block-scaled (MXFP8, NVFP4) quantisations of a seeded matrix
computed with torch alone -- float8_e4m3fn casts for the E4M3 roundings, torch.frexp for the power
of two, a sort-free nearest search for E2M1 -- an implementation independent of
oracle/mx_ref.py, which the CPU tests compare against this file (values, scales in the tiled
layout, dequantised matrix).

The reference holds no stored vectors for this format (its tests quantise random matrices at run
time, crates/cleandl/tests/matmul.rs:885-952), so the fixture pins the oracle to a second
implementation.  Run from the repository root:  python tests/golden/make_golden_mx.py
"""
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent


def sf_offsets(outer, blocks):
    o = torch.arange(outer).view(-1, 1)
    b = torch.arange(blocks).view(1, -1)
    tiles = (blocks + 3) // 4
    return ((o // 128) * tiles + b // 4) * 512 + (o % 32) * 16 + ((o % 128) // 32) * 4 + b % 4


def mxfp8(m, colwise):
    src = (m.T if colwise else m).contiguous()
    outer, inner = src.shape
    blk = src.view(outer, inner // 32, 32)
    amax = blk.abs().amax(dim=2)
    # smallest power of two s with amax / s <= 448:  amax / 448 = f * 2^e with f in [0.5, 1)
    f, e = torch.frexp(amax / 448.0)
    exp = torch.where(f == 0.5, e - 1, e)          # an exact power of two needs no rounding up
    exp = torch.where(amax == 0, torch.full_like(exp, -127), exp).clamp(-127, 127)
    scale = torch.exp2(exp.to(torch.float64))
    vals = (blk.to(torch.float64) / scale.unsqueeze(2)).to(torch.float32).to(torch.float8_e4m3fn)
    values = vals.view(torch.uint8).view(outer, inner)
    sf = torch.zeros(((outer + 127) // 128 * 128) * ((inner // 32 + 3) // 4 * 4), dtype=torch.uint8)
    sf[sf_offsets(outer, inner // 32).reshape(-1)] = (exp + 127).to(torch.uint8).reshape(-1)
    deq = (vals.to(torch.float64) * scale.unsqueeze(2)).view(outer, inner)
    return values.numpy(), sf.numpy(), (deq.T if colwise else deq).contiguous().to(torch.float32).numpy()


E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=torch.float64)


def e2m1_codes(q):
    a = q.abs().clamp(max=6.0).to(torch.float64)
    dist = (a.unsqueeze(-1) - E2M1).abs()
    best = dist.min(dim=-1, keepdim=True).values
    tie = dist == best                                   # one or two candidates
    idx = torch.arange(8).expand_as(dist)
    even_first = torch.where(tie & (idx % 2 == 0), idx, torch.where(tie, idx + 100, idx + 1000))
    code = even_first.min(dim=-1).values % 100           # ties go to the even code
    return (code + 8 * (torch.signbit(q)).to(torch.int64)).to(torch.uint8)


def nvfp4(m):
    outer, inner = m.shape
    blk = m.view(outer, inner // 16, 16)
    amax = blk.abs().amax(dim=2)
    s8 = (amax / 6.0).to(torch.float32).clamp(max=448.0).to(torch.float8_e4m3fn)  # satfinite
    scale = s8.to(torch.float32)
    inv = torch.where(scale == 0, torch.zeros_like(scale), 1.0 / scale)  # correctly rounded f32
    q = blk * inv.unsqueeze(2)
    codes = e2m1_codes(q.to(torch.float32)).view(outer, inner)
    values = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    sf = torch.zeros(((outer + 127) // 128 * 128) * ((inner // 16 + 3) // 4 * 4), dtype=torch.uint8)
    sf[sf_offsets(outer, inner // 16).reshape(-1)] = s8.view(torch.uint8).reshape(-1)
    mag = E2M1[(codes & 7).long()] * torch.where((codes & 8) != 0, -1.0, 1.0)
    deq = (mag.view(outer, inner // 16, 16) * scale.to(torch.float64).unsqueeze(2)).view(outer, inner)
    return values.numpy(), sf.numpy(), deq.to(torch.float32).numpy()


def main():
    gen = torch.Generator().manual_seed(20241)
    m = torch.randn(160, 96, generator=gen) * torch.exp(torch.randn(160, 96, generator=gen) * 2.0)
    m = m.to(torch.bfloat16).to(torch.float32)
    m[0, :32] = 0.0          # an all-zero block
    m[1, :32] = 448.0        # amax = 448 * 2^0 exactly
    m[2, 0] = 3.0e38         # close to the largest finite bf16
    rv, rs, rd = mxfp8(m, colwise=False)
    cv, cs, cd = mxfp8(m, colwise=True)
    nv, ns, nd = nvfp4(m)
    np.savez_compressed(OUT / "mx.npz", m=m.numpy(), row_values=rv, row_scales=rs, row_deq=rd,
                        col_values=cv, col_scales=cs, col_deq=cd, nv_values=nv, nv_scales=ns, nv_deq=nd)
    print("wrote", OUT / "mx.npz")


if __name__ == "__main__":
    main()
