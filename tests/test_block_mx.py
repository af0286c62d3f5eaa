"""sky-1 block with MXFP8 matrix products against the bf16 block of this library on the same
inputs: outputs, input gradient and every weight gradient agree within the error of the format.
E4M3 keeps three mantissa bits: an element's relative rounding error is uniform in +-2^-4, about
3.6e-2 rms; a product of two quantised operands carries 5e-2, and a sum of such products of random
sign keeps that RELATIVE error (signal and error both grow like sqrt(K)).  One GEMM therefore sits
near 5e-2 against its bf16 twin, a chain of them (the gradients) near 1e-1; the bounds below are
twice those figures.  The bf16 block itself is held to the f64 oracle elsewhere."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


@pytest.mark.parametrize("dims", [
    dict(batch=2, seqlen=256, hidden=256, heads=2, kv_heads=2, head_dim=128, ffn=512),
    dict(batch=1, seqlen=512, hidden=512, heads=4, kv_heads=2, head_dim=128, ffn=1024),
])
def test_mx_block_tracks_bf16_block(cdl, gpu_ok, dims):
    cfg = cdl.sky1.Sky1Config(**dims)
    params = cdl.sky1.init_params(cfg, 3, std=0.05)
    gen = torch.Generator().manual_seed(5)
    params["norm1"] = (1 + 0.1 * torch.randn(cfg.hidden, generator=gen)).to(torch.bfloat16)
    params["norm2"] = (1 + 0.1 * torch.randn(cfg.hidden, generator=gen)).to(torch.bfloat16)
    x = torch.randn(cfg.tokens, cfg.hidden, generator=gen).to(torch.bfloat16).cuda()
    dy = torch.randn(cfg.tokens, cfg.hidden, generator=gen).to(torch.bfloat16).cuda()
    ref_blk = cdl.sky1.Sky1Block(cfg, params)
    mx_blk = cdl.sky1_mx.Sky1BlockMX(cfg, params)
    y_ref, y_mx = ref_blk.forward(x), mx_blk.forward(x)
    dx_ref, dx_mx = ref_blk.backward(dy), mx_blk.backward(dy)
    torch.cuda.synchronize()
    print({"y": rel(y_mx, y_ref), "dx": rel(dx_mx, dx_ref),
           **{n: rel(mx_blk.grads[n], ref_blk.grads[n]) for n in mx_blk.grads}})
    assert torch.isfinite(y_mx.float()).all() and torch.isfinite(dx_mx.float()).all()
    assert rel(y_mx, y_ref) < 0.10, rel(y_mx, y_ref)
    assert rel(dx_mx, dx_ref) < 0.20, rel(dx_mx, dx_ref)
    for name in ("wqkv", "wo", "wup", "wgate", "wdown", "norm1", "norm2"):
        r = rel(mx_blk.grads[name], ref_blk.grads[name])
        assert r < 0.20, (name, r)
    # gradients accumulate: a second backward doubles them
    g1 = {n: v.clone() for n, v in mx_blk.grads.items()}
    mx_blk.forward(x)
    mx_blk.backward(dy)
    torch.cuda.synchronize()
    for n, v in mx_blk.grads.items():
        assert rel(v, 2 * g1[n]) < 1e-3, n
