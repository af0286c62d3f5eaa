"""GPU parity of the sky-1 decoder block (forward + backward) against the float64 restatement of
the reference's dataflow (oracle/block_ref.py), on reduced dimensions the CPU finishes in seconds
(and once at the full size of benchmark configuration 4, with the same restatement run in f32 on
the device), and of the elementwise kernels it uses.  Bound: the acceptance bound of 2e-2 of the largest magnitude for bf16
tensors produced by chains of bf16 GEMMs; gradients likewise."""
import numpy as np
import pytest
import torch

from helpers import to_f32
from oracle import block_ref

pytestmark = pytest.mark.gpu


def rel_err(got, ref):
    ref = ref.double().cpu()
    return ((got.double().cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-12)).item()


def test_rope_forward_backward(cdl, gpu_ok):
    L = cdl._lib
    gen = torch.Generator().manual_seed(0)
    b, s, heads, d = 2, 96, 6, 128
    x = torch.randn(b * s, heads, d, generator=gen).to(torch.bfloat16)
    table = block_ref.rope_table(s, d)
    for backward in (0, 1):
        dev = x.cuda().clone()
        tx, tt = L.tensor_arg(dev), L.tensor_arg(table.cuda())
        L.check(L.lib.cdl_b200_rope(L.ref(tx), L.ref(tt), 4, s, backward, None))
        torch.cuda.synchronize()
        t = table.double() if backward == 0 else torch.cat([table[:, :64], -table[:, 64:]], 1).double()
        ref = block_ref.rope(x.double().view(b, s, heads, d)[:, :, :4], t).reshape(b * s, 4, d)
        assert rel_err(dev[:, :4], ref) <= 2.0 ** -7
        assert torch.equal(dev[:, 4:].cpu(), x[:, 4:])  # heads beyond rot_heads are untouched


@pytest.mark.parametrize("ragged", [False, True])
def test_matmul_with_rope_epilogue(cdl, gpu_ok, ragged):
    """cdl_b200_matmul_rope: the fused QKV projection with RoPE on the q and k heads applied in the
    GEMM's epilogue (the call sites it fuses: decoder.rs:350-378), against the f64 product rotated
    by the oracle; heads beyond rot_heads (v) must equal the plain product bit for bit."""
    L = cdl._lib
    gen = torch.Generator().manual_seed(12)
    bsz, s, hidden, heads, rot = 2, 200, 256, 5, 3   # tokens 400: a partial 256-row tile
    tokens = bsz * s
    x = torch.randn(tokens, hidden, generator=gen).to(torch.bfloat16)
    w = (torch.randn(hidden, heads * 128, generator=gen) * 0.1).to(torch.bfloat16)
    if ragged:
        lens = [130, 1, 200, 40]  # 371 tokens, then 29 rows of padding
        cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
        table = block_ref.rope_table(max(lens), 128)
        seqlen = max(lens)
    else:
        cu, table, seqlen = None, block_ref.rope_table(s, 128), s
    d = torch.empty(tokens, heads * 128, dtype=torch.bfloat16, device="cuda")
    dev = [x.cuda(), w.cuda(), table.cuda(), cu.cuda() if ragged else None]  # kept alive for the call
    args = [L.tensor_arg(t) for t in dev[:3]]
    tcu = L.tensor_arg(dev[3]) if ragged else None
    td = L.tensor_arg(d)
    L.check(L.lib.cdl_b200_matmul_rope(L.ref(args[0]), L.ref(args[1]), L.ref(args[2]), rot, seqlen,
                                       L.ref(tcu), L.ref(td), None))
    torch.cuda.synchronize()
    prod = (x.double() @ w.double()).view(tokens, heads, 128)
    ref = prod.clone()
    if ragged:
        for b in range(len(lens)):
            r0, r1 = int(cu[b]), int(cu[b + 1])
            ref[r0:r1, :rot] = block_ref.rope(prod[None, r0:r1, :rot], table.double())[0]
    else:
        ref[:, :rot] = block_ref.rope(prod.view(bsz, s, heads, 128)[:, :, :rot], table.double()).reshape(tokens, rot, 128)
    got = d.cpu().double().view(tokens, heads, 128)
    tol = 2.0 ** -8 * ref.abs() + 1e-5 * (x.double().abs() @ w.double().abs()).view(tokens, heads, 128) * 2 + 1e-6
    assert ((got - ref).abs() <= tol).all(), ((got - ref).abs() / tol).max()
    plain = cdl.ops.matmul(x.cuda(), w.cuda()).view(tokens, heads, 128)
    assert torch.equal(plain[:, rot:], d.view(tokens, heads, 128)[:, rot:])
    with pytest.raises(cdl._lib.CdlError, match="RoPE epilogue"):
        d2 = torch.empty(tokens, 200, dtype=torch.bfloat16, device="cuda")
        w2_dev = w.cuda()[:, :200].contiguous()
        w2 = L.tensor_arg(w2_dev)
        td2 = L.tensor_arg(d2)
        L.check(L.lib.cdl_b200_matmul_rope(L.ref(args[0]), L.ref(w2), L.ref(args[2]), 1, seqlen, None, L.ref(td2), None))


def test_swiglu_forward_backward(cdl, gpu_ok):
    L = cdl._lib
    gen = torch.Generator().manual_seed(1)
    n = (257, 264)
    gate, up, dact = (torch.randn(n, generator=gen).to(torch.bfloat16) for _ in range(3))
    g, u, da = gate.cuda(), up.cuda(), dact.cuda()
    act = torch.empty_like(g)
    args = [L.tensor_arg(t) for t in (g, u, act)]
    L.check(L.lib.cdl_b200_swiglu_fwd(*(L.ref(a) for a in args), None))
    gd, ud = gate.double().requires_grad_(True), up.double().requires_grad_(True)
    ref = torch.nn.functional.silu(gd) * ud
    ref.backward(dact.double())
    torch.cuda.synchronize()
    assert rel_err(act, ref.detach()) <= 2.0 ** -7
    dg, du = torch.empty_like(g), torch.empty_like(g)
    args = [L.tensor_arg(t) for t in (da, g, u, dg, du)]
    L.check(L.lib.cdl_b200_swiglu_bwd(*(L.ref(a) for a in args), None))
    torch.cuda.synchronize()
    assert rel_err(dg, gd.grad) <= 2.0 ** -7 and rel_err(du, ud.grad) <= 2.0 ** -7


@pytest.mark.parametrize("dims", [
    dict(batch=2, seqlen=256, hidden=256, heads=2, kv_heads=2, head_dim=128, ffn=512),
    dict(batch=1, seqlen=200, hidden=384, heads=4, kv_heads=2, head_dim=128, ffn=264),
])
def test_block_forward_backward_vs_oracle(cdl, gpu_ok, dims):
    sky1 = cdl.sky1
    cfg = sky1.Sky1Config(**dims)
    params = sky1.init_params(cfg, seed=3, std=0.05)
    gen = torch.Generator().manual_seed(3)
    params["norm1"] = (1 + 0.1 * torch.randn(cfg.hidden, generator=gen)).to(torch.bfloat16)
    params["norm2"] = (1 + 0.1 * torch.randn(cfg.hidden, generator=gen)).to(torch.bfloat16)
    x = torch.randn(cfg.tokens, cfg.hidden, generator=gen).to(torch.bfloat16)
    dy = torch.randn(cfg.tokens, cfg.hidden, generator=gen).to(torch.bfloat16)
    blk = sky1.Sky1Block(cfg, params)
    g0 = {n: torch.randn(g.shape, generator=gen) * 0.5 for n, g in blk.grads.items()}
    for n, g in blk.grads.items():
        g.copy_(g0[n])
    out = blk.forward(x.cuda())
    dx = blk.backward(dy.cuda())
    torch.cuda.synchronize()

    c = dict(heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim, eps=cfg.eps)
    table = block_ref.rope_table(cfg.seqlen, cfg.head_dim)
    shape3 = (cfg.batch, cfg.seqlen, cfg.hidden)
    out_ref, dx_ref, g_ref = block_ref.block_forward_backward(
        x.view(shape3), params, dy.view(shape3), c, table)
    assert rel_err(out, out_ref.reshape(cfg.tokens, -1)) <= 2e-2
    assert rel_err(dx, dx_ref.reshape(cfg.tokens, -1)) <= 2e-2
    for n in sky1.PARAM_NAMES:
        # gradients are accumulated on top of the buffers' previous contents
        got = blk.grads[n].double().cpu() - g0[n].double()
        err = ((got - g_ref[n]).abs().max() / g_ref[n].abs().max()).item()
        assert err <= 2e-2, (n, err)


def test_block_config4_full_size_vs_f32_on_device(cdl, gpu_ok):
    """Benchmark configuration 4 at its full size (8 x 2048 tokens, hidden 2048, 16 heads, ffn
    5632): the f64 oracle on the host would take minutes, so the same restatement runs in f32 on
    the device (torch, TF32 off) and the bounds are those of the small cases."""
    sky1 = cdl.sky1
    cfg = sky1.Sky1Config()
    assert (cfg.batch, cfg.seqlen, cfg.hidden, cfg.heads, cfg.ffn) == (8, 2048, 2048, 16, 5632)
    params = sky1.init_params(cfg, seed=3)
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(cfg.tokens, cfg.hidden, generator=gen).to(torch.bfloat16).cuda()
    dy = torch.randn(cfg.tokens, cfg.hidden, generator=gen).to(torch.bfloat16).cuda()
    blk = sky1.Sky1Block(cfg, params)
    for g in blk.grads.values():
        g.zero_()
    out = blk.forward(x)
    dx = blk.backward(dy)
    torch.cuda.synchronize()

    assert not torch.backends.cuda.matmul.allow_tf32
    c = dict(heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim, eps=cfg.eps)
    table = block_ref.rope_table(cfg.seqlen, cfg.head_dim).cuda()
    shape3 = (cfg.batch, cfg.seqlen, cfg.hidden)
    out_ref, dx_ref, g_ref = block_ref.block_forward_backward(
        x.view(shape3), {k: v.cuda() for k, v in params.items()}, dy.view(shape3), c, table,
        dtype=torch.float32)

    def err(got, ref):
        return ((got.float() - ref.float()).abs().max() / ref.float().abs().max()).item()

    assert err(out, out_ref.reshape(cfg.tokens, -1)) <= 2e-2
    assert err(dx, dx_ref.reshape(cfg.tokens, -1)) <= 2e-2
    for n in sky1.PARAM_NAMES:
        assert err(blk.grads[n], g_ref[n]) <= 2e-2, n


def test_block_backward_records_an_event_per_gradient_group(cdl, gpu_ok):
    """cdl_b200_sky1_block_bwd_events: the whole backward with one event per group of weight
    gradients.  A second stream that waits for a group's event and copies that group's gradients
    must see their final values (that is what a data-parallel caller's all-reduce relies on), and
    dx and the gradients equal the plain backward's bit for bit (fixed summation order)."""
    sky1 = cdl.sky1
    cfg = sky1.Sky1Config(deterministic=True, batch=2, seqlen=512, hidden=512, heads=4, kv_heads=4,
                          head_dim=128, ffn=1024)
    params = sky1.init_params(cfg, seed=12, std=0.05)
    x = torch.randn(cfg.tokens, cfg.hidden, generator=torch.Generator().manual_seed(13)).to(torch.bfloat16).cuda()
    dy = torch.randn(cfg.tokens, cfg.hidden, generator=torch.Generator().manual_seed(14)).to(torch.bfloat16).cuda()
    ref = sky1.Sky1Block(cfg, params)
    ref.zero_grads()
    ref.forward(x)
    dx_ref = ref.backward(dy)
    blk = sky1.Sky1Block(cfg, params)
    blk.zero_grads()
    blk.forward(x)
    events = [torch.cuda.Event() for _ in blk.GRAD_GROUPS]
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    dx = blk.backward(dy, events=events)
    early = {}
    with torch.cuda.stream(side):
        for ev, group in zip(events, blk.GRAD_GROUPS):
            side.wait_event(ev)
            for n in group:
                early[n] = blk.grads[n].clone()
    torch.cuda.synchronize()
    assert cdl._lib.device_status() == 0
    assert torch.equal(dx, dx_ref)
    assert sorted(early) == sorted(sky1.PARAM_NAMES)
    for n in sky1.PARAM_NAMES:
        assert torch.equal(blk.grads[n], ref.grads[n]), n
        assert torch.equal(early[n], ref.grads[n]), f"{n}: not final when its event fired"
    with pytest.raises(cdl._lib.CdlError, match="events"):
        blk.backward(dy, events=events[:3])


def test_block_backward_in_two_phases_equals_whole_backward(cdl, gpu_ok):
    """The data-parallel step runs the backward as phase 1 (FFN half) then phase 2 (attention half)
    so that the FFN gradients can be reduced early.  With the fixed-summation-order option the two
    halves must reproduce the one-call backward bit for bit: dx and all seven weight gradients.
    (Without the option the weight gradients agree within the f32 summation bound, checked too.)"""
    sky1 = cdl.sky1
    dims = dict(batch=2, seqlen=512, hidden=512, heads=4, kv_heads=4, head_dim=128, ffn=1024)
    gen = torch.Generator().manual_seed(9)
    results = {}
    for det in (True, False):
        cfg = sky1.Sky1Config(deterministic=det, **dims)
        params = sky1.init_params(cfg, seed=9, std=0.05)
        x = torch.randn(cfg.tokens, cfg.hidden, generator=torch.Generator().manual_seed(10)).to(torch.bfloat16).cuda()
        dy = torch.randn(cfg.tokens, cfg.hidden, generator=torch.Generator().manual_seed(11)).to(torch.bfloat16).cuda()
        for split in (False, True):
            blk = sky1.Sky1Block(cfg, params)
            for g in blk.grads.values():
                g.zero_()
            blk.forward(x)
            dx = torch.empty_like(x)
            if split:
                blk.backward(dy, dx, phase=1)
                ffn_after_phase1 = {n: blk.grads[n].clone() for n in ("wdown", "wup", "wgate", "norm2")}
                blk.backward(dy, dx, phase=2)
                # phase 2 must not touch the gradients phase 1 declared final
                for n, g in ffn_after_phase1.items():
                    assert torch.equal(g, blk.grads[n]), n
            else:
                blk.backward(dy, dx)
            torch.cuda.synchronize()
            results[(det, split)] = (dx.clone(), {n: g.clone() for n, g in blk.grads.items()})
    dx_a, g_a = results[(True, False)]
    dx_b, g_b = results[(True, True)]
    assert torch.equal(dx_a, dx_b)
    for n in sky1.PARAM_NAMES:
        assert torch.equal(g_a[n], g_b[n]), n
    dx_c, g_c = results[(False, True)]
    assert torch.equal(dx_a, dx_c)  # activations never depend on the K-slice order
    for n in sky1.PARAM_NAMES:
        scale = g_a[n].abs().max().item()
        assert (g_a[n] - g_c[n]).abs().max().item() <= 1e-5 * scale + 1e-7, n


def test_block_rejects_bad_arguments(cdl, gpu_ok):
    sky1 = cdl.sky1
    cfg = sky1.Sky1Config(batch=1, seqlen=128, hidden=256, heads=2, kv_heads=2, head_dim=64, ffn=256)
    with pytest.raises(cdl._lib.CdlError, match="head_dim"):
        sky1.Sky1Block(cfg, sky1.init_params(cfg, 0))
    cfg = sky1.Sky1Config(batch=1, seqlen=128, hidden=256, heads=2, kv_heads=2, head_dim=128, ffn=256)
    blk = sky1.Sky1Block(cfg, sky1.init_params(cfg, 0))
    with pytest.raises(cdl._lib.CdlError, match="contiguous bf16"):
        blk.forward(torch.zeros(cfg.tokens, cfg.hidden, device="cuda"))
    with pytest.raises(cdl._lib.CdlError, match="before forward"):
        blk.backward(torch.zeros(cfg.tokens, cfg.hidden, device="cuda", dtype=torch.bfloat16))


def test_ragged_block_vs_oracle_per_sequence(cdl, gpu_ok):
    """Ragged batch (cu_seqlens; RoPE positions restart, attention stays inside a sequence; the
    layout of the reference's decoder_ragged_seqlen, decoder.rs:372-378, 440-455): outputs and dx
    of every sequence equal the dense oracle run on that sequence alone, and the weight gradients
    equal the sum of the per-sequence ones.  6 padding rows follow the last sequence."""
    sky1 = cdl.sky1
    seqlens = [150, 37, 260, 128]
    pad = 6
    total = sum(seqlens) + pad
    cfg = sky1.Sky1Config(batch=1, seqlen=total, hidden=256, heads=2, kv_heads=1, head_dim=128, ffn=384)
    params = sky1.init_params(cfg, seed=5, std=0.05)
    gen = torch.Generator().manual_seed(5)
    params["norm1"] = (1 + 0.1 * torch.randn(cfg.hidden, generator=gen)).to(torch.bfloat16)
    params["norm2"] = (1 + 0.1 * torch.randn(cfg.hidden, generator=gen)).to(torch.bfloat16)
    x = torch.randn(total, cfg.hidden, generator=gen).to(torch.bfloat16)
    dy = torch.randn(total, cfg.hidden, generator=gen).to(torch.bfloat16)
    dy[total - pad:] = 0  # padding rows carry no gradient
    cu = torch.tensor([0] + list(torch.tensor(seqlens).cumsum(0)), dtype=torch.int32)
    blk = sky1.Sky1Block(cfg, params, cu_seqlens=cu.cuda(), max_seqlen=max(seqlens))
    blk.saved["attn"].fill_(float("nan"))  # stale contents must not leak into the padding rows
    out = blk.forward(x.cuda())
    dx = blk.backward(dy.cuda())
    torch.cuda.synchronize()
    assert blk.saved["lse"].numel() == cfg.heads * total

    c = dict(heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim, eps=cfg.eps)
    g_sum = {n: torch.zeros(s, dtype=torch.float64) for n, s in cfg.param_shapes().items()}
    for b, n_tok in enumerate(seqlens):
        lo, hi = int(cu[b]), int(cu[b + 1])
        table = block_ref.rope_table(n_tok, cfg.head_dim)
        o_ref, dx_ref, g_ref = block_ref.block_forward_backward(x[None, lo:hi], params, dy[None, lo:hi], c, table)
        assert rel_err(out[lo:hi], o_ref[0]) <= 2e-2, b
        assert rel_err(dx[lo:hi], dx_ref[0]) <= 2e-2, b
        for n in g_sum:
            g_sum[n] += g_ref[n]
    for n in sky1.PARAM_NAMES:
        got = blk.grads[n].double().cpu()
        assert torch.isfinite(got).all(), n
        err = ((got - g_sum[n]).abs().max() / g_sum[n].abs().max()).item()
        assert err <= 2e-2, (n, err)


def test_rope_ragged_positions(cdl, gpu_ok):
    L = cdl._lib
    heads, d = 3, 128
    seqlens = [5, 1, 9]
    total = sum(seqlens) + 2
    gen = torch.Generator().manual_seed(1)
    x = torch.randn(total, heads, d, generator=gen).to(torch.bfloat16)
    table = block_ref.rope_table(max(seqlens), d)
    cu = torch.tensor([0, 5, 6, 15], dtype=torch.int32).cuda()
    xd = x.cuda().clone()
    tx, tt, tc = L.tensor_arg(xd), L.tensor_arg(table.float().cuda()), L.tensor_arg(cu)
    L.check(L.lib.cdl_b200_rope_ragged(L.ref(tx), L.ref(tt), 2, L.ref(tc), 0, None))
    torch.cuda.synchronize()
    lo = 0
    for n_tok in seqlens:
        ref = block_ref.rope(x.double()[None, lo:lo + n_tok, :2], table[:n_tok])[0]
        assert rel_err(xd[lo:lo + n_tok, :2], ref) <= 2.0 ** -7
        lo += n_tok
    assert torch.equal(xd[:, 2], x.cuda()[:, 2])      # the third head is not rotated
    assert torch.equal(xd[lo:], x.cuda()[lo:])        # padding rows are untouched
