"""GPU parity of the LM-step kernels (cross-entropy, embedding scatter-add, reduction, AdamW) and of
a 50-step training run of a small sky-1-style LM against the torch restatement (oracle/lm_ref.py):
The acceptance bound is a loss curve within 1 % of the reference over 50 steps."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import to_f32
from oracle import block_ref, lm_ref

pytestmark = pytest.mark.gpu


def test_cross_entropy_forward_and_gradient(cdl, gpu_ok):
    L = cdl._lib
    gen = torch.Generator().manual_seed(0)
    T, V = 300, 4096
    logits = (torch.randn(T, V, generator=gen) * 3).to(torch.bfloat16)
    targets = torch.randint(0, V, (T,), generator=gen, dtype=torch.int32)
    targets[5] = -1  # ignored row
    dev = logits.cuda().clone()
    loss = torch.empty(T, device="cuda")
    args = [L.tensor_arg(t) for t in (dev, targets.cuda(), loss)]
    L.check(L.lib.cdl_b200_cross_entropy(*(L.ref(a) for a in args), 0.25, None))
    torch.cuda.synchronize()
    x = logits.double().requires_grad_(True)
    valid = targets >= 0
    ref = torch.nn.functional.cross_entropy(x[valid], targets[valid].long(), reduction="none")
    (ref.sum() * 0.25).backward()
    got_loss = loss.cpu().double()
    assert got_loss[5] == 0 and torch.allclose(got_loss[valid], ref.detach(), rtol=1e-4, atol=1e-4)
    g = dev.float().cpu().double()
    assert (g[5] == 0).all()
    err = (g - x.grad).abs().max() / x.grad.abs().max()
    assert err <= 2.0 ** -7


def test_embedding_backward_and_sum(cdl, gpu_ok):
    L = cdl._lib
    gen = torch.Generator().manual_seed(1)
    T, V, H = 1000, 64, 256  # many repeats of every token: exercises the atomic accumulation
    tokens = torch.randint(0, V, (T,), generator=gen, dtype=torch.int32)
    dx = torch.randn(T, H, generator=gen).to(torch.bfloat16)
    table = torch.randn(V, H, generator=gen)
    dev = table.cuda().clone()
    args = [L.tensor_arg(t) for t in (tokens.cuda(), dx.cuda(), dev)]
    L.check(L.lib.cdl_b200_embedding_bwd(*(L.ref(a) for a in args), None))
    ref = table.double().index_add(0, tokens.long(), dx.double())
    assert torch.allclose(dev.cpu().double(), ref, rtol=1e-5, atol=1e-4)
    # deterministic reduction: sum of squares, scaled and accumulated
    x = torch.randn(1_000_003, generator=gen).cuda()
    out = torch.full((1,), 2.0, device="cuda")
    scr = torch.empty(4096, dtype=torch.uint8, device="cuda")
    for _ in range(2):
        out.fill_(2.0)
        L.check(L.lib.cdl_b200_sum(x.data_ptr(), x.numel(), out.data_ptr(), 0.5, 1, 1, scr.data_ptr(), 4096, None))
        first = out.clone() if _ == 0 else first
    assert torch.equal(out, first)
    assert abs(out.item() - (2.0 + 0.5 * (x.double() ** 2).sum().item())) <= 1e-5 * out.item()


def test_adamw_matches_reference_update(cdl, gpu_ok):
    L = cdl._lib
    gen = torch.Generator().manual_seed(2)
    n = 100_003
    w, g = torch.randn(n, generator=gen), torch.randn(n, generator=gen)
    m, v = torch.randn(n, generator=gen) * 0.1, torch.rand(n, generator=gen) * 0.1
    dw, dg, dm, dv = (t.cuda().clone() for t in (w, g, m, v))
    rep = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    sumsq = (g.double() ** 2).sum().float().reshape(1).cuda()
    hp = L.CdlAdamwParams(3e-4, 0.9, 0.95, 1e-8, 0.1, 7, 0.5, 1.0)
    L.check(L.lib.cdl_b200_adamw(dw.data_ptr(), rep.data_ptr(), dg.data_ptr(), dm.data_ptr(), dv.data_ptr(),
                                 n, sumsq.data_ptr(), ctypes.byref(hp), None))
    torch.cuda.synchronize()
    gd = g.double() * 0.5
    gd = gd * min(1.0, 1.0 / (gd.norm().item() + 1e-6))
    md = 0.9 * m.double() + 0.1 * gd
    vd = 0.95 * v.double() + 0.05 * gd * gd
    wd = w.double() - 3e-4 * ((md / (1 - 0.9 ** 7)) / ((vd / (1 - 0.95 ** 7)).sqrt() + 1e-8) + 0.1 * w.double())
    assert torch.allclose(dw.cpu().double(), wd, rtol=1e-5, atol=1e-6)
    assert torch.allclose(dm.cpu().double(), md, rtol=1e-5, atol=1e-7)
    assert torch.allclose(dv.cpu().double(), vd, rtol=1e-5, atol=1e-7)
    assert (dg == 0).all() and torch.equal(rep, dw.to(torch.bfloat16))


def small_lm(cdl, layers=2, vocab=2048, seed=4):
    sky1 = cdl.sky1
    blk = sky1.Sky1Config(batch=2, seqlen=256, hidden=256, heads=2, kv_heads=2, head_dim=128, ffn=512)
    return sky1.Sky1LMConfig(block=blk, layers=layers, vocab=vocab, lr=3e-3)


def _run_curve(cdl, cfg, batches, lr):
    sky1 = cdl.sky1
    model = sky1.Sky1LM(cfg, seed=4)
    b = cfg.block
    init = {name: model.view("master", name).detach().cpu().clone() for name, _, _ in model.layout}
    losses = []
    for tokens, targets in batches:
        t = tokens.reshape(1, -1).to(torch.int32).cuda()
        y = targets.reshape(1, -1).to(torch.int32).cuda()
        losses.append(model.train_step(t, y, lr=lr).item())
    assert cdl._lib.device_status() == 0
    c = dict(heads=b.heads, kv_heads=b.kv_heads, head_dim=b.head_dim, eps=b.eps)
    ref_losses, _ = lm_ref.train(init, batches, c, block_ref.rope_table(b.seqlen, b.head_dim), cfg.layers,
                                 lr=lr, beta1=cfg.beta1, beta2=cfg.beta2, eps=cfg.adam_eps,
                                 wd=cfg.weight_decay)
    return np.array(losses), np.array(ref_losses)


def test_lm_loss_curve_50_steps_baseline_regime(cdl, gpu_ok):
    """benchmark configuration 5's regime at reduced size: fresh uniform-random tokens every step, AdamW
    lr 3e-4, betas (0.9, 0.95), wd 0.1, 50 steps; every loss within 1 % of the torch restatement."""
    cfg = small_lm(cdl)
    b = cfg.block
    gen = torch.Generator().manual_seed(4)
    data = torch.randint(0, cfg.vocab, (50, b.batch, b.seqlen + 1), generator=gen)
    batches = [(data[i, :, :-1], data[i, :, 1:]) for i in range(50)]
    losses, ref = _run_curve(cdl, cfg, batches, 3e-4)
    rel = np.abs(losses - ref) / ref
    assert rel.max() <= 1e-2, (rel.max(), losses[-5:], ref[-5:])


def test_lm_loss_curve_50_steps_memorising_one_batch(cdl, gpu_ok):
    """A harder variant: the same batch every step with a larger learning rate, so the loss falls
    by more than a nat in 50 steps and any error in a gradient or in the optimizer shows up as a
    diverging curve."""
    cfg = small_lm(cdl)
    b = cfg.block
    gen = torch.Generator().manual_seed(6)
    data = torch.randint(0, cfg.vocab, (b.batch, b.seqlen + 1), generator=gen)
    batches = [(data[:, :-1], data[:, 1:])] * 50
    losses, ref = _run_curve(cdl, cfg, batches, 1e-3)
    assert ref[-1] < ref[0] - 1.0, "the reference run must actually learn"
    rel = np.abs(losses - ref) / ref
    assert rel.max() <= 1e-2, (rel.max(), losses[-5:], ref[-5:])


def test_lm_gradient_accumulation_equals_one_big_batch(cdl, gpu_ok):
    """Two microbatches accumulated == the same tokens as the reference's summed gradients
    (crates/sky-1/src/skyred/training.rs:290-304): compare the post-step weights with the torch
    restatement fed both microbatches as one batch."""
    sky1 = cdl.sky1
    cfg = small_lm(cdl, layers=1, vocab=1024)
    model = sky1.Sky1LM(cfg, seed=5)
    b = cfg.block
    gen = torch.Generator().manual_seed(5)
    data = torch.randint(0, cfg.vocab, (2, b.batch, b.seqlen + 1), generator=gen)
    init = {name: model.view("master", name).detach().cpu().clone() for name, _, _ in model.layout}
    t = data[:, :, :-1].reshape(2, -1).to(torch.int32).cuda()
    y = data[:, :, 1:].reshape(2, -1).to(torch.int32).cuda()
    loss = model.train_step(t, y, lr=cfg.lr).item()
    c = dict(heads=b.heads, kv_heads=b.kv_heads, head_dim=b.head_dim, eps=b.eps)
    big = (data[:, :, :-1].reshape(-1, b.seqlen), data[:, :, 1:].reshape(-1, b.seqlen))
    ref_losses, ref_master = lm_ref.train(init, [big], c, block_ref.rope_table(b.seqlen, b.head_dim), 1,
                                          lr=cfg.lr, beta1=cfg.beta1, beta2=cfg.beta2, eps=cfg.adam_eps,
                                          wd=cfg.weight_decay)
    assert abs(loss - ref_losses[0]) / ref_losses[0] <= 1e-2
    # After one Adam step every weight moved by about lr; the direction (sign of the gradient)
    # must agree for the bulk of the entries.
    for name in ("lm_head", "blocks.0.wqkv", "blocks.0.wdown", "embedding"):
        d_got = (model.view("master", name).cpu() - init[name]).flatten()
        d_ref = (ref_master[name] - init[name]).flatten()
        big_moves = d_ref.abs() > 0.5 * cfg.lr
        agree = (torch.sign(d_got[big_moves]) == torch.sign(d_ref[big_moves])).float().mean().item()
        assert agree >= 0.97, (name, agree)


def test_lm_config5_full_size_loss_curve_10_steps(cdl, gpu_ok):
    """Benchmark configuration 5 at its real size: 24 layers, hidden 2048, 16 x 128 heads, ffn 5632,
    vocabulary 32768, AdamW lr 3e-4 betas (0.9, 0.95) wd 0.1, one microbatch of 8 x 2048
    uniform-random tokens per step, seed 4.  Ten optimizer steps of the product against the torch
    restatement run in f32 on the same GPU (bf16-rounded weights, full f32 products, every block
    recomputed in its backward to fit): every loss within 1 % (the stated bound) and within 0.03
    nats (what f32-against-bf16 arithmetic leaves on a loss near ln 32768 = 10.4)."""
    sky1 = cdl.sky1
    free, _ = torch.cuda.mem_get_info()
    if free < 120 * 2 ** 30:
        pytest.skip("needs about 110 GB of free device memory")
    b = sky1.Sky1Config()
    cfg = sky1.Sky1LMConfig(block=b, layers=24, vocab=32768)
    model = sky1.Sky1LM(cfg, seed=4)
    steps = 10
    gen = torch.Generator().manual_seed(4)
    data = torch.randint(0, cfg.vocab, (steps, b.batch, b.seqlen + 1), generator=gen)
    init = {name: model.view("master", name).detach().clone() for name, _, _ in model.layout}
    losses = []
    for i in range(steps):
        t = data[i, :, :-1].reshape(1, -1).to(torch.int32).cuda()
        y = data[i, :, 1:].reshape(1, -1).to(torch.int32).cuda()
        losses.append(model.train_step(t, y).item())
    assert cdl._lib.device_status() == 0
    del model
    torch.cuda.empty_cache()
    c = dict(heads=b.heads, kv_heads=b.kv_heads, head_dim=b.head_dim, eps=b.eps)
    batches = [(data[i, :, :-1], data[i, :, 1:]) for i in range(steps)]
    ref, _ = lm_ref.train(init, batches, c, block_ref.rope_table(b.seqlen, b.head_dim), cfg.layers,
                          lr=cfg.lr, beta1=cfg.beta1, beta2=cfg.beta2, eps=cfg.adam_eps,
                          wd=cfg.weight_decay, device="cuda", checkpoint_blocks=True)
    losses, ref = np.array(losses), np.array(ref)
    print("config 5, 10 steps: product", np.round(losses, 4).tolist(), "torch f32", np.round(ref, 4).tolist())
    assert np.isfinite(losses).all()
    assert (np.abs(losses - ref) / ref).max() <= 1e-2, (losses, ref)
    assert np.abs(losses - ref).max() <= 0.03, (losses, ref)
