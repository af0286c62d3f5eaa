"""GPU parity of flash attention forward / backward against the f64 oracle, through the C ABI.

Follows crates/cleandl/tests/attention.rs: inputs N(0,1) rounded to bf16 (:251-259); tolerance
atol * max|expected| + rtol * |expected| (:541-556) with (1e-2, 1e-2) for the bf16 output,
(1e-4, 1e-3) for LSE and (2e-2, 2e-2) for bf16 gradients (:781-804); cases over masks, GQA and
Sq != Sk (:836-866), fused-QKV slicing (:589-613), backward (:984-1032), rejections (:1035-1105).
"""
import ctypes

import numpy as np
import pytest
import torch

from helpers import assert_all_close, to_f32
from oracle import cpu_oracle as oracle

pytestmark = pytest.mark.gpu


def make(b, sq, sk, hq, hk, seed=7, d=128):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(b, sq, hq, d, generator=gen).to(torch.bfloat16)
    k = torch.randn(b, sk, hk, d, generator=gen).to(torch.bfloat16)
    v = torch.randn(b, sk, hk, d, generator=gen).to(torch.bfloat16)
    do = torch.randn(b, sq, hq, d, generator=gen).to(torch.bfloat16)
    return q, k, v, do


def check_fwd(out, q, k, v, causal, scale=None):
    ref = oracle.attention(to_f32(q), to_f32(k), to_f32(v), None, scale=scale, causal=causal)
    assert_all_close("out", to_f32(out.out), ref["out"],
                     oracle.attention_tolerance(ref["out"], 1e-2, 1e-2))
    got_lse = np.where(np.isneginf(to_f32(out.lse)), -1e30, to_f32(out.lse))
    exp_lse = np.where(np.isneginf(ref["lse"]), -1e30, ref["lse"])
    assert_all_close("lse", got_lse, exp_lse, oracle.attention_tolerance(ref["lse"], 1e-4, 1e-3))
    return ref


FWD_CASES = [
    # b, sq, sk, hq, hk, causal
    (1, 128, 128, 1, 1, True),
    (1, 256, 256, 2, 2, True),
    (2, 384, 384, 2, 1, True),     # GQA, odd number of 128-row tiles
    (1, 200, 200, 2, 2, True),     # ragged tail
    (1, 77, 333, 2, 2, True),      # sq < sk: mask aligned to the bottom right
    (1, 300, 100, 1, 1, True),     # sq > sk: the first rows see no key
    (2, 256, 320, 4, 2, False),    # dense (no mask), GQA
    (1, 1, 1, 1, 1, True),
    (1, 640, 640, 1, 1, True),
    (3, 1100, 1100, 2, 2, True),   # five 256-row work items per head
    (1, 1536, 700, 1, 1, True),    # sq > sk over several work items: the first of them see no key
    (2, 520, 1300, 2, 1, False),   # dense, ragged in both directions
]


@pytest.mark.parametrize("variant", [1, 2], ids=["one_shot", "persistent"])
@pytest.mark.parametrize("b,sq,sk,hq,hk,causal", FWD_CASES)
def test_fwd_cases(cdl, gpu_ok, b, sq, sk, hq, hk, causal, variant):
    """Both forward kernels (cdl_attn_desc.variant: what a tuner enumerates) on every case."""
    q, k, v, _ = make(b, sq, sk, hq, hk)
    out = cdl.ops.attention_fwd(q.cuda(), k.cuda(), v.cuda(),
                                cdl.ops.AttentionOpts(causal=causal, variant=variant))
    check_fwd(out, q, k, v, causal)


def test_fwd_many_items_per_cluster(cdl, gpu_ok):
    """More work items than SMs (the persistent kernel walks several items per CTA: rings,
    barriers and tensor memory live across items): 4 x 40 heads x 4 query blocks = 640 items.  Run twice (bit-equal) and checked on three (batch, head) slices against the oracle
    and everywhere against the one-CTA kernel."""
    gen = torch.Generator().manual_seed(31)
    q, k, v = (torch.randn(4, 1024, 40, 128, generator=gen).to(torch.bfloat16).cuda() for _ in range(3))
    o1 = cdl.ops.attention_fwd(q, k, v)
    o2 = cdl.ops.attention_fwd(q, k, v)
    assert torch.equal(o1.out, o2.out) and torch.equal(o1.lse, o2.lse)
    ref = cdl.ops.attention_fwd(q, k, v, cdl.ops.AttentionOpts(variant=cdl._lib.ATTN_ONE_SHOT))
    assert (o1.out.float() - ref.out.float()).abs().max().item() <= 2e-2 * ref.out.float().abs().max().item()
    assert (o1.lse - ref.lse).abs().max().item() <= 2e-3
    for bi, hi in ((0, 0), (3, 39), (2, 17)):
        sl = (slice(bi, bi + 1), slice(None), slice(hi, hi + 1))
        r = oracle.attention(to_f32(q[sl]), to_f32(k[sl]), to_f32(v[sl]), None, causal=True)
        assert_all_close("out", to_f32(o1.out[sl]), r["out"], oracle.attention_tolerance(r["out"], 1e-2, 1e-2))
        assert_all_close("lse", to_f32(o1.lse[bi:bi + 1, hi:hi + 1]), r["lse"],
                         oracle.attention_tolerance(r["lse"], 1e-4, 1e-3))


def test_fwd_fused_qkv_views_and_scale(cdl, gpu_ok):
    """q, k, v as slices of one fused [B, S, 3H, D] buffer, custom softmax scale."""
    b, s, h = 2, 256, 2
    gen = torch.Generator().manual_seed(11)
    qkv = torch.randn(b, s, 3 * h, 128, generator=gen).to(torch.bfloat16)
    dq = qkv.cuda()
    q, k, v = dq[:, :, :h], dq[:, :, h:2 * h], dq[:, :, 2 * h:]
    out = cdl.ops.attention_fwd(q, k, v, cdl.ops.AttentionOpts(softmax_scale=0.05, causal=True))
    check_fwd(out, qkv[:, :, :h], qkv[:, :, h:2 * h], qkv[:, :, 2 * h:], True, scale=0.05)


def test_fwd_large_logits_rescale(cdl, gpu_ok):
    """Scores that grow along the sequence force the running max to move repeatedly."""
    q, k, v, _ = make(1, 512, 512, 1, 1, seed=5)
    ramp = torch.linspace(0.2, 6.0, 512).view(1, 512, 1, 1)
    k = (k.float() * ramp).to(torch.bfloat16)
    out = cdl.ops.attention_fwd(q.cuda(), k.cuda(), v.cuda(), cdl.ops.AttentionOpts(causal=True))
    check_fwd(out, q, k, v, True)


def test_fwd_deterministic_and_sdpa_at_config3_shape(cdl, gpu_ok):
    """benchmark configuration 3 shape (B=8, H=16, S=2048, D=128, seed 2): the f64 oracle would need
    minutes, so the full size is compared with torch's fp32 attention on the GPU and one
    (batch, head) slice with the oracle."""
    gen = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn(8, 2048, 16, 128, generator=gen).to(torch.bfloat16).cuda() for _ in range(3))
    o1 = cdl.ops.attention_fwd(q, k, v)
    o2 = cdl.ops.attention_fwd(q, k, v)
    assert torch.equal(o1.out, o2.out) and torch.equal(o1.lse, o2.lse)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q[:2].float().transpose(1, 2), k[:2].float().transpose(1, 2), v[:2].float().transpose(1, 2),
        is_causal=True).transpose(1, 2)
    err = (o1.out[:2].float() - ref).abs().max().item() / ref.abs().max().item()
    assert err <= 1e-2
    sl = (slice(7, 8), slice(None), slice(15, 16))
    r = oracle.attention(to_f32(q[sl]), to_f32(k[sl]), to_f32(v[sl]), None, causal=True)
    assert_all_close("out", to_f32(o1.out[sl]), r["out"], oracle.attention_tolerance(r["out"], 1e-2, 1e-2))
    assert_all_close("lse", to_f32(o1.lse[7:8, 15:16]), r["lse"],
                     oracle.attention_tolerance(r["lse"], 1e-4, 1e-3))


def test_fwd_rejections(cdl, gpu_ok):
    dev = "cuda"
    z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)
    with pytest.raises(cdl._lib.CdlError, match="head dimension"):
        cdl.ops.attention_fwd(z(1, 8, 1, 64), z(1, 8, 1, 64), z(1, 8, 1, 64))
    with pytest.raises(cdl._lib.CdlError, match="multiple of kv heads"):
        cdl.ops.attention_fwd(z(1, 8, 3, 128), z(1, 8, 2, 128), z(1, 8, 2, 128))
    with pytest.raises(cdl._lib.CdlError, match="shape"):
        cdl.ops.attention_fwd(z(1, 8, 2, 128), z(1, 8, 2, 128), z(1, 9, 2, 128))
    with pytest.raises(cdl._lib.CdlError, match="contiguous"):
        cdl.ops.attention_fwd(z(1, 8, 2, 256)[..., ::2], z(1, 8, 2, 128), z(1, 8, 2, 128))
    out = cdl.ops.attention_fwd(z(0, 8, 2, 128), z(0, 8, 2, 128), z(0, 8, 2, 128))
    assert out.out.shape == (0, 8, 2, 128)


def check_bwd(cdl, q, k, v, do, causal, scale=None, variant=0):
    dq_, dk_, dv_, ddo = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    opts = cdl.ops.AttentionOpts(softmax_scale=scale, causal=causal, variant=variant)
    fwd = cdl.ops.attention_fwd(dq_, dk_, dv_, opts)
    dq, dk, dv = cdl.ops.attention_bwd(dq_, dk_, dv_, fwd.out, ddo, fwd.lse, opts)
    ref = oracle.attention(to_f32(q), to_f32(k), to_f32(v), to_f32(do), scale=scale, causal=causal)
    for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert_all_close(name, to_f32(got), ref[name], oracle.attention_tolerance(ref[name], 2e-2, 2e-2))


BWD_CASES = [
    (1, 128, 128, 1, 1, True),
    (1, 256, 256, 2, 2, True),
    (2, 384, 384, 2, 1, True),     # GQA: dk/dv accumulate over the query heads of a group
    (1, 200, 200, 2, 2, True),     # ragged tail
    (1, 77, 333, 2, 2, True),      # sq < sk
    (1, 300, 100, 1, 1, True),     # sq > sk: rows without keys, key blocks without queries
    (2, 256, 320, 4, 2, False),    # dense, GQA
    (1, 1, 1, 1, 1, True),
    (1, 640, 512, 1, 1, True),
]


@pytest.mark.parametrize("variant", [1, 2], ids=["one_shot", "persistent"])
@pytest.mark.parametrize("b,sq,sk,hq,hk,causal", BWD_CASES)
def test_bwd_cases(cdl, gpu_ok, b, sq, sk, hq, hk, causal, variant):
    q, k, v, do = make(b, sq, sk, hq, hk)
    check_bwd(cdl, q, k, v, do, causal, variant=variant)


@pytest.mark.parametrize("b,s,hq,hk,causal", [(6, 1024, 8, 4, True), (3, 1100, 8, 8, False),
                                              (20, 300, 8, 8, True)])
def test_bwd_persistent_equals_one_shot(cdl, gpu_ok, b, s, hq, hk, causal):
    """More key blocks than SMs, so every CTA of the persistent dK/dV and dQ kernels takes several items
    (among them one-block items, whose hand-over to the next item is the shortest): the two forms
    run the same arithmetic in the same order and must agree bit for bit; one (batch, head)
    against the oracle."""
    q, k, v, do = (t.cuda() for t in make(b, s, s, hq, hk, seed=19))
    fwd = cdl.ops.attention_fwd(q, k, v, cdl.ops.AttentionOpts(causal=causal))
    res = {}
    for variant in (1, 2):
        opts = cdl.ops.AttentionOpts(causal=causal, variant=variant)
        for rep in range(2):     # twice: the second launch finds the work counter as the first left it
            res[variant] = cdl.ops.attention_bwd(q, k, v, fwd.out, do, fwd.lse, opts)
    for name, a, c in zip(("dq", "dk", "dv"), res[1], res[2]):
        assert torch.equal(a, c), name
    sl = (slice(b - 1, b), slice(None))
    g = hq // hk
    r = oracle.attention(to_f32(q[sl][:, :, :g]), to_f32(k[sl][:, :, :1]), to_f32(v[sl][:, :, :1]),
                         to_f32(do[sl][:, :, :g]), causal=causal)
    for name, got in (("dk", res[2][1]), ("dv", res[2][2])):
        assert_all_close(name, to_f32(got[sl][:, :, :1]), r[name], oracle.attention_tolerance(r[name], 2e-2, 2e-2))
    assert_all_close("dq", to_f32(res[2][0][sl][:, :, :g]), r["dq"], oracle.attention_tolerance(r["dq"], 2e-2, 2e-2))


def test_bwd_on_several_streams_at_once(cdl, gpu_ok):
    """Persistent backward launches on different streams draw from different work counters."""
    q, k, v, do = (t.cuda() for t in make(4, 1024, 1024, 8, 8, seed=23))
    fwd = cdl.ops.attention_fwd(q, k, v)
    opts = cdl.ops.AttentionOpts(variant=2)
    ref = cdl.ops.attention_bwd(q, k, v, fwd.out, do, fwd.lse, opts)
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream() for _ in range(3)]
    outs = []
    for rep in range(2):
        for st in streams:
            st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                outs.append(cdl.ops.attention_bwd(q, k, v, fwd.out, do, fwd.lse, opts))
    torch.cuda.synchronize()
    for got in outs:
        for a, c in zip(got, ref):
            assert torch.equal(a, c)


def test_bwd_fused_qkv_views(cdl, gpu_ok):
    """Inputs and gradients as slices of fused [B, S, 3H, D] buffers (the sky-1 block's layout)."""
    b, s, h = 1, 256, 2
    gen = torch.Generator().manual_seed(13)
    qkv = torch.randn(b, s, 3 * h, 128, generator=gen).to(torch.bfloat16)
    do = torch.randn(b, s, h, 128, generator=gen).to(torch.bfloat16)
    dev = qkv.cuda()
    q, k, v = dev[:, :, :h], dev[:, :, h:2 * h], dev[:, :, 2 * h:]
    fwd = cdl.ops.attention_fwd(q, k, v)
    dqkv = torch.zeros_like(dev)
    cdl.ops.attention_bwd(q, k, v, fwd.out, do.cuda(), fwd.lse, dq=dqkv[:, :, :h],
                          dk=dqkv[:, :, h:2 * h], dv=dqkv[:, :, 2 * h:])
    ref = oracle.attention(to_f32(qkv[:, :, :h]), to_f32(qkv[:, :, h:2 * h]), to_f32(qkv[:, :, 2 * h:]),
                           to_f32(do), causal=True)
    for i, name in enumerate(("dq", "dk", "dv")):
        assert_all_close(name, to_f32(dqkv[:, :, i * h:(i + 1) * h]), ref[name],
                         oracle.attention_tolerance(ref[name], 2e-2, 2e-2))


def test_bwd_config3_shape_vs_torch_autograd(cdl, gpu_ok):
    """benchmark configuration 3 (B=8, H=16, S=2048, D=128, seed 2) against fp32 autograd through
    torch's attention on the same GPU for two batches, and one (batch, head) against the oracle."""
    gen = torch.Generator().manual_seed(2)
    q, k, v, do = (torch.randn(8, 2048, 16, 128, generator=gen).to(torch.bfloat16).cuda()
                   for _ in range(4))
    fwd = cdl.ops.attention_fwd(q, k, v)
    dq, dk, dv = cdl.ops.attention_bwd(q, k, v, fwd.out, do, fwd.lse)
    qf, kf, vf = (t[:2].float().transpose(1, 2).detach().requires_grad_(True) for t in (q, k, v))
    out = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, is_causal=True)
    out.backward(do[:2].float().transpose(1, 2))
    for name, got, ref in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
        ref = ref.transpose(1, 2)
        err = (got[:2].float() - ref).abs().max().item() / ref.abs().max().item()
        assert err <= 2e-2, (name, err)
    sl = (slice(5, 6), slice(None), slice(3, 4))
    r = oracle.attention(to_f32(q[sl]), to_f32(k[sl]), to_f32(v[sl]), to_f32(do[sl]), causal=True)
    for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert_all_close(name, to_f32(got[sl]), r[name], oracle.attention_tolerance(r[name], 2e-2, 2e-2))


def test_bwd_scratch_is_checked(cdl, gpu_ok):
    q, k, v, do = (t.cuda() for t in make(1, 128, 128, 1, 1))
    fwd = cdl.ops.attention_fwd(q, k, v)
    small = torch.empty(64, dtype=torch.uint8, device="cuda")
    with pytest.raises(cdl._lib.CdlError, match="scratch"):
        cdl.ops.attention_bwd(q, k, v, fwd.out, do, fwd.lse, scratch=small)


# ---------------------------------------------------------------------------------------------
# Packed ("varlen") layout: QueryLayout::Packed / KvLayout::Packed of the reference
# (ops/attention/mod.rs:55-79), tested there by `Case::varlen` with 5 unused query rows and 3
# unused key rows at the end of the packed buffers (crates/cleandl/tests/attention.rs:118-127,
# 273-299).  The oracle runs one sequence at a time on the dense restatement.

def make_packed(seqlens_q, seqlens_k, hq, hk, pad_q=5, pad_k=3, seed=11, d=128):
    gen = torch.Generator().manual_seed(seed)
    tq, tk = sum(seqlens_q) + pad_q, sum(seqlens_k) + pad_k
    q = torch.randn(tq, hq, d, generator=gen).to(torch.bfloat16)
    k = torch.randn(tk, hk, d, generator=gen).to(torch.bfloat16)
    v = torch.randn(tk, hk, d, generator=gen).to(torch.bfloat16)
    do = torch.randn(tq, hq, d, generator=gen).to(torch.bfloat16)
    cu_q = torch.tensor([0] + list(np.cumsum(seqlens_q)), dtype=torch.int32)
    cu_k = torch.tensor([0] + list(np.cumsum(seqlens_k)), dtype=torch.int32)
    return q, k, v, do, cu_q, cu_k


PACKED_CASES = [
    # seqlens_q, seqlens_k, hq, hk, causal, give max_seqlen
    ([128, 256], [128, 256], 2, 2, True, True),
    ([200, 77, 333], [200, 77, 333], 2, 1, True, True),       # ragged, GQA
    ([100, 300, 1], [260, 300, 40], 2, 2, True, False),       # sq != sk per sequence, no bound given
    ([64, 0, 190], [64, 50, 190], 1, 1, True, True),          # an empty query sequence
    ([130, 250], [300, 129], 4, 2, False, True),              # dense mask
]


@pytest.mark.parametrize("variant", [1, 2], ids=["one_shot", "persistent"])
@pytest.mark.parametrize("sq,sk,hq,hk,causal,bound", PACKED_CASES)
def test_packed_fwd_bwd(cdl, gpu_ok, sq, sk, hq, hk, causal, bound, variant):
    q, k, v, do, cu_q, cu_k = make_packed(sq, sk, hq, hk)
    opts = cdl.ops.AttentionOpts(causal=causal, variant=variant, cu_seqlens_q=cu_q.cuda(), cu_seqlens_k=cu_k.cuda(),
                                 max_seqlen_q=max(sq) if bound else None,
                                 max_seqlen_k=max(sk) if bound else None)
    qd, kd, vd, dod = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    fwd = cdl.ops.attention_fwd(qd, kd, vd, opts)
    # rows outside every sequence are not written: mark them to check that
    dq = torch.full_like(qd, 7.0)
    dk = torch.full_like(kd, 7.0)
    dv = torch.full_like(vd, 7.0)
    cdl.ops.attention_bwd(qd, kd, vd, fwd.out, dod, fwd.lse, opts, dq=dq, dk=dk, dv=dv)
    assert fwd.lse.shape == (hq, q.shape[0])
    for b in range(len(sq)):
        q0, q1, k0, k1 = int(cu_q[b]), int(cu_q[b + 1]), int(cu_k[b]), int(cu_k[b + 1])
        if q1 == q0:
            assert float(dk[k0:k1].float().abs().max()) == 0.0 if k1 > k0 else True
            continue
        ref = oracle.attention(to_f32(q[None, q0:q1]), to_f32(k[None, k0:k1]), to_f32(v[None, k0:k1]),
                               to_f32(do[None, q0:q1]), causal=causal)
        assert_all_close(f"out[{b}]", to_f32(fwd.out[q0:q1])[None], ref["out"],
                         oracle.attention_tolerance(ref["out"], 1e-2, 1e-2))
        got_lse = to_f32(fwd.lse[:, q0:q1])[None]
        exp_lse = np.where(np.isneginf(ref["lse"]), -1e30, ref["lse"])
        assert_all_close(f"lse[{b}]", np.where(np.isneginf(got_lse), -1e30, got_lse), exp_lse,
                         oracle.attention_tolerance(ref["lse"], 1e-4, 1e-3))
        for name, got, lo, hi in (("dq", dq, q0, q1), ("dk", dk, k0, k1), ("dv", dv, k0, k1)):
            assert_all_close(f"{name}[{b}]", to_f32(got[lo:hi])[None], ref[name],
                             oracle.attention_tolerance(ref[name], 2e-2, 2e-2))
    # the unused rows at the end keep their marker
    assert float(dq[int(cu_q[-1]):].float().min()) == 7.0
    assert float(dk[int(cu_k[-1]):].float().min()) == 7.0
    assert float(dv[int(cu_k[-1]):].float().min()) == 7.0


def test_packed_equals_dense_for_equal_lengths(cdl, gpu_ok):
    """Equal-length sequences: the packed call must reproduce the dense call bit for bit."""
    b, s, h = 3, 384, 2
    q, k, v, do = make(b, s, s, h, h, seed=5)
    dense = cdl.ops.attention_fwd(q.cuda(), k.cuda(), v.cuda())
    ddq, ddk, ddv = cdl.ops.attention_bwd(q.cuda(), k.cuda(), v.cuda(), dense.out, do.cuda(), dense.lse)
    cu = torch.arange(0, (b + 1) * s, s, dtype=torch.int32).cuda()
    opts = cdl.ops.AttentionOpts(cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=s, max_seqlen_k=s)
    flat = lambda t: t.reshape(b * s, h, 128).cuda()
    packed = cdl.ops.attention_fwd(flat(q), flat(k), flat(v), opts)
    assert torch.equal(packed.out.view(b, s, h, 128), dense.out)
    assert torch.equal(packed.lse.view(h, b, s).permute(1, 0, 2), dense.lse)
    pdq, pdk, pdv = cdl.ops.attention_bwd(flat(q), flat(k), flat(v), packed.out, flat(do), packed.lse, opts)
    assert torch.equal(pdq.view(b, s, h, 128), ddq)
    assert torch.equal(pdk.view(b, s, h, 128), ddk)
    assert torch.equal(pdv.view(b, s, h, 128), ddv)


@pytest.mark.parametrize("variant", [1, 2], ids=["one_shot", "persistent"])
def test_packed_sequence_longer_than_the_bound_is_cut_and_reported(cdl, gpu_ok, variant):
    """max_seqlen_q / max_seqlen_k size the grids and the backward's statistics scratch.  A
    sequence longer than the bound must not make the backward read or write beyond that scratch:
    it is cut at the bound and the device status word reports code 921.  The sequences within the
    bound still get their exact gradients."""
    sq = [128, 300]
    q, k, v, do, cu_q, cu_k = make_packed(sq, sq, 2, 2)
    qd, kd, vd, dod = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    ok = cdl.ops.AttentionOpts(causal=True, variant=variant, cu_seqlens_q=cu_q.cuda(), cu_seqlens_k=cu_k.cuda(),
                               max_seqlen_q=300, max_seqlen_k=300)
    fwd = cdl.ops.attention_fwd(qd, kd, vd, ok)
    ref_dq, ref_dk, ref_dv = cdl.ops.attention_bwd(qd, kd, vd, fwd.out, dod, fwd.lse, ok)
    assert cdl._lib.device_status() == 0
    low = cdl.ops.AttentionOpts(causal=True, variant=variant, cu_seqlens_q=cu_q.cuda(), cu_seqlens_k=cu_k.cuda(),
                                max_seqlen_q=128, max_seqlen_k=128)
    # scratch sized exactly by the (too small) bound, followed by a guard region
    n = ctypes.c_size_t(0)
    cdl._lib.check(cdl._lib.lib.cdl_b200_attn_bwd_packed_scratch_bytes(2, 128, 2, ctypes.byref(n)))
    buf = torch.full((n.value + 4096,), 0x5A, dtype=torch.uint8, device="cuda")
    dq, dk, dv = cdl.ops.attention_bwd(qd, kd, vd, fwd.out, dod, fwd.lse, low, scratch=buf[:n.value])
    assert cdl._lib.device_status() == 921
    assert bool((buf[n.value:] == 0x5A).all()), "the backward wrote beyond its scratch"
    s0 = slice(0, 128)  # the sequence that fits the bound
    assert torch.equal(dq[s0], ref_dq[s0]) and torch.equal(dk[s0], ref_dk[s0]) and torch.equal(dv[s0], ref_dv[s0])


def _rope_table(positions, d=128):
    inv = 10000.0 ** (-torch.arange(0, d // 2, dtype=torch.float64) * 2 / d)
    ang = torch.arange(positions, dtype=torch.float64)[:, None] * inv[None]
    return torch.cat([ang.cos(), ang.sin()], 1).float()


def _assert_same_up_to_one_rounding(name, got, ref):
    """Both sides apply the same f32 arithmetic to the same bf16 values; the compiler may contract
    the two kernels' multiply-adds differently, so single results may differ by one bf16 step."""
    g, r = got.float(), ref.float()
    step = torch.maximum(g.abs(), r.abs()) * 2.0 ** -7 + 1e-30
    assert bool(((g - r).abs() <= step).all()), f"{name}: more than one bf16 step apart"
    assert (got == ref).float().mean().item() > 0.99, f"{name}: too many elements differ"


@pytest.mark.parametrize("variant", [1, 2], ids=["one_shot", "persistent"])
@pytest.mark.parametrize("b,s,hq,hk", [(2, 384, 2, 2), (1, 200, 4, 2), (2, 130, 2, 1)])
def test_bwd_with_rope_equals_bwd_then_inverse_rope(cdl, gpu_ok, b, s, hq, hk, variant):
    """cdl_b200_attn_bwd_rope: dq and dk with the transposed rotary rotation applied in the store
    epilogues equal the plain backward followed by cdl_b200_rope(backward = 1); dv is untouched."""
    L = cdl._lib
    q, k, v, do = make(b, s, s, hq, hk, seed=21)
    qd, kd, vd, dod = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    table = _rope_table(s).cuda()
    opts = cdl.ops.AttentionOpts(causal=True, variant=variant)
    fwd = cdl.ops.attention_fwd(qd, kd, vd, opts)
    dq, dk, dv = cdl.ops.attention_bwd(qd, kd, vd, fwd.out, dod, fwd.lse, opts)
    keep = []
    for t, heads in ((dq, hq), (dk, hk)):
        flat = t.view(b * s, heads, 128)
        tx, tt = L.tensor_arg(flat), L.tensor_arg(table)
        keep += [tx, tt]
        L.check(L.lib.cdl_b200_rope(L.ref(tx), L.ref(tt), heads, s, 1, None))
    fq, fk, fv = cdl.ops.attention_bwd(qd, kd, vd, fwd.out, dod, fwd.lse, opts, rope_table=table)
    torch.cuda.synchronize()
    assert L.device_status() == 0
    _assert_same_up_to_one_rounding("dq", fq, dq)
    _assert_same_up_to_one_rounding("dk", fk, dk)
    assert torch.equal(fv, dv)


@pytest.mark.parametrize("variant", [1, 2], ids=["one_shot", "persistent"])
def test_packed_bwd_with_rope_equals_bwd_then_inverse_rope(cdl, gpu_ok, variant):
    L = cdl._lib
    lens = [128, 300, 77]
    q, k, v, do, cu_q, cu_k = make_packed(lens, lens, 4, 2)
    qd, kd, vd, dod, cu = q.cuda(), k.cuda(), v.cuda(), do.cuda(), cu_q.cuda()
    table = _rope_table(max(lens)).cuda()
    opts = cdl.ops.AttentionOpts(causal=True, variant=variant, cu_seqlens_q=cu, cu_seqlens_k=cu,
                                 max_seqlen_q=max(lens), max_seqlen_k=max(lens))
    fwd = cdl.ops.attention_fwd(qd, kd, vd, opts)
    mark = lambda t: torch.full_like(t, 7.0)
    dq, dk, dv = cdl.ops.attention_bwd(qd, kd, vd, fwd.out, dod, fwd.lse, opts, dq=mark(qd), dk=mark(kd), dv=mark(vd))
    keep = []
    for t, heads in ((dq, 4), (dk, 2)):
        tx, tt, tc = L.tensor_arg(t), L.tensor_arg(table), L.tensor_arg(cu)
        keep += [tx, tt, tc]
        L.check(L.lib.cdl_b200_rope_ragged(L.ref(tx), L.ref(tt), heads, L.ref(tc), 1, None))
    fq, fk, fv = cdl.ops.attention_bwd(qd, kd, vd, fwd.out, dod, fwd.lse, opts, dq=mark(qd), dk=mark(kd),
                                       dv=mark(vd), rope_table=table)
    torch.cuda.synchronize()
    assert L.device_status() == 0
    _assert_same_up_to_one_rounding("dq", fq, dq)
    _assert_same_up_to_one_rounding("dk", fk, dk)
    assert torch.equal(fv, dv)
    # a table shorter than the longest sequence is refused
    with pytest.raises(L.CdlError, match="positions"):
        cdl.ops.attention_bwd(qd, kd, vd, fwd.out, dod, fwd.lse, opts, rope_table=table[:100].contiguous())


def test_forward_on_several_streams_at_once(cdl, gpu_ok):
    """The persistent forward hands its work items out through a counter that belongs to the
    launching stream.  Calls with many more items than SMs, enqueued on three streams so that they
    overlap on the device and repeated back to back on each stream, must all reproduce the call
    made alone bit for bit, and every launch must leave its counter at zero for the next one."""
    streams = [torch.cuda.Stream() for _ in range(3)]
    inputs = [tuple(t.cuda() for t in make(4, 2048, 2048, 16, 16, seed=40 + i)[:3]) for i in range(3)]  # 512 items each
    opts = cdl.ops.AttentionOpts(causal=True)
    want = [cdl.ops.attention_fwd(q, k, v, opts) for q, k, v in inputs]
    torch.cuda.synchronize()
    got = [[None] * 5 for _ in streams]
    for rep in range(5):
        for i, st in enumerate(streams):
            with torch.cuda.stream(st):
                got[i][rep] = cdl.ops.attention_fwd(*inputs[i], opts)
    torch.cuda.synchronize()
    assert cdl._lib.device_status() == 0
    for i in range(len(streams)):
        for rep in range(5):
            assert torch.equal(got[i][rep].out, want[i].out), (i, rep)
            assert torch.equal(got[i][rep].lse, want[i].lse), (i, rep)


def test_packed_rejections(cdl, gpu_ok):
    z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device="cuda")
    cu = torch.tensor([0, 8], dtype=torch.int32, device="cuda")
    with pytest.raises(cdl._lib.CdlError, match="together"):
        cdl.ops.attention_fwd(z(8, 2, 128), z(8, 2, 128), z(8, 2, 128), cdl.ops.AttentionOpts(cu_seqlens_q=cu))
    with pytest.raises(cdl._lib.CdlError, match="total_q, heads, head_dim"):
        cdl.ops.attention_fwd(z(1, 8, 2, 128), z(1, 8, 2, 128), z(1, 8, 2, 128),
                              cdl.ops.AttentionOpts(cu_seqlens_q=cu, cu_seqlens_k=cu))
    with pytest.raises(cdl._lib.CdlError, match="i32"):
        cdl.ops.attention_fwd(z(8, 2, 128), z(8, 2, 128), z(8, 2, 128),
                              cdl.ops.AttentionOpts(cu_seqlens_q=cu.float(), cu_seqlens_k=cu))
