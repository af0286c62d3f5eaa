"""GPU parity of RMSNorm forward / backward against the f64 oracle, through the C ABI.

Forward cases and tolerances follow crates/cleandl/tests/norm.rs: inputs x ~ N(0.5, 2.0),
scale ~ U(0.5, 1.5), bias ~ N(0, 1) (:220-228); specialized cases (:322-380); bf16 output within
1e-5 + 2^-7 |e| (:261-268), r_inv within 1e-6 + 1e-4 |e| (:309-315); strided rows (:586-621).
The backward has no reference test; it is held to the acceptance bound of 1e-2 and to the bf16 rounding
bound of the forward.
"""
import numpy as np
import pytest
import torch

from helpers import assert_all_close, to_f32
from oracle import cpu_oracle as oracle

pytestmark = pytest.mark.gpu

CASES = [(1, 128), (37, 4096), (300, 2048), (128, 8192), (100, 7168), (5, 1024), (96, 512),
         (333, 1536), (64, 136)]


def make_inputs(rows, cols, seed):
    gen = torch.Generator().manual_seed(seed)
    x = (torch.randn(rows, cols, generator=gen) * 2.0 + 0.5).to(torch.bfloat16)
    scale = (torch.rand(cols, generator=gen) + 0.5).to(torch.bfloat16)
    bias = torch.randn(cols, generator=gen).to(torch.bfloat16)
    return x, scale, bias


@pytest.mark.parametrize("rows,cols", CASES)
@pytest.mark.parametrize("affine", ["none", "scale", "scale_bias"])
def test_fwd_cases(cdl, gpu_ok, rows, cols, affine):
    x, scale, bias = make_inputs(rows, cols, 1)
    s = scale if affine != "none" else None
    b = bias if affine == "scale_bias" else None
    eps = 1e-2 if (rows, cols) == (333, 1536) else 1e-6
    out = cdl.ops.norm_fwd(x.cuda(), cdl.ops.NormFwdOpts(
        scale=None if s is None else s.cuda(), bias=None if b is None else b.cuda(), eps=eps,
        save_stats=True))
    y_ref, r_ref = oracle.rmsnorm_fwd(to_f32(x), None if s is None else to_f32(s),
                                      None if b is None else to_f32(b), eps)
    assert_all_close("y", to_f32(out.y), y_ref, oracle.abs_rel_tolerance(y_ref, 1e-5, 2.0 ** -7))
    assert_all_close("r_inv", to_f32(out.r_inv), r_ref, oracle.abs_rel_tolerance(r_ref, 1e-6, 1e-4))


def test_fwd_strided_rows_no_stats(cdl, gpu_ok):
    x, scale, _ = make_inputs(64, 1024, 2)
    big = torch.zeros(64, 2048, dtype=torch.bfloat16)
    big[:, 512:1536] = x
    xd = big.cuda()[:, 512:1536]
    out = cdl.ops.norm_fwd(xd, cdl.ops.NormFwdOpts(scale=scale.cuda()))
    assert out.r_inv is None
    y_ref, _ = oracle.rmsnorm_fwd(to_f32(x), to_f32(scale), None, 1e-6)
    assert_all_close("y", to_f32(out.y), y_ref, oracle.abs_rel_tolerance(y_ref, 1e-5, 2.0 ** -7))


def test_fwd_config2_and_determinism(cdl, gpu_ok):
    """benchmark configuration 2: x[16384, 2048] ~ N(0,1), weight 1 + N(0, 0.02), eps 1e-6, seed 1."""
    gen = torch.Generator().manual_seed(1)
    x = torch.randn(16384, 2048, generator=gen).to(torch.bfloat16)
    w = (1 + 0.02 * torch.randn(2048, generator=gen)).to(torch.bfloat16)
    opts = cdl.ops.NormFwdOpts(scale=w.cuda(), save_stats=True)
    o1 = cdl.ops.norm_fwd(x.cuda(), opts)
    o2 = cdl.ops.norm_fwd(x.cuda(), opts)
    assert torch.equal(o1.y, o2.y) and torch.equal(o1.r_inv, o2.r_inv)
    y_ref, r_ref = oracle.rmsnorm_fwd(to_f32(x), to_f32(w), None, 1e-6)
    assert_all_close("y", to_f32(o1.y), y_ref, oracle.abs_rel_tolerance(y_ref, 1e-5, 2.0 ** -7))
    assert_all_close("r_inv", to_f32(o1.r_inv), r_ref, oracle.abs_rel_tolerance(r_ref, 1e-6, 1e-4))
    rel = np.abs(to_f32(o1.y) - y_ref).max() / np.abs(y_ref).max()
    assert rel <= 1e-2


def test_fwd_empty_and_errors(cdl, gpu_ok):
    dev = "cuda"
    out = cdl.ops.norm_fwd(torch.zeros(0, 128, dtype=torch.bfloat16, device=dev))
    assert out.y.shape == (0, 128)
    with pytest.raises(cdl._lib.CdlError, match="2D"):
        cdl.ops.norm_fwd(torch.zeros(2, 4, 128, dtype=torch.bfloat16, device=dev))
    with pytest.raises(cdl._lib.CdlError, match=r"shape \[128\]"):
        cdl.ops.norm_fwd(torch.zeros(4, 128, dtype=torch.bfloat16, device=dev),
                         cdl.ops.NormFwdOpts(scale=torch.zeros(64, dtype=torch.bfloat16, device=dev)))
    with pytest.raises(cdl._lib.CdlError, match="f32 or bf16"):
        cdl.ops.norm_fwd(torch.zeros(4, 128, dtype=torch.float16, device=dev))
    with pytest.raises(cdl._lib.CdlError, match=r"r_inv must be f32 \[4\]"):
        L = cdl._lib
        x = torch.zeros(4, 100, dtype=torch.float32, device=dev)
        y, bad = torch.empty_like(x), torch.zeros(5, dtype=torch.float32, device=dev)
        args = [L.tensor_arg(t) for t in (x, None, None, y, bad)]
        L.check(L.lib.cdl_b200_rmsnorm_fwd(L.ref(args[0]), None, None, 1e-6, L.ref(args[3]),
                                           L.ref(args[4]), None))


@pytest.mark.parametrize("rows,cols", [(1, 128), (37, 2048), (300, 1536), (1000, 2048), (64, 136),
                                       (50, 4096), (33, 8192)])
@pytest.mark.parametrize("residual", [False, True])
@pytest.mark.parametrize("variant", [1, 2], ids=["warp_per_row", "pipelined"])
def test_bwd_cases(cdl, gpu_ok, rows, cols, residual, variant):
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(rows, cols, generator=gen).to(torch.bfloat16)
    dy = torch.randn(rows, cols, generator=gen).to(torch.bfloat16)
    w = (1 + 0.02 * torch.randn(cols, generator=gen)).to(torch.bfloat16)
    res = torch.randn(rows, cols, generator=gen).to(torch.bfloat16) if residual else None
    dscale0 = torch.randn(cols, generator=gen)
    fwd = cdl.ops.norm_fwd(x.cuda(), cdl.ops.NormFwdOpts(scale=w.cuda(), save_stats=True))
    dscale = dscale0.cuda().clone()
    dx = cdl.ops.norm_bwd(x.cuda(), dy.cuda(), w.cuda(), fwd.r_inv, dscale,
                          residual_dy=None if res is None else res.cuda(), variant=variant)
    dx_ref, ds_ref = oracle.rmsnorm_bwd(to_f32(x), to_f32(dy), to_f32(w),
                                        None if res is None else to_f32(res), 1e-6,
                                        dscale_init=to_f32(dscale0))
    assert_all_close("dx", to_f32(dx), dx_ref, oracle.abs_rel_tolerance(dx_ref, 1e-4, 2.0 ** -7))
    # dscale is an f32 sum over rows of products of bf16 values.
    bound = np.abs(to_f32(dy) * to_f32(x)).sum(axis=0) * 3.0 + np.abs(to_f32(dscale0))
    assert_all_close("dscale", to_f32(dscale), ds_ref, 1e-5 + 1e-5 * bound + 1e-4 * np.abs(ds_ref))


def test_bwd_config2_determinism(cdl, gpu_ok):
    gen = torch.Generator().manual_seed(1)
    x = torch.randn(16384, 2048, generator=gen).to(torch.bfloat16).cuda()
    w = (1 + 0.02 * torch.randn(2048, generator=gen)).to(torch.bfloat16).cuda()
    dy = torch.randn(16384, 2048, generator=gen).to(torch.bfloat16).cuda()
    fwd = cdl.ops.norm_fwd(x, cdl.ops.NormFwdOpts(scale=w, save_stats=True))
    ds1 = torch.zeros(2048, device="cuda")
    ds2 = torch.zeros(2048, device="cuda")
    dx1 = cdl.ops.norm_bwd(x, dy, w, fwd.r_inv, ds1)
    dx2 = cdl.ops.norm_bwd(x, dy, w, fwd.r_inv, ds2)
    assert torch.equal(dx1, dx2) and torch.equal(ds1, ds2)
    dx_ref, ds_ref = oracle.rmsnorm_bwd(to_f32(x), to_f32(dy), to_f32(w), None, 1e-6)
    assert np.abs(to_f32(dx1) - dx_ref).max() / np.abs(dx_ref).max() <= 1e-2
    assert np.abs(to_f32(ds1) - ds_ref).max() / np.abs(ds_ref).max() <= 1e-2


def test_bwd_many_launches_back_to_back(cdl, gpu_ok):
    """Thirty launches of the pipelined backward replayed from one CUDA graph on alternating
    buffers, 443 rows per CTA.  The consumer warps of its shared-memory ring run independently; a
    warp that reached a stage's next use before the previous use was taken once passed the parity
    wait on a stale phase (garbage rows, then a stalled ring: status 711 / 712).  Every launch must
    reproduce the single-launch result bit for bit and leave the status word clear."""
    rows, cols, nb, launches = 65536, 2048, 2, 30
    gen = torch.Generator(device="cuda").manual_seed(5)
    rnd = lambda: torch.randn(rows, cols, device="cuda", generator=gen).to(torch.bfloat16)
    xs, dys, rss = [rnd() for _ in range(nb)], [rnd() for _ in range(nb)], [rnd() for _ in range(nb)]
    w = (1 + 0.02 * torch.randn(cols, device="cuda", generator=gen)).to(torch.bfloat16)
    r_invs = [cdl.ops.norm_fwd(x, cdl.ops.NormFwdOpts(scale=w, save_stats=True)).r_inv for x in xs]
    scr = torch.empty(cdl.ops.norm_bwd_scratch_bytes(rows, cols), dtype=torch.uint8, device="cuda")
    want = []
    for j in range(nb):
        ds = torch.zeros(cols, device="cuda")
        want.append((cdl.ops.norm_bwd(xs[j], dys[j], w, r_invs[j], ds, residual_dy=rss[j], scratch=scr), ds))
    torch.cuda.synchronize()
    dxs = [torch.empty_like(xs[0]) for _ in range(nb)]
    dss = [torch.zeros(cols, device="cuda") for _ in range(launches)]
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(launches):
                j = i % nb
                cdl.ops.norm_bwd(xs[j], dys[j], w, r_invs[j], dss[i], residual_dy=rss[j], scratch=scr, dx=dxs[j])
        for _ in range(3):
            graph.replay()
    torch.cuda.synchronize()
    assert cdl._lib.device_status() == 0
    for j in range(nb):
        assert torch.equal(dxs[j], want[j][0])
    for i in range(launches):
        assert torch.equal(dss[i], want[i % nb][1] * 3), i  # three replays accumulate into dscale


def layernorm_reference(x, scale, bias, eps):
    """The reference's test oracle for NormType::LayerNorm (crates/cleandl/tests/norm.rs:97-130), f64."""
    x = x.astype(np.float64)
    mean = x.mean(axis=1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=1, keepdims=True)
    r = 1.0 / np.sqrt(var + eps)
    y = (x - mean) * r
    if scale is not None:
        y = y * scale.astype(np.float64)
    if bias is not None:
        y = y + bias.astype(np.float64)
    return y, mean[:, 0], r[:, 0]


@pytest.mark.parametrize("rows,cols", CASES)
@pytest.mark.parametrize("affine", ["none", "scale_bias"])
def test_layernorm_fwd_cases(cdl, gpu_ok, rows, cols, affine):
    """NormType::LayerNorm: y within 1e-5 + 2^-7 |e|, mean and r_inv within 1e-5 / 1e-6 + 1e-4 |e|
    (crates/cleandl/tests/norm.rs:261-268, 295-315)."""
    x, scale, bias = make_inputs(rows, cols, 1)
    s = scale if affine != "none" else None
    b = bias if affine != "none" else None
    out = cdl.ops.norm_fwd(x.cuda(), cdl.ops.NormFwdOpts(
        scale=None if s is None else s.cuda(), bias=None if b is None else b.cuda(), eps=1e-6,
        save_stats=True, norm_type="layer"))
    y_ref, m_ref, r_ref = layernorm_reference(to_f32(x), None if s is None else to_f32(s),
                                              None if b is None else to_f32(b), 1e-6)
    assert_all_close("y", to_f32(out.y), y_ref, oracle.abs_rel_tolerance(y_ref, 1e-5, 2.0 ** -7))
    assert_all_close("mean", to_f32(out.mean), m_ref, oracle.abs_rel_tolerance(m_ref, 1e-5, 1e-4))
    assert_all_close("r_inv", to_f32(out.r_inv), r_ref, oracle.abs_rel_tolerance(r_ref, 1e-6, 1e-4))


F32, BF16 = torch.float32, torch.bfloat16


def _general_case(cdl, rows, cols, norm_type, x_ty, out_ty, scale_ty, bias_ty, seed=2, eps=1e-6,
                  col_stride=1):
    gen = torch.Generator().manual_seed(seed)
    x = (torch.randn(rows, cols * col_stride, generator=gen) * 2.0 + 0.5).to(x_ty)[:, ::col_stride]
    scale = None if scale_ty is None else (torch.rand(cols, generator=gen) + 0.5).to(scale_ty)
    bias = None if bias_ty is None else torch.randn(cols, generator=gen).to(bias_ty)
    xd = torch.empty(0, dtype=x_ty).set_(x.untyped_storage()).cuda().as_strided(
        x.shape, x.stride(), x.storage_offset())
    out = cdl.ops.norm_fwd(xd, cdl.ops.NormFwdOpts(
        scale=None if scale is None else scale.cuda(), bias=None if bias is None else bias.cuda(),
        eps=eps, save_stats=True, norm_type=norm_type, out=out_ty))
    assert out.y.dtype == out_ty
    xs, ss, bs = to_f32(x), None if scale is None else to_f32(scale), None if bias is None else to_f32(bias)
    if norm_type == "layer":
        y_ref, m_ref, r_ref = layernorm_reference(xs, ss, bs, eps)
        assert_all_close("mean", to_f32(out.mean), m_ref, oracle.abs_rel_tolerance(m_ref, 1e-5, 1e-4))
    else:
        y_ref, r_ref = oracle.rmsnorm_fwd(xs, ss, bs, eps)
    rel = 2.0 ** -7 if out_ty == BF16 else 1e-4
    assert_all_close("y", to_f32(out.y), y_ref, oracle.abs_rel_tolerance(y_ref, 1e-5, rel))
    assert_all_close("r_inv", to_f32(out.r_inv), r_ref, oracle.abs_rel_tolerance(r_ref, 1e-6, 1e-4))


@pytest.mark.parametrize("norm_type", ["rms", "layer"])
@pytest.mark.parametrize("x_ty,out_ty", [(F32, F32), (F32, BF16), (BF16, F32), (BF16, BF16)])
@pytest.mark.parametrize("scale_ty,bias_ty", [(None, None), (F32, BF16), (BF16, F32)])
def test_general_path_type_matrix(cdl, gpu_ok, norm_type, x_ty, out_ty, scale_ty, bias_ty):
    """The type matrix of the reference's fallback_configurations test
    (crates/cleandl/tests/norm.rs:414-437) on its [77, 1000] shape: every combination of f32 / bf16
    input, output, scale and bias, both norm types; f32 outputs within 1e-5 + 1e-4 |e| (:266-268)."""
    _general_case(cdl, 77, 1000, norm_type, x_ty, out_ty, scale_ty, bias_ty)


@pytest.mark.parametrize("norm_type", ["rms", "layer"])
def test_general_path_shapes(cdl, gpu_ok, norm_type):
    """Long rows (tests/norm.rs:438-446), a column count past the vectorised kernels' 8192 (:471-475),
    one that is not a multiple of 8, eps 1e-3 on [50, 3000] (:454-462), strided columns."""
    _general_case(cdl, 9, 20000, norm_type, F32, F32, F32, None)
    _general_case(cdl, 31, 8200, norm_type, BF16, BF16, None, None)
    _general_case(cdl, 50, 3000, norm_type, BF16, BF16, BF16, None, eps=1e-3)
    _general_case(cdl, 13, 100, norm_type, BF16, BF16, BF16, BF16)
    _general_case(cdl, 20, 96, norm_type, BF16, F32, None, None, col_stride=2)
