"""GPU parity of the tcgen05 GEMM against the f64 oracle, through the C ABI.

Cases follow crates/cleandl/tests/matmul.rs: shapes and output types (:212-240), transposed views
(:268-310), sliced views (:313-339), batched (:666-687), batched + transposed + C with alpha/beta
(:632-663), accumulate into C (:690-725), unaligned operands (:604-630), f32 inputs (:243-265),
K = 0 (:825-843), rejection messages (:355-468), with the
tolerance of :199-202.  The acceptance bound of this build (max relative error 2e-2 against an
f32-accumulated reference) is checked as well.
"""
import numpy as np
import pytest
import torch

from helpers import assert_all_close, to_f32
from oracle import cpu_oracle as oracle

pytestmark = pytest.mark.gpu


def rand_bf16(gen, *shape):
    # Uniform(-1, 1) rounded to bf16, like random_bf16 of the reference tests (:120-148).
    return (torch.rand(*shape, generator=gen) * 2 - 1).to(torch.bfloat16)


def run_case(cdl, a, b, out_dtype, c=None, alpha=1.0, beta=0.0, in_place=False):
    """a, b, c: CPU tensors (possibly views). Runs on the GPU and compares with the oracle."""
    dev = "cuda"

    def to_dev(t):
        # Preserve the view's strides: move the base storage and re-view.
        base = torch.empty(0, dtype=t.dtype).set_(t.untyped_storage())
        return base.to(dev).as_strided(t.shape, t.stride(), t.storage_offset())

    da, db = to_dev(a), to_dev(b)
    dc = to_dev(c) if c is not None else None
    opts = cdl.ops.MatmulOpts(out=out_dtype, c=dc, alpha=alpha, beta=beta)
    d = cdl.ops.matmul(da, db, opts, out=dc if in_place else None)
    expected, bound = oracle.matmul(to_f32(a), to_f32(b), None if c is None else to_f32(c), alpha, beta)
    tol = oracle.matmul_tolerance(expected, bound, out_dtype == torch.bfloat16)
    assert_all_close("matmul", to_f32(d), expected, tol)
    # Acceptance bound: max relative error 2e-2 (relative to the largest magnitude of the output).
    scale = max(float(np.abs(expected).max()), 1e-6)
    assert float(np.abs(to_f32(d) - expected).max()) / scale <= 2e-2
    return d


@pytest.mark.parametrize("shape", [(64, 64, 64), (129, 264, 72), (1, 8, 8), (300, 520, 136),
                                   (512, 512, 512), (256, 1024, 4096 + 8)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_shapes_and_outputs(cdl, gpu_ok, shape, out_dtype):
    m, k, n = shape
    gen = torch.Generator().manual_seed(0)
    run_case(cdl, rand_bf16(gen, m, k), rand_bf16(gen, k, n), out_dtype)


@pytest.mark.parametrize("ta,tb", [(True, False), (False, True), (True, True)])
def test_transposed_views(cdl, gpu_ok, ta, tb):
    m, k, n = 136, 200, 264
    gen = torch.Generator().manual_seed(1)
    a = rand_bf16(gen, k, m).T if ta else rand_bf16(gen, m, k)
    b = rand_bf16(gen, n, k).T if tb else rand_bf16(gen, k, n)
    run_case(cdl, a, b, torch.bfloat16)


def test_sliced_views(cdl, gpu_ok):
    gen = torch.Generator().manual_seed(2)
    a = rand_bf16(gen, 200, 320)[8:136, 64:64 + 128]
    b = rand_bf16(gen, 256, 400)[16:16 + 128, 8:8 + 200]
    run_case(cdl, a, b, torch.float32)


def test_batched(cdl, gpu_ok):
    gen = torch.Generator().manual_seed(3)
    run_case(cdl, rand_bf16(gen, 3, 130, 72), rand_bf16(gen, 3, 72, 264), torch.bfloat16)


def test_batched_transposed_with_c(cdl, gpu_ok):
    gen = torch.Generator().manual_seed(4)
    a = rand_bf16(gen, 2, 72, 136).transpose(1, 2)
    b = rand_bf16(gen, 2, 200, 72).transpose(1, 2)
    c = rand_bf16(gen, 2, 136, 200)
    run_case(cdl, a, b, torch.bfloat16, c=c, alpha=2.0, beta=0.5)


@pytest.mark.parametrize("c_dtype", [torch.bfloat16, torch.float32])
def test_accumulate_c(cdl, gpu_ok, c_dtype):
    gen = torch.Generator().manual_seed(5)
    a, b = rand_bf16(gen, 150, 264), rand_bf16(gen, 264, 96)
    c = rand_bf16(gen, 150, 96).to(c_dtype)
    run_case(cdl, a, b, c_dtype, c=c, alpha=0.5, beta=-2.0)


def test_wgrad_shape_in_place_f32(cdl, gpu_ok):
    """dW[K_in, N_out] (f32) += X^T . dY with the reduction over tokens, written into C."""
    gen = torch.Generator().manual_seed(6)
    x, dy = rand_bf16(gen, 1000, 256), rand_bf16(gen, 1000, 520)
    w = torch.randn(256, 520, generator=gen)
    run_case(cdl, x.T, dy, torch.float32, c=w, alpha=1.0, beta=1.0, in_place=True)


def test_unaligned_output_rows(cdl, gpu_ok):
    """N not a multiple of 8: output rows are not 16-byte aligned, scalar stores take over."""
    gen = torch.Generator().manual_seed(7)
    a = rand_bf16(gen, 70, 64)
    b = rand_bf16(gen, 64, 72)[:, :65]
    run_case(cdl, a, b, torch.bfloat16)
    run_case(cdl, a, b, torch.float32)


@pytest.mark.parametrize("m,k,n", [(37, 64, 65), (40, 72, 1), (16, 24, 8), (200, 333, 129)])
def test_unaligned_operands(cdl, gpu_ok, m, k, n):
    """The reference's unaligned_operands test (crates/cleandl/tests/matmul.rs:604-630): A starts 3
    elements into rows of k + 3 elements (pointer and leading dimension off the 16-byte grid), B
    is the transposed view of an [n, k] matrix.  TMA cannot describe these; the general kernel
    computes them."""
    gen = torch.Generator().manual_seed(110)
    a = rand_bf16(gen, m, k + 3)[:, 3:]
    b = rand_bf16(gen, n, k).T
    run_case(cdl, a, b, torch.bfloat16)
    run_case(cdl, a, b, torch.float32)
    c = torch.randn(m, n, generator=gen)
    run_case(cdl, a, b, torch.float32, c=c, alpha=0.5, beta=2.0)


def test_unaligned_batched(cdl, gpu_ok):
    gen = torch.Generator().manual_seed(111)
    a = rand_bf16(gen, 3, 50, 45)[:, :, 1:41]     # [3, 50, 40], row stride 45
    b = rand_bf16(gen, 3, 33, 40).transpose(1, 2)  # [3, 40, 33], K contiguous
    run_case(cdl, a, b, torch.bfloat16)


@pytest.mark.parametrize("shape", [(96, 200, 136), (130, 64, 70)])
def test_f32_inputs(cdl, gpu_ok, shape):
    """The reference's f32_tf32_matmul test (tests/matmul.rs:243-265): f32 x f32 -> f32 within the
    TF32 tolerance 2e-3 * sum |a b| + 1e-5 (the products here are full f32)."""
    m, k, n = shape
    gen = torch.Generator().manual_seed(10)
    a = torch.rand(m, k, generator=gen) * 2 - 1
    b = torch.rand(k, n, generator=gen) * 2 - 1
    d = cdl.ops.matmul(a.cuda(), b.cuda(), cdl.ops.MatmulOpts(out=torch.float32))
    expected, bound = oracle.matmul(to_f32(a), to_f32(b), None, 1.0, 0.0)
    assert_all_close("f32 inputs", to_f32(d), expected, 2e-3 * bound + 1e-5)
    dt = cdl.ops.matmul(a.T.contiguous().cuda().T, b.cuda(), cdl.ops.MatmulOpts(out=torch.bfloat16))
    assert_all_close("f32 inputs, transposed a, bf16 out", to_f32(dt), expected,
                     oracle.matmul_tolerance(expected, bound, True))


def test_deterministic(cdl, gpu_ok):
    gen = torch.Generator().manual_seed(8)
    a, b = rand_bf16(gen, 1024, 2048).cuda(), rand_bf16(gen, 2048, 1536).cuda()
    d1 = cdl.ops.matmul(a, b)
    d2 = cdl.ops.matmul(a, b)
    assert torch.equal(d1, d2)


def test_pair_kernel_on_several_streams_at_once(cdl, gpu_ok):
    """The CTA-pair kernel draws its work units from a counter that belongs to the launching
    stream.  Products with many more tiles than the device has clusters, enqueued on four streams
    so that they overlap on the device, each repeated back to back on its stream, must all equal
    the product computed alone (bit for bit: bf16 output, no K slices), and the next launch on a
    stream must find its counter at zero again."""
    gen = torch.Generator(device="cuda").manual_seed(17)
    m, k, n = 4096, 512, 4096  # 256 tiles of 256 x 256 on 74 clusters
    streams = [torch.cuda.Stream() for _ in range(4)]
    ab = [(torch.randn(m, k, device="cuda", generator=gen).to(torch.bfloat16),
           torch.randn(k, n, device="cuda", generator=gen).to(torch.bfloat16)) for _ in streams]
    want = [cdl.ops.matmul(a, b) for a, b in ab]
    torch.cuda.synchronize()
    got = [[None] * 6 for _ in streams]
    for rep in range(6):
        for i, st in enumerate(streams):
            with torch.cuda.stream(st):
                got[i][rep] = cdl.ops.matmul(*ab[i])
    torch.cuda.synchronize()
    assert cdl._lib.device_status() == 0
    for i in range(len(streams)):
        for rep in range(6):
            assert torch.equal(got[i][rep], want[i]), (i, rep)


def test_weight_gradient_form_summation_order_option(cdl, gpu_ok):
    """D (f32) += A^T . B with a long contraction: by default the K slices meet in D through f32
    atomics, so two runs agree only within the f32 summation bound; with the `deterministic`
    option (cdl_matmul_options) two runs are bit-equal.  Both agree with the oracle, and every
    candidate the library enumerates for the problem gives a result within tolerance."""
    gen = torch.Generator().manual_seed(12)
    x, dy = rand_bf16(gen, 8192, 512).cuda(), rand_bf16(gen, 8192, 768).cuda()
    w0 = torch.randn(512, 768, generator=gen).cuda()
    expected, bound = oracle.matmul(to_f32(x.T), to_f32(dy), to_f32(w0), 1.0, 1.0)
    tol = oracle.matmul_tolerance(expected, bound, False)

    def run(**kw):
        w = w0.clone()
        cdl.ops.matmul(x.T, dy, cdl.ops.MatmulOpts(out=torch.float32, c=w, beta=1.0, **kw), out=w)
        return w

    d1, d2 = run(deterministic=True), run(deterministic=True)
    assert torch.equal(d1, d2)
    assert_all_close("deterministic wgrad", to_f32(d1), expected, tol)
    f1, f2 = run(), run()
    assert_all_close("sliced wgrad", to_f32(f1), expected, tol)
    assert (f1 - f2).abs().max().item() <= 1e-5 * float(np.abs(bound).max())
    cands = cdl.ops.matmul_candidates(x.T, dy, w0)
    assert cands[0] == (cdl._lib.GEMM_CTA_PAIR, False) and len(cands) >= 3
    for variant, det in cands:
        assert_all_close(f"candidate {variant} {det}", to_f32(run(variant=variant, deterministic=det)),
                         expected, tol)


def test_large_vs_f32_accumulated(cdl, gpu_ok):
    """A block-sized forward GEMM against a float32-accumulated torch product on the same GPU
    (the f64 oracle would take minutes at this size)."""
    gen = torch.Generator().manual_seed(9)
    a = (torch.randn(4096, 2048, generator=gen)).to(torch.bfloat16).cuda()
    b = (torch.randn(2048, 5632, generator=gen) * 0.02).to(torch.bfloat16).cuda()
    d = cdl.ops.matmul(a, b).float()
    ref = a.float() @ b.float()
    rel = (d - ref).abs().max() / ref.abs().max()
    assert rel.item() <= 2e-2
    # dgrad (B transposed view) and wgrad (A transposed view) of the same layer
    dy = torch.randn(4096, 5632, generator=gen).to(torch.bfloat16).cuda()
    dx = cdl.ops.matmul(dy, b.T).float()
    ref = dy.float() @ b.float().T
    assert ((dx - ref).abs().max() / ref.abs().max()).item() <= 2e-2
    dw = cdl.ops.matmul(a.T, dy, cdl.ops.MatmulOpts(out=torch.float32))
    ref = a.float().T @ dy.float()
    assert ((dw - ref).abs().max() / ref.abs().max()).item() <= 2e-2


def test_empty_and_errors(cdl, gpu_ok):
    dev = "cuda"
    a = torch.zeros(0, 64, dtype=torch.bfloat16, device=dev)
    b = torch.zeros(64, 32, dtype=torch.bfloat16, device=dev)
    assert cdl.ops.matmul(a, b).shape == (0, 32)  # empty output: silent success
    with pytest.raises(cdl._lib.CdlError, match="K is zero"):
        cdl.ops.matmul(torch.zeros(8, 0, dtype=torch.bfloat16, device=dev),
                       torch.zeros(0, 8, dtype=torch.bfloat16, device=dev))
    with pytest.raises(cdl._lib.CdlError, match="contraction"):
        cdl.ops.matmul(torch.zeros(8, 16, dtype=torch.bfloat16, device=dev),
                       torch.zeros(24, 8, dtype=torch.bfloat16, device=dev))
    with pytest.raises(cdl._lib.CdlError, match="rank"):
        cdl.ops.matmul(torch.zeros(8, 16, dtype=torch.bfloat16, device=dev),
                       torch.zeros(2, 16, 8, dtype=torch.bfloat16, device=dev))
    with pytest.raises(cdl._lib.CdlError, match="f32 or bf16"):
        cdl.ops.matmul(torch.zeros(8, 16, dtype=torch.bfloat16, device=dev),
                       torch.zeros(16, 8, dtype=torch.float32, device=dev))
    with pytest.raises(cdl._lib.CdlError, match="contiguous"):
        cdl.ops.matmul(torch.zeros(16, 32, dtype=torch.bfloat16, device=dev)[::2, ::2],
                       torch.zeros(16, 8, dtype=torch.bfloat16, device=dev))
    # The fused epilogues exist on the tensor-memory path only: unaligned operands are rejected there.
    L = cdl._lib
    a65 = torch.zeros(37, 65, dtype=torch.bfloat16, device=dev)[:, :64]
    b8 = torch.zeros(64, 8, dtype=torch.bfloat16, device=dev)
    up = torch.zeros(37, 8, dtype=torch.bfloat16, device=dev)
    gate, act = torch.empty_like(up), torch.empty_like(up)
    args = [L.tensor_arg(t) for t in (a65, b8, up, gate, act)]
    with pytest.raises(L.CdlError, match="16-byte"):
        L.check(L.lib.cdl_b200_matmul_swiglu_gate(*(L.ref(t) for t in args), None))


@pytest.mark.parametrize("m,n,k", [(300, 264, 136), (128, 72, 64), (1024, 512, 256)])
def test_fused_swiglu_epilogues(cdl, gpu_ok, m, n, k):
    """GEMM + SwiGLU in one kernel (the reference's swiglu_gate_train_fwd / swiglu_down_train_dgrad
    kernels) against float64: gate/act forward and d_up/d_gate backward."""
    L = cdl._lib
    gen = torch.Generator().manual_seed(21)
    a = rand_bf16(gen, m, k)
    b = (torch.randn(k, n, generator=gen) * 0.3).to(torch.bfloat16)
    up = rand_bf16(gen, m, n)
    gate_in = (torch.randn(m, n, generator=gen) * 2).to(torch.bfloat16)
    da, db, dup, dgi = a.cuda(), b.cuda(), up.cuda(), gate_in.cuda()
    gate_out, act_out = torch.empty_like(dup), torch.empty_like(dup)
    args = [L.tensor_arg(t) for t in (da, db, dup, gate_out, act_out)]
    L.check(L.lib.cdl_b200_matmul_swiglu_gate(*(L.ref(x) for x in args), None))
    d_up, d_gate = torch.empty_like(dup), torch.empty_like(dup)
    args = [L.tensor_arg(t) for t in (da, db, dgi, dup, d_up, d_gate)]
    L.check(L.lib.cdl_b200_matmul_swiglu_dgrad(*(L.ref(x) for x in args), None))
    torch.cuda.synchronize()
    prod = a.double() @ b.double()
    sig = torch.sigmoid

    def rel(got, ref):
        return ((got.double().cpu() - ref).abs().max() / ref.abs().max()).item()

    assert rel(gate_out, prod) <= 2.0 ** -7
    assert rel(act_out, prod * sig(prod) * up.double()) <= 2.0 ** -6
    g = gate_in.double()
    assert rel(d_up, g * sig(g) * prod) <= 2.0 ** -6
    assert rel(d_gate, prod * up.double() * (sig(g) + g * sig(g) * (1 - sig(g)))) <= 2.0 ** -6
