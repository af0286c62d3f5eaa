"""Block-scaled (MXFP8) tensors: oracle pins on CPU, GPU parity through the C ABI.

Follows the reference's tests of the format: the host quantiser and the dequantised checks of
crates/cleandl/tests/matmul.rs:885-952, 1041-1060 (block-scaled matmul inputs, tolerance of
`tolerance(out, bounds)` :199-202), and the block-scaled norm outputs of
crates/cleandl/tests/norm.rs:134-149, 322-380 (|got - y| <= 0.07 |y| + 2^-9 * block scale).
"""
import ctypes

import numpy as np
import pytest
import torch

from helpers import assert_all_close, to_f32
from oracle import cpu_oracle as oracle
from oracle import mx_ref

ROW, COL = mx_ref.ROWWISE, mx_ref.COLWISE


# ------------------------------------------------------------------------------ CPU: the oracle
def test_e4m3_table_pins():
    t = mx_ref.E4M3_VALUES
    assert t[0x00] == 0.0 and t[0x01] == 2.0 ** -9 and t[0x08] == 2.0 ** -6
    assert t[0x38] == 1.0 and t[0x7E] == 448.0 and np.isnan(t[0x7F]) and t[0xFE] == -448.0
    finite = t[:0x7F]
    assert np.all(np.diff(finite) > 0)
    # every code encodes to itself; ties go to the even code; overflow saturates
    codes = np.arange(0x7F, dtype=np.uint8)
    assert np.array_equal(mx_ref.e4m3_encode(finite), codes)
    ties = (finite[:-1] + finite[1:]) / 2
    enc = mx_ref.e4m3_encode(ties)
    assert np.all(enc % 2 == 0) and np.all(np.abs(enc.astype(int) - codes[:-1]) <= 1)
    assert mx_ref.e4m3_encode(np.array([1e9, -1e9, 449.0]))[:].tolist() == [0x7E, 0xFE, 0x7E]


def test_e4m3_encode_matches_torch():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(100000) * rng.choice([1e-3, 0.02, 1, 40, 200], 100000)).astype(np.float32)
    x = np.clip(x, -448, 448)
    want = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(mx_ref.e4m3_encode(x), want)


def test_scale_factor_index_is_a_bijection_on_tiles():
    # closed form of crates/cleandl/tests/common/mod.rs:124-129 on a padded 256 x 8 block grid
    r, b = np.meshgrid(np.arange(256), np.arange(8), indexing="ij")
    idx = mx_ref.sf_index(r, b, 8)
    assert sorted(idx.ravel().tolist()) == list(range(256 * 8))
    assert mx_ref.sf_index(0, 0, 8) == 0 and mx_ref.sf_index(1, 0, 8) == 16
    assert mx_ref.sf_index(32, 0, 8) == 4 and mx_ref.sf_index(0, 1, 8) == 1
    assert mx_ref.sf_index(0, 4, 8) == 512 and mx_ref.sf_index(128, 0, 8) == 1024
    assert mx_ref.sf_index(5, 2, 3) == 5 * 16 + 2  # 3 block columns pad to one tile of 4


def test_scale_exponent():
    # amax = 448 * 2^k needs exactly scale 2^k; anything above rounds up; zero blocks get 2^-127
    e = mx_ref.scale_exponent(np.array([448.0, 448.0001, 1.0, 0.0, 3.4e38], dtype=np.float32))
    assert e.tolist() == [127, 128, 127 - 8, 0, 247]


@pytest.mark.parametrize("dim", [ROW, COL])
def test_quantize_roundtrip_within_format_error(dim):
    rng = np.random.default_rng(1)
    m = (rng.standard_normal((192, 160)) * np.exp(rng.standard_normal((192, 160)) * 2)).astype(np.float32)
    v, s = mx_ref.quantize(m, dim)
    outer, inner, sf_rows, sf_cols = mx_ref.layout(192, 160, dim)
    assert v.shape == (outer, inner) and s.shape == (sf_rows * sf_cols,)
    d, es = mx_ref.dequantize(v, s, 192, 160, dim)
    assert np.all(np.abs(d - m) <= 2.0 ** -4 * np.abs(m) + 2.0 ** -10 * es * 1.0001)
    # no element overflows its block: |x| / scale <= 448
    assert np.all(np.abs(m) <= 448.0 * es)


def test_layout_through_the_c_abi(cdl):
    for rows, cols in [(1, 128), (300, 2048), (96, 512), (256, 160)]:
        for dim in (ROW, COL):
            try:
                outer, inner, sf_rows, sf_cols = mx_ref.layout(rows, cols, dim)
            except ValueError:
                with pytest.raises(cdl._lib.CdlError, match="block size"):
                    cdl.mx.layout_bytes(rows, cols, dim)
                continue
            assert cdl.mx.layout_bytes(rows, cols, dim) == (outer * inner, sf_rows * sf_cols)
    with pytest.raises(cdl._lib.CdlError, match="unknown format"):
        cdl.mx.layout_bytes(128, 128, ROW, fmt=7)


def test_host_validation_needs_no_gpu(cdl):
    L = cdl._lib
    x = L.CdlTensor(ptr=256, dtype=L.CDL_BF16, rank=2)
    x.shape[0], x.shape[1], x.stride[0], x.stride[1] = 4, 48, 48, 1
    y = L.CdlMxTensor(512, 1024, L.CDL_MXFP8, L.CDL_MX_ROWWISE, 4, 48)
    st = L.lib.cdl_b200_rmsnorm_fwd_mx(ctypes.byref(x), None, None, 1e-6, ctypes.byref(y), None, None, None)
    assert st == -1 and "block size" in L.last_error()
    x.shape[0], x.shape[1], x.stride[0] = 48, 64, 64
    y = L.CdlMxTensor(512, 1024, L.CDL_MXFP8, L.CDL_MX_ROWWISE, 48, 64)
    yc = L.CdlMxTensor(512, 1024, L.CDL_MXFP8, L.CDL_MX_COLWISE, 48, 64)
    st = L.lib.cdl_b200_rmsnorm_fwd_mx(ctypes.byref(x), None, None, 1e-6, ctypes.byref(y), ctypes.byref(yc),
                                       None, None)
    assert st == -1 and "block size" in L.last_error()
    # matmul: A must be rowwise, B colwise, contraction dimensions equal
    a = L.CdlMxTensor(512, 1024, L.CDL_MXFP8, L.CDL_MX_COLWISE, 128, 64)
    b = L.CdlMxTensor(512, 1024, L.CDL_MXFP8, L.CDL_MX_COLWISE, 64, 128)
    d = L.CdlTensor(ptr=2048, dtype=L.CDL_BF16, rank=2)
    d.shape[0], d.shape[1], d.stride[0], d.stride[1] = 128, 128, 128, 1
    st = L.lib.cdl_b200_matmul_mx(ctypes.byref(a), ctypes.byref(b), None, ctypes.byref(d), 1.0, 0.0, None)
    assert st == -1 and "contraction" in L.last_error()
    a = L.CdlMxTensor(512, 1024, L.CDL_MXFP8, L.CDL_MX_ROWWISE, 128, 64)
    b = L.CdlMxTensor(512, 1024, L.CDL_MXFP8, L.CDL_MX_COLWISE, 96, 128)
    st = L.lib.cdl_b200_matmul_mx(ctypes.byref(a), ctypes.byref(b), None, ctypes.byref(d), 1.0, 0.0, None)
    assert st == -1 and "contraction" in L.last_error()


# ------------------------------------------------------------------------------ GPU parity
def valid_scales(t, scales_np):
    """Scale bytes of the real blocks of an MxTensor (padding bytes are unspecified)."""
    outer, inner, _, _ = mx_ref.layout(t.rows, t.cols, t.dim)
    blocks = inner // 32
    o, b = np.meshgrid(np.arange(outer), np.arange(blocks), indexing="ij")
    return scales_np[mx_ref.sf_index(o, b, blocks)]


def rand_bf16(rows, cols, seed, spread=2.0):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=gen) * torch.exp(torch.randn(rows, cols, generator=gen) * spread)
    return x.to(torch.bfloat16)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", [(1, 128), (37, 4096), (300, 2048), (128, 8192), (96, 512),
                                        (64, 160), (256, 7168), (4, 16384), (32, 12288), (8, 256),
                                        (64, 768), (160, 1280), (32, 2304)])
def test_quantize_is_bit_exact(cdl, gpu_ok, rows, cols):
    x = rand_bf16(rows, cols, 10)
    x[0, :32] = 0  # an all-zero block
    if rows > 1:
        x[1, :32] = 448.0  # exactly representable amax
    col = rows % 32 == 0
    yr, yc = cdl.mx.quantize(x.cuda(), rowwise=True, colwise=col)
    for t, dim in ((yr, ROW), (yc, COL)):
        if t is None:
            continue
        v_ref, s_ref = mx_ref.quantize(to_f32(x), dim)
        assert np.array_equal(t.values.cpu().numpy(), v_ref), f"values dim {dim}"
        assert np.array_equal(valid_scales(t, t.scale_factors.cpu().numpy()), valid_scales(t, s_ref))
        d_ref, _ = mx_ref.dequantize(v_ref, s_ref, rows, cols, dim)
        assert np.array_equal(to_f32(cdl.mx.dequantize(t)), d_ref)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", [(64, 512), (96, 4352), (32, 72)])
def test_quantize_colwise_only_is_bit_exact(cdl, gpu_ok, rows, cols):
    x = rand_bf16(rows, cols, 12)
    yr, yc = cdl.mx.quantize(x.cuda(), rowwise=False, colwise=True)
    assert yr is None
    v_ref, s_ref = mx_ref.quantize(to_f32(x), COL)
    assert np.array_equal(yc.values.cpu().numpy(), v_ref)
    assert np.array_equal(valid_scales(yc, yc.scale_factors.cpu().numpy()), valid_scales(yc, s_ref))


@pytest.mark.gpu
def test_quantize_strided_rows(cdl, gpu_ok):
    big = rand_bf16(64, 1024, 11).cuda()
    x = big[:, 256:768]
    yr, yc = cdl.mx.quantize(x, rowwise=True, colwise=True)
    v_ref, _ = mx_ref.quantize(to_f32(x), ROW)
    assert np.array_equal(yr.values.cpu().numpy(), v_ref)
    v_ref, _ = mx_ref.quantize(to_f32(x), COL)
    assert np.array_equal(yc.values.cpu().numpy(), v_ref)


NORM_CASES = [(1, 128), (37, 4096), (300, 2048), (128, 8192), (100, 7168), (5, 1024), (96, 512),
              (320, 1536), (16384, 2048), (3, 16384), (64, 256), (40, 768), (64, 4096),
              (32, 6144), (64, 5120), (32, 3584)]


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", NORM_CASES)
@pytest.mark.parametrize("affine", ["none", "scale", "scale_bias"])
def test_norm_fwd_mx(cdl, gpu_ok, rows, cols, affine):
    if rows == 16384 and affine != "scale":
        pytest.skip("the full-size case runs once")
    gen = torch.Generator().manual_seed(1)
    x = (torch.randn(rows, cols, generator=gen) * 2.0 + 0.5).to(torch.bfloat16)
    scale = (torch.rand(cols, generator=gen) + 0.5).to(torch.bfloat16) if affine != "none" else None
    bias = torch.randn(cols, generator=gen).to(torch.bfloat16) if affine == "scale_bias" else None
    col = rows % 32 == 0
    out = cdl.mx.norm_fwd_mx(x.cuda(), None if scale is None else scale.cuda(),
                             None if bias is None else bias.cuda(), 1e-6, colwise=col, save_stats=True)
    y_ref, r_ref = oracle.rmsnorm_fwd(to_f32(x), None if scale is None else to_f32(scale),
                                      None if bias is None else to_f32(bias), 1e-6)
    assert_all_close("r_inv", to_f32(out.r_inv), r_ref, oracle.abs_rel_tolerance(r_ref, 1e-6, 1e-4))
    # what quantising the bf16-rounded f64 result gives; the kernel's f32 result can differ from
    # it by a bf16 ulp in a few places, so bits are compared statistically, values by tolerance
    yb = oracle.bf16_round(y_ref.astype(np.float32))
    for t, dim in ((out.y, ROW), (out.y_col, COL)):
        if t is None:
            continue
        got, es = mx_ref.dequantize(t.values.cpu().numpy(), t.scale_factors.cpu().numpy(), rows, cols, dim)
        assert_all_close(f"y dim {dim}", got, y_ref, mx_ref.output_tolerance(y_ref, es))
        v_ref, s_ref = mx_ref.quantize(yb, dim)
        same_scale = valid_scales(t, t.scale_factors.cpu().numpy()) == valid_scales(t, s_ref)
        assert same_scale.mean() > 0.995, f"scales dim {dim}: {same_scale.mean()}"
        assert (t.values.cpu().numpy() == v_ref).mean() > 0.98, f"codes dim {dim}"
        # the device's own dequantiser agrees with the oracle's
        assert np.array_equal(to_f32(cdl.mx.dequantize(t)), got)


MM_CASES = [(192, 256, 160), (128, 32, 64), (128, 128, 256), (256, 2048, 512), (100, 96, 24),
            (384, 416, 296), (1024, 1024, 2048)]


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,n", MM_CASES)
@pytest.mark.parametrize("out", ["bf16", "f32"])
def test_matmul_mx(cdl, gpu_ok, m, k, n, out):
    """The reference's mxfp8_inputs test: the expected product is the f64 product of the
    DEQUANTISED operands; tolerance as for a plain matmul of those values."""
    gen = torch.Generator().manual_seed(80)
    a = torch.randn(m, k, generator=gen).to(torch.bfloat16)
    b = torch.randn(k, n, generator=gen).to(torch.bfloat16)
    qa, _ = cdl.mx.quantize(a.cuda(), rowwise=True)
    _, qb = cdl.mx.quantize(b.cuda(), rowwise=False, colwise=True)
    da, _ = mx_ref.dequantize(qa.values.cpu().numpy(), qa.scale_factors.cpu().numpy(), m, k, ROW)
    db, _ = mx_ref.dequantize(qb.values.cpu().numpy(), qb.scale_factors.cpu().numpy(), k, n, COL)
    dtype = torch.bfloat16 if out == "bf16" else torch.float32
    d = cdl.mx.matmul_mx(qa, qb, out_dtype=dtype)
    expected = da.astype(np.float64) @ db.astype(np.float64)
    bound = np.abs(da).astype(np.float64) @ np.abs(db).astype(np.float64)
    assert_all_close(f"mxfp8 {m}x{k}x{n} -> {out}", to_f32(d), expected,
                     oracle.matmul_tolerance(expected, bound, out == "bf16"))


@pytest.mark.gpu
def test_matmul_mx_many_tiles_and_alpha(cdl, gpu_ok):
    """More tiles than SMs (both accumulators and their shared columns in use), alpha != 1, and
    linearity in the block scales: doubling every scale of A doubles the product exactly."""
    m, k, n = 2048, 512, 4864
    gen = torch.Generator().manual_seed(81)
    a = torch.randn(m, k, generator=gen).to(torch.bfloat16)
    b = torch.randn(k, n, generator=gen).to(torch.bfloat16)
    qa, _ = cdl.mx.quantize(a.cuda(), rowwise=True)
    _, qb = cdl.mx.quantize(b.cuda(), rowwise=False, colwise=True)
    d1 = cdl.mx.matmul_mx(qa, qb, out_dtype=torch.float32)
    da, _ = mx_ref.dequantize(qa.values.cpu().numpy(), qa.scale_factors.cpu().numpy(), m, k, ROW)
    db, _ = mx_ref.dequantize(qb.values.cpu().numpy(), qb.scale_factors.cpu().numpy(), k, n, COL)
    expected = da.astype(np.float64) @ db.astype(np.float64)
    bound = np.abs(da).astype(np.float64) @ np.abs(db).astype(np.float64)
    assert_all_close("product", to_f32(d1), expected, oracle.matmul_tolerance(expected, bound, False))
    d_half = cdl.mx.matmul_mx(qa, qb, out_dtype=torch.float32, alpha=0.5)
    assert torch.equal(d_half, d1 * 0.5)
    qa2 = cdl.mx.MxTensor(qa.values, qa.scale_factors + 1, qa.dim, qa.rows, qa.cols)
    d2 = cdl.mx.matmul_mx(qa2, qb, out_dtype=torch.float32)
    assert torch.equal(d2, d1 * 2)
    # repeated runs give identical bits (a fixed accumulation order)
    assert torch.equal(cdl.mx.matmul_mx(qa, qb, out_dtype=torch.float32), d1)


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,n", [(256, 128, 192), (100, 96, 64), (1024, 512, 2048)])
@pytest.mark.parametrize("dim", [ROW, COL])
def test_matmul_mx_block_scaled_output(cdl, gpu_ok, m, k, n, dim):
    """The reference's block_scaled_outputs test (crates/cleandl/tests/matmul.rs:1083-1115): the
    dequantised output against the f64 product of the dequantised operands, within half an ulp of
    E4M3 relative to the block scale plus the accumulation error."""
    if dim == COL and m % 32:
        pytest.skip("a colwise output needs a row count that is a multiple of 32")
    gen = torch.Generator().manual_seed(100)
    a = torch.randn(m, k, generator=gen).to(torch.bfloat16)
    b = torch.randn(k, n, generator=gen).to(torch.bfloat16)
    qa, _ = cdl.mx.quantize(a.cuda(), rowwise=True)
    _, qb = cdl.mx.quantize(b.cuda(), rowwise=False, colwise=True)
    da, _ = mx_ref.dequantize(qa.values.cpu().numpy(), qa.scale_factors.cpu().numpy(), m, k, ROW)
    db, _ = mx_ref.dequantize(qb.values.cpu().numpy(), qb.scale_factors.cpu().numpy(), k, n, COL)
    expected = da.astype(np.float64) @ db.astype(np.float64)
    bound = np.abs(da).astype(np.float64) @ np.abs(db).astype(np.float64)
    d = cdl.mx.matmul_mx_out(qa, qb, dim=dim)
    assert d.dim == dim and (d.rows, d.cols) == (m, n)
    got, es = mx_ref.dequantize(d.values.cpu().numpy(), d.scale_factors.cpu().numpy(), m, n, dim)
    assert_all_close(f"mxfp8 output dim {dim}", got, expected,
                     2.0 ** -4 * np.abs(expected) + 2.0 ** -9 * es + 1e-4 * bound)
    # the output equals quantising the plain f32 product of the same kernel (same accumulation
    # order), bit for bit
    plain = cdl.mx.matmul_mx(qa, qb, out_dtype=torch.float32)
    v_ref, s_ref = mx_ref.quantize(to_f32(plain), dim)
    assert np.array_equal(d.values.cpu().numpy(), v_ref)
    assert np.array_equal(valid_scales(d, d.scale_factors.cpu().numpy()), valid_scales(d, s_ref))
    # and feeds a following matmul: (A.B) rowwise times a colwise C
    if dim == ROW and n % 32 == 0:
        c = torch.randn(n, 64, generator=gen).to(torch.bfloat16)
        _, qc = cdl.mx.quantize(c.cuda(), rowwise=False, colwise=True)
        dc, _ = mx_ref.dequantize(qc.values.cpu().numpy(), qc.scale_factors.cpu().numpy(), n, 64, COL)
        e2 = got.astype(np.float64) @ dc.astype(np.float64)
        b2 = np.abs(got).astype(np.float64) @ np.abs(dc).astype(np.float64)
        out2 = cdl.mx.matmul_mx(d, qc, out_dtype=torch.float32)
        assert_all_close("chained", to_f32(out2), e2, oracle.matmul_tolerance(e2, b2, False))


# ------------------------------------------------------------------------------ NVFP4
def test_nvfp4_oracle_pins():
    assert mx_ref.e2m1_decode(np.arange(16)).tolist() == [0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6]
    # nearest with ties to the even code, saturating
    assert mx_ref.e2m1_encode(np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.3, 0.2])).tolist() == \
        [0, 2, 2, 4, 4, 6, 6, 7, 9, 0]
    rng = np.random.default_rng(3)
    m = rng.standard_normal((64, 128)).astype(np.float32)
    for dim in (ROW, COL):
        v, s = mx_ref.quantize_nvfp4(m, dim)
        outer, inner, sf_rows, sf_cols = mx_ref.layout(64, 128, dim, mx_ref.NVFP4)
        assert v.shape == (outer, inner // 2) and s.shape == (sf_rows * sf_cols,)
        d, es = mx_ref.dequantize_nvfp4(v, s, 64, 128, dim)
        # the tolerance the reference's tests give an NVFP4 result (crates/cleandl/tests/norm.rs:144)
        assert np.all(np.abs(d - m) <= 0.34 * np.abs(m) + 0.5 * es)


def nv_valid_scales(t, scales_np):
    outer, inner, _, _ = mx_ref.layout(t.rows, t.cols, t.dim, mx_ref.NVFP4)
    blocks = inner // 16
    o, b = np.meshgrid(np.arange(outer), np.arange(blocks), indexing="ij")
    return scales_np[mx_ref.sf_index(o, b, blocks)]


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", [(1, 128), (37, 4096), (300, 2048), (128, 8192), (64, 144), (5, 1024)])
def test_nvfp4_quantize_is_bit_exact(cdl, gpu_ok, rows, cols):
    x = rand_bf16(rows, cols, 20, spread=1.0)
    x[0, :16] = 0
    yr, _ = cdl.mx.quantize(x.cuda(), rowwise=True, fmt=cdl.mx.NVFP4)
    v_ref, s_ref = mx_ref.quantize_nvfp4(to_f32(x), ROW)
    assert np.array_equal(yr.values.cpu().numpy(), v_ref)
    assert np.array_equal(nv_valid_scales(yr, yr.scale_factors.cpu().numpy()), nv_valid_scales(yr, s_ref))
    d_ref, _ = mx_ref.dequantize_nvfp4(v_ref, s_ref, rows, cols, ROW)
    assert np.array_equal(to_f32(cdl.mx.dequantize(yr)), d_ref)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", [(1, 128), (37, 4096), (300, 2048), (100, 7168), (5, 1024)])
@pytest.mark.parametrize("affine", ["none", "scale_bias"])
def test_norm_fwd_nvfp4(cdl, gpu_ok, rows, cols, affine):
    """NormOutput::Nvfp4Rowwise: |got - y| <= 0.34 |y| + 0.5 * block scale (tests/norm.rs:144)."""
    gen = torch.Generator().manual_seed(1)
    x = (torch.randn(rows, cols, generator=gen) * 2.0 + 0.5).to(torch.bfloat16)
    scale = (torch.rand(cols, generator=gen) + 0.5).to(torch.bfloat16) if affine != "none" else None
    bias = torch.randn(cols, generator=gen).to(torch.bfloat16) if affine != "none" else None
    out = cdl.mx.norm_fwd_mx(x.cuda(), None if scale is None else scale.cuda(),
                             None if bias is None else bias.cuda(), 1e-6, save_stats=True,
                             fmt=cdl.mx.NVFP4)
    y_ref, r_ref = oracle.rmsnorm_fwd(to_f32(x), None if scale is None else to_f32(scale),
                                      None if bias is None else to_f32(bias), 1e-6)
    assert_all_close("r_inv", to_f32(out.r_inv), r_ref, oracle.abs_rel_tolerance(r_ref, 1e-6, 1e-4))
    got, es = mx_ref.dequantize_nvfp4(out.y.values.cpu().numpy(), out.y.scale_factors.cpu().numpy(),
                                      rows, cols, ROW)
    assert_all_close("y", got, y_ref, 0.34 * np.abs(y_ref) + 0.5 * es + 1e-30)
    v_ref, _ = mx_ref.quantize_nvfp4(oracle.bf16_round(y_ref.astype(np.float32)), ROW)
    assert (out.y.values.cpu().numpy() == v_ref).mean() > 0.97


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,n", [(128, 256, 64), (128, 64, 256), (192, 320, 160), (512, 2048, 768),
                                   (2048, 512, 4864)])
@pytest.mark.parametrize("out", ["bf16", "f32"])
def test_matmul_nvfp4(cdl, gpu_ok, m, k, n, out):
    """The reference's nvfp4_inputs test (crates/cleandl/tests/matmul.rs:1063-1080)."""
    gen = torch.Generator().manual_seed(90)
    a = torch.randn(m, k, generator=gen).to(torch.bfloat16)
    b = torch.randn(k, n, generator=gen).to(torch.bfloat16)
    qa, _ = cdl.mx.quantize(a.cuda(), rowwise=True, fmt=cdl.mx.NVFP4)
    qb = cdl.mx.quantize(b.cuda().T.contiguous(), rowwise=True, fmt=cdl.mx.NVFP4)[0].transposed()
    assert (qb.dim, qb.rows, qb.cols) == (COL, k, n)
    da, _ = mx_ref.dequantize_nvfp4(qa.values.cpu().numpy(), qa.scale_factors.cpu().numpy(), m, k, ROW)
    db, _ = mx_ref.dequantize_nvfp4(qb.values.cpu().numpy(), qb.scale_factors.cpu().numpy(), k, n, COL)
    d = cdl.mx.matmul_mx(qa, qb, out_dtype=torch.bfloat16 if out == "bf16" else torch.float32)
    expected = da.astype(np.float64) @ db.astype(np.float64)
    bound = np.abs(da).astype(np.float64) @ np.abs(db).astype(np.float64)
    assert_all_close(f"nvfp4 {m}x{k}x{n} -> {out}", to_f32(d), expected,
                     oracle.matmul_tolerance(expected, bound, out == "bf16"))


def test_nvfp4_host_validation(cdl):
    L = cdl._lib
    a = L.CdlMxTensor(512, 1024, L.CDL_NVFP4, L.CDL_MX_ROWWISE, 128, 96)
    b = L.CdlMxTensor(512, 1024, L.CDL_NVFP4, L.CDL_MX_COLWISE, 96, 128)
    d = L.CdlTensor(ptr=2048, dtype=L.CDL_BF16, rank=2)
    d.shape[0], d.shape[1], d.stride[0], d.stride[1] = 128, 128, 128, 1
    st = L.lib.cdl_b200_matmul_mx(ctypes.byref(a), ctypes.byref(b), None, ctypes.byref(d), 1.0, 0.0, None)
    assert st == -2 and "multiple of 64" in L.last_error()
    b = L.CdlMxTensor(512, 1024, L.CDL_MXFP8, L.CDL_MX_COLWISE, 96, 128)
    st = L.lib.cdl_b200_matmul_mx(ctypes.byref(a), ctypes.byref(b), None, ctypes.byref(d), 1.0, 0.0, None)
    assert st == -2 and "mixed" in L.last_error()
    assert cdl.mx.layout_bytes(128, 256, ROW, fmt=cdl.mx.NVFP4) == (128 * 128, 128 * 16)
    with pytest.raises(cdl._lib.CdlError, match="block size 16"):
        cdl.mx.layout_bytes(128, 40, ROW, fmt=cdl.mx.NVFP4)


@pytest.mark.gpu
def test_mx_edge_shapes(cdl, gpu_ok):
    """Empty shapes are a silent success; single rows, the smallest K and ragged N work."""
    dev = "cuda"
    # empty
    x0 = torch.empty(0, 64, dtype=torch.bfloat16, device=dev)
    yr, _ = cdl.mx.quantize(x0, rowwise=True)
    assert yr.values.numel() == 0
    out = cdl.mx.norm_fwd_mx(x0, save_stats=True)
    assert out.y.values.numel() == 0 and out.r_inv.numel() == 0
    qa = cdl.mx.MxTensor.empty(0, 64, ROW, dev)
    qb = cdl.mx.MxTensor.empty(64, 16, COL, dev)
    assert cdl.mx.matmul_mx(qa, qb).shape == (0, 16)
    # one row, K = 32, N = 8; and 129 rows (a pair tile with one row in the second CTA)
    gen = torch.Generator().manual_seed(7)
    for m, k, n in [(1, 32, 8), (129, 64, 40), (257, 160, 264)]:
        a = torch.randn(m, k, generator=gen).to(torch.bfloat16)
        b = torch.randn(k, n, generator=gen).to(torch.bfloat16)
        qa, _ = cdl.mx.quantize(a.cuda(), rowwise=True)
        _, qb = cdl.mx.quantize(b.cuda(), rowwise=False, colwise=True)
        da, _ = mx_ref.dequantize(qa.values.cpu().numpy(), qa.scale_factors.cpu().numpy(), m, k, ROW)
        db, _ = mx_ref.dequantize(qb.values.cpu().numpy(), qb.scale_factors.cpu().numpy(), k, n, COL)
        expected = da.astype(np.float64) @ db.astype(np.float64)
        bound = np.abs(da).astype(np.float64) @ np.abs(db).astype(np.float64)
        d = cdl.mx.matmul_mx(qa, qb, out_dtype=torch.float32)
        assert_all_close(f"{m}x{k}x{n}", to_f32(d), expected, oracle.matmul_tolerance(expected, bound, False))
    # the one-CTA kernel is still reachable and agrees bit for bit with the pair kernel
    a = torch.randn(512, 256, generator=gen).to(torch.bfloat16)
    b = torch.randn(256, 384, generator=gen).to(torch.bfloat16)
    qa, _ = cdl.mx.quantize(a.cuda(), rowwise=True)
    _, qb = cdl.mx.quantize(b.cuda(), rowwise=False, colwise=True)
    d_pair = cdl.mx.matmul_mx(qa, qb, out_dtype=torch.float32)
    d_single = cdl.mx.matmul_mx(qa, qb, out_dtype=torch.float32, variant=cdl._lib.GEMM_ONE_CTA)
    assert torch.equal(d_pair, d_single)


def test_oracle_against_torch_golden():
    """tests/golden/mx.npz was produced by an independent torch implementation
    (tests/golden/make_golden_mx.py): the oracle reproduces it bit for bit."""
    from pathlib import Path

    g = np.load(Path(__file__).resolve().parent / "golden" / "mx.npz")
    m = g["m"]
    rows, cols = m.shape
    for dim, key in ((ROW, "row"), (COL, "col")):
        v, s = mx_ref.quantize(m, dim)
        assert np.array_equal(v, g[key + "_values"]) and np.array_equal(s, g[key + "_scales"])
        assert np.array_equal(mx_ref.dequantize(v, s, rows, cols, dim)[0], g[key + "_deq"])
    v, s = mx_ref.quantize_nvfp4(m, ROW)
    assert np.array_equal(v, g["nv_values"]) and np.array_equal(s, g["nv_scales"])
    assert np.array_equal(mx_ref.dequantize_nvfp4(v, s, rows, cols, ROW)[0], g["nv_deq"])


@pytest.mark.gpu
def test_gpu_against_torch_golden(cdl, gpu_ok):
    """The same fixture against the CUDA quantisers (the committed bits, not only the oracle)."""
    from pathlib import Path

    g = np.load(Path(__file__).resolve().parent / "golden" / "mx.npz")
    x = torch.from_numpy(g["m"]).to(torch.bfloat16).cuda()
    yr, yc = cdl.mx.quantize(x, rowwise=True, colwise=True)
    assert np.array_equal(yr.values.cpu().numpy(), g["row_values"])
    assert np.array_equal(yc.values.cpu().numpy(), g["col_values"])
    assert np.array_equal(valid_scales(yr, yr.scale_factors.cpu().numpy()), valid_scales(yr, g["row_scales"]))
    assert np.array_equal(valid_scales(yc, yc.scale_factors.cpu().numpy()), valid_scales(yc, g["col_scales"]))
    yn, _ = cdl.mx.quantize(x, rowwise=True, fmt=cdl.mx.NVFP4)
    assert np.array_equal(yn.values.cpu().numpy(), g["nv_values"])
    assert np.array_equal(nv_valid_scales(yn, yn.scale_factors.cpu().numpy()), nv_valid_scales(yn, g["nv_scales"]))
    assert np.array_equal(to_f32(cdl.mx.dequantize(yn)), g["nv_deq"])


@pytest.mark.gpu
@pytest.mark.parametrize("dim", [ROW, COL])
@pytest.mark.parametrize("in_fmt", ["mxfp8", "nvfp4"])
def test_matmul_nvfp4_block_scaled_output(cdl, gpu_ok, dim, in_fmt):
    """The (Nvfp4, Rowwise) case of the reference's block_scaled_outputs test
    (crates/cleandl/tests/matmul.rs:1083-1115), with either operand format, and the colwise form:
    |got - e| <= 0.25 |e| + 0.5 * block scale + 1e-4 * sum |a b|."""
    m, k, n = 256, 128, 192
    gen = torch.Generator().manual_seed(100)
    a = torch.randn(m, k, generator=gen).to(torch.bfloat16)
    b = torch.randn(k, n, generator=gen).to(torch.bfloat16)
    if in_fmt == "nvfp4":
        qa, _ = cdl.mx.quantize(a.cuda(), rowwise=True, fmt=cdl.mx.NVFP4)
        qb = cdl.mx.quantize(b.cuda().T.contiguous(), rowwise=True, fmt=cdl.mx.NVFP4)[0].transposed()
        da, _ = mx_ref.dequantize_nvfp4(qa.values.cpu().numpy(), qa.scale_factors.cpu().numpy(), m, k, ROW)
        db, _ = mx_ref.dequantize_nvfp4(qb.values.cpu().numpy(), qb.scale_factors.cpu().numpy(), k, n, COL)
    else:
        qa, _ = cdl.mx.quantize(a.cuda(), rowwise=True)
        _, qb = cdl.mx.quantize(b.cuda(), rowwise=False, colwise=True)
        da, _ = mx_ref.dequantize(qa.values.cpu().numpy(), qa.scale_factors.cpu().numpy(), m, k, ROW)
        db, _ = mx_ref.dequantize(qb.values.cpu().numpy(), qb.scale_factors.cpu().numpy(), k, n, COL)
    expected = da.astype(np.float64) @ db.astype(np.float64)
    bound = np.abs(da).astype(np.float64) @ np.abs(db).astype(np.float64)
    d = cdl.mx.matmul_mx_out(qa, qb, dim=dim, fmt=cdl.mx.NVFP4)
    assert (d.format, d.dim, d.rows, d.cols) == (cdl.mx.NVFP4, dim, m, n)
    got, es = mx_ref.dequantize_nvfp4(d.values.cpu().numpy(), d.scale_factors.cpu().numpy(), m, n, dim)
    assert_all_close(f"nvfp4 output dim {dim}", got, expected, 0.25 * np.abs(expected) + 0.5 * es + 1e-4 * bound)
    plain = cdl.mx.matmul_mx(qa, qb, out_dtype=torch.float32)
    v_ref, s_ref = mx_ref.quantize_nvfp4(to_f32(plain), dim)
    assert np.array_equal(d.values.cpu().numpy(), v_ref)
    assert np.array_equal(nv_valid_scales(d, d.scale_factors.cpu().numpy()), nv_valid_scales(d, s_ref))


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_matmul_mx_with_c(cdl, gpu_ok, fmt):
    """alpha / beta / C with block-scaled operands, C bf16 and f32, and accumulation in place (the
    weight-gradient form D (f32) += A . B), after the reference's accumulate_c test
    (crates/cleandl/tests/matmul.rs:690-726)."""
    m, k, n = 384, 256, 320
    gen = torch.Generator().manual_seed(110)
    a = torch.randn(m, k, generator=gen).to(torch.bfloat16)
    b = torch.randn(k, n, generator=gen).to(torch.bfloat16)
    if fmt == "nvfp4":
        qa, _ = cdl.mx.quantize(a.cuda(), rowwise=True, fmt=cdl.mx.NVFP4)
        qb = cdl.mx.quantize(b.cuda().T.contiguous(), rowwise=True, fmt=cdl.mx.NVFP4)[0].transposed()
        da, _ = mx_ref.dequantize_nvfp4(qa.values.cpu().numpy(), qa.scale_factors.cpu().numpy(), m, k, ROW)
        db, _ = mx_ref.dequantize_nvfp4(qb.values.cpu().numpy(), qb.scale_factors.cpu().numpy(), k, n, COL)
    else:
        qa, _ = cdl.mx.quantize(a.cuda(), rowwise=True)
        _, qb = cdl.mx.quantize(b.cuda(), rowwise=False, colwise=True)
        da, _ = mx_ref.dequantize(qa.values.cpu().numpy(), qa.scale_factors.cpu().numpy(), m, k, ROW)
        db, _ = mx_ref.dequantize(qb.values.cpu().numpy(), qb.scale_factors.cpu().numpy(), k, n, COL)
    prod = da.astype(np.float64) @ db.astype(np.float64)
    bound = np.abs(da).astype(np.float64) @ np.abs(db).astype(np.float64)
    for c_dtype, out_dtype in ((torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32),
                               (torch.bfloat16, torch.float32)):
        c = torch.randn(m, n, generator=gen).to(c_dtype)
        d = cdl.mx.matmul_mx(qa, qb, out_dtype=out_dtype, alpha=0.5, c=c.cuda(), beta=-2.0)
        expected = 0.5 * prod - 2.0 * c.double().numpy()
        tol = oracle.matmul_tolerance(expected, 0.5 * bound + 2.0 * np.abs(c.double().numpy()),
                                      out_dtype == torch.bfloat16)
        assert_all_close(f"{fmt} c {c_dtype} -> {out_dtype}", to_f32(d), expected, tol)
    # in place, twice: D = C0 + 2 A.B
    acc = torch.randn(m, n, generator=gen)
    d = acc.cuda().clone()
    for _ in range(2):
        cdl.mx.matmul_mx(qa, qb, out=d, c=d, beta=1.0)
    expected = acc.double().numpy() + 2.0 * prod
    assert_all_close("in place", to_f32(d), expected,
                     oracle.matmul_tolerance(expected, 2.0 * bound + np.abs(acc.double().numpy()), False))
