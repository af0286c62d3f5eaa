"""CPU checks of the drop-in boundary: the shared library loads without a GPU, exports every
symbol that include/cleandl_b200.h declares, and the Python binding knows all of them."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "cleandl_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cdl_b200_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for must in ("cdl_b200_matmul", "cdl_b200_rmsnorm_fwd", "cdl_b200_rmsnorm_bwd",
                 "cdl_b200_attn_fwd", "cdl_b200_attn_bwd", "cdl_b200_last_error"):
        assert must in syms


def test_library_exports_every_declared_symbol(cdl):
    lib = ctypes.CDLL(str(cdl._lib.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_binding_covers_header(cdl):
    assert sorted(cdl._lib.SIGNATURES) == declared_symbols()


def test_last_error_is_empty_string_initially(cdl):
    assert isinstance(cdl._lib.last_error(), str)


def test_host_validation_needs_no_gpu(cdl):
    """Operand validation happens before any CUDA call, so it can be exercised on CPU."""
    L = cdl._lib
    a = L.CdlTensor(ptr=256, dtype=L.CDL_BF16, rank=2)
    a.shape[0], a.shape[1], a.stride[0], a.stride[1] = 8, 16, 16, 1
    b = L.CdlTensor(ptr=512, dtype=L.CDL_BF16, rank=2)
    b.shape[0], b.shape[1], b.stride[0], b.stride[1] = 24, 8, 8, 1
    d = L.CdlTensor(ptr=1024, dtype=L.CDL_BF16, rank=2)
    d.shape[0], d.shape[1], d.stride[0], d.stride[1] = 8, 8, 8, 1
    st = L.lib.cdl_b200_matmul(ctypes.byref(a), ctypes.byref(b), None, ctypes.byref(d), 1.0, 0.0,
                               None, 0, None)
    assert st == -1 and "contraction" in L.last_error()
    b.shape[0] = 16
    a.shape[1] = b.shape[0] = 0
    st = L.lib.cdl_b200_matmul(ctypes.byref(a), ctypes.byref(b), None, ctypes.byref(d), 1.0, 0.0,
                               None, 0, None)
    assert st == -1 and "K is zero" in L.last_error()
    x = L.CdlTensor(ptr=256, dtype=L.CDL_BF16, rank=3)
    st = L.lib.cdl_b200_rmsnorm_fwd(ctypes.byref(x), None, None, 1e-6, ctypes.byref(x), None, None)
    assert st == -1 and "2D" in L.last_error()


def test_candidates_need_no_gpu_and_put_the_heuristic_first(cdl):
    """cdl_b200_matmul_candidates only inspects shapes and layouts (what the reference's
    Executor::candidates does, op.rs:301-318)."""
    L = cdl._lib

    def t(ptr, rows, cols, dtype=None, transposed=False):
        x = L.CdlTensor(ptr=ptr, dtype=L.CDL_BF16 if dtype is None else dtype, rank=2)
        x.shape[0], x.shape[1] = rows, cols
        x.stride[0], x.stride[1] = (1, rows) if transposed else (cols, 1)
        return x

    buf = (L.CdlMatmulOptions * 8)()
    n = ctypes.c_int32(0)
    a, b, d = t(4096, 1024, 512), t(8192, 512, 256), t(1 << 20, 1024, 256)
    L.check(L.lib.cdl_b200_matmul_candidates(ctypes.byref(a), ctypes.byref(b), ctypes.byref(d), buf, 8,
                                             ctypes.byref(n)))
    assert [(buf[i].variant, buf[i].deterministic) for i in range(n.value)] == [
        (L.GEMM_CTA_PAIR, 0), (L.GEMM_ONE_CTA, 0)]
    # the weight-gradient form (f32 output) adds the fixed-order variant of the pair kernel
    a, d = t(4096, 512, 1024, transposed=True), t(1 << 20, 512, 256, dtype=L.CDL_F32)
    b = t(8192, 1024, 256)
    L.check(L.lib.cdl_b200_matmul_candidates(ctypes.byref(a), ctypes.byref(b), ctypes.byref(d), buf, 8,
                                             ctypes.byref(n)))
    assert [(buf[i].variant, buf[i].deterministic) for i in range(n.value)] == [
        (L.GEMM_CTA_PAIR, 0), (L.GEMM_CTA_PAIR, 1), (L.GEMM_ONE_CTA, 0)]
    # one 128-row slab: the one-CTA kernel is the default; unaligned operands: the general kernel
    a, d = t(4096, 64, 512), t(1 << 20, 64, 256)
    b = t(8192, 512, 256)
    L.check(L.lib.cdl_b200_matmul_candidates(ctypes.byref(a), ctypes.byref(b), ctypes.byref(d), buf, 8,
                                             ctypes.byref(n)))
    assert buf[0].variant == L.GEMM_ONE_CTA
    a = t(4098, 64, 512)
    L.check(L.lib.cdl_b200_matmul_candidates(ctypes.byref(a), ctypes.byref(b), ctypes.byref(d), buf, 8,
                                             ctypes.byref(n)))
    assert n.value == 1 and buf[0].variant == L.GEMM_AUTO
    # an unknown variant is rejected before any CUDA call
    mo = L.CdlMatmulOptions(7, 0)
    a = t(4096, 64, 512)
    st = L.lib.cdl_b200_matmul_opt(ctypes.byref(a), ctypes.byref(b), None, ctypes.byref(d), 1.0, 0.0,
                                   ctypes.byref(mo), None, 0, None)
    assert st == -1 and "variant" in L.last_error()
