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
