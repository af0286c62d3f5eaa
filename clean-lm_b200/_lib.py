"""ctypes binding of libcleandl_b200.so.  There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

# The in-tree build; CLEANDL_B200_LIB names another build of the same sources (a variant made by
# build.py with other tunable macros) for side-by-side measurements.
LIB_PATH = Path(os.environ.get("CLEANDL_B200_LIB") or Path(__file__).resolve().parent / "libcleandl_b200.so")

CDL_BF16, CDL_F32, CDL_I32 = 0, 1, 2


class CdlError(RuntimeError):
    """A C-ABI call returned a negative status; `.status` holds it."""

    def __init__(self, status: int, message: str):
        super().__init__(f"cleandl_b200 error {status}: {message}")
        self.status = status
        self.message = message


class CdlTensor(ctypes.Structure):
    _fields_ = [
        ("ptr", ctypes.c_void_p),
        ("dtype", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("shape", ctypes.c_int64 * 4),
        ("stride", ctypes.c_int64 * 4),
    ]


class CdlAttnDesc(ctypes.Structure):
    _fields_ = [("softmax_scale", ctypes.c_float), ("causal", ctypes.c_int32),
                ("variant", ctypes.c_int32)]


ATTN_AUTO, ATTN_ONE_SHOT, ATTN_PERSISTENT = 0, 1, 2


class CdlProfileRecord(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("ms", ctypes.c_float), ("work", ctypes.c_double)]


class CdlAdamwParams(ctypes.Structure):
    _fields_ = [("lr", ctypes.c_float), ("beta1", ctypes.c_float), ("beta2", ctypes.c_float),
                ("eps", ctypes.c_float), ("weight_decay", ctypes.c_float), ("step", ctypes.c_int32),
                ("grad_scale", ctypes.c_float), ("max_grad_norm", ctypes.c_float)]


class CdlSky1Config(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in
                ("batch", "seqlen", "hidden", "heads", "kv_heads", "head_dim", "ffn")] + [
                    ("eps", ctypes.c_float), ("flags", ctypes.c_int32)]


CDL_SKY1_DETERMINISTIC = 1


class CdlMatmulOptions(ctypes.Structure):
    """cdl_matmul_options: variant (GEMM_AUTO / GEMM_ONE_CTA / GEMM_CTA_PAIR), deterministic."""

    _fields_ = [("variant", ctypes.c_int32), ("deterministic", ctypes.c_int32)]


class CdlNormOptions(ctypes.Structure):
    """cdl_norm_options: variant (NORM_AUTO / NORM_WARP_PER_ROW / NORM_PIPELINED)."""

    _fields_ = [("variant", ctypes.c_int32)]


GEMM_AUTO, GEMM_ONE_CTA, GEMM_CTA_PAIR = 0, 1, 2
NORM_AUTO, NORM_WARP_PER_ROW, NORM_PIPELINED = 0, 1, 2


class CdlSky1Ragged(ctypes.Structure):
    _fields_ = [("cu_seqlens", ctypes.c_void_p), ("num_seqs", ctypes.c_int32),
                ("max_seqlen", ctypes.c_int32)]


class CdlSky1GradEvents(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("wdown", "wup", "wgate_norm2", "wo", "wqkv_norm1")]


class CdlMxTensor(ctypes.Structure):
    _fields_ = [("values", ctypes.c_void_p), ("scale_factors", ctypes.c_void_p),
                ("format", ctypes.c_int32), ("dim", ctypes.c_int32),
                ("rows", ctypes.c_int64), ("cols", ctypes.c_int64)]


CDL_MXFP8, CDL_NVFP4 = 0, 1
CDL_MX_ROWWISE, CDL_MX_COLWISE = 0, 1

_BLOCK_PARAMS = ("norm1", "wqkv", "wo", "norm2", "wup", "wgate", "wdown")


class CdlSky1Weights(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in _BLOCK_PARAMS]


class CdlSky1Grads(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in _BLOCK_PARAMS]


class CdlSky1Saved(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("qkv", "attn", "lse", "o", "up", "gate", "act")]


if not LIB_PATH.exists():
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python clean-lm_b200/build.py` "
        "(needs nvcc; the library holds sm_100a code only and has no CPU fallback)"
    )

lib = ctypes.CDLL(str(LIB_PATH))

_T = ctypes.POINTER(CdlTensor)
_MX = ctypes.POINTER(CdlMxTensor)
_MO = ctypes.POINTER(CdlMatmulOptions)
_NO = ctypes.POINTER(CdlNormOptions)
_vp = ctypes.c_void_p
_sz = ctypes.c_size_t

# name -> argtypes; every entry point declared in include/cleandl_b200.h
SIGNATURES = {
    "cdl_b200_last_error": ([], ctypes.c_char_p),
    "cdl_b200_device_ok": ([ctypes.c_int32], ctypes.c_int32),
    "cdl_b200_device_status": ([ctypes.POINTER(ctypes.c_int32)], ctypes.c_int32),
    "cdl_b200_profile_start": ([ctypes.c_int32], ctypes.c_int32),
    "cdl_b200_profile_stop": ([ctypes.POINTER(CdlProfileRecord), ctypes.c_int32,
                               ctypes.POINTER(ctypes.c_int32)], ctypes.c_int32),
    "cdl_b200_embedding_fwd": ([_T, _T, _T, _vp], ctypes.c_int32),
    "cdl_b200_matmul": ([_T, _T, _T, _T, ctypes.c_float, ctypes.c_float, _vp, _sz, _vp],
                        ctypes.c_int32),
    "cdl_b200_matmul_opt": ([_T, _T, _T, _T, ctypes.c_float, ctypes.c_float, _MO, _vp, _sz, _vp],
                            ctypes.c_int32),
    "cdl_b200_matmul_candidates": ([_T, _T, _T, _MO, ctypes.c_int32, ctypes.POINTER(ctypes.c_int32)],
                                   ctypes.c_int32),
    "cdl_b200_matmul_rope": ([_T, _T, _T, ctypes.c_int32, ctypes.c_int32, _T, _T, _vp], ctypes.c_int32),
    "cdl_b200_matmul_swiglu_gate": ([_T, _T, _T, _T, _T, _vp], ctypes.c_int32),
    "cdl_b200_matmul_swiglu_dgrad": ([_T, _T, _T, _T, _T, _T, _vp], ctypes.c_int32),
    "cdl_b200_matmul_scratch_bytes": ([_T, _T, _T, ctypes.POINTER(_sz)], ctypes.c_int32),
    "cdl_b200_rmsnorm_fwd": ([_T, _T, _T, ctypes.c_float, _T, _T, _vp], ctypes.c_int32),
    "cdl_b200_rmsnorm_fwd_opt": ([_T, _T, _T, ctypes.c_float, _T, _T, _NO, _vp], ctypes.c_int32),
    "cdl_b200_rmsnorm_bwd_opt": ([_T, _T, _T, _T, _T, _T, _T, _NO, _vp, _sz, _vp], ctypes.c_int32),
    "cdl_b200_layernorm_fwd": ([_T, _T, _T, ctypes.c_float, _T, _T, _T, _vp], ctypes.c_int32),
    "cdl_b200_rmsnorm_bwd": ([_T, _T, _T, _T, _T, _T, _T, _vp, _sz, _vp], ctypes.c_int32),
    "cdl_b200_rmsnorm_bwd_static": ([_T, _T, _T, _T, _T, _T, _T, _vp], ctypes.c_int32),
    "cdl_b200_rmsnorm_bwd_scratch_bytes": ([ctypes.c_int64, ctypes.c_int64, ctypes.POINTER(_sz)],
                                           ctypes.c_int32),
    "cdl_b200_mx_layout": ([ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64,
                            ctypes.POINTER(_sz), ctypes.POINTER(_sz)], ctypes.c_int32),
    "cdl_b200_mx_quantize": ([_T, _MX, _MX, _vp], ctypes.c_int32),
    "cdl_b200_mx_dequantize": ([_MX, _T, _vp], ctypes.c_int32),
    "cdl_b200_rmsnorm_fwd_mx": ([_T, _T, _T, ctypes.c_float, _MX, _MX, _T, _vp], ctypes.c_int32),
    "cdl_b200_matmul_mx": ([_MX, _MX, _T, _T, ctypes.c_float, ctypes.c_float, _vp], ctypes.c_int32),
    "cdl_b200_matmul_mx_opt": ([_MX, _MX, _T, _T, ctypes.c_float, ctypes.c_float, _MO, _vp],
                               ctypes.c_int32),
    "cdl_b200_matmul_mx_out": ([_MX, _MX, _MX, ctypes.c_float, _vp], ctypes.c_int32),
    "cdl_b200_attn_fwd": ([ctypes.POINTER(CdlAttnDesc), _T, _T, _T, _T, _T, _vp], ctypes.c_int32),
    "cdl_b200_attn_bwd": ([ctypes.POINTER(CdlAttnDesc), _T, _T, _T, _T, _T, _T, _T, _T, _T, _vp,
                           _sz, _vp], ctypes.c_int32),
    "cdl_b200_attn_bwd_scratch_bytes": ([_T, _T, ctypes.POINTER(_sz)], ctypes.c_int32),
    "cdl_b200_attn_fwd_packed": ([ctypes.POINTER(CdlAttnDesc), _T, _T, _T, _T, _T, ctypes.c_int64,
                                  ctypes.c_int64, _T, _T, _vp], ctypes.c_int32),
    "cdl_b200_attn_bwd_packed": ([ctypes.POINTER(CdlAttnDesc), _T, _T, _T, _T, _T, _T, _T, _T,
                                  ctypes.c_int64, ctypes.c_int64, _T, _T, _T, _vp, _sz, _vp],
                                 ctypes.c_int32),
    "cdl_b200_attn_bwd_rope": ([ctypes.POINTER(CdlAttnDesc), _T, _T, _T, _T, _T, _T, _T, _T, _T, _T, _vp,
                                _sz, _vp], ctypes.c_int32),
    "cdl_b200_attn_bwd_packed_rope": ([ctypes.POINTER(CdlAttnDesc), _T, _T, _T, _T, _T, _T, _T, _T,
                                       ctypes.c_int64, ctypes.c_int64, _T, _T, _T, _T, _vp, _sz, _vp],
                                      ctypes.c_int32),
    "cdl_b200_attn_bwd_packed_scratch_bytes": ([ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                                ctypes.POINTER(_sz)], ctypes.c_int32),
    "cdl_b200_rope": ([_T, _T, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, _vp], ctypes.c_int32),
    "cdl_b200_rope_ragged": ([_T, _T, ctypes.c_int32, _T, ctypes.c_int32, _vp], ctypes.c_int32),
    "cdl_b200_swiglu_fwd": ([_T, _T, _T, _vp], ctypes.c_int32),
    "cdl_b200_swiglu_bwd": ([_T, _T, _T, _T, _T, _vp], ctypes.c_int32),
    "cdl_b200_cross_entropy": ([_T, _T, _T, ctypes.c_float, _vp], ctypes.c_int32),
    "cdl_b200_embedding_bwd": ([_T, _T, _T, _vp], ctypes.c_int32),
    "cdl_b200_sum": ([_vp, ctypes.c_int64, _vp, ctypes.c_float, ctypes.c_int32, ctypes.c_int32, _vp,
                      _sz, _vp], ctypes.c_int32),
    "cdl_b200_adamw": ([_vp, _vp, _vp, _vp, _vp, ctypes.c_int64, _vp,
                        ctypes.POINTER(CdlAdamwParams), _vp], ctypes.c_int32),
    "cdl_b200_sky1_block_workspace_bytes": ([ctypes.POINTER(CdlSky1Config), ctypes.POINTER(_sz),
                                             ctypes.POINTER(_sz)], ctypes.c_int32),
    "cdl_b200_sky1_block_workspace_bytes_ragged": ([ctypes.POINTER(CdlSky1Config),
                                                    ctypes.POINTER(CdlSky1Ragged), ctypes.POINTER(_sz),
                                                    ctypes.POINTER(_sz)], ctypes.c_int32),
    "cdl_b200_sky1_block_fwd_ragged": ([ctypes.POINTER(CdlSky1Config), ctypes.POINTER(CdlSky1Weights),
                                        _vp, _vp, ctypes.POINTER(CdlSky1Ragged),
                                        ctypes.POINTER(CdlSky1Saved), _vp, _vp, _sz, _vp], ctypes.c_int32),
    "cdl_b200_sky1_block_bwd_ragged": ([ctypes.POINTER(CdlSky1Config), ctypes.POINTER(CdlSky1Weights),
                                        _vp, _vp, ctypes.POINTER(CdlSky1Ragged),
                                        ctypes.POINTER(CdlSky1Saved), _vp, ctypes.POINTER(CdlSky1Grads),
                                        _vp, _vp, _sz, ctypes.c_int32, _vp], ctypes.c_int32),
    "cdl_b200_sky1_block_fwd": ([ctypes.POINTER(CdlSky1Config), ctypes.POINTER(CdlSky1Weights), _vp,
                                 _vp, ctypes.POINTER(CdlSky1Saved), _vp, _vp, _sz, _vp],
                                ctypes.c_int32),
    "cdl_b200_sky1_block_bwd": ([ctypes.POINTER(CdlSky1Config), ctypes.POINTER(CdlSky1Weights), _vp,
                                 _vp, ctypes.POINTER(CdlSky1Saved), _vp,
                                 ctypes.POINTER(CdlSky1Grads), _vp, _vp, _sz, ctypes.c_int32, _vp],
                                ctypes.c_int32),
    "cdl_b200_sky1_block_bwd_events": ([ctypes.POINTER(CdlSky1Config), ctypes.POINTER(CdlSky1Weights),
                                        _vp, _vp, ctypes.POINTER(CdlSky1Ragged),
                                        ctypes.POINTER(CdlSky1Saved), _vp, ctypes.POINTER(CdlSky1Grads),
                                        _vp, _vp, _sz, ctypes.POINTER(CdlSky1GradEvents), _vp],
                               ctypes.c_int32),
}

for _name, (_args, _res) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.argtypes = _args
    _fn.restype = _res


def last_error() -> str:
    return lib.cdl_b200_last_error().decode()


def check(status: int) -> None:
    if status != 0:
        raise CdlError(status, last_error())


def tensor_arg(t):
    """Wraps a torch tensor (any strides) as a cdl_tensor; None stays None (a NULL pointer)."""
    if t is None:
        return None
    import torch

    dt = {torch.bfloat16: CDL_BF16, torch.float32: CDL_F32, torch.int32: CDL_I32}.get(t.dtype)
    if dt is None:
        raise CdlError(-1, f"unsupported element type {t.dtype}: f32 or bf16 expected")
    if t.dim() > 4:
        raise CdlError(-1, f"rank {t.dim()} exceeds 4")
    ct = CdlTensor()
    ct.ptr = t.data_ptr()
    ct.dtype = dt
    ct.rank = t.dim()
    for i in range(t.dim()):
        ct.shape[i] = t.shape[i]
        ct.stride[i] = t.stride(i)
    return ct


def ref(ct):
    return None if ct is None else ctypes.byref(ct)


def device_status() -> int:
    """Synchronises the device; returns (and clears) the kernel status word."""
    out = ctypes.c_int32(0)
    check(lib.cdl_b200_device_status(ctypes.byref(out)))
    return out.value


PROFILE_KINDS = {1: "gemm", 2: "norm_fwd", 3: "norm_bwd", 4: "attn_fwd", 5: "attn_bwd",
                 6: "elementwise"}


def profile_start(max_records: int = 4096) -> None:
    check(lib.cdl_b200_profile_start(max_records))


def profile_stop(max_records: int = 4096):
    """Synchronises the device; returns [(kind name, ms, work), ...] in launch order."""
    buf = (CdlProfileRecord * max_records)()
    n = ctypes.c_int32(0)
    check(lib.cdl_b200_profile_stop(buf, max_records, ctypes.byref(n)))
    return [(PROFILE_KINDS.get(buf[i].kind, "?"), buf[i].ms, buf[i].work) for i in range(n.value)]
