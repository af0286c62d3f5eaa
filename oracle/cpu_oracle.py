"""TEST INFRASTRUCTURE — numpy front end of the CPU oracle (oracle/cpu_ref.c).

Only tests, `__graft_entry__.smoke()` and the bench's cpu_baseline / reference legs import this
module; the product library never does.  PARITY UNPINNED: see the header of cpu_ref.c.

All arrays are float32 holding values already rounded to bf16 where the device stores bf16.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_SRC = _DIR / "cpu_ref.c"
_LIB = _DIR / "liboracle.so"
_lib = None


def build(force: bool = False) -> Path:
    """Compiles cpu_ref.c with gcc (OpenMP) next to its source."""
    if force or not _LIB.exists() or _LIB.stat().st_mtime < _SRC.stat().st_mtime:
        subprocess.run(
            ["gcc", "-O3", "-fopenmp", "-shared", "-fPIC", str(_SRC), "-o", str(_LIB), "-lm"],
            check=True,
        )
    return _LIB


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(_LIB))
        f32p = ctypes.POINTER(ctypes.c_float)
        f64p = ctypes.POINTER(ctypes.c_double)
        i64 = ctypes.c_int64
        _lib.oracle_matmul.argtypes = [f32p, f32p, f32p, ctypes.c_float, ctypes.c_float,
                                       i64, i64, i64, i64, f32p, f32p]
        _lib.oracle_rmsnorm_fwd.argtypes = [f32p, f32p, f32p, ctypes.c_float, i64, i64, f32p, f32p]
        _lib.oracle_rmsnorm_bwd.argtypes = [f32p, f32p, f32p, f32p, ctypes.c_float, i64, i64,
                                            f32p, f64p]
        _lib.oracle_attention.argtypes = [f32p, f32p, f32p, f32p, i64, i64, i64, i64, i64, i64,
                                          ctypes.c_float, ctypes.c_int, f32p, f32p, f32p, f32p, f32p]
        for fn in (_lib.oracle_matmul, _lib.oracle_rmsnorm_fwd, _lib.oracle_rmsnorm_bwd,
                   _lib.oracle_attention):
            fn.restype = None
    return _lib


def num_threads() -> int:
    """Threads the OpenMP loops use (all host cores unless OMP_NUM_THREADS says otherwise)."""
    env = os.environ.get("OMP_NUM_THREADS")
    return int(env) if env else (os.cpu_count() or 1)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _p(a, ty=ctypes.c_float):
    return None if a is None else a.ctypes.data_as(ctypes.POINTER(ty))


def bf16_round(a: np.ndarray) -> np.ndarray:
    """Rounds float32 values to the nearest bf16 (ties to even); result stays float32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32)
    bias = ((u >> 16) & 1) + np.uint32(0x7FFF)
    r = ((u + bias) & np.uint32(0xFFFF0000)).astype(np.uint32)
    out = r.view(np.float32).copy()
    nan = np.isnan(a)
    out[nan] = np.nan
    return out


def matmul(a, b, c=None, alpha=1.0, beta=0.0, with_bound=True):
    """alpha * a @ b + beta * c in f64; a [.., M, K], b [.., K, N]. Returns (value, bound)."""
    lib = _load()
    a, b, c = _f32(a), _f32(b), _f32(c)
    batched = a.ndim == 3
    batch = a.shape[0] if batched else 1
    m, k = a.shape[-2:]
    n = b.shape[-1]
    assert b.shape[-2] == k
    out = np.empty(((batch, m, n) if batched else (m, n)), dtype=np.float32)
    bound = np.empty_like(out) if with_bound else None
    lib.oracle_matmul(_p(a), _p(b), _p(c), alpha, beta, batch, m, k, n, _p(out), _p(bound))
    return out, bound


def rmsnorm_fwd(x, scale=None, bias=None, eps=1e-6):
    """Returns (y, r_inv) as float32 arrays computed in f64."""
    lib = _load()
    x, scale, bias = _f32(x), _f32(scale), _f32(bias)
    rows, cols = x.shape
    y = np.empty_like(x)
    r_inv = np.empty(rows, dtype=np.float32)
    lib.oracle_rmsnorm_fwd(_p(x), _p(scale), _p(bias), eps, rows, cols, _p(y), _p(r_inv))
    return y, r_inv


def rmsnorm_bwd(x, dy, scale, residual=None, eps=1e-6, dscale_init=None):
    """Returns (dx f32, dscale f64 = dscale_init + sum over rows)."""
    lib = _load()
    x, dy, scale, residual = _f32(x), _f32(dy), _f32(scale), _f32(residual)
    rows, cols = x.shape
    dx = np.empty_like(x)
    acc = (np.zeros(cols, dtype=np.float64) if dscale_init is None
           else np.ascontiguousarray(dscale_init, dtype=np.float64).copy())
    lib.oracle_rmsnorm_bwd(_p(x), _p(dy), _p(residual), _p(scale), eps, rows, cols, _p(dx),
                           _p(acc, ctypes.c_double))
    return dx, acc


def attention(q, k, v, d_out=None, scale=None, causal=True):
    """Dense [B, S, H, D] attention. Returns dict(out, lse[, dq, dk, dv]) as float32."""
    lib = _load()
    q, k, v, d_out = _f32(q), _f32(k), _f32(v), _f32(d_out)
    b, sq, hq, d = q.shape
    _, sk, hk, _ = k.shape
    if scale is None:
        scale = 1.0 / np.sqrt(d)
    out = np.empty_like(q)
    lse = np.empty((b, hq, sq), dtype=np.float32)
    res = {"out": out, "lse": lse}
    dq = dk = dv = None
    if d_out is not None:
        dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
        res.update(dq=dq, dk=dk, dv=dv)
    lib.oracle_attention(_p(q), _p(k), _p(v), _p(d_out), b, sq, sk, hq, hk, d, float(scale),
                         1 if causal else 0, _p(out), _p(lse), _p(dq), _p(dk), _p(dv))
    return res


# ---- tolerances of the reference's own tests ----------------------------------------------

def matmul_tolerance(expected, bound, out_is_bf16):
    """crates/cleandl/tests/matmul.rs:199-202."""
    rounding = 2.0 ** -8 if out_is_bf16 else 0.0
    return rounding * np.abs(expected) + 1e-5 * bound + 1e-6


def abs_rel_tolerance(expected, atol, rtol):
    """crates/cleandl/tests/norm.rs:261-268, 309-315."""
    return atol + rtol * np.abs(expected)


def attention_tolerance(expected, atol, rtol):
    """crates/cleandl/tests/attention.rs:541-556: atol * max|expected| + rtol * |expected|."""
    fin = np.isfinite(expected)
    scale = max(float(np.max(np.abs(expected[fin]))) if fin.any() else 0.0, 1e-3)
    return atol * scale + rtol * np.abs(np.where(fin, expected, 0.0))
