"""CPU restatement of the reference's block-scaled (MX) tensor format.  TEST INFRASTRUCTURE ONLY:
nothing in the product path may import this file.

Follows the host-side quantiser and checks of the reference's own tests:
  * layout of values and scale factors      crates/cleandl/src/mx_tensor.rs:339-372 (MxLayout::new)
  * scale-factor index (128x4 tiles)        crates/cleandl/tests/common/mod.rs:124-129
  * quantize_mx                             crates/cleandl/tests/matmul.rs:885-952
  * UE8M0 decode                            crates/cleandl/tests/common/mod.rs:131-137
  * tolerances of a block-scaled output     crates/cleandl/tests/norm.rs:134-149,
                                            crates/cleandl/tests/matmul.rs:1100-1110
Parity unpinned against the reference itself: its tests draw their inputs from Rust random
streams and hold no stored vectors for this format.  The oracle is pinned instead by the format's
definition (the e4m3 table against its 256 codes, the index against the closed form), by torch's
float8_e4m3fn cast, and bit for bit by tests/golden/mx.npz, which an independent torch
implementation produced (tests/golden/make_golden_mx.py).

MXFP8: blocks of 32 elements along the block dimension share one UE8M0 scale 2^(e - 127); values
are FP8 E4M3 (bias 7, no infinities, 0x7F / 0xFF NaN, largest finite 448).

NVFP4 (no global scale factor, as in the reference's NormOutput::Nvfp4Rowwise): blocks of 16
elements share one E4M3 scale; values are FP4 E2M1 (magnitudes 0, 0.5, 1, 1.5, 2, 3, 4, 6), two per
byte, the even element in the low nibble.  The quantiser here is the device's: scale = amax / 6
rounded to nearest E4M3 (the reference's kernel, crates/cleandl-specialized-kernels/src/utils/
block_scale.rs:28-31, 55-66), elements x * (1 / scale) rounded to nearest E2M1 with ties to even
and saturation, all zero when the scale rounds to zero; the reciprocal and the product are
correctly rounded f32 operations (the reference multiplies by an approximate bf16 reciprocal),
which keeps the bits reproducible on any IEEE machine.  The reference's HOST test quantiser
(tests/matmul.rs:922-935) floors the scale at 2^-9 and breaks ties toward the smaller magnitude;
both lie within the tolerance its tests allow an NVFP4 result (0.34 |y| + 0.5 scale).
"""
from __future__ import annotations

import numpy as np

BLOCK = 32
E4M3_MAX = 448.0
ROWWISE, COLWISE = 0, 1
MXFP8, NVFP4 = 0, 1
E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float64)


def block_size(fmt: int) -> int:
    return 32 if fmt == MXFP8 else 16


def _e4m3_table() -> np.ndarray:
    out = np.zeros(256, dtype=np.float64)
    for code in range(256):
        s = -1.0 if code & 0x80 else 1.0
        e = (code >> 3) & 0xF
        m = code & 0x7
        if e == 0xF and m == 0x7:
            out[code] = np.nan
        elif e == 0:
            out[code] = s * (m / 8.0) * 2.0 ** -6
        else:
            out[code] = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
    return out


E4M3_VALUES = _e4m3_table()
_POS = E4M3_VALUES[:0x7F]  # 127 finite non-negative values, increasing


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    return E4M3_VALUES[np.asarray(codes, dtype=np.uint8)].astype(np.float32)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """Round to nearest (ties to the even code), saturating at +-448; NaN -> 0x7F."""
    x = np.asarray(x, dtype=np.float64)
    a = np.minimum(np.abs(x), E4M3_MAX)
    hi = np.clip(np.searchsorted(_POS, a, side="left"), 0, len(_POS) - 1)
    lo = np.maximum(hi - 1, 0)
    d_lo, d_hi = a - _POS[lo], _POS[hi] - a
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & (hi % 2 == 0))
    code = np.where(pick_hi, hi, lo).astype(np.uint8)
    code = np.where(np.signbit(x), code | 0x80, code).astype(np.uint8)
    return np.where(np.isnan(x), np.uint8(0x7F), code).astype(np.uint8)


def e2m1_decode(nibbles: np.ndarray) -> np.ndarray:
    n = np.asarray(nibbles, dtype=np.uint8)
    return (np.where(n & 0x8, -1.0, 1.0) * E2M1_VALUES[n & 0x7]).astype(np.float32)


def e2m1_encode(x: np.ndarray) -> np.ndarray:
    """Round to nearest (ties to the even code), saturating at +-6."""
    x = np.asarray(x, dtype=np.float64)
    a = np.minimum(np.abs(x), 6.0)
    hi = np.clip(np.searchsorted(E2M1_VALUES, a, side="left"), 0, 7)
    lo = np.maximum(hi - 1, 0)
    d_lo, d_hi = a - E2M1_VALUES[lo], E2M1_VALUES[hi] - a
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & (hi % 2 == 0))
    code = np.where(pick_hi, hi, lo).astype(np.uint8)
    return np.where(np.signbit(x), code | 0x8, code).astype(np.uint8)


def ue8m0_decode(bits: np.ndarray) -> np.ndarray:
    b = np.asarray(bits, dtype=np.int32)
    return np.where(b == 0xFF, np.nan, np.exp2((b - 127).astype(np.float64))).astype(np.float64)


def sf_index(row, block_col, num_block_cols):
    """Offset of the scale of block (row, block_col) in the 128 x 4 tiled layout."""
    row = np.asarray(row, dtype=np.int64)
    block_col = np.asarray(block_col, dtype=np.int64)
    tiles_per_row = (num_block_cols + 3) // 4
    return ((row // 128) * tiles_per_row + block_col // 4) * 512 + (row % 32) * 16 + \
        ((row % 128) // 32) * 4 + block_col % 4


def layout(rows: int, cols: int, dim: int, fmt: int = MXFP8):
    """(outer, inner, sf_rows, sf_cols): values are a packed [outer, inner] matrix of elements (the
    transpose of the logical matrix when the blocks run down the columns; one byte per element for
    MXFP8, two elements per byte for NVFP4); the scale buffer holds sf_rows * sf_cols bytes."""
    outer, inner = (rows, cols) if dim == ROWWISE else (cols, rows)
    blk = block_size(fmt)
    if inner % blk:
        raise ValueError(f"block dimension {inner} must be a multiple of {blk}")
    blocks = inner // blk
    return outer, inner, -(-outer // 128) * 128, -(-blocks // 4) * 4


def scale_exponent(amax: np.ndarray) -> np.ndarray:
    """Biased UE8M0 exponent of a block: the smallest power of two s with amax / s <= 448."""
    amax = np.asarray(amax, dtype=np.float32)
    q = (amax / np.float32(E4M3_MAX)).astype(np.float32)
    with np.errstate(divide="ignore"):
        e = np.where(q > 0, np.ceil(np.log2(q.astype(np.float64))), -127.0)
    return (np.clip(e, -127, 127) + 127).astype(np.uint8)


def quantize(m: np.ndarray, dim: int):
    """m: [rows, cols] float32.  Returns (values uint8 [outer, inner], scales uint8 [sf_rows * sf_cols])."""
    m = np.asarray(m, dtype=np.float32)
    rows, cols = m.shape
    outer, inner, sf_rows, sf_cols = layout(rows, cols, dim)
    src = m if dim == ROWWISE else m.T
    blocks = inner // BLOCK
    blk = np.ascontiguousarray(src).reshape(outer, blocks, BLOCK)
    e = scale_exponent(np.abs(blk).max(axis=2))
    scale = np.exp2(e.astype(np.float64) - 127.0)
    values = e4m3_encode(blk.astype(np.float64) / scale[:, :, None]).reshape(outer, inner)
    scales = np.zeros(sf_rows * sf_cols, dtype=np.uint8)
    o, b = np.meshgrid(np.arange(outer), np.arange(blocks), indexing="ij")
    scales[sf_index(o, b, blocks)] = e
    return values, scales


def dequantize(values: np.ndarray, scales: np.ndarray, rows: int, cols: int, dim: int):
    """Returns (matrix float32 [rows, cols], element_scales float32 [rows, cols])."""
    outer, inner, _, _ = layout(rows, cols, dim)
    blocks = inner // BLOCK
    o, b = np.meshgrid(np.arange(outer), np.arange(blocks), indexing="ij")
    s = ue8m0_decode(np.asarray(scales, dtype=np.uint8).reshape(-1)[sf_index(o, b, blocks)])
    s = np.repeat(s, BLOCK, axis=1)
    v = e4m3_decode(np.asarray(values, dtype=np.uint8).reshape(outer, inner)).astype(np.float64) * s
    if dim == COLWISE:
        v, s = v.T, s.T
    return np.ascontiguousarray(v).astype(np.float32), np.ascontiguousarray(s).astype(np.float32)


def output_tolerance(expected: np.ndarray, element_scales: np.ndarray, rel=0.07, unit=2.0 ** -9):
    """Allowed |got - expected| for a block-scaled output checked against unquantised values:
    three mantissa bits plus the rounding of the input to bf16, and the subnormal step."""
    return rel * np.abs(expected) + unit * element_scales + 1e-30


def quantize_nvfp4(m: np.ndarray, dim: int):
    """m: [rows, cols] float32.  Returns (values uint8 [outer, inner / 2], scales uint8 flat)."""
    m = np.asarray(m, dtype=np.float32)
    rows, cols = m.shape
    outer, inner, sf_rows, sf_cols = layout(rows, cols, dim, NVFP4)
    src = np.ascontiguousarray(m if dim == ROWWISE else m.T)
    blocks = inner // 16
    blk = src.reshape(outer, blocks, 16)
    amax = np.abs(blk).max(axis=2)
    sbits = e4m3_encode((amax / np.float32(6.0)).astype(np.float32))
    scale = e4m3_decode(sbits)  # float32
    with np.errstate(divide="ignore", invalid="ignore"):
        inv = np.where(scale == 0, np.float32(0), np.float32(1) / scale).astype(np.float32)
    q = (blk * inv[:, :, None]).astype(np.float32)
    codes = e2m1_encode(q).reshape(outer, inner)
    values = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    scales = np.zeros(sf_rows * sf_cols, dtype=np.uint8)
    o, b = np.meshgrid(np.arange(outer), np.arange(blocks), indexing="ij")
    scales[sf_index(o, b, blocks)] = sbits
    return values, scales


def dequantize_nvfp4(values: np.ndarray, scales: np.ndarray, rows: int, cols: int, dim: int):
    """Returns (matrix float32 [rows, cols], element_scales float32 [rows, cols])."""
    outer, inner, _, _ = layout(rows, cols, dim, NVFP4)
    blocks = inner // 16
    v = np.asarray(values, dtype=np.uint8).reshape(outer, inner // 2)
    codes = np.empty((outer, inner), dtype=np.uint8)
    codes[:, 0::2] = v & 0xF
    codes[:, 1::2] = v >> 4
    o, b = np.meshgrid(np.arange(outer), np.arange(blocks), indexing="ij")
    s = e4m3_decode(np.asarray(scales, dtype=np.uint8).reshape(-1)[sf_index(o, b, blocks)])
    s = np.repeat(s.astype(np.float64), 16, axis=1)
    out = e2m1_decode(codes).astype(np.float64) * s
    if dim == COLWISE:
        out, s = out.T, s.T
    return np.ascontiguousarray(out).astype(np.float32), np.ascontiguousarray(s).astype(np.float32)
