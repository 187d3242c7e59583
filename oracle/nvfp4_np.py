"""CPU oracle (test infrastructure, never shipped): the NVFP4 codec in numpy.

This file restates, with numpy only, the reference's codec
(muse_moe_w4a16/nvfp4.py, identical copy in muse_decode_layer/nvfp4.py):

* a stored value is  e2m1 code * e4m3 block scale * fp32 global scale     (nvfp4.py:1-8)
* two E2M1 codes per byte, element 2i in the low nibble                   (nvfp4.py:40-57)
* one E4M3 scale per 16 contiguous elements of the last dim               (nvfp4.py:16, 66-87)
* rounding to the E2M1 grid goes through the midpoints with
  ``bucketize(right=False)``: an exact midpoint goes to the smaller
  magnitude, |v| clamps to 6, values that round to 0 never carry a sign   (nvfp4.py:50-57)

Only tests, ``__graft_entry__.smoke`` and the ``cpu_baseline`` / reference arm of
``bench.py`` may import it; the product path never does.  It is pinned against
vectors produced by the reference's own module (tests/golden/make_golden.py).
"""
from __future__ import annotations

import numpy as np

BLOCK = 16
E2M1_MAX = np.float32(6.0)
E4M3_MAX = np.float32(448.0)

# magnitude of each 3-bit E2M1 code, sign is bit 3 (nvfp4.py:22-25)
E2M1_GRID = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_MIDS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)


def _e4m3_table() -> np.ndarray:
    """All 256 float8_e4m3fn bit patterns as float32 (0x7f / 0xff are NaN)."""
    t = np.empty(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 0x7
        if e == 0xF and m == 0x7:
            v = float("nan")
        elif e == 0:
            v = s * (m / 8.0) * 2.0 ** -6
        else:
            v = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[b] = v
    return t


E4M3_TABLE = _e4m3_table()
_E4M3_POS = E4M3_TABLE[:0x7F].copy()  # codes 0x00..0x7e: 0 .. 448, strictly increasing


def e4m3_to_f32(codes: np.ndarray) -> np.ndarray:
    """uint8 e4m3 bit patterns -> float32 (what ``sf.float()`` gives, nvfp4.py:83,96)."""
    return E4M3_TABLE[np.asarray(codes, dtype=np.uint8)]


def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    """float32 -> e4m3 bit patterns, round to nearest, ties to the even code.

    Stands for ``.to(torch.float8_e4m3fn)`` at nvfp4.py:82 on inputs already clamped to
    [-448, 448] (the only inputs the codec produces).
    """
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x)
    hi = np.searchsorted(_E4M3_POS, a, side="left")          # first code with value >= a
    hi = np.clip(hi, 0, len(_E4M3_POS) - 1)
    lo = np.clip(hi - 1, 0, None)
    d_hi = _E4M3_POS[hi].astype(np.float64) - a.astype(np.float64)
    d_lo = a.astype(np.float64) - _E4M3_POS[lo].astype(np.float64)
    pick_lo = (d_lo < d_hi) | ((d_lo == d_hi) & ((lo & 1) == 0))
    pick_lo &= hi != lo
    code = np.where(pick_lo, lo, hi).astype(np.uint8)
    return (code | (np.signbit(x).astype(np.uint8) << 7)).astype(np.uint8)


def unpack_e2m1(packed: np.ndarray) -> np.ndarray:
    """uint8 [..., K/2] -> float32 [..., K] unscaled E2M1 values (nvfp4.py:40-47)."""
    p = np.asarray(packed, dtype=np.uint8)
    codes = np.stack((p & 0x0F, (p >> 4) & 0x0F), axis=-1).reshape(*p.shape[:-1], p.shape[-1] * 2)
    mag = E2M1_GRID[codes & 0x7]
    return np.where((codes & 0x8) != 0, -mag, mag).astype(np.float32)


def pack_e2m1(values: np.ndarray) -> np.ndarray:
    """float [..., K] (already divided by the scale) -> uint8 [..., K/2] (nvfp4.py:50-57)."""
    v = np.asarray(values, dtype=np.float32)
    a = np.minimum(np.abs(v), E2M1_MAX)
    mag = np.searchsorted(E2M1_MIDS, a, side="left").astype(np.uint8)   # bucketize(right=False)
    sign = ((v < 0) & (mag > 0)).astype(np.uint8) << 3
    codes = (sign | mag).reshape(*v.shape[:-1], v.shape[-1] // 2, 2)
    return (codes[..., 0] | (codes[..., 1] << 4)).astype(np.uint8)


def global_scale_for(amax) -> np.float32:
    """Tensor scale that puts the largest block scale at the top of E4M3 (nvfp4.py:60-63)."""
    amax = np.float32(amax)
    return np.float32(amax / np.float32(float(E2M1_MAX) * float(E4M3_MAX))) if amax > 0 else np.float32(1.0)


def quantize(x: np.ndarray, global_scale=None):
    """Quantise the last dim to NVFP4 (nvfp4.py:66-87).

    Returns (packed uint8 [..., K/2], e4m3 codes uint8 [..., K/16], global scale float32).
    """
    xf = np.asarray(x, dtype=np.float32)
    k = xf.shape[-1]
    if k % BLOCK:
        raise ValueError(f"last dim {k} is not a multiple of {BLOCK}")
    gs = global_scale_for(np.abs(xf).max()) if global_scale is None else np.float32(global_scale)
    blocks = xf.reshape(*xf.shape[:-1], k // BLOCK, BLOCK)
    block_amax = np.abs(blocks).max(axis=-1)
    sf = f32_to_e4m3(np.minimum((block_amax / E2M1_MAX / gs).astype(np.float32), E4M3_MAX))
    scale = (e4m3_to_f32(sf) * gs).astype(np.float32)[..., None]
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(scale > 0, blocks / scale, np.float32(0.0)).astype(np.float32)
    return pack_e2m1(q.reshape(xf.shape)), sf, gs


def dequantize(packed: np.ndarray, sf: np.ndarray, global_scale) -> np.ndarray:
    """Inverse of quantize, float32 [..., K] (nvfp4.py:90-97)."""
    vals = unpack_e2m1(packed)
    k = vals.shape[-1]
    blocks = vals.reshape(*vals.shape[:-1], k // BLOCK, BLOCK)
    scale = (e4m3_to_f32(sf) * np.float32(global_scale)).astype(np.float32)[..., None]
    return (blocks * scale).astype(np.float32).reshape(vals.shape)


def fake_quantize(x: np.ndarray, global_scale=None) -> np.ndarray:
    """quantize then dequantize (nvfp4.py:100-102)."""
    return dequantize(*quantize(x, global_scale))
