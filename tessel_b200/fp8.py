"""FP8 (E4M3) row quantisation on the host: the weight side of the engine's FP8 mode.

A separate, NON-PARITY mode (the reference computes in f16 throughout): weights are stored as
E4M3 bytes with one f32 scale per output row, activations are quantised per row on the device
just before each projection, and the projections run on the tensor cores' 8-bit path
(``tcgen05.mma.kind::f8f6f4``) with f32 accumulation; the product is scaled back by
``row scale x column scale`` in the epilogue. Everything else (attention, RoPE, the KV cache,
norms, the LM head) stays f16 / f32.

E4M3 here is the OCP "FN" format CUDA's ``__NV_E4M3`` implements: 1 sign, 4 exponent (bias 7),
3 mantissa bits, no infinities, largest finite value 448, subnormals down to 2^-9. Conversion
rounds to nearest, ties to even, and saturates at +-448, as ``__nv_cvt_float_to_fp8(x,
__NV_SATFINITE, __NV_E4M3)`` does, so that the device's quantiser and this one give the same bytes.
"""
from __future__ import annotations

import numpy as np

E4M3_MAX = 448.0


def _positive_values() -> np.ndarray:
    """The 127 non-negative finite E4M3 values; index = bit pattern (0x00 .. 0x7e)."""
    v = np.zeros(127, np.float64)
    for code in range(127):
        e, m = code >> 3, code & 7
        v[code] = (m / 8.0) * 2.0 ** -6 if e == 0 else (1.0 + m / 8.0) * 2.0 ** (e - 7)
    return v


_VALUES = _positive_values()
_MIDS = (_VALUES[:-1] + _VALUES[1:]) / 2.0
_DECODE = np.concatenate([_VALUES, [np.nan], -_VALUES, [np.nan]]).astype(np.float32)


def encode(x: np.ndarray) -> np.ndarray:
    """f32 -> E4M3 bytes: round to nearest even, saturate at +-448 (NaN -> 0x7f)."""
    x = np.asarray(x, np.float32)
    ax = np.abs(x).astype(np.float64)
    code = np.searchsorted(_MIDS, ax, side="left")        # mids strictly below |x|
    code = np.minimum(code, 126)
    # A value exactly on a midpoint goes to the neighbour with the even bit pattern.
    k = np.minimum(code, 125)
    tie = (ax == _MIDS[k]) & (code <= 125)
    code = np.where(tie & (k % 2 == 1), k + 1, code)
    out = code.astype(np.uint8) | np.where(np.signbit(x), 0x80, 0).astype(np.uint8)
    return np.where(np.isnan(x), np.uint8(0x7F), out).astype(np.uint8)


def decode(q: np.ndarray) -> np.ndarray:
    """E4M3 bytes -> f32."""
    return _DECODE[np.asarray(q, np.uint8)]


def quantize_rows(w: np.ndarray):
    """Per-row quantisation of a matrix: returns (q uint8 [rows, cols], scale f32 [rows]) with
    ``w ~= decode(q) * scale[:, None]``. scale = max|row| / 448 (1 for an all-zero row), the
    division and the rounding done in f32 exactly as the device's ``quant_rows`` does them."""
    w = np.asarray(w, np.float32)
    amax = np.abs(w).max(axis=1) if w.shape[1] else np.zeros(w.shape[0], np.float32)
    scale = np.where(amax > 0, amax / np.float32(E4M3_MAX), np.float32(1.0)).astype(np.float32)
    return encode(w / scale[:, None]), scale
