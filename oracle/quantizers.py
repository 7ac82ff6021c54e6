"""numpy restatement of the reference's Q/K/V quantizers (test infrastructure).

Every function takes float32 arrays laid out ``[batch, heads, sequence, head_dim]``
whose values are exactly the FP16/BF16 inputs widened to FP32, and performs the
arithmetic in IEEE float32 exactly as the reference does with torch on CPU:
true division, round-half-to-even, then clamp.

Reference locations (paths inside the reference project):
  * src/piper_kernels/attention/kernels/qk_quantization/int8/sage/reference.py:5-74
  * src/piper_kernels/attention/piper/reference.py:27-37
  * src/piper_kernels/attention/sage2pp/reference.py:25-28
"""

from __future__ import annotations

import numpy as np

QUERY_BLOCK = 32  # sage/reference.py:5
KEY_BLOCK = 64  # sage/reference.py:6
SCALE_EPSILON = np.float32(1e-7)  # sage/reference.py:7, piper/reference.py:24

_F32 = np.float32


def _as_f32(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x)
    if x.dtype != np.float32:
        x = x.astype(np.float32)
    return x


def _pad_sequence(x: np.ndarray, multiple: int) -> tuple[np.ndarray, int]:
    """Zero-pad the sequence axis to a multiple (sage/reference.py:10-17)."""
    length = x.shape[2]
    padded_length = -(-length // multiple) * multiple
    if padded_length == length:
        return x, length
    out = np.zeros((*x.shape[:2], padded_length, x.shape[3]), dtype=x.dtype)
    out[:, :, :length] = x
    return out, length


def _codes(grouped: np.ndarray, scale: np.ndarray, qrange: int) -> np.ndarray:
    # (x / scale).round().clamp(-r, r).to(int8): IEEE division, ties to even.
    q = np.rint(grouped / scale)
    return np.clip(q, -qrange, qrange).astype(np.int8)


def sequence_mean(x: np.ndarray) -> np.ndarray:
    """Per-(batch, head, feature) mean over the sequence, ``[B,H,1,D]`` float32.

    The reference calls ``tensor.float().mean(dim=2, keepdim=True)``
    (piper/reference.py:58,60-64; sage2pp/reference.py:49).  torch's FP32 reduction
    order is an implementation detail, so this restatement defines the mean as the
    float64 sum divided by the length, rounded once to float32 (the correctly
    rounded mean).  The CUDA prepass accumulates in FP64 for the same reason, and
    both accept an injected mean for bit-exact comparisons with the reference.
    """
    x = _as_f32(x)
    s = x.sum(axis=2, keepdims=True, dtype=np.float64)
    return (s / np.float64(x.shape[2])).astype(np.float32)


def quantize_per_group(x: np.ndarray, group_size: int, qrange: int = 127):
    """One scale per ``group_size`` consecutive rows (sage/reference.py:58-74).

    Returns ``(int8 codes [B,H,S,D], float32 scale [B,H,ceil(S/group)])``.
    """
    x = _as_f32(x)
    padded, length = _pad_sequence(x, group_size)
    b, h, _, d = padded.shape
    grouped = padded.reshape(b, h, -1, group_size, d)
    scale = np.abs(grouped).max(axis=(3, 4)) / _F32(qrange) + SCALE_EPSILON
    q = _codes(grouped, scale[..., None, None], qrange)
    return q.reshape(padded.shape)[:, :, :length], scale.astype(np.float32)


def quantize_query_per_thread(x: np.ndarray, qrange: int = 127):
    """Four interleaved rows {t, t+8, t+16, t+24} of each 32-row block share a scale
    (sage/reference.py:20-36).  Returns codes and a per-row scale ``[B,H,S]``."""
    x = _as_f32(x)
    padded, length = _pad_sequence(x, QUERY_BLOCK)
    b, h, _, d = padded.shape
    grouped = padded.reshape(b, h, -1, 4, 8, d)
    scale_group = np.abs(grouped).max(axis=(3, 5)) / _F32(qrange) + SCALE_EPSILON
    scale = np.broadcast_to(scale_group[:, :, :, None, :, None], grouped.shape)
    q = _codes(grouped, scale, qrange)
    row_scale = scale[..., 0].reshape(padded.shape[:3])
    return q.reshape(padded.shape)[:, :, :length], np.ascontiguousarray(row_scale[:, :, :length])


def quantize_key_per_thread(x: np.ndarray, qrange: int = 127):
    """Sixteen interleaved rows ``8a + 2t + c`` (a<8, c<2) of each 64-row block share
    scale ``t`` (sage/reference.py:39-55).  Returns codes and per-row scale."""
    x = _as_f32(x)
    padded, length = _pad_sequence(x, KEY_BLOCK)
    b, h, _, d = padded.shape
    grouped = padded.reshape(b, h, -1, 8, 4, 2, d)
    scale_group = np.abs(grouped).max(axis=(3, 5, 6)) / _F32(qrange) + SCALE_EPSILON
    scale = np.broadcast_to(scale_group[:, :, :, None, :, None, None], grouped.shape)
    q = _codes(grouped, scale, qrange)
    row_scale = scale[..., 0].reshape(padded.shape[:3])
    return q.reshape(padded.shape)[:, :, :length], np.ascontiguousarray(row_scale[:, :, :length])


def quantize_value_per_key(v: np.ndarray):
    """Signed INT8 with one scale per key row (piper/reference.py:27-37)."""
    v = _as_f32(v)
    scale = np.abs(v).max(axis=-1) / _F32(127.0) + SCALE_EPSILON
    q = np.clip(np.rint(v / scale[..., None]), -127.0, 127.0).astype(np.int8)
    return q, scale.astype(np.float32)


# ---------------------------------------------------------------------------
# E4M3 (float8_e4m3fn): 1 sign, 4 exponent (bias 7), 3 mantissa bits, no inf,
# max finite 448.  torch's cast rounds to nearest even; the values met on this
# path satisfy |x| <= 448, so saturation never triggers.
# ---------------------------------------------------------------------------

def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """Round float32 to E4M3 (nearest, ties to even) and return the byte codes."""
    x = _as_f32(x)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    a = np.abs(x).astype(np.float64)
    a = np.minimum(a, 448.0)
    # exponent of the binade, clamped to the subnormal binade (2^-6)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.maximum(e, -6.0)
    step = np.exp2(e - 3.0)  # spacing inside the binade (subnormals: 2^-9)
    m = np.rint(a / step)  # integer in [0, 16]
    val = m * step  # rounded magnitude (may have carried into the next binade)
    # re-derive fields from the rounded value
    with np.errstate(divide="ignore"):
        e2 = np.floor(np.log2(np.where(val > 0, val, 1.0)))
    e2 = np.maximum(e2, -6.0)
    is_sub = val < 2.0**-6
    mant = np.where(is_sub, val / 2.0**-9, val / np.exp2(e2 - 3.0) - 8.0)
    expo = np.where(is_sub, 0.0, e2 + 7.0)
    code = (expo.astype(np.uint8) << 3) | mant.astype(np.uint8)
    return (code | sign).astype(np.uint8)


def e4m3_decode(code: np.ndarray) -> np.ndarray:
    """Byte codes to float32 values."""
    code = np.asarray(code, dtype=np.uint8)
    sign = np.where(code & 0x80, -1.0, 1.0)
    expo = ((code >> 3) & 0xF).astype(np.int32)
    mant = (code & 0x7).astype(np.float64)
    val = np.where(expo == 0, mant * 2.0**-9, (8.0 + mant) * np.exp2(expo.astype(np.float64) - 10.0))
    return (sign * val).astype(np.float32)


def quantize_value_per_channel_e4m3(v: np.ndarray):
    """Sage2++ V: one scale per (batch, head, feature) = amax over keys / 2.25 + 1e-7;
    codes = E4M3(v / scale) (sage2pp/reference.py:25-28).  Returns (uint8 codes, scale [B,H,D])."""
    v = _as_f32(v)
    scale = np.abs(v).max(axis=2) / _F32(2.25) + SCALE_EPSILON
    codes = e4m3_encode(v / scale[:, :, None, :])
    return codes, scale.astype(np.float32)


def round_to_dtype(x: np.ndarray, dtype: str) -> np.ndarray:
    """Round float32 to 'f16' / 'bf16' (nearest even) and widen back to float32; 'f32' is identity."""
    x = _as_f32(x)
    if dtype == "f32":
        return x
    if dtype == "f16":
        return x.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        bits = x.view(np.uint32).astype(np.uint64)
        rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
        out = rounded.astype(np.uint32).view(np.float32)
        return np.where(np.isnan(x), x, out)
    raise ValueError(f"unknown dtype {dtype}")
