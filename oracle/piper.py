"""numpy restatement of the reference's portable Piper attention (test infrastructure).

Follows src/piper_kernels/attention/piper/reference.py:40-156 of the reference
project step by step: K smoothing, optional V centering, optional centered-row-range
ordering, INT8 Q/K in either granularity, per-key INT8 V, then the 64-key online
softmax loop with a UINT8 probability operand and the mean-restoring epilogue.
"""

from __future__ import annotations

import numpy as np

from .quantizers import (
    KEY_BLOCK,
    QUERY_BLOCK,
    quantize_key_per_thread,
    quantize_per_group,
    quantize_query_per_thread,
    quantize_value_per_key,
    round_to_dtype,
    sequence_mean,
)

PV_BLOCK = 64  # piper/reference.py:21
P_RANGE = np.float32(255.0)  # piper/reference.py:22


def centered_value_order(value_centered: np.ndarray) -> np.ndarray:
    """Stable ascending order of ``max_d |v - mean|`` per key row (piper/reference.py:67-68)."""
    row_range = np.abs(value_centered).max(axis=-1)
    return np.argsort(row_range, axis=-1, kind="stable").astype(np.int64)


def piper_prepare_oracle(
    q: np.ndarray,
    k: np.ndarray,
    v: np.ndarray,
    *,
    center_value: bool,
    qk_quantization: str = "per_warp",
    sort_value_rows: bool = False,
    k_mean: np.ndarray | None = None,
    v_mean: np.ndarray | None = None,
) -> dict:
    """Everything the reference computes before its tile loop (piper/reference.py:55-91).

    ``k_mean`` / ``v_mean`` (``[B,H,1,D]`` float32) replace the computed means when
    given, so that codes can be compared bit-for-bit with a run that used another
    summation order.
    """
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    if k_mean is None:
        k_mean = sequence_mean(k)
    k_centered = k - k_mean
    if center_value:
        if v_mean is None:
            v_mean = sequence_mean(v)
    else:
        v_mean = np.zeros_like(v[:, :, :1])
    v_centered = v - v_mean

    order = None
    if sort_value_rows:
        order = centered_value_order(v_centered)
        k_centered = np.take_along_axis(k_centered, order[..., None], axis=2)
        v_centered = np.take_along_axis(v_centered, order[..., None], axis=2)

    if qk_quantization == "per_warp":
        q8, q_group_scale = quantize_per_group(q, QUERY_BLOCK)
        k8, k_group_scale = quantize_per_group(k_centered, KEY_BLOCK)
        q_scale = np.repeat(q_group_scale, QUERY_BLOCK, axis=2)[:, :, : q.shape[2]]
        k_scale = np.repeat(k_group_scale, KEY_BLOCK, axis=2)[:, :, : k.shape[2]]
    elif qk_quantization == "per_thread":
        q8, q_scale = quantize_query_per_thread(q)
        k8, k_scale = quantize_key_per_thread(k_centered)
        q_group_scale, k_group_scale = q_scale, k_scale
    else:
        raise ValueError(f"unknown Q/K quantization granularity: {qk_quantization}")
    v8, v_scale = quantize_value_per_key(v_centered)
    return {
        "k_mean": k_mean,
        "v_mean": v_mean,
        "order": order,
        "q_codes": q8,
        "k_codes": k8,
        "v_codes": v8,
        "q_scale": q_scale,  # per row
        "k_scale": k_scale,  # per row
        "q_group_scale": q_group_scale,  # in the reference's own layout
        "k_group_scale": k_group_scale,
        "v_scale": v_scale,
    }


def piper_attention_oracle(
    q: np.ndarray,
    k: np.ndarray,
    v: np.ndarray,
    scale: float,
    is_causal: bool,
    *,
    center_value: bool,
    qk_quantization: str = "per_warp",
    sort_value_rows: bool = False,
    out_dtype: str = "f32",
    k_mean: np.ndarray | None = None,
    v_mean: np.ndarray | None = None,
    heads: slice | None = None,
) -> np.ndarray:
    """Piper attention forward on CPU; returns float32 values rounded to ``out_dtype``.

    ``heads`` restricts the tile loop to a slice of the flattened (batch*heads) axis
    (used to time a bounded sample); the result then has shape ``[n, Sq, D]``.
    """
    if sort_value_rows and is_causal:
        raise ValueError("value-row ordering is valid only for non-causal attention")
    prep = piper_prepare_oracle(
        q, k, v, center_value=center_value, qk_quantization=qk_quantization,
        sort_value_rows=sort_value_rows, k_mean=k_mean, v_mean=v_mean,
    )
    b, h, sq, d = prep["q_codes"].shape
    flat = lambda a: a.reshape(b * h, *a.shape[2:])  # noqa: E731
    q8, k8, v8 = flat(prep["q_codes"]), flat(prep["k_codes"]), flat(prep["v_codes"])
    qs, ks, vs = flat(prep["q_scale"]), flat(prep["k_scale"]), flat(prep["v_scale"])
    vmean = flat(prep["v_mean"])
    sel = range(b * h)[heads] if heads is not None else range(b * h)
    out = np.empty((len(sel), sq, d), dtype=np.float32)
    for oi, bh in enumerate(sel):
        out[oi] = piper_tile_loop(q8[bh], qs[bh], k8[bh], ks[bh], v8[bh], vs[bh], vmean[bh], scale, is_causal)
    out = round_to_dtype(out, out_dtype)
    if heads is None:
        out = out.reshape(b, h, sq, d)
    return out


def piper_tile_loop(q8, qs, k8, ks, v8, vs, vmean, scale, is_causal, row0: int = 0) -> np.ndarray:
    """The 64-key online-softmax loop of one head (piper/reference.py:93-156) for the query
    rows given (``row0`` is the position of the first one, used by the causal mask).
    Inputs: int8 codes ``q8 [R,D]``, ``k8 [Sk,D]``, ``v8 [Sk,D]``; per-row float32 scales
    ``qs [R]``, ``ks [Sk]``, ``vs [Sk]``; ``vmean [1,D]``.  Returns float32 ``[R,D]``."""
    sq, d = q8.shape
    sk = k8.shape[0]
    scale32 = np.float32(scale)
    qpos = np.arange(row0, row0 + sq)
    qf = q8.astype(np.float32)
    num = np.zeros((sq, d), dtype=np.float32)
    den = np.zeros((sq,), dtype=np.float32)
    run_max = np.full((sq,), -np.inf, dtype=np.float32)
    for start in range(0, sk, PV_BLOCK):
        stop = min(start + PV_BLOCK, sk)
        kf = k8[start:stop].astype(np.float32)
        int_scores = qf @ kf.T  # exact: |sum| < 2^24
        scores = int_scores * qs[:, None] * ks[None, start:stop] * scale32
        if is_causal:
            kpos = np.arange(start, stop)
            scores = np.where(kpos[None, :] > qpos[:, None], np.float32(-np.inf), scores)
        bvs = vs[start:stop]
        shifted = scores + np.log(bvs)[None, :]
        block_max = shifted.max(axis=-1)
        next_max = np.maximum(run_max, block_max)
        with np.errstate(invalid="ignore", over="ignore"):
            old_w = np.exp(run_max - next_max)
            cur_w = np.exp(block_max - next_max)
            p = np.exp(scores - block_max[:, None])
        p = np.nan_to_num(p)  # piper/reference.py:135
        num *= old_w[:, None]
        den = den * old_w + p.sum(axis=-1, dtype=np.float32) * cur_w
        p8 = np.clip(np.rint(p * bvs[None, :] * P_RANGE), 0.0, P_RANGE)
        partial = p8 @ v8[start:stop].astype(np.float32)  # exact integers
        num += partial * (cur_w[:, None] / P_RANGE)
        run_max = next_max
    o = num / np.maximum(den, np.float32(1e-30))[:, None]
    return o + vmean
