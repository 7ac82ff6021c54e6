"""numpy restatement of the reference's portable SageAttention2++ 8+8 forward
(test infrastructure).  Follows src/piper_kernels/attention/sage2pp/reference.py:31-121
of the reference project: K smoothing, INT8 Q/K, per-channel E4M3 V (range 2.25),
E4M3 probabilities (range 448) relative to the running maximum, 64-key PV partials
rounded once to FP16 and accumulated in FP32.
"""

from __future__ import annotations

import numpy as np

from .quantizers import (
    KEY_BLOCK,
    QUERY_BLOCK,
    e4m3_decode,
    e4m3_encode,
    quantize_key_per_thread,
    quantize_per_group,
    quantize_query_per_thread,
    quantize_value_per_channel_e4m3,
    round_to_dtype,
    sequence_mean,
)

PV_BLOCK = 64  # sage2pp/reference.py:19
P_FP8_RANGE = np.float32(448.0)  # sage2pp/reference.py:20


def sage_prepare_oracle(q, k, v, *, qk_quantization: str = "per_thread", k_mean=None) -> dict:
    """Quantities computed before the tile loop (sage2pp/reference.py:46-68)."""
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    if k_mean is None:
        k_mean = sequence_mean(k)
    k_centered = k - k_mean
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
    v8, v_scale = quantize_value_per_channel_e4m3(v)
    return {
        "k_mean": k_mean, "q_codes": q8, "k_codes": k8, "v_codes": v8,
        "q_scale": q_scale, "k_scale": k_scale,
        "q_group_scale": q_group_scale, "k_group_scale": k_group_scale, "v_scale": v_scale,
    }


def sage_attention_2pp_oracle(
    q, k, v, scale: float, is_causal: bool, *,
    qk_quantization: str = "per_thread", out_dtype: str = "f32", k_mean=None,
    heads: slice | None = None,
) -> np.ndarray:
    """SageAttention2++ forward on CPU; float32 values rounded to ``out_dtype``."""
    prep = sage_prepare_oracle(q, k, v, qk_quantization=qk_quantization, k_mean=k_mean)
    b, h, sq, d = prep["q_codes"].shape
    sk = prep["k_codes"].shape[2]
    flat = lambda a: a.reshape(b * h, *a.shape[2:])  # noqa: E731
    q8, k8 = flat(prep["q_codes"]), flat(prep["k_codes"])
    vf = flat(e4m3_decode(prep["v_codes"]))
    qs, ks, vs = flat(prep["q_scale"]), flat(prep["k_scale"]), flat(prep["v_scale"])
    sel = range(b * h)[heads] if heads is not None else range(b * h)
    out = np.empty((len(sel), sq, d), dtype=np.float32)
    scale32 = np.float32(scale)
    qpos = np.arange(sq)
    for oi, bh in enumerate(sel):
        qf = q8[bh].astype(np.float32)
        acc = np.zeros((sq, d), dtype=np.float32)
        den = np.zeros((sq,), dtype=np.float32)
        run_max = np.full((sq,), -np.inf, dtype=np.float32)
        for start in range(0, sk, PV_BLOCK):
            stop = min(start + PV_BLOCK, sk)
            int_scores = qf @ k8[bh, start:stop].astype(np.float32).T
            scores = int_scores * qs[bh][:, None] * ks[bh][None, start:stop] * scale32
            if is_causal:
                kpos = np.arange(start, stop)
                scores = np.where(kpos[None, :] > qpos[:, None], np.float32(-np.inf), scores)
            block_max = scores.max(axis=-1)
            next_max = np.maximum(run_max, block_max)
            with np.errstate(invalid="ignore", over="ignore"):
                old_w = np.exp(run_max - next_max)
                p = np.exp(scores - next_max[:, None])
            p = np.nan_to_num(p)
            acc *= old_w[:, None]
            den = den * old_w + p.sum(axis=-1, dtype=np.float32)
            p8 = e4m3_decode(e4m3_encode(p * P_FP8_RANGE))
            partial = p8 @ vf[bh, start:stop]
            partial = partial.astype(np.float16).astype(np.float32)  # sage2pp/reference.py:113-116
            acc += partial * (vs[bh][None, :] / P_FP8_RANGE)
            run_max = next_max
        out[oi] = acc / np.maximum(den, np.float32(1e-30))[:, None]
    out = round_to_dtype(out, out_dtype)
    if heads is None:
        out = out.reshape(b, h, sq, d)
    return out
