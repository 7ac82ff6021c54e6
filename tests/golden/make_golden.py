"""Generate the golden fixtures in this directory from the reference project itself.

Run once, in a container where the reference source tree is present:

    PIPER_REF_SRC=/path/to/reference/src python tests/golden/make_golden.py

It imports the reference's portable PyTorch implementation (CPU), runs it on small
seeded inputs, and stores inputs, intermediate integer codes / scales / means / order
and outputs as ``.npz`` files.  The fixtures pin the numpy oracle under ``oracle/``;
nothing in the test-suite needs the reference tree at run time.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

REF = os.environ["PIPER_REF_SRC"]  # path of the reference project's src/ directory
sys.path.insert(0, REF)

from piper_kernels.attention.kernels.qk_quantization.int8.sage.reference import (  # noqa: E402
    quantize_key_per_thread,
    quantize_per_group,
    quantize_query_per_thread,
)
from piper_kernels.attention.piper.reference import (  # noqa: E402
    _quantize_value_per_key,
    reference_piper_attention,
)
from piper_kernels.attention.sage2pp.reference import (  # noqa: E402
    _quantize_value_per_channel,
    reference_sage_attention_2pp,
)

HERE = Path(__file__).resolve().parent
torch.set_num_threads(1)  # fixed reduction order for the stored means


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().astype(np.uint16)


def quantizer_outputs(q, kc, granularity):
    if granularity == "per_warp":
        q8, qs = quantize_per_group(q, 32, 127)
        k8, ks = quantize_per_group(kc, 64, 127)
    else:
        q8, qs = quantize_query_per_thread(q, 127)
        k8, ks = quantize_key_per_thread(kc, 127)
    return q8.numpy(), qs.numpy(), k8.numpy(), ks.numpy()


def piper_case(name, q, k, v, *, causal, center, sort, scale=None):
    d = q.shape[-1]
    scale = d**-0.5 if scale is None else scale
    rec = {
        "kind": "piper", "dtype": str(q.dtype).split(".")[-1], "causal": causal, "center": center,
        "sort": sort, "scale": np.float64(scale),
        "q": bits16(q), "k": bits16(k), "v": bits16(v),
    }
    kf, vf = k.float(), v.float()
    k_mean = kf.mean(dim=2, keepdim=True)
    v_mean = vf.mean(dim=2, keepdim=True) if center else torch.zeros_like(vf[:, :, :1])
    kc, vc = kf - k_mean, vf - v_mean
    rec["k_mean"], rec["v_mean"] = k_mean.numpy(), v_mean.numpy()
    if sort:
        order = torch.argsort(vc.abs().amax(dim=-1), dim=-1, stable=True)
        rec["order"] = order.numpy()
        idx = order[..., None].expand_as(kc)
        kc, vc = torch.gather(kc, 2, idx), torch.gather(vc, 2, idx)
    v8, vs = _quantize_value_per_key(vc)
    rec["v_codes"], rec["v_scale"] = v8.numpy(), vs.numpy()
    for gran in ("per_warp", "per_thread"):
        q8, qs, k8, ks = quantizer_outputs(q, kc, gran)
        rec[f"q_codes_{gran}"], rec[f"q_scale_{gran}"] = q8, qs
        rec[f"k_codes_{gran}"], rec[f"k_scale_{gran}"] = k8, ks
        if sort and gran == "per_thread":
            continue  # the reference only orders rows with grouped (per-warp) Q/K
        out32 = reference_piper_attention(
            q.float(), k.float(), v.float(), scale, causal,
            center_value=center, qk_quantization=gran, sort_value_rows=sort)
        out16 = reference_piper_attention(
            q, k, v, scale, causal, center_value=center, qk_quantization=gran, sort_value_rows=sort)
        rec[f"out32_{gran}"] = out32.numpy()
        rec[f"out16_{gran}"] = bits16(out16)
    np.savez_compressed(HERE / f"{name}.npz", **rec)
    print("wrote", name)


def sage_case(name, q, k, v, *, causal, scale=None):
    d = q.shape[-1]
    scale = d**-0.5 if scale is None else scale
    rec = {
        "kind": "sage2pp", "dtype": str(q.dtype).split(".")[-1], "causal": causal,
        "scale": np.float64(scale), "q": bits16(q), "k": bits16(k), "v": bits16(v),
    }
    kf = k.float()
    k_mean = kf.mean(dim=2, keepdim=True)
    kc = kf - k_mean
    rec["k_mean"] = k_mean.numpy()
    v8, vs = _quantize_value_per_channel(v)
    rec["v_codes"] = v8.view(torch.uint8).numpy()
    rec["v_scale"] = vs.numpy()
    for gran in ("per_warp", "per_thread"):
        q8, qs, k8, ks = quantizer_outputs(q, kc, gran)
        rec[f"q_codes_{gran}"], rec[f"q_scale_{gran}"] = q8, qs
        rec[f"k_codes_{gran}"], rec[f"k_scale_{gran}"] = k8, ks
        out32 = reference_sage_attention_2pp(q.float(), k.float(), v.float(), scale, causal, qk_quantization=gran)
        out16 = reference_sage_attention_2pp(q, k, v, scale, causal, qk_quantization=gran)
        rec[f"out32_{gran}"] = out32.numpy()
        rec[f"out16_{gran}"] = bits16(out16)
    np.savez_compressed(HERE / f"{name}.npz", **rec)
    print("wrote", name)


def randn(gen, shape, dtype):
    return torch.randn(shape, generator=gen, dtype=torch.float32).to(dtype)


def main() -> None:
    g = torch.Generator().manual_seed(20251)

    # ragged lengths, both head sizes, both dtypes (shapes of the reference's own GPU tests)
    q = randn(g, (1, 2, 193, 64), torch.float16)
    k = randn(g, (1, 2, 193, 64), torch.float16) + randn(g, (1, 1, 1, 64), torch.float16) * 0.5
    v = randn(g, (1, 2, 193, 64), torch.float16)
    piper_case("piper_d64_s193_f16", q, k, v, causal=False, center=False, sort=False)
    piper_case("piper_d64_s193_f16_causal", q, k, v, causal=True, center=False, sort=False)

    q = randn(g, (1, 2, 193, 128), torch.bfloat16)
    k = randn(g, (1, 2, 193, 128), torch.bfloat16)
    v = randn(g, (1, 2, 193, 128), torch.bfloat16) + randn(g, (1, 2, 1, 128), torch.bfloat16) * 2
    piper_case("piper_d128_s193_bf16_center", q, k, v, causal=False, center=True, sort=False)
    piper_case("piper_d128_s193_bf16_center_sort", q, k, v, causal=False, center=True, sort=True)
    piper_case("piper_d128_s193_bf16_causal", q, k, v, causal=True, center=False, sort=False)

    # rectangular, non-causal
    q = randn(g, (2, 1, 70, 128), torch.float16)
    k = randn(g, (2, 1, 300, 128), torch.float16)
    v = randn(g, (2, 1, 300, 128), torch.float16) * 3
    piper_case("piper_d128_rect_f16_center", q, k, v, causal=False, center=True, sort=False)

    # constant V with centering returns V exactly
    q = randn(g, (1, 2, 65, 64), torch.float16)
    k = randn(g, (1, 2, 65, 64), torch.float16)
    v = randn(g, (1, 2, 1, 64), torch.float16).expand(1, 2, 65, 64).contiguous()
    piper_case("piper_d64_constant_v", q, k, v, causal=False, center=True, sort=False)

    # one huge V entry keeps every scale finite
    q = randn(g, (1, 1, 80, 128), torch.float16)
    k = randn(g, (1, 1, 80, 128), torch.float16)
    v = randn(g, (1, 1, 80, 128), torch.float16)
    v[0, 0, 3, 5] = 40000.0
    piper_case("piper_d128_huge_v", q, k, v, causal=False, center=False, sort=False)

    # Sage2++: ragged, offset keys, rectangular
    q = randn(g, (1, 2, 193, 64), torch.float16)
    k = randn(g, (1, 2, 193, 64), torch.float16) + randn(g, (1, 1, 1, 64), torch.float16)
    v = randn(g, (1, 2, 193, 64), torch.float16)
    sage_case("sage_d64_s193_f16", q, k, v, causal=False)
    sage_case("sage_d64_s193_f16_causal", q, k, v, causal=True)
    q = randn(g, (1, 2, 33, 128), torch.bfloat16)
    k = randn(g, (1, 2, 17, 128), torch.bfloat16) + 100.0
    v = randn(g, (1, 2, 17, 128), torch.bfloat16)
    sage_case("sage_d128_sk17_offset_bf16", q, k, v, causal=False)
    q = randn(g, (2, 2, 96, 64), torch.float16)
    k = randn(g, (2, 2, 260, 64), torch.float16)
    v = randn(g, (2, 2, 260, 64), torch.float16)
    sage_case("sage_d64_rect_f16", q, k, v, causal=False)


if __name__ == "__main__":
    main()
