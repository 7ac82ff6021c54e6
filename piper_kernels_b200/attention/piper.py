"""Public ``piper_attention`` — drop-in for ``piper_kernels.attention.piper_attention``
(src/piper_kernels/attention/piper/dispatch.py:114-165 of the reference project).

Signature, validation and error behaviour are the reference's.  The backend is the
hand-written sm_100a library; there is no portable fallback, so non-CUDA tensors are
rejected after validation.
"""

from __future__ import annotations

import torch

from ._validation import validate_inputs


def default_center_value(query: torch.Tensor, key: torch.Tensor, is_causal: bool) -> bool:
    """Centering policy when ``center_value`` is None.

    The reference enables centering by default only in its measured region: non-causal,
    head_dim 128, both lengths >= 1024, on the consumer-Blackwell target it was tuned on
    (piper/dispatch.py:96-111).  This build applies the same shape rule on B200.
    """
    return (
        query.device.type == "cuda"
        and not is_causal
        and query.shape[-1] == 128
        and query.shape[2] >= 1024
        and key.shape[2] >= 1024
    )


def should_sort_value_rows(*, center_value: bool, is_causal: bool, head_dim: int, key_length: int) -> bool:
    """Exact centred-row-range key ordering only where its cost is amortised: centred,
    non-causal, head_dim 128, >= 16384 keys (piper/triton.py:1034-1051)."""
    return bool(center_value) and not is_causal and head_dim == 128 and key_length >= 16384


def piper_attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    *,
    scale: float | None = None,
    is_causal: bool = False,
    center_value: bool | None = None,
) -> torch.Tensor:
    """Piper's key-scaled UINT8-P / INT8-V forward attention on B200.

    ``[batch, heads, sequence, head_dim]`` FP16/BF16 tensors with contiguous head dimension;
    rectangular shapes when non-causal; ``scale`` defaults to ``head_dim**-0.5``;
    ``center_value=True`` subtracts the per-feature sequence mean of V before quantization and
    restores it in the epilogue; ``None`` selects it in the long non-causal D=128 region.
    Inference only.
    """
    converted_scale = validate_inputs("Piper Attention", query, key, value, scale, is_causal)
    centering = default_center_value(query, key, is_causal) if center_value is None else bool(center_value)
    from .. import _ops

    return _ops.piper_attention_op(query, key, value, converted_scale, bool(is_causal), centering)
