"""Public ``sage_attention_2pp`` — drop-in for ``piper_kernels.attention.sage_attention_2pp``
(src/piper_kernels/attention/sage2pp/dispatch.py:96-120 of the reference project)."""

from __future__ import annotations

import torch

from ._validation import validate_inputs


def sage_attention_2pp(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    *,
    scale: float | None = None,
    is_causal: bool = False,
) -> torch.Tensor:
    """SageAttention2++ 8+8 forward attention on B200: INT8 QK^T, E4M3 P and V, 64-key PV
    partials rounded to FP16 and accumulated in FP32.  Same layout rules as
    :func:`piper_attention`.  Inference only."""
    converted_scale = validate_inputs("SageAttention2++", query, key, value, scale, is_causal)
    from .. import _ops

    return _ops.sage_attention_2pp_op(query, key, value, converted_scale, bool(is_causal))
