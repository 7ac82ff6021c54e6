"""GPU-side helpers for the parity tests: every call goes through the C ABI of
libpiper_b200.so (ctypes), with torch used only to hold device memory."""

from __future__ import annotations

import numpy as np
import torch

from piper_kernels_b200.runtime import AttentionCall

TORCH_DTYPE = {"float16": torch.float16, "bfloat16": torch.bfloat16}


def to_device(bits: np.ndarray, dtype: str) -> torch.Tensor:
    """uint16 bit patterns -> CUDA tensor of the given 16-bit float type."""
    t = torch.from_numpy(bits.astype(np.int16)).view(TORCH_DTYPE[dtype])
    return t.cuda()


class Call(AttentionCall):
    def fwd(self):
        """A prepare call to obtain the views of the workspace, then pk_*_attention_fwd
        (which repeats the prepass and runs the fused kernel, so the status words are its)."""
        self.prepare()
        return super().fwd()


def f32(t: torch.Tensor) -> np.ndarray:
    return t.float().cpu().numpy()
