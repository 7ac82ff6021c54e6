"""Fused quantized attention operators (same names as ``piper_kernels.attention``)."""

from .piper import piper_attention
from .sage2pp import sage_attention_2pp

__all__ = ["piper_attention", "sage_attention_2pp"]
