"""piper_kernels_b200 — B200-native (sm_100a) fused quantized attention.

Drop-in for the attention operators of Boffee/piper-kernels:
``piper_attention`` and ``sage_attention_2pp`` keep the reference's signatures and
validation and dispatch through ``torch.library`` operators into ``libpiper_b200.so``.
"""

from .attention import piper_attention, sage_attention_2pp

__all__ = ["piper_attention", "sage_attention_2pp"]
__version__ = "0.1.0"
