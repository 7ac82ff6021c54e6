"""CPU oracle for the fused quantized attention path (TEST INFRASTRUCTURE ONLY).

This package restates, in numpy, the portable algorithm of the reference
project's ``piper_attention`` and ``sage_attention_2pp`` operators.  It exists
to check the CUDA implementation; it is never imported by the product package.
Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import it.

Parity status: PINNED.  ``tests/golden/*.npz`` hold inputs and outputs produced
by importing the reference's own Python modules (generator script:
``tests/golden/make_golden.py``); ``tests/test_oracle_golden.py`` checks every
function here against them (integer codes and scales bit-exactly when the
reference's means are injected; outputs within 2e-5).
"""

from .quantizers import (  # noqa: F401
    KEY_BLOCK,
    QUERY_BLOCK,
    e4m3_decode,
    e4m3_encode,
    quantize_key_per_thread,
    quantize_per_group,
    quantize_query_per_thread,
    quantize_value_per_channel_e4m3,
    quantize_value_per_key,
    round_to_dtype,
    sequence_mean,
)
from .piper import centered_value_order, piper_attention_oracle, piper_prepare_oracle, piper_tile_loop  # noqa: F401
from .sage2pp import sage_attention_2pp_oracle, sage_prepare_oracle  # noqa: F401
