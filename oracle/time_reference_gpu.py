"""Time the reference project's own GPU paths on this box (TEST INFRASTRUCTURE; needs oracle/_ref).

    python -m oracle.time_reference_gpu [--workload c5] [--heads 4]

Runs, on CUDA tensors, (a) the reference's portable PyTorch loop (device-agnostic), (b) its
Triton backend through the reference's own dispatch (``sage_attention_2pp`` takes the Triton
kernel on compute capability >= 8.9; ``piper_attention`` has no optimized backend on capability
10.0 and falls back to the portable loop) and (c) for Piper the Triton kernel with the affine
signed-INT8 fallback through the reference's private entry point.  Whatever Triton emits for sm_100 is JIT output of
the reference's kernels, not a shipped Blackwell kernel; a compile failure is reported as such.
Prints one JSON line per measurement.  Nothing here is part of the product or of its benchmark.
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def main() -> None:
    import torch

    from oracle.build_ref import import_reference
    from piper_kernels_b200.workloads import WORKLOADS, make_inputs

    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="c5")
    ap.add_argument("--heads", type=int, default=4)
    a = ap.parse_args()
    ref = import_reference()
    from piper_kernels.attention.piper.reference import reference_piper_attention
    from piper_kernels.attention.sage2pp.reference import reference_sage_attention_2pp

    w = WORKLOADS[a.workload]
    dev = torch.device("cuda:0")
    q, k, v = make_inputs(w, dev, range(0, a.heads))
    ops = 4.0 * a.heads * (w.q_len * (w.q_len + 1) / 2 if w.causal else w.q_len * w.kv_len) * w.head_dim

    def timed(name, fn, reps):
        try:
            t0 = time.perf_counter(); out = fn(); torch.cuda.synchronize(); first = time.perf_counter() - t0
            ts = []
            for _ in range(reps):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record(); fn(); e.record(); torch.cuda.synchronize(); ts.append(s.elapsed_time(e))
            ms = sorted(ts)[len(ts) // 2]
            print(json.dumps({"impl": name, "workload": w.name, "heads": a.heads, "ms": ms, "tops": ops / ms / 1e9,
                              "first_call_s": first, "gpu": torch.cuda.get_device_name(0)}), flush=True)
            return out
        except Exception as exc:  # a JIT failure is a result, not an error of this script
            print(json.dumps({"impl": name, "workload": w.name, "error": f"{type(exc).__name__}: {str(exc)[:300]}"}), flush=True)
            return None

    scale = w.head_dim ** -0.5
    if w.op == "piper":
        center = (not w.causal and w.head_dim == 128 and min(w.q_len, w.kv_len) >= 1024) if w.center is None else w.center
        sort = center and not w.causal and w.head_dim == 128 and w.kv_len >= 16384
        timed("reference portable loop on CUDA tensors (reference_piper_attention)",
              lambda: reference_piper_attention(q.float(), k.float(), v.float(), scale, w.causal, center_value=center,
                                                qk_quantization="per_warp", sort_value_rows=sort), 3)
        timed("reference public piper_attention on this GPU (its own dispatch)",
              lambda: ref.piper_attention(q, k, v, is_causal=w.causal), 3)
        # The reference's Triton Piper kernel with the affine signed-INT8 PV fallback: plain tl.dot, no
        # compiler hook, reachable on any capability through its private entry (piper/triton.py:1292-1316).
        from piper_kernels.attention.piper.triton import _run_piper_attention
        timed("reference Triton JIT Piper kernel, affine INT8 PV fallback (_run_piper_attention, native_uint8=False)",
              lambda: _run_piper_attention(q, k, v, scale, w.causal, center, native_uint8=False, sort_value_rows=False,
                                           use_tensor_descriptors=False), 10)
    else:
        timed("reference portable loop on CUDA tensors (reference_sage_attention_2pp)",
              lambda: reference_sage_attention_2pp(q.float(), k.float(), v.float(), scale, w.causal, qk_quantization="per_thread"), 3)
        timed("reference public sage_attention_2pp on this GPU (Triton JIT via its own dispatch)",
              lambda: ref.sage_attention_2pp(q, k, v, is_causal=w.causal), 10)


if __name__ == "__main__":
    main()
