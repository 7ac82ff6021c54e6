#!/usr/bin/env python
"""Per-role timeline of one CTA of the fused kernel (profiling aid, beside bench.py).

    python bench_timeline.py [--workload c2] [--bh 5] [--q-tile 7]

Runs the ordinary fused kernel through ``pk_debug_timeline`` and prints, per warp role, the
average cycles per key tile spent waiting and working, plus the steady-state tile period.
"""

from __future__ import annotations

import argparse
import ctypes as C

import numpy as np
import torch

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

from piper_kernels_b200 import _cabi  # noqa: E402
from piper_kernels_b200.attention.piper import default_center_value, should_sort_value_rows  # noqa: E402
from piper_kernels_b200.runtime import AttentionCall  # noqa: E402
from piper_kernels_b200.workloads import WORKLOADS, make_inputs  # noqa: E402

ROLES = 7


def capture(call: AttentionCall, bh: int, q_tile: int, max_tiles: int = 1024) -> np.ndarray:
    buf = torch.zeros(ROLES * max_tiles * 8, dtype=torch.int64, device=call.q.device)
    call._sync_stream()
    _cabi.check(call.lib.pk_debug_timeline(C.byref(call.p), int(call.algo != "piper"), bh, q_tile, buf.data_ptr(), max_tiles))
    torch.cuda.synchronize(call.q.device)
    return buf.cpu().numpy().reshape(ROLES, max_tiles, 8)


def summarize(tr: np.ndarray, n_tiles: int, nswg: int) -> str:
    """Average cycles per key tile, per role.  Stamp slots: softmax 0 start, 1 scores ready,
    4 scores in registers, 2 tile max known / score buffer released, 5 codes computed,
    6 probability buffer free, 7 probabilities stored, 3 published; dequant 0 start, 1 rescaled,
    2 first chunk loaded, 4 early chunks folded, 7 next statistics done, 5 next tile's product
    complete, 6 all chunks folded, 3 buffer released (when the fold starts from the top of the tile: 0 start,
    7 statistics done, 5 product complete, 1 rescaled, 2 first chunk loaded, 6, 3; slot 4 stays empty); issue warps 0 start, 1 operands
    ready, 2 issued; producer 0 start, 1 K stage free, 2 copies issued."""
    n = min(n_tiles, tr.shape[1])
    t0 = tr[tr > 0].min()
    tr = np.where(tr > 0, tr - t0, -1)[:, :n]
    lo, hi = min(8, n // 4), n - 2
    d = lambda x, a, b: float(np.mean(x[:, b] - x[:, a]))  # noqa: E731
    lines = [f"tiles {n}; total {int(tr.max())} cycles; steady-state period {(tr[nswg, hi, 3] - tr[nswg, lo, 3]) / (hi - lo):.0f} cycles per tile"]
    for w in range(nswg):
        x = tr[w, lo + ((w - lo) % nswg):hi:nswg]
        if x[:, 4].min() >= 0:  # single-pass softmax stamps
            lines.append(f"softmax{w}: wait scores {d(x, 0, 1):.0f} | load {d(x, 1, 4):.0f} | scale+max+release {d(x, 4, 2):.0f} | "
                         f"exp+codes {d(x, 2, 5):.0f} | wait P buffer {d(x, 5, 6):.0f} | store P {d(x, 6, 7):.0f} | publish {d(x, 7, 3):.0f} | "
                         f"per own tile {np.mean(np.diff(x[:, 0])):.0f}")
        else:
            lines.append(f"softmax{w}: wait {d(x, 0, 1):.0f} | pass 1 {d(x, 1, 2):.0f} | pass 2 + publish {d(x, 2, 3):.0f} | per own tile {np.mean(np.diff(x[:, 0])):.0f}")
    x = tr[nswg, lo:hi]
    top = x[:, 4].min() < 0  # the fold starts from the top of the tile: statistics and product wait come first
    if top:
        lines.append(f"dequant : statistics {d(x, 0, 7):.0f} | product wait {d(x, 7, 5):.0f} | rescale {d(x, 5, 1):.0f} | first chunk {d(x, 1, 2):.0f} | "
                     f"other chunks {d(x, 2, 6):.0f} | release {d(x, 6, 3):.0f} | per tile {np.mean(np.diff(x[:, 0])):.0f}")
    else:
        lines.append(f"dequant : rescale {d(x, 0, 1):.0f} | first chunk {d(x, 1, 2):.0f} | early chunks {d(x, 2, 4):.0f} | "
                     f"next tile's statistics {d(x, 4, 7):.0f} | next tile's product wait {d(x, 7, 5):.0f} | remaining chunks {d(x, 5, 6):.0f} | "
                     f"release {d(x, 6, 3):.0f} | per tile {np.mean(np.diff(x[:, 0])):.0f}")
    for r, name in ((nswg + 1, "S issue "), (nswg + 2, "PV issue")):
        x = tr[r, lo:hi]
        lines.append(f"{name}: wait {d(x, 0, 1):.0f} | issue {d(x, 1, 2):.0f} | per tile {np.mean(np.diff(x[:, 0])):.0f}")
    x = tr[nswg + 3, lo:hi]
    if x[:, 2].min() >= 0:
        lines.append(f"producer: wait K stage {d(x, 0, 1):.0f} | wait V stage + issue copies {d(x, 1, 2):.0f} | per tile {np.mean(np.diff(x[:, 0])):.0f}")
    own = np.arange(n) % nswg
    p_done = tr[own, np.arange(n), 3]
    lines.append(f"P published -> PV issued {np.mean(tr[nswg + 2, lo:hi, 2] - p_done[lo:hi]):.0f} | PV issued -> fold begins {np.mean(tr[nswg, lo:hi, 5 if top else 0] - tr[nswg + 2, lo:hi, 2]):.0f} | "
                 f"S issued -> softmax picks it up {np.mean(tr[own, np.arange(n), 1][lo:hi] - tr[nswg + 1, lo:hi, 2]):.0f}")
    return "\n".join(lines)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--bh", type=int, default=5)
    ap.add_argument("--q-tile", type=int, default=7)
    ap.add_argument("--save", default=None, help="write the raw stamps to this .npy file")
    a = ap.parse_args()
    w = WORKLOADS[a.workload]
    dev = torch.device("cuda:0")
    q, k, v = make_inputs(w, dev)
    scale = w.head_dim ** -0.5
    if w.op == "piper":
        center = default_center_value(q, k, w.causal) if w.center is None else bool(w.center)
        sort = should_sort_value_rows(center_value=center, is_causal=w.causal, head_dim=w.head_dim, key_length=w.kv_len)
        call = AttentionCall("piper", q, k, v, scale, w.causal, center=center, sort=sort)
    else:
        call = AttentionCall("sage2pp", q, k, v, scale, w.causal)
    call.prepare().run()
    torch.cuda.synchronize()
    tr = capture(call, a.bh, a.q_tile)
    n_tiles = (w.kv_len + 63) // 64
    if w.causal:
        n_tiles = min(n_tiles, 2 * a.q_tile + 2)
    print(summarize(tr, n_tiles, 2))
    if a.save:
        np.save(a.save, tr)


if __name__ == "__main__":
    main()
