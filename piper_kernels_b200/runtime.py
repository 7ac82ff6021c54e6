"""Prepared-call helper over the C ABI: quantise once, launch the fused kernel many times.

Mirrors the reference's split between ``_prepare_piper_attention`` and
``_launch_piper_attention`` (src/piper_kernels/attention/piper/triton.py:1054-1289), which
its benchmarks use to time "prepared execution" apart from the whole operator
(benchmarks/lib/attention_providers.py:201-216).  torch only owns the device buffers.
"""

from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _cabi, _ops


class AttentionCall:
    """One attention problem bound to its output and workspace buffers."""

    def __init__(self, algo: str, q, k, v, scale: float, causal: bool, *, center: bool = False,
                 sort: bool = False, gran: str | None = None, out_dtype=None, k_mean=None, v_mean=None):
        if algo not in ("piper", "sage2pp"):
            raise ValueError(f"unknown operator {algo}")
        self.algo = algo
        self.q, self.k, self.v = q, k, v
        self.out_dtype = out_dtype or q.dtype
        self.out = torch.empty(q.shape, dtype=self.out_dtype, device=q.device)
        as_dev = lambda m: None if m is None else torch.as_tensor(  # noqa: E731
            np.ascontiguousarray(m, dtype=np.float32)).to(q.device)
        self.k_mean, self.v_mean = as_dev(k_mean), as_dev(v_mean)
        gran = gran or _ops.DEFAULT_GRANULARITY[algo]
        self.p = _ops.make_problem(q, k, v, scale, causal, center_value=center, sort_value_rows=sort,
                                   granularity=gran, out=self.out, k_mean=self.k_mean, v_mean=self.v_mean,
                                   out_dtype=self.out_dtype)
        nbytes = _ops.workspace_bytes(algo, self.p)
        self.ws = torch.zeros(nbytes + 256, dtype=torch.uint8, device=q.device)
        self.p.workspace, self.p.workspace_bytes = self.ws.data_ptr(), nbytes
        self.views = _cabi.PkViews()
        self.lib = _cabi.lib()

    def _fn(self, what: str):
        return getattr(self.lib, ("pk_piper_" if self.algo == "piper" else "pk_sage2pp_") + what)

    def _sync_stream(self):
        self.p.stream = torch.cuda.current_stream(self.q.device).cuda_stream

    def prepare(self):
        """Quantisation prepass only; fills ``views``."""
        self._sync_stream()
        _cabi.check(self._fn("prepare")(C.byref(self.p), C.byref(self.views)))
        return self

    def prepare_kv(self):
        """Key/value side of the prepass only (means, key order, K and V codes, per-key vectors)."""
        self._sync_stream()
        _cabi.check(self._fn("prepare_kv")(C.byref(self.p), C.byref(self.views)))
        return self

    def requantize_q(self, new_q=None):
        """Query side of the prepass only, on this call's workspace.  ``new_q`` (same shape and
        dtype as the original query, any strides) replaces the query; K/V stay as prepared."""
        if new_q is not None:
            if new_q.shape != self.q.shape or new_q.dtype != self.q.dtype or new_q.device != self.q.device:
                raise ValueError("requantize_q needs a query of the prepared shape, dtype and device")
            self.q = new_q
            self.p.q = new_q.data_ptr()
            self.p.q_stride = (C.c_int64 * 3)(new_q.stride(0), new_q.stride(1), new_q.stride(2))
        self._sync_stream()
        _cabi.check(self._fn("prepare_q")(C.byref(self.p), C.byref(self.views)))
        return self

    def stalled_wait_drill(self, skip_key_tile: int = 1):
        """pk_debug_stalled_wait on the prepared workspace (see include/piper_b200.h)."""
        self._sync_stream()
        _cabi.check(self.lib.pk_debug_stalled_wait(C.byref(self.p), int(self.algo != "piper"), int(skip_key_tile)))
        return self

    def run(self):
        """Fused kernel only, on the prepared workspace."""
        self._sync_stream()
        _cabi.check(self._fn("run")(C.byref(self.p)))
        return self

    def fwd(self):
        """pk_*_attention_fwd: prepass + fused kernel in one call."""
        self._sync_stream()
        _cabi.check(self._fn("attention_fwd")(C.byref(self.p)))
        return self

    def status(self) -> list[int]:
        st = (C.c_int32 * 16)()
        _cabi.check(self.lib.pk_device_status(C.byref(self.p), C.byref(st)))
        return list(st)

    def view(self, name: str, dtype, shape):
        """Workspace region named in ``pk_views`` as a torch tensor (no copy); needs prepare()."""
        ptr = getattr(self.views, name)
        if not ptr:
            raise RuntimeError(f"view {name} is not available (call prepare() first)")
        off = ptr - self.ws.data_ptr()
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        return self.ws[off:off + n].view(dtype).reshape(shape)

    def debug_tile(self, bh: int = 0, q_tile: int = 0):
        """Raw first-key-tile intermediates of one query tile (int32 scores, 8-bit P codes, PV partial)."""
        d = self.p.head_dim
        nbytes = 128 * 64 * 4 + 128 * 64 + 128 * d * 4
        dump = torch.zeros(nbytes, dtype=torch.uint8, device=self.q.device)
        self._sync_stream()
        _cabi.check(self.lib.pk_debug_first_tile(C.byref(self.p), int(self.algo != "piper"), bh, q_tile, dump.data_ptr()))
        torch.cuda.synchronize(self.q.device)
        raw = dump.cpu().numpy()
        s = raw[: 128 * 64 * 4].view(np.int32).reshape(128, 64)
        pc = raw[128 * 64 * 4: 128 * 64 * 5].reshape(128, 64)
        o = raw[128 * 64 * 5:].view(np.int32).reshape(128, d)
        return s, pc, o


class GraphedAttention:
    """prepare + run of an :class:`AttentionCall` captured once in a CUDA graph and replayed.

    A small problem's eight launches take longer to issue than to run (c1: 54 us of kernels in a
    127 us step); the library allocates nothing and never synchronises, so the whole call can be
    captured.  The call's q/k/v tensors are the graph's inputs (copy new data into them in place)
    and ``call.out`` its output.  The first launches on a device set function attributes and map
    the pinned fault word, so the call runs once eagerly before the capture."""

    def __init__(self, call: AttentionCall):
        self.call = call
        dev = call.q.device
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            call.fwd()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            call.fwd()

    def replay(self):
        self.graph.replay()
        return self.call.out
