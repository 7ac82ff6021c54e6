"""GPU-side helpers for the parity tests: every call goes through the C ABI of
libpiper_b200.so (ctypes), with torch used only to hold device memory."""

from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from piper_kernels_b200 import _cabi, _ops

TORCH_DTYPE = {"float16": torch.float16, "bfloat16": torch.bfloat16}


def to_device(bits: np.ndarray, dtype: str) -> torch.Tensor:
    """uint16 bit patterns -> CUDA tensor of the given 16-bit float type."""
    t = torch.from_numpy(bits.astype(np.int16)).view(TORCH_DTYPE[dtype])
    return t.cuda()


class Call:
    """One prepared problem: owns output, workspace and the ctypes structs."""

    def __init__(self, algo, q, k, v, scale, causal, *, center=False, sort=False, gran="per_warp",
                 out_dtype=None, k_mean=None, v_mean=None):
        self.algo = algo
        self.q, self.k, self.v = q, k, v
        self.out_dtype = out_dtype or q.dtype
        self.out = torch.empty(q.shape, dtype=self.out_dtype, device=q.device)
        self.k_mean = None if k_mean is None else torch.from_numpy(np.ascontiguousarray(k_mean, dtype=np.float32)).cuda()
        self.v_mean = None if v_mean is None else torch.from_numpy(np.ascontiguousarray(v_mean, dtype=np.float32)).cuda()
        self.p = _ops.make_problem(q, k, v, scale, causal, center_value=center, sort_value_rows=sort,
                                   granularity=gran, out=self.out, k_mean=self.k_mean, v_mean=self.v_mean,
                                   out_dtype=self.out_dtype)
        nbytes = _ops.workspace_bytes(algo, self.p)
        self.ws = torch.zeros(nbytes + 256, dtype=torch.uint8, device=q.device)
        self.p.workspace, self.p.workspace_bytes = self.ws.data_ptr(), nbytes
        self.views = _cabi.PkViews()
        self.lib = _cabi.lib()

    def _fn(self, what):
        prefix = "pk_piper_" if self.algo == "piper" else "pk_sage2pp_"
        return getattr(self.lib, prefix + what)

    def prepare(self):
        _cabi.check(self._fn("prepare")(C.byref(self.p), C.byref(self.views)))
        return self

    def run(self):
        _cabi.check(self._fn("run")(C.byref(self.p)))
        return self

    def fwd(self):
        _cabi.check(self._fn("attention_fwd")(C.byref(self.p)))
        return self

    def status(self):
        st = (C.c_int32 * 16)()
        _cabi.check(self.lib.pk_device_status(C.byref(self.p), C.byref(st)))
        return list(st)

    def view(self, name, dtype, shape):
        """Workspace region named in pk_views as a torch tensor (no copy)."""
        ptr = getattr(self.views, name)
        assert ptr, name
        off = ptr - self.ws.data_ptr()
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        return self.ws[off:off + n].view(dtype).reshape(shape)

    def debug_tile(self, bh=0, q_tile=0):
        d = self.p.head_dim
        nbytes = 128 * 64 * 4 + 128 * 64 + 128 * d * 4
        dump = torch.zeros(nbytes, dtype=torch.uint8, device=self.q.device)
        _cabi.check(self.lib.pk_debug_first_tile(C.byref(self.p), int(self.algo != "piper"), bh, q_tile, dump.data_ptr()))
        torch.cuda.synchronize()
        raw = dump.cpu().numpy()
        s = raw[: 128 * 64 * 4].view(np.int32).reshape(128, 64)
        pc = raw[128 * 64 * 4: 128 * 64 * 5].reshape(128, 64)
        o = raw[128 * 64 * 5:].view(np.int32).reshape(128, d)
        return s, pc, o


def f32(t: torch.Tensor) -> np.ndarray:
    return t.float().cpu().numpy()
