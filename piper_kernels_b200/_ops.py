"""torch.library operators over the C ABI.

Schemas mirror the reference project's operators
(``piper_kernels::piper_attention`` — src/piper_kernels/attention/piper/triton.py:1319-1348,
``piper_kernels::sage_attention_2pp`` — src/piper_kernels/attention/sage2pp/triton.py:434-443,682-690)
under the ``piper_b200`` namespace, with the same fake (meta) kernel: a fresh contiguous
tensor shaped like the query.  torch is used only for device memory, streams and the
operator registry; all arithmetic happens inside ``libpiper_b200.so``.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _cabi

_DTYPE = {torch.float16: _cabi.PK_F16, torch.bfloat16: _cabi.PK_BF16, torch.float32: _cabi.PK_F32}
_GRAN = {"per_warp": _cabi.PK_QK_PER_BLOCK, "per_block": _cabi.PK_QK_PER_BLOCK, "per_thread": _cabi.PK_QK_PER_THREAD}

# Q/K scale granularity used by the public functions (the reference's portable default is
# "per_thread" for both operators; its optimized Piper backend uses per-block scales).
DEFAULT_GRANULARITY = {"piper": "per_warp", "sage2pp": "per_thread"}


def make_problem(query, key, value, scale, is_causal, *, center_value=False, sort_value_rows=False,
                 granularity="per_warp", out=None, workspace=None, k_mean=None, v_mean=None,
                 out_dtype=None) -> _cabi.PkProblem:
    """Fill a ``pk_problem`` from torch tensors (no copies; pointers are borrowed)."""
    p = _cabi.PkProblem()
    p.batch, p.heads, p.q_len, p.head_dim = query.shape
    p.kv_len = key.shape[2]
    p.in_dtype = _DTYPE[query.dtype]
    p.out_dtype = _DTYPE[out_dtype if out_dtype is not None else query.dtype]
    p.is_causal = int(bool(is_causal))
    p.center_value = int(bool(center_value))
    p.sort_value_rows = int(bool(sort_value_rows))
    p.qk_granularity = _GRAN[granularity]
    p.scale = float(scale)
    for name, t in (("q", query), ("k", key), ("v", value)):
        setattr(p, name, t.data_ptr())
        setattr(p, name + "_stride", (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2)))
    p.out = out.data_ptr() if out is not None else None
    p.k_mean_override = k_mean.data_ptr() if k_mean is not None else None
    p.v_mean_override = v_mean.data_ptr() if v_mean is not None else None
    if workspace is not None:
        p.workspace = workspace.data_ptr()
        p.workspace_bytes = workspace.numel() * workspace.element_size()
    dev = query.device
    p.device = dev.index if dev.index is not None else torch.cuda.current_device()
    p.stream = torch.cuda.current_stream(dev).cuda_stream
    return p


def workspace_bytes(algo: str, problem: _cabi.PkProblem) -> int:
    n = C.c_uint64(0)
    fn = _cabi.lib().pk_piper_workspace_bytes if algo == "piper" else _cabi.lib().pk_sage2pp_workspace_bytes
    _cabi.check(fn(C.byref(problem), C.byref(n)))
    return int(n.value)


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if t.device.type != "cuda":
        raise RuntimeError(
            f"piper_b200::{name} runs only on CUDA tensors (B200, sm_100a); there is no CPU path")


def poll_device_fault(device_index: int) -> None:
    """Raise if a fused kernel launched earlier on this device gave up a bounded wait (its output
    rows were filled with NaN).  Reads one pinned host word: no synchronisation, no device work."""
    code = C.c_int32(0)
    _cabi.check(_cabi.lib().pk_poll_device_fault(int(device_index), C.byref(code)))


def _run(algo: str, query, key, value, scale, is_causal, center_value, sort_value_rows, granularity):
    _require_cuda(query, algo)
    out = torch.empty(query.shape, dtype=query.dtype, device=query.device)
    with torch.cuda.device(query.device):
        dev_index = query.device.index if query.device.index is not None else torch.cuda.current_device()
        poll_device_fault(dev_index)
        p = make_problem(query, key, value, scale, is_causal, center_value=center_value,
                         sort_value_rows=sort_value_rows, granularity=granularity, out=out)
        ws = torch.empty(workspace_bytes(algo, p), dtype=torch.uint8, device=query.device)
        p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        fn = _cabi.lib().pk_piper_attention_fwd if algo == "piper" else _cabi.lib().pk_sage2pp_attention_fwd
        _cabi.check(fn(C.byref(p)))
        # The kernels run asynchronously on the current stream.  The scratch was allocated on that
        # stream, so the caching allocator only hands it to work queued behind them: no
        # record_stream (and its events) needed.
    return out


@torch.library.custom_op("piper_b200::piper_attention", mutates_args=())
def piper_attention_op(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, scale: float,
                       is_causal: bool, center_value: bool) -> torch.Tensor:
    from .attention.piper import should_sort_value_rows  # policy lives beside the public function

    sort = should_sort_value_rows(center_value=center_value, is_causal=is_causal,
                                  head_dim=query.shape[-1], key_length=key.shape[2])
    return _run("piper", query, key, value, scale, is_causal, center_value, sort,
                DEFAULT_GRANULARITY["piper"])


@piper_attention_op.register_fake
def _(query, key, value, scale, is_causal, center_value):
    return torch.empty_like(query, memory_format=torch.contiguous_format)


@torch.library.custom_op("piper_b200::sage_attention_2pp", mutates_args=())
def sage_attention_2pp_op(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, scale: float,
                          is_causal: bool) -> torch.Tensor:
    return _run("sage2pp", query, key, value, scale, is_causal, False, False,
                DEFAULT_GRANULARITY["sage2pp"])


@sage_attention_2pp_op.register_fake
def _(query, key, value, scale, is_causal):
    return torch.empty_like(query, memory_format=torch.contiguous_format)
