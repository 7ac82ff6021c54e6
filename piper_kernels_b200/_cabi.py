"""ctypes binding of ``libpiper_b200.so`` (the C ABI declared in ``include/piper_b200.h``).

There is no fallback: if the shared library is missing or a call fails, an exception is
raised.  Build the library with ``python -m piper_kernels_b200.csrc.build``.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libpiper_b200.so"

PK_OK = 0
PK_ERR_BAD_ARG, PK_ERR_UNSUPPORTED_ARCH, PK_ERR_WORKSPACE, PK_ERR_CUDA, PK_ERR_DEVICE_STATUS = 1, 2, 3, 4, 5
PK_F16, PK_BF16, PK_F32 = 0, 1, 2
PK_QK_PER_BLOCK, PK_QK_PER_THREAD = 0, 1

EXPORTS = (
    "pk_version", "pk_last_error",
    "pk_piper_workspace_bytes", "pk_piper_prepare", "pk_piper_run", "pk_piper_attention_fwd",
    "pk_sage2pp_workspace_bytes", "pk_sage2pp_prepare", "pk_sage2pp_run", "pk_sage2pp_attention_fwd",
    "pk_device_status", "pk_debug_first_tile", "pk_kv_means_static", "pk_debug_timeline",
    "pk_piper_prepare_kv", "pk_piper_prepare_q", "pk_sage2pp_prepare_kv", "pk_sage2pp_prepare_q",
    "pk_poll_device_fault", "pk_debug_stalled_wait",
)


class PkProblem(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("heads", C.c_int32), ("q_len", C.c_int32), ("kv_len", C.c_int32),
        ("head_dim", C.c_int32), ("in_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("is_causal", C.c_int32), ("center_value", C.c_int32), ("sort_value_rows", C.c_int32),
        ("qk_granularity", C.c_int32), ("scale", C.c_float),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
        ("out", C.c_void_p),
        ("k_mean_override", C.c_void_p), ("v_mean_override", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_uint64),
        ("device", C.c_int32), ("stream", C.c_void_p),
    ]


class PkViews(C.Structure):
    _fields_ = [
        ("q_codes", C.c_void_p), ("k_codes", C.c_void_p), ("v_codes_t", C.c_void_p),
        ("q_group_scale", C.c_void_p), ("k_group_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("k_mean", C.c_void_p), ("v_mean", C.c_void_p), ("order", C.c_void_p),
        ("q_row_mul", C.c_void_p), ("k_col_mul", C.c_void_p), ("k_col_add", C.c_void_p),
        ("k_col_inv", C.c_void_p), ("status", C.c_void_p),
        ("sq_pad", C.c_int32), ("sk_pad", C.c_int32),
    ]


class PiperB200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libpiper_b200 error {code}: {message}")
        self.code = code


_lib = None


def lib() -> C.CDLL:
    """Load the shared library once; raise if it is absent (no fallback path exists)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m piper_kernels_b200.csrc.build` "
                "(needs nvcc with sm_100a support); piper_kernels_b200 has no other backend")
        handle = C.CDLL(str(LIB_PATH))
        P, V = C.POINTER(PkProblem), C.POINTER(PkViews)
        handle.pk_version.restype = C.c_int
        handle.pk_last_error.restype = C.c_char_p
        for name in ("pk_piper_workspace_bytes", "pk_sage2pp_workspace_bytes"):
            getattr(handle, name).argtypes = [P, C.POINTER(C.c_uint64)]
        for name in ("pk_piper_prepare", "pk_sage2pp_prepare", "pk_piper_prepare_kv", "pk_piper_prepare_q",
                     "pk_sage2pp_prepare_kv", "pk_sage2pp_prepare_q"):
            getattr(handle, name).argtypes = [P, V]
        for name in ("pk_piper_run", "pk_piper_attention_fwd", "pk_sage2pp_run", "pk_sage2pp_attention_fwd"):
            getattr(handle, name).argtypes = [P]
        handle.pk_device_status.argtypes = [P, C.POINTER(C.c_int32 * 16)]
        handle.pk_debug_first_tile.argtypes = [P, C.c_int, C.c_int, C.c_int, C.c_void_p]
        handle.pk_debug_timeline.argtypes = [P, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]
        handle.pk_kv_means_static.argtypes = [P, C.c_void_p, C.c_void_p]
        handle.pk_poll_device_fault.argtypes = [C.c_int32, C.POINTER(C.c_int32)]
        handle.pk_debug_stalled_wait.argtypes = [P, C.c_int, C.c_int]
        for name in EXPORTS[2:]:
            getattr(handle, name).restype = C.c_int
        _lib = handle
    return _lib


def check(code: int) -> None:
    if code != PK_OK:
        raise PiperB200Error(code, lib().pk_last_error().decode("utf-8", "replace"))
