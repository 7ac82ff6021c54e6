"""CPU tests of the host side: validation messages mirror the reference's, the C ABI library
loads and exports every declared symbol, and argument errors come back as codes (no GPU)."""

import ctypes as C
import re
from pathlib import Path

import pytest
import torch

import piper_kernels_b200 as pk
from piper_kernels_b200 import _cabi, _ops
from piper_kernels_b200.attention.piper import default_center_value, should_sort_value_rows

ROOT = Path(__file__).resolve().parents[1]


def _qkv(dtype=torch.float16, sq=8, sk=8, d=64, b=1, h=2):
    return (torch.randn(b, h, sq, d).to(dtype), torch.randn(b, h, sk, d).to(dtype), torch.randn(b, h, sk, d).to(dtype))


@pytest.mark.parametrize("fn,name", [(pk.piper_attention, "Piper Attention"), (pk.sage_attention_2pp, "SageAttention2++")])
def test_validation_messages(fn, name):
    q, k, v = _qkv()
    with pytest.raises(ValueError, match="float16 or bfloat16"):
        fn(q.float(), k.float(), v.float())
    with pytest.raises(ValueError, match="share a dtype"):
        fn(q, k.to(torch.bfloat16), v)
    with pytest.raises(ValueError, match="head dimensions 64 and 128"):
        fn(*_qkv(d=32))
    with pytest.raises(ValueError, match="key/value lengths"):
        fn(q, k, v[:, :, :4])
    with pytest.raises(ValueError, match="equal batch and head dimensions"):
        fn(q, k[:, :1], v[:, :1])
    with pytest.raises(ValueError, match="equal query and key lengths"):
        fn(*_qkv(sq=4, sk=8), is_causal=True)
    with pytest.raises(ValueError, match="does not accept empty"):
        fn(q[:, :, :0], k, v)
    with pytest.raises(ValueError, match="head dimension must be contiguous"):
        fn(q.transpose(2, 3).contiguous().transpose(2, 3), k, v)
    with pytest.raises(ValueError, match="finite and positive"):
        fn(q, k, v, scale=0.0)
    with pytest.raises(ValueError, match="shape"):
        fn(q[0], k[0], v[0])
    with pytest.raises(RuntimeError, match="inference-only"):
        fn(q.requires_grad_(), k, v)
    assert name in str(pytest.raises(ValueError, fn, q.detach().float(), k.float(), v.float()).value)


def test_no_cpu_fallback():
    q, k, v = _qkv()
    with pytest.raises(RuntimeError, match="no CPU path"):
        pk.piper_attention(q, k, v)
    with pytest.raises(RuntimeError, match="no CPU path"):
        pk.sage_attention_2pp(q, k, v)


def test_default_policies():
    q = torch.empty(1, 1, 1024, 128, device="meta")
    assert not default_center_value(torch.empty(1, 1, 1024, 128), torch.empty(1, 1, 1024, 128), False)  # CPU tensor
    assert should_sort_value_rows(center_value=True, is_causal=False, head_dim=128, key_length=16384)
    assert not should_sort_value_rows(center_value=True, is_causal=False, head_dim=128, key_length=16383)
    assert not should_sort_value_rows(center_value=False, is_causal=False, head_dim=128, key_length=32768)
    assert not should_sort_value_rows(center_value=True, is_causal=True, head_dim=128, key_length=32768)
    assert not should_sort_value_rows(center_value=True, is_causal=False, head_dim=64, key_length=32768)
    del q


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "piper_b200.h").read_text()
    declared = set(re.findall(r"PK_API\s+(?:const\s+char\*|int)\s+(pk_\w+)\(", header))
    assert declared == set(_cabi.EXPORTS)
    lib = _cabi.lib()
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.pk_version() == 1


def test_struct_layout_matches_header(tmp_path):
    """The ctypes mirror must agree with what a C compiler makes of include/piper_b200.h."""
    import shutil
    import subprocess

    if shutil.which("gcc") is None:
        pytest.skip("gcc not available")
    fields_p = [f[0] for f in _cabi.PkProblem._fields_]
    fields_v = [f[0] for f in _cabi.PkViews._fields_]
    src = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{ROOT}/include/piper_b200.h"', "int main(void){",
           'printf("%zu %zu\\n", sizeof(pk_problem), sizeof(pk_views));']
    src += [f'printf("%zu\\n", offsetof(pk_problem, {f}));' for f in fields_p]
    src += [f'printf("%zu\\n", offsetof(pk_views, {f}));' for f in fields_v]
    src += ["return 0;}"]
    (tmp_path / "layout.c").write_text("\n".join(src))
    subprocess.run(["gcc", "-o", str(tmp_path / "layout"), str(tmp_path / "layout.c")], check=True)
    out = subprocess.run([str(tmp_path / "layout")], check=True, capture_output=True, text=True).stdout.split()
    nums = [int(x) for x in out]
    assert nums[0] == C.sizeof(_cabi.PkProblem) and nums[1] == C.sizeof(_cabi.PkViews)
    want = [getattr(_cabi.PkProblem, f).offset for f in fields_p] + [getattr(_cabi.PkViews, f).offset for f in fields_v]
    assert nums[2:] == want


def _problem(**over):
    p = _cabi.PkProblem()
    p.batch, p.heads, p.q_len, p.kv_len, p.head_dim = 1, 2, 100, 200, 128
    p.in_dtype = p.out_dtype = _cabi.PK_BF16
    p.scale = 0.1
    p.q = p.k = p.v = 256
    for k_, v_ in over.items():
        setattr(p, k_, v_)
    return p


def test_abi_argument_errors_without_gpu():
    lib = _cabi.lib()
    n = C.c_uint64()
    assert lib.pk_piper_workspace_bytes(C.byref(_problem()), C.byref(n)) == _cabi.PK_OK
    assert n.value > 2 * (128 * 128 + 256 * 128 * 2)
    bad = [dict(head_dim=96), dict(q_len=0), dict(in_dtype=_cabi.PK_F32), dict(scale=float("nan")),
           dict(is_causal=1), dict(qk_granularity=7), dict(sort_value_rows=1), dict(q=None)]
    for over in bad:
        assert lib.pk_piper_workspace_bytes(C.byref(_problem(**over)), C.byref(n)) == _cabi.PK_ERR_BAD_ARG, over
        assert lib.pk_last_error()
    assert lib.pk_sage2pp_workspace_bytes(C.byref(_problem(head_dim=64)), C.byref(n)) == _cabi.PK_OK
    # run without a workspace is refused before anything touches a device
    p = _problem(out=256)
    assert lib.pk_piper_attention_fwd(C.byref(p)) == _cabi.PK_ERR_WORKSPACE
    p.workspace, p.workspace_bytes = 4096, 16
    assert lib.pk_piper_attention_fwd(C.byref(p)) == _cabi.PK_ERR_WORKSPACE
    assert b"too small" in lib.pk_last_error()


def test_abi_rejects_more_flat_heads_than_a_grid_dimension_holds():
    lib = _cabi.lib()
    n = C.c_uint64()
    assert lib.pk_piper_workspace_bytes(C.byref(_problem(batch=65535, heads=1, q_len=8, kv_len=8)), C.byref(n)) == _cabi.PK_OK
    assert lib.pk_piper_workspace_bytes(C.byref(_problem(batch=256, heads=256, q_len=8, kv_len=8)), C.byref(n)) == _cabi.PK_ERR_BAD_ARG
    assert b"65535" in lib.pk_last_error()


def test_fault_poll_reports_nothing_before_any_launch_and_maps_errors():
    lib = _cabi.lib()
    code = C.c_int32(7)
    assert lib.pk_poll_device_fault(0, C.byref(code)) == _cabi.PK_OK and code.value == 0
    assert lib.pk_poll_device_fault(-1, C.byref(code)) == _cabi.PK_ERR_BAD_ARG
    with pytest.raises(_cabi.PiperB200Error) as exc:
        _cabi.check(lib.pk_poll_device_fault(1000, C.byref(code)))
    assert exc.value.code == _cabi.PK_ERR_BAD_ARG


def test_workspace_grows_with_sorting_and_granularity():
    lib = _cabi.lib()
    a, b = C.c_uint64(), C.c_uint64()
    lib.pk_piper_workspace_bytes(C.byref(_problem(center_value=1)), C.byref(a))
    lib.pk_piper_workspace_bytes(C.byref(_problem(center_value=1, sort_value_rows=1)), C.byref(b))
    assert b.value > a.value


def test_fake_kernel_shapes():
    q = torch.empty(2, 3, 5, 64, dtype=torch.float16, device="meta").permute(1, 0, 2, 3)
    out = _ops.piper_attention_op(q, q, q, 0.125, False, False)
    assert out.shape == q.shape and out.is_contiguous() and out.dtype == q.dtype
    out = _ops.sage_attention_2pp_op(q, q, q, 0.125, False)
    assert out.shape == q.shape and out.is_contiguous()


def test_host_pipeline_chunk_plan_covers_every_head_and_ramps():
    from piper_kernels_b200.scheduler import plan_chunks

    for flat in range(1, 70):
        for max_chunk in (1, 2, 3, 4, 8, 16):
            plan = plan_chunks(flat, max_chunk)
            assert sum(plan) == flat
            assert all(1 <= n <= max_chunk for n in plan)
            assert plan[0] == 1 and plan[-1] == 1  # the exposed first upload / last download are one head
            # an upload never exceeds twice the chunk whose compute hides it
            assert all(b <= 2 * a for a, b in zip(plan, plan[1:]))
    assert plan_chunks(40, 8) == [1, 1, 2, 4, 8, 8, 8, 4, 2, 1, 1]


def test_chunk_size_follows_the_work_per_head():
    """About half a millisecond of fused-kernel time per chunk, at most eight heads and at most a
    quarter of the heads (so that the pipeline has something to overlap)."""
    from piper_kernels_b200.scheduler import suggest_heads_per_chunk
    from piper_kernels_b200.workloads import WORKLOADS

    got = {n: suggest_heads_per_chunk(w.ops(1), w.flat_heads) for n, w in WORKLOADS.items()}
    assert got == {"c1": 2, "c2": 8, "c3": 8, "c4": 1, "c5": 8}
    assert suggest_heads_per_chunk(WORKLOADS["c4"].ops(1), 5) == 1  # a strong-scaling shard of five heads
    assert suggest_heads_per_chunk(1e15, 64) == 1 and suggest_heads_per_chunk(1.0, 3) == 1


def test_magic_number_rounding_equals_rint_and_yields_the_code_byte():
    """The arithmetic the quantisers use for an INT8 code, restated in numpy: adding 1.5 * 2^23 to
    t in FP32 rounds it to an integer like rint (ties to even), and the low byte of the sum's bit
    pattern is that integer in two's complement.  The guard that sends elements near a
    half-integer to the exact division is wider than the distance between x * fl(1/s) and x / s."""
    import numpy as np

    rng = np.random.default_rng(7)
    t = np.concatenate([
        rng.uniform(-127.4, 127.4, 200000),
        np.arange(-127, 127) + 0.5,                       # exact ties
        np.arange(-127, 127) + 0.5 + 2.0 ** -17,          # just above a tie
        np.arange(-127, 127) + 0.5 - 2.0 ** -17,
        [0.0, -0.0, 127.0, -127.0, 126.5, -126.5],
    ]).astype(np.float32)
    magic = np.float32(12582912.0)
    tm = (t + magic).astype(np.float32)
    q = (tm - magic).astype(np.float32)
    assert np.array_equal(q, np.rint(t))
    code = (tm.view(np.uint32) & 0xFF).astype(np.uint8).view(np.int8)
    assert np.array_equal(code.astype(np.float32), np.rint(t))
    # |x * fl(1/s) - x / s| for |x / s| <= 127: far inside the 1e-4 guard around half-integers
    x = rng.standard_normal(200000).astype(np.float32) * 3
    s = (np.abs(x).max() / np.float32(127.0) + np.float32(1e-7)).astype(np.float32)
    r = (np.float32(1.0) / s).astype(np.float32)
    gap = np.abs((x * r).astype(np.float32).astype(np.float64) - x.astype(np.float64) / np.float64(s))
    assert gap.max() < 2.4e-5
    exact = np.rint((x / s).astype(np.float32))
    fast = np.rint((x * r).astype(np.float32))
    near_half = np.abs(np.abs((x * r).astype(np.float32) - fast) - 0.5) < 1e-4
    assert np.array_equal(fast[~near_half], exact[~near_half])
