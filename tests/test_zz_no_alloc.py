"""The allocation-free entry point pk_kv_means_static.

Some hosts cannot allocate device memory at the point where they call this library (a memory
pool frozen for the life of a serving process, a plug-in runtime that hands out fixed buffers).
For them the K/V sequence means can be computed with the scratch held in a static array inside
the library.  This test calls that entry point through the C ABI twice in a row and checks both
results, bit for bit, against the workspace-based prepare call.  It lives in a file of its own
that pytest collects last."""

import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(shape_k, dtype, seed):
    gen = torch.Generator().manual_seed(seed)
    b, h, sk, d = shape_k
    q = torch.randn(b, h, 40, d, generator=gen).to(dtype).cuda()
    k = (torch.randn(shape_k, generator=gen) + 0.3).to(dtype).cuda()
    v = (torch.randn(shape_k, generator=gen) * 2 - 1.0).to(dtype).cuda()
    return q, k, v


@pytest.mark.parametrize("shape_k,dtype", [((2, 3, 1500, 128), torch.bfloat16), ((1, 4, 777, 64), torch.float16)])
def test_static_scratch_means_match_workspace_means_twice(shape_k, dtype):
    from piper_kernels_b200 import _cabi
    from piper_kernels_b200.runtime import AttentionCall

    lib = _cabi.lib()
    b, h, sk, d = shape_k
    for round_, seed in enumerate((11, 12)):  # two calls in a row share the static array
        q, k, v = _inputs(shape_k, dtype, seed)
        call = AttentionCall("piper", q, k, v, d ** -0.5, False, center=True).prepare()
        torch.cuda.synchronize()
        want_k = call.view("k_mean", torch.float32, (b * h, d)).cpu().numpy()
        want_v = call.view("v_mean", torch.float32, (b * h, d)).cpu().numpy()
        got_k = torch.full((b * h, d), float("nan"), dtype=torch.float32, device="cuda")
        got_v = torch.full((b * h, d), float("nan"), dtype=torch.float32, device="cuda")
        _cabi.check(lib.pk_kv_means_static(C.byref(call.p), got_k.data_ptr(), got_v.data_ptr()))
        torch.cuda.synchronize()
        assert np.array_equal(got_k.cpu().numpy(), want_k), f"K mean differs on call {round_}"
        assert np.array_equal(got_v.cpu().numpy(), want_v), f"V mean differs on call {round_}"


def test_static_scratch_rejects_oversized_problems():
    from piper_kernels_b200 import _cabi, _ops

    q = torch.empty(1, 1, 8, 128, dtype=torch.float16, device="cuda")
    p = _ops.make_problem(q, q, q, 0.1, False)
    p.batch, p.heads, p.kv_len = 64, 64, 4096  # 64*64*8*128 partial sums per tensor: over the limit
    out = torch.empty(8, dtype=torch.float32, device="cuda")
    rc = _cabi.lib().pk_kv_means_static(C.byref(p), out.data_ptr(), out.data_ptr())
    assert rc == _cabi.PK_ERR_BAD_ARG
    assert b"exceeds the built-in scratch" in _cabi.lib().pk_last_error()
