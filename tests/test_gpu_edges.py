"""GPU edge cases: tiny and ragged lengths, exact tile multiples, many small heads, large
magnitudes, C-ABI error codes on a device, and bounded-wait status reporting."""

import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import piper_kernels_b200 as pk
from _util import cosine

pytestmark = pytest.mark.gpu


def _np(t):
    return t.float().cpu().numpy()


def _rand(shape, dtype, seed, scale=1.0, shift=0.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale + shift).to(dtype).cuda()


@pytest.mark.parametrize("sq,sk", [(1, 1), (1, 17), (17, 1), (63, 64), (64, 65), (65, 63), (128, 128), (129, 257), (257, 129)])
@pytest.mark.parametrize("d", [64, 128])
def test_ragged_lengths_piper_and_sage(sq, sk, d):
    q = _rand((1, 2, sq, d), torch.float16, 100 + sq)
    k = _rand((1, 2, sk, d), torch.float16, 200 + sk, shift=0.25)
    v = _rand((1, 2, sk, d), torch.float16, 300 + sk)
    for center in (False, True):
        out = _np(pk.piper_attention(q, k, v, center_value=center))
        want = oracle.piper_attention_oracle(_np(q), _np(k), _np(v), d ** -0.5, False, center_value=center,
                                             qk_quantization="per_warp")
        assert np.isfinite(out).all()
        assert np.all(np.abs(out - want) <= 2e-3 + np.abs(want) * 2.0 ** -10)
    out = _np(pk.sage_attention_2pp(q, k, v))
    want = oracle.sage_attention_2pp_oracle(_np(q), _np(k), _np(v), d ** -0.5, False, qk_quantization="per_thread")
    assert np.all(np.abs(out - want) <= 2e-3 + np.abs(want) * 2.0 ** -10)


@pytest.mark.parametrize("s", [1, 64, 100, 257])
def test_causal_lengths(s):
    q = _rand((2, 1, s, 128), torch.bfloat16, 400 + s)
    k = _rand((2, 1, s, 128), torch.bfloat16, 500 + s)
    v = _rand((2, 1, s, 128), torch.bfloat16, 600 + s)
    out = _np(pk.piper_attention(q, k, v, is_causal=True))
    want = oracle.piper_attention_oracle(_np(q), _np(k), _np(v), 128 ** -0.5, True, center_value=False,
                                         qk_quantization="per_warp")
    assert np.all(np.abs(out - want) <= 2e-3 + np.abs(want) * 2.0 ** -7)
    out = _np(pk.sage_attention_2pp(q, k, v, is_causal=True))
    want = oracle.sage_attention_2pp_oracle(_np(q), _np(k), _np(v), 128 ** -0.5, True, qk_quantization="per_thread")
    assert np.all(np.abs(out - want) <= 2e-3 + np.abs(want) * 2.0 ** -7)


def test_many_small_heads_and_custom_scale():
    q = _rand((8, 16, 40, 64), torch.float16, 7)
    k = _rand((8, 16, 72, 64), torch.float16, 8)
    v = _rand((8, 16, 72, 64), torch.float16, 9)
    out = _np(pk.piper_attention(q, k, v, scale=0.2, center_value=True))
    want = oracle.piper_attention_oracle(_np(q), _np(k), _np(v), 0.2, False, center_value=True, qk_quantization="per_warp")
    # With 72 keys and a sharp softmax a single probability code that rounds the other way
    # (the CUDA path works in base 2, the oracle in base e: ~1e-3 of the codes differ by one
    # step) moves one output row by up to ~1/255 of a value; the bulk stays at ~3e-5.
    diff = np.abs(out - want)
    assert diff.mean() <= 1e-4
    assert (diff > 2e-3 + np.abs(want) * 2.0 ** -10).mean() < 1e-4
    assert diff.max() <= 6e-3
    assert cosine(out, want) >= 0.9999


def test_large_magnitudes_and_zero_rows():
    q = _rand((1, 2, 150, 128), torch.bfloat16, 21, scale=8.0)
    k = _rand((1, 2, 190, 128), torch.bfloat16, 22, scale=8.0, shift=30.0)
    v = _rand((1, 2, 190, 128), torch.bfloat16, 23, scale=50.0)
    v[:, :, 5] = 0  # an all-zero value row (scale = epsilon)
    q[:, :, 3] = 0  # an all-zero query row (uniform attention)
    out = _np(pk.piper_attention(q, k, v, center_value=False))
    want = oracle.piper_attention_oracle(_np(q), _np(k), _np(v), 128 ** -0.5, False, center_value=False,
                                         qk_quantization="per_warp")
    assert np.isfinite(out).all()
    mag = float(np.abs(want).max())
    assert np.all(np.abs(out - want) <= 2e-3 * mag + np.abs(want) * 2.0 ** -7)


def test_abi_rejects_bad_arguments_on_device():
    from piper_kernels_b200 import _cabi, _ops

    q = _rand((1, 1, 64, 64), torch.float16, 1)
    out = torch.empty_like(q)
    ws = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    p = _ops.make_problem(q, q, q, 0.125, False, out=out, workspace=ws)
    lib = _cabi.lib()
    assert lib.pk_piper_attention_fwd(C.byref(p)) == _cabi.PK_OK
    p.workspace_bytes = 128
    assert lib.pk_piper_attention_fwd(C.byref(p)) == _cabi.PK_ERR_WORKSPACE
    p.workspace_bytes = ws.numel()
    p.workspace = ws.data_ptr() + 8
    assert lib.pk_piper_attention_fwd(C.byref(p)) == _cabi.PK_ERR_WORKSPACE
    p.workspace = ws.data_ptr()
    p.out = out.data_ptr() + 2
    assert lib.pk_piper_attention_fwd(C.byref(p)) == _cabi.PK_ERR_BAD_ARG
    torch.cuda.synchronize()


def test_status_words_are_clean_after_runs():
    from piper_kernels_b200.runtime import AttentionCall

    q = _rand((1, 3, 500, 128), torch.float16, 31)
    call = AttentionCall("piper", q, q, q, 128 ** -0.5, True).fwd()
    assert call.status() == [0] * 16
    call = AttentionCall("sage2pp", q, q, q, 128 ** -0.5, False).fwd()
    assert call.status() == [0] * 16
