"""GPU parity on the five benchmark shapes (c1-c5) and on the host-pipelined entry point.

The gate is the one stated for the path: un-rounded FP32 output of the CUDA kernels against the
FP32 oracle, max-abs <= 2e-3 and cosine >= 0.9999, with no allowance for the output type.  The
16-bit output of the public operator is checked separately: it is the FP32 output rounded once
to the output type.  Whole tensors or whole heads
are compared where the oracle finishes in seconds (c1, a c2 head, a c5 head); for c3 and c4 one
head runs on the GPU at full length and several row blocks spread over the sequence are
compared (rows are independent given the head's K/V).  Size-independent properties
(constant-V exactness, bitwise determinism) run at full c4 length."""

import numpy as np
import pytest
import torch

import oracle
import piper_kernels_b200 as pk
from _util import cosine
from piper_kernels_b200.attention.piper import default_center_value, should_sort_value_rows
from piper_kernels_b200.runtime import AttentionCall
from piper_kernels_b200.workloads import WORKLOADS, make_inputs

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-3  # the path's stated tolerance, on FP32 outputs
MIN_COS = 0.9999
SHORT = {torch.float16: "f16", torch.bfloat16: "bf16"}


def _np(t):
    return t.float().cpu().numpy()


def _ulp16(x, dtype):
    """Spacing of the 16-bit format at |x| (float16: 10 fraction bits, bfloat16: 7)."""
    frac = 10 if dtype == torch.float16 else 7
    emin = -14 if dtype == torch.float16 else -126
    e = np.floor(np.log2(np.maximum(np.abs(x), 2.0 ** emin)))
    return 2.0 ** (e - frac)


def _gate32(out32, want32):
    assert np.isfinite(out32).all()
    err = float(np.abs(out32 - want32).max())
    assert err <= MAX_ABS, f"max-abs {err:.3e} exceeds {MAX_ABS}"
    assert cosine(out32, want32) >= MIN_COS
    return err


def _gate16(out16, out32, want32, dtype):
    """The 16-bit output of the public operator is the FP32 output rounded once (so the only
    difference between the two outputs is the output type's own rounding), and it lies within
    the gate plus one unit in the last place of the rounded oracle."""
    assert np.array_equal(out16, oracle.round_to_dtype(out32, SHORT[dtype]))
    want16 = oracle.round_to_dtype(want32, SHORT[dtype])
    assert np.all(np.abs(out16 - want16) <= MAX_ABS + _ulp16(want16, dtype))


def _policy(w, q, k):
    center = default_center_value(q, k, w.causal) if w.center is None else bool(w.center)
    sort = w.op == "piper" and should_sort_value_rows(center_value=center, is_causal=w.causal, head_dim=w.head_dim,
                                                      key_length=w.kv_len)
    return center, sort


def _gpu32(w, q, k, v):
    """FP32 output of the CUDA path with the public operator's policy for this workload."""
    center, sort = _policy(w, q, k)
    if w.op == "piper":
        call = AttentionCall("piper", q, k, v, w.head_dim ** -0.5, w.causal, center=center, sort=sort,
                             out_dtype=torch.float32).fwd()
    else:
        call = AttentionCall("sage2pp", q, k, v, w.head_dim ** -0.5, w.causal, out_dtype=torch.float32).fwd()
    assert call.status()[0] == 0
    return _np(call.out)


def _gpu16(w, q, k, v):
    if w.op == "piper":
        return _np(pk.piper_attention(q, k, v, is_causal=w.causal, center_value=w.center))
    return _np(pk.sage_attention_2pp(q, k, v, is_causal=w.causal))


def _piper_rows(w, q, k, v, rows):
    """Oracle FP32 output for query rows `rows` (32-row aligned start) of a one-head input."""
    center, sort = _policy(w, q, k)
    qf, kf, vf = _np(q), _np(k), _np(v)
    prep = oracle.piper_prepare_oracle(qf[:, :, rows], kf, vf, center_value=center, qk_quantization="per_warp",
                                       sort_value_rows=sort)
    return oracle.piper_tile_loop(prep["q_codes"][0, 0], prep["q_scale"][0, 0], prep["k_codes"][0, 0],
                                  prep["k_scale"][0, 0], prep["v_codes"][0, 0], prep["v_scale"][0, 0],
                                  prep["v_mean"][0, 0], w.head_dim ** -0.5, w.causal, row0=rows.start)


def test_c1_whole_tensor():
    w = WORKLOADS["c1"]
    q, k, v = make_inputs(w, "cuda")
    want = oracle.piper_attention_oracle(_np(q), _np(k), _np(v), w.head_dim ** -0.5, False, center_value=False,
                                         qk_quantization="per_warp")
    out32 = _gpu32(w, q, k, v)
    err = _gate32(out32, want)
    print(f"c1 whole tensor: max-abs {err:.3e}")
    _gate16(_gpu16(w, q, k, v), out32, want, w.dtype)


def test_c2_whole_head():
    w = WORKLOADS["c2"]
    q, k, v = make_inputs(w, "cuda", range(7, 8))
    assert _policy(w, q, k) == (True, False)
    want = _piper_rows(w, q, k, v, slice(0, w.q_len))
    out32 = _gpu32(w, q, k, v)[0, 0]
    err = _gate32(out32, want)
    print(f"c2 head 7, all {w.q_len} rows: max-abs {err:.3e}, |out| max {np.abs(want).max():.2f}")
    _gate16(_gpu16(w, q, k, v)[0, 0], out32, want, w.dtype)


C3_BLOCKS = [slice(0, 128), slice(2048 + 32, 2048 + 288), slice(5120 - 64, 5120 + 64), slice(8192 - 256, 8192)]
C4_BLOCKS = [slice(0, 128), slice(4096, 4224), slice(16384 - 32, 16384 + 96), slice(32760 - 120 - 128, 32760)]


@pytest.mark.parametrize("name,head,blocks", [
    ("c3", 5, C3_BLOCKS),
    ("c3", 127, C3_BLOCKS[1:3]),
    ("c4", 3, C4_BLOCKS),
    ("c4", 39, C4_BLOCKS[1:3]),
])
def test_c3_c4_one_head_row_blocks(name, head, blocks):
    w = WORKLOADS[name]
    q, k, v = make_inputs(w, "cuda", range(head, head + 1))
    center, sort = _policy(w, q, k)
    assert center == (name == "c4") and sort == (name == "c4")
    out32 = _gpu32(w, q, k, v)[0, 0]
    out16 = _gpu16(w, q, k, v)[0, 0]
    for rows in blocks:
        want = _piper_rows(w, q, k, v, rows)
        err = _gate32(out32[rows], want)
        print(f"{name} head {head} rows {rows.start}:{rows.stop}: max-abs {err:.3e}, |out| max {np.abs(want).max():.2f}")
        _gate16(out16[rows], out32[rows], want, w.dtype)


def test_c5_sage_strided_rectangular_whole_head():
    w = WORKLOADS["c5"]
    q, k, v = make_inputs(w, "cuda", range(11, 12))
    assert k.stride(2) == 2 * w.head_dim and not k.is_contiguous()
    want = oracle.sage_attention_2pp_oracle(_np(q), _np(k), _np(v), w.head_dim ** -0.5, False,
                                            qk_quantization="per_thread")
    out32 = _gpu32(w, q, k, v)
    err = _gate32(out32, want)
    print(f"c5 head 11, all {w.q_len} rows: max-abs {err:.3e}")
    _gate16(_gpu16(w, q, k, v), out32, want, w.dtype)


# ---------------------------------------------------------------------------------------------
# Quantised codes, scales and key order of one whole head of every configuration, bit for bit
# against the oracle (which is itself pinned to the reference's quantizers), with the oracle's
# means injected so that both sides quantise the same numbers.
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,head", [("c1", 3), ("c2", 30), ("c3", 64), ("c4", 17), ("c5", 20)])
def test_codes_scales_order_bit_exact_on_config_heads(name, head):
    w = WORKLOADS[name]
    q, k, v = make_inputs(w, "cuda", range(head, head + 1))
    center, sort = _policy(w, q, k)
    qf, kf, vf = _np(q), _np(k), _np(v)
    d, sq, sk = w.head_dim, w.q_len, w.kv_len
    if w.op == "piper":
        gran = "per_warp"
        prep = oracle.piper_prepare_oracle(qf, kf, vf, center_value=center, qk_quantization=gran, sort_value_rows=sort)
        call = AttentionCall("piper", q, k, v, d ** -0.5, w.causal, center=center, sort=sort, gran=gran,
                             k_mean=prep["k_mean"][0, :, 0], v_mean=prep["v_mean"][0, :, 0]).prepare()
    else:
        gran = "per_thread"
        prep = oracle.sage_prepare_oracle(qf, kf, vf, qk_quantization=gran)
        call = AttentionCall("sage2pp", q, k, v, d ** -0.5, w.causal, gran=gran, k_mean=prep["k_mean"][0, :, 0]).prepare()
    torch.cuda.synchronize()
    vw = call.views
    qc = call.view("q_codes", torch.int8, (1, vw.sq_pad, d)).cpu().numpy()
    kc = call.view("k_codes", torch.int8, (1, vw.sk_pad, d)).cpu().numpy()
    vt = call.view("v_codes_t", torch.uint8, (1, d, vw.sk_pad)).cpu().numpy()
    assert np.array_equal(qc[:, :sq], prep["q_codes"][0]) and not qc[:, sq:].any()
    assert np.array_equal(kc[:, :sk], prep["k_codes"][0]) and not kc[:, sk:].any()
    want_v = prep["v_codes"][0]
    assert np.array_equal(vt.transpose(0, 2, 1)[:, :sk].view(want_v.dtype), want_v) and not vt[:, :, sk:].any()
    qg, kg, vs = prep["q_group_scale"][0], prep["k_group_scale"][0], prep["v_scale"][0]
    assert np.array_equal(call.view("q_group_scale", torch.float32, (1, qg.shape[1])).cpu().numpy(), qg.reshape(1, -1))
    assert np.array_equal(call.view("k_group_scale", torch.float32, (1, kg.shape[1])).cpu().numpy(), kg.reshape(1, -1))
    assert np.array_equal(call.view("v_scale", torch.float32, (1, vs.size)).cpu().numpy(), vs.reshape(1, -1))
    if sort:
        order = call.view("order", torch.int32, (1, sk)).cpu().numpy()
        assert np.array_equal(order, prep["order"][0].astype(np.int32))
    else:
        assert not call.views.order


@pytest.mark.parametrize("name,head", [("c4", 8), ("c5", 2), ("c3", 1)])
def test_means_equal_oracle_means_at_config_length(name, head):
    """The FP64-accumulated chunked means equal the oracle's mean bit for bit at full length
    (c4: 64 chunks of 512 rows, the last one ragged; c5: sequence stride 2*D)."""
    w = WORKLOADS[name]
    q, k, v = make_inputs(w, "cuda", range(head, head + 1))
    call = AttentionCall("piper", q, k, v, w.head_dim ** -0.5, False, center=True).prepare()
    torch.cuda.synchronize()
    km = call.view("k_mean", torch.float32, (1, w.head_dim)).cpu().numpy()
    vm = call.view("v_mean", torch.float32, (1, w.head_dim)).cpu().numpy()
    assert np.array_equal(km, oracle.sequence_mean(_np(k))[0, :, 0])
    assert np.array_equal(vm, oracle.sequence_mean(_np(v))[0, :, 0])


def test_key_order_with_ties_and_skipped_digit_passes():
    """Multi-chunk radix sort against a stable argsort: 5000 keys (five 1024-key chunks) with
    duplicated value rows (exact ties keep their original order).  Ranges in [1, 2) share the
    two high digits of their bit patterns, so two of the four passes are skipped (an even
    number of passes ran: the order is already in the first index buffer); the second case
    spreads the ranges over several binades so that three passes run (odd: copied back)."""
    gen = torch.Generator().manual_seed(77)
    for spread in (False, True):
        sk, d = 5000, 128
        base = torch.rand(1, 1, sk, d, generator=gen) * 0.5
        base[..., 0] = 1.0 + torch.rand(1, 1, sk, generator=gen) * (0.999 if not spread else 0.0)
        if spread:
            base[..., 0] = torch.exp2(torch.randint(-3, 4, (1, 1, sk), generator=gen).float()) * (1 + torch.rand(1, 1, sk, generator=gen))
        v = base.to(torch.float16)
        v[:, :, 1000:1500] = v[:, :, 2000:2500]  # exact duplicate rows: ties
        v[:, :, 4000:4064] = v[:, :, 17:18]
        v = v.cuda()
        q = torch.randn(1, 1, 64, d, generator=gen).to(torch.float16).cuda()
        k = torch.randn(1, 1, sk, d, generator=gen).to(torch.float16).cuda()
        zero = np.zeros((1, d), dtype=np.float32)
        call = AttentionCall("piper", q, k, v, d ** -0.5, False, center=True, sort=True, v_mean=zero).prepare()
        torch.cuda.synchronize()
        order = call.view("order", torch.int32, (1, sk)).cpu().numpy()[0]
        rng = np.abs(_np(v)[0, 0]).max(axis=-1)
        assert len(np.unique(rng)) < sk  # ties are present
        assert np.array_equal(order, np.argsort(rng, kind="stable").astype(np.int32))


def _reference_functions():
    """The reference project's own portable loops, when its package is installed beside the
    oracle (oracle/_ref, filled by oracle/build_ref.py where the reference tree exists)."""
    try:
        from oracle.build_ref import import_reference
        import_reference()
        from piper_kernels.attention.piper.reference import reference_piper_attention
        from piper_kernels.attention.sage2pp.reference import reference_sage_attention_2pp
    except ImportError as exc:
        pytest.skip(f"reference package not installed beside the oracle: {exc}")
    return reference_piper_attention, reference_sage_attention_2pp


@pytest.mark.parametrize("name,head", [("c2", 21), ("c5", 5), ("c1", 6)])
def test_whole_head_against_the_reference_loop_on_cuda_tensors(name, head):
    """Second, whole-tensor oracle: the reference's own portable loop (device-agnostic PyTorch)
    run on CUDA tensors with FP32 inputs, against the FP32 output of the CUDA kernels."""
    ref_piper, ref_sage = _reference_functions()
    w = WORKLOADS[name]
    q, k, v = make_inputs(w, "cuda", range(head, head + 1))
    center, sort = _policy(w, q, k)
    with torch.no_grad():
        if w.op == "piper":
            want = ref_piper(q.float(), k.float(), v.float(), w.head_dim ** -0.5, w.causal, center_value=center,
                             qk_quantization="per_warp", sort_value_rows=sort)
        else:
            want = ref_sage(q.float(), k.float(), v.float(), w.head_dim ** -0.5, w.causal, qk_quantization="per_thread")
    assert want.dtype == torch.float32
    err = _gate32(_gpu32(w, q, k, v), want.cpu().numpy())
    print(f"{name} head {head} vs the reference's loop on CUDA: max-abs {err:.3e}")


def test_c4_size_constant_value_is_restored_exactly():
    w = WORKLOADS["c4"]
    q, k, _ = make_inputs(w, "cuda", range(0, 2))
    row = torch.randn(1, 2, 1, w.head_dim, device="cuda").to(w.dtype)
    v = row.expand(1, 2, w.kv_len, w.head_dim).contiguous()
    out = pk.piper_attention(q, k, v, center_value=True)
    assert torch.equal(out, row.expand_as(out))


def test_c4_size_bitwise_determinism_and_head_independence():
    w = WORKLOADS["c4"]
    q, k, v = make_inputs(w, "cuda", range(4, 7))
    a = pk.piper_attention(q, k, v)
    b = pk.piper_attention(q, k, v)
    assert torch.equal(a, b)
    one = pk.piper_attention(q[:, 1:2], k[:, 1:2], v[:, 1:2])  # a head alone equals the head in a batch
    assert torch.equal(one, a[:, 1:2])


def _small32(algo, q, k, v, scale, causal, **kw):
    call = AttentionCall(algo, q, k, v, scale, causal, out_dtype=torch.float32, **kw).fwd()
    assert call.status()[0] == 0
    return _np(call.out)


def test_strided_batch_head_permuted_inputs():
    gen = torch.Generator(device="cuda").manual_seed(9)
    base = torch.randn(3, 2, 300, 128, generator=gen, device="cuda").to(torch.float16)
    q = base.permute(1, 0, 2, 3)  # [2,3,300,128] with swapped batch/head strides
    k = torch.randn(2, 3, 600, 128, generator=gen, device="cuda").to(torch.float16)[:, :, ::2]  # sequence stride 2*D
    v = torch.randn(2, 3, 300, 128, generator=gen, device="cuda").to(torch.float16)
    want = oracle.piper_attention_oracle(_np(q), _np(k), _np(v), 128 ** -0.5, False, center_value=True,
                                         qk_quantization="per_warp")
    out32 = _small32("piper", q, k, v, 128 ** -0.5, False, center=True)
    _gate32(out32, want)
    _gate16(_np(pk.piper_attention(q, k, v, center_value=True)), out32, want, torch.float16)
    want = oracle.sage_attention_2pp_oracle(_np(q), _np(k), _np(v), 128 ** -0.5, False, qk_quantization="per_thread")
    out32 = _small32("sage2pp", q, k, v, 128 ** -0.5, False)
    _gate32(out32, want)
    _gate16(_np(pk.sage_attention_2pp(q, k, v)), out32, want, torch.float16)


def test_unaligned_head_dim_view_uses_elementwise_loads():
    gen = torch.Generator(device="cuda").manual_seed(10)
    wide = torch.randn(1, 2, 200, 67, generator=gen, device="cuda").to(torch.float16)
    q = wide[..., 3:67]  # 6-byte offset: rows are not 16-byte aligned
    k, v = wide[..., 1:65], wide[..., 2:66]
    want = oracle.piper_attention_oracle(_np(q), _np(k), _np(v), 64 ** -0.5, False, center_value=False,
                                         qk_quantization="per_warp")
    out32 = _small32("piper", q, k, v, 64 ** -0.5, False, center=False)
    _gate32(out32, want)
    _gate16(_np(pk.piper_attention(q, k, v, center_value=False)), out32, want, torch.float16)


def test_attention_from_host_equals_device_call():
    from piper_kernels_b200.scheduler import attention_from_host

    gen = torch.Generator().manual_seed(12)
    q = torch.randn(2, 5, 700, 128, generator=gen).to(torch.bfloat16).pin_memory()
    k = torch.randn(2, 5, 900, 128, generator=gen).to(torch.bfloat16).pin_memory()
    v = (torch.randn(2, 5, 900, 128, generator=gen) + 1).to(torch.bfloat16).pin_memory()
    out = torch.empty_like(q).pin_memory()
    attention_from_host(pk.piper_attention, q, k, v, out, "cuda:0", heads_per_chunk=3, center_value=True)
    want = pk.piper_attention(q.cuda(), k.cuda(), v.cuda(), center_value=True).cpu()
    assert torch.equal(out, want)


def test_sharded_attention_on_one_device_equals_unsharded():
    """The head split of the multi-GPU scheduler with the real operator: two "ranks" run their
    chunks of flat heads one after the other on this device and reproduce the unsharded output
    bit for bit (heads are independent)."""
    from piper_kernels_b200.scheduler import shard_heads, sharded_attention

    gen = torch.Generator(device="cuda").manual_seed(14)
    q = torch.randn(1, 5, 600, 128, generator=gen, device="cuda").to(torch.bfloat16)
    k = torch.randn(1, 5, 1100, 128, generator=gen, device="cuda").to(torch.bfloat16)
    v = (torch.randn(1, 5, 1100, 128, generator=gen, device="cuda") + 2).to(torch.bfloat16)
    whole = pk.piper_attention(q, k, v, center_value=True)
    pieces = []
    for rank in range(2):
        out, mine = sharded_attention(pk.piper_attention, q, k, v, world=2, rank=rank, center_value=True)
        assert mine == shard_heads(5, 2, rank) and out.shape[1] == len(mine)
        pieces.append(out)
    assert torch.equal(torch.cat(pieces, dim=1), whole)


def test_torch_compile_fullgraph_matches_eager():
    """The operators trace under torch.compile(fullgraph=True) through their fake kernels, on
    batch/head-permuted inputs, as the reference's compile tests do."""
    gen = torch.Generator(device="cuda").manual_seed(13)
    q = torch.randn(2, 2, 160, 64, generator=gen, device="cuda").to(torch.float16).permute(1, 0, 2, 3)
    k = torch.randn(2, 2, 160, 64, generator=gen, device="cuda").to(torch.float16)
    v = torch.randn(2, 2, 160, 64, generator=gen, device="cuda").to(torch.float16)

    def f(a, b, c):
        return pk.piper_attention(a, b, c, is_causal=True) + pk.sage_attention_2pp(a, b, c)

    compiled = torch.compile(f, fullgraph=True, backend="aot_eager")
    assert torch.equal(compiled(q, k, v), f(q, k, v))
