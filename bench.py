#!/usr/bin/env python
"""Benchmark of the fused quantized attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c4]
                    [--scaling weak|strong] [--heads H] [--quality] [--records out.jsonl]

Metric: attention TOPS = 4*B*H*pairs*D / t, pairs = Sq*Sk (Sq*(Sq+1)/2 for causal problems, the
reference benchmark's convention).  A step is one call of the public operator (quantisation
prepass + fused kernel) on one batch of seeded synthetic input.  The default workload is the
D=128, S=32760 non-causal centred configuration ("c4").

Multi-GPU (one process per GPU, no collective on the data path; heads are independent):
  --scaling weak    every rank processes its own copy of the workload's heads (default)
  --scaling strong  the workload's flat heads are split into contiguous chunks, one per rank
Box value = operations all ranks processed / max-over-ranks time.

One JSON line is printed by rank 0.  ``--impl reference`` times the reference's own portable
CPU loop (installed under oracle/_ref; the numpy port when that is absent) on the host cores.
"""

from __future__ import annotations

import argparse
import datetime
import json
import os
import platform
import statistics
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "attention_tops"
UNIT = "TOPS"
NOMINAL_INT8_TOPS = 4500.0
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one fused-kernel launch per flat
# head, from ncu captures summarised under profiles/: c4 from a capture of a 4-head slice of c4
# itself, c2 from a capture of the whole workload.  Every head has its own Q/K/V codes, vectors
# and output, so the traffic of a launch is proportional to the heads it processes.
FUSED_DRAM_BYTES_PER_HEAD = {
    # 4-head slice of c4: 52.55 MB read per launch (codes and vectors, each read once; K/V of a head stay in L2
    # for all of its query tiles).  The slice's 33.5 MB of output were still in L2 when the kernel ended
    # (3-6 MB written); the full workload's 335 MB cannot be, so the output bytes are counted as written.
    "c4": 52.55e6 / 4 + 32760 * 128 * 2,
    "c2": 99.3e6 / 48,
}

_JSON_OUT = None  # duplicate of the original standard output, set in main()


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--heads", type=int, default=0, help="use only the first HEADS flat heads of the workload")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="target CPU time of the cpu_baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-peaks", action="store_true", help="skip the library 8-bit GEMM yardsticks")
    ap.add_argument("--quality", action="store_true", help="SQNR / MAE / rel-L1 / max-abs against FP32 SDPA")
    ap.add_argument("--records", type=Path, default=None, help="append benchmark records (schema v1) as JSON lines")
    return ap.parse_args()


def pairs(w) -> float:
    return w.q_len * (w.q_len + 1) / 2 if w.causal else float(w.q_len) * w.kv_len


def metric_ops(w, flat_heads: int) -> float:
    """Operation count of the metric: 4 * heads * pairs * D."""
    return 4.0 * flat_heads * pairs(w) * w.head_dim


def workload_config(w, n_gpus, scaling, heads_per_rank):
    how = (f"{n_gpus} x independent copies of the workload's heads" if scaling == "weak"
           else f"the workload's {sum(heads_per_rank)} flat heads split over {n_gpus} ranks as {heads_per_rank}")
    return {
        "workload": f"{w.name}: {w.note}", "op": w.op, "batch": w.batch, "heads": w.heads,
        "q_len": w.q_len, "kv_len": w.kv_len, "head_dim": w.head_dim, "in_dtype": str(w.dtype).split(".")[-1],
        "causal": w.causal, "sharding": how + ", no collective on the data path",
        "l2": "inputs of one step exceed the 126 MB L2 (c4: 1 GB), no explicit flush" if w.name in ("c3", "c4")
              else "inputs of one step may fit the 126 MB L2; the whole operator (prepass included) re-reads them from where they are",
    }


def policy(w):
    """Centering / key-order policy of the public operator for a workload (mirrors
    piper_kernels_b200.attention.piper without needing a tensor)."""
    center = bool(w.center) if w.center is not None else (w.op == "piper" and not w.causal and w.head_dim == 128
                                                          and min(w.q_len, w.kv_len) >= 1024)
    sort = w.op == "piper" and center and not w.causal and w.head_dim == 128 and w.kv_len >= 16384
    return center, sort


# --------------------------------------------------------------------------------------
# CPU arm: the reference's portable loop (or its numpy port) on the host cores
# --------------------------------------------------------------------------------------
def _reference_module():
    try:
        from oracle.build_ref import import_reference
        import_reference()
        from piper_kernels.attention.piper.reference import reference_piper_attention
        from piper_kernels.attention.sage2pp.reference import reference_sage_attention_2pp
        return reference_piper_attention, reference_sage_attention_2pp
    except Exception:  # the installed reference is optional: fall back to the port
        return None


def cpu_reference_tops(w, target_seconds: float, threads: int):
    """Times the reference's CPU implementation of the path on one head of the workload: all
    keys, a bounded number of query rows (the whole head for causal problems).  Returns
    (tops, kind, description).  kind "reference": the reference's own torch loop with
    torch.set_num_threads(threads); kind "port": the numpy restatement, one thread per core."""
    import torch

    from piper_kernels_b200.workloads import make_inputs

    q, k, v = make_inputs(w, "cpu", range(0, 1))
    scale = w.head_dim ** -0.5
    center, sort = policy(w)
    ref = _reference_module()
    if ref is not None:
        ref_piper, ref_sage = ref
        torch.set_num_threads(threads)
        qf, kf, vf = q.float(), k.float().contiguous(), v.float().contiguous()

        def run(rows: int) -> float:
            t0 = time.perf_counter()
            with torch.no_grad():
                if w.op == "piper":
                    ref_piper(qf[:, :, :rows], kf, vf, scale, w.causal, center_value=center,
                              qk_quantization="per_warp", sort_value_rows=sort)
                else:
                    ref_sage(qf[:, :, :rows], kf, vf, scale, w.causal, qk_quantization="per_thread")
            return time.perf_counter() - t0

        if w.causal:
            rows = w.q_len
            t = min(run(rows) for _ in range(2))
        else:
            probe = min(w.q_len, 2048)
            t_probe = run(probe)
            rows = int(min(w.q_len, max(probe, probe * target_seconds / max(t_probe, 1e-3)))) // 32 * 32 or w.q_len
            t = run(rows)
        n_pairs = rows * (rows + 1) / 2 if w.causal else float(rows) * w.kv_len
        desc = (f"{w.name} head 0 through the reference's reference_{'piper_attention' if w.op == 'piper' else 'sage_attention_2pp'} "
                f"(torch CPU, {threads} threads): first {rows} of {w.q_len} query rows, all {w.kv_len} keys, {t:.1f} s wall")
        return 4.0 * n_pairs * w.head_dim / t / 1e12, "reference", desc

    from threadpoolctl import threadpool_limits

    import oracle

    qf, kf, vf = (t.float().numpy() for t in (q, k, v))
    chunk = 1024  # rows per work item: large enough that numpy's per-call overhead is negligible

    def run_port(rows: int, nthreads: int) -> float:
        t0 = time.perf_counter()
        if w.op == "piper":
            prep = oracle.piper_prepare_oracle(qf[:, :, :rows], kf, vf, center_value=center,
                                               qk_quantization="per_warp", sort_value_rows=sort)
            args = (prep["k_codes"][0, 0], prep["k_scale"][0, 0], prep["v_codes"][0, 0], prep["v_scale"][0, 0],
                    prep["v_mean"][0, 0])

            def work(r0):
                r1 = min(rows, r0 + chunk)
                return oracle.piper_tile_loop(prep["q_codes"][0, 0, r0:r1], prep["q_scale"][0, 0, r0:r1], *args,
                                              scale, w.causal, row0=r0)
        else:
            def work(r0):
                r1 = min(rows, r0 + chunk)
                return oracle.sage_attention_2pp_oracle(qf[:, :, r0:r1], kf, vf, scale, False, qk_quantization="per_thread")
        with threadpool_limits(limits=1), ThreadPoolExecutor(nthreads) as ex:
            list(ex.map(work, range(0, rows, chunk)))
        return time.perf_counter() - t0

    probe_rows = min(w.q_len, chunk)
    t_probe = run_port(probe_rows, 1)
    rounds = max(1, int(target_seconds / max(t_probe, 1e-3)))
    rows = min(w.q_len, probe_rows * threads * rounds)
    rows = max(chunk, rows // chunk * chunk) if w.q_len >= chunk else w.q_len
    t = run_port(rows, threads)
    desc = (f"{w.name} head 0, numpy port of the reference's portable loop: prepass of the head + tile loop over the "
            f"first {rows} of {w.q_len} query rows, all {w.kv_len} keys, {threads} threads, {t:.1f} s wall")
    return 4.0 * rows * w.kv_len * w.head_dim / t / 1e12, "port", desc


def reference_arm(args, w, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    per_step = max(2.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    vals, times = [], []
    kind, desc = "port", ""
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        tops, kind, desc = cpu_reference_tops(w, per_step, threads)
        if i >= args.warmup:
            vals.append(tops)
            times.append((time.perf_counter() - t0) * 1e3)
    value = statistics.mean(vals)
    flat = args.heads or w.flat_heads
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": statistics.mean(times), "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": workload_config(w, args.gpus, args.scaling, [flat] * args.gpus if args.scaling == "weak" else [flat]),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), file=_JSON_OUT or sys.stdout, flush=True)


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(index)],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.file.read().splitlines():
            f = [x.strip() for x in row.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [s for s, p in zip(sm, power) if p >= 0.6 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


def timed(fn, steps, sync, barrier):
    import torch
    barrier(); sync()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    sync(); barrier()
    return a.elapsed_time(b) / steps  # ms per step on this rank


def timed_each(fn, steps, sync):
    """Per-call device times (ms) of `steps` calls, for median / p20 / p80 records."""
    import torch
    sync()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in evs:
        a.record(); fn(); b.record()
    sync()
    return sorted(a.elapsed_time(b) for a, b in evs)


def quantile(ordered, q):
    if len(ordered) == 1:
        return ordered[0]
    pos = q * (len(ordered) - 1)
    lo = int(pos)
    hi = min(lo + 1, len(ordered) - 1)
    return ordered[lo] + (ordered[hi] - ordered[lo]) * (pos - lo)


def library_peaks(dev):
    """Same-box 8-bit GEMM throughput of the vendor library (torch._int_mm, torch._scaled_mm on
    8192^3, best of 10): a yardstick for the tensor pipe, measured outside every timed region and
    never part of the attention path."""
    import torch
    out = {}
    n = 8192

    def best(fn):
        fn(); torch.cuda.synchronize(dev)
        ts = []
        for _ in range(10):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record(); torch.cuda.synchronize(dev)
            ts.append(a.elapsed_time(b))
        return 2.0 * n ** 3 / (min(ts) * 1e-3) / 1e12

    try:
        x = torch.randint(-127, 127, (n, n), dtype=torch.int8, device=dev)
        y = torch.randint(-127, 127, (n, n), dtype=torch.int8, device=dev).t()
        out["int8"] = best(lambda: torch._int_mm(x, y))
        del x, y
    except Exception as exc:
        out["int8_error"] = f"{type(exc).__name__}: {exc}"[:120]
    try:
        x = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        y = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev)
        out["fp8"] = best(lambda: torch._scaled_mm(x, y, scale_a=one, scale_b=one, out_dtype=torch.bfloat16))
        del x, y
    except Exception as exc:
        out["fp8_error"] = f"{type(exc).__name__}: {exc}"[:120]
    return out


def library_attention(dev, q, k, v, causal, steps=3):
    """The vendor library's 16-bit attention (torch SDPA, whichever fused backend torch picks) on the
    same tensors: a comparison row like the reference benchmark's SDPA provider
    (benchmarks/lib/attention_providers.py), measured outside every timed region and never part of
    the path under test.  Returns milliseconds per call, or an error string."""
    import torch
    import torch.nn.functional as F
    try:
        fn = lambda: F.scaled_dot_product_attention(q, k, v, is_causal=causal)  # noqa: E731
        fn(); torch.cuda.synchronize(dev)
        ts = []
        for _ in range(steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record(); torch.cuda.synchronize(dev)
            ts.append(a.elapsed_time(b))
        return sorted(ts)[len(ts) // 2]
    except Exception as exc:  # noqa: BLE001 - a yardstick must not fail the run
        return f"{type(exc).__name__}: {exc}"[:120]


def quality_metrics(actual, reference):
    """Metric definitions of the reference's benchmarks (benchmarks/lib/quality.py:107-180):
    finite pairs only, float64 accumulation."""
    import torch
    a, r = actual.double().flatten(), reference.double().flatten()
    fin = torch.isfinite(a) & torch.isfinite(r)
    a, r = a[fin], r[fin]
    err = a - r
    tiny = torch.finfo(torch.float64).tiny
    return {
        "mean_absolute_error": float(err.abs().mean()), "max_absolute_error": float(err.abs().max()),
        "relative_l1_error": float(err.abs().sum() / r.abs().sum().clamp_min(tiny)),
        "relative_l2_error": float(err.square().sum().sqrt() / r.square().sum().sqrt().clamp_min(tiny)),
        "sqnr_db": float(10 * torch.log10(r.square().sum() / err.square().sum())),
        "cosine_similarity": float((a @ r) / (a.norm() * r.norm()).clamp_min(tiny)),
        "actual_nonfinite_count": int((~torch.isfinite(actual)).sum()),
        "reference_nonfinite_count": int((~torch.isfinite(reference)).sum()),
        "nonfinite_mismatch_count": int((torch.isfinite(actual) != torch.isfinite(reference)).sum()), "saturation": {},
    }


def environment_info(dev):
    import torch
    rev = dirty = None
    try:
        rev = subprocess.run(["git", "-C", str(ROOT), "rev-parse", "HEAD"], capture_output=True, text=True, timeout=5).stdout.strip() or None
        dirty = bool(subprocess.run(["git", "-C", str(ROOT), "status", "--porcelain"], capture_output=True, text=True, timeout=5).stdout.strip())
    except (OSError, subprocess.SubprocessError):
        pass
    cap = torch.cuda.get_device_capability(dev)
    return {
        "captured_at_utc": datetime.datetime.now(datetime.timezone.utc).isoformat(), "python_version": platform.python_version(),
        "platform": platform.platform(), "torch_version": torch.__version__, "triton_version": None,
        "accelerator_backend": "cuda", "accelerator_runtime_version": torch.version.cuda,
        "accelerator_driver_version": None, "gpu_name": torch.cuda.get_device_name(dev),
        "gpu_architecture": f"sm_{cap[0]}{cap[1]}", "gpu_index": dev.index, "git_revision": rev, "git_dirty": dirty,
    }


def ours_arm(args, w, rank, local_rank, world):
    import torch

    import piper_kernels_b200 as pk
    from piper_kernels_b200.runtime import AttentionCall
    from piper_kernels_b200.scheduler import shard_heads
    from piper_kernels_b200.workloads import make_inputs

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()

    def sync():
        torch.cuda.synchronize(dev)

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    flat_total = min(args.heads, w.flat_heads) if args.heads else w.flat_heads
    if args.scaling == "strong":
        mine = shard_heads(flat_total, world, rank)
        heads_per_rank = [len(shard_heads(flat_total, world, r)) for r in range(world)]
        total_heads = flat_total
    else:
        mine = range(flat_total)
        heads_per_rank = [flat_total] * world
        total_heads = flat_total * world
    if len(mine) == 0:
        raise RuntimeError(f"rank {rank} received no heads: {flat_total} heads over {world} ranks")
    whole = args.scaling == "weak" and not args.heads
    q, k, v = make_inputs(w, dev, None if whole else mine)
    scale = w.head_dim ** -0.5
    if w.op == "piper":
        op = lambda a, b, c: pk.piper_attention(a, b, c, is_causal=w.causal, center_value=w.center)  # noqa: E731
    else:
        op = lambda a, b, c: pk.sage_attention_2pp(a, b, c, is_causal=w.causal)  # noqa: E731
    step = lambda: op(q, k, v)  # noqa: E731

    warmup = max(3, args.warmup)
    t_first0 = time.perf_counter()
    step(); sync()
    first_call_ms = (time.perf_counter() - t_first0) * 1e3
    for _ in range(warmup - 1):
        step()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms = max_over_ranks(timed(step, args.steps, sync, barrier))
    clocks = sampler.stop() if sampler else None
    total_ops = metric_ops(w, total_heads)
    value = total_ops / (ms * 1e-3) / 1e12

    # dominant kernel alone: the fused attention kernel on a prepared workspace
    center, sort = policy(w)
    if w.op == "piper":
        call = AttentionCall("piper", q, k, v, scale, w.causal, center=center, sort=sort)
    else:
        call = AttentionCall("sage2pp", q, k, v, scale, w.causal)
    call.prepare(); call.run(); sync()
    fused_ms = max_over_ranks(timed(lambda: call.run(), args.steps, sync, barrier))
    prep_ms = max_over_ranks(timed(lambda: call.prepare(), args.steps, sync, barrier))
    fused_each = timed_each(lambda: call.run(), max(args.steps, 5), sync)
    prep_each = timed_each(lambda: call.prepare(), max(args.steps, 5), sync)
    status = call.status()
    out_prepared = call.out.clone() if args.quality else None
    # the same whole call (prepass + fused kernel) replayed from a CUDA graph: what a caller who
    # captures the launch-bound small problems gets (c1: 8 launches of 54 us in a 100 us eager step)
    graph_ms = None
    try:
        from piper_kernels_b200.runtime import GraphedAttention
        graphed = GraphedAttention(call)
        graph_ms = max_over_ranks(timed(graphed.replay, args.steps, sync, barrier))
        del graphed
    except Exception as e:  # noqa: BLE001 - a side measurement must not fail the run
        print(f"graph replay not measured: {e}", file=sys.stderr)
    del call

    # end to end from pinned host memory through the public host entry point: per-head-chunk upload,
    # prepass, fused kernel and download overlap on four streams (heads are independent)
    e2e = None
    if not args.no_e2e:
        from piper_kernels_b200.scheduler import HostAttentionPipeline, suggest_heads_per_chunk

        hq = q.contiguous().cpu().pin_memory()
        if w.name == "c5":  # keep the interleaved K/V layout (sequence stride 2*D) in host memory too
            kv_host = torch.stack((k, v), dim=3).contiguous().cpu().pin_memory()
            hk, hv = kv_host[:, :, :, 0, :], kv_host[:, :, :, 1, :]
        else:
            hk, hv = k.contiguous().cpu().pin_memory(), v.contiguous().cpu().pin_memory()
        hout = torch.empty(q.shape, dtype=q.dtype).pin_memory()
        kwargs = dict(is_causal=w.causal, center_value=w.center) if w.op == "piper" else dict(is_causal=w.causal)
        fn = pk.piper_attention if w.op == "piper" else pk.sage_attention_2pp
        local_heads = q.shape[0] * q.shape[1]
        chunk = suggest_heads_per_chunk(w.ops(1), local_heads)
        pipe = HostAttentionPipeline(dev, heads_per_chunk=chunk, slots=4)

        def e2e_step():
            pipe(fn, hq, hk, hv, hout, **kwargs)

        for _ in range(2):
            e2e_step()
        e2e_ms = max_over_ranks(timed(e2e_step, args.steps, sync, barrier))
        # the same transfers with the kernels left out: the ceiling the host link sets for this rank count
        copy_only = lambda: pipe(fn, hq, hk, hv, hout, copy_only=True, **kwargs)  # noqa: E731
        copy_only()
        copy_ms = max_over_ranks(timed(copy_only, max(2, args.steps // 2), sync, barrier))
        h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv))
        d2h = hout.numel() * hout.element_size()
        e2e = {"value": total_ops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "copy_only_ms_per_step": copy_ms, "copy_only_gbs_per_rank": (h2d + d2h) / (copy_ms * 1e-3) / 1e9,
               "frac_of_copy_ceiling": copy_ms / e2e_ms,
               "api": f"scheduler.HostAttentionPipeline, chunks of up to {chunk} heads, 4 staging slots, pinned host buffers"}

    quality = None
    if args.quality and rank == 0:
        import torch.nn.functional as F
        nq = min(q.shape[0] * q.shape[1], 4)  # FP32 SDPA on a bounded number of heads (a library call, yardstick only)
        fq, fk, fv = (t.flatten(0, 1)[:nq].float().unsqueeze(0) for t in (q, k, v))
        exact = torch.cat([F.scaled_dot_product_attention(fq[:, i:i + 1], fk[:, i:i + 1], fv[:, i:i + 1], is_causal=w.causal)
                           for i in range(nq)], dim=1)
        quality = quality_metrics(out_prepared.flatten(0, 1)[:nq].float().unsqueeze(0), exact)
        quality["heads_compared"] = nq
        quality["against"] = "torch SDPA in FP32 on the same 16-bit inputs"

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks = {}
    pf = ROOT / "MEASURED_PEAKS.json"
    if pf.exists():
        peaks = json.loads(pf.read_text())
    # The fused kernel is timed alone (back-to-back launches, no throttling seen): the burst figure
    # is the denominator; 8-bit MMA issues at twice the bf16 rate.
    if "bf16_tflops" in peaks:
        peak, peak_note = 2.0 * peaks["bf16_tflops"], "2 x measured burst cuBLAS bf16 (8-bit MMA runs at twice the bf16 rate); of measured"
    else:
        peak, peak_note = 2.0 * 1590.0, "2 x fallback burst bf16 1.59 PFLOP/s; of fallback"
    local_heads = len(mine)
    achieved = metric_ops(w, local_heads) / (fused_ms * 1e-3) / 1e12
    per_head = FUSED_DRAM_BYTES_PER_HEAD.get(w.name)
    roofline = {
        "bound": "tensor", "kernel": "fused_attention_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
        "frac": achieved / peak, "traffic": per_head * local_heads if per_head else None,
        "traffic_note": "dram bytes read + written per launch: ncu capture of a slice of this workload x heads per launch" if per_head else None,
        "peak_note": peak_note, "frac_of_nominal_int8": achieved / NOMINAL_INT8_TOPS,
        "ms_per_launch": fused_ms, "prepass_ms": prep_ms,
    }
    if not args.no_peaks:
        lib = library_peaks(dev)
        roofline["peak_int8_measured"] = lib.get("int8")
        roofline["peak_fp8_measured"] = lib.get("fp8")
        if lib.get("int8"):
            roofline["frac_of_measured_int8"] = achieved / lib["int8"]
        if lib.get("fp8") and w.op == "sage2pp":
            roofline["frac_of_measured_fp8"] = achieved / lib["fp8"]
        roofline["peaks_measured_how"] = "torch._int_mm / torch._scaled_mm 8192^3, best of 10, outside the timed region"
        for key in ("int8_error", "fp8_error"):
            if key in lib:
                roofline[key] = lib[key]
    sdpa = None
    if not args.no_peaks:
        t = library_attention(dev, q, k, v, w.causal)
        sdpa = {"provider": f"torch SDPA, {str(w.dtype).split('.')[-1]} (library kernel, comparison row only)"}
        if isinstance(t, float):
            sdpa.update(ms_per_step=t, value=metric_ops(w, local_heads) / (t * 1e-3) / 1e12, unit=UNIT)
        else:
            sdpa["error"] = t
    # The prepass is byte work bound by HBM: 2 bytes read + 1 byte written per input element of
    # q, k and v (the second read of K/V for "statistics, then quantise" should hit L2), plus the
    # per-key vectors; the whole prepass (all its launches) is timed as one unit.
    hbm_peak = peaks.get("hbm_gbs")
    prepass_bytes = 3 * local_heads * (w.q_len + 2 * w.kv_len) * w.head_dim + 16 * local_heads * w.kv_len
    prepass_gbs = prepass_bytes / (prep_ms * 1e-3) / 1e9
    roofline_prepass = {
        "bound": "hbm", "kernel": "prepass (all launches of one call)", "achieved": prepass_gbs,
        "peak": hbm_peak if hbm_peak else 6650.0, "unit": "GB/s",
        "frac": prepass_gbs / (hbm_peak if hbm_peak else 6650.0), "algorithmic_bytes": prepass_bytes,
        "peak_note": "measured copy bandwidth; of measured" if hbm_peak else "of fallback", "ms": prep_ms,
    }
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        tops, kind, desc = cpu_reference_tops(w, args.cpu_seconds, threads)
        cpu_baseline = {"value": tops, "unit": UNIT, "cores": threads, "kind": kind, "sample": desc}

    # status words, Q codes, column statistics (two launches), K codes, V codes; with a key order the row ranges are one
    # more launch and the sort shares its launch with the Q codes
    prepass_launches = 6 + (1 if sort else 0)
    # heads with few query tiles split their keys over several CTAs and add a merge launch (piper only)
    n_qt, n_kt = -(-w.q_len // 128), -(-w.kv_len // 64)
    key_split = w.op == "piper" and not w.causal and n_qt <= 8 and min(8, 16 // n_qt, n_kt // 4) >= 2
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "int8",
        "data": "synthetic", "config": workload_config(w, world, args.scaling, heads_per_rank), "clocks": clocks, "e2e": e2e,
        "gpu_launches": (prepass_launches + 1 + (1 if key_split else 0)) * args.steps, "roofline": roofline, "cpu_baseline": cpu_baseline,
        "roofline_prepass": roofline_prepass, "device_status": status[0],
        "library_attention": sdpa,
        "graph_replay": None if graph_ms is None else {"ms_per_step": graph_ms, "value": total_ops / (graph_ms * 1e-3) / 1e12, "unit": UNIT},
        "per_gpu_value": value / world,
        "value_full_rectangle": (4.0 * total_heads * w.q_len * w.kv_len * w.head_dim / (ms * 1e-3) / 1e12) if w.causal else None,
        "quality": quality,
    }
    print(json.dumps(line), file=_JSON_OUT or sys.stdout, flush=True)

    if args.records is not None:
        def timing(ordered, clock):
            return {"median_ms": quantile(ordered, 0.5), "p20_ms": quantile(ordered, 0.2), "p80_ms": quantile(ordered, 0.8), "clock": clock}
        rec = {
            "schema_version": 1, "benchmark": "attention", "provider": "piper_b200_" + w.op,
            "shape": {"batch_size": w.batch, "num_query_heads": w.heads, "num_key_value_heads": w.heads, "query_length": w.q_len,
                      "key_value_length": w.kv_len, "head_dim": w.head_dim, "flat_heads_run": local_heads},
            "configuration": {"dtype": str(w.dtype).split(".")[-1], "is_causal": w.causal, "center_value": center,
                              "sort_value_rows": sort, "workload": w.name},
            "timings": {"warmup_ms": 0, "measurement_time_ms": max(1, int(ms * args.steps)), "first_call_ms": first_call_ms,
                        "first_call_clock": "synchronized_wall", "preparation": timing(prep_each, "device_event"),
                        "prepared_execution": timing(fused_each, "device_event"),
                        "operator_end_to_end": {"median_ms": ms, "p20_ms": ms, "p80_ms": ms, "clock": "device_event"}},
            "quality": quality, "environment": environment_info(dev),
            "extra": {"effective_tflops": metric_ops(w, local_heads) / (quantile(fused_each, 0.5) * 1e-3) / 1e12,
                      "effective_tflops_end_to_end": value / world},
        }
        args.records.parent.mkdir(parents=True, exist_ok=True)
        with args.records.open("a", encoding="utf-8") as f:
            f.write(json.dumps(rec, separators=(",", ":")) + "\n")
            if sdpa is not None and "ms_per_step" in sdpa:
                t = sdpa["ms_per_step"]
                ref_rec = dict(rec, provider="torch_sdpa", quality=None,
                               configuration={"dtype": str(w.dtype).split(".")[-1], "is_causal": w.causal, "workload": w.name},
                               timings={"warmup_ms": 0, "measurement_time_ms": max(1, int(3 * t)), "first_call_ms": None,
                                        "first_call_clock": "synchronized_wall", "preparation": None, "prepared_execution": None,
                                        "operator_end_to_end": {"median_ms": t, "p20_ms": t, "p80_ms": t, "clock": "device_event"}},
                               extra={"effective_tflops_end_to_end": sdpa["value"]})
                f.write(json.dumps(ref_rec, separators=(",", ":")) + "\n")
    if dist is not None:
        dist.destroy_process_group()


def main():
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world == 1 and args.impl == "ours":
        # convenience: relaunch under torchrun, one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29533"),
               str(Path(__file__).resolve()), *sys.argv[1:]]
        raise SystemExit(subprocess.call(cmd))
    from piper_kernels_b200.workloads import WORKLOADS

    # Standard output carries exactly one JSON line.  Libraries loaded below write banners to
    # file descriptor 1 from C code (NCCL prints its version there), so descriptor 1 is pointed at
    # standard error for the run and the JSON line goes to a duplicate of the original.
    sys.stdout.flush()
    json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    global _JSON_OUT
    _JSON_OUT = json_out

    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        reference_arm(args, w, rank, world)
    else:
        ours_arm(args, w, rank, local_rank, world)


if __name__ == "__main__":
    main()
