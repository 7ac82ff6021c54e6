#!/usr/bin/env python
"""Benchmark of the fused quantized attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c4]

Metric: attention TOPS = 4*B*H*Sq*Sk*D / t.  A step is one call of the public operator
(quantisation prepass + fused kernel) on one batch of seeded synthetic input.  The default
workload is the D=128, S=32760 non-causal centred configuration ("c4").  With N GPUs every
rank processes its own copy of the workload's heads (independent heads, no collective):
weak scaling, box value = N * ops / max-over-ranks time.

One JSON line is printed by rank 0.  ``--impl reference`` times the CPU restatement of the
reference's portable path (oracle/) on the host cores instead.
"""

from __future__ import annotations

import argparse
import json
import os
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
# DRAM bytes per launch of the fused kernel per query row (read + write), from the ncu capture of
# workload c2 summarised in profiles/fused_attention_kernel_c2_ncu_full.md: 99.3 MB for 48 heads
# x 4096 rows at D=128.  Traffic grows with batch*heads*rows (K/V of a head stay in L2 while its
# query tiles run), so other D=128 workloads scale by their row count.
FUSED_DRAM_BYTES_PER_ROW_D128 = 99.3e6 / (48 * 4096)


_JSON_OUT = None  # duplicate of the original standard output, set in main()


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="target CPU time of the cpu_baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def workload_config(w, n_gpus):
    return {
        "workload": f"{w.name}: {w.note}", "op": w.op, "batch_per_gpu": w.batch, "heads": w.heads,
        "q_len": w.q_len, "kv_len": w.kv_len, "head_dim": w.head_dim, "in_dtype": str(w.dtype).split(".")[-1],
        "causal": w.causal, "sharding": f"{n_gpus} x independent copies of the workload's heads, no collective",
        "l2": "inputs (>= 1 GB at c4) exceed the 126 MB L2, no explicit flush",
    }


# --------------------------------------------------------------------------------------
# CPU arm: the oracle port on the host cores
# --------------------------------------------------------------------------------------
def cpu_reference_tops(w, target_seconds: float, threads: int):
    """Times the numpy restatement of the reference's portable path on one head of the
    workload: the prepass of that head plus the tile loop over a bounded number of query
    rows, split over `threads` host threads.  Returns (tops, description)."""
    import numpy as np
    import torch
    from threadpoolctl import threadpool_limits

    import oracle
    from piper_kernels_b200.workloads import make_inputs

    q, k, v = make_inputs(w, "cpu", range(0, 1))
    qf, kf, vf = (t.float().numpy() for t in (q, k, v))
    scale = w.head_dim ** -0.5
    center = bool(w.center) if w.center is not None else (not w.causal and w.head_dim == 128 and min(w.q_len, w.kv_len) >= 1024)
    sort = w.op == "piper" and center and not w.causal and w.head_dim == 128 and w.kv_len >= 16384
    chunk = 1024  # rows per work item: large enough that numpy's per-call overhead is negligible

    def run(rows: int, nthreads: int) -> float:
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
    t_probe = run(probe_rows, 1)  # one work item on one thread
    rounds = max(1, int(target_seconds / max(t_probe, 1e-3)))
    rows = min(w.q_len, probe_rows * threads * rounds)
    rows = max(chunk, rows // chunk * chunk) if w.q_len >= chunk else w.q_len
    t = run(rows, threads)
    ops = 4.0 * rows * w.kv_len * w.head_dim
    desc = (f"{w.name} head 0: prepass of the head + tile loop over the first {rows} of {w.q_len} query rows, "
            f"all {w.kv_len} keys, {threads} threads, {t:.1f} s wall")
    return ops / t / 1e12, desc


def reference_arm(args, w, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    per_step = max(2.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    vals, times = [], []
    desc = ""
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        tops, desc = cpu_reference_tops(w, per_step, threads)
        if i >= args.warmup:
            vals.append(tops)
            times.append((time.perf_counter() - t0) * 1e3)
    value = statistics.mean(vals)
    rows_ops = None
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": statistics.mean(times), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": workload_config(w, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
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


def ours_arm(args, w, rank, local_rank, world):
    import torch

    import piper_kernels_b200 as pk
    from piper_kernels_b200.attention.piper import default_center_value, should_sort_value_rows
    from piper_kernels_b200.runtime import AttentionCall
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

    q, k, v = make_inputs(w, dev)
    scale = w.head_dim ** -0.5
    if w.op == "piper":
        op = lambda a, b, c: pk.piper_attention(a, b, c, is_causal=w.causal, center_value=w.center)  # noqa: E731
    else:
        op = lambda a, b, c: pk.sage_attention_2pp(a, b, c, is_causal=w.causal)  # noqa: E731
    step = lambda: op(q, k, v)  # noqa: E731

    for _ in range(max(3, args.warmup)):
        step()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms = max_over_ranks(timed(step, args.steps, sync, barrier))
    clocks = sampler.stop() if sampler else None
    ops_per_gpu = w.ops()
    value = world * ops_per_gpu / (ms * 1e-3) / 1e12

    # dominant kernel alone: the fused attention kernel on a prepared workspace
    center = default_center_value(q, k, w.causal) if w.center is None else bool(w.center)
    if w.op == "piper":
        sort = should_sort_value_rows(center_value=center, is_causal=w.causal, head_dim=w.head_dim, key_length=w.kv_len)
        call = AttentionCall("piper", q, k, v, scale, w.causal, center=center, sort=sort)
    else:
        call = AttentionCall("sage2pp", q, k, v, scale, w.causal)
    call.prepare(); call.run(); sync()
    fused_ms = max_over_ranks(timed(lambda: call.run(), args.steps, sync, barrier))
    prep_ms = max_over_ranks(timed(lambda: call.prepare(), args.steps, sync, barrier))
    status = call.status()
    del call

    # end to end from pinned host memory through the public host entry point: per-head-chunk upload,
    # prepass, fused kernel and download overlap on four streams (heads are independent)
    e2e = None
    if not args.no_e2e:
        from piper_kernels_b200.scheduler import HostAttentionPipeline

        hq = q.contiguous().cpu().pin_memory()
        if w.name == "c5":  # keep the interleaved K/V layout (sequence stride 2*D) in host memory too
            kv_host = torch.stack((k, v), dim=3).contiguous().cpu().pin_memory()
            hk, hv = kv_host[:, :, :, 0, :], kv_host[:, :, :, 1, :]
        else:
            hk, hv = k.contiguous().cpu().pin_memory(), v.contiguous().cpu().pin_memory()
        hout = torch.empty(q.shape, dtype=q.dtype).pin_memory()
        kwargs = dict(is_causal=w.causal, center_value=w.center) if w.op == "piper" else dict(is_causal=w.causal)
        fn = pk.piper_attention if w.op == "piper" else pk.sage_attention_2pp
        chunk = max(1, min(4, w.flat_heads // 4))
        pipe = HostAttentionPipeline(dev, heads_per_chunk=chunk)

        def e2e_step():
            pipe(fn, hq, hk, hv, hout, **kwargs)

        for _ in range(2):
            e2e_step()
        e2e_ms = max_over_ranks(timed(e2e_step, args.steps, sync, barrier))
        h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv))
        e2e = {"value": world * ops_per_gpu / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": hout.numel() * hout.element_size(),
               "api": f"scheduler.HostAttentionPipeline, ramped chunks of up to {chunk} heads, pinned host buffers"}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks = {}
    pf = ROOT / "MEASURED_PEAKS.json"
    if pf.exists():
        peaks = json.loads(pf.read_text())
    if "bf16_tflops_sustained" in peaks:
        peak, peak_note = 2.0 * peaks["bf16_tflops_sustained"], "2 x measured sustained cuBLAS bf16 (8-bit MMA runs at twice the bf16 rate); of measured"
    else:
        peak, peak_note = 2.0 * 1400.0, "2 x fallback sustained bf16 1.4 PFLOP/s; of fallback"
    achieved = ops_per_gpu / (fused_ms * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "kernel": "fused_attention_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
        "frac": achieved / peak,
        "traffic": (FUSED_DRAM_BYTES_PER_ROW_D128 * w.flat_heads * w.q_len if (w.head_dim == 128 and w.q_len == w.kv_len) else None),
        "traffic_note": "bytes per launch, scaled from the ncu capture of c2 by rows processed",
        "peak_note": peak_note,
        "frac_of_nominal_int8": achieved / NOMINAL_INT8_TOPS, "ms_per_launch": fused_ms, "prepass_ms": prep_ms,
    }
    # The prepass is byte work bound by HBM: 2 bytes read + 1 byte written per input element of
    # q, k and v (the second read of K/V for "statistics, then quantise" should hit L2), plus the
    # per-key vectors; the whole prepass (all its launches) is timed as one unit.
    hbm_peak = peaks.get("hbm_gbs")
    prepass_bytes = 3 * w.flat_heads * (w.q_len + 2 * w.kv_len) * w.head_dim + 16 * w.flat_heads * w.kv_len
    prepass_gbs = prepass_bytes / (prep_ms * 1e-3) / 1e9
    roofline_prepass = {
        "bound": "hbm", "kernel": "prepass (all launches of one call)", "achieved": prepass_gbs,
        "peak": hbm_peak if hbm_peak else 6650.0, "unit": "GB/s",
        "frac": prepass_gbs / (hbm_peak if hbm_peak else 6650.0), "algorithmic_bytes": prepass_bytes,
        "peak_note": "measured copy bandwidth; of measured" if hbm_peak else "of fallback", "ms": prep_ms,
    }
    # The reference's benchmark counts Sq(Sq+1)/2 query-key pairs for causal problems.
    causal_pairs_value = None
    if w.causal:
        causal_pairs_value = world * 4.0 * w.flat_heads * w.head_dim * (w.q_len * (w.q_len + 1) / 2) / (ms * 1e-3) / 1e12
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        tops, desc = cpu_reference_tops(w, args.cpu_seconds, threads)
        cpu_baseline = {"value": tops, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc}

    prepass_launches = 6 + (2 if (w.op == "piper" and w.kv_len >= 16384 and w.head_dim == 128 and not w.causal) else 0)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic", "config": workload_config(w, world), "clocks": clocks, "e2e": e2e,
        "gpu_launches": (prepass_launches + 1) * args.steps, "roofline": roofline, "cpu_baseline": cpu_baseline,
        "roofline_prepass": roofline_prepass, "value_causal_pairs": causal_pairs_value, "device_status": status[0],
    }
    print(json.dumps(line), file=_JSON_OUT or sys.stdout, flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world == 1:
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
