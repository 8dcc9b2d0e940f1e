#!/usr/bin/env python
"""Benchmark of the hot path: segmented sum-reduction of fp16 arrays on B200.

One step = one pass of the reference's segmented-reduction sweep over one batch
of synthetic input: 2^28 fp16 elements per GPU, uniform in [-1, 1), reduced to
fp32 per-segment sums at segment sizes 16, 32, 64, 256, 1024 and 16384 (six
launches).  Segments are sharded over the GPUs with no communication (weak
scaling: every GPU holds its own 2^28 elements).  Throughput is elements
processed per second, the reference's counter
(src/reduction/seg_wmma_16n.cu:75-81), in Gelem/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

For N > 1 launch one rank per GPU with torch.distributed.run.  Rank 0 prints
one JSON line.  ``--impl reference`` times the plain CPU implementation of the
same sweep on the host cores (the reference project has no CPU path of its
own; its validation loops are compiled out).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LOG2_ELEMS = 28
SWEEP = [16, 32, 64, 256, 1024, 16384]
FALLBACK_HBM_GBS = 6650.0  # earlier measurement on this pool, used only without MEASURED_PEAKS.json
# dram__bytes_read.sum + dram__bytes_write.sum of one seg_reduce_kernel<4> launch over 2^28
# elements, from the ncu capture summarised in profiles/; None until measured.
NCU_TRAFFIC_BYTES_S16 = None


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--algo", default="auto", choices=["auto", "mma", "shuffle"])
    ap.add_argument("--log2-elems", type=int, default=LOG2_ELEMS,
                    help="elements per GPU (default 28, the reference sweep's size)")
    ap.add_argument("--profile", default=None, choices=["reduce", "scan", "full"],
                    help="run ONE untimed pass of the named kernels at --log2-elems and exit "
                         "(the small case an ncu capture wraps)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the other configurations, the e2e leg and the CPU baseline")
    return ap.parse_args()


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi sampled every 200 ms while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU arm
def cpu_sweep(log2_sample: int, min_seconds: float, max_passes: int):
    """Times the plain CPU segmented reduction over the sweep on a bounded sample.
    Returns (Gelem/s, cores, passes, seconds)."""
    import numpy as np
    import oracle
    lib = oracle.c_lib()
    n = 1 << log2_sample
    x = oracle.c_fill_f16(n, 2024, 0, "uniform_pm1")
    outs = {s: np.empty(n // s, dtype=np.float32) for s in SWEEP}
    cores = lib.tcu_cpu_available_cores()
    for s in SWEEP:  # warm-up: page in
        lib.tcu_cpu_segmented_reduce(x.ctypes.data, outs[s].ctypes.data, n // s, s, 0)
    t0 = time.perf_counter()
    passes = 0
    while passes < max_passes and (passes == 0 or time.perf_counter() - t0 < min_seconds):
        for s in SWEEP:
            lib.tcu_cpu_segmented_reduce(x.ctypes.data, outs[s].ctypes.data, n // s, s, 0)
        passes += 1
    dt = time.perf_counter() - t0
    return passes * len(SWEEP) * n / dt / 1e9, cores, passes, dt


def run_reference_arm(args, rank: int):
    """The CPU implementation of the sweep, all host threads, rank 0 only."""
    if rank != 0:
        return
    import numpy as np
    import oracle
    lib = oracle.c_lib()
    log2_sample = min(args.log2_elems, 26)
    n = 1 << log2_sample
    x = oracle.c_fill_f16(n, 2024, 0, "uniform_pm1")
    outs = {s: np.empty(n // s, dtype=np.float32) for s in SWEEP}
    cores = lib.tcu_cpu_available_cores()

    def step():
        for s in SWEEP:
            lib.tcu_cpu_segmented_reduce(x.ctypes.data, outs[s].ctypes.data, n // s, s, 0)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = args.steps * len(SWEEP) * n / dt / 1e9
    sample = f"{len(SWEEP)} segment sizes x 2^{log2_sample} elements per step"
    print(json.dumps({
        "impl": "reference", "metric": "segmented_reduce_sweep_throughput", "value": value,
        "unit": "Gelem/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, 1),
        "cpu_baseline": {"value": value, "unit": "Gelem/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "Gelem/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def workload_config(args, world: int):
    return {"workload": f"segmented sum reduction sweep, 2^{args.log2_elems} fp16 elements per GPU, "
                        "uniform[-1,1), segment sizes 16/32/64/256/1024/16384, fp32 outputs",
            "elements_per_gpu": 1 << args.log2_elems, "segment_sizes": SWEEP,
            "sharding": f"whole segments over {world} GPU(s), no communication",
            "l2": "inputs (512 MiB) exceed L2 (126 MB) and rotate over 2 buffers",
            "algo": args.algo}


# --------------------------------------------------------------------------- GPU arm
def time_op(torch, fn, reps: int, warm: int = 3):
    """Median and min CUDA-event time (ms) of fn() on the current stream."""
    for _ in range(warm):
        fn()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(reps)]
    torch.cuda.synchronize()
    for a, b in evs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = [a.elapsed_time(b) for a, b in evs]
    return statistics.median(ts), min(ts)


def extras(torch, tcu, dist, args, rank, world, peak_gbs):
    """The other configurations of the benchmark definition, a few repetitions each."""
    out = {}
    dev = torch.device("cuda")
    n28 = 1 << min(args.log2_elems, 28)

    def gelem(n, ms):
        return n / (ms * 1e-3) / 1e9

    def entry(n, bytes_per_elem, ms_med, ms_min):
        g = gelem(n, ms_med)
        return {"gelem_per_s": round(g, 1), "gelem_per_s_best": round(gelem(n, ms_min), 1),
                "gbytes_per_s": round(g * bytes_per_elem, 1),
                "hbm_frac": round(g * bytes_per_elem / peak_gbs, 4), "ms": round(ms_med, 4)}

    # C1: 2^24 elements, S=16, cold cache: rotate over 8 buffer sets (256 MiB of input > 2x L2)
    n24 = 1 << 24
    xs = [tcu.fill(torch.empty(n24, dtype=torch.float16, device=dev), 1, i * n24) for i in range(8)]
    os_ = [torch.empty(n24 // 16, dtype=torch.float32, device=dev) for _ in range(8)]
    k = [0]

    def c1():
        i = k[0] % 8
        k[0] += 1
        tcu.segmented_reduce(xs[i], 16, out=os_[i], algo=args.algo)
    out["C1_seg_reduce_2^24_S16_cold"] = entry(n24, 2.25, *time_op(torch, c1, 40, 8))
    del xs, os_

    x = [tcu.fill(torch.empty(n28, dtype=torch.float16, device=dev), 2, rank * n28 + i * (1 << 40))
         for i in range(2)]
    k[0] = 0
    # C3: segmented scans
    for s, dt, bpe in [(16, torch.float16, 4), (256, torch.float16, 4), (4096, torch.float32, 6)]:
        o = torch.empty(n28, dtype=dt, device=dev)

        def c3():
            k[0] += 1
            tcu.segmented_scan(x[k[0] % 2], s, out=o, algo=args.algo)
        name = f"C3_seg_scan_2^28_S{s}_{'f32' if dt == torch.float32 else 'f16'}"
        out[name] = entry(n28, bpe, *time_op(torch, c3, 10))
        del o
    del x

    # C4 / C5: full reduce and full scan over 2^30 elements in total per GPU at N=1; with more
    # GPUs each rank holds a contiguous 2^30-element shard and one all-gather of per-shard totals.
    n30 = 1 << min(args.log2_elems + 2, 30)
    x = tcu.fill(torch.empty(n30, dtype=torch.float16, device=dev), 3, rank * n30, "uniform_01")
    ws = torch.empty(max(tcu.workspace_bytes(tcu.OP_FULL_SCAN, n30, n30),
                         tcu.workspace_bytes(tcu.OP_FULL_REDUCE, n30, n30)),
                     dtype=torch.uint8, device=dev)
    o32, o64 = torch.empty(1, dtype=torch.float32, device=dev), torch.empty(1, dtype=torch.float64, device=dev)

    def local_total():
        tcu.full_reduce(x, workspace=ws, out=o32, out_f64=o64)
        return o64

    def c4():
        tcu.sharded_full_reduce(local_total)
    ms_med, ms_min = time_op(torch, c4, 10)
    if world > 1:
        t = torch.tensor([ms_med, ms_min], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_med, ms_min = t.tolist()
    out["C4_full_reduce_2^30_per_gpu"] = entry(n30 * world, 2, ms_med, ms_min)

    o = torch.empty(n30, dtype=torch.float32, device=dev)

    def c5():
        if world == 1:
            tcu.full_scan(x, out=o, workspace=ws, algo=args.algo)
        else:  # reduce pass -> all-gather of totals -> scan seeded with the earlier shards
            tcu.sharded_full_scan(local_total, lambda totals, r: tcu.full_scan(
                x, out=o, workspace=ws, shard_totals=totals, shard_index=r))
    ms_med, ms_min = time_op(torch, c5, 8)
    if world > 1:
        t = torch.tensor([ms_med, ms_min], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_med, ms_min = t.tolist()
    out["C5_full_scan_2^30_per_gpu_f32"] = entry(n30 * world, 6, ms_med, ms_min)
    return out


def run_e2e(torch, tcu, dist, args, rank, world):
    """Same sweep through the host-buffer entry point: pinned host input, results read back."""
    import numpy as np
    n = 1 << args.log2_elems
    h_in = torch.empty(n, dtype=torch.float16).pin_memory()
    dev_x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 2024, rank * n)
    h_in.copy_(dev_x)
    del dev_x
    h_out = {s: torch.empty(n // s, dtype=torch.float32).pin_memory() for s in SWEEP}
    ctx = tcu.HostContext(chunk_elements=1 << 25)
    steps = max(2, min(args.steps, 5))

    def step():
        for s in SWEEP:
            ctx.run(tcu.OP_SEGMENTED_REDUCE, h_in, h_out[s], s, algo=args.algo)

    step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()  # each call returns only when its results are in host memory
    dt = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([dt], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t[0])
    ctx.close()
    h2d = len(SWEEP) * n * 2
    d2h = sum(n // s * 4 for s in SWEEP)
    # spot check: the results that came back are the right ones
    import oracle
    ref = oracle.np_segmented_reduce(h_in[:1 << 20].view(torch.int16).numpy().view(np.uint16), 1024)
    assert np.array_equal(h_out[1024][:1 << 10].numpy(), ref.astype(np.float32))
    return {"value": steps * len(SWEEP) * n * world / dt / 1e9, "unit": "Gelem/s",
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": steps,
            "note": "pinned host buffers, chunked copies overlapped with kernels on two streams"}


def profile_pass(torch, tcu, args, n):
    """One launch of each kernel of a family, for a profiler to capture."""
    x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 2024, 0)
    if args.profile == "reduce":
        for s in SWEEP:
            tcu.segmented_reduce(x, s, algo=args.algo)
    elif args.profile == "scan":
        for s, dt in [(16, torch.float16), (256, torch.float16), (4096, torch.float32)]:
            tcu.segmented_scan(x, s, out_dtype=dt, algo=args.algo)
    else:
        tcu.fill(x, 2024, 0, "uniform_01")
        tcu.full_reduce(x)
        tcu.full_scan(x, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert tcu.device_error() == 0
    print(json.dumps({"profile": args.profile, "log2_elems": args.log2_elems, "algo": args.algo}))


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import torch
    import torch.distributed as dist
    import tcu_scope_b200 as tcu

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if args.gpus != world and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)

    n = 1 << args.log2_elems
    dev = torch.device("cuda")
    peak_gbs, peak_kind = hbm_peak()
    if args.profile:
        profile_pass(torch, tcu, args, n)
        return

    # this rank's shard of the logical array: elements [rank*n, (rank+1)*n), two buffers to rotate
    xs = [tcu.fill(torch.empty(n, dtype=torch.float16, device=dev), 2024 + i, rank * n) for i in range(2)]
    outs = {s: torch.empty(n // s, dtype=torch.float32, device=dev) for s in SWEEP}
    counter = [0]

    def step(events=None):
        for j, s in enumerate(SWEEP):
            x = xs[counter[0] % 2]
            counter[0] += 1
            if events is not None:
                events[j][0].record()
            tcu.segmented_reduce(x, s, out=outs[s], algo=args.algo)
            if events is not None:
                events[j][1].record()

    for _ in range(max(args.warmup, 0)):
        step()
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in SWEEP] for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    t_begin.record()
    for k in range(args.steps):
        step(ev[k])
    t_end.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if sampler else None
    total_ms = t_begin.elapsed_time(t_end)
    if world > 1:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t[0])
    assert tcu.device_error() == 0, "a bounded device-side wait ran out"

    per_size = {}
    for j, s in enumerate(SWEEP):
        ts = [ev[k][j][0].elapsed_time(ev[k][j][1]) for k in range(args.steps)]
        ms = statistics.mean(ts)
        bpe = 2 + 4 / s
        per_size[str(s)] = {"ms": round(ms, 4), "gelem_per_s": round(n / ms / 1e6, 1),
                            "gbytes_per_s": round(n * bpe / ms / 1e6, 1),
                            "hbm_frac": round(n * bpe / ms / 1e6 / peak_gbs, 4)}
    value = args.steps * len(SWEEP) * n * world / (total_ms * 1e-3) / 1e9

    # dominant kernel: the 16-element launch moves the most bytes (2 + 4/16 per element)
    dom = per_size["16"]
    roofline = {"bound": "hbm", "kernel": "seg_reduce_kernel<4> (segment size 16)",
                "achieved": dom["gbytes_per_s"], "peak": peak_gbs, "unit": "GB/s",
                "frac": dom["hbm_frac"], "peak_source": f"of {peak_kind}",
                "algorithmic_bytes_per_launch": int(n * 2.25),
                "traffic": NCU_TRAFFIC_BYTES_S16 if args.log2_elems == 28 else None}

    result = {
        "metric": "segmented_reduce_sweep_throughput", "value": round(value, 2), "unit": "Gelem/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(total_ms / args.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, world), "roofline": roofline, "per_segment_size": per_size,
        "gpu_launches": args.steps * len(SWEEP), "clocks": clocks,
    }

    if not args.no_extras:
        result["e2e"] = run_e2e(torch, tcu, dist, args, rank, world)
        result["other_configs"] = extras(torch, tcu, dist, args, rank, world, peak_gbs)
        if rank == 0 and world == 1:
            v, cores, passes, secs = cpu_sweep(26, 8.0, 2000)
            result["cpu_baseline"] = {
                "value": round(v, 3), "unit": "Gelem/s", "cores": cores, "kind": "port",
                "sample": f"{passes} passes of the 6-size sweep over 2^26 elements ({secs:.1f} s)"}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(result))


if __name__ == "__main__":
    main()
