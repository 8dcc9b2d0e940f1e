#!/usr/bin/env python
"""Benchmark of the hot path: segmented sum-reduction of fp16 arrays on B200.

One step = one pass of the reference's segmented-reduction sweep over one batch
of synthetic input: 2^28 fp16 elements per GPU, uniform in [-1, 1), reduced to
fp32 per-segment sums at segment sizes 16, 32, 64, 256, 1024 and 16384 (six
launches).  Segments are sharded over the GPUs with no communication (weak
scaling: every GPU holds its own 2^28 elements).  Throughput is elements
processed per second, the reference's counter
(src/reduction/seg_wmma_16n.cu:75-81), in Gelem/s.  With more than one GPU the
line also carries the strong-scaling form of every configuration (the fixed
totals of the benchmark definition cut into one shard per GPU), each with its
outputs checked against the fp64 oracle on every rank.

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
NOMINAL_HBM_GBS = 8000.0   # the HBM figure the benchmark definition quotes its target against
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "seg_reduce_kernel_S16_traffic.json")
KERNEL_SOURCES = ["tcu_scope_b200/csrc/common.cuh", "tcu_scope_b200/csrc/reduce_kernels.cuh"]


def kernel_source_hash():
    import hashlib
    h = hashlib.sha256()
    for rel in KERNEL_SOURCES:
        with open(os.path.join(ROOT, rel), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def ncu_traffic(n_elems: int):
    """DRAM bytes of one seg_reduce_kernel<4> launch over n_elems elements, scaled from the ncu
    capture recorded next to its summary (traffic grows with the element count; the full-size
    launch is too large to capture).  None, with the reason, when the record is missing or was
    taken from other kernel sources than the ones this run was built from."""
    try:
        rec = json.load(open(TRAFFIC_FILE))
    except Exception:
        return None, "no capture recorded"
    if rec.get("kernel_source_sha16") != kernel_source_hash():
        return None, "capture predates the current kernel sources"
    per_elem = (rec["dram_bytes_read"] + rec["dram_bytes_write"]) / float(1 << rec["log2_elems"])
    return int(per_elem * n_elems), f"ncu capture at 2^{rec['log2_elems']} elements, scaled"

def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--algo", default="auto", choices=["auto", "mma", "shuffle", "tcgen05"],
                    help="tcgen05 covers reductions up to 2048 and scans up to 16384 elements per "
                         "segment: use it with --profile reduce or --profile scan")
    ap.add_argument("--log2-elems", type=int, default=LOG2_ELEMS,
                    help="elements per GPU (default 28, the reference sweep's size)")
    ap.add_argument("--profile", default=None, choices=["reduce", "scan", "scan16", "scan32", "full", "shard", "general"],
                    help="run ONE untimed pass of the named kernels at --log2-elems and exit "
                         "(the small case an ncu capture wraps)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the other configurations, the e2e leg and the CPU baseline")
    args = ap.parse_args()
    if args.algo == "tcgen05" and args.profile not in ("reduce", "scan", "scan16", "scan32"):
        ap.error("--algo tcgen05 does not cover every size of the sweep: use it with --profile reduce "
                 "or --profile scan (the timed run reports it under ablation_tensor_core_vs_shuffle)")
    return args


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """SM clock and throttle reasons of one GPU through NVML (read-only queries; nothing is
    set).  sample() is called by the benchmark while it waits for the timed region to finish,
    so every sample is taken under load."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if index < len(ids) and ids[index].isdigit():
                    phys = int(ids[index])
            self._n = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
            self._get_reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            self._bits = {
                "hw_slowdown": getattr(pynvml, "nvmlClocksEventReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(pynvml, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(pynvml, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(pynvml, "nvmlClocksEventReasonSwPowerCap", 0x4),
            }
        except Exception as e:  # no NVML: report that instead of a number
            self._n = None
            self.reasons.add(f"nvml unavailable: {type(e).__name__}")

    def sample(self):
        if self._n is None:
            return
        try:
            self.samples.append(self._n.nvmlDeviceGetClockInfo(self._h, self._n.NVML_CLOCK_SM))
            r = self._get_reasons(self._h)
            for name, bit in self._bits.items():
                if r & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def wait_for(self, event):
        """Sample until the CUDA event has completed (the GPU is busy with the timed steps)."""
        self.sample()
        while not event.query():
            self.sample()
            time.sleep(0.0002)

    def result(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "samples": len(self.samples),
                "reasons": sorted(self.reasons)}


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


def run_reference_arm(args, rank: int, json_fd: int):
    """The CPU implementation of the sweep, all host threads, rank 0 only."""
    if rank != 0:
        return
    import numpy as np
    import oracle
    lib = oracle.c_lib()
    log2_sample = args.log2_elems  # the same 2^28 elements per size as the GPU arm
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
    emit(json_fd, {
        "impl": "reference", "metric": "segmented_reduce_sweep_throughput", "value": value,
        "unit": "Gelem/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(workload_config(args, 1), sharding="one host, all cores, whole segments per thread",
                       l2="host memory", timing="wall clock around the K steps",
                       algo="plain C loops (oracle/tcu_oracle.c), fp32 accumulate"),
        "cpu_baseline": {"value": value, "unit": "Gelem/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "Gelem/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })


def workload_config(args, world: int):
    return {"workload": f"segmented sum reduction sweep, 2^{args.log2_elems} fp16 elements per GPU, "
                        "uniform[-1,1), segment sizes 16/32/64/256/1024/16384, fp32 outputs",
            "elements_per_gpu": 1 << args.log2_elems, "segment_sizes": SWEEP,
            "sharding": f"whole segments over {world} GPU(s), no communication",
            "l2": "inputs (512 MiB) exceed L2 (126 MB) and rotate over 2 buffers",
            "timing": "one CUDA-graph replay (6 launches) per step, CUDA events around the K steps",
            "algo": args.algo}


# --------------------------------------------------------------------------- GPU arm
def time_op(torch, fn, reps: int, warm: int = 3):
    """Average CUDA-event time (ms) of fn() over `reps` back-to-back calls on the current
    stream, taken twice: returns (mean of the two batches, the faster batch)."""
    for _ in range(warm):
        fn()
    out = []
    for _ in range(2):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b) / reps)
    return statistics.mean(out), min(out)


def time_graph(torch, fn, launches_per_graph: int, replays: int):
    """fn() is called launches_per_graph times inside one CUDA graph; the graph is replayed
    `replays` times between two events.  Returns ms per fn() call.  For launches far shorter
    than the host's launch overhead (the 2^24-element configuration: ~10 us of GPU work)."""
    for _ in range(launches_per_graph):
        fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for _ in range(launches_per_graph):
                fn()
    torch.cuda.current_stream().wait_stream(side)
    g.replay()
    torch.cuda.synchronize()
    out = []
    for _ in range(2):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(replays):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b) / (replays * launches_per_graph))
    return statistics.mean(out), min(out)


def time_rotating(torch, launch, nbuf: int, replays: int):
    """launch(i) queues one kernel on buffer set i; one CUDA graph holds 12 launches or more,
    cycling over the buffer sets (so consecutive launches never touch the same data and nbuf
    sets exceed twice the L2; the cost of starting a graph is spread over a dozen kernels),
    replayed `replays` times between two events.  Returns ms per launch (mean of 2 batches, best)."""
    per_graph = -(-12 // nbuf) * nbuf
    for i in range(nbuf):
        launch(i)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for i in range(per_graph):
                launch(i % nbuf)
    torch.cuda.current_stream().wait_stream(side)
    g.replay()
    torch.cuda.synchronize()
    out = []
    for _ in range(2):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(replays):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b) / (replays * per_graph))
    return statistics.mean(out), min(out)


def max_over_ranks(torch, dist, world, *vals):
    if world == 1:
        return vals
    t = torch.tensor(list(vals), dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return tuple(t.tolist())


def extras(torch, tcu, dist, args, rank, world, peak_gbs, sweep_gelem_per_gpu):
    """The other configurations of the benchmark definition, a few repetitions each.  With one
    GPU: every configuration at its stated size.  With several: the same per-GPU sizes (weak
    scaling) here, the stated totals cut into shards (strong scaling) in strong_scaling()."""
    out = {}
    dev = torch.device("cuda")
    n28 = 1 << min(args.log2_elems, 28)

    def gelem(n, ms):
        return n / (ms * 1e-3) / 1e9

    def entry(n, bytes_per_elem, ms_med, ms_min, gpus=1):
        g = gelem(n, ms_med)  # n = elements over all `gpus` GPUs; hbm_frac is per GPU
        return {"gelem_per_s": round(g, 1), "gelem_per_s_best": round(gelem(n, ms_min), 1),
                "gbytes_per_s": round(g * bytes_per_elem, 1),
                "hbm_frac": round(g * bytes_per_elem / peak_gbs / gpus, 4),
                "hbm_frac_of_nominal_8tbs": round(g * bytes_per_elem / NOMINAL_HBM_GBS / gpus, 4),
                "ms": round(ms_med, 4)}

    # C1: 2^24 elements, S=16, cold cache: rotate over 8 buffer sets (256 MiB of input > 2x L2)
    n24 = 1 << 24
    xs = [tcu.fill(torch.empty(n24, dtype=torch.float16, device=dev), 1, i * n24) for i in range(8)]
    os_ = [torch.empty(n24 // 16, dtype=torch.float32, device=dev) for _ in range(8)]
    k = [0]

    def c1():
        i = k[0] % 8
        k[0] += 1
        tcu.segmented_reduce(xs[i], 16, out=os_[i], algo=args.algo)
    out["C1_seg_reduce_2^24_S16_cold"] = entry(n24, 2.25, *time_graph(torch, c1, 16, 10))
    c1_entry = out["C1_seg_reduce_2^24_S16_cold"]
    c1_entry["timing"] = "16 launches per CUDA graph, 8 rotating buffer sets"
    # What bounds a launch this short: its HBM time plus the fixed cost of ANY launch of this
    # shape in this graph, measured with the same kernel on an input of one tile per CTA
    # (every CTA starts, loads once and leaves: launch, ramp and drain, next to no data).
    tiny_n = tcu.num_sms() * 16384
    tiny_x = tcu.fill(torch.empty(tiny_n, dtype=torch.float16, device=dev), 1, 0)
    tiny_o = torch.empty(tiny_n // 16, dtype=torch.float32, device=dev)
    ms_fixed, _ = time_graph(torch, lambda: tcu.segmented_reduce(tiny_x, 16, out=tiny_o, algo=args.algo), 16, 10)
    hbm_ms = n24 * 2.25 / (peak_gbs * 1e9) * 1e3
    c1_entry["fixed_cost_ms"] = round(ms_fixed, 4)
    c1_entry["hbm_time_ms"] = round(hbm_ms, 4)
    c1_entry["bound_ms"] = round(ms_fixed + hbm_ms, 4)
    c1_entry["note"] = ("fixed_cost_ms = the same kernel on one tile per CTA in the same kind of graph; "
                        "bound_ms = fixed cost + bytes / measured HBM peak")
    del xs, os_, tiny_x, tiny_o

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

    # C4 / C5: full reduce and full scan over 2^30 elements per GPU.  One GPU: the single-pass
    # kernels.  More GPUs (weak scaling): each rank holds a contiguous 2^30-element shard; the
    # totals travel either inside the kernels (PeerGroup) or through one all-gather per call.
    n30 = 1 << min(args.log2_elems + 2, 30)
    x = tcu.fill(torch.empty(n30, dtype=torch.float16, device=dev), 3, rank * n30, "uniform_01")
    ws = torch.empty(max(tcu.workspace_bytes(tcu.OP_FULL_SCAN, n30, n30),
                         tcu.workspace_bytes(tcu.OP_FULL_REDUCE, n30, n30)),
                     dtype=torch.uint8, device=dev)
    o32, o64 = torch.empty(1, dtype=torch.float32, device=dev), torch.empty(1, dtype=torch.float64, device=dev)
    o = torch.empty(n30, dtype=torch.float32, device=dev)

    def local_total():
        tcu.full_reduce(x, workspace=ws, out=o32, out_f64=o64)
        return o64

    ms = max_over_ranks(torch, dist, world, *time_op(torch, local_total, 10))
    out["C4_full_reduce_2^30_one_gpu"] = entry(n30, 2, *ms)
    ms = max_over_ranks(torch, dist, world, *time_op(
        torch, lambda: tcu.full_scan(x, out=o, workspace=ws, algo=args.algo), 8))
    out["C5_full_scan_2^30_one_gpu_f32"] = entry(n30, 6, *ms)
    one_gpu = {"C2": round(sweep_gelem_per_gpu, 1),
               "C4": out["C4_full_reduce_2^30_one_gpu"]["gelem_per_s"],
               "C5": out["C5_full_scan_2^30_one_gpu_f32"]["gelem_per_s"]}

    grp = tcu.PeerGroup()  # collective
    # the two-pass scan of the multi-GPU path (reduce, then scan seeded by the earlier totals)
    ms = max_over_ranks(torch, dist, world, *time_op(torch, lambda: grp.full_scan(x, out=o), 8))
    key = "C5_full_scan_2^30_per_gpu_f32" if world > 1 else "C5_full_scan_2^30_two_pass_f32"
    out[key] = entry(n30 * world, 6, *ms, world)
    out[key]["exchange"] = "totals stored by the kernels into every rank's memory"
    if world > 1:
        ms = max_over_ranks(torch, dist, world, *time_op(torch, lambda: grp.full_reduce(x, out=o32, out_f64=o64), 10))
        out["C4_full_reduce_2^30_per_gpu"] = entry(n30 * world, 2, *ms, world)
        out["C4_full_reduce_2^30_per_gpu"]["exchange"] = "totals stored by the kernels into every rank's memory"
        ms = max_over_ranks(torch, dist, world, *time_op(
            torch, lambda: tcu.sharded_full_reduce(local_total), 10))
        out["C4_full_reduce_2^30_per_gpu_all_gather"] = entry(n30 * world, 2, *ms, world)
        ms = max_over_ranks(torch, dist, world, *time_op(torch, lambda: tcu.sharded_full_scan(
            local_total, lambda totals, r: tcu.full_scan(x, out=o, workspace=ws, shard_totals=totals,
                                                         shard_index=r)), 8))
        out["C5_full_scan_2^30_per_gpu_f32_all_gather"] = entry(n30 * world, 6, *ms, world)
    del x, o, ws
    if world > 1:
        out["strong_scaling"] = strong_scaling(torch, tcu, dist, args, rank, world, peak_gbs, grp,
                                               one_gpu, out)
    grp.close()  # collective
    return out


def strong_scaling(torch, tcu, dist, args, rank, world, peak_gbs, grp, one_gpu, weak):
    """The configurations of the benchmark definition at their STATED totals (2^28 elements for
    the segmented operations, 2^30 for the full ones) cut into one contiguous shard per GPU.
    Every output is checked against the fp64 oracle on every rank before it is timed; a
    mismatch raises.  Shards of this size fit L2, so each timing rotates over enough buffer
    sets to exceed twice the L2 (segmented legs: one launch per set in a CUDA graph)."""
    import numpy as np
    import oracle
    from tcu_scope_b200.sharded import shard_range
    dev = torch.device("cuda")
    res = {}
    L2_X2 = 2 * 126_000_000

    def bits(t):
        return t.cpu().view(torch.int16).numpy().view(np.uint16)

    def entry(n_total, bpe, ms_med, ms_min, one_gpu_gelem, **kw):
        g = n_total / ms_med / 1e6
        e = {"gelem_per_s": round(g, 1), "gelem_per_s_best": round(n_total / ms_min / 1e6, 1),
             "hbm_frac_per_gpu": round(g * bpe / peak_gbs / world, 4),
             "hbm_frac_of_nominal_8tbs_per_gpu": round(g * bpe / NOMINAL_HBM_GBS / world, 4),
             "ms": round(ms_med, 4), "one_gpu_gelem_per_s": one_gpu_gelem,
             "x_over_1gpu": round(g / one_gpu_gelem, 3) if one_gpu_gelem else None}
        e.update(kw)
        return e

    def all_ok(ok: bool, worst: float):
        t = torch.tensor([0.0 if ok else 1.0, worst], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if t[0].item() != 0.0:
            raise AssertionError("a sharded output does not match the fp64 oracle")
        return float(t[1])

    # ---- C2 / C3: whole segments per rank, no communication
    n_total = 1 << min(args.log2_elems, 28)
    SAMPLE = 1 << 18  # elements per checked chunk: the head, the middle and the tail of the shard

    def seg_leg(kind, s, out_dtype):
        segs = n_total // s
        sb, se = shard_range(segs, rank, world)
        n = (se - sb) * s
        out_elems = (se - sb) if kind == "reduce" else n
        per_set = n * 2 + out_elems * (4 if out_dtype == torch.float32 else 2)
        nbuf = max(2, -(-L2_X2 // per_set))
        xs = [tcu.fill(torch.empty(n, dtype=torch.float16, device=dev), 2024 + i, sb * s) for i in range(nbuf)]
        os_ = [torch.empty(out_elems, dtype=out_dtype, device=dev) for _ in range(nbuf)]

        def launch(i):
            if kind == "reduce":
                tcu.segmented_reduce(xs[i], s, out=os_[i], algo=args.algo)
            else:
                tcu.segmented_scan(xs[i], s, out=os_[i], algo=args.algo)
        launch(0)
        torch.cuda.synchronize()
        worst, ok = 0.0, True
        chunk = max(SAMPLE // s, 1) * s
        for first in sorted({0, (n // 2) // chunk * chunk, max(n - chunk, 0)}):
            xb = oracle.c_fill_f16(chunk, 2024, sb * s + first, "uniform_pm1")
            assert np.array_equal(xb, bits(xs[0][first:first + chunk]))
            if kind == "reduce":
                ref = oracle.c_segmented_reduce(xb, s)
                got = os_[0][first // s:(first + chunk) // s]
            else:
                ref = oracle.c_segmented_scan(xb, s)
                got = os_[0][first:first + chunk]
            if out_dtype == torch.float32:
                bad, max_abs, _ = oracle.np_check_f32(got.cpu().numpy(), ref)
                worst = max(worst, max_abs)
            else:
                bad, w = oracle.np_check_f16(bits(got), ref, 2)
                worst = max(worst, float(w))
            ok = ok and bad == 0
        worst = all_ok(ok, worst)
        ms = max_over_ranks(torch, dist, world, *time_rotating(torch, launch, nbuf, 4))
        del xs, os_
        return ms, worst, nbuf

    sweep_ms, sweep_best, worst_all = 0.0, 0.0, 0.0
    per = {}
    for s in SWEEP:
        (ms, best), worst, nbuf = seg_leg("reduce", s, torch.float32)
        sweep_ms += ms
        sweep_best += best
        worst_all = max(worst_all, worst)
        per[str(s)] = {"ms": round(ms, 4), "gelem_per_s": round(n_total / ms / 1e6, 1),
                       "hbm_frac_per_gpu": round(n_total * (2 + 4 / s) / ms / 1e6 / peak_gbs / world, 4)}
    res["C2_seg_reduce_sweep_2^28_total"] = {
        "gelem_per_s": round(len(SWEEP) * n_total / sweep_ms / 1e6, 1),
        "one_gpu_gelem_per_s": one_gpu["C2"],
        "x_over_1gpu": round(len(SWEEP) * n_total / sweep_ms / 1e6 / one_gpu["C2"], 3),
        "gelem_per_s_best": round(len(SWEEP) * n_total / sweep_best / 1e6, 1),
        "ms_per_sweep": round(sweep_ms, 4), "per_segment_size": per, "checked": True,
        "max_abs_err": worst_all, "buffer_sets": nbuf,
        "timing": "per size: 12 launches per CUDA graph cycling over the buffer sets, max over ranks"}
    for s, dt, bpe in [(16, torch.float16, 4), (256, torch.float16, 4), (4096, torch.float32, 6)]:
        (ms, best), worst, nbuf = seg_leg("scan", s, dt)
        tag = "f32" if dt == torch.float32 else "f16"
        one_g = weak.get(f"C3_seg_scan_2^28_S{s}_{tag}", {}).get("gelem_per_s")
        res[f"C3_seg_scan_2^28_total_S{s}_{tag}"] = entry(
            n_total, bpe, ms, best, one_g, checked=True, buffer_sets=nbuf,
            **({"max_abs_err": worst} if dt == torch.float32 else {"worst_half_ulp": worst}))

    # ---- C4 / C5: contiguous shards of 2^30 elements in total
    n_total = 1 << min(args.log2_elems + 2, 30)
    b, e = shard_range(n_total // 16, rank, world)
    b, e = b * 16, e * 16
    n = e - b
    nbuf = max(1, -(-L2_X2 // (n * 2)))
    xs = [tcu.fill(torch.empty(n, dtype=torch.float16, device=dev), 3, b, "uniform_01") for _ in range(nbuf)]
    o = torch.empty(n, dtype=torch.float32, device=dev)
    o32, o64 = torch.empty(1, dtype=torch.float32, device=dev), torch.empty(1, dtype=torch.float64, device=dev)
    ws = torch.empty(max(tcu.workspace_bytes(tcu.OP_FULL_SCAN, n, n), tcu.workspace_bytes(tcu.OP_FULL_REDUCE, n, n)),
                     dtype=torch.uint8, device=dev)
    k = [0]

    def nxt():
        k[0] += 1
        return xs[k[0] % nbuf]

    def local_total(x=None):
        tcu.full_reduce(xs[k[0] % nbuf] if x is None else x, workspace=ws, out=o32, out_f64=o64)
        return o64

    # the oracle's view of this shard, block by block: totals of all shards, then the scan
    BLOCK = 1 << 22
    run, blocks = 0.0, []
    for first in range(0, n, BLOCK):
        m = min(BLOCK, n - first)
        v = oracle.c_fill_f16(m, 3, b + first, "uniform_01").view(np.float16).astype(np.float64)
        blocks.append((first, m, run))
        run += v.sum()
    t = torch.zeros(world, dtype=torch.float64, device=dev)
    t[rank] = run
    dist.all_reduce(t)
    ref_totals = t.cpu().numpy()
    ref_total, ref_carry = float(ref_totals.sum()), float(ref_totals[:rank].sum())

    def check_scan(got, label):
        worst, ok = 0.0, True
        picks = sorted({0, len(blocks) // 2, len(blocks) - 1})
        for i in picks:
            first, m, before = blocks[i]
            v = oracle.c_fill_f16(m, 3, b + first, "uniform_01").view(np.float16).astype(np.float64)
            ref = np.cumsum(v) + (ref_carry + before)
            bad, max_abs, max_rel = oracle.np_check_f32(got[first:first + m].cpu().numpy(), ref)
            ok = ok and bad == 0
            worst = max(worst, max_rel)
        return all_ok(ok, worst)

    # kernel-level exchange
    grp.full_reduce(xs[0], out=o32, out_f64=o64)
    torch.cuda.synchronize()
    err4 = all_ok(abs(float(o64[0]) - ref_total) <= 1e-9 * abs(ref_total), abs(float(o64[0]) - ref_total))
    grp.full_scan(xs[0], out=o)
    torch.cuda.synchronize()
    err5 = check_scan(o, "peer")
    ms = max_over_ranks(torch, dist, world, *time_op(torch, lambda: grp.full_reduce(nxt(), out=o32, out_f64=o64), 20))
    res["C4_full_reduce_2^30_total"] = entry(n_total, 2, *ms, one_gpu["C4"], checked=True, abs_err=err4,
                                             exchange="totals stored by the kernels into every rank's memory",
                                             buffer_sets=nbuf)
    ms = max_over_ranks(torch, dist, world, *time_op(torch, lambda: grp.full_scan(nxt(), out=o), 12))
    res["C5_full_scan_2^30_total_f32"] = entry(n_total, 6, *ms, one_gpu["C5"], checked=True, max_rel_err=err5,
                                               exchange="totals stored by the kernels into every rank's memory",
                                               traffic="each shard is read twice: 8 B/elem against 6 algorithmic, "
                                                       "less what the second read finds in L2",
                                               buffer_sets=nbuf)
    # L2 residency of the second read: what the first pass asks L2 to keep
    sweep = {}
    for keep_mib in (0, 32, 96):
        grp.set_l2_keep_bytes(keep_mib << 20)
        m2 = max_over_ranks(torch, dist, world, *time_op(torch, lambda: grp.full_scan(nxt(), out=o), 8))
        sweep[f"{keep_mib}MiB"] = round(n_total / m2[0] / 1e6, 1)
    grp.set_l2_keep_bytes(64 << 20)
    sweep["64MiB"] = res["C5_full_scan_2^30_total_f32"]["gelem_per_s"]
    res["C5_full_scan_2^30_total_f32"]["gelem_per_s_by_l2_keep"] = sweep

    # all-gather variant
    total = tcu.sharded_full_reduce(lambda: local_total(xs[0]))
    torch.cuda.synchronize()
    err4 = all_ok(abs(float(total[0]) - ref_total) <= 1e-9 * abs(ref_total), abs(float(total[0]) - ref_total))
    tcu.sharded_full_scan(lambda: local_total(xs[0]), lambda totals, r: tcu.full_scan(
        xs[0], out=o, workspace=ws, shard_totals=totals, shard_index=r))
    torch.cuda.synchronize()
    err5 = check_scan(o, "all_gather")

    def c4_gather():
        nxt()
        tcu.sharded_full_reduce(local_total)

    def c5_gather():
        x = nxt()
        tcu.sharded_full_scan(local_total, lambda totals, r: tcu.full_scan(
            x, out=o, workspace=ws, shard_totals=totals, shard_index=r))
    ms = max_over_ranks(torch, dist, world, *time_op(torch, c4_gather, 20))
    res["C4_full_reduce_2^30_total_all_gather"] = entry(n_total, 2, *ms, one_gpu["C4"], checked=True, abs_err=err4)
    ms = max_over_ranks(torch, dist, world, *time_op(torch, c5_gather, 12))
    res["C5_full_scan_2^30_total_f32_all_gather"] = entry(n_total, 6, *ms, one_gpu["C5"], checked=True,
                                                          max_rel_err=err5)
    return res


def reference_kernels_leg(torch, tcu, args):
    """Baseline leg, beside the CPU one: the reference's OWN WMMA kernels (compiled unmodified
    for sm_100a into oracle/_ref where the reference checkout was present) timed on this GPU on
    the same sweep.  They accumulate and store fp16 and are not checked here; the tests compare
    them with the oracle on exactly summable inputs.  Returns None when the file is missing."""
    import oracle
    ref = oracle.ref_lib()
    if ref is None:
        return None
    n = 1 << min(args.log2_elems, 28)
    x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 2024, 0)
    stream = torch.cuda.current_stream().cuda_stream
    # the launch shapes the reference's own plots pick (figures/spec/segmented_reduction_16n.yml:30-42,
    # paper_tune_segmented_reduction.yml:36-48, paper_tune_segmented_prefixsum.yml:30-54)
    reduce_shapes = {16: (0, 8), 32: (0, 8), 64: (0, 8), 256: (1, 8), 1024: (1, 8), 16384: (1, 8)}
    scan_shapes = {16: (0, 8), 256: (1, 8), 4096: (1, 4)}
    out = {"reduce_gelem_per_s": {}, "scan_f16_gelem_per_s": {}}
    total_ms = 0.0
    for s, (variant, wpb) in reduce_shapes.items():
        o = torch.empty(n // s, dtype=torch.float16, device="cuda")

        def call():
            rc = ref.tcu_ref_segmented_reduce(x.data_ptr(), o.data_ptr(), n // s, s, variant, wpb, stream)
            assert rc == 0, rc
        ms, _ = time_op(torch, call, 5, 2)
        total_ms += ms
        out["reduce_gelem_per_s"][str(s)] = round(n / ms / 1e6, 1)
    out["sweep_gelem_per_s"] = round(len(reduce_shapes) * n / total_ms / 1e6, 1)
    for s, (variant, wpb) in scan_shapes.items():
        o = torch.empty(n, dtype=torch.float16, device="cuda")

        def call():
            rc = ref.tcu_ref_segmented_scan(x.data_ptr(), o.data_ptr(), n // s, s, variant, wpb, stream)
            assert rc == 0, rc
        ms, _ = time_op(torch, call, 5, 2)
        out["scan_f16_gelem_per_s"][str(s)] = round(n / ms / 1e6, 1)
        del o
    out["note"] = "reference kernels, fp16 accumulate and fp16 outputs, unvalidated at this size"
    return out


def cub_leg(torch, tcu, args):
    """Baseline leg: CUB device-wide primitives (the CUDA toolkit's CCCL) on the same inputs --
    the library comparison the reference itself makes.  None when oracle/libtcu_cub.so is missing."""
    import ctypes
    import oracle
    cub = oracle.cub_lib()
    if cub is None:
        return None
    stream = torch.cuda.current_stream().cuda_stream
    n28 = 1 << min(args.log2_elems, 28)
    n30 = 1 << min(args.log2_elems + 2, 30)
    out = {"unit": "Gelem/s", "seg_reduce_f32": {}, "seg_scan": {}}

    def timed(op, x, o, n, seg, reps):
        need = ctypes.c_size_t(oracle.cub_temp_bytes(op, n, seg))
        tmp = torch.empty(need.value, dtype=torch.uint8, device="cuda")

        def call():
            rc = cub.tcu_cub_run(op, x.data_ptr(), o.data_ptr(), n, seg, tmp.data_ptr(),
                                 ctypes.byref(need), stream)
            assert rc == 0, rc
        ms, _ = time_op(torch, call, reps, 2)
        return round(n / ms / 1e6, 1)

    x = tcu.fill(torch.empty(n28, dtype=torch.float16, device="cuda"), 2024, 0)
    total_ms = 0.0
    for s in SWEEP:
        o = torch.empty(n28 // s, dtype=torch.float32, device="cuda")
        g = timed(oracle.CUB_SEG_REDUCE, x, o, n28, s, 3 if s < 64 else 5)
        out["seg_reduce_f32"][str(s)] = g
        total_ms += n28 / g / 1e6
    out["seg_reduce_sweep"] = round(len(SWEEP) * n28 / total_ms / 1e6, 1)
    o16 = torch.empty(n28, dtype=torch.float16, device="cuda")
    for s in (16, 256):
        out["seg_scan"][f"{s}_f16"] = timed(oracle.CUB_SEG_SCAN_F16, x, o16, n28, s, 5)
    del o16
    o32 = torch.empty(n28, dtype=torch.float32, device="cuda")
    out["seg_scan"]["4096_f32"] = timed(oracle.CUB_SEG_SCAN_F32, x, o32, n28, 4096, 5)
    del o32, x
    x = tcu.fill(torch.empty(n30, dtype=torch.float16, device="cuda"), 3, 0, "uniform_01")
    o1 = torch.empty(1, dtype=torch.float32, device="cuda")
    out["full_reduce"] = timed(oracle.CUB_FULL_REDUCE, x, o1, n30, n30, 5)
    o = torch.empty(n30, dtype=torch.float32, device="cuda")
    out["full_scan_f32"] = timed(oracle.CUB_FULL_SCAN, x, o, n30, n30, 5)
    out["note"] = ("cub::DeviceSegmentedReduce / DeviceScan::InclusiveSumByKey / DeviceReduce / "
                   "DeviceScan, fp16 inputs widened to fp32 by a transform iterator")
    # Thrust, the reference's other comparison set (src/reduction/seg_thrust.cu:50,
    # src/prefixsum/seg_thrust.cu:46, src/reduction/thrust.cu, src/prefixsum/thrust.cu)
    th = {"seg_reduce_f32": {}, "seg_scan_f32": {}}

    def thrust_timed(op, x, o, n, seg, reps):
        def call():
            rc = cub.tcu_thrust_run(op, x.data_ptr(), o.data_ptr(), n, seg, stream)
            assert rc == 0, rc
        ms, _ = time_op(torch, call, reps, 1)
        return round(n / ms / 1e6, 1)
    x = tcu.fill(torch.empty(n28, dtype=torch.float16, device="cuda"), 2024, 0)
    for s in (16, 256, 16384):
        o = torch.empty(n28 // s, dtype=torch.float32, device="cuda")
        th["seg_reduce_f32"][str(s)] = thrust_timed(oracle.THRUST_REDUCE_BY_KEY, x, o, n28, s, 3)
    o32 = torch.empty(n28, dtype=torch.float32, device="cuda")
    for s in (16, 256, 4096):
        th["seg_scan_f32"][str(s)] = thrust_timed(oracle.THRUST_SCAN_BY_KEY, x, o32, n28, s, 3)
    th["full_scan_f32_2^28"] = thrust_timed(oracle.THRUST_SCAN, x, o32, n28, n28, 3)
    th["full_reduce_2^28"] = thrust_timed(oracle.THRUST_REDUCE, x, o32, n28, n28, 3)
    th["note"] = "thrust::reduce_by_key / inclusive_scan_by_key / inclusive_scan / reduce, 2^28 elements"
    out["thrust"] = th
    return out


def adjacent_sizes_leg(torch, tcu, args, peak_gbs):
    """Segment sizes next to the benchmark definition's: multiples of 8 / 16 that are not powers of
    two (the reference's 16n kernels accept the latter) and whole segments longer than 16384
    elements with 16-bit outputs.  Fractions of the measured copy bandwidth."""
    n_max = 1 << min(args.log2_elems, 28)
    xs = [tcu.fill(torch.empty(n_max, dtype=torch.float16, device="cuda"), 77 + i, 0) for i in range(2)]
    k = [0]

    def timed(fn, bytes_moved):
        ms, _ = time_op(torch, fn, 8, 3)
        return round(bytes_moved / ms / 1e6 / peak_gbs, 3)

    out = {"unit": "fraction of the measured copy bandwidth", "reduce_f32": {}, "scan_f32": {},
           "scan_f16": {}, "scan_f16_long_segments": {}}
    for s in (48, 240, 1000, 2000):
        n = n_max // s * s
        o = torch.empty(n // s, dtype=torch.float32, device="cuda")

        def red():
            k[0] += 1
            tcu.segmented_reduce(xs[k[0] % 2][:n], s, out=o)
        out["reduce_f32"][str(s)] = timed(red, n * 2 + n // s * 4)
        if s % 16:
            continue
        for dt, key, width in ((torch.float32, "scan_f32", 4), (torch.float16, "scan_f16", 2)):
            o2 = torch.empty(n, dtype=dt, device="cuda")

            def scan():
                k[0] += 1
                tcu.segmented_scan(xs[k[0] % 2][:n], s, out=o2)
            out[key][str(s)] = timed(scan, n * (2 + width))
            del o2
    o16 = torch.empty(n_max, dtype=torch.float16, device="cuda")
    for lg in (15, 16, 17, 18):
        s = 1 << lg
        if n_max // s < 2:
            continue
        ws = torch.empty(tcu.workspace_bytes(tcu.OP_SEGMENTED_SCAN, n_max, s), dtype=torch.uint8, device="cuda")
        row = {}
        for algo in ("auto", "mma"):  # mma: the single-pass look-back kernel
            def scan():
                k[0] += 1
                tcu.segmented_scan(xs[k[0] % 2], s, out=o16, algo=algo, workspace=ws)
            row[algo] = timed(scan, n_max * 4)
        out["scan_f16_long_segments"][f"2^{lg}"] = row
    return out


def ablation_leg(torch, tcu, args):
    """In-run ablation: the same TMA pipeline with CUDA-core adds and warp shuffles in place of
    the tensor-core contraction (TCU_ALGO_SHUFFLE), on the sweep and on the segmented scans, and
    the tcgen05 / tensor-memory form of the reductions up to 2048 elements (TCU_ALGO_TCGEN05)."""
    n = 1 << min(args.log2_elems, 28)
    xs = [tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 2024 + i, 0) for i in range(2)]
    k = [0]
    out = {"unit": "Gelem/s", "reduce": {}, "scan": {}}
    for algo in ("mma", "shuffle"):
        red, total_ms = {}, 0.0
        for s in SWEEP:
            o = torch.empty(n // s, dtype=torch.float32, device="cuda")

            def call():
                k[0] += 1
                tcu.segmented_reduce(xs[k[0] % 2], s, out=o, algo=algo)
            ms, _ = time_op(torch, call, 10, 3)
            total_ms += ms
            red[str(s)] = round(n / ms / 1e6, 1)
        red["sweep"] = round(len(SWEEP) * n / total_ms / 1e6, 1)
        out["reduce"][algo] = red
        sc = {}
        for s, dt in [(16, torch.float16), (256, torch.float16), (4096, torch.float32)]:
            o = torch.empty(n, dtype=dt, device="cuda")

            def call():
                k[0] += 1
                tcu.segmented_scan(xs[k[0] % 2], s, out=o, algo=algo)
            ms, _ = time_op(torch, call, 10, 3)
            sc[f"{s}_{'f32' if dt == torch.float32 else 'f16'}"] = round(n / ms / 1e6, 1)
            del o
        out["scan"][algo] = sc
    red = {}
    for s in [v for v in SWEEP if v <= 2048]:
        o = torch.empty(n // s, dtype=torch.float32, device="cuda")

        def call():
            k[0] += 1
            tcu.segmented_reduce(xs[k[0] % 2], s, out=o, algo="tcgen05")
        ms, _ = time_op(torch, call, 10, 3)
        red[str(s)] = round(n / ms / 1e6, 1)
    out["reduce"]["tcgen05"] = red
    sc = {}
    for s, dt in [(16, torch.float16), (256, torch.float16), (2048, torch.float16), (16384, torch.float16),
                  (4096, torch.float32)]:
        o = torch.empty(n, dtype=dt, device="cuda")
        for algo in ("mma", "tcgen05"):
            def call():
                k[0] += 1
                tcu.segmented_scan(xs[k[0] % 2], s, out=o, algo=algo)
            ms, _ = time_op(torch, call, 10, 3)
            sc.setdefault(algo, {})[f"{s}_{'f32' if dt == torch.float32 else 'f16'}"] = round(n / ms / 1e6, 1)
        del o
    out["scan_mma_sync_vs_tcgen05"] = sc
    out["note"] = ("direct launches, CUDA events around 10 back-to-back calls; the shuffle variant "
                   "does not split inputs into exact parts (plain fp32 rounding); tcgen05 = "
                   "tcgen05.mma with the accumulator in tensor memory: reductions up to 2048 elements per "
                   "segment with plain fp32 accumulation, scans with the exact parts of the mma.sync path "
                   "(the default for 16-bit outputs of 16- and 256...16384-element segments)")
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

    def step():  # one call: every chunk is uploaded once and reduced at all six segment sizes
        ctx.reduce_sweep(h_in, SWEEP, [h_out[s] for s in SWEEP], algo=args.algo)

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
    h2d = n * 2
    d2h = sum(n // s * 4 for s in SWEEP)
    # spot check: the results that came back are the right ones
    import oracle
    ref = oracle.np_segmented_reduce(h_in[:1 << 20].view(torch.int16).numpy().view(np.uint16), 1024)
    assert np.array_equal(h_out[1024][:1 << 10].numpy(), ref.astype(np.float32))
    res = {"value": steps * len(SWEEP) * n * world / dt / 1e9, "unit": "Gelem/s",
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": steps,
           "h2d_gbytes_per_s_per_rank": round(steps * h2d / dt / 1e9, 1),
           "note": "tcu_host_segmented_reduce_sweep_f16: pinned host buffers, each 64 MiB chunk "
                   "copied once and reduced at all six sizes, copies overlap kernels on two streams"}
    # What ONE segmented reduction of a host array gets (tcu_host_run_f16): every element crosses
    # the bus for a single pass, so the call runs at the host-to-device copy rate.
    single = {}
    for s in (16, 16384):
        def one():
            ctx.run(tcu.OP_SEGMENTED_REDUCE, h_in, h_out[s], s, algo=args.algo)
        one()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(2):
            one()
        d1 = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([d1], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            d1 = float(t[0])
        single[str(s)] = {"gelem_per_s": round(2 * n * world / d1 / 1e9, 2),
                          "h2d_gbytes_per_s_per_rank": round(2 * h2d / d1 / 1e9, 1)}
    res["single_size_calls"] = single
    ctx.close()
    return res


def profile_pass(torch, tcu, args, n, json_fd):
    """One launch of each kernel of a family, for a profiler to capture."""
    x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 2024, 0)
    if args.profile == "reduce":
        for s in (SWEEP if args.algo != "tcgen05" else [v for v in SWEEP if v <= 2048]):
            tcu.segmented_reduce(x, s, algo=args.algo)
    elif args.profile == "scan":
        for s, dt in [(16, torch.float16), (256, torch.float16), (4096, torch.float32)]:
            tcu.segmented_scan(x, s, out_dtype=dt, algo=args.algo)
    elif args.profile == "scan16":  # the classes with 16-bit outputs that stay under 0.90
        for s in (2048, 4096, 16384):
            tcu.segmented_scan(x, s, out_dtype=torch.float16, algo=args.algo)
    elif args.profile == "scan32":  # the fp32-output classes under 0.90, and their neighbours
        for s in (16, 32, 64, 128):
            tcu.segmented_scan(x, s, out_dtype=torch.float32, algo=args.algo)
    elif args.profile == "general":  # a segment size that is a multiple of 16 but no power of two
        x = x[:n // 48 * 48]
        tcu.segmented_reduce(x, 48)
        tcu.segmented_scan(x, 48, out_dtype=torch.float32)
        tcu.segmented_scan(x, 48, out_dtype=torch.float16)
    elif args.profile == "shard":  # the two passes of the sharded full scan, one rank
        tcu.fill(x, 2024, 0, "uniform_01")
        grp = tcu.PeerGroup()
        o = torch.empty(n, dtype=torch.float32, device="cuda")
        grp.full_scan(x, out=o)          # pass 1 asks L2 to keep 64 MiB for pass 2
        grp.set_l2_keep_bytes(0)
        grp.full_scan(x, out=o)          # ... and nothing
        torch.cuda.synchronize()
        grp.close()
    else:
        tcu.fill(x, 2024, 0, "uniform_01")
        tcu.full_reduce(x)
        tcu.full_scan(x, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert tcu.device_error() == 0
    emit(json_fd, {"profile": args.profile, "log2_elems": args.log2_elems, "algo": args.algo})


def main():
    args = parse_args()
    # Libraries (NCCL's version banner, for one) write to stdout; the contract is ONE JSON line
    # there.  Everything else goes to stderr: fd 1 is pointed at fd 2 for the run and the result
    # is written to the saved descriptor at the end.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    try:
        _main(args, json_fd)
    finally:
        sys.stdout.flush()
        os.dup2(json_fd, 1)
        os.close(json_fd)


def emit(json_fd: int, obj) -> None:
    os.write(json_fd, (json.dumps(obj) + "\n").encode())


def _main(args, json_fd):
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, json_fd)
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
        profile_pass(torch, tcu, args, n, json_fd)
        return

    # this rank's shard of the logical array: elements [rank*n, (rank+1)*n), two buffers to rotate
    xs = [tcu.fill(torch.empty(n, dtype=torch.float16, device=dev), 2024 + i, rank * n) for i in range(2)]
    outs = {s: torch.empty(n // s, dtype=torch.float32, device=dev) for s in SWEEP}
    counter = [0]

    def launch(s):
        x = xs[counter[0] % 2]  # consecutive launches alternate between the two input buffers
        counter[0] += 1
        tcu.segmented_reduce(x, s, out=outs[s], algo=args.algo)

    def step():
        for s in SWEEP:
            launch(s)

    def capture(fn):
        """fn() captured into one CUDA graph (every launch goes through the C ABI on the
        capturing stream); None if capture is not possible."""
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(g, stream=side):
                    fn()
            torch.cuda.current_stream().wait_stream(side)
            g.replay()
            torch.cuda.synchronize()
            return g
        except Exception as e:  # keep measuring, say why
            print(f"warning: CUDA graph capture failed ({e}); timing direct launches", file=sys.stderr)
            return None

    step()  # first call of every kernel: one-time function attributes, before any capture
    torch.cuda.synchronize()
    step_graph = capture(step)  # six launches; an even count, so replays keep alternating buffers
    run_step = step_graph.replay if step_graph is not None else step

    for _ in range(max(args.warmup, 0)):
        run_step()
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    t_begin.record()
    for k in range(args.steps):
        run_step()
    t_end.record()
    if sampler:
        sampler.wait_for(t_end)
    torch.cuda.synchronize()
    clocks = sampler.result() if sampler else None
    if world > 1:
        dist.barrier()
    total_ms = t_begin.elapsed_time(t_end)
    if world > 1:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t[0])
    assert tcu.device_error() == 0, "a bounded device-side wait ran out"
    value = args.steps * len(SWEEP) * n * world / (total_ms * 1e-3) / 1e9

    # Per-kernel durations: every size on its own, six back-to-back launches per graph replay,
    # CUDA events around `steps` replays on the launching stream.
    per_size = {}
    for s in SWEEP:
        g = capture(lambda: [launch(s) for _ in range(6)])
        fn = g.replay if g is not None else (lambda: [launch(s) for _ in range(6)])
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn()
        torch.cuda.synchronize()
        a.record()
        for _ in range(max(args.steps, 1)):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / (6 * max(args.steps, 1))
        bpe = 2 + 4 / s
        per_size[str(s)] = {"ms": round(ms, 4), "gelem_per_s": round(n / ms / 1e6, 1),
                            "gbytes_per_s": round(n * bpe / ms / 1e6, 1),
                            "hbm_frac": round(n * bpe / ms / 1e6 / peak_gbs, 4),
                            "hbm_frac_of_nominal_8tbs": round(n * bpe / ms / 1e6 / NOMINAL_HBM_GBS, 4)}

    # dominant kernel: the 16-element launch moves the most bytes (2 + 4/16 per element)
    dom = per_size["16"]
    traffic, traffic_source = ncu_traffic(n)
    roofline = {"bound": "hbm", "kernel": "seg_reduce_kernel<4> (segment size 16)",
                "achieved": dom["gbytes_per_s"], "peak": peak_gbs, "unit": "GB/s",
                "frac": dom["hbm_frac"], "peak_source": f"of {peak_kind}",
                "frac_of_nominal_8tbs": dom["hbm_frac_of_nominal_8tbs"],
                "algorithmic_bytes_per_launch": int(n * 2.25),
                "timing": "back-to-back launches of this kernel (6 per graph replay), CUDA events",
                "traffic": traffic, "traffic_source": traffic_source}

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
        result["other_configs"] = extras(torch, tcu, dist, args, rank, world, peak_gbs, value / world)
        if rank == 0 and world == 1:
            v, cores, passes, secs = cpu_sweep(26, 8.0, 2000)
            result["cpu_baseline"] = {
                "value": round(v, 3), "unit": "Gelem/s", "cores": cores, "kind": "port",
                "sample": f"{passes} passes of the 6-size sweep over 2^26 elements ({secs:.1f} s)"}
            rk = reference_kernels_leg(torch, tcu, args)
            if rk is not None:
                result["reference_kernels_on_this_gpu"] = rk
            cb = cub_leg(torch, tcu, args)
            if cb is not None:
                result["cub_on_this_gpu"] = cb
            result["ablation_tensor_core_vs_shuffle"] = ablation_leg(torch, tcu, args)
            result["adjacent_sizes"] = adjacent_sizes_leg(torch, tcu, args, peak_gbs)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        emit(json_fd, result)


if __name__ == "__main__":
    main()
