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
# dram__bytes_read.sum + dram__bytes_write.sum of one seg_reduce_kernel<4> launch: captured by
# ncu at 2^27 elements (268.461 MB read + 25.693 MB written; the capture is summarised under profiles/)
# and doubled for the 2^28-element launch of this benchmark (traffic grows with the element count).
NCU_TRAFFIC_BYTES_S16 = 2 * (268_460_800 + 25_693_440)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--algo", default="auto", choices=["auto", "mma", "shuffle", "tcgen05"],
                    help="tcgen05 only exists for segment sizes up to 2048: use it with --profile reduce")
    ap.add_argument("--log2-elems", type=int, default=LOG2_ELEMS,
                    help="elements per GPU (default 28, the reference sweep's size)")
    ap.add_argument("--profile", default=None, choices=["reduce", "scan", "full"],
                    help="run ONE untimed pass of the named kernels at --log2-elems and exit "
                         "(the small case an ncu capture wraps)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the other configurations, the e2e leg and the CPU baseline")
    args = ap.parse_args()
    if args.algo == "tcgen05" and args.profile != "reduce":
        ap.error("--algo tcgen05 covers segment sizes up to 2048 only: use it with --profile reduce "
                 "(the timed sweep reports it under ablation_tensor_core_vs_shuffle)")
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
    emit(json_fd, {
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


def extras(torch, tcu, dist, args, rank, world, peak_gbs):
    """The other configurations of the benchmark definition, a few repetitions each."""
    out = {}
    dev = torch.device("cuda")
    n28 = 1 << min(args.log2_elems, 28)

    def gelem(n, ms):
        return n / (ms * 1e-3) / 1e9

    def entry(n, bytes_per_elem, ms_med, ms_min, gpus=1):
        g = gelem(n, ms_med)  # n = elements over all `gpus` GPUs; hbm_frac is per GPU
        return {"gelem_per_s": round(g, 1), "gelem_per_s_best": round(gelem(n, ms_min), 1),
                "gbytes_per_s": round(g * bytes_per_elem, 1),
                "hbm_frac": round(g * bytes_per_elem / peak_gbs / gpus, 4), "ms": round(ms_med, 4)}

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
    out["C1_seg_reduce_2^24_S16_cold"]["timing"] = "16 launches per CUDA graph, 8 rotating buffer sets"
    # context for a launch this short: a plain device-to-device copy moving the same 37.7 MB
    # (half read, half written), timed the same way -- what the box gives ANY kernel of this size
    half = n24 * 9 // 16  # halves: 2 B read + 2 B written each = 2.25 B x 2^24
    dsts = [torch.empty(half, dtype=torch.float16, device=dev) for _ in range(8)]

    def copy_same_bytes():
        i = k[0] % 8
        k[0] += 1
        dsts[i].copy_(xs[(i + 3) % 8][:half])
    c1_entry = out["C1_seg_reduce_2^24_S16_cold"]
    try:
        ms_copy, _ = time_graph(torch, copy_same_bytes, 16, 10)
        c1_entry["copy_of_same_bytes_ms"] = round(ms_copy, 4)
        c1_entry["frac_of_copy_at_this_size"] = round(ms_copy / c1_entry["ms"], 3)
    except RuntimeError as e:  # context only: never fail the run for it
        c1_entry["copy_of_same_bytes_ms"] = None
        print(f"copy context skipped: {e}", file=sys.stderr)
    del xs, os_, dsts

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
        if world == 1:
            local_total()  # one GPU: the kernel's own total is the result
        else:
            tcu.sharded_full_reduce(local_total)
    ms_med, ms_min = time_op(torch, c4, 10)
    if world > 1:
        t = torch.tensor([ms_med, ms_min], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_med, ms_min = t.tolist()
    out["C4_full_reduce_2^30_per_gpu"] = entry(n30 * world, 2, ms_med, ms_min, world)

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
    out["C5_full_scan_2^30_per_gpu_f32"] = entry(n30 * world, 6, ms_med, ms_min, world)
    return out


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
    out["note"] = ("direct launches, CUDA events around 10 back-to-back calls; the shuffle variant "
                   "does not split inputs into exact parts (plain fp32 rounding); tcgen05 = "
                   "tcgen05.mma with the accumulator in tensor memory, segment sizes up to 2048 (plain fp32 "
                   "accumulation, no exact parts)")
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
    ctx.close()
    h2d = n * 2
    d2h = sum(n // s * 4 for s in SWEEP)
    # spot check: the results that came back are the right ones
    import oracle
    ref = oracle.np_segmented_reduce(h_in[:1 << 20].view(torch.int16).numpy().view(np.uint16), 1024)
    assert np.array_equal(h_out[1024][:1 << 10].numpy(), ref.astype(np.float32))
    return {"value": steps * len(SWEEP) * n * world / dt / 1e9, "unit": "Gelem/s",
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": steps,
            "note": "tcu_host_segmented_reduce_sweep_f16: pinned host buffers, each 64 MiB chunk "
                    "copied once and reduced at all six sizes, copies overlap kernels on two streams"}


def profile_pass(torch, tcu, args, n, json_fd):
    """One launch of each kernel of a family, for a profiler to capture."""
    x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 2024, 0)
    if args.profile == "reduce":
        for s in (SWEEP if args.algo != "tcgen05" else [v for v in SWEEP if v <= 2048]):
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
                            "hbm_frac": round(n * bpe / ms / 1e6 / peak_gbs, 4)}

    # dominant kernel: the 16-element launch moves the most bytes (2 + 4/16 per element)
    dom = per_size["16"]
    roofline = {"bound": "hbm", "kernel": "seg_reduce_kernel<4> (segment size 16)",
                "achieved": dom["gbytes_per_s"], "peak": peak_gbs, "unit": "GB/s",
                "frac": dom["hbm_frac"], "peak_source": f"of {peak_kind}",
                "algorithmic_bytes_per_launch": int(n * 2.25),
                "timing": "back-to-back launches of this kernel (6 per graph replay), CUDA events",
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
            rk = reference_kernels_leg(torch, tcu, args)
            if rk is not None:
                result["reference_kernels_on_this_gpu"] = rk
            cb = cub_leg(torch, tcu, args)
            if cb is not None:
                result["cub_on_this_gpu"] = cb
            result["ablation_tensor_core_vs_shuffle"] = ablation_leg(torch, tcu, args)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        emit(json_fd, result)


if __name__ == "__main__":
    main()
