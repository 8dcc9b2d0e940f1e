"""The C++ benchmark runner keeps the reference's benchmark names and JSON fields."""
import json
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "tcu_scope_b200", "tcu_bench")


@pytest.fixture(scope="module")
def bench_binary(built_library):
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "tcu_scope_b200_build", os.path.join(ROOT, "tcu_scope_b200", "build.py"))
    build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build)
    return build.build_bench()


def list_names(binary, flt):
    out = subprocess.run([binary, "--benchmark_list_tests", f"--benchmark_filter={flt}"],
                         check=True, capture_output=True, text=True).stdout
    return out.strip().splitlines()


def test_registered_names_match_the_reference_format(bench_binary):
    # the regexes of the reference's plot specs (figures/spec/segmented_reduction_16n.yml:30,
    # full_reduction_ker2.yml:89, segmented_prefixsum_256n.yml) select what they should
    names = list_names(bench_binary, r"^CUDA_WMMA_SEGMENTED_REDUCTION_16N<8>.*/segment_size:16/.*")
    assert len(names) == 19  # 2^12 .. 2^30 elements (src/reduction/args.hpp:39-40)
    assert ("CUDA_WMMA_SEGMENTED_REDUCTION_16N<8>/num_segments:1048576/segment_size:16/"
            "num_elements:16777216/manual_time") in names
    names = list_names(bench_binary, r"^CUDA_WMMA_FULL_REDUCTION_2KERS_BLOCK_BASE_256<64 \* 256, 8>.*")
    assert "CUDA_WMMA_FULL_REDUCTION_2KERS_BLOCK_BASE_256<64 * 256, 8>/num_elements:1073741824/manual_time" in names
    names = list_names(bench_binary, r"^CUDA_WMMA_SEGMENTED_PREFIXSUM_256N<8>.*/segment_size:4096/.*")
    assert any("/num_elements:268435456/" in n for n in names)
    names = list_names(bench_binary, r"^CUDA_WMMA_FULL_PREFIXSUM_3KERS<4 \* 256, 8>")
    assert names and all(re.match(r".*/num_elements:\d+/manual_time$", n) for n in names)
    names = list_names(bench_binary, r"^CUDA_WMMA_TUNE_SEGMENTED_REDUCTION_16N<1>/")
    assert len(names) == 27  # segment size 16 .. 2^30 at 2^30 elements (Tuning16_x_30)
    for fam in ("CUDA_WMMA_SEGMENTED_REDUCTION_256N_BLOCK", "CUDA_WMMA_SEGMENTED_PREFIXSUM_16N",
                "CUDA_WMMA_TUNE_SEGMENTED_PREFIXSUM_256N", "CUDA_WMMA_FULL_REDUCTION_2KERS_BASE_16",
                "CUDA_WMMA_FULL_PREFIXSUM_3KERS_BLOCK"):
        assert list_names(bench_binary, "^" + fam + "<"), fam


def test_unsafe_names_are_registered_like_the_safe_ones(bench_binary):
    # src/unsafe_reduction/seg_wmma_16n.cu:183-229, src/unsafe_prefixsum/seg_wmma_16n.cu:188-194 and
    # siblings register the same sweeps under CUDA_UNSAFE_WMMA_*
    safe = list_names(bench_binary, r"^CUDA_WMMA_")
    unsafe = list_names(bench_binary, r"^CUDA_UNSAFE_WMMA")
    assert len(safe) == len(unsafe) > 10000
    renamed = {n.replace("CUDA_WMMA_", "CUDA_UNSAFE_WMMA_", 1) for n in safe}
    # the unsafe tree spells two families without the underscore (src/unsafe_reduction/wmma_atomic.cu:166,172)
    renamed = {n.replace("CUDA_UNSAFE_WMMA_FULL_REDUCTION_ATOMIC", "CUDA_UNSAFE_WMMAFULL_REDUCTION_ATOMIC")
               for n in renamed}
    assert renamed == set(unsafe)
    assert ("CUDA_UNSAFE_WMMA_TUNE_SEGMENTED_REDUCTION_16N<16>/num_segments:67108864/segment_size:16/"
            "base_segment_size:16/max_elements_log2:30/manual_time") in unsafe


@pytest.mark.gpu
def test_runner_output_has_the_reference_schema(bench_binary, tmp_path):
    out = tmp_path / "r.json"
    flt = (r"^CUDA_WMMA_(SEGMENTED_REDUCTION_16N<8>.*segment_size:16/num_elements:(4096|16777216)/|"
           r"SEGMENTED_PREFIXSUM_256N<8>.*segment_size:4096/num_elements:1048576/|"
           r"FULL_REDUCTION_2KERS_BASE_256<256, 8>/num_elements:1048576/|"
           r"FULL_PREFIXSUM_3KERS<256, 8>/num_elements:4194304/|"
           r"TUNE_SEGMENTED_REDUCTION_256N<8>/num_segments:2/.*max_elements_log2:22)")
    subprocess.run([BENCH, f"--benchmark_filter={flt}", f"--benchmark_out={out}",
                    "--benchmark_out_format=json", "--benchmark_min_time=0.02", "--validate"],
                   check=True, capture_output=True, text=True)
    j = json.loads(out.read_text())
    assert len(j["benchmarks"]) == 6
    for b in j["benchmarks"]:
        assert not b.get("error_occurred", False), b
        # the fields tools/plot.py and the reference's counters use
        for field in ("name", "iterations", "real_time", "cpu_time", "time_unit", "flops",
                      "num_elements", "num_segments", "segment_size", "warps_per_block"):
            assert field in b, field
        assert b["flops"] > 0 and b["time_unit"] == "ns"
        # "flops" is elements per second: consistent with the manual time
        assert b["flops"] == pytest.approx(b["num_elements"] / (b["real_time"] * 1e-9), rel=1e-3)
        assert "inert" in b["label"]  # what the template arguments in the name mean here


@pytest.mark.gpu
def test_runner_on_several_gpus(bench_binary, tmp_path):
    import torch
    gpus = torch.cuda.device_count()
    if gpus < 2:
        pytest.skip("needs two or more GPUs")
    out = tmp_path / "m.json"
    flt = (r"^CUDA_(UNSAFE_)?WMMA_(SEGMENTED_REDUCTION_256N<8>.*segment_size:1024/num_elements:4194304/|"
           r"SEGMENTED_PREFIXSUM_16N<8>.*segment_size:64/num_elements:4194304/|"
           r"FULL_REDUCTION_2KERS_BASE_256<256, 8>/num_elements:16777216/|"
           r"FULL_PREFIXSUM_3KERS<256, 8>/num_elements:16777216/)")
    g = min(gpus, 4)
    subprocess.run([BENCH, f"--benchmark_filter={flt}", f"--benchmark_out={out}", f"--num_gpus={g}",
                    "--benchmark_min_time=0.02", "--validate"], check=True, capture_output=True, text=True)
    j = json.loads(out.read_text())
    assert len(j["benchmarks"]) == 8
    for b in j["benchmarks"]:
        assert not b.get("error_occurred", False), b
        assert b["num_gpus"] == g and b["flops"] > 0
