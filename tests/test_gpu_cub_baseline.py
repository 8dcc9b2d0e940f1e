"""The CUB library baseline (oracle/libtcu_cub.so) computes the same operations: checked against
the oracle at a small size so that its timings in bench.py compare like with like."""
import ctypes

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def test_cub_baseline_matches_oracle():
    cub = oracle.cub_lib()
    if cub is None:
        pytest.skip("oracle/libtcu_cub.so not built")
    import tcu_scope_b200 as tcu
    n, s = 1 << 20, 256
    x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 61, 0, "uniform_pm1")
    xb = x.cpu().view(torch.int16).numpy().view(np.uint16)
    st = torch.cuda.current_stream().cuda_stream

    def run(op, out, seg):
        need = ctypes.c_size_t(oracle.cub_temp_bytes(op, n, seg))
        tmp = torch.empty(need.value, dtype=torch.uint8, device="cuda")
        assert cub.tcu_cub_run(op, x.data_ptr(), out.data_ptr(), n, seg, tmp.data_ptr(),
                               ctypes.byref(need), st) == 0
        torch.cuda.synchronize()
        return out

    tot = run(oracle.CUB_FULL_REDUCE, torch.empty(1, dtype=torch.float32, device="cuda"), n)
    assert oracle.np_check_f32(tot.cpu().numpy(), oracle.np_segmented_reduce(xb, n), 1e-3, 1e-3)[0] == 0
    red = run(oracle.CUB_SEG_REDUCE, torch.empty(n // s, dtype=torch.float32, device="cuda"), s)
    assert oracle.np_check_f32(red.cpu().numpy(), oracle.np_segmented_reduce(xb, s), 1e-3, 1e-4)[0] == 0
    sc = run(oracle.CUB_SEG_SCAN_F32, torch.empty(n, dtype=torch.float32, device="cuda"), s)
    assert oracle.np_check_f32(sc.cpu().numpy(), oracle.np_segmented_scan(xb, s), 1e-3, 1e-4)[0] == 0
    fs = run(oracle.CUB_FULL_SCAN, torch.empty(n, dtype=torch.float32, device="cuda"), n)
    assert oracle.np_check_f32(fs.cpu().numpy(), oracle.np_segmented_scan(xb, n), 1e-3, 1e-2)[0] == 0


def test_thrust_baseline_matches_oracle():
    cub = oracle.cub_lib()
    if cub is None:
        pytest.skip("oracle/libtcu_cub.so not built")
    import tcu_scope_b200 as tcu
    n, s = 1 << 20, 256
    x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 62, 0, "uniform_pm1")
    xb = x.cpu().view(torch.int16).numpy().view(np.uint16)
    st = torch.cuda.current_stream().cuda_stream

    def run(op, out, seg):
        assert cub.tcu_thrust_run(op, x.data_ptr(), out.data_ptr(), n, seg, st) == 0
        torch.cuda.synchronize()
        return out

    tot = run(oracle.THRUST_REDUCE, torch.empty(1, dtype=torch.float32, device="cuda"), n)
    assert oracle.np_check_f32(tot.cpu().numpy(), oracle.np_segmented_reduce(xb, n), 1e-3, 1e-3)[0] == 0
    red = run(oracle.THRUST_REDUCE_BY_KEY, torch.empty(n // s, dtype=torch.float32, device="cuda"), s)
    assert oracle.np_check_f32(red.cpu().numpy(), oracle.np_segmented_reduce(xb, s), 1e-3, 1e-4)[0] == 0
    sc = run(oracle.THRUST_SCAN_BY_KEY, torch.empty(n, dtype=torch.float32, device="cuda"), s)
    assert oracle.np_check_f32(sc.cpu().numpy(), oracle.np_segmented_scan(xb, s), 1e-3, 1e-4)[0] == 0
    fs = run(oracle.THRUST_SCAN, torch.empty(n, dtype=torch.float32, device="cuda"), n)
    assert oracle.np_check_f32(fs.cpu().numpy(), oracle.np_segmented_scan(xb, n), 1e-3, 1e-2)[0] == 0
