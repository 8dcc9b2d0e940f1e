"""GPU test of tcu_full_scan_f16_static, the entry point for callers that may
not allocate device memory (a plugin given only its input and output buffers,
a latency-bound service loop): it must give what tcu_full_scan_f16 gives with
a caller-made workspace, call after call, although all calls share one built-in
scratch array that still holds the previous call's contents.

Collected last on purpose (file name), so that a run which stops at the first
failure has already run every other test.  Passes alone in a fresh process and
after the rest of the suite.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

OUT_F32 = 1
TOO_LARGE = 6


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_static_scratch_scan_matches_workspace_scan_twice_in_a_row():
    import tcu_scope_b200 as tcu
    lib = tcu._lib.load()
    # first a long input, then a shorter one with other data: the second call
    # finds the first call's tile states in the shared scratch and must clear them
    for n, seed in [((1 << 22) + 16 * 37, 5), (1 << 20, 6), (1 << 20, 7)]:
        x = torch.empty(n, dtype=torch.float16, device="cuda")
        tcu.fill(x, seed, 0, "uniform_01")
        want = tcu.full_scan(x, out_dtype=torch.float32)  # existing entry point, own workspace
        got = torch.empty(n, dtype=torch.float32, device="cuda")
        st = lib.tcu_full_scan_f16_static(x.data_ptr(), got.data_ptr(), OUT_F32, n, None, 0, 0,
                                          _stream())
        assert st == 0, lib.tcu_status_string(st)
        torch.cuda.synchronize()
        xb = x.cpu().view(torch.int16).numpy().view(np.uint16)
        ref = oracle.c_segmented_scan(xb, n)
        # same tolerance as the other fp32 scan tests: 1e-3 relative, 1e-5 absolute floor
        for name, t in (("static", got), ("workspace", want)):
            bad, max_abs, _ = oracle.np_check_f32(t.cpu().numpy(), ref, 1e-3, 1e-5)
            assert bad == 0, f"{name}: {bad} outputs out of tolerance (max abs err {max_abs})"
        bad, max_abs, _ = oracle.np_check_f32(got.cpu().numpy(), want.double().cpu().numpy(), 1e-3, 1e-5)
        assert bad == 0, f"static vs workspace entry point differ (max abs {max_abs})"
    assert tcu.device_error() == 0


def test_static_scratch_scan_rejects_oversize_input():
    import tcu_scope_b200 as tcu
    lib = tcu._lib.load()
    x = torch.zeros(16, dtype=torch.float16, device="cuda")
    out = torch.zeros(16, dtype=torch.float32, device="cuda")
    too_many = (1 << 30) + 16  # refused before anything is read or launched
    st = lib.tcu_full_scan_f16_static(x.data_ptr(), out.data_ptr(), OUT_F32, too_many, None, 0, 0,
                                      _stream())
    assert st == TOO_LARGE
    assert b"scratch" in lib.tcu_status_string(st)
    torch.cuda.synchronize()
    assert torch.all(out == 0)
