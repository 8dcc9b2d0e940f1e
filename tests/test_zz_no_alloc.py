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


def test_static_scratch_scan_allocates_nothing_and_takes_a_seed():
    """Free device memory is the same before and after the calls (the scratch is part of the
    library's device image, not an allocation), and the multi-GPU seed -- the totals of the
    earlier shards -- goes through this entry point as it does through tcu_full_scan_f16."""
    import tcu_scope_b200 as tcu
    lib = tcu._lib.load()
    n = (1 << 21) + 16 * 5
    x = torch.empty(n, dtype=torch.float16, device="cuda")
    tcu.fill(x, 8, 0, "uniform_01")
    got = torch.empty(n, dtype=torch.float32, device="cuda")
    totals = torch.tensor([1000.5, 250.25, 7.0], dtype=torch.float64, device="cuda")
    want = tcu.full_scan(x, out_dtype=torch.float32, shard_totals=totals, shard_index=2)
    # first call on this device (if no other test made it) does the one-time address look-up
    assert lib.tcu_full_scan_f16_static(x.data_ptr(), got.data_ptr(), OUT_F32, n, totals.data_ptr(), 2,
                                        0, _stream()) == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert lib.tcu_full_scan_f16_static(x.data_ptr(), got.data_ptr(), OUT_F32, n,
                                            totals.data_ptr(), 2, 0, _stream()) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the call changed the amount of free device memory"
    assert torch.equal(got, want)
    xb = x.cpu().view(torch.int16).numpy().view(np.uint16)
    ref = oracle.c_segmented_scan(xb, n) + 1250.75  # the two earlier shards
    assert oracle.np_check_f32(got.cpu().numpy(), ref, 1e-3, 1e-5)[0] == 0
    assert tcu.device_error() == 0


def test_static_scratch_scan_at_its_size_limit():
    """2^30 elements is the largest input the built-in scratch is sized for: accepted, and equal
    to the scan with a caller-made workspace."""
    import tcu_scope_b200 as tcu
    lib = tcu._lib.load()
    n = 1 << 30
    free, _ = torch.cuda.mem_get_info()
    if free < 12 * (1 << 30):
        pytest.skip("needs 12 GiB of free device memory")
    x = torch.empty(n, dtype=torch.float16, device="cuda")
    tcu.fill(x, 9, 0, "uniform_01")
    got = torch.empty(n, dtype=torch.float32, device="cuda")
    assert lib.tcu_full_scan_f16_static(x.data_ptr(), got.data_ptr(), OUT_F32, n, None, 0, 0,
                                        _stream()) == 0
    want = tcu.full_scan(x, out_dtype=torch.float32)
    # The look-back adds tile aggregates in the order they become available; at 2^29 and beyond a
    # prefix no longer fits a double exactly, so two runs may round a handful of the 2^30 outputs
    # to neighbouring floats: compare to one float32 ulp (the tests' tolerance is 1e-3 relative).
    want.sub_(got).abs_()
    want.div_(got.abs().clamp_(min=1.0))
    assert float(want.max()) <= 1.2e-7
    del want
    tail = got[-(1 << 16):].cpu().numpy()
    assert np.all(np.diff(tail) >= 0) and abs(tail[-1] / (n / 2) - 1) < 1e-3  # mean of [0,1) inputs
    assert tcu.device_error() == 0
