"""Every device-side wait of the library is bounded; these tests make three of
them run out -- an mbarrier that is never armed, a look-back on a status word
nobody publishes, a total another rank never sends -- with the limits
shortened to about a millisecond, and check that the call returns, that
tcu_device_error names the wait, and that the next ordinary call is correct.
Nothing here faults, traps or spins without a bound."""
import ctypes

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

BARRIER, LOOKBACK, PEER = 1, 2, 4
SKIP_TILE_LOAD, LOOKBACK_TICKET = 1, 2
TIMEOUT = 4


def bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


@pytest.fixture()
def lib():
    import tcu_scope_b200 as tcu
    lib = tcu._lib.load()
    assert tcu.device_error() == 0
    yield lib
    lib.tcu_test_inject(0, 0)
    assert lib.tcu_test_set_wait_limits(0, 0, 0, 0) == 0  # defaults back for every later test
    tcu.device_error()


def error_bits(lib, clear=1):
    b = ctypes.c_uint(0)
    status = lib.tcu_device_error(ctypes.byref(b), clear)
    return status, b.value


def test_unarmed_barrier_runs_out_and_the_kernel_returns(lib):
    import tcu_scope_b200 as tcu
    n = 64 * 16384
    x = torch.empty(n, dtype=torch.float16, device="cuda")
    tcu.fill(x, 3, 0)
    ref = oracle.c_segmented_reduce(bits(x), 256)
    assert lib.tcu_test_set_wait_limits(3000, 0, 0, 0) == 0  # ~3 ms instead of ~2 s
    assert lib.tcu_test_inject(SKIP_TILE_LOAD, 5) == 0       # tile 5 is never loaded
    out = tcu.segmented_reduce(x, 256)                       # returns: the wait gave up
    status, b = error_bits(lib)
    assert status == TIMEOUT and (b & BARRIER), (status, b)
    assert error_bits(lib) == (0, 0)                         # cleared
    # the stall was one-shot: the same call is now right, also with the short limit in place
    out = tcu.segmented_reduce(x, 256)
    assert np.array_equal(out.cpu().numpy(), ref.astype(np.float32))
    assert error_bits(lib) == (0, 0)
    # full reduction (the long class shares the producer)
    assert lib.tcu_test_inject(SKIP_TILE_LOAD, 0) == 0
    tcu.full_reduce(x)
    status, b = error_bits(lib)
    assert status == TIMEOUT and (b & BARRIER)
    assert tcu.full_reduce(x)[1].cpu().numpy()[0] == oracle.c_segmented_reduce(bits(x), n)[0]
    assert error_bits(lib) == (0, 0)


def test_lookback_on_a_tile_nobody_scans_runs_out(lib):
    import tcu_scope_b200 as tcu
    n = 40 * 16384  # more than one block of 32 tiles
    x = torch.empty(n, dtype=torch.float16, device="cuda")
    tcu.fill(x, 4, 0, "uniform_01")
    assert lib.tcu_test_set_wait_limits(0, 1500, 0, 0) == 0  # ~0.4 ms of polls
    assert lib.tcu_test_inject(LOOKBACK_TICKET, 1) == 0      # tile 0 is never handed out
    tcu.full_scan(x)
    status, b = error_bits(lib)
    assert status == TIMEOUT and b == LOOKBACK, (status, b)
    got = tcu.full_scan(x)
    assert oracle.np_check_f32(got.cpu().numpy(), oracle.c_segmented_scan(bits(x), n))[0] == 0
    assert error_bits(lib) == (0, 0)
    assert lib.tcu_test_inject(LOOKBACK_TICKET, 0) == 1      # tickets start at 1..255
    assert lib.tcu_test_inject(77, 0) == 2


def test_a_total_that_never_arrives_runs_out(lib):
    import tcu_scope_b200 as tcu
    n = 1 << 18
    x = torch.empty(n, dtype=torch.float16, device="cuda")
    tcu.fill(x, 5, 0, "uniform_01")
    out = torch.zeros(n, dtype=torch.float32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def group():
        ctx = (ctypes.c_void_p * 2)()
        for r in range(2):
            c = ctypes.c_void_p()
            assert lib.tcu_mgpu_ctx_create(ctypes.byref(c), r, 2, None) == 0
            ctx[r] = c
        for r in range(2):
            assert lib.tcu_mgpu_ctx_connect_local(ctx[r], ctx) == 0
        return ctx

    ctx = group()
    assert lib.tcu_test_set_wait_limits(0, 0, 0, 3000) == 0  # ~1 ms of polls
    # rank 1 scans its half; rank 0 never makes the matching call
    assert lib.tcu_mgpu_full_scan_f16(ctx[1], x.data_ptr() + n, out.data_ptr() + 2 * n, 1, n // 2,
                                      stream) == 0
    status, b = error_bits(lib)
    assert status == TIMEOUT and b == PEER, (status, b)
    for r in range(2):
        lib.tcu_mgpu_ctx_destroy(ctx[r])
    # a group that timed out is out of step: a fresh one works
    ctx = group()
    for r in range(2):
        assert lib.tcu_mgpu_full_scan_f16(ctx[r], x.data_ptr() + r * n, out.data_ptr() + 2 * r * n, 1,
                                          n // 2, stream) == 0
    assert error_bits(lib) == (0, 0)
    assert oracle.np_check_f32(out.cpu().numpy(), oracle.c_segmented_scan(bits(x), n))[0] == 0
    for r in range(2):
        lib.tcu_mgpu_ctx_destroy(ctx[r])
