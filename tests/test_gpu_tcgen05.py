"""The tcgen05 / tensor-memory variant of the segmented reduction (TCU_ALGO_TCGEN05, segments of 16 ... 2048)
against the oracle and against the mma.sync path."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


@pytest.mark.parametrize("s", [16, 32, 64, 128, 256, 512, 1024, 2048])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
def test_tcgen05_reduce_matches_oracle(s, out_dtype):
    import tcu_scope_b200 as tcu
    # one row, a partial tile, whole tiles, many tiles per SM (ring and accumulators wrap)
    for n in (64, 64 * 37, 8192, 8192 * 5 + 64 * 3, 1 << 20, (1 << 25) + 64 * 11):
        n = max(s, n // s * s)  # whole segments (and still whole 64-element rows)
        x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 70 + s, 0)
        buf = torch.full((n // s + 128,), -777.0, dtype=out_dtype, device="cuda")
        out = buf[64:64 + n // s]
        tcu.segmented_reduce(x, s, out=out, algo="tcgen05")
        ref = oracle.c_segmented_reduce(bits(x), s)
        if out_dtype == torch.float32:
            bad, max_abs, _ = oracle.np_check_f32(out.cpu().numpy(), ref, 1e-3, 1e-5)
            assert bad == 0, (n, max_abs)
        else:
            assert oracle.np_check_f16(bits(out), ref, 2)[0] == 0
        guards = torch.cat([buf[:64], buf[64 + n // s:]]).float().cpu()
        assert torch.all(guards == -777.0)
        assert tcu.device_error() == 0
    ints = tcu.fill(torch.empty(1 << 18, dtype=torch.float16, device="cuda"), 5, 0, "small_int")
    assert torch.equal(tcu.segmented_reduce(ints, s, algo="tcgen05"), tcu.segmented_reduce(ints, s, algo="mma"))


def test_tcgen05_rejects_what_it_does_not_cover():
    import tcu_scope_b200 as tcu
    x = tcu.fill(torch.empty(4096, dtype=torch.float16, device="cuda"), 1, 0)
    with pytest.raises(tcu.TcuError) as e:
        tcu.segmented_reduce(x, 4096, algo="tcgen05")  # only segments of 16 ... 2048 elements
    assert e.value.status == 2
    with pytest.raises(tcu.TcuError):
        tcu.segmented_reduce(x[:4096 - 16], 16, algo="tcgen05")  # element count not a multiple of 64


@pytest.mark.parametrize("s", [16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
def test_tcgen05_scan_matches_oracle(s, out_dtype):
    """The tensor-memory scan keeps the exact (hi, lo) parts: fp32 outputs equal the fp64 prefix
    rounded once, fp16 outputs are within one half of it -- the bars of the mma.sync path."""
    import tcu_scope_b200 as tcu
    # ... and, for segments spread over several tiles, groups of four segments that are not full
    for n in (64, 64 * 37, 8192, 8192 * 5 + 64 * 3, 1 << 20, (1 << 24) + 64 * 11, 7 * s, 1197 * s):
        n = max(s, n // s * s)
        if n % 64:
            continue
        x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 80 + s, 0)
        buf = torch.full((n + 128,), -777.0, dtype=out_dtype, device="cuda")
        out = buf[64:64 + n]
        tcu.segmented_scan(x, s, out=out, algo="tcgen05")
        ref = oracle.c_segmented_scan(bits(x), s)
        if out_dtype == torch.float32:
            got = out.cpu().numpy()
            bad, max_abs, _ = oracle.np_check_f32(got, ref, 1e-3, 1e-5)
            assert bad == 0, (n, max_abs)
            assert np.array_equal(got, ref.astype(np.float32)), n
        else:
            bad, worst = oracle.np_check_f16(bits(out), ref, 2)
            assert bad == 0 and worst <= 1, (n, worst)
        guards = torch.cat([buf[:64], buf[64 + n:]]).float().cpu()
        assert torch.all(guards == -777.0)
        assert tcu.device_error() == 0
    # sums that leave the exactly representable range: integers, and uniform [0, 1) prefixes
    ints = tcu.fill(torch.empty(1 << 18, dtype=torch.float16, device="cuda"), 5, 0, "small_int")
    assert torch.equal(tcu.segmented_scan(ints, s, out_dtype=out_dtype, algo="tcgen05"),
                       tcu.segmented_scan(ints, s, out_dtype=out_dtype, algo="mma"))
    if out_dtype == torch.float32:
        pos = tcu.fill(torch.empty(1 << 18, dtype=torch.float16, device="cuda"), 6, 0, "uniform_01")
        got = tcu.segmented_scan(pos, s, out_dtype=out_dtype, algo="tcgen05").cpu().numpy()
        bad, max_abs, max_rel = oracle.np_check_f32(got, oracle.c_segmented_scan(bits(pos), s), 1e-3, 1e-5)
        assert bad == 0 and max_rel < 2e-7, (max_abs, max_rel)


def test_tcgen05_scan_rejects_what_it_does_not_cover():
    import tcu_scope_b200 as tcu
    x = tcu.fill(torch.empty(1 << 15, dtype=torch.float16, device="cuda"), 1, 0)
    with pytest.raises(tcu.TcuError) as e:
        tcu.segmented_scan(x, 32768, out_dtype=torch.float32, algo="tcgen05")  # fp32 outputs: up to 16384 elements
    assert e.value.status == 2
    with pytest.raises(tcu.TcuError) as e:
        tcu.segmented_scan(x, 32768, out_dtype=torch.float16, algo="tcgen05")  # one segment is the full scan's job
    assert e.value.status == 2
    with pytest.raises(tcu.TcuError):
        tcu.segmented_scan(x[:4096 - 16], 16, algo="tcgen05")  # element count not a multiple of 64


@pytest.mark.parametrize("s,out_dtype", [(16, torch.float16), (2048, torch.float16), (16384, torch.float16),
                                         (16, torch.float32)])
def test_auto_runs_the_tcgen05_scan_on_large_arrays(s, out_dtype):
    """TCU_ALGO_AUTO switches to the tensor-memory scan from 2^26 / 2^27 elements on: the default
    path of a large scan is checked against the oracle like the explicit one."""
    import tcu_scope_b200 as tcu
    n = 1 << 27
    x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 123, 0)
    out = tcu.segmented_scan(x, s, out_dtype=out_dtype)
    ref = oracle.c_segmented_scan(bits(x), s)
    if out_dtype == torch.float32:
        assert np.array_equal(out.cpu().numpy(), ref.astype(np.float32))
    else:
        bad, worst = oracle.np_check_f16(bits(out), ref, 2)
        assert bad == 0 and worst <= 1
    assert torch.equal(out, tcu.segmented_scan(x, s, out_dtype=out_dtype, algo="tcgen05"))
    assert tcu.device_error() == 0


@pytest.mark.parametrize("s", [1 << 15, 1 << 16, 1 << 18, 1 << 20])
def test_tcgen05_scan_of_long_segments_with_16bit_outputs(s):
    """Whole segments of 2^15 ... 2^20 elements are spread over tiles like the 4096 ... 16384-element
    ones: no look-back, no workspace traffic."""
    import tcu_scope_b200 as tcu
    for segs in (2, 3, 8, 9, 37):
        n = s * segs
        if n > 1 << 26:
            continue
        x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 300 + segs, 0)
        buf = torch.full((n + 128,), -777.0, dtype=torch.float16, device="cuda")
        out = buf[64:64 + n]
        tcu.segmented_scan(x, s, out=out, algo="tcgen05")
        bad, worst = oracle.np_check_f16(bits(out), oracle.c_segmented_scan(bits(x), s), 2)
        assert bad == 0 and worst <= 1, (s, segs, worst)
        guards = torch.cat([buf[:64], buf[64 + n:]]).float().cpu()
        assert torch.all(guards == -777.0)
        assert tcu.device_error() == 0
    if s <= 1 << 16:  # sums beyond the exactly representable range (and still finite in fp16)
        pos = tcu.fill(torch.empty(4 * s, dtype=torch.float16, device="cuda"), 6, 0, "uniform_01")
        got = tcu.segmented_scan(pos, s, out_dtype=torch.float16, algo="tcgen05")
        assert oracle.np_check_f16(bits(got), oracle.c_segmented_scan(bits(pos), s), 2)[0] == 0


@pytest.mark.parametrize("s", [16, 256, 2048, 4096, 16384])
def test_auto_runs_the_tcgen05_scan_for_large_exclusive_scans(s):
    """Exclusive scans with 16-bit outputs take the tensor-memory kernel on large arrays: a strictly
    triangular U inside a row for 16-element segments, rows shifted by one column above."""
    import tcu_scope_b200 as tcu
    n = (1 << 26) + 64 * s  # not a whole number of work units for the long segments
    x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 321 + s, 0)
    buf = torch.full((n + 128,), -777.0, dtype=torch.float16, device="cuda")
    out = buf[64:64 + n]
    tcu.segmented_scan(x, s, out=out, exclusive=True)
    ref = oracle.c_segmented_scan(bits(x), s) - bits(x).view(np.float16).astype(np.float64)
    bad, worst = oracle.np_check_f16(bits(out), ref, 2)
    assert bad == 0 and worst <= 1, (s, worst)
    guards = torch.cat([buf[:64], buf[64 + n:]]).float().cpu()
    assert torch.all(guards == -777.0)
    assert tcu.device_error() == 0
