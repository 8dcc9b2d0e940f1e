"""bfloat16 inputs (tcu_*_bf16 entry points) against the numpy oracle: the same sums, the 16-bit
element type switched.  fp32 outputs within 1e-3 relative / 1e-5 absolute of the float64 result,
bfloat16 outputs within two representable bfloat16 values of its correct rounding."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def check(out, ref):
    if out.dtype == torch.float32:
        bad, max_abs, _ = oracle.np_check_f32(out.cpu().numpy(), ref, 1e-3, 1e-5)
        assert bad == 0, max_abs
    else:
        bad, worst = oracle.np_check_f16(bits(out), ref, 2, fmt="bf16")
        assert bad == 0, worst


def test_fill_matches_the_oracle_bit_for_bit():
    import tcu_scope_b200 as tcu
    for dist in ("uniform_pm1", "uniform_01", "small_int", "const_0p001"):
        x = tcu.fill(torch.empty(1 << 16, dtype=BF, device="cuda"), 77, 12345, dist)
        assert np.array_equal(bits(x), oracle.np_fill_f16(1 << 16, 77, 12345, dist, fmt="bf16"))


@pytest.mark.parametrize("s", [16, 32, 64, 128, 256, 1024, 4096, 16384, 65536, 48, 1000, 7])
@pytest.mark.parametrize("out_dtype", [torch.float32, BF])
def test_segmented_reduce_bf16(s, out_dtype):
    import tcu_scope_b200 as tcu
    n = s * max(3, (1 << 20) // s + 5)
    x = tcu.fill(torch.empty((n + 7) // 8 * 8, dtype=BF, device="cuda"), 300 + s, 0)[:n]
    out = tcu.segmented_reduce(x, s, out_dtype=out_dtype)
    check(out, oracle.np_segmented_reduce(bits(x), s, fmt="bf16"))
    assert tcu.device_error() == 0


@pytest.mark.parametrize("s", [16, 32, 64, 128, 256, 1024, 4096, 16384, 65536, 48, 1000, 7])
@pytest.mark.parametrize("out_dtype", [torch.float32, BF])
@pytest.mark.parametrize("exclusive", [False, True])
def test_segmented_scan_bf16(s, out_dtype, exclusive):
    import tcu_scope_b200 as tcu
    n = s * max(3, (1 << 19) // s + 3)
    x = tcu.fill(torch.empty((n + 7) // 8 * 8, dtype=BF, device="cuda"), 400 + s, 0)[:n]
    out = tcu.segmented_scan(x, s, out_dtype=out_dtype, exclusive=exclusive)
    ref = oracle.np_segmented_scan(bits(x), s, fmt="bf16")
    if exclusive:
        ref = ref - oracle._as_f64(bits(x), "bf16")
    check(out, ref)
    assert tcu.device_error() == 0


@pytest.mark.parametrize("n", [16, 16 * 1001, 1 << 20, (1 << 22) + 64 * 5, (1 << 22) + 16 * 3])
def test_full_reduce_and_scan_bf16(n):
    import tcu_scope_b200 as tcu
    x = tcu.fill(torch.empty(n, dtype=BF, device="cuda"), 55, 0, "uniform_01")
    xs = oracle._as_f64(bits(x), "bf16")
    o32, o64 = tcu.full_reduce(x)
    total = xs.sum()
    assert abs(o64.item() - total) <= 1e-6 * abs(total)
    assert abs(o32.item() - total) <= 1e-6 * abs(total)
    ref = np.cumsum(xs)
    check(tcu.full_scan(x, out_dtype=torch.float32), ref)
    check(tcu.full_scan(x, out_dtype=BF), ref)
    check(tcu.full_scan(x, out_dtype=torch.float32, exclusive=True), ref - xs)
    assert tcu.device_error() == 0


@pytest.mark.parametrize("algo", ["shuffle", "tcgen05"])
def test_other_algorithms_bf16(algo):
    import tcu_scope_b200 as tcu
    x = tcu.fill(torch.empty(1 << 20, dtype=BF, device="cuda"), 9, 0)
    for s in (16, 32, 64):
        check(tcu.segmented_reduce(x, s, algo=algo), oracle.np_segmented_reduce(bits(x), s, fmt="bf16"))
    if algo == "shuffle":
        check(tcu.segmented_scan(x, 256, out_dtype=torch.float32, algo=algo),
              oracle.np_segmented_scan(bits(x), 256, fmt="bf16"))
    assert tcu.device_error() == 0


@pytest.mark.parametrize("s", [16, 64, 256, 2048, 4096, 16384, 65536])
@pytest.mark.parametrize("out_dtype", [torch.float32, BF])
def test_tcgen05_scan_bf16(s, out_dtype):
    """The tensor-memory scan with bfloat16 inputs: single tiles, segments spread over tiles, and
    (16-bit outputs) whole segments longer than 16384 elements."""
    import tcu_scope_b200 as tcu
    if s > 16384 and out_dtype == torch.float32:
        pytest.skip("segments longer than 16384 elements: 16-bit outputs only")
    n = s * max(3, (1 << 20) // s + 5)
    n = (n + 63) // 64 * 64 if s < 64 else n  # whole 64-element rows
    x = tcu.fill(torch.empty(n, dtype=BF, device="cuda"), 500 + s, 0)
    out = tcu.segmented_scan(x, s, out_dtype=out_dtype, algo="tcgen05")
    check(out, oracle.np_segmented_scan(bits(x), s, fmt="bf16"))
    assert tcu.device_error() == 0


@pytest.mark.parametrize("s", [16, 4096])
def test_large_exclusive_scan_bf16(s):
    """Large exclusive scans with 16-bit outputs run the tensor-memory kernel by default."""
    import tcu_scope_b200 as tcu
    n = 1 << 26
    x = tcu.fill(torch.empty(n, dtype=BF, device="cuda"), 600 + s, 0)
    out = tcu.segmented_scan(x, s, out_dtype=BF, exclusive=True)
    ref = oracle.np_segmented_scan(bits(x), s, fmt="bf16") - oracle._as_f64(bits(x), "bf16")
    check(out, ref)
    assert tcu.device_error() == 0


def test_exact_cases_bf16():
    import tcu_scope_b200 as tcu
    ones = torch.ones(1 << 16, dtype=BF, device="cuda")
    for s in (16, 256, 4096):
        assert torch.all(tcu.segmented_reduce(ones, s) == float(s))
        scan = tcu.segmented_scan(ones, s, out_dtype=torch.float32).cpu().view(-1, s)
        assert torch.equal(scan, torch.arange(1, s + 1, dtype=torch.float32).expand_as(scan))
    ints = tcu.fill(torch.empty(1 << 18, dtype=BF, device="cuda"), 5, 0, "small_int")
    ref = oracle.np_segmented_reduce(bits(ints), 1024, fmt="bf16")
    assert np.array_equal(tcu.segmented_reduce(ints, 1024).cpu().numpy(), ref.astype(np.float32))
    # 16-bit outputs take the input's type
    with pytest.raises(TypeError):
        tcu.segmented_reduce(ones, 16, out=torch.empty(1 << 12, dtype=torch.float16, device="cuda"))
