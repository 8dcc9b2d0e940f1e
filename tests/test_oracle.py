"""CPU tests of the oracle: numpy vs C restatement, golden fixtures, closed forms."""
import os

import numpy as np
import pytest

import oracle

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "golden.npz")
DIST_NAMES = {v: k for k, v in oracle.DIST.items()}


def golden_cases():
    g = np.load(GOLDEN)
    names = sorted({k.split("/")[0] for k in g.files})
    return g, names


def test_golden_file_has_cases():
    g, names = golden_cases()
    assert len(names) >= 10


@pytest.mark.parametrize("impl", ["numpy", "c"])
def test_oracle_matches_golden(impl):
    g, names = golden_cases()
    for name in names:
        seed, first, dist, n, s, is_scan = (int(v) for v in g[name + "/meta"])
        fill = oracle.np_fill_f16 if impl == "numpy" else oracle.c_fill_f16
        x = fill(n, seed, first, DIST_NAMES[dist])
        assert np.array_equal(x[:64], g[name + "/head_bits"]), name
        if is_scan:
            ref = (oracle.np_segmented_scan if impl == "numpy" else oracle.c_segmented_scan)(x, s)
        else:
            ref = (oracle.np_segmented_reduce if impl == "numpy" else oracle.c_segmented_reduce)(x, s)
        # float64 sums of multiples of 2^-24 this small are exact: bit equality
        assert np.array_equal(ref, g[name + "/ref"]), name


@pytest.mark.parametrize("dist", list(oracle.DIST))
def test_fill_numpy_equals_c(dist):
    for n, seed, first in [(8, 0, 0), (4096, 1, 0), (4096, 1, 4096), (1000, 2 ** 40 + 3, 2 ** 35)]:
        assert np.array_equal(oracle.np_fill_f16(n, seed, first, dist),
                              oracle.c_fill_f16(n, seed, first, dist))


def test_fill_is_counter_based():
    whole = oracle.np_fill_f16(4096, 11, 0)
    part = oracle.np_fill_f16(1024, 11, 2048)
    assert np.array_equal(whole[2048:3072], part)


def test_fill_value_ranges():
    pm1 = oracle.np_fill_f16(1 << 16, 3, 0, "uniform_pm1").view(np.float16).astype(np.float64)
    u01 = oracle.np_fill_f16(1 << 16, 3, 0, "uniform_01").view(np.float16).astype(np.float64)
    ints = oracle.np_fill_f16(1 << 12, 3, 0, "small_int").view(np.float16).astype(np.float64)
    assert -1.0 <= pm1.min() < -0.99 and 0.99 < pm1.max() <= 1.0 and abs(pm1.mean()) < 0.01
    assert 0.0 <= u01.min() and u01.max() <= 1.0 and abs(u01.mean() - 0.5) < 0.01
    assert set(np.unique(ints)) == {-2.0, -1.0, 0.0, 1.0, 2.0}


def test_half_conversion_exhaustive():
    lib = oracle.c_lib()
    bits = np.arange(0, 1 << 16, dtype=np.uint16)
    vals = bits.view(np.float16).astype(np.float64)
    finite = np.isfinite(vals)
    for b in bits[finite][::13]:
        v = lib.tcu_oracle_f16_to_f64(int(b))
        assert v == float(np.uint16(b).view(np.float16))
        assert lib.tcu_oracle_f64_to_f16(v) == int(b) or v == 0.0
    pos = np.arange(0, 0x7BFF, dtype=np.uint16).view(np.float16).astype(np.float64)
    mids = (pos[:-1] + pos[1:]) / 2  # exact ties: must round to even
    want = mids.astype(np.float16).view(np.uint16)
    for m, w in zip(mids[::11], want[::11]):
        assert lib.tcu_oracle_f64_to_f16(float(m)) == int(w)
    assert lib.tcu_oracle_f64_to_f16(65520.0) == 0x7C00  # rounds up to inf
    assert lib.tcu_oracle_f64_to_f16(65519.9) == 0x7BFF
    assert lib.tcu_oracle_f64_to_f16(2.0 ** -25) == 0  # tie to even (0)
    assert lib.tcu_oracle_f64_to_f16(2.0 ** -25 * 1.0001) == 1


def test_closed_forms():
    ones = np.full(4096, 0x3C00, dtype=np.uint16)
    for s in (16, 256, 2048):
        assert np.all(oracle.c_segmented_reduce(ones, s) == s)
        assert np.array_equal(oracle.c_segmented_scan(ones, s), np.tile(np.arange(1, s + 1.0), 4096 // s))
    alt = np.tile(np.array([0x3800, 0xB800], dtype=np.uint16), 2048)  # +0.5, -0.5
    assert np.all(oracle.c_segmented_reduce(alt, 64) == 0.0)
    const = oracle.c_fill_f16(1024, 0, 0, "const_0p001")
    h = float(np.float16(0.001))
    assert np.allclose(oracle.c_segmented_reduce(const, 1024), 1024 * h, rtol=0, atol=1e-12)


def test_tile_algebra_is_a_scan():
    x = oracle.np_fill_f16(256, 21, 0)
    want = oracle.np_segmented_scan(x, 256)
    assert np.array_equal(oracle.np_tile256_scan_algebra(x), want)
    out = np.empty(256, dtype=np.float64)
    oracle.c_lib().tcu_oracle_tile256_scan_algebra(x.ctypes.data, out.ctypes.data)
    assert np.allclose(out, want, rtol=0, atol=1e-12)


def test_checkers_agree_and_flag_errors():
    x = oracle.np_fill_f16(8192, 5, 0)
    ref = oracle.np_segmented_scan(x, 1024)
    good32 = ref.astype(np.float32)
    assert oracle.np_check_f32(good32, ref)[0] == 0 and oracle.c_check_f32(good32, ref)[0] == 0
    bad32 = good32.copy()
    bad32[7] += 0.01 * max(1.0, abs(bad32[7]))
    bad32[9] = np.nan
    assert oracle.np_check_f32(bad32, ref)[0] == 2 and oracle.c_check_f32(bad32, ref)[0] == 2
    good16 = ref.astype(np.float16).view(np.uint16)
    assert oracle.np_check_f16(good16, ref) == (0, 0) and oracle.c_check_f16(good16, ref) == (0, 0)
    off = good16.copy()
    off[3] += 3  # three representable halves away
    off[5] += 2  # allowed
    assert oracle.np_check_f16(off, ref) == (1, 3) and oracle.c_check_f16(off, ref) == (1, 3)


def test_cpu_baseline_within_tolerance():
    lib = oracle.c_lib()
    x = oracle.np_fill_f16(1 << 18, 8, 0)
    for s in (16, 256, 16384):
        out = np.empty(x.size // s, dtype=np.float32)
        used = lib.tcu_cpu_segmented_reduce(x.ctypes.data, out.ctypes.data, out.size, s, 2)
        assert used == 2
        assert oracle.np_check_f32(out, oracle.np_segmented_reduce(x, s))[0] == 0
    out16 = np.empty(x.size, dtype=np.uint16)
    lib.tcu_cpu_segmented_scan(x.ctypes.data, out16.ctypes.data, 0, x.size // 16, 16, 0)
    assert oracle.np_check_f16(out16, oracle.np_segmented_scan(x, 16))[0] == 0
    y = oracle.np_fill_f16(1 << 18, 8, 0, "uniform_01")
    tot = np.empty(1, dtype=np.float32)
    lib.tcu_cpu_full_reduce(y.ctypes.data, tot.ctypes.data, y.size, 0)
    assert oracle.np_check_f32(tot, oracle.np_segmented_reduce(y, y.size))[0] == 0
    fs = np.empty(y.size, dtype=np.float32)
    lib.tcu_cpu_full_scan(y.ctypes.data, fs.ctypes.data, y.size, 3)
    assert oracle.np_check_f32(fs, oracle.np_segmented_scan(y, y.size))[0] == 0


def test_bf16_side_of_the_oracle_agrees_with_torch_on_cpu():
    """The bfloat16 conversions of the oracle against an independent implementation."""
    import torch
    rng = np.random.default_rng(5)
    v = np.concatenate([rng.uniform(-1, 1, 4096), rng.uniform(-1e-6, 1e-6, 512), [0.0, 1.0, -1.0, 0.001,
                        1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -9]]).astype(np.float32)  # incl. rounding ties
    mine = oracle.f32_to_bf16_bits(v)
    theirs = torch.from_numpy(v).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(mine, theirs)
    back = torch.from_numpy(mine.view(np.int16)).view(torch.bfloat16).double().numpy()
    assert np.array_equal(oracle._as_f64(mine, "bf16"), back)
    x = oracle.np_fill_f16(1 << 12, 9, 0, "uniform_pm1", fmt="bf16")
    t = torch.from_numpy(x.view(np.int16)).view(torch.bfloat16).double()
    assert np.array_equal(oracle.np_segmented_reduce(x, 64, fmt="bf16"), t.view(-1, 64).sum(1).numpy())
    assert np.allclose(oracle.np_segmented_scan(x, 256, fmt="bf16"),
                       torch.cumsum(t.view(-1, 256), 1).reshape(-1).numpy(), rtol=0, atol=1e-12)
    # a correctly rounded bfloat16 is zero representable values away from itself, its neighbour one
    ref = oracle._as_f64(x, "bf16")
    assert oracle.np_check_f16(x, ref, 0, fmt="bf16") == (0, 0)
    assert oracle.np_check_f16(x + np.uint16(1), ref, 0, fmt="bf16")[1] == 1
