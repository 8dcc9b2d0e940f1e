"""GPU parity tests: the CUDA path, called through the C ABI, against the fp64
oracle on the same seeded inputs.

Tolerances (from the task statement): fp32 outputs within 1e-3 relative with a
1e-5 absolute floor; fp16 outputs within 2 representable halves of the fp64
result rounded to half.  The tensor-core path is built to do better -- exact
partial sums, one final rounding -- and the tests also assert that.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

REL, ABS_FLOOR, MAX_HALF_ULP = 1e-3, 1e-5, 2
TILE = 16384
ALL_SIZES = [16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384]


@pytest.fixture(scope="module")
def tcu():
    import tcu_scope_b200
    assert torch.cuda.is_available()
    yield tcu_scope_b200
    assert tcu_scope_b200.device_error() == 0, "a bounded device wait ran out during the tests"


def device_input(tcu, n, seed, first=0, dist="uniform_pm1"):
    x = torch.empty(n, dtype=torch.float16, device="cuda")
    tcu.fill(x, seed, first, dist)
    return x


def bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def guarded(n, dtype):
    """Output buffer with 64 canary elements on each side."""
    buf = torch.full((n + 128,), -777.0, dtype=dtype, device="cuda")
    return buf, buf[64:64 + n]


def assert_guards(buf, n):
    g = torch.cat([buf[:64], buf[64 + n:]]).float().cpu()
    assert torch.all(g == -777.0), "kernel wrote outside its output"


def check_f32(got, ref, exact=False):
    g = got.float().cpu().numpy()
    bad, max_abs, max_rel = oracle.np_check_f32(g, ref, REL, ABS_FLOOR)
    assert bad == 0, f"{bad} outputs out of tolerance (max abs {max_abs:.3e}, max rel {max_rel:.3e})"
    if exact:  # one rounding of the exact sum
        assert np.array_equal(g, ref.astype(np.float32))


def check_f16(got, ref, max_ulp=MAX_HALF_ULP):
    bad, worst = oracle.np_check_f16(bits(got), ref, max_ulp)
    assert bad == 0, f"{bad} outputs more than {max_ulp} halves off (worst {worst})"
    return worst


# --------------------------------------------------------------------- fill
@pytest.mark.parametrize("dist", list(oracle.DIST))
def test_fill_matches_oracle_bit_for_bit(tcu, dist):
    for n, seed, first in [(8, 1, 0), (4096, 2, 0), (1 << 20, 3, 12345 * 8), (4096, 2 ** 40, 2 ** 36)]:
        x = device_input(tcu, n, seed, first, dist)
        assert np.array_equal(bits(x), oracle.np_fill_f16(n, seed, first, dist))


# ------------------------------------------------------------------- reduce
@pytest.mark.parametrize("s", ALL_SIZES)
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
def test_segmented_reduce_sizes(tcu, s, out_dtype):
    # ragged counts: one segment, a partial slice, a partial tile, several tiles + tail
    for segs in sorted({1, 3, max(1, 2048 // s) + 1, max(1, TILE // s) * 3 + 1, (5 * TILE + 4096) // s}):
        n = segs * s
        x = device_input(tcu, n, 100 + s, 0)
        buf, out = guarded(segs, out_dtype)
        # guards shift the output by 64 elements: still 16-byte aligned for both dtypes
        tcu.segmented_reduce(x, s, out=out)
        ref = oracle.np_segmented_reduce(bits(x), s)
        if out_dtype == torch.float32:
            check_f32(out, ref, exact=(s >= 256))
        else:
            check_f16(out, ref)
        assert_guards(buf, segs)


@pytest.mark.parametrize("s", [16, 64, 1024, 16384])
def test_segmented_reduce_many_tiles(tcu, s):
    n = 1 << 25  # 2048 tiles: every CTA wraps its ring more than twice
    x = device_input(tcu, n, 7, 0)
    out = tcu.segmented_reduce(x, s)
    check_f32(out, oracle.c_segmented_reduce(bits(x), s), exact=(s >= 256))


@pytest.mark.parametrize("s", [32768, 65536, 1 << 20])
def test_segmented_reduce_long_segments(tcu, s):
    for segs in (1, 3, 40):
        x = device_input(tcu, segs * s, 11, 5 * s)
        buf, out = guarded(segs, torch.float32)
        tcu.segmented_reduce(x, s, out=out)
        check_f32(out, oracle.c_segmented_reduce(bits(x), s), exact=True)
        assert_guards(buf, segs)


@pytest.mark.parametrize("n", [16, 48, 16384, 16384 * 3 + 160, 1 << 24, (1 << 26) + 4096])
@pytest.mark.parametrize("dist", ["uniform_01", "uniform_pm1"])
def test_full_reduce(tcu, n, dist):
    x = device_input(tcu, n, 13, 0, dist)
    out32, out64 = tcu.full_reduce(x)
    ref = oracle.c_segmented_reduce(bits(x), n)
    check_f32(out32, ref, exact=True)
    assert out64.cpu().numpy()[0] == ref[0]  # sums of halves this size are exact in double


def test_reduce_exact_on_integers(tcu):
    for s in ALL_SIZES + [65536]:
        n = max(s * 5, 1 << 18) // s * s
        x = device_input(tcu, n, 17, 0, "small_int")
        out = tcu.segmented_reduce(x, s)
        assert np.array_equal(out.cpu().numpy().astype(np.float64), oracle.np_segmented_reduce(bits(x), s))


# --------------------------------------------------------------------- scan
@pytest.mark.parametrize("s", ALL_SIZES)
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
def test_segmented_scan_sizes(tcu, s, out_dtype):
    for segs in sorted({1, 3, max(1, 2048 // s) + 1, max(1, TILE // s) * 3 + 1, (5 * TILE + 4096) // s}):
        n = segs * s
        x = device_input(tcu, n, 200 + s, 0)
        buf, out = guarded(n, out_dtype)
        tcu.segmented_scan(x, s, out=out)
        ref = oracle.np_segmented_scan(bits(x), s)
        if out_dtype == torch.float32:
            check_f32(out, ref, exact=True)
        else:
            assert check_f16(out, ref) <= 1
        assert_guards(buf, n)


@pytest.mark.parametrize("s,out_dtype", [(16, torch.float16), (256, torch.float16), (4096, torch.float32)])
def test_segmented_scan_many_tiles(tcu, s, out_dtype):
    n = 1 << 25
    x = device_input(tcu, n, 9, 0)
    out = tcu.segmented_scan(x, s, out_dtype=out_dtype)
    ref = oracle.c_segmented_scan(bits(x), s)
    if out_dtype == torch.float32:
        check_f32(out, ref, exact=True)
    else:
        assert check_f16(out, ref) <= 1


@pytest.mark.parametrize("s", [32768, 1 << 18])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
def test_segmented_scan_long_segments(tcu, s, out_dtype):
    for segs in (1, 3, 17):
        n = segs * s
        x = device_input(tcu, n, 23, 0)
        buf, out = guarded(n, out_dtype)
        tcu.segmented_scan(x, s, out=out)
        ref = oracle.c_segmented_scan(bits(x), s)
        if out_dtype == torch.float32:
            check_f32(out, ref)
        else:
            check_f16(out, ref)
        assert_guards(buf, n)


@pytest.mark.parametrize("n", [16, 2064, 16384, 16384 * 3 + 160, 1 << 22, (1 << 25) + 16 * 999])
def test_full_scan(tcu, n):
    x = device_input(tcu, n, 29, 0, "uniform_01")
    out = tcu.full_scan(x, out_dtype=torch.float32)
    check_f32(out, oracle.c_segmented_scan(bits(x), n))
    # repeated launches reuse a caller-owned workspace
    ws = torch.empty(tcu.workspace_bytes(tcu.OP_FULL_SCAN, n, n), dtype=torch.uint8, device="cuda")
    again = tcu.full_scan(x, out_dtype=torch.float32, workspace=ws)
    again2 = tcu.full_scan(x, out_dtype=torch.float32, workspace=ws)
    assert torch.equal(again, out) and torch.equal(again2, out)


def test_full_scan_seeded_by_earlier_shards(tcu):
    n, shards = 1 << 20, 4
    x = device_input(tcu, n, 31, 0, "uniform_01")
    ref = oracle.c_segmented_scan(bits(x), n)
    per = n // shards
    totals = torch.empty(shards, dtype=torch.float64, device="cuda")
    for r in range(shards):
        _, t64 = tcu.full_reduce(x[r * per:(r + 1) * per])
        totals[r] = t64[0]
    for r in range(shards):
        out = tcu.full_scan(x[r * per:(r + 1) * per], shard_totals=totals, shard_index=r)
        check_f32(out, ref[r * per:(r + 1) * per])


def test_scan_exact_on_integers(tcu):
    for s in [16, 128, 256, 2048, 16384, 65536]:
        n = max(s * 3, 1 << 18) // s * s
        x = device_input(tcu, n, 37, 0, "small_int")
        for dt in (torch.float16, torch.float32):
            out = tcu.segmented_scan(x, s, out_dtype=dt)
            assert np.array_equal(out.float().cpu().numpy().astype(np.float64),
                                  oracle.np_segmented_scan(bits(x), s))


@pytest.mark.parametrize("s", [16, 64, 256, 4096, 16384, 65536])
def test_exclusive_scan(tcu, s):
    """out[i] = prefix before i: the inclusive oracle shifted by one inside each segment."""
    n = max(3 * s, 5 * TILE + 2048) // s * s
    x = device_input(tcu, n, 300 + s, 0)
    incl = oracle.np_segmented_scan(bits(x), s).reshape(-1, s)
    ref = np.concatenate([np.zeros((incl.shape[0], 1)), incl[:, :-1]], axis=1).reshape(-1)
    buf, out = guarded(n, torch.float32)
    tcu.segmented_scan(x, s, out=out, exclusive=True)
    check_f32(out, ref, exact=True)
    assert_guards(buf, n)
    assert check_f16(tcu.segmented_scan(x, s, out_dtype=torch.float16, exclusive=True), ref) <= 1
    if s == 65536:
        y = device_input(tcu, n, 301, 0, "uniform_01")
        full = oracle.np_segmented_scan(bits(y), n)
        check_f32(tcu.full_scan(y, exclusive=True), np.concatenate([[0.0], full[:-1]]))


# -------------------------------------------------------------- closed forms
def test_closed_forms(tcu):
    ones = torch.ones(1 << 16, dtype=torch.float16, device="cuda")
    for s in (16, 256, 2048):
        assert torch.all(tcu.segmented_reduce(ones, s) == s)
        want = torch.arange(1, s + 1, device="cuda", dtype=torch.float32).repeat((1 << 16) // s)
        assert torch.equal(tcu.segmented_scan(ones, s, out_dtype=torch.float32), want)
        assert torch.equal(tcu.segmented_scan(ones, s, out_dtype=torch.float16).float(), want)
    alt = torch.tensor([0.5, -0.5], dtype=torch.float16, device="cuda").repeat(1 << 15)
    assert torch.all(tcu.segmented_reduce(alt, 64) == 0)
    # the reference's fill: every element half(0.001)
    const = device_input(tcu, 1 << 16, 0, 0, "const_0p001")
    h = float(np.float16(0.001))
    got = tcu.segmented_reduce(const, 1024).cpu().numpy()
    assert np.array_equal(got, np.full(64, np.float32(1024 * h)))
    # a single non-zero element at every position of a segment
    for s in (16, 256):
        x = torch.zeros(s * s, dtype=torch.float16, device="cuda")
        x[torch.arange(s, device="cuda") * s + torch.arange(s, device="cuda")] = 1.0
        assert torch.all(tcu.segmented_reduce(x, s) == 1)
        sc = tcu.segmented_scan(x, s, out_dtype=torch.float32).view(s, s)
        assert torch.equal(sc, torch.triu(torch.ones(s, s, device="cuda")))


# -------------------------------------------------------------------- errors
def test_error_behaviour(tcu):
    x = device_input(tcu, 4096, 1)
    with pytest.raises(ValueError):
        tcu.segmented_reduce(x, 48)  # 4096 is not a multiple of 48
    with pytest.raises(tcu.TcuError) as e:
        tcu.segmented_reduce(x[:4032], 48, algo="shuffle")  # the ablation: powers of two only
    # a segment size of zero is rejected like the reference's "invalid segment
    # size" (src/reduction/seg_wmma_16n.cu:172)
    lib = tcu._lib.load()
    out = torch.empty(4096, dtype=torch.float32, device="cuda")
    assert lib.tcu_segmented_reduce_f16(x.data_ptr(), out.data_ptr(), 1, 4, 0, 0, None, 0, None) == 2
    assert lib.tcu_segmented_reduce_f16(x.data_ptr() + 2, out.data_ptr(), 1, 16, 16, 0, None, 0, None) == 1
    # long segments without a workspace
    big = device_input(tcu, 1 << 16, 2)
    assert lib.tcu_segmented_reduce_f16(big.data_ptr(), out.data_ptr(), 1, 2, 1 << 15, 0, None, 0, None) == 5
    assert lib.tcu_full_scan_f16(big.data_ptr(), out.data_ptr(), 1, 1 << 12, None, 0, 0, None, 0, None) == 5
    # empty input: nothing launched, ok
    assert lib.tcu_segmented_scan_f16(None, None, 0, 0, 16, 0, None, 0, None) == 0
    assert e.value.status == 2


# ------------------------------------------------------------------ ablation
@pytest.mark.parametrize("s", [16, 64, 256, 4096, 16384])
def test_shuffle_ablation_agrees(tcu, s):
    """The CUDA-core variant carries plain fp32 rounding: it meets the fp32
    tolerance on reductions; its scans are compared at a looser bound."""
    n = (3 * TILE + 2048) // s * s if s <= 2048 else 5 * s
    x = device_input(tcu, n, 41, 0)
    red = tcu.segmented_reduce(x, s, algo="shuffle")
    bad, max_abs, _ = oracle.np_check_f32(red.cpu().numpy(), oracle.np_segmented_reduce(bits(x), s),
                                          REL, 1e-4)
    assert bad == 0, max_abs
    sc = tcu.segmented_scan(x, s, out_dtype=torch.float32, algo="shuffle")
    bad, max_abs, _ = oracle.np_check_f32(sc.cpu().numpy(), oracle.np_segmented_scan(bits(x), s),
                                          REL, 1e-4)
    assert bad == 0, max_abs


# ---------------------------------------------------------------- host path
def test_host_buffers_match_device_path(tcu):
    ctx = tcu.HostContext(chunk_elements=1 << 18)
    n = (1 << 20) + (1 << 16)
    h_in = torch.from_numpy(oracle.np_fill_f16(n, 43, 0).view(np.int16)).view(torch.float16).pin_memory()
    xb = bits(h_in)
    out = torch.empty(n // 256, dtype=torch.float32).pin_memory()
    ctx.run(tcu.OP_SEGMENTED_REDUCE, h_in, out, 256)
    assert np.array_equal(out.numpy(), oracle.np_segmented_reduce(xb, 256).astype(np.float32))
    sizes = [16, 256, 16384]
    outs = [torch.empty(n // s, dtype=torch.float32).pin_memory() for s in sizes]
    ctx.reduce_sweep(h_in, sizes, outs)
    for s, o in zip(sizes, outs):
        want = oracle.np_segmented_reduce(xb, s)
        if s >= 256:
            assert np.array_equal(o.numpy(), want.astype(np.float32))
        else:
            assert oracle.np_check_f32(o.numpy(), want)[0] == 0
    sc = torch.empty(n, dtype=torch.float16).pin_memory()
    ctx.run(tcu.OP_SEGMENTED_SCAN, h_in, sc, 4096)
    assert oracle.np_check_f16(sc.view(torch.int16).numpy().view(np.uint16),
                               oracle.np_segmented_scan(xb, 4096), 1)[0] == 0
    h01 = torch.from_numpy(oracle.np_fill_f16(n, 44, 0, "uniform_01").view(np.int16)).view(torch.float16).pin_memory()
    tot = torch.empty(1, dtype=torch.float32).pin_memory()
    ctx.run(tcu.OP_FULL_REDUCE, h01, tot)
    ref = oracle.np_segmented_scan(bits(h01), n)
    assert tot.numpy()[0] == np.float32(ref[-1])
    fs = torch.empty(n, dtype=torch.float32).pin_memory()
    ctx.run(tcu.OP_FULL_SCAN, h01, fs)
    assert oracle.np_check_f32(fs.numpy(), ref)[0] == 0
    ctx.close()


def test_host_sweep_with_sizes_that_are_not_powers_of_two(tcu):
    """Chunks of the sweep must hold whole segments of every size: with {48, 64} a chunk is a
    multiple of 192, not of 64; small chunks make the array span many of them."""
    ctx = tcu.HostContext(chunk_elements=1 << 14)  # the smallest staging buffer: one tile
    sizes = [48, 64, 16]
    n = 192 * 1000  # 12 chunks of 16320 elements (85 x 192) and a short one
    h_in = torch.from_numpy(oracle.np_fill_f16(n, 45, 0).view(np.int16)).view(torch.float16).pin_memory()
    outs = [torch.empty(n // s, dtype=torch.float32).pin_memory() for s in sizes]
    ctx.reduce_sweep(h_in, sizes, outs)
    for s, o in zip(sizes, outs):
        assert oracle.np_check_f32(o.numpy(), oracle.np_segmented_reduce(bits(h_in), s))[0] == 0, s
    # sizes whose common multiple exceeds the staging buffer are refused, not mangled
    big = [16384, 48]
    m = 16384 * 3 * 2
    h2 = torch.zeros(m, dtype=torch.float16).pin_memory()
    with pytest.raises(tcu.TcuError) as e:
        ctx.reduce_sweep(h2, big, [torch.empty(m // s, dtype=torch.float32).pin_memory() for s in big])
    assert e.value.status == 2
    ctx.close()
