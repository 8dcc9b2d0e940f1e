"""The benchmark configurations at their FULL sizes (2^28 elements for the segmented operations,
2^30 for the full ones), where the float64 oracle cannot be run over every output in test time.
Checked through what does not depend on the size:

  * sampled segments / chunks against the oracle, with the tolerances of the small tests;
  * a checksum of checksums: sums at one segment size folded into the next larger one, and into
    the full reduction;
  * consistency between operations: the last element of every scanned segment is its reduction;
  * linearity: doubling the input (exact in fp16) doubles every output bit for bit;
  * integer inputs (-2..2): every result is exact, so all of the above must hold with equality.
"""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

SWEEP = [16, 32, 64, 256, 1024, 16384]
REL, ABS_FLOOR = 1e-3, 1e-5


@pytest.fixture(scope="module")
def tcu():
    import tcu_scope_b200
    yield tcu_scope_b200
    assert tcu_scope_b200.device_error() == 0
    torch.cuda.empty_cache()


def bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def sample_rows(num_rows, count, seed):
    rng = np.random.default_rng(seed)
    idx = np.unique(np.concatenate([[0, num_rows - 1], rng.integers(0, num_rows, count)]))
    return torch.from_numpy(idx).cuda()


def within_spec(got64: torch.Tensor, ref64: torch.Tensor):
    err = (got64 - ref64).abs()
    return bool(torch.all(err <= torch.clamp(REL * ref64.abs(), min=ABS_FLOOR)))


def test_c2_segmented_reduce_sweep_at_2p28(tcu):
    n = 1 << 28
    x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 2024, 0)
    sums = {}
    for s in SWEEP:
        out = tcu.segmented_reduce(x, s)
        rows = sample_rows(n // s, 4096 if s <= 1024 else 512, s)
        ref = oracle.np_segmented_reduce(bits(x.view(-1, s)[rows]).reshape(-1), s)
        got = out[rows].cpu().numpy()
        bad, max_abs, _ = oracle.np_check_f32(got, ref, REL, ABS_FLOOR)
        assert bad == 0, (s, max_abs)
        if s >= 256:  # exact parts: the float32 nearest to the float64 sum
            assert np.array_equal(got, ref.astype(np.float32)), s
        sums[s] = out
    # checksum of checksums, level by level and down to the single total
    for a, b in zip(SWEEP[:-1], SWEEP[1:]):
        assert within_spec(sums[a].double().view(-1, b // a).sum(1), sums[b].double()), (a, b)
    total64 = tcu.full_reduce(x)[1].item()
    assert abs(sums[16384].double().sum().item() - total64) <= 1e-6 * max(1.0, abs(total64))
    # linearity: 2x is exact in fp16, and doubles every partial sum exactly
    y = x * 2
    for s in SWEEP:
        assert torch.equal(tcu.segmented_reduce(y, s), sums[s] * 2), s
    del y, sums
    # integers: every level exact
    xi = tcu.fill(x, 7, 0, "small_int")
    prev, prev_s = None, None
    for s in SWEEP:
        out = tcu.segmented_reduce(xi, s)
        if prev is not None:
            assert torch.equal(prev.view(-1, s // prev_s).sum(1), out), (prev_s, s)
        prev, prev_s = out, s
    assert prev.double().sum().item() == tcu.full_reduce(xi)[1].item()


@pytest.mark.parametrize("s,out_dtype", [(16, torch.float16), (256, torch.float16), (4096, torch.float32)])
def test_c3_segmented_scan_at_2p28(tcu, s, out_dtype):
    n = 1 << 28
    x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 2025, 0)
    out = tcu.segmented_scan(x, s, out_dtype=out_dtype)
    rows = sample_rows(n // s, 4096 if s <= 256 else 1024, s)
    ref = oracle.np_segmented_scan(bits(x.view(-1, s)[rows]).reshape(-1), s)
    got = out.view(-1, s)[rows].reshape(-1)
    if out_dtype == torch.float32:
        assert np.array_equal(got.cpu().numpy(), ref.astype(np.float32))  # exact parts, one rounding
    else:
        bad, worst = oracle.np_check_f16(bits(got), ref, 2)
        assert bad == 0 and worst <= 1, worst
    # the last element of every scanned segment is the segment's sum
    red = tcu.segmented_reduce(x, s)
    assert within_spec(out.view(-1, s)[:, -1].double(), red.double())
    # first element = the input itself
    assert torch.equal(out.view(-1, s)[:, 0].float(), x.view(-1, s)[:, 0].float())
    # linearity (fp32 outputs double exactly; fp16 outputs too, away from subnormal prefix sums)
    out2 = tcu.segmented_scan(x * 2, s, out_dtype=out_dtype)
    if out_dtype == torch.float32:
        assert torch.equal(out2, out * 2)
    else:
        normal = out.abs() >= 2.0 ** -13
        assert torch.equal(out2[normal], (out * 2)[normal])
    del out2
    # integers: exact running sums, any output type
    xi = tcu.fill(x, 8, 0, "small_int")
    oi = tcu.segmented_scan(xi, s, out_dtype=out_dtype)
    assert torch.equal(oi.view(-1, s)[:, -1].float(), tcu.segmented_reduce(xi, s))
    ref_i = oracle.np_segmented_scan(bits(xi.view(-1, s)[rows]).reshape(-1), s)
    assert np.array_equal(oi.view(-1, s)[rows].reshape(-1).float().cpu().numpy().astype(np.float64), ref_i)


def test_c4_full_reduce_at_2p30(tcu):
    n = 1 << 30
    x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 2026, 0, "uniform_01")
    o32, o64 = tcu.full_reduce(x)
    # the whole array through the C oracle: 2^20-element chunk sums, exact in double, then added up
    chunk = oracle.c_segmented_reduce(bits(x), 1 << 20)
    ref = float(np.sum(chunk, dtype=np.float64))
    assert abs(o64.item() - ref) <= 1e-12 * ref
    assert o32.item() == np.float32(ref)
    # checksum of checksums on the device: long-segment sums fold into the total
    seg = tcu.segmented_reduce(x, 1 << 20)
    assert np.array_equal(seg.cpu().numpy(), chunk.astype(np.float32))
    assert abs(seg.double().sum().item() - ref) <= 1e-6 * ref
    # linearity
    d32, d64 = tcu.full_reduce(x * 2)
    assert d64.item() == 2 * o64.item() and d32.item() == 2 * o32.item()


def test_c5_full_scan_at_2p30(tcu):
    n, chunk = 1 << 30, 1 << 20
    x = tcu.fill(torch.empty(n, dtype=torch.float16, device="cuda"), 2027, 0, "uniform_01")
    out = tcu.full_scan(x, out_dtype=torch.float32)
    # prefix at the end of every 2^20-element chunk = running sum of exact chunk sums
    chunk_sums = oracle.c_segmented_reduce(bits(x), chunk)
    ends = np.cumsum(chunk_sums, dtype=np.float64)
    got_ends = out.view(-1, chunk)[:, -1].cpu().numpy()
    bad, max_abs, max_rel = oracle.np_check_f32(got_ends, ends, REL, ABS_FLOOR)
    assert bad == 0 and max_rel <= 1e-6, (max_abs, max_rel)
    # inside sampled chunks: offset of the chunk + the oracle's scan of the chunk
    for c in (0, 1, 511, 1023):
        local = oracle.c_segmented_scan(bits(x.view(-1, chunk)[c]), chunk)
        ref = local + (ends[c - 1] if c else 0.0)
        bad, max_abs, max_rel = oracle.np_check_f32(out.view(-1, chunk)[c].cpu().numpy(), ref, REL, ABS_FLOOR)
        assert bad == 0 and max_rel <= 1e-6, (c, max_abs, max_rel)
    # inputs are non-negative: the prefix never steps down (each output is rounded once, at its
    # own magnitude; one float32 ulp of slack for ties); consistent with the reduction
    assert bool(torch.all(out[1:] - out[:-1] >= -out[1:] * 2.0 ** -23))
    assert abs(out[-1].item() - tcu.full_reduce(x)[1].item()) <= 1e-6 * out[-1].item()
    # linearity, to the last bit but one: the carry of a tile is split into a coarse and a fine
    # float at a fixed absolute scale, so doubling the data may move one rounding
    twice = tcu.full_scan(x * 2, out_dtype=torch.float32)
    assert bool(torch.all((twice - out * 2).abs() <= out * 2.0 ** -22))
