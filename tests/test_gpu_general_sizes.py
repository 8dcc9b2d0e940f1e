"""Segment sizes the tiled kernels do not take, against the oracle: multiples of 16 that are not a
power of two (the reference's kernels accept them: src/reduction/seg_wmma_16n.cu:137-172 only asks
for multiples of 16) and, beyond the reference, every other size from 1 up (masked tails)."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

SIZES = [48, 80, 240, 272, 768, 1008, 4112, 16000, 3 * 16384, 100016,   # multiples of 16
         1, 2, 3, 8, 12, 20, 24, 100, 255, 257, 1000, 1001, 2040, 4099, 65537]  # everything else


def bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def filled(tcu, n, seed):
    """n seeded halves; the fill writes whole 16-byte vectors, so it gets a padded buffer."""
    full = tcu.fill(torch.empty((n + 7) // 8 * 8, dtype=torch.float16, device="cuda"), seed, 0)
    return full[:n]


def guarded(n_out, dtype):
    buf = torch.full((n_out + 128,), -777.0, dtype=dtype, device="cuda")
    return buf, buf[64:64 + n_out]


def guards_intact(buf, n_out):
    return bool(torch.all(torch.cat([buf[:64], buf[64 + n_out:]]).float() == -777.0))


@pytest.mark.parametrize("s", SIZES)
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
def test_general_reduce_matches_oracle(s, out_dtype):
    import tcu_scope_b200 as tcu
    for segs in (1, 7, 300 if s < 20000 else 33):
        n = s * segs
        x = filled(tcu, n, 900 + s)
        buf, out = guarded(segs, out_dtype)
        tcu.segmented_reduce(x, s, out=out)
        ref = oracle.c_segmented_reduce(bits(x), s)
        if out_dtype == torch.float32:
            # exact parts, one rounding: the fp32 result is the rounded fp64 sum
            assert np.array_equal(out.cpu().numpy(), ref.astype(np.float32)), (s, segs)
        else:
            assert oracle.np_check_f16(bits(out), ref, 2)[0] == 0
        assert guards_intact(buf, segs)
    assert tcu.device_error() == 0


@pytest.mark.parametrize("s", SIZES)
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("exclusive", [False, True])
def test_general_scan_matches_oracle(s, out_dtype, exclusive):
    import tcu_scope_b200 as tcu
    for segs in (1, 5, 130 if s < 20000 else 9):
        n = s * segs
        x = filled(tcu, n, 950 + s)
        buf, out = guarded(n, out_dtype)
        tcu.segmented_scan(x, s, out=out, exclusive=exclusive)
        ref = oracle.c_segmented_scan(bits(x), s)
        if exclusive:
            ref = ref - bits(x).view(np.float16).astype(np.float64)  # exact: inclusive minus the element
        if out_dtype == torch.float32:
            bad, max_abs, _ = oracle.np_check_f32(out.cpu().numpy(), ref, 1e-3, 1e-5)
            assert bad == 0, (s, segs, max_abs)
        else:
            assert oracle.np_check_f16(bits(out), ref, 2)[0] == 0
        assert guards_intact(buf, n)
    assert tcu.device_error() == 0


def test_general_sizes_closed_form():
    import tcu_scope_b200 as tcu
    s, segs = 48 * 7, 19
    ones = torch.ones(s * segs, dtype=torch.float16, device="cuda")
    assert torch.all(tcu.segmented_reduce(ones, s) == float(s))
    scan = tcu.segmented_scan(ones, s, out_dtype=torch.float32).cpu().view(segs, s)
    assert torch.equal(scan, torch.arange(1, s + 1, dtype=torch.float32).expand(segs, s))
    # one non-zero element per segment, at every position of a 48-element segment
    for pos in range(48):
        x = torch.zeros(48 * 4, dtype=torch.float16, device="cuda")
        x[pos::48] = 0.5
        assert torch.all(tcu.segmented_reduce(x, 48) == 0.5)
        sc = tcu.segmented_scan(x, 48, out_dtype=torch.float32).cpu().view(4, 48)
        assert torch.all(sc[:, :pos] == 0) and torch.all(sc[:, pos:] == 0.5)


def test_other_algorithms_cover_powers_of_two_only():
    import tcu_scope_b200 as tcu
    x = tcu.fill(torch.empty(48 * 4, dtype=torch.float16, device="cuda"), 1, 0)
    for algo in ("shuffle", "tcgen05"):
        with pytest.raises(tcu.TcuError) as e:
            tcu.segmented_reduce(x, 48, algo=algo)
        assert e.value.status == 2
    with pytest.raises(tcu.TcuError):
        tcu.segmented_scan(x, 48, algo="shuffle")
