"""Pins the oracle against outputs of the REFERENCE ITSELF: its WMMA kernels,
compiled unmodified for sm_100a (oracle/_ref, built where the reference checkout
is present), run on the GPU on inputs whose sums are exact in fp16 -- integers in
[-2, 2] -- so that the reference's fp16-accumulating kernels must agree with the
fp64 oracle bit for bit, and with this library's outputs.
"""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    lib = oracle.ref_lib()
    if lib is None:
        pytest.skip("oracle/_ref/libtcu_ref.so not built (needs the reference checkout)")
    return lib


def bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def stream():
    return torch.cuda.current_stream().cuda_stream


# (segment_size, variant 0=16n / 1=256n, warps_per_block)
REDUCE_CASES = [(16, 0, 8), (32, 0, 8), (64, 0, 1), (256, 0, 1), (1024, 0, 1),
                (256, 1, 8), (1024, 1, 8)]
SCAN_CASES = [(16, 0, 8), (32, 0, 8), (256, 0, 1), (256, 1, 8), (256, 1, 4)]


@pytest.mark.parametrize("s,variant,wpb", REDUCE_CASES)
def test_reference_reduction_equals_oracle_and_library(ref, s, variant, wpb):
    import tcu_scope_b200 as tcu
    segs = 128 * 16  # a multiple of every block shape
    x = tcu.fill(torch.empty(segs * s, dtype=torch.float16, device="cuda"), 51, 0, "small_int")
    out = torch.full((segs,), -1.0, dtype=torch.float16, device="cuda")
    assert ref.tcu_ref_segmented_reduce(x.data_ptr(), out.data_ptr(), segs, s, variant, wpb, stream()) == 0
    torch.cuda.synchronize()
    want = oracle.np_segmented_reduce(bits(x), s)
    assert np.abs(want).max() <= 2048  # exactly representable in fp16
    assert np.array_equal(out.float().cpu().numpy().astype(np.float64), want)
    mine = tcu.segmented_reduce(x, s, out_dtype=torch.float16)
    assert torch.equal(mine, out)


@pytest.mark.parametrize("s,variant,wpb", SCAN_CASES)
def test_reference_scan_equals_oracle_and_library(ref, s, variant, wpb):
    import tcu_scope_b200 as tcu
    segs = 64 * 16
    x = tcu.fill(torch.empty(segs * s, dtype=torch.float16, device="cuda"), 52, 0, "small_int")
    out = torch.full((segs * s,), -1.0, dtype=torch.float16, device="cuda")
    assert ref.tcu_ref_segmented_scan(x.data_ptr(), out.data_ptr(), segs, s, variant, wpb, stream()) == 0
    torch.cuda.synchronize()
    want = oracle.np_segmented_scan(bits(x), s)
    assert np.array_equal(out.float().cpu().numpy().astype(np.float64), want)
    mine = tcu.segmented_scan(x, s, out_dtype=torch.float16)
    assert torch.equal(mine, out)


def test_reference_fill_value_is_a_distribution_here(ref):
    """The reference fills its inputs with half(0.001) (seg_wmma_16n.cu:38); on that input its
    16-element reduction and this library agree to fp16 rounding."""
    import tcu_scope_b200 as tcu
    segs = 128 * 16
    x = tcu.fill(torch.empty(segs * 16, dtype=torch.float16, device="cuda"), 0, 0, "const_0p001")
    out = torch.empty(segs, dtype=torch.float16, device="cuda")
    assert ref.tcu_ref_segmented_reduce(x.data_ptr(), out.data_ptr(), segs, 16, 0, 8, stream()) == 0
    torch.cuda.synchronize()
    want = oracle.np_segmented_reduce(bits(x), 16)
    assert oracle.np_check_f16(bits(out), want, 2)[0] == 0
    assert oracle.np_check_f16(bits(tcu.segmented_reduce(x, 16, out_dtype=torch.float16)), want, 1)[0] == 0
