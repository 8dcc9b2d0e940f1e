"""Writes tests/golden/golden.npz: seeded cases with their float64 oracle outputs.

The reference project holds no golden vectors for this path, so these pin the
oracle itself (numpy restatement, checked by the tests against the C one and
against closed forms); regenerate with ``python tests/golden/make_golden.py``.
Inputs are not stored: a case is (seed, first_index, dist, n, segment_size),
and the generator is part of what is pinned (the first 64 input bit patterns
of each case are stored too).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402

CASES = [
    # name, op, seed, first_index, dist, n, segment_size
    ("reduce_s16", "reduce", 1, 0, "uniform_pm1", 4096, 16),
    ("reduce_s64", "reduce", 2, 12345, "uniform_pm1", 4096, 64),
    ("reduce_s256", "reduce", 3, 0, "uniform_pm1", 8192, 256),
    ("reduce_s4096", "reduce", 4, 1 << 33, "uniform_01", 16384, 4096),
    ("reduce_const", "reduce", 5, 0, "const_0p001", 2048, 1024),
    ("scan_s16", "scan", 6, 0, "uniform_pm1", 1024, 16),
    ("scan_s256", "scan", 7, 99, "uniform_pm1", 2048, 256),
    ("scan_s4096", "scan", 8, 0, "uniform_pm1", 8192, 4096),
    ("scan_full_01", "scan", 9, 0, "uniform_01", 8192, 8192),
    ("scan_ints", "scan", 10, 7, "small_int", 2048, 512),
]


def main():
    out = {}
    for name, op, seed, first, dist, n, s in CASES:
        x = oracle.np_fill_f16(n, seed, first, dist)
        ref = oracle.np_segmented_reduce(x, s) if op == "reduce" else oracle.np_segmented_scan(x, s)
        out[name + "/head_bits"] = x[:64].copy()
        out[name + "/ref"] = ref
        out[name + "/meta"] = np.array([seed, first, oracle.DIST[dist], n, s, 0 if op == "reduce" else 1],
                                       dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
    print("wrote", len(CASES), "cases")


if __name__ == "__main__":
    main()
