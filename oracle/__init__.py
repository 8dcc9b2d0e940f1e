"""CPU oracle for the segmented / full reduce and inclusive scan -- TEST INFRASTRUCTURE ONLY.

Two restatements of the same definition, checked against each other and against
the fixtures in tests/golden/:
  * numpy (this file): float64 sums over the fp16-rounded inputs;
  * C (tcu_oracle.c, built by ``make -C oracle``): the same loops, plus the
    timed plain-CPU baseline.

PARITY UNPINNED: the reference (c3sr/tcu_scope) has no golden vectors or tests
for this path; its validation blocks are compiled out
(src/reduction/seg_wmma_16n.cu:82-109, src/prefixsum/wmma_3kers.cu:92-129).
They intended a sequential running sum per segment compared element by
element -- that is what is restated here, in double precision.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may
import this package; the shipped library never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
C_LIB_PATH = os.path.join(HERE, "libtcu_oracle.so")

DIST = {"uniform_pm1": 0, "uniform_01": 1, "small_int": 2, "const_0p001": 3}

# ----------------------------------------------------------------- numpy side

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        x = ((x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        x = ((x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return x ^ (x >> np.uint64(31))


def np_fill_f16(n: int, seed: int, first_index: int = 0, dist: str = "uniform_pm1",
                fmt: str = "f16") -> np.ndarray:
    """uint16 bit patterns of the seeded input, element i = f(seed, first_index + i), rounded
    to fp16 or (fmt="bf16") to bfloat16."""
    key = _splitmix64(np.array([seed], dtype=np.uint64))[0]
    with np.errstate(over="ignore"):
        idx = (np.arange(n, dtype=np.uint64) + np.uint64(first_index) + key) & _M64
    u24 = (_splitmix64(idx) >> np.uint64(40)).astype(np.int64)
    code = DIST[dist]
    if code == 0:
        v = (u24 - (1 << 23)).astype(np.float32) * np.float32(2.0 ** -23)
    elif code == 1:
        v = u24.astype(np.float32) * np.float32(2.0 ** -24)
    elif code == 2:
        v = ((u24 % 5) - 2).astype(np.float32)
    else:
        v = np.full(n, 0.001, dtype=np.float32)
    if fmt == "bf16":
        return f32_to_bf16_bits(v)
    return v.astype(np.float16).view(np.uint16)


def _as_f64(in_u16: np.ndarray, fmt: str = "f16") -> np.ndarray:
    """float64 values of 16-bit patterns: fp16 (the reference's type) or bfloat16."""
    u = np.ascontiguousarray(in_u16, dtype=np.uint16)
    if fmt == "bf16":  # a bfloat16 is the upper half of a float32
        return (u.astype(np.uint32) << np.uint32(16)).view(np.float32).astype(np.float64)
    return u.view(np.float16).astype(np.float64)


def f32_to_bf16_bits(v: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (finite inputs)."""
    u = np.ascontiguousarray(v, dtype=np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def np_segmented_reduce(in_u16: np.ndarray, segment_size: int, fmt: str = "f16") -> np.ndarray:
    """Segment j = in[j*S:(j+1)*S] (src/reduction/seg_wmma_16n.cu:14-25); float64 sums."""
    x = _as_f64(in_u16, fmt).reshape(-1, segment_size)
    return x.sum(axis=1, dtype=np.float64)


def np_segmented_scan(in_u16: np.ndarray, segment_size: int, fmt: str = "f16") -> np.ndarray:
    """Inclusive running sum inside each segment (U[i][j]=1 for i<=j,
    src/prefixsum/kernel.cuh:60,79-81; the check the authors intended,
    src/prefixsum/wmma_3kers.cu:97-108)."""
    x = _as_f64(in_u16, fmt).reshape(-1, segment_size)
    return np.cumsum(x, axis=1, dtype=np.float64).reshape(-1)


def np_tile256_scan_algebra(in_u16: np.ndarray) -> np.ndarray:
    """A.U + (L.A).1 over one row-major 16x16 tile (src/prefixsum/kernel.cuh:316-361)."""
    a = _as_f64(in_u16).reshape(16, 16)
    i, j = np.indices((16, 16))
    u = (i <= j).astype(np.float64)
    l = (i > j).astype(np.float64)
    ones = np.ones((16, 16))
    return (a @ u + (l @ a) @ ones).reshape(-1)


def half_order_key(bits: np.ndarray) -> np.ndarray:
    b = bits.astype(np.int32)
    mag = b & 0x7FFF
    return np.where(b & 0x8000, -mag, mag)


def np_check_f32(got: np.ndarray, ref: np.ndarray, rel: float = 1e-3, abs_floor: float = 1e-5):
    """Returns (violations, max_abs_err, max_rel_err): |got-ref| <= max(rel*|ref|, abs_floor)."""
    g = got.astype(np.float64)
    err = np.abs(g - ref)
    tol = np.maximum(rel * np.abs(ref), abs_floor)
    bad = ~np.isfinite(g) | (err > tol)
    big = np.abs(ref) > abs_floor
    max_rel = float((err[big] / np.abs(ref[big])).max()) if big.any() else 0.0
    return int(bad.sum()), float(np.nanmax(err)) if err.size else 0.0, max_rel


def np_check_f16(got_bits: np.ndarray, ref: np.ndarray, max_ulp: int = 2, fmt: str = "f16"):
    """Returns (violations, worst): distance in representable halves (bfloat16s) from the
    correctly rounded reference."""
    g = np.ascontiguousarray(got_bits, dtype=np.uint16)
    if fmt == "bf16":
        ref_bits = f32_to_bf16_bits(ref.astype(np.float32))
        nan = ((g & 0x7F80) == 0x7F80) & ((g & 0x7F) != 0)
    else:
        ref_bits = ref.astype(np.float16).view(np.uint16)
        nan = ((g & 0x7C00) == 0x7C00) & ((g & 0x3FF) != 0)
    d = np.abs(half_order_key(g) - half_order_key(ref_bits))
    bad = nan | (d > max_ulp)
    return int(bad.sum()), int(d[~nan].max()) if (~nan).any() else 0


# --------------------------------------------------------------------- C side

_c = None


def build_c(force: bool = False) -> str:
    if force or not os.path.exists(C_LIB_PATH) or (
            os.path.getmtime(C_LIB_PATH) < os.path.getmtime(os.path.join(HERE, "tcu_oracle.c"))):
        subprocess.run(["make", "-C", HERE, "libtcu_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return C_LIB_PATH


def c_lib() -> ctypes.CDLL:
    global _c
    if _c is not None:
        return _c
    build_c()
    lib = ctypes.CDLL(C_LIB_PATH)
    vp, sz, i32, u64 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_uint64
    dbl_p = ctypes.POINTER(ctypes.c_double)
    sig = {
        "tcu_oracle_f32_to_f16": (ctypes.c_uint16, [ctypes.c_float]),
        "tcu_oracle_f64_to_f16": (ctypes.c_uint16, [ctypes.c_double]),
        "tcu_oracle_f16_to_f64": (ctypes.c_double, [ctypes.c_uint16]),
        "tcu_oracle_hash": (u64, [u64, u64]),
        "tcu_oracle_fill_f16": (None, [vp, sz, u64, u64, i32]),
        "tcu_oracle_segmented_reduce": (None, [vp, vp, sz, sz]),
        "tcu_oracle_segmented_scan": (None, [vp, vp, sz, sz]),
        "tcu_oracle_tile256_scan_algebra": (None, [vp, vp]),
        "tcu_oracle_check_f32": (sz, [vp, vp, sz, ctypes.c_double, ctypes.c_double, dbl_p, dbl_p]),
        "tcu_oracle_check_f16": (sz, [vp, vp, sz, i32, ctypes.POINTER(i32)]),
        "tcu_cpu_segmented_reduce": (i32, [vp, vp, sz, sz, i32]),
        "tcu_cpu_segmented_scan": (i32, [vp, vp, i32, sz, sz, i32]),
        "tcu_cpu_full_reduce": (i32, [vp, vp, sz, i32]),
        "tcu_cpu_full_scan": (i32, [vp, vp, sz, i32]),
        "tcu_cpu_available_cores": (i32, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _c = lib
    return lib


def _ptr(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def c_fill_f16(n: int, seed: int, first_index: int = 0, dist: str = "uniform_pm1") -> np.ndarray:
    out = np.empty(n, dtype=np.uint16)
    c_lib().tcu_oracle_fill_f16(_ptr(out), n, seed, first_index, DIST[dist])
    return out


def c_segmented_reduce(in_u16: np.ndarray, segment_size: int) -> np.ndarray:
    x = np.ascontiguousarray(in_u16, dtype=np.uint16)
    out = np.empty(x.size // segment_size, dtype=np.float64)
    c_lib().tcu_oracle_segmented_reduce(_ptr(x), _ptr(out), out.size, segment_size)
    return out


def c_segmented_scan(in_u16: np.ndarray, segment_size: int) -> np.ndarray:
    x = np.ascontiguousarray(in_u16, dtype=np.uint16)
    out = np.empty(x.size, dtype=np.float64)
    c_lib().tcu_oracle_segmented_scan(_ptr(x), _ptr(out), x.size // segment_size, segment_size)
    return out


def c_check_f32(got: np.ndarray, ref: np.ndarray, rel: float = 1e-3, abs_floor: float = 1e-5):
    g = np.ascontiguousarray(got, dtype=np.float32)
    r = np.ascontiguousarray(ref, dtype=np.float64)
    ma, mr = ctypes.c_double(0), ctypes.c_double(0)
    bad = c_lib().tcu_oracle_check_f32(_ptr(g), _ptr(r), g.size, rel, abs_floor,
                                       ctypes.byref(ma), ctypes.byref(mr))
    return int(bad), ma.value, mr.value


def c_check_f16(got_bits: np.ndarray, ref: np.ndarray, max_ulp: int = 2):
    g = np.ascontiguousarray(got_bits, dtype=np.uint16)
    r = np.ascontiguousarray(ref, dtype=np.float64)
    worst = ctypes.c_int(0)
    bad = c_lib().tcu_oracle_check_f16(_ptr(g), _ptr(r), g.size, max_ulp, ctypes.byref(worst))
    return int(bad), worst.value


# ------------------------------------------------- the reference's own kernels
REF_LIB_PATH = os.path.join(HERE, "_ref", "libtcu_ref.so")
_ref = None


def ref_lib():
    """oracle/_ref/libtcu_ref.so: the reference's WMMA kernels compiled unmodified for
    sm_100a by ``make -C oracle ref`` (needs the reference checkout; the built file
    travels to the GPU box).  Returns None when it has not been built."""
    global _ref
    if _ref is not None:
        return _ref
    if not os.path.exists(REF_LIB_PATH):
        return None
    lib = ctypes.CDLL(REF_LIB_PATH)
    vp, sz, i32 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    for name in ("tcu_ref_segmented_reduce", "tcu_ref_segmented_scan"):
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = i32, [vp, vp, sz, sz, i32, i32, vp]
    _ref = lib
    return lib


# ---------------------------------------------------------- CUB library baseline
CUB_LIB_PATH = os.path.join(HERE, "libtcu_cub.so")
_cub = None


def cub_lib():
    """oracle/libtcu_cub.so (``make -C oracle cub``): CUB device-wide and Thrust reduce / scan
    on the same inputs, the library baselines.  None when it has not been built."""
    global _cub
    if _cub is not None:
        return _cub
    if not os.path.exists(CUB_LIB_PATH):
        return None
    lib = ctypes.CDLL(CUB_LIB_PATH)
    vp, sz, i32 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    lib.tcu_cub_run.restype = i32
    lib.tcu_cub_run.argtypes = [i32, vp, vp, sz, sz, vp, ctypes.POINTER(sz), vp]
    lib.tcu_thrust_run.restype = i32
    lib.tcu_thrust_run.argtypes = [i32, vp, vp, sz, sz, vp]
    _cub = lib
    return lib


CUB_FULL_REDUCE, CUB_SEG_REDUCE, CUB_FULL_SCAN, CUB_SEG_SCAN_F32, CUB_SEG_SCAN_F16 = range(5)
THRUST_REDUCE, THRUST_REDUCE_BY_KEY, THRUST_SCAN, THRUST_SCAN_BY_KEY = range(4)


def cub_temp_bytes(op: int, n: int, segment_size: int) -> int:
    need = ctypes.c_size_t(0)
    rc = cub_lib().tcu_cub_run(op, None, None, n, segment_size, None, ctypes.byref(need), None)
    assert rc == 0, rc
    return max(int(need.value), 1)
