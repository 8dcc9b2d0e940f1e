"""CPU tests of the boundary: the library builds, loads and exports every
symbol include/tcu_scope.h declares; argument validation that needs no GPU."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tcu_scope.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tcu_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_operator_surface():
    syms = declared_symbols()
    for must in ["tcu_segmented_reduce_f16", "tcu_segmented_scan_f16", "tcu_full_reduce_f16",
                 "tcu_full_scan_f16", "tcu_workspace_bytes", "tcu_fill_f16", "tcu_host_run_f16",
                 "tcu_status_string"]:
        assert must in syms


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(built_library)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/tcu_scope.h but not exported"


def test_python_binding_covers_every_symbol(built_library):
    from tcu_scope_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    _lib.load()


def test_no_gpu_calls_needed_for_sizes(built_library):
    import tcu_scope_b200 as tcu
    tile = tcu._lib.load().tcu_tile_elements()
    assert tile == 16384
    assert tcu.workspace_bytes(tcu.OP_SEGMENTED_REDUCE, 1 << 20, 256) == 0
    assert tcu.workspace_bytes(tcu.OP_SEGMENTED_SCAN, 1 << 20, tile) == 0
    assert tcu.workspace_bytes(tcu.OP_SEGMENTED_REDUCE, 1 << 20, 2 * tile) > 0
    n = 1 << 24
    assert tcu.workspace_bytes(tcu.OP_FULL_SCAN, n, n) >= (n // tile) * 8
    assert tcu.workspace_bytes(tcu.OP_FULL_REDUCE, n, n) > 0
    assert b"workspace" in tcu._lib.load().tcu_status_string(5)


def test_validation_rejects_before_touching_the_gpu(built_library):
    """These paths return before any CUDA call, so they run on a GPU-less box."""
    import tcu_scope_b200 as tcu
    lib = tcu._lib.load()
    # segment size zero
    assert lib.tcu_segmented_reduce_f16(None, None, 1, 4, 0, 0, None, 0, None) == 2
    assert lib.tcu_segmented_scan_f16(None, None, 0, 4, 0, 0, None, 0, None) == 2
    # the ablation and tcgen05 variants exist for powers of two >= 16 only
    for algo in (2, 3):
        assert lib.tcu_segmented_reduce_f16(None, None, 1, 4, 48, algo, None, 0, None) == 2
    # zero segments is a no-op
    assert lib.tcu_segmented_reduce_f16(None, None, 1, 0, 16, 0, None, 0, None) == 0
    # unknown output type / algorithm
    assert lib.tcu_segmented_reduce_f16(None, None, 7, 4, 16, 0, None, 0, None) == 2
    assert lib.tcu_segmented_reduce_f16(None, None, 1, 4, 16, 9, None, 0, None) == 2
    # null and misaligned pointers
    assert lib.tcu_segmented_reduce_f16(None, None, 1, 4, 16, 0, None, 0, None) == 1
    assert lib.tcu_segmented_scan_f16(0x1008, 0x2000, 0, 4, 16, 0, None, 0, None) == 1
    # size overflow
    assert lib.tcu_segmented_reduce_f16(0x1000, 0x2000, 1, 1 << 62, 1 << 20, 0, None, 0, None) == 1
    # full ops: element count must be a positive multiple of 16
    assert lib.tcu_full_reduce_f16(0x1000, 0x2000, None, 24, 0, None, 0, None) == 1
    assert lib.tcu_full_scan_f16(0x1000, 0x2000, 1, 40, None, 0, 0, None, 0, None) == 1
    assert lib.tcu_fill_f16(0x1000, 12, 0, 0, 0, None) == 1
    assert lib.tcu_fill_f16(0x1000, 16, 0, 0, 17, None) == 2
