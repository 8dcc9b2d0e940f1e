"""ctypes binding of libtcu_scope.so: one Python callable per symbol of include/tcu_scope.h.

There is no fallback: if the shared library is missing or a symbol cannot be
resolved, importing fails with the reason.
"""
from __future__ import annotations

import ctypes
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libtcu_scope.so")

c_size_t, c_int, c_void_p = ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p

# name -> (restype, argtypes); kept in the order of the header.
SIGNATURES = {
    "tcu_segmented_reduce_f16": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_size_t, c_int,
                                         c_void_p, c_size_t, c_void_p]),
    "tcu_segmented_scan_f16": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_size_t, c_int,
                                       c_void_p, c_size_t, c_void_p]),
    "tcu_full_reduce_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_void_p,
                                    c_size_t, c_void_p]),
    "tcu_full_scan_f16": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_void_p, c_int, c_int,
                                  c_void_p, c_size_t, c_void_p]),
    "tcu_segmented_exclusive_scan_f16": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_size_t,
                                                 c_void_p, c_size_t, c_void_p]),
    "tcu_full_exclusive_scan_f16": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_void_p,
                                            c_size_t, c_void_p]),
    "tcu_segmented_reduce_bf16": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_size_t, c_int,
                                          c_void_p, c_size_t, c_void_p]),
    "tcu_segmented_scan_bf16": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_size_t, c_int,
                                        c_void_p, c_size_t, c_void_p]),
    "tcu_segmented_exclusive_scan_bf16": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_size_t,
                                                  c_void_p, c_size_t, c_void_p]),
    "tcu_full_exclusive_scan_bf16": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_void_p,
                                             c_size_t, c_void_p]),
    "tcu_full_reduce_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_void_p,
                                     c_size_t, c_void_p]),
    "tcu_full_scan_bf16": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_void_p, c_int, c_int,
                                   c_void_p, c_size_t, c_void_p]),
    "tcu_fill_bf16": (c_int, [c_void_p, c_size_t, ctypes.c_uint64, ctypes.c_uint64, c_int,
                              c_void_p]),
    "tcu_full_scan_f16_static": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_void_p, c_int,
                                         c_int, c_void_p]),
    "tcu_workspace_bytes": (c_size_t, [c_int, c_size_t, c_size_t]),
    "tcu_fill_f16": (c_int, [c_void_p, c_size_t, ctypes.c_uint64, ctypes.c_uint64, c_int,
                             c_void_p]),
    "tcu_host_ctx_create": (c_int, [ctypes.POINTER(c_void_p), c_size_t]),
    "tcu_host_ctx_destroy": (None, [c_void_p]),
    "tcu_host_run_f16": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_size_t, c_size_t,
                                 c_int]),
    "tcu_host_segmented_reduce_sweep_f16": (c_int, [c_void_p, c_void_p, c_size_t, c_int,
                                                    ctypes.POINTER(c_size_t),
                                                    ctypes.POINTER(c_void_p), c_int, c_int]),
    "tcu_mgpu_ctx_create": (c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_void_p]),
    "tcu_mgpu_ctx_connect": (c_int, [c_void_p, c_void_p]),
    "tcu_mgpu_ctx_connect_local": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "tcu_mgpu_ctx_set_l2_keep_bytes": (c_int, [c_void_p, c_size_t]),
    "tcu_mgpu_ctx_destroy": (None, [c_void_p]),
    "tcu_mgpu_full_reduce_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "tcu_mgpu_full_scan_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_void_p]),
    "tcu_device_error": (c_int, [ctypes.POINTER(ctypes.c_uint), c_int]),
    "tcu_test_set_wait_limits": (c_int, [ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_uint]),
    "tcu_test_inject": (c_int, [c_int, ctypes.c_ulonglong]),
    "tcu_tile_elements": (c_int, []),
    "tcu_num_sms": (c_int, []),
    "tcu_status_string": (ctypes.c_char_p, [c_int]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library once and type every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python tcu_scope_b200/build.py` "
            "(there is no CPU or PyTorch fallback for these operators)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib
