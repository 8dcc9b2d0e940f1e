"""tcu_scope_b200: segmented / full sum-reduction and inclusive prefix sum over
fp16 arrays on B200 tensor cores, behind a C ABI (include/tcu_scope.h).

The CUDA library is the product; this package is the thin host layer the tests
and the benchmark use.  Importing it loads ``libtcu_scope.so`` and fails loudly
if it has not been built.
"""
from . import _lib

_lib.load()

from .ops import (  # noqa: E402
    ALGO, DIST, OP_FULL_REDUCE, OP_FULL_SCAN, OP_SEGMENTED_REDUCE, OP_SEGMENTED_SCAN,
    HostContext, TcuError, device_error, fill, full_reduce, full_scan, num_sms, segmented_reduce,
    segmented_scan, workspace_bytes,
)
from .sharded import PeerGroup, sharded_full_reduce, sharded_full_scan, shard_range  # noqa: E402

__all__ = [
    "ALGO", "DIST", "OP_FULL_REDUCE", "OP_FULL_SCAN", "OP_SEGMENTED_REDUCE", "OP_SEGMENTED_SCAN",
    "HostContext", "TcuError", "device_error", "fill", "full_reduce", "full_scan", "num_sms",
    "segmented_reduce", "segmented_scan", "workspace_bytes", "sharded_full_reduce",
    "sharded_full_scan", "shard_range", "PeerGroup",
]
