"""Host-side operators over torch CUDA tensors, calling the C ABI.

torch is used for device memory and streams only.  Names and argument meaning
follow the reference's benchmark drivers: ``num_segments`` segments of
``segment_size`` consecutive halves (src/reduction/seg_wmma_16n.cu:14-25); an
unsupported segment size is an error, as in the reference's dispatch
(src/reduction/seg_wmma_16n.cu:172 "invalid segment size").
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

OK = 0
ALGO = {"auto": 0, "mma": 1, "shuffle": 2, "tcgen05": 3}
OUT_F16, OUT_F32 = 0, 1
OP_SEGMENTED_REDUCE, OP_SEGMENTED_SCAN, OP_FULL_REDUCE, OP_FULL_SCAN = 0, 1, 2, 3
DIST = {"uniform_pm1": 0, "uniform_01": 1, "small_int": 2, "const_0p001": 3}


class TcuError(RuntimeError):
    def __init__(self, status: int, where: str):
        msg = _lib.load().tcu_status_string(status).decode()
        super().__init__(f"{where}: status {status} ({msg})")
        self.status = status


def _check(status: int, where: str) -> None:
    if status != OK:
        raise TcuError(status, where)


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _out_code(dtype: torch.dtype, in_dtype: torch.dtype = torch.float16) -> int:
    """16-bit outputs have the type of the input (float16 or bfloat16)."""
    if dtype == torch.float32:
        return OUT_F32
    if dtype == in_dtype and dtype in (torch.float16, torch.bfloat16):
        return OUT_F16
    raise TypeError(f"output dtype must be float32 or the input's {in_dtype}, got {dtype}")


def _require_input(x: torch.Tensor) -> str:
    """Checks the input and returns the suffix of the entry points for its type."""
    if not x.is_cuda:
        raise RuntimeError("input must be a CUDA tensor: there is no CPU path in this library")
    if x.dtype not in (torch.float16, torch.bfloat16) or not x.is_contiguous():
        raise TypeError("input must be a contiguous float16 or bfloat16 tensor")
    return "f16" if x.dtype == torch.float16 else "bf16"


def _default_out(out_dtype: torch.dtype, x: torch.Tensor) -> torch.dtype:
    return x.dtype if out_dtype in (torch.float16, torch.bfloat16) else out_dtype


def workspace_bytes(op: int, num_elements: int, segment_size: int) -> int:
    return int(_lib.load().tcu_workspace_bytes(op, num_elements, segment_size))


def _workspace(op: int, n: int, segment_size: int, device, workspace):
    need = workspace_bytes(op, n, segment_size)
    if need == 0:
        return None, 0, 0
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=device)
    return workspace, workspace.data_ptr(), workspace.numel()


def fill(out: torch.Tensor, seed: int, first_index: int = 0, dist: str = "uniform_pm1") -> torch.Tensor:
    """Fill a float16 or bfloat16 CUDA tensor with element i = f(seed, first_index + i)."""
    t = _require_input(out)
    fn = getattr(_lib.load(), f"tcu_fill_{t}")
    _check(fn(out.data_ptr(), out.numel(), seed, first_index, DIST[dist], _stream()),
           f"tcu_fill_{t}")
    return out


def segmented_reduce(x: torch.Tensor, segment_size: int, out_dtype=torch.float32, algo="auto",
                     out: torch.Tensor | None = None, workspace: torch.Tensor | None = None):
    """out[j] = sum(x[j*segment_size:(j+1)*segment_size])."""
    t = _require_input(x)
    n = x.numel()
    if segment_size <= 0 or n % segment_size:
        raise ValueError("num_elements must be a multiple of segment_size")
    segs = n // segment_size
    if out is None:
        out = torch.empty(segs, dtype=_default_out(out_dtype, x), device=x.device)
    ws, ws_ptr, ws_bytes = _workspace(OP_SEGMENTED_REDUCE, n, segment_size, x.device, workspace)
    fn = getattr(_lib.load(), f"tcu_segmented_reduce_{t}")
    _check(fn(x.data_ptr(), out.data_ptr(), _out_code(out.dtype, x.dtype), segs, segment_size,
              ALGO[algo], ws_ptr, ws_bytes, _stream()), f"tcu_segmented_reduce_{t}")
    return out


def segmented_scan(x: torch.Tensor, segment_size: int, out_dtype=torch.float16, algo="auto",
                   out: torch.Tensor | None = None, workspace: torch.Tensor | None = None,
                   exclusive: bool = False):
    """Prefix sum inside every segment of segment_size elements (inclusive unless ``exclusive``)."""
    t = _require_input(x)
    n = x.numel()
    if segment_size <= 0 or n % segment_size:
        raise ValueError("num_elements must be a multiple of segment_size")
    if out is None:
        out = torch.empty(n, dtype=_default_out(out_dtype, x), device=x.device)
    ws, ws_ptr, ws_bytes = _workspace(OP_SEGMENTED_SCAN, n, segment_size, x.device, workspace)
    code = _out_code(out.dtype, x.dtype)
    if exclusive:
        fn = getattr(_lib.load(), f"tcu_segmented_exclusive_scan_{t}")
        _check(fn(x.data_ptr(), out.data_ptr(), code, n // segment_size, segment_size, ws_ptr,
                  ws_bytes, _stream()), f"tcu_segmented_exclusive_scan_{t}")
        return out
    fn = getattr(_lib.load(), f"tcu_segmented_scan_{t}")
    _check(fn(x.data_ptr(), out.data_ptr(), code, n // segment_size, segment_size, ALGO[algo],
              ws_ptr, ws_bytes, _stream()), f"tcu_segmented_scan_{t}")
    return out


def full_reduce(x: torch.Tensor, algo="auto", workspace: torch.Tensor | None = None,
                out: torch.Tensor | None = None, out_f64: torch.Tensor | None = None):
    """Sum of all elements; returns (float32[1], float64[1]) device tensors."""
    t = _require_input(x)
    n = x.numel()
    if out is None:
        out = torch.empty(1, dtype=torch.float32, device=x.device)
    if out_f64 is None:
        out_f64 = torch.empty(1, dtype=torch.float64, device=x.device)
    ws, ws_ptr, ws_bytes = _workspace(OP_FULL_REDUCE, n, n, x.device, workspace)
    fn = getattr(_lib.load(), f"tcu_full_reduce_{t}")
    _check(fn(x.data_ptr(), out.data_ptr(), out_f64.data_ptr(), n, ALGO[algo], ws_ptr, ws_bytes,
              _stream()), f"tcu_full_reduce_{t}")
    return out, out_f64


def full_scan(x: torch.Tensor, out_dtype=torch.float32, algo="auto",
              shard_totals: torch.Tensor | None = None, shard_index: int = 0,
              out: torch.Tensor | None = None, workspace: torch.Tensor | None = None,
              exclusive: bool = False):
    """Inclusive prefix sum over the whole tensor (seeded by earlier shards' totals)."""
    t = _require_input(x)
    n = x.numel()
    if out is None:
        out = torch.empty(n, dtype=_default_out(out_dtype, x), device=x.device)
    if shard_totals is not None and shard_totals.dtype != torch.float64:
        raise TypeError("shard_totals must be float64")
    ws, ws_ptr, ws_bytes = _workspace(OP_FULL_SCAN, n, n, x.device, workspace)
    if exclusive:
        if shard_totals is not None:
            raise ValueError("the exclusive full scan has no multi-GPU seed")
        fn = getattr(_lib.load(), f"tcu_full_exclusive_scan_{t}")
        _check(fn(x.data_ptr(), out.data_ptr(), _out_code(out.dtype, x.dtype), n, ws_ptr, ws_bytes,
                  _stream()), f"tcu_full_exclusive_scan_{t}")
        return out
    st_ptr = shard_totals.data_ptr() if shard_totals is not None else None
    fn = getattr(_lib.load(), f"tcu_full_scan_{t}")
    _check(fn(x.data_ptr(), out.data_ptr(), _out_code(out.dtype, x.dtype), n, st_ptr, shard_index,
              ALGO[algo], ws_ptr, ws_bytes, _stream()), f"tcu_full_scan_{t}")
    return out


def num_sms() -> int:
    """Streaming multiprocessors of the current device (the grid size of the persistent kernels)."""
    return int(_lib.load().tcu_num_sms())


def device_error(clear: bool = True) -> int:
    """Synchronise and return the device-side error bits (0 = none)."""
    bits = ctypes.c_uint(0)
    _lib.load().tcu_device_error(ctypes.byref(bits), 1 if clear else 0)
    return int(bits.value)


class HostContext:
    """Runs the operators on HOST buffers (pinned torch tensors or numpy arrays).

    Owns two staging buffers of ``chunk_elements`` halves on the device and two
    streams; host -> device copies, kernels and device -> host copies of
    consecutive chunks overlap.
    """

    def __init__(self, chunk_elements: int = 1 << 26):
        self._ctx = ctypes.c_void_p()
        _check(_lib.load().tcu_host_ctx_create(ctypes.byref(self._ctx), chunk_elements),
               "tcu_host_ctx_create")

    def close(self) -> None:
        if self._ctx:
            _lib.load().tcu_host_ctx_destroy(self._ctx)
            self._ctx = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def reduce_sweep(self, h_in: torch.Tensor, segment_sizes, h_outs, algo="auto"):
        """Segmented reductions of one host array at several segment sizes; each chunk of the
        input crosses the bus once.  h_outs[i]: host tensor of h_in.numel() // segment_sizes[i]."""
        if h_in.is_cuda or h_in.dtype != torch.float16 or not h_in.is_contiguous():
            raise TypeError("h_in must be a contiguous float16 host tensor")
        k = len(segment_sizes)
        if k != len(h_outs) or k == 0:
            raise ValueError("one output per segment size")
        code = _out_code(h_outs[0].dtype)
        for s, o in zip(segment_sizes, h_outs):
            if o.is_cuda or not o.is_contiguous() or _out_code(o.dtype) != code:
                raise TypeError("outputs must be contiguous host tensors of one dtype")
            if o.numel() * s != h_in.numel():
                raise ValueError("output size does not match num_elements / segment_size")
        sizes = (ctypes.c_size_t * k)(*segment_sizes)
        outs = (ctypes.c_void_p * k)(*[o.data_ptr() for o in h_outs])
        _check(_lib.load().tcu_host_segmented_reduce_sweep_f16(
            self._ctx, h_in.data_ptr(), h_in.numel(), k, sizes, outs, code, ALGO[algo]),
            "tcu_host_segmented_reduce_sweep_f16")
        return h_outs

    def run(self, op: int, h_in: torch.Tensor, h_out: torch.Tensor, segment_size: int = 0,
            algo="auto") -> torch.Tensor:
        if h_in.is_cuda or h_out.is_cuda:
            raise RuntimeError("HostContext.run takes host tensors")
        if h_in.dtype != torch.float16 or not h_in.is_contiguous() or not h_out.is_contiguous():
            raise TypeError("h_in must be contiguous float16, h_out contiguous")
        _check(_lib.load().tcu_host_run_f16(self._ctx, op, h_in.data_ptr(), h_out.data_ptr(),
                                            _out_code(h_out.dtype), h_in.numel(), segment_size,
                                            ALGO[algo]), "tcu_host_run_f16")
        return h_out
