"""Multi-GPU layer: one process per GPU, work sharded by whole segments.

Segmented operations need no communication at all: rank r owns the contiguous
segments ``shard_range(num_segments, r, world)`` and keeps its outputs.  The
full reduction and the full scan add ONE collective: an all-gather of one
double per rank (the per-shard totals).  The reference is single-GPU
(src/init/cuda.cpp:45 selects one device), so this layer has no counterpart
there.

Two ways to move those totals:

* ``PeerGroup`` (the fast one): the kernels exchange the totals themselves.  The
  reduction kernel's last thread block stores {total, sequence number} into a
  slot array in every rank's memory; the scan kernel waits, bounded, for the
  earlier ranks' totals in its own memory.  No collective per call; the process
  group is used once, at set-up, to pass around the handles of the slot arrays.
* ``sharded_full_reduce`` / ``sharded_full_scan``: one ``all_gather`` per call.
  The gather step is a parameter so that the host logic can be exercised on CPU
  with the ``gloo`` backend: ``local_total`` / ``local_scan`` are callables that
  run the device kernels in production and a CPU stand-in in the CPU tests.
"""
from __future__ import annotations

import ctypes
from typing import Callable

import torch
import torch.distributed as dist

HANDLE_BYTES = 64  # TCU_MGPU_HANDLE_BYTES


def shard_range(num_units: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, balanced split of ``num_units`` whole units (segments or
    16-element groups) over ``world`` ranks: [begin, end) of rank ``rank``."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    return num_units * rank // world, num_units * (rank + 1) // world


def gather_totals(local_total: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather one float64 per rank; returns float64[world] on the same device."""
    if local_total.dtype != torch.float64 or local_total.numel() != 1:
        raise TypeError("local_total must be a float64 tensor with one element")
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return local_total.reshape(1).clone()
    out = torch.empty(world, dtype=torch.float64, device=local_total.device)
    dist.all_gather_into_tensor(out, local_total.reshape(1), group=group)
    return out


def sharded_full_reduce(local_total_fn: Callable[[], torch.Tensor], group=None) -> torch.Tensor:
    """Each rank reduces its shard to one float64, the totals are gathered and
    every rank adds them in rank order (same result everywhere).  Returns a
    float64[1] tensor holding the global sum."""
    totals = gather_totals(local_total_fn(), group)
    return totals.sum(dtype=torch.float64).reshape(1)


def sharded_full_scan(local_total_fn: Callable[[], torch.Tensor],
                      local_scan_fn: Callable[[torch.Tensor, int], torch.Tensor],
                      group=None) -> torch.Tensor:
    """Full inclusive scan of an array sharded contiguously over the ranks.

    ``local_total_fn()`` -> float64[1]: sum of this rank's shard.
    ``local_scan_fn(totals, rank)`` -> the shard's scan seeded with the sum of
    ``totals[:rank]`` (the device kernel adds that carry itself, inside its
    first tile; no extra pass over the output).
    """
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    totals = gather_totals(local_total_fn(), group)
    return local_scan_fn(totals, rank)


def exchange_handles(handle: bytes, group=None) -> bytes:
    """All ranks' set-up handles in rank order (one all-gather of HANDLE_BYTES bytes each).
    With the ``gloo`` backend the bytes travel as a CPU tensor, with ``nccl`` as a CUDA tensor."""
    if len(handle) != HANDLE_BYTES:
        raise ValueError("a handle is HANDLE_BYTES bytes")
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return handle
    world = dist.get_world_size(group)
    on_gpu = dist.get_backend(group) == "nccl"
    mine = torch.frombuffer(bytearray(handle), dtype=torch.uint8)
    if on_gpu:
        mine = mine.cuda()
    out = torch.empty(world * HANDLE_BYTES, dtype=torch.uint8, device=mine.device)
    dist.all_gather_into_tensor(out, mine, group=group)
    return bytes(out.cpu().numpy().tobytes())


class PeerGroup:
    """One rank's end of the kernel-level exchange (``tcu_mgpu_*`` of the C ABI).

    Every rank constructs one after ``init_process_group`` (collective: the
    handles of the slot arrays are gathered once), then makes the same sequence
    of ``full_reduce`` / ``full_scan`` calls; ``close`` is collective as well --
    peers store into this rank's memory until their last call has finished.
    """

    def __init__(self, group=None, l2_keep_bytes: int | None = None):
        from . import _lib, ops
        self._lib, self._ops, self._group = _lib.load(), ops, group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self._ctx = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(HANDLE_BYTES)
        ops._check(self._lib.tcu_mgpu_ctx_create(ctypes.byref(self._ctx), self.rank, self.world, handle),
                   "tcu_mgpu_ctx_create")
        if self.world > 1:
            handles = exchange_handles(handle.raw, group)
            ops._check(self._lib.tcu_mgpu_ctx_connect(self._ctx, handles), "tcu_mgpu_ctx_connect")
            dist.barrier(group)  # nobody stores into a slot array that is not mapped everywhere yet
        if l2_keep_bytes is not None:
            self.set_l2_keep_bytes(l2_keep_bytes)

    def set_l2_keep_bytes(self, nbytes: int) -> None:
        self._ops._check(self._lib.tcu_mgpu_ctx_set_l2_keep_bytes(self._ctx, nbytes),
                         "tcu_mgpu_ctx_set_l2_keep_bytes")

    def full_reduce(self, x: torch.Tensor, out: torch.Tensor | None = None,
                    out_f64: torch.Tensor | None = None):
        """Sum over ALL ranks' shards, on every rank: (float32[1], float64[1])."""
        ops = self._ops
        if x.dtype != torch.float16 or not x.is_cuda or not x.is_contiguous():
            raise TypeError("the shard must be a contiguous float16 CUDA tensor")
        if out is None:
            out = torch.empty(1, dtype=torch.float32, device=x.device)
        if out_f64 is None:
            out_f64 = torch.empty(1, dtype=torch.float64, device=x.device)
        ops._check(self._lib.tcu_mgpu_full_reduce_f16(self._ctx, x.data_ptr(), out.data_ptr(),
                                                      out_f64.data_ptr(), x.numel(), ops._stream()),
                   "tcu_mgpu_full_reduce_f16")
        return out, out_f64

    def full_scan(self, x: torch.Tensor, out: torch.Tensor | None = None,
                  out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """This rank's part of the inclusive scan of the whole (sharded) array."""
        ops = self._ops
        if x.dtype != torch.float16 or not x.is_cuda or not x.is_contiguous():
            raise TypeError("the shard must be a contiguous float16 CUDA tensor")
        if out is None:
            out = torch.empty(x.numel(), dtype=out_dtype, device=x.device)
        ops._check(self._lib.tcu_mgpu_full_scan_f16(self._ctx, x.data_ptr(), out.data_ptr(),
                                                    ops._out_code(out.dtype), x.numel(),
                                                    ops._stream()), "tcu_mgpu_full_scan_f16")
        return out

    def close(self) -> None:
        if not self._ctx:
            return
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(self._group)  # every rank's last kernel is done: nobody writes here any more
        self._lib.tcu_mgpu_ctx_destroy(self._ctx)
        self._ctx = ctypes.c_void_p()
