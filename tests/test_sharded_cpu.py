"""World-size-2 gloo tests of the multi-GPU host logic (no GPU): the sharding
arithmetic and the one collective (all-gather of per-shard totals)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_range_partitions_whole_units():
    from tcu_scope_b200.sharded import shard_range
    for units in (1, 7, 8, 1000, 2 ** 24):
        for world in (1, 2, 3, 8):
            edges = [shard_range(units, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == units
            for a, b in zip(edges, edges[1:]):
                assert a[1] == b[0]
            sizes = [e - b for b, e in edges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


def _worker(rank, world, port, n, seed, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from tcu_scope_b200.sharded import shard_range, sharded_full_reduce, sharded_full_scan
    b, e = shard_range(n // 16, rank, world)
    b, e = b * 16, e * 16
    x = oracle.np_fill_f16(e - b, seed, b, "uniform_01").view(np.float16).astype(np.float64)

    # CPU stand-ins for the device kernels: same contract as ops.full_reduce / ops.full_scan
    def local_total():
        return torch.tensor([x.sum()], dtype=torch.float64)

    def local_scan(totals, r):
        carry = float(totals[:r].sum())
        return torch.from_numpy((np.cumsum(x) + carry).astype(np.float32))

    total = sharded_full_reduce(local_total)
    scan = sharded_full_scan(local_total, local_scan)
    ret[rank] = (float(total[0]), scan.numpy(), (b, e))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_full_ops_gloo(world):
    import oracle
    n, seed = 16 * 1001, 77
    port = 29500 + (os.getpid() % 2000) + world
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    ret = mgr.dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, seed, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    whole = oracle.np_fill_f16(n, seed, 0, "uniform_01")
    ref_scan = oracle.np_segmented_scan(whole, n)
    for r in range(world):
        total, scan, (b, e) = ret[r]
        assert total == pytest.approx(ref_scan[-1], rel=1e-12)
        assert oracle.np_check_f32(scan, ref_scan[b:e])[0] == 0


def _handle_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from tcu_scope_b200.sharded import HANDLE_BYTES, exchange_handles
    mine = bytes([rank * 16 + k % 16 for k in range(HANDLE_BYTES)])
    ret[rank] = exchange_handles(mine)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_setup_handles_are_gathered_in_rank_order(world):
    """The one collective of the kernel-level exchange happens at set-up: every rank's 64-byte
    handle, in rank order, on every rank (here over gloo; the bytes mean nothing without a GPU)."""
    from tcu_scope_b200.sharded import HANDLE_BYTES, exchange_handles
    port = 29900 + (os.getpid() % 1500) + world
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_handle_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    want = b"".join(bytes([r * 16 + k % 16 for k in range(HANDLE_BYTES)]) for r in range(world))
    for r in range(world):
        assert ret[r] == want
    # without a process group there is nothing to exchange
    one = bytes(range(HANDLE_BYTES))
    assert exchange_handles(one) == one
    with pytest.raises(ValueError):
        exchange_handles(b"short")
