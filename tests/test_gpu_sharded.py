"""GPU tests of the sharded (multi-GPU) full reduction and full scan.

Three layers:
  * one GPU, several ranks' contexts in one process: the two-pass kernels, the
    slot arrays and the sequence numbers, with the shards processed in rank
    order on one stream (a scan only waits for EARLIER ranks, whose totals are
    then already there, so nothing ever waits on a later launch);
  * two or more GPUs, one process per GPU (child processes, or the ranks of a
    ``torch.distributed.run -m pytest`` launch): the kernel-level exchange over
    NVLink and the all-gather variant, every rank checking its own outputs
    against the fp64 oracle;
  * segmented operations on shards: no communication, outputs of the shards
    concatenate to the oracle's.
"""
import ctypes
import os
import sys

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REL, ABS_FLOOR = 1e-3, 1e-5
OUT_F16, OUT_F32 = 0, 1


def bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class LocalGroup:
    """`world` contexts on the current device, connected through their device pointers."""

    def __init__(self, lib, world):
        self.lib, self.world = lib, world
        self.ctx = (ctypes.c_void_p * world)()
        for r in range(world):
            c = ctypes.c_void_p()
            assert lib.tcu_mgpu_ctx_create(ctypes.byref(c), r, world, None) == 0
            self.ctx[r] = c
        for r in range(world):
            assert lib.tcu_mgpu_ctx_connect_local(self.ctx[r], self.ctx) == 0

    def close(self):
        torch.cuda.synchronize()
        for r in range(self.world):
            self.lib.tcu_mgpu_ctx_destroy(self.ctx[r])


@pytest.mark.parametrize("world,n,keep", [
    (1, 16, None), (1, 5 * 16384 + 48, None), (2, 1 << 20, None), (3, 16 * 100001, 0),
    (4, (1 << 23) + 16 * 7, None), (4, 16 * 3, None), (2, 1 << 25, 1 << 22)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
def test_two_pass_scan_with_emulated_ranks(world, n, keep, out_dtype):
    import tcu_scope_b200 as tcu
    from tcu_scope_b200.sharded import shard_range
    lib = tcu._lib.load()
    dist_name = "uniform_01" if out_dtype == torch.float32 else "uniform_pm1"
    x = torch.empty(n, dtype=torch.float16, device="cuda")
    tcu.fill(x, 90 + world, 0, dist_name)
    out = torch.full((n,), -7.0, dtype=out_dtype, device="cuda")
    grp = LocalGroup(lib, world)
    code = OUT_F32 if out_dtype == torch.float32 else OUT_F16
    for rep in range(3):  # the slots rotate with the call number: go round more than once
        out.fill_(-7.0)
        for r in range(world):  # rank order: a rank's scan finds the earlier totals in place
            b, e = shard_range(n // 16, r, world)
            b, e = b * 16, e * 16
            if keep is not None:
                assert lib.tcu_mgpu_ctx_set_l2_keep_bytes(grp.ctx[r], keep) == 0
            st = lib.tcu_mgpu_full_scan_f16(grp.ctx[r], x.data_ptr() + 2 * b,
                                            out.data_ptr() + out.element_size() * b, code, e - b,
                                            _stream())
            assert st == 0, lib.tcu_status_string(st)
        torch.cuda.synchronize()
    grp.close()
    ref = oracle.c_segmented_scan(bits(x), n)
    if out_dtype == torch.float32:
        bad, max_abs, max_rel = oracle.np_check_f32(out.cpu().numpy(), ref, REL, ABS_FLOOR)
        assert bad == 0, f"{bad} outputs out of tolerance (max abs {max_abs}, max rel {max_rel})"
        assert max_rel < 1e-6  # one rounding of an exact prefix
    else:
        bad, worst = oracle.np_check_f16(bits(out), ref, 2)
        assert bad == 0, f"{bad} outputs more than 2 halves off (worst {worst})"
    assert tcu.device_error() == 0


def test_mgpu_full_reduce_single_rank_and_validation():
    import tcu_scope_b200 as tcu
    lib = tcu._lib.load()
    grp = LocalGroup(lib, 1)
    for n in (16, 16384 * 3 + 160, (1 << 24) + 4096):
        x = torch.empty(n, dtype=torch.float16, device="cuda")
        tcu.fill(x, 13, 0, "uniform_01")
        o32 = torch.zeros(1, dtype=torch.float32, device="cuda")
        o64 = torch.zeros(1, dtype=torch.float64, device="cuda")
        for _ in range(2):
            assert lib.tcu_mgpu_full_reduce_f16(grp.ctx[0], x.data_ptr(), o32.data_ptr(),
                                                o64.data_ptr(), n, _stream()) == 0
        ref = oracle.c_segmented_reduce(bits(x), n)
        assert o64.cpu().numpy()[0] == ref[0]
        assert o32.cpu().numpy()[0] == np.float32(ref[0])
    x = torch.zeros(64, dtype=torch.float16, device="cuda")
    o32 = torch.zeros(1, dtype=torch.float32, device="cuda")
    assert lib.tcu_mgpu_full_reduce_f16(grp.ctx[0], x.data_ptr(), o32.data_ptr(), None, 24, _stream()) == 1
    assert lib.tcu_mgpu_full_reduce_f16(None, x.data_ptr(), o32.data_ptr(), None, 32, _stream()) == 1
    assert lib.tcu_mgpu_full_scan_f16(grp.ctx[0], x.data_ptr(), o32.data_ptr(), 9, 16, _stream()) == 2
    grp.close()
    c = ctypes.c_void_p()
    assert lib.tcu_mgpu_ctx_create(ctypes.byref(c), 3, 2, None) == 1   # rank outside the group
    assert lib.tcu_mgpu_ctx_create(ctypes.byref(c), 0, 17, None) == 1  # more ranks than slots
    # a context that was never connected refuses to run
    assert lib.tcu_mgpu_ctx_create(ctypes.byref(c), 0, 2, None) == 0
    assert lib.tcu_mgpu_full_reduce_f16(c, x.data_ptr(), o32.data_ptr(), None, 32, _stream()) == 1
    lib.tcu_mgpu_ctx_destroy(c)
    assert tcu.device_error() == 0


# ------------------------------------------------------------------ several GPUs
def sharded_checks(rank, world):
    """Run by every rank with its GPU current and the process group up.  Returns a dict of
    what was checked; raises on any mismatch."""
    import torch.distributed as dist
    import tcu_scope_b200 as tcu
    from tcu_scope_b200.sharded import shard_range
    report = {}
    n_total = (1 << 24) + 16 * 5 * world + 16  # ragged: shards differ in length
    b, e = shard_range(n_total // 16, rank, world)
    b, e = b * 16, e * 16
    x = torch.empty(e - b, dtype=torch.float16, device="cuda")
    tcu.fill(x, 2025, b, "uniform_01")
    xb = bits(x)
    assert np.array_equal(xb, oracle.c_fill_f16(e - b, 2025, b, "uniform_01"))
    whole = oracle.c_fill_f16(n_total, 2025, 0, "uniform_01")
    ref_scan = oracle.c_segmented_scan(whole, n_total)

    grp = tcu.PeerGroup()
    for rep in range(5):
        o32, o64 = grp.full_reduce(x)
        sc = grp.full_scan(x)
        sc16 = grp.full_scan(x, out_dtype=torch.float16) if rep == 0 else None
        torch.cuda.synchronize()
        assert o64.cpu().numpy()[0] == ref_scan[-1], "sum over all ranks (kernel-level exchange)"
        assert o32.cpu().numpy()[0] == np.float32(ref_scan[-1])
        bad, max_abs, max_rel = oracle.np_check_f32(sc.cpu().numpy(), ref_scan[b:e], REL, ABS_FLOOR)
        assert bad == 0, f"rank {rank}: {bad} scan outputs out of tolerance (max abs {max_abs})"
        assert max_rel < 1e-6
        if sc16 is not None:  # fp16 outputs saturate late in a [0,1) scan; compare where they are finite
            m = ref_scan[b:e] < 60000.0
            if m.any():
                badh, worst = oracle.np_check_f16(bits(sc16)[m], ref_scan[b:e][m], 2)
                assert badh == 0, worst
    report["peer_exchange"] = "ok"

    # the all-gather variant: reduce pass, one collective, seeded look-back scan
    ws = torch.empty(max(tcu.workspace_bytes(tcu.OP_FULL_SCAN, e - b, e - b),
                         tcu.workspace_bytes(tcu.OP_FULL_REDUCE, e - b, e - b)),
                     dtype=torch.uint8, device="cuda")

    def local_total():
        return tcu.full_reduce(x, workspace=ws)[1]
    total = tcu.sharded_full_reduce(local_total)
    sc = tcu.sharded_full_scan(local_total, lambda totals, r: tcu.full_scan(
        x, workspace=ws, shard_totals=totals, shard_index=r))
    torch.cuda.synchronize()
    assert total.cpu().numpy()[0] == ref_scan[-1]
    bad, max_abs, _ = oracle.np_check_f32(sc.cpu().numpy(), ref_scan[b:e], REL, ABS_FLOOR)
    assert bad == 0, f"rank {rank}: all-gather variant, {bad} out of tolerance (max abs {max_abs})"
    report["all_gather"] = "ok"

    # segmented operations: whole segments per rank, no communication
    for s in (16, 256, 4096):
        segs = (1 << 22) // s + 3
        sb, se = shard_range(segs, rank, world)
        xs = torch.empty((se - sb) * s, dtype=torch.float16, device="cuda")
        tcu.fill(xs, 31, sb * s, "uniform_pm1")
        red = tcu.segmented_reduce(xs, s)
        scn = tcu.segmented_scan(xs, s, out_dtype=torch.float32)
        w = oracle.c_fill_f16(segs * s, 31, 0, "uniform_pm1")
        assert oracle.np_check_f32(red.cpu().numpy(), oracle.c_segmented_reduce(w, s)[sb:se])[0] == 0
        assert oracle.np_check_f32(scn.cpu().numpy(),
                                   oracle.c_segmented_scan(w, s)[sb * s:se * s])[0] == 0
    report["segmented"] = "ok"
    assert tcu.device_error() == 0
    grp.close()
    dist.barrier()
    return report


def _child(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ret[rank] = sharded_checks(rank, world)
    finally:
        dist.destroy_process_group()


def test_sharded_ops_on_several_gpus():
    env_world = int(os.environ.get("WORLD_SIZE", "1"))
    if env_world > 1:  # launched as one rank per GPU (torch.distributed.run -m pytest ...)
        import torch.distributed as dist
        rank, local = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        assert sharded_checks(rank, env_world) == {"peer_exchange": "ok", "all_gather": "ok",
                                                   "segmented": "ok"}
        return
    gpus = torch.cuda.device_count()
    if gpus < 2:
        pytest.skip("needs two or more GPUs")
    import torch.multiprocessing as mp
    world = min(gpus, 4)
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29800 + os.getpid() % 1500
    procs = [ctx.Process(target=_child, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
        assert p.exitcode == 0, "a rank failed"
    assert len(ret) == world
