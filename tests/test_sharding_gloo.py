"""CPU, world_size 2 over gloo: the host-side logic of the column-sharded linear (slab bounds,
unique-id distribution, slab-major <-> row-major layout), with the oracle standing in for the
per-rank device GEMM."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import open64_b200 as o
        import oracle
        from open64_b200 import sharded

        M, N, K = 24, 64, 96
        A, B = o.workloads.c5_int8(M, N, K)               # identical on every rank (seeded)
        lo, hi = sharded.slab_bounds(N, rank, world)
        slab = o.workloads.shard_rows(B, rank, world)
        assert slab.shape[0] == hi - lo and torch.equal(slab, B[lo:hi])
        mine = torch.from_numpy(oracle.gemm_s8s8_s32(A.numpy(), slab.numpy()))   # [M, N/g]

        # the exchange: an all-gather of contiguous [M, N/g] slabs -> slab-major [g*M, N/g]
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        slabs = torch.cat(parts, dim=0)
        full = sharded.slab_major_to_row_major(slabs, world)
        ref = torch.from_numpy(oracle.gemm_s8s8_s32(A.numpy(), B.numpy()))
        assert torch.equal(full, ref)

        # unique-id distribution: rank 0 makes it, everybody holds the same 128 bytes
        made = []

        def make_id():
            made.append(1)
            return bytes(range(128))

        idb = sharded.broadcast_unique_id(make_id)
        assert idb == bytes(range(128)) and len(made) == (1 if rank == 0 else 0)
        # a damaged id is refused
        try:
            sharded.broadcast_unique_id(lambda: b"short")
            ok = False
        except RuntimeError:
            ok = True
        assert ok
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"fail: {e!r}"))
    finally:
        dist.destroy_process_group()


def test_column_sharding_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_slab_bounds_edges():
    sys.path.insert(0, ROOT)
    from open64_b200 import sharded
    assert sharded.slab_bounds(8192, 0, 8) == (0, 1024)
    assert sharded.slab_bounds(8192, 7, 8) == (7168, 8192)
    with pytest.raises(ValueError):
        sharded.slab_bounds(100, 0, 8)
    with pytest.raises(ValueError):
        sharded.slab_bounds(64, 2, 2)
    t = torch.arange(2 * 3 * 4).view(6, 4)      # g=2, M=3, ns=4
    rm = sharded.slab_major_to_row_major(t, 2)
    assert rm.shape == (3, 8) and rm[1].tolist() == [4, 5, 6, 7, 16, 17, 18, 19]
