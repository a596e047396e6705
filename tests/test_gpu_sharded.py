"""GPU: the column-sharded int8 GEMM.  On one GPU the three gather modes must agree with the
plain GEMM; with two or more GPUs the ranks run as child processes over NCCL and every rank
must hold the full exact product."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

import open64_b200 as o
import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_single_rank_modes(eng):
    M, N, K = 300, 512, 400
    A, B = o.workloads.c5_int8(M, N, K, seed=21)
    ref = oracle.gemm_s8s8_s32(A.numpy(), B.numpy())
    Ad, Bd = A.to(DEV), B.to(DEV)
    for mode in (o.GATHER_NONE, o.GATHER_ROWMAJOR, o.GATHER_SLABS):
        C = eng.gemm_s8_sharded(Ad, Bd, N, gather=mode)
        assert np.array_equal(C.cpu().numpy(), ref), mode
    assert eng.lib.o64_gemm_s8_sharded_workspace(M, N, 1, o.GATHER_ROWMAJOR) == M * N * 4
    # the fused form needs the engine's own result buffer
    import pytest as _pt
    with _pt.raises(o.O64Error):
        eng.gemm_s8_sharded(Ad, Bd, N, gather=o.GATHER_PUSH)
    out = eng.alloc_result(M, N)
    out.fill_(-1)
    eng.gemm_s8_sharded(Ad, Bd, N, gather=o.GATHER_PUSH, out=out)
    assert np.array_equal(out.cpu().numpy(), ref)


def test_single_rank_bf16_modes(eng):
    from util import TOL_LOWP, bits16, relmax
    M, N, K = 300, 512, 264
    g = torch.Generator().manual_seed(8)
    A = (torch.randn(M, K, generator=g) * 0.2).to(torch.bfloat16)
    B = torch.randn(N, K, generator=g).to(torch.bfloat16)
    bias = torch.randn(N, generator=g)
    ref = oracle.gemm_bf16(bits16(A), bits16(B), bias=bias.numpy(), act=oracle.ACT_SILU, transB=True)
    Ad, Bd, bd = A.to(DEV), B.to(DEV), bias.to(DEV)
    for mode in (o.GATHER_NONE, o.GATHER_SLABS):
        C = eng.gemm_bf16_sharded(Ad, Bd, N, gather=mode, bias=bd, act="silu")
        assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP, mode
    out = eng.alloc_result(M, N, dtype=torch.bfloat16)
    eng.gemm_bf16_sharded(Ad, Bd, N, gather=o.GATHER_PUSH, bias=bd, act="silu", out=out)
    assert relmax(out.float().cpu().numpy(), ref) <= TOL_LOWP
    with pytest.raises(o.O64Error):
        eng.gemm_bf16_sharded(Ad, Bd, N, gather=o.GATHER_ROWMAJOR, bias=bd)


def _rank_main(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import open64_b200 as oo
        import oracle as orc
        from open64_b200 import sharded
        dev = torch.device("cuda", rank)
        eng = oo.Engine(rank)
        M, N, K = 520, 1024, 640
        A, B = oo.workloads.c5_int8(M, N, K, seed=33)
        ref = torch.from_numpy(orc.gemm_s8s8_s32(A.numpy(), B.numpy()))
        lin = sharded.ShardedInt8Linear(eng, oo.workloads.shard_rows(B, rank, world).to(dev), N)
        Ad = A.to(dev)
        full = lin(Ad, gather=oo.GATHER_ROWMAJOR)
        assert torch.equal(full.cpu(), ref), "row-major gather"
        slabs = lin(Ad, gather=oo.GATHER_SLABS)
        assert torch.equal(sharded.slab_major_to_row_major(slabs.view(world * M, N // world), world).cpu(), ref)
        mine = torch.full((M, N), -1, dtype=torch.int32, device=dev)
        lin(Ad, gather=oo.GATHER_NONE, out=mine)
        lo, hi = sharded.slab_bounds(N, rank, world)
        assert torch.equal(mine[:, lo:hi].cpu(), ref[:, lo:hi]) and (mine[:, :lo] == -1).all()
        # fused GEMM + exchange: one kernel stores its tiles into every rank's result buffer
        out = eng.alloc_result(M, N)
        for rep in range(2):
            out.fill_(-1 - rep)
            lin(Ad, gather=oo.GATHER_PUSH, out=out)
            torch.cuda.synchronize()
            assert torch.equal(out.cpu(), ref), f"fused push, call {rep}"
        # the fused form replayed from a CUDA graph: the call number the ranks compare lives in device
        # memory, so the frozen launch parameters are good for every replay
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            lin(Ad, gather=oo.GATHER_PUSH, out=out)          # warm-up on the capturing stream
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                lin(Ad, gather=oo.GATHER_PUSH, out=out)
        torch.cuda.current_stream().wait_stream(side)
        for rep in range(3):
            out.fill_(-20 - rep)
            torch.cuda.synchronize()
            dist.barrier()                                   # every rank has refilled before anyone replays
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out.cpu(), ref), f"fused push replayed from a graph, replay {rep}"
        del graph
        # a taller product through the fused form: more tiles than CTA pairs, the last row block ragged
        M2, K2 = 4200, 256
        A2, B2 = oo.workloads.c5_int8(M2, N, K2, seed=35)
        ref2 = torch.from_numpy(orc.gemm_s8s8_s32(A2.numpy(), B2.numpy()))
        out2 = eng.alloc_result(M2, N)
        B2s = oo.workloads.shard_rows(B2, rank, world).contiguous().to(dev)
        for rep in range(3):
            out2.fill_(-1 - rep)
            eng.gemm_s8_sharded(A2.to(dev), B2s, N, gather=oo.GATHER_PUSH, out=out2)
            torch.cuda.synchronize()
            assert torch.equal(out2.cpu(), ref2), f"fused push of a tall product, call {rep}"
        out = eng.alloc_result(M, N)   # the engine holds one result buffer at a time
        # the bf16 linear with a fused bias + GELU, sharded the same way
        from util import TOL_LOWP, bits16, relmax
        g = torch.Generator().manual_seed(44)
        Ab = (torch.randn(M, K, generator=g) * 0.2).to(torch.bfloat16)
        Bb = torch.randn(N, K, generator=g).to(torch.bfloat16)
        bias = torch.randn(N, generator=g)
        refb = orc.gemm_bf16(bits16(Ab), bits16(Bb), bias=bias.numpy(), act=orc.ACT_GELU_TANH, transB=True)
        Bs = oo.workloads.shard_rows(Bb, rank, world).contiguous().to(dev)
        outb = eng.alloc_result(M, N, dtype=torch.bfloat16)
        for rep in range(2):
            outb.fill_(float(rep + 3))
            eng.gemm_bf16_sharded(Ab.to(dev), Bs, N, gather=oo.GATHER_PUSH, bias=bias.to(dev), act="gelu_tanh", out=outb)
            torch.cuda.synchronize()
            assert relmax(outb.float().cpu().numpy(), refb) <= TOL_LOWP, f"bf16 fused push, call {rep}"
        slb = eng.gemm_bf16_sharded(Ab.to(dev), Bs, N, gather=oo.GATHER_SLABS, bias=bias.to(dev), act="gelu_tanh")
        rm = sharded.slab_major_to_row_major(slb.view(world * M, N // world), world)
        assert relmax(rm.float().cpu().numpy(), refb) <= TOL_LOWP, "bf16 slab-major gather"
        st, detail = eng.last_status()
        assert st == 0
        # a rank that never makes the call: the other's kernel waits for its arrival for the handle's budget,
        # gives up, stores nothing to the peer, and says which wait ran out; the context stays usable and a
        # fresh result buffer (new counters on both ranks) works again.  Nothing faults, traps or hangs.
        torch.cuda.synchronize()
        dist.barrier()
        out = eng.alloc_result(M, N)
        out.fill_(-99)
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            eng.set_wait_budget_us(30_000)
            lin(Ad, gather=oo.GATHER_PUSH, out=out)
            torch.cuda.synchronize()
            st, detail = eng.last_status()
            # 0x501: the wait for the peers' arrival (0x581 when a CTA other than the one that watches the
            # peers' counters was the first to give up)
            assert st == oo.ERR_TIMEOUT and (detail & 0xf7f) == 0x501, (st, hex(detail))
            eng.set_wait_budget_us(0)
            assert eng.last_status()[0] == 0
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 1:
            assert (out == -99).all(), "a kernel whose wait ran out must not have stored into its peer"
        dist.barrier()
        out = eng.alloc_result(M, N)                             # collective: counters start afresh
        out.fill_(-1)
        torch.cuda.synchronize()
        dist.barrier()
        lin(Ad, gather=oo.GATHER_PUSH, out=out)
        torch.cuda.synchronize()
        assert torch.equal(out.cpu(), ref), "fused push after a timed-out call"
        st, detail = eng.last_status()
        assert st == 0
        torch.cuda.synchronize()
        dist.barrier()
        eng.close()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"fail: {e!r}"))
    finally:
        dist.destroy_process_group()


def test_two_ranks_all_gather(built):
    world = min(torch.cuda.device_count(), 2)
    if world < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(r, "ok") for r in range(world)], results
