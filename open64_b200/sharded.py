"""Column-sharded linears over the GPUs of one node.

Rank r of g owns rows [r*N/g, (r+1)*N/g) of the [N,K] weight and produces the matching
columns of C = A W^T; no reduction is needed.  The only exchange is an all-gather of the
column slabs when every rank wants the whole C (NCCL, inside libo64gemm.so).

This module holds the host-side bookkeeping: slab bounds, distribution of the NCCL unique id
over an existing torch.distributed group, and the slab-major <-> row-major layout rule.
"""
import ctypes

import torch

from . import _lib
from ._lib import GATHER_NONE, GATHER_ROWMAJOR, GATHER_SLABS, check


def slab_bounds(N, rank, world):
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    if N % world:
        raise ValueError(f"N={N} does not divide over {world} ranks")
    ns = N // world
    return rank * ns, (rank + 1) * ns


def broadcast_unique_id(make_id, group=None):
    """Rank 0 of `group` calls make_id() -> bytes; every rank returns those bytes."""
    import torch.distributed as dist
    rank = dist.get_rank(group)
    payload = [make_id() if rank == 0 else None]
    src = dist.get_global_rank(group, 0) if group is not None else 0
    dist.broadcast_object_list(payload, src=src, group=group)
    if not isinstance(payload[0], (bytes, bytearray)) or len(payload[0]) != _lib.UNIQUE_ID_BYTES:
        raise RuntimeError("unique id did not arrive intact")
    return bytes(payload[0])


def slab_major_to_row_major(slabs, world):
    """[g*M, N/g] (slab-major, what the all-gather delivers) -> [M, N] row-major."""
    gM, ns = slabs.shape
    M = gM // world
    return slabs.view(world, M, ns).permute(1, 0, 2).reshape(M, world * ns)


class ShardedInt8Linear:
    """C = A W^T, int8 -> int32, W's rows (C's columns) split over the ranks of `group`."""

    def __init__(self, eng, W_slab, N, group=None):
        import torch.distributed as dist
        self.eng = eng
        self.W_slab = W_slab
        self.N = N
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        lo, hi = slab_bounds(N, self.rank, self.world)
        if W_slab.shape[0] != hi - lo:
            raise ValueError("W_slab has the wrong number of rows for this rank")
        if self.world > 1:
            lib = eng.lib

            def make_id():
                buf = (ctypes.c_char * _lib.UNIQUE_ID_BYTES)()
                check(lib.o64_comm_unique_id(buf), "o64_comm_unique_id")
                return bytes(buf)

            idb = broadcast_unique_id(make_id, group)
            check(lib.o64_comm_init(eng._h, ctypes.create_string_buffer(idb, _lib.UNIQUE_ID_BYTES),
                                    self.rank, self.world), "o64_comm_init")

    def __call__(self, A, gather=GATHER_ROWMAJOR, out=None, workspace=None):
        return self.eng.gemm_s8_sharded(A, self.W_slab, self.N, gather=gather, out=out,
                                        workspace=workspace)
