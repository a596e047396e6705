"""GPU: the failure path of the tensor-core kernels.  Every device-side wait carries a budget; when it
runs out the kernel records which wait gave up, leaves its role loops, frees its tensor memory and
RETURNS.  The test makes a wait run out in the allowed way: a hooked instantiation of each kernel whose
loader leaves out one K block (nothing traps, faults or spins without a limit), a budget of a tenth of a
second, then the status is read and an ordinary product on the same handle must be exact again."""
import numpy as np
import pytest
import torch

import open64_b200 as o
import oracle
from util import TOL_LOWP, bits16, relmax

pytestmark = pytest.mark.gpu

# (name, pin, M): the pin selects the kernel; M = 64 with split_k = -1 is the few-rows kernel
KERNELS = [
    ("one CTA per tile", dict(cta_group=1, tile_m=128, tile_n=256, split_k=1), 512),
    ("CTA pair per 256-row tile", dict(cta_group=2, tile_m=256, tile_n=256), 512),
    ("CTA pair per 512-row tile", dict(cta_group=2, tile_m=512, tile_n=256), 1024),
    ("few rows, cluster split of K", dict(split_k=-2, tile_n=256), 64),
]


@pytest.mark.parametrize("name,pin,M", KERNELS, ids=[k[0] for k in KERNELS])
def test_a_wait_that_runs_out_ends_the_kernel_with_a_status(eng, name, pin, M):
    dev = torch.device("cuda", eng.device)
    N, K = 512, 1024                       # 16 K blocks of 64
    A, B = o.workloads.c2_gemm_bf16(M, N, K)
    Ad, Bd = A.to(dev), B.to(dev)
    eng.plan_set(o.KIND_BF16, **pin)
    eng.set_wait_budget_us(100_000)
    try:
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        eng.test_gemm_bf16_withheld(Ad, Bd, withhold_kblock=5)
        t1.record()
        st, detail = eng.last_status()
        assert st == o.ERR_TIMEOUT, f"{name}: status {st}, detail 0x{detail:x}"
        assert (detail & 0xf) in (1, 2, 3, 4), f"{name}: detail 0x{detail:x} names no wait"
        ms = t0.elapsed_time(t1)
        assert 50.0 <= ms <= 2000.0, f"{name}: the kernel took {ms:.0f} ms for a 100 ms budget"
        assert eng.last_status() == (o.OK, 0)          # reading the status cleared it
        # the context is intact and the same kernel is exact again
        c = eng.gemm_bf16(Ad, Bd, transB=True).float().cpu().numpy()
        assert eng.last_status() == (o.OK, 0)
        ref = oracle.gemm_bf16(bits16(A), bits16(B))
        assert relmax(c, ref) <= TOL_LOWP
        assert torch.cuda.memory_allocated(dev) >= 0   # the allocator still answers
    finally:
        eng.set_wait_budget_us(0)
        eng.plan_set(o.KIND_BF16)


def test_hook_is_refused_where_no_hooked_kernel_exists(eng):
    dev = torch.device("cuda", eng.device)
    A, B = o.workloads.c2_gemm_bf16(256, 256, 256)
    eng.plan_set(o.KIND_BF16, cta_group=1, tile_m=128, tile_n=128, split_k=1)
    try:
        with pytest.raises(o.O64Error) as e:
            eng.test_gemm_bf16_withheld(A.to(dev), B.to(dev), withhold_kblock=1)
        assert e.value.status == o.ERR_DTYPE
    finally:
        eng.plan_set(o.KIND_BF16)


def test_empty_sum_is_the_epilogue_of_zero(eng):
    """K == 0: C = act(bias) for bf16, bias for the scaled fp8 product, zeros for int8 and SwiGLU
    (the runtime's kernels zero C, osprey/libfi/matrix/xgemmx.h:185-196)."""
    dev = torch.device("cuda", eng.device)
    M, N = 70, 200
    bias = torch.linspace(-2, 2, N)
    A = torch.empty((M, 0), dtype=torch.bfloat16, device=dev)
    B = torch.empty((N, 0), dtype=torch.bfloat16, device=dev)
    c = eng.gemm_bf16(A, B, transB=True, bias=bias.to(dev), act="relu").float().cpu()
    want = torch.relu(bias).to(torch.bfloat16).float().expand(M, N)
    assert torch.equal(c, want)
    c = eng.gemm_bf16(A, B, transB=True, out=torch.full((M, N), 7.0, dtype=torch.bfloat16, device=dev))
    assert torch.count_nonzero(c).item() == 0
    A8 = torch.empty((M, 0), dtype=torch.int8, device=dev)
    B8 = torch.empty((N, 0), dtype=torch.int8, device=dev)
    c = eng.gemm_s8(A8, B8, out=torch.full((M, N), 7, dtype=torch.int32, device=dev))
    assert torch.count_nonzero(c).item() == 0
    host = torch.full((M, N), 7, dtype=torch.int32)          # a host result is staged and copied back
    eng.gemm_s8(A8.cpu(), B8.cpu(), out=host)
    assert torch.count_nonzero(host).item() == 0
    assert eng.last_status() == (o.OK, 0)
