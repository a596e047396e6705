"""GPU: the K split of a last, partly filled wave of tiles in the CTA-pair kernels.  When the tile count
does not divide by the number of CTA pairs, the tiles of the last wave are cut along K over the pairs;
pieces meet through slots in global memory, flags carry a per-launch epoch.  Every case checks that the
split really ran (o64_test_last_tail_split) and the result against the CPU oracle: bf16 / fp8 within the
contract's tolerance and a tight 4e-3, int8 bit for bit, twice in a row (slots and flags are reused)."""
import numpy as np
import pytest
import torch

import open64_b200 as o
import oracle
from util import TOL_LOWP, bits16, bits8, relmax

pytestmark = pytest.mark.gpu
TIGHT = 4e-3

PAIR = dict(cta_group=2, tile_m=256, tile_n=256)
PAIR128 = dict(cta_group=2, tile_m=256, tile_n=128)

# (pin, M, N, K): fewer tiles than pairs, ragged edges, more than one wave
SHAPES = [
    (PAIR, 512, 2560, 2048),
    (PAIR, 300, 1000, 1100),
    (PAIR, 2048, 2560, 2048),      # 80 tiles on 74 pairs: one whole wave, six tiles cut
    (PAIR128, 256, 4096, 2048),
    (PAIR128, 1000, 1200, 1544),
]


def _dev(eng):
    return torch.device("cuda", eng.device)


@pytest.fixture(autouse=True)
def forced(eng, request):
    """Correctness cases take the split wherever a last wave is partly filled, also where the model
    expects no gain from it; the policy test runs with the model in charge."""
    eng.force_tail_split(-1 if "automatic" in request.node.name else 1)
    yield
    eng.force_tail_split(-1)


@pytest.mark.parametrize("pin,M,N,K", SHAPES)
def test_bf16_with_bias_and_activation(eng, pin, M, N, K):
    dev = _dev(eng)
    A, B = o.workloads.c2_gemm_bf16(M, N, K, seed=M + N + K)
    bias = torch.linspace(-1, 1, N)
    eng.plan_set(o.KIND_BF16, **pin)
    try:
        ref = oracle.gemm_bf16(bits16(A), bits16(B), bias=bias.numpy(), act=oracle.ACT_GELU_TANH)
        for call in range(2):
            c = eng.gemm_bf16(A.to(dev), B.to(dev), transB=True, bias=bias.to(dev), act="gelu_tanh")
            tiles, pairs = eng.last_tail_split()
            assert tiles > 0 and pairs > tiles, f"no split for {pin} {M}x{N}x{K}: {tiles}, {pairs}"
            err = relmax(c.float().cpu().numpy(), ref)
            assert err <= TOL_LOWP and err <= TIGHT, (call, err)
        assert eng.last_status() == (o.OK, 0)
    finally:
        eng.plan_set(o.KIND_BF16)


@pytest.mark.parametrize("pin,M,N,K", [(PAIR, 512, 2560, 4096), (PAIR128, 1024, 1024, 8192), (PAIR, 2100, 2400, 1000)])
def test_int8_bit_exact(eng, pin, M, N, K):
    dev = _dev(eng)
    A, B = o.workloads.c5_int8(M, N, K, seed=K)
    want = oracle.gemm_s8s8_s32(A.numpy(), B.numpy())
    eng.plan_set(o.KIND_S8, **pin)
    try:
        for call in range(2):
            c = eng.gemm_s8(A.to(dev), B.to(dev))
            assert eng.last_tail_split()[0] > 0
            assert np.array_equal(c.cpu().numpy(), want), call
        assert eng.last_status() == (o.OK, 0)
    finally:
        eng.plan_set(o.KIND_S8)


def test_fp8_scaled(eng):
    dev = _dev(eng)
    A8, W8, sA, sB, b = o.workloads.c4_fp8(512, 2560, 4096)
    ref = oracle.gemm_fp8_scaled(bits8(A8), bits8(W8), sA.numpy(), sB.numpy(), b.numpy())
    eng.plan_set(o.KIND_FP8, **PAIR)
    try:
        c = eng.gemm_fp8_scaled(A8.to(dev), W8.to(dev), sA.to(dev), sB.to(dev), b.to(dev))
        assert eng.last_tail_split()[0] > 0
        err = relmax(c.float().cpu().numpy(), ref)
        assert err <= TOL_LOWP and err <= TIGHT, err
    finally:
        eng.plan_set(o.KIND_FP8)


@pytest.mark.parametrize("pin", [PAIR])
def test_swiglu_and_kn_weights(eng, pin):
    dev = _dev(eng)
    T, D, F = 1024, 2048, 1280
    x, Wg, Wu, Wd = o.workloads.c3_swiglu(T, D, F)
    eng.plan_set(o.KIND_BF16, **pin)
    try:
        h = eng.swiglu(x.to(dev), Wg.to(dev), Wu.to(dev))
        assert eng.last_tail_split()[0] > 0, "SwiGLU GEMM ran whole tiles"
        h_ref = oracle.swiglu_bf16(bits16(x), bits16(Wg), bits16(Wu))
        hf = oracle.bf16_to_f32(h_ref)
        assert relmax(h.float().cpu().numpy(), hf) <= TOL_LOWP
        out = eng.gemm_bf16(h, Wd.to(dev), transB=False)
        ref = oracle.gemm_bf16(bits16(h.cpu()), bits16(Wd), transB=False)
        err = relmax(out.float().cpu().numpy(), ref)
        assert err <= TOL_LOWP and err <= TIGHT, err
        assert eng.last_status() == (o.OK, 0)
    finally:
        eng.plan_set(o.KIND_BF16)


def test_split_is_deterministic(eng):
    """Pieces are added in a fixed order, not in order of arrival: the same call twice gives the same bits."""
    dev = _dev(eng)
    A, B = o.workloads.c2_gemm_bf16(768, 2560, 4096, seed=5)
    Ad, Bd = A.to(dev), B.to(dev)
    eng.plan_set(o.KIND_BF16, **PAIR)
    try:
        first = eng.gemm_bf16(Ad, Bd, transB=True).clone()
        assert eng.last_tail_split()[0] > 0
        for _ in range(3):
            assert torch.equal(eng.gemm_bf16(Ad, Bd, transB=True), first)
    finally:
        eng.plan_set(o.KIND_BF16)


def test_replayed_from_a_cuda_graph(eng):
    """A captured launch has frozen parameters: the flag words must be back at zero after every launch
    by themselves.  Three products on different operands, captured once, replayed three times; between
    replays the operands change, so a consumer that ran ahead of its contributors would read stale sums."""
    dev = _dev(eng)
    M, N, K = 512, 2560, 2048
    eng.plan_set(o.KIND_S8, **PAIR)
    try:
        As = [torch.empty((M, K), dtype=torch.int8, device=dev) for _ in range(3)]
        Bs = [torch.empty((N, K), dtype=torch.int8, device=dev) for _ in range(3)]
        Cs = [torch.empty((M, N), dtype=torch.int32, device=dev) for _ in range(3)]
        eng.gemm_s8(As[0], Bs[0], out=Cs[0])                       # set-up and allocations before the capture
        assert eng.last_tail_split()[0] > 0
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for i in range(3):
                    eng.gemm_s8(As[i], Bs[i], out=Cs[i])
        for rep in range(3):
            hosts = [o.workloads.c5_int8(M, N, K, seed=100 * rep + i) for i in range(3)]
            for i, (a, b) in enumerate(hosts):
                As[i].copy_(a)
                Bs[i].copy_(b)
            torch.cuda.synchronize()
            graph.replay()
            torch.cuda.synchronize()
            for i, (a, b) in enumerate(hosts):
                assert np.array_equal(Cs[i].cpu().numpy(), oracle.gemm_s8s8_s32(a.numpy(), b.numpy())), (rep, i)
        assert eng.last_status() == (o.OK, 0)
    finally:
        eng.plan_set(o.KIND_S8)


def test_automatic_policy(eng):
    """The model in charge: a 768-row product on 256 x 256 tiles (96 tiles on 74 pairs) takes the split,
    64 tiles on 74 pairs and the 8192^3 headline shape (68 of 74 pairs busy in the last wave) do not."""
    dev = _dev(eng)
    eng.plan_set(o.KIND_BF16, **PAIR)
    try:
        for M, want in ((768, True), (512, False)):
            A, B = o.workloads.c2_gemm_bf16(M, 8192, 4096, seed=M)
            c = eng.gemm_bf16(A.to(dev), B.to(dev), transB=True)
            assert (eng.last_tail_split()[0] > 0) == want, (M, eng.last_tail_split())
            ref = oracle.gemm_bf16(bits16(A), bits16(B))
            assert relmax(c.float().cpu().numpy(), ref) <= TIGHT
    finally:
        eng.plan_set(o.KIND_BF16)
    plan = eng.plan_get(o.KIND_BF16, 8192, 8192, 8192)
    assert (plan["tile_m"], plan["tile_n"]) == (512, 256)
    assert eng.last_status() == (o.OK, 0)
