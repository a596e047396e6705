"""GPU: the kernel for few rows of A (M <= 128) against a large weight — only the existing rows
of A are loaded, every 128 x 256 tile is split along K over a cluster of CTAs and the partial sums
are added through distributed shared memory.  Same gates as the tile kernels:
bf16 / fp8 max|y - ref| / max|ref| <= 2e-2 against the fp32 loop nest, int8 -> int32 bit exact."""
import numpy as np
import pytest
import torch

import open64_b200 as o
import oracle
from util import TOL_LOWP, bits16, bits8, relmax

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ACTS = {"none": oracle.ACT_NONE, "relu": oracle.ACT_RELU, "gelu_tanh": oracle.ACT_GELU_TANH,
        "gelu_erf": oracle.ACT_GELU_ERF, "silu": oracle.ACT_SILU}

# every A-box height (16 / 32 / 64 / 128), ragged N and K, one tile and many, every cluster size
# (8 tiles or fewer: 8 CTAs per tile ... more than 74 tiles: one)
SHAPES = [(1, 2048, 1024), (7, 1000, 2056), (16, 4096, 1024), (17, 520, 4104), (33, 768, 2048),
          (64, 8192, 512), (100, 1304, 1096), (128, 2048, 2048), (5, 256, 8192), (20, 19200, 128),
          (128, 9000, 512), (3, 72, 16384), (9, 8, 131072)]


def _bf16_case(M, N, K, transB, seed=0):
    g = torch.Generator().manual_seed(seed + M * 131 + N * 17 + K)
    A = torch.randn(M, K, generator=g).to(torch.bfloat16)
    B = torch.randn((N, K) if transB else (K, N), generator=g).to(torch.bfloat16)
    return A, B


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("transB", [True, False])
def test_bf16_few_rows(eng, shape, transB):
    M, N, K = shape
    plan = eng.plan_get(o.KIND_BF16, M, N, K)
    assert plan["split_k"] in (-1, -2, -4, -8) and plan["tile_m"] in (16, 32, 64, 128) and plan["tile_m"] >= M
    A, B = _bf16_case(M, N, K, transB)
    ref = oracle.gemm_bf16(bits16(A), bits16(B), transB=transB)
    Ad, Bd = A.to(DEV), B.to(DEV)
    for rep in range(2):
        C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        eng.gemm_bf16(Ad, Bd, transB=transB, out=C)
        assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP, rep
    assert eng.last_status() == (o.OK, 0)


@pytest.mark.parametrize("act", list(ACTS))
def test_bf16_few_rows_bias_and_activation(eng, act):
    M, N, K = 24, 1544, 2048
    A, B = _bf16_case(M, N, K, True, seed=5)
    A = (A.float() * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(9))
    C = eng.gemm_bf16(A.to(DEV), B.to(DEV), transB=True, bias=bias.to(DEV), act=act)
    ref = oracle.gemm_bf16(bits16(A), bits16(B), bias=bias.numpy(), act=ACTS[act], transB=True)
    assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP


def test_few_rows_agrees_with_the_tile_kernels_and_respects_pins(eng):
    M, N, K = 48, 2048, 4096
    A, B = _bf16_case(M, N, K, True, seed=3)
    Ad, Bd = A.to(DEV), B.to(DEV)
    ref = oracle.gemm_bf16(bits16(A), bits16(B), transB=True)
    C_auto = eng.gemm_bf16(Ad, Bd, transB=True)
    try:
        eng.plan_set(o.KIND_BF16, split_k=1)                       # rules the kernel out
        assert eng.plan_get(o.KIND_BF16, M, N, K)["split_k"] == 1
        C_tile = eng.gemm_bf16(Ad, Bd, transB=True)
        others = []
        for pin in (dict(split_k=-1, num_ctas=7),                 # fewer CTAs than tiles: one CTA per tile
                    dict(split_k=-2), dict(split_k=-4), dict(split_k=-8)):   # fixed cluster sizes
            eng.plan_set(o.KIND_BF16, **pin)
            others.append(eng.gemm_bf16(Ad, Bd, transB=True))
    finally:
        eng.plan_set(o.KIND_BF16)
    for C in [C_auto, C_tile] + others:
        assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP
    # fp32 sums in a different order: equal up to the last bf16 bit of a few elements
    assert relmax(C_auto.float().cpu().numpy(), C_tile.float().cpu().numpy()) <= 1e-2


def test_few_rows_padded_pitches_and_unaligned_result(eng):
    M, N, K = 20, 600, 2048
    g = torch.Generator().manual_seed(4)
    Ap = torch.randn(M, K + 8, generator=g).to(torch.bfloat16).to(DEV)
    Bp = torch.randn(N, K + 16, generator=g).to(torch.bfloat16).to(DEV)
    Cp = torch.full((M, N + 3), 5.0, dtype=torch.bfloat16, device=DEV)   # odd pitch: scalar stores
    eng.gemm_bf16(Ap[:, :K], Bp[:, :K], transB=True, out=Cp[:, :N])
    ref = oracle.gemm_bf16(bits16(Ap[:, :K].cpu().contiguous()), bits16(Bp[:, :K].cpu().contiguous()), transB=True)
    assert relmax(Cp[:, :N].float().cpu().numpy(), ref) <= TOL_LOWP
    assert (Cp[:, N:] == 5.0).all()


@pytest.mark.parametrize("shape", [(3, 1024, 2048), (16, 4096, 4096), (50, 1000, 2176), (128, 1536, 2048)])
def test_int8_few_rows_bit_exact(eng, shape):
    M, N, K = shape
    assert eng.plan_get(o.KIND_S8, M, N, K)["split_k"] < 0
    A, B = o.workloads.c5_int8(M, N, K, seed=M + K)
    ref = oracle.gemm_s8s8_s32(A.numpy(), B.numpy())
    Cpad = torch.full((M, N + 4), -9, dtype=torch.int32, device=DEV)
    for rep in range(2):
        eng.gemm_s8(A.to(DEV), B.to(DEV), out=Cpad[:, :N])
        assert np.array_equal(Cpad[:, :N].cpu().numpy(), ref)
    assert (Cpad[:, N:] == -9).all()


@pytest.mark.parametrize("shape", [(8, 2048, 2048), (40, 1000, 4224), (128, 4096, 1024)])
def test_fp8_few_rows(eng, shape):
    M, N, K = shape
    assert eng.plan_get(o.KIND_FP8, M, N, K)["split_k"] < 0
    A8, W8, sA, sB, bias = o.workloads.c4_fp8(M, N, K, seed=M + N + K)
    ref = oracle.gemm_fp8_scaled(bits8(A8), bits8(W8), sA.numpy(), sB.numpy(), bias.numpy())
    for rep in range(2):
        C = eng.gemm_fp8_scaled(A8.to(DEV), W8.to(DEV), sA.to(DEV), sB.to(DEV), bias.to(DEV))
        assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP
    C2 = eng.gemm_fp8_scaled(A8.to(DEV), W8.to(DEV))
    assert relmax(C2.float().cpu().numpy(), oracle.gemm_fp8_scaled(bits8(A8), bits8(W8))) <= TOL_LOWP


def test_few_rows_full_size_weight_against_the_reference_kernel(eng):
    """16 x 8192 x 8192 (the weight of the headline configuration): every element against the
    one-thread-per-output kernel, sampled rows against the CPU oracle."""
    M, N, K = 16, 8192, 8192
    A, B = o.workloads.c2_gemm_bf16(M, N, K)
    Ad, Bd = A.to(DEV), B.to(DEV)
    C = eng.gemm_bf16(Ad, Bd, transB=True)
    Cn = eng.naive(o.KIND_BF16, Ad, Bd, transB=True)
    assert relmax(C.float().cpu().numpy(), Cn.float().cpu().numpy()) <= TOL_LOWP
    ref = oracle.gemm_bf16(bits16(A[:4]), bits16(B), transB=True)
    assert relmax(C[:4].float().cpu().numpy(), ref) <= TOL_LOWP
    assert eng.last_status() == (o.OK, 0)


@pytest.mark.parametrize("shape", [(129, 1024, 1024), (200, 2048, 2056), (256, 1304, 1024), (300, 512, 4096), (512, 768, 512)])
def test_several_row_tiles_per_column_block(eng, shape):
    """128 < M <= 512 when asked for: up to four 128-row tiles share each 256-column block of the
    weight; every (row tile, column block) has its own cluster."""
    M, N, K = shape
    A, B = _bf16_case(M, N, K, True, seed=13)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(2))
    ref = oracle.gemm_bf16(bits16(A), bits16(B), bias=bias.numpy(), act=oracle.ACT_RELU, transB=True)
    Ai, Bi = o.workloads.c5_int8(M, N, K, seed=M)
    refi = oracle.gemm_s8s8_s32(Ai.numpy(), Bi.numpy())
    try:
        for sk in (-1, -2, -4):
            eng.plan_set(o.KIND_BF16, split_k=sk)
            eng.plan_set(o.KIND_S8, split_k=sk)
            plan = eng.plan_get(o.KIND_BF16, M, N, K)
            assert plan["split_k"] < 0 and plan["tile_m"] == 128
            C = eng.gemm_bf16(A.to(DEV), B.to(DEV), transB=True, bias=bias.to(DEV), act="relu")
            assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP, sk
            Ci = eng.gemm_s8(Ai.to(DEV), Bi.to(DEV))
            assert np.array_equal(Ci.cpu().numpy(), refi), sk
    finally:
        eng.plan_set(o.KIND_BF16)
        eng.plan_set(o.KIND_S8)
    assert eng.last_status() == (o.OK, 0)


@pytest.mark.parametrize("shape", [(1, 2048, 1024), (17, 520, 4104), (64, 1304, 1096), (128, 4096, 2048),
                                   (100, 9000, 512), (300, 640, 2048), (9, 8, 131072)])
def test_128_column_tiles(eng, shape):
    """tile_n = 128: twice the tiles and half the partial sums to exchange per CTA; clusters of
    1, 2 and 4 (the plan reports what it took), both layouts of B, bias + activation, int8 and fp8."""
    M, N, K = shape
    A, B = _bf16_case(M, N, K, True, seed=21)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(4))
    ref = oracle.gemm_bf16(bits16(A), bits16(B), bias=bias.numpy(), act=oracle.ACT_SILU, transB=True)
    Ai, Bi = o.workloads.c5_int8(M, N, K, seed=M + 1)
    refi = oracle.gemm_s8s8_s32(Ai.numpy(), Bi.numpy())
    Bkn = B.t().contiguous()
    A8, W8, sA, sB, b8 = o.workloads.c4_fp8(M, N, K, seed=M + N)
    ref8 = oracle.gemm_fp8_scaled(bits8(A8), bits8(W8), sA.numpy(), sB.numpy(), b8.numpy())
    try:
        for sk in (-1, -2, -4, -8):
            eng.plan_set(o.KIND_BF16, split_k=sk, tile_n=128)
            eng.plan_set(o.KIND_S8, split_k=sk, tile_n=128)
            eng.plan_set(o.KIND_FP8, split_k=sk, tile_n=128)
            plan = eng.plan_get(o.KIND_BF16, M, N, K)
            assert plan["tile_n"] == 128 and -4 <= plan["split_k"] <= -1
            C = eng.gemm_bf16(A.to(DEV), B.to(DEV), transB=True, bias=bias.to(DEV), act="silu")
            assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP, sk
            C = eng.gemm_bf16(A.to(DEV), Bkn.to(DEV), transB=False, bias=bias.to(DEV), act="silu")
            assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP, sk
            Ci = eng.gemm_s8(Ai.to(DEV), Bi.to(DEV))
            assert np.array_equal(Ci.cpu().numpy(), refi), sk
            C8 = eng.gemm_fp8_scaled(A8.to(DEV), W8.to(DEV), sA.to(DEV), sB.to(DEV), b8.to(DEV))
            assert relmax(C8.float().cpu().numpy(), ref8) <= TOL_LOWP, sk
    finally:
        eng.plan_set(o.KIND_BF16)
        eng.plan_set(o.KIND_S8)
        eng.plan_set(o.KIND_FP8)
    assert eng.last_status() == (o.OK, 0)


def test_back_to_back_calls_that_depend_on_each_other(eng):
    """The kernel is launched so that it may be placed on SMs before the previous kernel of the
    stream has finished, and prefetches weight lines into L2 before it waits for that kernel.
    Chains without any synchronisation in between must still read what the previous call wrote:
    its result as the next A, and its result as the next WEIGHT (lines prefetched early are
    overwritten afterwards)."""
    g = torch.Generator().manual_seed(77)
    K, N = 4096, 8192
    W1 = (torch.randn(N, K, generator=g) / 64).to(torch.bfloat16).to(DEV)
    W2 = (torch.randn(1024, N, generator=g) / 64).to(torch.bfloat16).to(DEV)
    X = torch.randn(16, N, generator=g).to(torch.bfloat16).to(DEV)
    C1 = torch.zeros(128, N, dtype=torch.bfloat16, device=DEV)
    y1 = torch.zeros(16, N, dtype=torch.bfloat16, device=DEV)
    y2 = torch.zeros(16, 1024, dtype=torch.bfloat16, device=DEV)
    y3 = torch.zeros(16, 128, dtype=torch.bfloat16, device=DEV)
    try:
        eng.plan_set(o.KIND_BF16, split_k=-1)
        for rep in range(6):
            A16 = torch.randn(16, K, generator=g).to(torch.bfloat16).to(DEV)
            A128 = torch.randn(128, K, generator=g).to(torch.bfloat16).to(DEV)
            torch.cuda.synchronize()
            eng.gemm_bf16(A16, W1, transB=True, out=y1)      # layer 1
            eng.gemm_bf16(y1, W2, transB=True, out=y2)       # layer 2 reads layer 1's result as A
            eng.gemm_bf16(A128, W1, transB=True, out=C1)     # a 128 x 8192 product ...
            eng.gemm_bf16(X, C1, transB=True, out=y3)        # ... that is the next call's weight
            torch.cuda.synchronize()
            assert relmax(y1.float().cpu().numpy(), (A16.float() @ W1.float().t()).cpu().numpy()) <= TOL_LOWP
            assert relmax(y2.float().cpu().numpy(), (y1.float() @ W2.float().t()).cpu().numpy()) <= TOL_LOWP, rep
            assert relmax(C1.float().cpu().numpy(), (A128.float() @ W1.float().t()).cpu().numpy()) <= TOL_LOWP
            assert relmax(y3.float().cpu().numpy(), (X.float() @ C1.float().t()).cpu().numpy()) <= TOL_LOWP, rep
    finally:
        eng.plan_set(o.KIND_BF16)
    assert eng.last_status() == (o.OK, 0)
