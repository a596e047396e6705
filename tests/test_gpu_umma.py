"""GPU: the tcgen05 GEMM kernels through the C ABI against the CPU oracle.
bf16 / fp8 gate: max|y - ref| / max|ref| <= 2e-2 against the fp32 loop nest on the upcast or
dequantised operands.  int8 -> int32: bit exact."""
import numpy as np
import pytest
import torch

import open64_b200 as o
import oracle
from util import TOL_LOWP, bits16, bits8, from_bits16, from_bits8_e4m3, relmax

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ACTS = {"none": oracle.ACT_NONE, "relu": oracle.ACT_RELU, "gelu_tanh": oracle.ACT_GELU_TANH,
        "gelu_erf": oracle.ACT_GELU_ERF, "silu": oracle.ACT_SILU}

# one tile, several K blocks, ragged edges in every dimension, several tiles per CTA
SHAPES = [(128, 256, 64), (1, 8, 8), (7, 24, 40), (100, 200, 72), (129, 257, 136), (300, 520, 264),
          (256, 512, 1024), (640, 1536, 192)]


def _bf16_case(M, N, K, transB, seed=0):
    g = torch.Generator().manual_seed(seed + M * 131 + N * 17 + K)
    A = torch.randn(M, K, generator=g).to(torch.bfloat16)
    B = torch.randn((N, K) if transB else (K, N), generator=g).to(torch.bfloat16)
    return A, B


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("transB", [True, False])
def test_bf16_shapes(eng, shape, transB):
    M, N, K = shape
    A, B = _bf16_case(M, N, K, transB)
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    eng.gemm_bf16(A.to(DEV), B.to(DEV), transB=transB, out=C)
    ref = oracle.gemm_bf16(bits16(A), bits16(B), transB=transB)
    assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP


def test_bf16_golden_fixture(eng, golden):
    A = from_bits16(golden["c2_A"], DEV)
    B = from_bits16(golden["c2_B"], DEV)
    C = eng.gemm_bf16(A, B, transB=True)
    assert relmax(C.float().cpu().numpy(), golden["c2_C"]) <= TOL_LOWP


@pytest.mark.parametrize("act", list(ACTS))
def test_bf16_bias_and_activation_epilogues(eng, act):
    M, N, K = 200, 328, 136
    A, B = _bf16_case(M, N, K, True, seed=5)
    A = (A.float() * 0.2).to(torch.bfloat16)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(9))
    C = eng.gemm_bf16(A.to(DEV), B.to(DEV), transB=True, bias=bias.to(DEV), act=act)
    ref = oracle.gemm_bf16(bits16(A), bits16(B), bias=bias.numpy(), act=ACTS[act], transB=True)
    assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP


def test_bf16_both_tile_widths_and_rasters(eng):
    M, N, K = 700, 1100, 200
    A, B = _bf16_case(M, N, K, True, seed=2)
    ref = oracle.gemm_bf16(bits16(A), bits16(B), transB=True)
    Ad, Bd = A.to(DEV), B.to(DEV)
    try:
        for pin in (dict(tile_n=128), dict(tile_n=256), dict(tile_n=256, group_m=1),
                    dict(tile_n=128, group_m=3, raster=1), dict(tile_n=256, num_ctas=5),
                    dict(cta_group=1, tile_n=256), dict(cta_group=2, tile_n=256),
                    dict(cta_group=2, tile_n=128, group_m=2), dict(cta_group=2, tile_n=256, num_ctas=6)):
            eng.plan_set(o.KIND_BF16, **pin)
            C = eng.gemm_bf16(Ad, Bd, transB=True)
            assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP, pin
    finally:
        eng.plan_set(o.KIND_BF16)


def test_bf16_padded_leading_dimensions_and_unaligned_result(eng):
    M, N, K = 150, 200, 96
    g = torch.Generator().manual_seed(4)
    Ap = torch.randn(M, K + 8, generator=g).to(torch.bfloat16).to(DEV)
    Bp = torch.randn(N, K + 16, generator=g).to(torch.bfloat16).to(DEV)
    Cp = torch.full((M, N + 3), 5.0, dtype=torch.bfloat16, device=DEV)   # odd pitch: scalar stores
    eng.gemm_bf16(Ap[:, :K], Bp[:, :K], transB=True, out=Cp[:, :N])
    ref = oracle.gemm_bf16(bits16(Ap[:, :K].contiguous()), bits16(Bp[:, :K].contiguous()), transB=True)
    assert relmax(Cp[:, :N].float().cpu().numpy(), ref) <= TOL_LOWP
    assert (Cp[:, N:] == 5.0).all()


def test_bf16_operands_tma_cannot_address(eng):
    """Row pitches that are not multiples of 16 bytes and a misaligned base: the engine copies such
    operands into aligned scratch first."""
    M, N, K = 150, 90, 60                      # 120-byte rows; [K,N] rows of 180 bytes
    A, B = _bf16_case(M, N, K, True, seed=12)
    ref = oracle.gemm_bf16(bits16(A), bits16(B), transB=True)
    C = eng.gemm_bf16(A.to(DEV), B.to(DEV), transB=True)
    assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP
    Bkn = B.t().contiguous()
    C = eng.gemm_bf16(A.to(DEV), Bkn.to(DEV), transB=False)
    assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP
    flat = torch.zeros(M * K + 1, dtype=torch.bfloat16, device=DEV)
    flat[1:] = A.to(DEV).reshape(-1)
    C = eng.gemm_bf16(flat[1:].view(M, K), B.to(DEV), transB=True)   # base off by 2 bytes
    assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP
    X = A
    Wg = (torch.randn(K, 50, generator=torch.Generator().manual_seed(1)) * 0.1).to(torch.bfloat16)
    Wu = (torch.randn(K, 50, generator=torch.Generator().manual_seed(2)) * 0.1).to(torch.bfloat16)
    H = eng.swiglu(X.to(DEV), Wg.to(DEV), Wu.to(DEV))
    href = oracle.bf16_to_f32(oracle.swiglu_bf16(bits16(X), bits16(Wg), bits16(Wu)))
    assert relmax(H.float().cpu().numpy(), href) <= TOL_LOWP


def test_bf16_host_operands(eng):
    A, B = _bf16_case(130, 136, 72, True, seed=8)
    C = eng.gemm_bf16(A, B, transB=True)
    assert not C.is_cuda
    ref = oracle.gemm_bf16(bits16(A), bits16(B), transB=True)
    assert relmax(C.float().numpy(), ref) <= TOL_LOWP


@pytest.mark.parametrize("shape", [(128, 128, 64), (32, 48, 64), (300, 264, 136), (512, 1024, 320)])
def test_swiglu(eng, shape):
    M, N, K = shape
    g = torch.Generator().manual_seed(M + N + K)
    X = torch.randn(M, K, generator=g).to(torch.bfloat16)
    Wg = (torch.randn(K, N, generator=g) * 0.1).to(torch.bfloat16)
    Wu = (torch.randn(K, N, generator=g) * 0.1).to(torch.bfloat16)
    H = eng.swiglu(X.to(DEV), Wg.to(DEV), Wu.to(DEV))
    ref = oracle.bf16_to_f32(oracle.swiglu_bf16(bits16(X), bits16(Wg), bits16(Wu)))
    assert relmax(H.float().cpu().numpy(), ref) <= TOL_LOWP


def test_swiglu_golden_and_mlp(eng, golden):
    X, Wg, Wu = (from_bits16(golden[k], DEV) for k in ("c3_X", "c3_Wg", "c3_Wu"))
    H = eng.swiglu(X, Wg, Wu)
    assert relmax(H.float().cpu().numpy(), golden["c3_H"]) <= TOL_LOWP
    # the whole MLP: h stays bf16 between the two GEMMs, in the oracle too
    x, wg, wu, wd = o.workloads.c3_swiglu(96, 128, 192)
    out = eng.mlp_swiglu(x.to(DEV), wg.to(DEV), wu.to(DEV), wd.to(DEV))
    h = oracle.swiglu_bf16(bits16(x), bits16(wg), bits16(wu))
    ref = oracle.gemm_bf16(h, bits16(wd), transB=False)
    assert relmax(out.float().cpu().numpy(), ref) <= TOL_LOWP


@pytest.mark.parametrize("shape", [(128, 256, 128), (5, 16, 16), (100, 200, 144), (300, 520, 400),
                                   (512, 768, 1024)])
def test_fp8_scaled(eng, shape):
    M, N, K = shape
    A8, W8, sA, sB, bias = o.workloads.c4_fp8(M, N, K, seed=M + N + K)
    C = eng.gemm_fp8_scaled(A8.to(DEV), W8.to(DEV), sA.to(DEV), sB.to(DEV), bias.to(DEV))
    ref = oracle.gemm_fp8_scaled(bits8(A8), bits8(W8), sA.numpy(), sB.numpy(), bias.numpy())
    assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP
    # scales and bias are optional
    C2 = eng.gemm_fp8_scaled(A8.to(DEV), W8.to(DEV))
    ref2 = oracle.gemm_fp8_scaled(bits8(A8), bits8(W8))
    assert relmax(C2.float().cpu().numpy(), ref2) <= TOL_LOWP


def test_fp8_golden_fixture(eng, golden):
    A8 = from_bits8_e4m3(golden["c4_A8"], DEV)
    B8 = from_bits8_e4m3(golden["c4_B8"], DEV)
    sA, sB, bias = (torch.from_numpy(golden[k]).to(DEV) for k in ("c4_sA", "c4_sB", "c4_bias"))
    C = eng.gemm_fp8_scaled(A8, B8, sA, sB, bias)
    assert relmax(C.float().cpu().numpy(), golden["c4_C"]) <= TOL_LOWP


@pytest.mark.parametrize("shape", [(128, 256, 128), (1, 4, 16), (3, 20, 48), (100, 200, 144),
                                   (300, 520, 400), (512, 768, 2048)])
def test_int8_bit_exact(eng, shape):
    M, N, K = shape
    A, B = o.workloads.c5_int8(M, N, K, seed=M * 3 + N + K)
    C = torch.full((M, N), -1, dtype=torch.int32, device=DEV)
    eng.gemm_s8(A.to(DEV), B.to(DEV), out=C)
    assert np.array_equal(C.cpu().numpy(), oracle.gemm_s8s8_s32(A.numpy(), B.numpy()))


def test_int8_golden_and_extremes(eng, golden):
    A = torch.from_numpy(golden["c5_A"]).to(DEV)
    B = torch.from_numpy(golden["c5_B"]).to(DEV)
    assert np.array_equal(eng.gemm_s8(A, B).cpu().numpy(), golden["c5_C"])
    # the largest magnitudes the contract allows, K = 8192: |acc| = 8192 * 127^2 < 2^31
    K = 8192
    A = torch.full((130, K), -127, dtype=torch.int8, device=DEV)
    B = torch.full((24, K), 127, dtype=torch.int8, device=DEV)
    B[1::2] = -127
    C = eng.gemm_s8(A, B)
    exp = torch.tensor([-K * 127 * 127, K * 127 * 127], dtype=torch.int32, device=DEV).repeat(12)
    assert torch.equal(C, exp.expand(130, 24))


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("tile_n", [128, 256])
def test_every_kind_on_one_cta_and_on_cta_pairs(eng, cta_group, tile_n):
    """Pins the plan so that both kernel families (one CTA per tile, a pair of CTAs per tile)
    are exercised for every element kind, on shapes with ragged edges and several tiles per CTA."""
    M, N, K = 700, 1160, 328
    try:
        for kind in (o.KIND_BF16, o.KIND_FP8, o.KIND_S8):
            eng.plan_set(kind, cta_group=cta_group, tile_n=tile_n, num_ctas=8)
        A, B = _bf16_case(M, N, K, True, seed=3)
        C = eng.gemm_bf16(A.to(DEV), B.to(DEV), transB=True)
        assert relmax(C.float().cpu().numpy(), oracle.gemm_bf16(bits16(A), bits16(B), transB=True)) <= TOL_LOWP
        Bkn = B.t().contiguous()
        C = eng.gemm_bf16(A.to(DEV), Bkn.to(DEV), transB=False, act="gelu_tanh")
        ref = oracle.gemm_bf16(bits16(A), bits16(Bkn), transB=False, act=oracle.ACT_GELU_TANH)
        assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP
        if not (cta_group == 2 and tile_n == 128):      # the fused gate/up kernel on pairs is 256 wide only
            Wg = (Bkn.float() * 0.1).to(torch.bfloat16)
            Wu = (torch.randn(K, N, generator=torch.Generator().manual_seed(6)) * 0.1).to(torch.bfloat16)
            H = eng.swiglu(A.to(DEV), Wg.to(DEV), Wu.to(DEV))
            href = oracle.bf16_to_f32(oracle.swiglu_bf16(bits16(A), bits16(Wg), bits16(Wu)))
            assert relmax(H.float().cpu().numpy(), href) <= TOL_LOWP
        A8, W8, sA, sB, bias = o.workloads.c4_fp8(M, N, K, seed=5)
        C = eng.gemm_fp8_scaled(A8.to(DEV), W8.to(DEV), sA.to(DEV), sB.to(DEV), bias.to(DEV))
        ref = oracle.gemm_fp8_scaled(bits8(A8), bits8(W8), sA.numpy(), sB.numpy(), bias.numpy())
        assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP
        Ai, Bi = o.workloads.c5_int8(M, N, K, seed=7)
        Ci = eng.gemm_s8(Ai.to(DEV), Bi.to(DEV))
        assert np.array_equal(Ci.cpu().numpy(), oracle.gemm_s8s8_s32(Ai.numpy(), Bi.numpy()))
    finally:
        for kind in (o.KIND_BF16, o.KIND_FP8, o.KIND_S8):
            eng.plan_set(kind)


@pytest.mark.parametrize("shape", [(16, 256, 2048), (200, 512, 4096), (129, 256, 8192), (40, 300, 1096)])
def test_split_k_for_skinny_shapes(eng, shape):
    """Few output tiles and a long K: slices of K go to separate CTAs and meet in scratch memory
    (fp32 atomics + a finishing kernel for 16-bit results, int32 atomics in place for int8)."""
    M, N, K = shape
    assert eng.plan_get(o.KIND_BF16, M, N, K)["split_k"] > 1
    A, B = _bf16_case(M, N, K, True, seed=21)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(3))
    ref = oracle.gemm_bf16(bits16(A), bits16(B), bias=bias.numpy(), act=oracle.ACT_RELU, transB=True)
    for rep in range(2):   # the scratch is re-zeroed by every call
        C = eng.gemm_bf16(A.to(DEV), B.to(DEV), transB=True, bias=bias.to(DEV), act="relu")
        assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP
    try:
        eng.plan_set(o.KIND_BF16, cta_group=1, tile_n=256, split_k=5)
        C = eng.gemm_bf16(A.to(DEV), B.to(DEV), transB=True, bias=bias.to(DEV), act="relu")
        assert relmax(C.float().cpu().numpy(), ref) <= TOL_LOWP
    finally:
        eng.plan_set(o.KIND_BF16)
    Ai, Bi = o.workloads.c5_int8(M, N, K, seed=M + K)
    Cpad = torch.full((M, N + 4), -9, dtype=torch.int32, device=DEV)
    eng.gemm_s8(Ai.to(DEV), Bi.to(DEV), out=Cpad[:, :N])
    assert np.array_equal(Cpad[:, :N].cpu().numpy(), oracle.gemm_s8s8_s32(Ai.numpy(), Bi.numpy()))
    assert (Cpad[:, N:] == -9).all()
    A8, W8, sA, sB, b8 = o.workloads.c4_fp8(M, N, K, seed=9)
    C8 = eng.gemm_fp8_scaled(A8.to(DEV), W8.to(DEV), sA.to(DEV), sB.to(DEV), b8.to(DEV))
    ref8 = oracle.gemm_fp8_scaled(bits8(A8), bits8(W8), sA.numpy(), sB.numpy(), b8.numpy())
    assert relmax(C8.float().cpu().numpy(), ref8) <= TOL_LOWP


@pytest.mark.parametrize("pinned", [True, False])
def test_tall_host_operands_travel_in_row_blocks(eng, pinned):
    """Host A and host C with at least 2048 rows: the rows are copied, multiplied and copied back in
    blocks on separate streams.  Same results as with device operands; the last block is ragged."""
    M, N, K = 2304, 384, 256
    A, B = _bf16_case(M, N, K, True, seed=31)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(5))
    Ah = A.pin_memory() if pinned else A
    Ch = torch.full((M, N), float("nan"), dtype=torch.bfloat16)
    if pinned:
        Ch = Ch.pin_memory()
    for rep in range(2):
        eng.gemm_bf16(Ah, B.to(DEV), transB=True, bias=bias.to(DEV), act="gelu_tanh", out=Ch)
        Cd = eng.gemm_bf16(A.to(DEV), B.to(DEV), transB=True, bias=bias.to(DEV), act="gelu_tanh")
        assert torch.equal(Ch, Cd.cpu())
    ref = oracle.gemm_bf16(bits16(A[-300:]), bits16(B), bias=bias.numpy(), act=oracle.ACT_GELU_TANH, transB=True)
    assert relmax(Ch[-300:].float().numpy(), ref) <= TOL_LOWP
    # int8 (exact) and fp8 with per-row scales (the scale vector is offset per block), B on the host too
    Ai, Bi = o.workloads.c5_int8(M, N, K, seed=77)
    Ci = torch.empty((M, N), dtype=torch.int32)
    eng.gemm_s8(Ai, Bi, out=Ci)
    assert np.array_equal(Ci.numpy(), oracle.gemm_s8s8_s32(Ai.numpy(), Bi.numpy()))
    A8, W8, sA, sB, b8 = o.workloads.c4_fp8(M, N, K, seed=78)
    C8 = torch.empty((M, N), dtype=torch.bfloat16)
    eng.gemm_fp8_scaled(A8, W8.to(DEV), sA.to(DEV), sB.to(DEV), b8.to(DEV), out=C8)
    ref8 = oracle.gemm_fp8_scaled(bits8(A8), bits8(W8), sA.numpy(), sB.numpy(), b8.numpy())
    assert relmax(C8.float().numpy(), ref8) <= TOL_LOWP
    assert eng.last_status() == (o.OK, 0)


def test_measured_plans(eng):
    """o64_plan_tune times the kernel shapes for one problem size and the engine then uses the fastest
    for that size (until a pin says otherwise); results stay correct."""
    M, N, K = 768, 2048, 1024
    A, B = _bf16_case(M, N, K, True, seed=41)
    ref = oracle.gemm_bf16(bits16(A[:64]), bits16(B), transB=True)
    Ad, Bd = A.to(DEV), B.to(DEV)

    def time_default():
        for _ in range(3):
            eng.gemm_bf16(Ad, Bd, transB=True)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(40):
            eng.gemm_bf16(Ad, Bd, transB=True)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 40

    before = time_default()
    try:
        best = eng.plan_tune(o.KIND_BF16, M, N, K)
        assert best["predicted_ms"] > 0 and best["tile_n"] in (128, 256)
        got = eng.plan_get(o.KIND_BF16, M, N, K)
        assert all(got[k] == best[k] for k in ("cta_group", "tile_m", "tile_n", "split_k"))
        assert eng.plan_get(o.KIND_BF16, M + 128, N, K) is not None          # other sizes: the model as before
        C = eng.gemm_bf16(Ad, Bd, transB=True)
        assert relmax(C[:64].float().cpu().numpy(), ref) <= TOL_LOWP
        after = time_default()
        assert after <= before * 1.3, (before, after, best)   # a sanity bound: eager timing of a 25 us kernel is noisy
        # a pin still wins over a measured plan
        eng.plan_set(o.KIND_BF16, cta_group=1, tile_n=128, split_k=1)
        assert eng.plan_get(o.KIND_BF16, M, N, K)["cta_group"] == 1
        eng.plan_set(o.KIND_BF16)
        # few rows: the cluster kernel's cluster sizes are among the candidates
        few = eng.plan_tune(o.KIND_S8, 32, 4096, 4096)
        Ai, Bi = o.workloads.c5_int8(32, 4096, 4096, seed=3)
        assert np.array_equal(eng.gemm_s8(Ai.to(DEV), Bi.to(DEV)).cpu().numpy(), oracle.gemm_s8s8_s32(Ai.numpy(), Bi.numpy()))
        assert few["predicted_ms"] > 0
    finally:
        eng.plan_set(o.KIND_BF16)
        eng.plan_tune_clear()
    assert eng.last_status() == (o.OK, 0)
