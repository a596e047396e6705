"""GPU: the scaled products with a fused activation and a requantised result.
int8 operands: the accumulator is an exact integer and the tail is specified operation by operation
(nothing fused), so bf16 and int8 results must equal the oracle's BIT FOR BIT where the activation is
exact (none, ReLU); with GELU / SiLU (libm vs the device's expf / tanhf) an int8 result may differ by
one step in a few places.  e4m3 operands accumulate in a different order on the tensor cores: results
are held to the contract's tolerance, e4m3 results to one step of that format."""
import numpy as np
import pytest
import torch

import open64_b200 as o
import oracle
from util import TOL_LOWP, bits8, from_bits8_e4m3, relmax

pytestmark = pytest.mark.gpu
ACTS = {"none": oracle.ACT_NONE, "relu": oracle.ACT_RELU, "gelu_tanh": oracle.ACT_GELU_TANH, "silu": oracle.ACT_SILU}

PINS = [None, dict(cta_group=1, tile_m=128, tile_n=256, split_k=1), dict(cta_group=1, tile_m=128, tile_n=128, split_k=1),
        dict(cta_group=2, tile_m=256, tile_n=256), dict(cta_group=2, tile_m=256, tile_n=128)]


def _int8_case(M, N, K, seed):
    A, B = o.workloads.c5_int8(M, N, K, seed=seed)
    g = torch.Generator().manual_seed(seed + 1)
    sA = (torch.rand(M, generator=g) * 0.01 + 0.002).float()
    sB = (torch.rand(N, generator=g) * 0.01 + 0.002).float()
    bias = (torch.rand(N, generator=g) * 8 - 4).float()
    return A, B, sA, sB, bias


@pytest.mark.parametrize("pin", PINS, ids=["auto", "1cta256", "1cta128", "pair256", "pair128"])
@pytest.mark.parametrize("M,N,K", [(256, 512, 384), (300, 1000, 1100), (130, 72, 200)])
def test_int8_scaled_exact(eng, pin, M, N, K):
    dev = torch.device("cuda", eng.device)
    A, B, sA, sB, bias = _int8_case(M, N, K, seed=M + N)
    if pin:
        eng.plan_set(o.KIND_S8, **pin)
    try:
        for act in ("none", "relu"):
            for out_kind, okind in ((o.OUT_S8, 1), (o.OUT_BF16, 3)):
                want = oracle.gemm_s8_scaled(A.numpy(), B.numpy(), sA.numpy(), sB.numpy(), bias.numpy(), ACTS[act], okind)
                got = eng.gemm_s8_scaled(A.to(dev), B.to(dev), sA.to(dev), sB.to(dev), bias.to(dev), act, out_kind)
                got = got.cpu().numpy() if out_kind == o.OUT_S8 else got.view(torch.int16).cpu().numpy().view(np.uint16)
                assert np.array_equal(got, want), (pin, act, out_kind, int((got != want).sum()))
            if act == "relu":
                assert (want >= 0).all() if okind == 1 else True
        assert eng.last_status() == (o.OK, 0)
    finally:
        eng.plan_set(o.KIND_S8)


def test_int8_requant_saturates_and_rounds_to_even(eng):
    dev = torch.device("cuda", eng.device)
    M, N, K = 128, 128, 64
    A = torch.ones((M, K), dtype=torch.int8)
    B = torch.ones((N, K), dtype=torch.int8)                      # acc = 64 everywhere
    sB = torch.ones(N)
    # 64 * s: halves round to even, large magnitudes saturate
    sA = torch.tensor([0.0078125 * v for v in (1, 3, 5, 7)] * (M // 4))    # 0.5, 1.5, 2.5, 3.5
    got = eng.gemm_s8_scaled(A.to(dev), B.to(dev), sA.to(dev), sB.to(dev), None, "none", o.OUT_S8).cpu()
    assert got[:4, 0].tolist() == [0, 2, 2, 4]
    big = eng.gemm_s8_scaled(A.to(dev), B.to(dev), torch.full((M,), 100.0, device=dev), None,
                             None, "none", o.OUT_S8).cpu()
    assert (big == 127).all()
    neg = eng.gemm_s8_scaled(A.to(dev), (-B).to(dev), torch.full((M,), 100.0, device=dev), None,
                             None, "none", o.OUT_S8).cpu()
    assert (neg == -128).all()


@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
def test_int8_scaled_with_transcendental_activation(eng, act):
    dev = torch.device("cuda", eng.device)
    A, B, sA, sB, bias = _int8_case(256, 512, 512, seed=9)
    ref = oracle.gemm_s8_scaled(A.numpy(), B.numpy(), sA.numpy(), sB.numpy(), bias.numpy(), ACTS[act], 0)
    got = eng.gemm_s8_scaled(A.to(dev), B.to(dev), sA.to(dev), sB.to(dev), bias.to(dev), act, o.OUT_BF16)
    assert relmax(got.float().cpu().numpy(), ref) <= 4e-3
    q = eng.gemm_s8_scaled(A.to(dev), B.to(dev), sA.to(dev), sB.to(dev), bias.to(dev), act, o.OUT_S8).cpu().numpy()
    want = oracle.gemm_s8_scaled(A.numpy(), B.numpy(), sA.numpy(), sB.numpy(), bias.numpy(), ACTS[act], 1)
    diff = np.abs(q.astype(np.int32) - want.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 1e-3


@pytest.mark.parametrize("pin", [None, dict(cta_group=2, tile_m=256, tile_n=256), dict(cta_group=1, tile_m=128, tile_n=128, split_k=1)],
                         ids=["auto", "pair256", "1cta128"])
def test_fp8_scaled_activation_and_e4m3_result(eng, pin):
    dev = torch.device("cuda", eng.device)
    A8, W8, sA, sB, b = o.workloads.c4_fp8(300, 1000, 1100)
    a8, w8 = bits8(A8), bits8(W8)
    if pin:
        eng.plan_set(o.KIND_FP8, **pin)
    try:
        for act in ("none", "silu"):
            ref = oracle.gemm_fp8_scaled_ex(a8, w8, sA.numpy(), sB.numpy(), b.numpy(), ACTS[act], 0)
            got = eng.gemm_fp8_scaled_ex(A8.to(dev), W8.to(dev), sA.to(dev), sB.to(dev), b.to(dev), act, o.OUT_BF16)
            assert relmax(got.float().cpu().numpy(), ref) <= 4e-3
            # requantised: scale so that the result spans e4m3's range
            s_out = (200.0 / np.abs(ref).max()).astype(np.float32)
            ref8 = oracle.gemm_fp8_scaled_ex(a8, w8, sA.numpy() * s_out, sB.numpy(), b.numpy() * s_out, ACTS["none"], 2)
            got8 = eng.gemm_fp8_scaled_ex(A8.to(dev), W8.to(dev), (sA * float(s_out)).to(dev), sB.to(dev),
                                          (b * float(s_out)).to(dev), "none", o.OUT_E4M3)
            g = oracle.e4m3_to_f32(bits8(got8))
            r = oracle.e4m3_to_f32(ref8)
            assert np.isfinite(g).all()
            # one step of e4m3 is 1/8 of the value's binade: 12.5 % of it at most
            assert (np.abs(g - r) <= 0.126 * np.maximum(np.abs(r), 2.0 ** -6)).all()
            assert (g == r).mean() > 0.9
        assert eng.last_status() == (o.OK, 0)
    finally:
        eng.plan_set(o.KIND_FP8)


def test_host_operands_and_errors(eng):
    A, B, sA, sB, bias = _int8_case(128, 256, 128, seed=4)
    want = oracle.gemm_s8_scaled(A.numpy(), B.numpy(), sA.numpy(), sB.numpy(), bias.numpy(), oracle.ACT_RELU, 1)
    out = torch.empty((128, 256), dtype=torch.int8)
    eng.gemm_s8_scaled(A, B, sA, sB, bias, "relu", o.OUT_S8, out=out)             # all on the host: staged
    assert np.array_equal(out.numpy(), want)
    with pytest.raises(o.O64Error) as e:
        eng.gemm_s8_scaled(A, B, sA, sB, bias, "relu", o.OUT_E4M3, out=out)
    assert e.value.status == o.ERR_DTYPE


@pytest.mark.parametrize("shape", [(300, 1000, 1100), (64, 130, 70), (1, 16, 16)])
def test_fp8_weight_stored_k_by_n(eng, shape):
    """The [K,N] entry point gives bit for bit what the [N,K] entry point gives on the transposed
    weight (the same kernels run on a transposed copy), also with a padded leading dimension."""
    dev = torch.device("cuda", eng.device)
    M, N, K = shape
    A8, W8, sA, sB, b = o.workloads.c4_fp8(M, N, K)
    a8, w8 = A8.to(dev), W8.to(dev)
    want = eng.gemm_fp8_scaled_ex(a8, w8, sA.to(dev), sB.to(dev), b.to(dev), "silu", o.OUT_BF16)
    w_kn = w8.view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn)          # [K, N]
    got = eng.gemm_fp8_scaled_kn(a8, w_kn, sA.to(dev), sB.to(dev), b.to(dev), "silu", o.OUT_BF16)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    ref = oracle.gemm_fp8_scaled_ex(bits8(A8), bits8(W8), sA.numpy(), sB.numpy(), b.numpy(), ACTS["silu"], 0)
    assert relmax(got.float().cpu().numpy(), ref) <= 4e-3
    wide = torch.zeros((K, N + 24), dtype=torch.uint8, device=dev)
    wide[:, :N] = w_kn.view(torch.uint8)
    got2 = eng.gemm_fp8_scaled_kn(a8, wide.view(torch.float8_e4m3fn)[:, :N], sA.to(dev), sB.to(dev), b.to(dev), "silu", o.OUT_BF16)
    assert torch.equal(got2.view(torch.int16), want.view(torch.int16))
    with pytest.raises(o.O64Error):
        eng.gemm_fp8_scaled_kn(a8, w_kn.cpu(), sA.to(dev), sB.to(dev), b.to(dev))


@pytest.mark.parametrize("out_kind", ["bf16", "e4m3"])
def test_fp8_weight_stored_k_by_n_read_in_place(eng, out_kind):
    """An aligned [K,N] e4m3 weight is multiplied as it lies (N-major shared-memory descriptor, 256 x 256
    tiles of the CTA-pair kernel): same bits as the [N,K] kernels on the transposed weight; ragged M, N
    and K; no scratch copy of the weight is made."""
    dev = torch.device("cuda", eng.device)
    M, N, K = 700, 1200, 1000            # N a multiple of 16: the pitch of the [K,N] weight is TMA-addressable
    A8, W8, sA, sB, b = o.workloads.c4_fp8(M, N, K)
    a8, w8 = A8.to(dev), W8.to(dev)
    w_kn = w8.view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn)
    kind = o.OUT_E4M3 if out_kind == "e4m3" else o.OUT_BF16
    scale = 0.05 if out_kind == "e4m3" else 1.0
    args = ((sA * scale).to(dev), sB.to(dev), (b * scale).to(dev), "relu", kind)
    free0 = torch.cuda.mem_get_info()[0]
    got = eng.gemm_fp8_scaled_kn(a8, w_kn, *args)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free0 - got.numel() * got.element_size() - (1 << 20)  # the result only
    want = eng.gemm_fp8_scaled_ex(a8, w8, *args)
    assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
    ref = oracle.gemm_fp8_scaled_ex(bits8(A8), bits8(W8), (sA * scale).numpy(), sB.numpy(), (b * scale).numpy(), ACTS["relu"],
                                    2 if out_kind == "e4m3" else 0)
    if out_kind == "bf16":
        assert relmax(got.float().cpu().numpy(), ref) <= 4e-3
    else:
        g8 = got.float().cpu().numpy()
        r8 = from_bits8_e4m3(ref).float().numpy()
        assert relmax(g8, r8) <= 7e-2    # one e4m3 rounding of the largest value
