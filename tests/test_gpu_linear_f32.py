"""GPU: the fp32 fused linear (CUDA cores) through the C ABI against the CPU oracle.
Gate: max|y - ref| / max|ref| <= 1e-4."""
import numpy as np
import pytest
import torch

import open64_b200 as o
import oracle
from util import TOL_F32, relmax

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ACTS = {"none": oracle.ACT_NONE, "relu": oracle.ACT_RELU, "gelu_tanh": oracle.ACT_GELU_TANH,
        "gelu_erf": oracle.ACT_GELU_ERF, "silu": oracle.ACT_SILU}


def test_c1_full_config(eng):
    A, B, bias = o.workloads.c1_linear_f32()
    y = eng.linear_f32(A.to(DEV), B.to(DEV), bias.to(DEV), "relu").cpu().numpy()
    ref = oracle.linear_f32(A.numpy(), B.numpy(), bias.numpy(), oracle.ACT_RELU)
    assert relmax(y, ref) <= TOL_F32
    assert (y >= 0).all() and ((y == 0) == (ref == 0)).mean() > 0.999
    # the second device implementation (one thread per output, unfused multiply-add) is the
    # loop nest verbatim: identical to the oracle except for the device's expf-free ReLU path
    yn = eng.naive(o.KIND_F32, A.to(DEV), B.to(DEV), transB=False, bias=bias.to(DEV), act="relu")
    assert np.array_equal(yn.cpu().numpy(), ref)


def test_golden_fixture(eng, golden):
    A, B, bias = (torch.from_numpy(golden[k]).to(DEV) for k in ("c1_A", "c1_B", "c1_bias"))
    y = eng.linear_f32(A, B, bias, "relu").cpu().numpy()
    assert relmax(y, golden["c1_Y"]) <= TOL_F32


@pytest.mark.parametrize("shape", [(1, 1, 1), (1, 7, 3), (5, 1, 9), (33, 65, 17), (64, 64, 16),
                                   (77, 131, 93), (200, 300, 1), (129, 257, 513), (1000, 40, 7)])
@pytest.mark.parametrize("act", ["none", "silu"])
def test_ragged_shapes(eng, shape, act):
    M, N, K = shape
    g = torch.Generator().manual_seed(M * 31 + N * 7 + K)
    A = torch.randn(M, K, generator=g)
    B = torch.randn(K, N, generator=g)
    bias = torch.randn(N, generator=g)
    y = eng.linear_f32(A.to(DEV), B.to(DEV), bias.to(DEV), act).cpu().numpy()
    ref = oracle.linear_f32(A.numpy(), B.numpy(), bias.numpy(), ACTS[act])
    assert relmax(y, ref) <= TOL_F32


@pytest.mark.parametrize("act", list(ACTS))
def test_every_activation(eng, act):
    A, B, bias = o.workloads.c1_linear_f32(96, 80, 64, seed=7)
    y = eng.linear_f32(A.to(DEV), B.to(DEV), bias.to(DEV), act).cpu().numpy()
    ref = oracle.linear_f32(A.numpy(), B.numpy(), bias.numpy(), ACTS[act])
    assert relmax(y, ref) <= TOL_F32


def test_big_tile_path_and_padded_leading_dimensions(eng):
    # enough 64x64 tiles to take the large-tile kernel; operands are views with padding
    M, N, K = 1500, 1300, 70
    g = torch.Generator().manual_seed(11)
    Ap = torch.randn(M, K + 5, generator=g)
    Bp = torch.randn(K, N + 3, generator=g)
    Yp = torch.full((M, N + 9), -7.0, device=DEV)
    A, B = Ap[:, :K], Bp[:, :N]
    eng.linear_f32(A.to(DEV)[:, :K], B.to(DEV)[:, :N], None, "none", out=Yp[:, :N])
    ref = oracle.linear_f32(A.contiguous().numpy(), B.contiguous().numpy())
    assert relmax(Yp[:, :N].cpu().numpy(), ref) <= TOL_F32
    assert (Yp[:, N:] == -7.0).all()          # nothing written beyond N


def test_empty_extents(eng):
    A = torch.zeros(0, 8, device=DEV)
    B = torch.zeros(8, 5, device=DEV)
    assert eng.linear_f32(A, B).shape == (0, 5)
    # K == 0: the empty sum is zero, so Y = act(bias)
    A = torch.zeros(4, 0, device=DEV)
    B = torch.zeros(0, 5, device=DEV)
    bias = torch.arange(5, dtype=torch.float32, device=DEV) - 2
    y = eng.linear_f32(A, B, bias, "relu")
    assert torch.equal(y, torch.relu(bias).expand(4, 5))


def test_host_operands_are_staged(eng):
    A, B, bias = o.workloads.c1_linear_f32(70, 50, 30, seed=3)
    y = eng.linear_f32(A, B, bias, "relu")          # CPU tensors in, CPU tensor out
    assert not y.is_cuda
    ref = oracle.linear_f32(A.numpy(), B.numpy(), bias.numpy(), oracle.ACT_RELU)
    assert relmax(y.numpy(), ref) <= TOL_F32


def test_pinned_tiles_of_the_dense_kernel(eng):
    """tile_m x tile_n of the CUDA-core kernel can be pinned (what `#pragma blocking size` on the i and
    j loops of a rewritten nest turns into); sizes without a kernel are refused."""
    g = torch.Generator().manual_seed(12)
    A, B = torch.rand(200, 136, generator=g) - 0.5, torch.rand(136, 328, generator=g) - 0.5
    bias = torch.rand(328, generator=g)
    ref = oracle.linear_f32(A.numpy(), B.numpy(), bias.numpy(), oracle.ACT_RELU)
    try:
        for tm, tn in ((32, 32), (32, 64), (64, 64)):
            eng.plan_set(o.KIND_F32, tile_m=tm, tile_n=tn)
            p = eng.plan_get(o.KIND_F32, 200, 328, 136)
            assert (p["tile_m"], p["tile_n"]) == (tm, tn)
            y = eng.linear_f32(A.to(DEV), B.to(DEV), bias.to(DEV), act="relu")
            assert relmax(y.cpu().numpy(), ref) <= TOL_F32
        for bad in (dict(tile_m=64, tile_n=32), dict(tile_m=128), dict(tile_n=48), dict(tile_k=32)):
            with pytest.raises(o.O64Error) as e:
                eng.plan_set(o.KIND_F32, **bad)
            assert e.value.status == o.ERR_RANK
    finally:
        eng.plan_set(o.KIND_F32)
