"""GPU: the benchmark configurations at their full sizes.

The CPU oracle checks sampled rows and columns (seconds of CPU work); the full matrices are
compared on the device against the one-thread-per-output reference kernels (the loop nest run
verbatim, themselves checked against the oracle on the same samples); and size-independent
properties are checked on the full results: power-of-two scaling and row-permutation
equivariance (bit exact), and a checksum of checksums for the integer product."""
import numpy as np
import pytest
import torch

import open64_b200 as o
import oracle
from util import TOL_LOWP, bits16, bits8, relmax

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def sample_idx(n, count, seed):
    rng = np.random.default_rng(seed)
    idx = np.unique(np.concatenate([[0, n - 1, 127, 128], rng.integers(0, n, count)]))
    return torch.from_numpy(idx[idx < n])


def dev_relmax(y, ref):
    return ((y.double() - ref.double()).abs().max() / ref.double().abs().max()).item()


def test_c2_bf16_8192(eng):
    M = N = K = 8192
    A, B = o.workloads.c2_gemm_bf16(M, N, K)
    Ad, Bd = A.to(DEV), B.to(DEV)
    C = eng.gemm_bf16(Ad, Bd, transB=True)
    ref_dev = eng.naive(o.KIND_BF16, Ad, Bd, transB=True)
    assert dev_relmax(C, ref_dev) <= TOL_LOWP
    rows = sample_idx(M, 24, 1)
    cols = sample_idx(N, 24, 2)
    ref_rows = oracle.gemm_bf16(bits16(A[rows]), bits16(B), transB=True)
    ref_cols = oracle.gemm_bf16(bits16(A), bits16(B[cols]), transB=True)
    assert np.array_equal(ref_dev[rows.to(DEV)].cpu().numpy(), ref_rows)      # nest run verbatim
    assert relmax(C[rows.to(DEV)].float().cpu().numpy(), ref_rows) <= TOL_LOWP
    assert relmax(C[:, cols.to(DEV)].float().cpu().numpy(), ref_cols) <= TOL_LOWP
    # scaling an operand by two commutes with every rounding in the path
    C2 = eng.gemm_bf16((Ad.float() * 2).to(torch.bfloat16), Bd, transB=True)
    assert torch.equal(C2.float(), C.float() * 2)
    # permuting rows of A permutes rows of C
    perm = torch.randperm(M, device=DEV, generator=torch.Generator(DEV).manual_seed(3))
    Cp = eng.gemm_bf16(Ad[perm].contiguous(), Bd, transB=True)
    assert torch.equal(Cp, C[perm])


def test_c3_swiglu_mlp(eng):
    T, D, F = 4096, 4096, 14336
    x, Wg, Wu, Wd = o.workloads.c3_swiglu(T, D, F)
    xd, Wgd, Wud, Wdd = (t.to(DEV) for t in (x, Wg, Wu, Wd))
    h = torch.empty(T, F, dtype=torch.bfloat16, device=DEV)
    out = eng.mlp_swiglu(xd, Wgd, Wud, Wdd, h=h)
    # device reference: the two products by the verbatim nest, SiLU-multiply in fp32, h rounded
    # to bf16 as the engine keeps it
    g_ref = eng.naive(o.KIND_BF16, xd, Wgd, transB=False)
    u_ref = eng.naive(o.KIND_BF16, xd, Wud, transB=False)
    h_ref = (torch.nn.functional.silu(g_ref) * u_ref)
    assert dev_relmax(h, h_ref) <= TOL_LOWP
    out_ref = eng.naive(o.KIND_BF16, h_ref.to(torch.bfloat16), Wdd, transB=False)
    assert dev_relmax(out, out_ref) <= TOL_LOWP
    del g_ref, u_ref
    rows = sample_idx(T, 12, 4)
    h_o = oracle.swiglu_bf16(bits16(x[rows]), bits16(Wg), bits16(Wu))
    assert relmax(h[rows.to(DEV)].float().cpu().numpy(), oracle.bf16_to_f32(h_o)) <= TOL_LOWP
    out_o = oracle.gemm_bf16(h_o, bits16(Wd), transB=False)
    assert relmax(out[rows.to(DEV)].float().cpu().numpy(), out_o) <= TOL_LOWP


def test_c4_fp8_scaled(eng):
    M, N, K = 4096, 8192, 8192
    A8, W8, sA, sB, bias = o.workloads.c4_fp8(M, N, K)
    A8d, W8d, sAd, sBd, bd = (t.to(DEV) for t in (A8, W8, sA, sB, bias))
    C = eng.gemm_fp8_scaled(A8d, W8d, sAd, sBd, bd)
    ref_dev = eng.naive(o.KIND_FP8, A8d, W8d, transB=True, scaleA=sAd, scaleB=sBd, bias=bd)
    assert dev_relmax(C, ref_dev) <= TOL_LOWP
    rows = sample_idx(M, 24, 5)
    ref_rows = oracle.gemm_fp8_scaled(bits8(A8[rows]), bits8(W8), sA[rows].numpy(), sB.numpy(),
                                      bias.numpy())
    assert relmax(ref_dev[rows.to(DEV)].cpu().numpy(), ref_rows) <= 1e-6
    assert relmax(C[rows.to(DEV)].float().cpu().numpy(), ref_rows) <= TOL_LOWP
    cols = sample_idx(N, 24, 6)
    ref_cols = oracle.gemm_fp8_scaled(bits8(A8), bits8(W8[cols]), sA.numpy(), sB[cols].numpy(),
                                      bias[cols].numpy())
    assert relmax(C[:, cols.to(DEV)].float().cpu().numpy(), ref_cols) <= TOL_LOWP
    # a power-of-two change of a scale vector scales (C - bias) exactly
    C0 = eng.gemm_fp8_scaled(A8d, W8d, sAd, sBd, None)
    C1 = eng.gemm_fp8_scaled(A8d, W8d, sAd * 4, sBd, None)
    assert torch.equal(C1.float(), C0.float() * 4)


def test_c5_int8_exact(eng):
    M, N, K = 16384, 8192, 8192
    A, B = o.workloads.c5_int8(M, N, K)
    Ad, Bd = A.to(DEV), B.to(DEV)
    C = eng.gemm_s8(Ad, Bd)
    assert torch.equal(C, eng.naive(o.KIND_S8, Ad, Bd))
    rows = sample_idx(M, 24, 7)
    cols = sample_idx(N, 24, 8)
    assert np.array_equal(C[rows.to(DEV)].cpu().numpy(), oracle.gemm_s8s8_s32(A[rows].numpy(), B.numpy()))
    assert np.array_equal(C[:, cols.to(DEV)].cpu().numpy(),
                          oracle.gemm_s8s8_s32(A.numpy(), B[cols].numpy()))
    # checksum of checksums, exact in float64 (|sum| < 2^53): column sums of C against
    # (column sums of A) . B^T, row sums against A . (column sums of B)
    col_sums = C.sum(dim=0, dtype=torch.int64).cpu().numpy()
    a_sum = A.to(torch.float64).sum(dim=0).numpy()
    exp_cols = np.concatenate([B[i:i + 1024].to(torch.float64).numpy() @ a_sum for i in range(0, N, 1024)])
    assert np.array_equal(col_sums.astype(np.float64), exp_cols)
    row_sums = C.sum(dim=1, dtype=torch.int64).cpu().numpy()
    b_sum = B.to(torch.float64).sum(dim=0).numpy()
    exp_rows = np.concatenate([A[i:i + 1024].to(torch.float64).numpy() @ b_sum for i in range(0, M, 1024)])
    assert np.array_equal(row_sums.astype(np.float64), exp_rows)


def test_int8_operand_and_result_beyond_4_gib(eng):
    """Offsets that do not fit 32 bits: A is 4.6 GB, the int32 result 4.5 GB; rows at the far end of both
    against the oracle (bit exact), and a checksum of checksums over the whole result."""
    M, N, K = 140000, 8064, 32768          # M*K = 4.59e9 bytes, M*N*4 = 4.52e9 bytes
    g = torch.Generator(device=DEV).manual_seed(77)
    A = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=DEV, generator=g)
    B = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=DEV, generator=g)
    C = torch.full((M, N), -7, dtype=torch.int32, device=DEV)
    eng.gemm_s8(A, B, out=C)
    torch.cuda.synchronize()
    rows = torch.tensor([0, 1, 65535, 65536, 131071, 131072, M - 257, M - 2, M - 1])
    ref = oracle.gemm_s8s8_s32(A[rows.to(DEV)].cpu().numpy(), B.cpu().numpy())
    assert np.array_equal(C[rows.to(DEV)].cpu().numpy(), ref)
    # sum over all of C = (column sums of A) . (column sums of B), in exact integer arithmetic
    sa = A.sum(dim=0, dtype=torch.int64)
    sb = B.sum(dim=0, dtype=torch.int64)
    assert int(C.sum(dtype=torch.int64).item()) == int((sa * sb).sum().item())
    st, detail = eng.last_status()
    assert st == 0
