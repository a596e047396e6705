"""GPU: the Fortran-ABI compat entry points (sgemm_, _s4gemmx__, _s4gemvx__) against the CPU
restatement of the reference runtime's kernels, and the error conventions of the C ABI."""
import ctypes

import numpy as np
import pytest
import torch

import open64_b200 as o
import oracle
from util import TOL_F32, relmax

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_xgemmx_golden_strided_transposed(eng, golden):
    m, n, k = (int(v) for v in golden["x_mnk"])
    alpha, beta = (float(v) for v in golden["x_alpha_beta"])
    a, b = torch.from_numpy(golden["x_a"]), torch.from_numpy(golden["x_b"])
    for where in ("host", "device"):
        c = torch.from_numpy(golden["x_c"].copy())
        if where == "device":
            a, b, c = a.to(DEV), b.to(DEV), c.to(DEV)
        eng.s4gemmx(m, n, k, alpha, a, 1, m, b, 1, k, beta, c, n, 1)
        assert relmax(c.cpu().numpy().reshape(m, n), golden["x_C"]) <= TOL_F32
    y = torch.from_numpy(golden["v_y"].copy())
    eng.s4gemvx(m, k, 0.75, torch.from_numpy(golden["x_a"]), 1, m, torch.from_numpy(golden["v_x"]), 1,
                2.0, y, 1)
    assert relmax(y.numpy(), golden["v_Y"]) <= TOL_F32


@pytest.mark.parametrize("shape", [(1, 1, 1), (19, 13, 17), (64, 64, 64), (130, 70, 33), (300, 200, 150)])
def test_xgemmx_matches_oracle(eng, shape):
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal(m * k).astype(np.float32)
    b = rng.standard_normal(k * n).astype(np.float32)
    c0 = rng.standard_normal(m * n).astype(np.float32)
    for (alpha, beta) in ((1.0, 0.0), (0.5, 1.0), (-2.0, 0.25)):
        cref = c0.copy()
        oracle.s4gemmx(m, n, k, alpha, a, 1, m, b, 1, k, beta, cref, 1, m)
        c = torch.from_numpy(c0.copy())
        eng.s4gemmx(m, n, k, alpha, torch.from_numpy(a), 1, m, torch.from_numpy(b), 1, k, beta, c, 1, m)
        assert relmax(c.numpy(), cref) <= TOL_F32


def test_xgemmx_quick_returns_and_zero_skip(eng):
    rng = np.random.default_rng(3)
    m, n, k = 5, 4, 3
    a = torch.from_numpy(rng.standard_normal(m * k).astype(np.float32))
    b = torch.from_numpy(rng.standard_normal(k * n).astype(np.float32))
    c0 = torch.from_numpy(rng.standard_normal(m * n).astype(np.float32))
    c = c0.clone()
    eng.s4gemmx(m, n, k, 0.0, a, 1, m, b, 1, k, 1.0, c, 1, m)
    assert torch.equal(c, c0)                                  # alpha = 0, beta = 1: untouched
    c = c0.clone()
    eng.s4gemmx(m, n, 0, 1.0, a, 1, m, b, 1, k, 3.0, c, 1, m)
    assert not c.any()                                         # K = 0: zeroed
    c = c0.clone()
    eng.s4gemmx(m, n, k, 0.0, a, 1, m, b, 1, k, 2.0, c, 1, m)
    assert torch.allclose(c, 2.0 * c0)                         # alpha = 0: scaled
    c = torch.full((m * n,), float("nan"))
    eng.s4gemmx(m, n, k, 1.0, a, 1, m, b, 1, k, 0.0, c, 1, m)
    assert torch.isfinite(c).all()                             # beta = 0: C is not read
    a2, b2 = a.clone(), b.clone()
    a2[0 + 1 * m] = float("inf")
    b2[1::k] = 0.0
    c = torch.zeros(m * n)
    eng.s4gemmx(m, n, k, 1.0, a2, 1, m, b2, 1, k, 0.0, c, 1, m)
    assert torch.isfinite(c).all()                             # zero B(l,j) skips the term
    y = c0[:m].clone()
    eng.s4gemvx(m, 0, 1.0, a, 1, m, b, 1, 5.0, y, 1)
    assert not y.any()                                         # empty sum zeroes y


@pytest.mark.parametrize("ta,tb", [("n", "n"), ("t", "n"), ("n", "t"), ("T", "T")])
def test_sgemm_blas_hook(eng, ta, tb):
    m, n, k = 37, 29, 41
    rng = np.random.default_rng(7)
    A = rng.standard_normal((m, k))
    B = rng.standard_normal((k, n))
    C0 = rng.standard_normal((m, n))
    # column-major storage of op-ed operands
    a = np.asfortranarray(A if ta in "nN" else A.T).astype(np.float32)
    b = np.asfortranarray(B if tb in "nN" else B.T).astype(np.float32)
    c = np.asfortranarray(C0).astype(np.float32)
    at = torch.from_numpy(a.ravel(order="F").copy())
    bt = torch.from_numpy(b.ravel(order="F").copy())
    ct = torch.from_numpy(c.ravel(order="F").copy())
    eng.sgemm(ta, tb, m, n, k, 1.5, at, a.shape[0], bt, b.shape[0], -0.5, ct, m)
    ref = 1.5 * A.astype(np.float32).astype(np.float64) @ B.astype(np.float32).astype(np.float64) \
        - 0.5 * C0.astype(np.float32).astype(np.float64)
    assert relmax(ct.numpy().reshape(n, m).T, ref) <= TOL_F32


def test_sgemm_as_called_by_the_matmul_runtime(eng):
    """('n','n',m,n,k,1,A,m,B,k,0,R,m) on contiguous column-major operands: the dot-product
    form the hook replaces."""
    m, n, k = 48, 40, 56
    rng = np.random.default_rng(9)
    a = rng.standard_normal(m * k).astype(np.float32)
    b = rng.standard_normal(k * n).astype(np.float32)
    r = torch.full((m * n,), float("nan"))
    eng.sgemm("n", "n", m, n, k, 1.0, torch.from_numpy(a), m, torch.from_numpy(b), k, 0.0, r, m)
    ref = oracle.internal_mm_f32(a, b, m, n, k)
    assert relmax(r.numpy(), ref) <= TOL_F32


def test_gemv_row_and_column_major(eng):
    m, n = 5000, 70
    rng = np.random.default_rng(11)
    a = rng.standard_normal(m * n).astype(np.float32)
    x = rng.standard_normal(n).astype(np.float32)
    x[3] = 0.0
    y0 = rng.standard_normal(m).astype(np.float32)
    for (inc1, inc2) in ((1, m), (n, 1)):
        yref = y0.copy()
        oracle.s4gemvx(m, n, 1.25, a, inc1, inc2, x, 1, 0.5, yref, 1)
        y = torch.from_numpy(y0.copy())
        eng.s4gemvx(m, n, 1.25, torch.from_numpy(a), inc1, inc2, torch.from_numpy(x), 1, 0.5, y, 1)
        assert relmax(y.numpy(), yref) <= TOL_F32


def test_error_codes(eng):
    lib, h = eng.lib, eng._h
    A = torch.zeros(128, 64, dtype=torch.bfloat16, device=DEV)
    B = torch.zeros(256, 64, dtype=torch.bfloat16, device=DEV)
    C = torch.zeros(128, 256, dtype=torch.bfloat16, device=DEV)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    f = lib.o64_gemm_bf16
    assert f(h, 128, 256, 64, p(A), 64, p(B), 64, 1, p(C), 256, None, None) == o.OK
    assert f(h, -1, 256, 64, p(A), 64, p(B), 64, 1, p(C), 256, None, None) == o.ERR_RANK
    assert f(h, 128, 256, 64, None, 64, p(B), 64, 1, p(C), 256, None, None) == o.ERR_RANK
    assert f(h, 128, 256, 64, p(A), 32, p(B), 64, 1, p(C), 256, None, None) == o.ERR_CONFORM   # lda < K
    assert f(h, 128, 256, 64, p(A), 64, p(B), 64, 1, p(C), 100, None, None) == o.ERR_CONFORM   # ldc < N
    # operands TMA cannot address directly (120-byte pitch, base off by 2 bytes) are repacked
    assert f(h, 128, 256, 60, p(A), 60, p(B), 60, 1, p(C), 256, None, None) == o.OK
    assert f(h, 128, 256, 56, ctypes.c_void_p(A.data_ptr() + 2), 64, p(B), 64, 1, p(C), 256, None,
             None) == o.OK
    assert f(h, 0, 256, 64, p(A), 64, p(B), 64, 1, p(C), 256, None, None) == o.OK               # empty
    epi = o._lib.Epilogue(None, 99)
    assert f(h, 128, 256, 64, p(A), 64, p(B), 64, 1, p(C), 256, ctypes.byref(epi), None) == o.ERR_RANK
    with pytest.raises(o.O64Error) as e:
        eng.gemm_bf16(A, torch.zeros(256, 32, dtype=torch.bfloat16, device=DEV))
    assert e.value.status == o.ERR_CONFORM
    with pytest.raises(o.O64Error):
        eng.plan_set(o.KIND_BF16, tile_n=192)
    # sharded call without a communicator on one rank degenerates to the plain GEMM
    assert lib.o64_gemm_s8_sharded(h, 8, 12, 16, p(A), 16, p(B), 16, None, 1, None, None) == o.ERR_RANK
    st, detail = eng.last_status()
    assert st == o.OK and detail == 0


def test_plan_query(eng):
    p = eng.plan_get(o.KIND_BF16, 8192, 8192, 8192)
    assert p["tile_m"] in (128, 256, 512) and p["tile_n"] in (128, 256) and p["num_ctas"] <= 148
    p = eng.plan_get(o.KIND_F32, 512, 512, 512)
    assert p["tile_m"] in (32, 64)
