"""CPU: the oracle against the committed golden vectors and against independent numpy math."""
import numpy as np
import pytest

import oracle
from util import relmax


def test_codecs_known_answers(golden):
    dec = oracle.e4m3_to_f32(np.arange(256, dtype=np.uint8))
    exp = golden["e4m3_decode"]
    assert np.array_equal(np.isnan(dec), np.isnan(exp))
    assert np.array_equal(dec[~np.isnan(exp)], exp[~np.isnan(exp)])
    assert np.array_equal(oracle.f32_to_e4m3(golden["e4m3_probe"]), golden["e4m3_encode"])
    assert np.array_equal(oracle.f32_to_bf16(golden["bf16_probe"]), golden["bf16_encode"])
    # round trip of every finite e4m3 code
    fin = ~np.isnan(exp)
    assert np.array_equal(oracle.f32_to_e4m3(exp[fin]) & 0x7f, np.arange(256, dtype=np.uint8)[fin] & 0x7f)


def test_c1_linear_golden(golden):
    y = oracle.linear_f32(golden["c1_A"], golden["c1_B"], golden["c1_bias"], oracle.ACT_RELU)
    assert relmax(y, golden["c1_Y"]) < 1e-6
    y64 = oracle.linear_f32_acc64(golden["c1_A"], golden["c1_B"], golden["c1_bias"], oracle.ACT_RELU)
    assert relmax(y64, golden["c1_Y"]) < 2e-7


def test_c2_bf16_golden(golden):
    c = oracle.gemm_bf16(golden["c2_A"], golden["c2_B"], transB=True)
    assert relmax(c, golden["c2_C"]) < 1e-6
    # the [K,N] form gives the same numbers
    Bkn = np.ascontiguousarray(golden["c2_B"].T)
    assert np.array_equal(oracle.gemm_bf16(golden["c2_A"], Bkn, transB=False), c)


def test_c3_swiglu_golden(golden):
    h = oracle.bf16_to_f32(oracle.swiglu_bf16(golden["c3_X"], golden["c3_Wg"], golden["c3_Wu"]))
    assert relmax(h, golden["c3_H"]) < 4e-3  # one bf16 rounding


def test_c4_fp8_golden(golden):
    c = oracle.gemm_fp8_scaled(golden["c4_A8"], golden["c4_B8"], golden["c4_sA"], golden["c4_sB"],
                               golden["c4_bias"])
    assert relmax(c, golden["c4_C"]) < 1e-6


def test_c5_int8_golden(golden):
    assert np.array_equal(oracle.gemm_s8s8_s32(golden["c5_A"], golden["c5_B"]), golden["c5_C"])


def test_xgemmx_golden(golden):
    m, n, k = (int(v) for v in golden["x_mnk"])
    alpha, beta = (float(v) for v in golden["x_alpha_beta"])
    c = golden["x_c"].copy()
    oracle.s4gemmx(m, n, k, alpha, golden["x_a"], 1, m, golden["x_b"], 1, k, beta, c, n, 1)
    assert relmax(c.reshape(m, n), golden["x_C"]) < 1e-6
    y = golden["v_y"].copy()
    oracle.s4gemvx(m, k, 0.75, golden["x_a"], 1, m, golden["v_x"], 1, 2.0, y, 1)
    assert relmax(y, golden["v_Y"]) < 1e-6


def test_xgemmx_quick_returns_and_zero_skip():
    rng = np.random.default_rng(3)
    m, n, k = 5, 4, 3
    a = rng.standard_normal(m * k).astype(np.float32)
    b = rng.standard_normal(k * n).astype(np.float32)
    c0 = rng.standard_normal(m * n).astype(np.float32)
    # alpha == 0 and beta == 1: untouched
    c = c0.copy()
    oracle.s4gemmx(m, n, k, 0.0, a, 1, m, b, 1, k, 1.0, c, 1, m)
    assert np.array_equal(c, c0)
    # K == 0: zeroed whatever beta is
    c = c0.copy()
    oracle.s4gemmx(m, n, 0, 1.0, a, 1, m, b, 1, k, 3.0, c, 1, m)
    assert not c.any()
    # alpha == 0: scaled by beta
    c = c0.copy()
    oracle.s4gemmx(m, n, k, 0.0, a, 1, m, b, 1, k, 2.0, c, 1, m)
    assert np.allclose(c, 2.0 * c0)
    # beta == 0: C is not read (NaN does not propagate)
    c = np.full(m * n, np.nan, np.float32)
    oracle.s4gemmx(m, n, k, 1.0, a, 1, m, b, 1, k, 0.0, c, 1, m)
    ref = a.reshape(k, m).T.astype(np.float64) @ b.reshape(n, k).T.astype(np.float64)
    assert relmax(c.reshape(n, m).T, ref) < 1e-6
    # a zero in B skips the axpy: an infinity in the matching column of A stays out
    a2 = a.copy()
    a2[0 + 1 * m] = np.inf          # A(0, l=1)
    b2 = b.copy()
    b2[1::k] = 0.0                  # B(l=1, j) = 0 for every j
    c = np.zeros(m * n, np.float32)
    oracle.s4gemmx(m, n, k, 1.0, a2, 1, m, b2, 1, k, 0.0, c, 1, m)
    assert np.isfinite(c).all()
    # the matrix-vector sibling: N == 0 zeroes y, x(j) == 0 skips
    y = c0[:m].copy()
    oracle.s4gemvx(m, 0, 1.0, a, 1, m, b, 1, 5.0, y, 1)
    assert not y.any()


def test_internal_mm_matches_strided_kernel():
    rng = np.random.default_rng(4)
    m, n, k = 9, 7, 11
    a = rng.standard_normal(m * k).astype(np.float32)
    b = rng.standard_normal(k * n).astype(np.float32)
    r = oracle.internal_mm_f32(a, b, m, n, k)
    c = np.zeros(m * n, np.float32)
    oracle.s4gemmx(m, n, k, 1.0, a, 1, m, b, 1, k, 0.0, c, 1, m)
    assert relmax(r, c) < 1e-6


@pytest.mark.parametrize("act", [oracle.ACT_NONE, oracle.ACT_RELU, oracle.ACT_GELU_TANH,
                                 oracle.ACT_GELU_ERF, oracle.ACT_SILU])
def test_activations_against_numpy(act):
    import math
    rng = np.random.default_rng(5)
    A = rng.standard_normal((6, 8)).astype(np.float32)
    B = rng.standard_normal((8, 5)).astype(np.float32)
    x = A.astype(np.float64) @ B.astype(np.float64)
    ref = {
        oracle.ACT_NONE: x,
        oracle.ACT_RELU: np.maximum(x, 0),
        oracle.ACT_GELU_TANH: 0.5 * x * (1 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3))),
        oracle.ACT_GELU_ERF: 0.5 * x * (1 + np.vectorize(math.erf)(x / math.sqrt(2))),
        oracle.ACT_SILU: x / (1 + np.exp(-x)),
    }[act]
    assert relmax(oracle.linear_f32(A, B, None, act), ref) < 1e-5


def test_reassociation_spread_is_far_inside_tolerance():
    """How far a legal re-association (fp64 accumulate as the extreme) moves the fp32 answer at
    the C1 size: orders of magnitude inside the 1e-4 gate."""
    import open64_b200 as o
    A, B, bias = o.workloads.c1_linear_f32()
    y = oracle.linear_f32(A.numpy(), B.numpy(), bias.numpy(), oracle.ACT_RELU)
    y64 = oracle.linear_f32_acc64(A.numpy(), B.numpy(), bias.numpy(), oracle.ACT_RELU)
    assert relmax(y, y64) < 1e-5


_INTS = (np.int8, np.int16, np.int32, np.int64)
PAIRS = ([(np.float64, np.float64), (np.float32, np.float64)] +
         [(a, c) for i, a in enumerate(_INTS) for c in _INTS[i:]] +
         [(a, c) for a in _INTS for c in (np.float32, np.float64)])


@pytest.mark.parametrize("ta,tc", PAIRS, ids=lambda t: np.dtype(t).name)
def test_xgemmx_other_kinds_against_numpy(ta, tc):
    """REAL*8 and the integer kinds of the strided kernel (A of kind ta; B, C of kind tc): numpy on
    the same strided views; integers with magnitudes that overflow, so the wrap-around in the kind
    of C is exercised."""
    rng = np.random.default_rng(11)
    m, n, k = 13, 9, 21
    real = tc in (np.float32, np.float64)
    if real:
        b, c0 = (rng.standard_normal(s).astype(tc) for s in (k * n, m * n))
        if ta in _INTS:
            a = rng.integers(-1000, 1000, m * k * 2, dtype=ta) if ta is not np.int8 else rng.integers(-128, 127, m * k * 2, dtype=ta)
        else:
            a = rng.standard_normal(m * k * 2).astype(ta)
        alpha, beta = 1.5, -0.5
    else:
        a = rng.integers(np.iinfo(ta).min, np.iinfo(ta).max, m * k * 2, dtype=ta, endpoint=True)
        big = np.iinfo(tc).max // 3
        b, c0 = (rng.integers(-big, big, s, dtype=tc) for s in (k * n, m * n))
        alpha, beta = 3, -7
    b[::5] = 0
    # A(i,l) at a[2*i + 2*m*l] (a section with stride 2), B transposed storage, C column-major
    c = oracle.xgemmx(m, n, k, alpha, a, 2, 2 * m, b, n, 1, beta, c0.copy(), 1, m)
    A = a[: 2 * m * k : 2].reshape(k, m).T.astype(tc)
    B = b.reshape(k, n)
    with np.errstate(over="ignore"):
        want = (tc(alpha) * (A @ B) + tc(beta) * c0.reshape(n, m).T).astype(tc)
    got = c.reshape(n, m).T
    if tc is np.float64:
        assert relmax(got, want) < 1e-14
    elif tc is np.float32:
        assert relmax(got, want) < 1e-5
    else:
        assert np.array_equal(got, want)


def test_sgemvx_f64_against_numpy():
    rng = np.random.default_rng(12)
    m, n = 17, 23
    a, x, y0 = rng.standard_normal(m * n), rng.standard_normal(n), rng.standard_normal(m)
    y = oracle.sgemvx_f64(m, n, 0.5, a, 1, m, x, 1, 2.0, y0.copy(), 1)
    assert relmax(y, 0.5 * (a.reshape(n, m).T @ x) + 2.0 * y0) < 1e-14


@pytest.mark.parametrize("dtype", [np.complex64, np.complex128])
def test_complex_kernels_against_numpy(dtype):
    rng = np.random.default_rng(21)
    m, n, k = 11, 7, 13
    cplx = lambda size: (rng.standard_normal(size) + 1j * rng.standard_normal(size)).astype(dtype)
    a, b, c0 = cplx(m * k), cplx(k * n), cplx(m * n)
    A, B, C0 = a.reshape(k, m).T, b.reshape(n, k).T, c0.reshape(n, m).T          # column-major views
    tol = 1e-5 if dtype is np.complex64 else 1e-13
    for conja, conjb in ((False, False), (True, False), (False, True), (True, True)):
        c = oracle.cgemmx(m, n, k, 0.5 - 2j, a, 1, m, b, 1, k, 1.5 + 0.25j, c0.copy(), 1, m, conja, conjb)
        want = (0.5 - 2j) * ((A.conj() if conja else A) @ (B.conj() if conjb else B)) + (1.5 + 0.25j) * C0
        assert np.abs(c.reshape(n, m).T - want).max() / np.abs(want).max() < tol
    assert not oracle.cgemmx(m, n, 0, 1.0, a, 1, m, b, 1, k, 3.0, c0.copy(), 1, m).any()   # K = 0: zeroed
    x, y0 = cplx(k), cplx(m)
    for conj in (False, True):
        y = oracle.cgemvx(m, k, 2.0 + 1j, a, 1, m, x, 1, -1j, y0.copy(), 1, conj)
        want = (2.0 + 1j) * ((A.conj() if conj else A) @ x) + (-1j) * y0
        assert np.abs(y - want).max() / np.abs(want).max() < tol


def test_logical_kernel_against_numpy():
    rng = np.random.default_rng(31)
    m, n, k = 9, 14, 22
    a = ((rng.random(m * k) < 0.1) * rng.integers(1, 50, m * k)).astype(np.int8)
    b = ((rng.random(k * n) < 0.1) * -rng.integers(1, 50, k * n)).astype(np.int32)
    c0 = (rng.random(m * n) < 0.3).astype(np.int32) * 5
    A, B, C0 = a.reshape(k, m).T != 0, b.reshape(n, k).T != 0, c0.reshape(n, m).T != 0
    prod = (A.astype(int) @ B.astype(int)) > 0
    for alpha, beta, want in ((1, 0, prod), (1, 1, prod | C0), (0, 0, np.zeros_like(prod))):
        c = oracle.lgemmx(m, n, k, alpha, a, 1, m, b, 1, k, beta, c0.copy(), 1, m)
        assert np.array_equal(c.reshape(n, m).T, want.astype(np.int32))
    assert np.array_equal(oracle.lgemmx(m, n, k, 0, a, 1, m, b, 1, k, 1, c0.copy(), 1, m), c0)   # untouched
    assert not oracle.lgemmx(m, n, 0, 1, a, 1, m, b, 1, k, 1, c0.copy(), 1, m).any()


@pytest.mark.parametrize("ka,kb", [("c4", "s4"), ("s4", "c4"), ("c4", "i1"), ("j", "c4"), ("c", "s4"), ("s", "c4"),
                                   ("c4", "c"), ("c", "c4"), ("c", "i2"), ("i4", "c"), ("c", "s"), ("s", "c")])
def test_complex_with_other_kinds_through_the_real_kernels(ka, kb):
    """MATMUL of a COMPLEX operand with a REAL / INTEGER / other-width COMPLEX one, formed as the
    entry points of osprey/libfi/matrix/matmul_c4s4.c, matmul_c4i1.c, matmul_c4c.c do: real and
    imaginary parts as separate products of the REAL kernel, increments of COMPLEX arrays doubled,
    C' = B'A' where MATRIX_A has the wider components.  The same sequence of kernel calls the GPU
    parity test replays, here against numpy's complex product."""
    import test_gpu_compat_complex_mixed as cm
    rng = np.random.default_rng(5)
    m, k, n = 13, 11, 17
    a, b = cm._rand(ka, rng, m * k), cm._rand(kb, rng, k * n)
    got = cm._ref_product(ka, kb, a, b, m, n, k, (1, m), (1, k))
    kc = cm._result_kind(ka, kb)
    assert got.dtype == cm.DT[kc]
    want = a.reshape(k, m).T.astype(np.complex128) @ b.reshape(n, k).T.astype(np.complex128)
    assert cm._close(kc, got.reshape(n, m).T, want)
