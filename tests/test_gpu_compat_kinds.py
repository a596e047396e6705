"""GPU: the runtime's MATMUL family for REAL*8, INTEGER*4 and INTEGER*8 — the strided kernels
(_sgemmx__, _sgemvx__, _i4gemmx__, _jgemmx__: osprey/libfi/matrix/sgemmx.f, sgemvx.f, i4gemmx.f,
jgemmx.f over the template xgemmx.h), the BLAS hook dgemm_ and the operator entry points
_MATMUL_SS / _MATMUL_I4I4 / _MATMUL_JJ — against the CPU restatement.  Integer results are
bit-exact including wrap-around; REAL*8 within 1e-12 of the largest magnitude."""
import ctypes

import numpy as np
import pytest
import torch

import open64_b200 as o
import oracle
from open64_b200._lib import DopeVector
from util import relmax

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL_F64 = 1e-12
KINDS = {"f64": np.float64, "i32": np.int32, "i64": np.int64}


def _operands(kind, rng, sizes, overflow=True):
    dt = KINDS[kind]
    if kind == "f64":
        return [rng.standard_normal(s) for s in sizes]
    hi = np.iinfo(dt).max // 3 if overflow else 1000
    return [rng.integers(-hi, hi, s, dtype=dt) for s in sizes]


def _same(kind, got, want):
    if kind == "f64":
        return relmax(got, want) <= TOL_F64
    return np.array_equal(got, want)


@pytest.mark.parametrize("kind", ["f64", "i32", "i64"])
@pytest.mark.parametrize("shape", [(1, 1, 1), (19, 13, 17), (64, 64, 64), (130, 70, 33), (257, 129, 200)])
def test_xgemmx_kinds_match_oracle(eng, kind, shape):
    m, n, k = shape
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    a, b, c0 = _operands(kind, rng, (m * k, k * n, m * n))
    b[::7] = 0
    scal = ((1, 0), (3, 1), (-2, 5)) if kind != "f64" else ((1.0, 0.0), (0.5, 1.0), (-2.0, 0.25))
    for alpha, beta in scal:
        cref = oracle.xgemmx(m, n, k, alpha, a, 1, m, b, 1, k, beta, c0.copy(), 1, m)
        for where in ("host", "device"):
            ta, tb, tc = (torch.from_numpy(v.copy()) for v in (a, b, c0))
            if where == "device":
                ta, tb, tc = ta.to(DEV), tb.to(DEV), tc.to(DEV)
            eng.xgemmx(kind, m, n, k, alpha, ta, 1, m, tb, 1, k, beta, tc, 1, m)
            assert _same(kind, tc.cpu().numpy(), cref), (where, alpha, beta)


@pytest.mark.parametrize("kind", ["f64", "i32", "i64"])
def test_xgemmx_kinds_strided_sections(eng, kind):
    """A(1:2m:2, :) through inc1a = 2, B stored transposed, C row-major."""
    rng = np.random.default_rng(5)
    m, n, k = 45, 37, 29
    a, b, c0 = _operands(kind, rng, (2 * m * k, k * n, m * n))
    one = 1 if kind != "f64" else 1.0
    zero = 0 if kind != "f64" else 0.0
    cref = oracle.xgemmx(m, n, k, one, a, 2, 2 * m, b, n, 1, zero, c0.copy(), n, 1)
    tc = torch.from_numpy(c0.copy())
    eng.xgemmx(kind, m, n, k, one, torch.from_numpy(a), 2, 2 * m, torch.from_numpy(b), n, 1, zero, tc, n, 1)
    assert _same(kind, tc.numpy(), cref)


@pytest.mark.parametrize("kind", ["f64", "i32", "i64"])
def test_xgemmx_kinds_quick_returns(eng, kind):
    rng = np.random.default_rng(6)
    m, n, k = 5, 4, 3
    a, b, c0 = (torch.from_numpy(v) for v in _operands(kind, rng, (m * k, k * n, m * n), overflow=False))
    c = c0.clone()
    eng.xgemmx(kind, m, n, k, 0, a, 1, m, b, 1, k, 1, c, 1, m)
    assert torch.equal(c, c0)                                  # alpha = 0, beta = 1: untouched
    c = c0.clone()
    eng.xgemmx(kind, m, n, 0, 1, a, 1, m, b, 1, k, 3, c, 1, m)
    assert not c.any()                                         # K = 0: zeroed
    c = c0.clone()
    eng.xgemmx(kind, m, n, k, 0, a, 1, m, b, 1, k, 2, c, 1, m)
    assert torch.equal(c, 2 * c0)                              # alpha = 0: scaled
    eng.xgemmx(kind, 0, n, k, 1, a, 1, m, b, 1, k, 0, c, 1, m)
    assert eng.lib.o64_compat_last_status() == o.OK            # empty extent: nothing to do
    with pytest.raises(o.O64Error) as e:
        eng.xgemmx(kind, -1, n, k, 1, a, 1, m, b, 1, k, 0, c, 1, m)
    assert e.value.status == o.ERR_RANK
    if kind == "f64":
        c = torch.full((m * n,), float("nan"), dtype=torch.float64)
        a2, b2 = a.clone(), b.clone()
        a2[0 + 1 * m] = float("inf")
        b2[1::k] = 0.0
        eng.xgemmx(kind, m, n, k, 1.0, a2, 1, m, b2, 1, k, 0.0, c, 1, m)
        assert torch.isfinite(c).all()                         # beta = 0 ignores C; zero B(l,j) skips


def test_sgemvx_f64(eng):
    rng = np.random.default_rng(7)
    for (m, n) in ((1, 1), (33, 45), (300, 129)):
        a, x, y0 = rng.standard_normal(m * n), rng.standard_normal(2 * n), rng.standard_normal(m)
        x[::6] = 0.0
        for alpha, beta in ((1.0, 0.0), (0.75, 2.0)):
            yref = oracle.sgemvx_f64(m, n, alpha, a, 1, m, x, 2, beta, y0.copy(), 1)
            y = torch.from_numpy(y0.copy())
            eng.sgemvx(m, n, alpha, torch.from_numpy(a), 1, m, torch.from_numpy(x), 2, beta, y, 1)
            assert relmax(y.numpy(), yref) <= TOL_F64
    y = torch.from_numpy(rng.standard_normal(4))
    eng.sgemvx(4, 0, 1.0, y, 1, 4, y, 1, 5.0, y, 1)
    assert not y.any()                                         # empty sum zeroes y


@pytest.mark.parametrize("ta", "nt")
@pytest.mark.parametrize("tb", "nt")
def test_dgemm_blas_hook(eng, ta, tb):
    rng = np.random.default_rng(8)
    m, n, k = 31, 23, 19
    A = rng.standard_normal((m, k))
    B = rng.standard_normal((k, n))
    C0 = rng.standard_normal((m, n))
    a = np.asfortranarray(A if ta == "n" else A.T)
    b = np.asfortranarray(B if tb == "n" else B.T)
    c = np.asfortranarray(C0.copy())
    tc = torch.from_numpy(c.ravel(order="F").copy())
    eng.dgemm(ta, tb, m, n, k, 1.25, torch.from_numpy(a.ravel(order="F").copy()), a.shape[0],
              torch.from_numpy(b.ravel(order="F").copy()), b.shape[0], -0.5, tc, m)
    want = 1.25 * (A @ B) - 0.5 * C0
    assert relmax(tc.numpy().reshape(n, m).T, want) <= TOL_F64


ENTRY = {"f64": ("_MATMUL_SS", 64, DopeVector.TYPE_REAL), "i32": ("_MATMUL_I4I4", 32, DopeVector.TYPE_INTEGER),
         "i64": ("_MATMUL_JJ", 64, DopeVector.TYPE_INTEGER)}


def _dv(kind, arr, extents, strides, assoc=True):
    _, bits, code = ENTRY[kind]
    return DopeVector.make(arr.ctypes.data if arr is not None else None, extents, strides, bits, code, assoc)


@pytest.mark.parametrize("kind", ["f64", "i32", "i64"])
def test_matmul_entry_points(eng, kind):
    fn = getattr(eng.lib, ENTRY[kind][0])
    dt = KINDS[kind]
    rng = np.random.default_rng(9)
    m, k, n = 37, 29, 41
    a, b = _operands(kind, rng, (m * k, k * n))
    one, zero = dt(1), dt(0)
    # matrix x matrix, column-major
    c = np.zeros(m * n, dt)
    fn(ctypes.byref(_dv(kind, c, (m, n), (1, m))), ctypes.byref(_dv(kind, a, (m, k), (1, m))),
       ctypes.byref(_dv(kind, b, (k, n), (1, k))))
    assert eng.lib.o64_compat_last_status() == o.OK
    ref = oracle.xgemmx(m, n, k, one, a, 1, m, b, 1, k, zero, np.zeros(m * n, dt), 1, m)
    assert _same(kind, c, ref)
    # matrix x vector and vector x matrix
    x = b[:k].copy()
    y = np.zeros(m, dt)
    fn(ctypes.byref(_dv(kind, y, (m,), (1,))), ctypes.byref(_dv(kind, a, (m, k), (1, m))),
       ctypes.byref(_dv(kind, x, (k,), (1,))))
    assert eng.lib.o64_compat_last_status() == o.OK
    assert _same(kind, y, oracle.xgemmx(m, 1, k, one, a, 1, m, x, 1, 1, zero, np.zeros(m, dt), 1, 1))
    xv = a[:m].copy()
    y2 = np.zeros(k, dt)
    fn(ctypes.byref(_dv(kind, y2, (k,), (1,))), ctypes.byref(_dv(kind, xv, (m,), (1,))),
       ctypes.byref(_dv(kind, a, (m, k), (1, m))))
    assert eng.lib.o64_compat_last_status() == o.OK
    assert _same(kind, y2, oracle.xgemmx(1, k, m, one, xv, 1, 1, a, 1, m, zero, np.zeros(k, dt), 1, 1))
    # a RESULT that is not associated is allocated by the runtime and handed to the caller
    R = _dv(kind, None, (0, 0), (0, 0), assoc=False)
    R.flags1 = 2 << 29
    fn(ctypes.byref(R), ctypes.byref(_dv(kind, a, (m, k), (1, m))), ctypes.byref(_dv(kind, b, (k, n), (1, k))))
    assert eng.lib.o64_compat_last_status() == o.OK and R.ptr and (R.flags0 & 1)
    assert R.dimension[0].extent == m and R.dimension[1].extent == n
    assert R.orig_size == m * n * ENTRY[kind][1]
    got = np.ctypeslib.as_array(ctypes.cast(R.ptr, ctypes.POINTER(np.ctypeslib.as_ctypes_type(dt))), (m * n,))
    assert _same(kind, got.copy(), ref)
    ctypes.CDLL(None).free(ctypes.c_void_p(R.ptr))
    # extents that do not conform
    fn(ctypes.byref(_dv(kind, c, (m, n), (1, m))), ctypes.byref(_dv(kind, a, (m, k), (1, m))),
       ctypes.byref(_dv(kind, b, (k + 1, n), (1, k + 1))))
    assert eng.lib.o64_compat_last_status() == o.ERR_CONFORM
