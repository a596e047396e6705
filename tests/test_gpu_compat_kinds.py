"""GPU: the runtime's MATMUL family beyond REAL*4 — REAL*8, every pair of integer kinds, and the
mixed pairs with a REAL result (REAL*4 x REAL*8, integer x real).
The strided kernels (_sgemmx__, _sgemvx__, _i1gemmx__ ... _jgemmx__: osprey/libfi/matrix/sgemmx.f,
sgemvx.f and the integer instances of the template xgemmx.h), the BLAS hook dgemm_ and the
operator entry points _MATMUL_SS, _MATMUL_I1I1 ... _MATMUL_JJ, against the CPU restatement.
Integer results are bit-exact including wrap-around in the result kind; REAL*8 within 1e-12 of
the largest magnitude."""
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
DT = {"s": np.float64, "s4": np.float32, "i1": np.int8, "i2": np.int16, "i4": np.int32, "j": np.int64}
INTS = ["i1", "i2", "i4", "j"]
ORDER = INTS + ["s4", "s"]      # the later kind of a pair is the kind of the result
# kernel name -> (kind of A, kind of B and C)
KERNELS = {"s": ("s", "s"), "s4s": ("s4", "s")}
for _i, _a in enumerate(INTS):
    for _c in INTS[_i:]:
        KERNELS[_a if _a == _c else _a + _c] = (_a, _c)
    KERNELS[_a + "s4"] = (_a, "s4")
    KERNELS[_a + "s"] = (_a, "s")


def _rand(kind, rng, size, overflow=True):
    dt = DT[kind]
    if kind in ("s", "s4"):
        return rng.standard_normal(size).astype(dt)
    info = np.iinfo(dt)
    if not overflow:
        return rng.integers(-11, 11, size, dtype=dt)
    return rng.integers(info.min // 3, info.max // 3, size, dtype=dt)


def _same(kind, got, want):
    if kind == "s":
        return relmax(got, want) <= TOL_F64
    if kind == "s4":
        return relmax(got, want) <= 1e-4
    return np.array_equal(got, want)


@pytest.mark.parametrize("kernel", list(KERNELS))
@pytest.mark.parametrize("shape", [(1, 1, 1), (19, 13, 17), (64, 64, 64), (130, 70, 33), (257, 129, 200)])
def test_xgemmx_kinds_match_oracle(eng, kernel, shape):
    ka, kc = KERNELS[kernel]
    m, n, k = shape
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    a, b, c0 = _rand(ka, rng, m * k), _rand(kc, rng, k * n), _rand(kc, rng, m * n)
    b[::7] = 0
    scal = ((1, 0), (3, 1), (-2, 5)) if kc in INTS else ((1.0, 0.0), (0.5, 1.0), (-2.0, 0.25))
    for alpha, beta in scal:
        cref = oracle.xgemmx(m, n, k, alpha, a, 1, m, b, 1, k, beta, c0.copy(), 1, m)
        for where in ("host", "device"):
            ta, tb, tc = (torch.from_numpy(v.copy()) for v in (a, b, c0))
            if where == "device":
                ta, tb, tc = ta.to(DEV), tb.to(DEV), tc.to(DEV)
            eng.xgemmx(kernel, m, n, k, alpha, ta, 1, m, tb, 1, k, beta, tc, 1, m)
            assert _same(kc, tc.cpu().numpy(), cref), (where, alpha, beta)


@pytest.mark.parametrize("kernel", ["s", "i1", "i1i4", "i2j", "i4", "j", "s4s", "i2s4", "js"])
def test_xgemmx_kinds_strided_sections(eng, kernel):
    """A(1:2m:2, :) through inc1a = 2, B stored transposed, C row-major."""
    ka, kc = KERNELS[kernel]
    rng = np.random.default_rng(5)
    m, n, k = 45, 37, 29
    a, b, c0 = _rand(ka, rng, 2 * m * k), _rand(kc, rng, k * n), _rand(kc, rng, m * n)
    one, zero = (1, 0) if kc in INTS else (1.0, 0.0)
    cref = oracle.xgemmx(m, n, k, one, a, 2, 2 * m, b, n, 1, zero, c0.copy(), n, 1)
    tc = torch.from_numpy(c0.copy())
    eng.xgemmx(kernel, m, n, k, one, torch.from_numpy(a), 2, 2 * m, torch.from_numpy(b), n, 1, zero, tc, n, 1)
    assert _same(kc, tc.numpy(), cref)


@pytest.mark.parametrize("kernel", ["s", "i1", "i2", "i4", "j", "i1i4"])
def test_xgemmx_kinds_quick_returns(eng, kernel):
    ka, kc = KERNELS[kernel]
    rng = np.random.default_rng(6)
    m, n, k = 5, 4, 3
    a = torch.from_numpy(_rand(ka, rng, m * k, overflow=False))
    b, c0 = (torch.from_numpy(_rand(kc, rng, s, overflow=False)) for s in (k * n, m * n))
    c = c0.clone()
    eng.xgemmx(kernel, m, n, k, 0, a, 1, m, b, 1, k, 1, c, 1, m)
    assert torch.equal(c, c0)                                  # alpha = 0, beta = 1: untouched
    c = c0.clone()
    eng.xgemmx(kernel, m, n, 0, 1, a, 1, m, b, 1, k, 3, c, 1, m)
    assert not c.any()                                         # K = 0: zeroed
    c = c0.clone()
    eng.xgemmx(kernel, m, n, k, 0, a, 1, m, b, 1, k, 2, c, 1, m)
    assert torch.equal(c, 2 * c0)                              # alpha = 0: scaled
    eng.xgemmx(kernel, 0, n, k, 1, a, 1, m, b, 1, k, 0, c, 1, m)
    assert eng.lib.o64_compat_last_status() == o.OK            # empty extent: nothing to do
    with pytest.raises(o.O64Error) as e:
        eng.xgemmx(kernel, -1, n, k, 1, a, 1, m, b, 1, k, 0, c, 1, m)
    assert e.value.status == o.ERR_RANK
    if kernel == "s":
        c = torch.full((m * n,), float("nan"), dtype=torch.float64)
        a2, b2 = a.clone(), b.clone()
        a2[0 + 1 * m] = float("inf")
        b2[1::k] = 0.0
        eng.xgemmx(kernel, m, n, k, 1.0, a2, 1, m, b2, 1, k, 0.0, c, 1, m)
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
    tc = torch.from_numpy(np.asfortranarray(C0).ravel(order="F").copy())
    eng.dgemm(ta, tb, m, n, k, 1.25, torch.from_numpy(a.ravel(order="F").copy()), a.shape[0],
              torch.from_numpy(b.ravel(order="F").copy()), b.shape[0], -0.5, tc, m)
    want = 1.25 * (A @ B) - 0.5 * C0
    assert relmax(tc.numpy().reshape(n, m).T, want) <= TOL_F64


def _entry(ka, kb):
    """(_MATMUL_<A><B>, result kind) for operand kinds ka, kb."""
    up = {"s": "S", "s4": "S4", "i1": "I1", "i2": "I2", "i4": "I4", "j": "J"}
    kc = ORDER[max(ORDER.index(ka), ORDER.index(kb))]
    return "_MATMUL_" + up[ka] + up[kb], kc


def _dv(kind, arr, extents, strides, assoc=True):
    code = DopeVector.TYPE_REAL if kind in ("s", "s4") else DopeVector.TYPE_INTEGER
    return DopeVector.make(arr.ctypes.data if arr is not None else None, extents, strides,
                           8 * np.dtype(DT[kind]).itemsize, code, assoc)


def _ref_product(ka, kb, kc, a, b, m, n, k):
    """The product through the oracle kernel the entry point of (ka, kb) calls: directly, or as
    C' = B'A' when MATRIX_A is the wider kind."""
    c = np.zeros(m * n, DT[kc])
    one, zero = (1, 0) if kc in INTS else (1.0, 0.0)
    if ORDER.index(ka) <= ORDER.index(kb):
        return oracle.xgemmx(m, n, k, one, a, 1, m, b, 1, k, zero, c, 1, m)
    return oracle.xgemmx(n, m, k, one, b, k, 1, a, m, 1, zero, c, m, 1)


PAIRS = ([("s", "s"), ("s4", "s"), ("s", "s4")] + [(x, y) for x in INTS for y in INTS] +
         [p for x in INTS for p in ((x, "s4"), ("s4", x), (x, "s"), ("s", x))])


@pytest.mark.parametrize("ka,kb", PAIRS)
def test_matmul_entry_points(eng, ka, kb):
    name, kc = _entry(ka, kb)
    fn = getattr(eng.lib, name)
    rng = np.random.default_rng(9)
    m, k, n = 37, 29, 41
    a, b = _rand(ka, rng, m * k), _rand(kb, rng, k * n)
    # matrix x matrix, column-major
    c = np.zeros(m * n, DT[kc])
    fn(ctypes.byref(_dv(kc, c, (m, n), (1, m))), ctypes.byref(_dv(ka, a, (m, k), (1, m))),
       ctypes.byref(_dv(kb, b, (k, n), (1, k))))
    assert eng.lib.o64_compat_last_status() == o.OK
    ref = _ref_product(ka, kb, kc, a, b, m, n, k)
    assert _same(kc, c, ref)
    if kc in INTS:   # independent check of the wrap-around in the result kind
        with np.errstate(over="ignore"):
            want = (a.reshape(k, m).T.astype(DT[kc]) @ b.reshape(n, k).T.astype(DT[kc])).astype(DT[kc])
        assert np.array_equal(c.reshape(n, m).T, want)
    # matrix x vector and vector x matrix
    x = b[:k].copy()
    y = np.zeros(m, DT[kc])
    fn(ctypes.byref(_dv(kc, y, (m,), (1,))), ctypes.byref(_dv(ka, a, (m, k), (1, m))),
       ctypes.byref(_dv(kb, x, (k,), (1,))))
    assert eng.lib.o64_compat_last_status() == o.OK
    assert _same(kc, y, _ref_product(ka, kb, kc, a, x, m, 1, k))
    xv = a[:k].copy()
    y2 = np.zeros(n, DT[kc])
    fn(ctypes.byref(_dv(kc, y2, (n,), (1,))), ctypes.byref(_dv(ka, xv, (k,), (1,))),
       ctypes.byref(_dv(kb, b, (k, n), (1, k))))
    assert eng.lib.o64_compat_last_status() == o.OK
    assert _same(kc, y2, _ref_product(ka, kb, kc, xv, b, 1, n, k))
    # a RESULT that is not associated is allocated by the runtime and handed to the caller
    R = _dv(kc, None, (0, 0), (0, 0), assoc=False)
    R.flags1 = 2 << 29
    fn(ctypes.byref(R), ctypes.byref(_dv(ka, a, (m, k), (1, m))), ctypes.byref(_dv(kb, b, (k, n), (1, k))))
    assert eng.lib.o64_compat_last_status() == o.OK and R.ptr and (R.flags0 & 1)
    assert R.dimension[0].extent == m and R.dimension[1].extent == n
    assert R.orig_size == m * n * 8 * np.dtype(DT[kc]).itemsize
    got = np.ctypeslib.as_array(ctypes.cast(R.ptr, ctypes.POINTER(np.ctypeslib.as_ctypes_type(DT[kc]))), (m * n,))
    assert _same(kc, got.copy(), ref)
    ctypes.CDLL(None).free(ctypes.c_void_p(R.ptr))
    # extents that do not conform
    fn(ctypes.byref(_dv(kc, c, (m, n), (1, m))), ctypes.byref(_dv(ka, a, (m, k), (1, m))),
       ctypes.byref(_dv(kb, b, (k + 1, n), (1, k + 1))))
    assert eng.lib.o64_compat_last_status() == o.ERR_CONFORM


@pytest.mark.parametrize("shape", [(200, 136, 96), (70, 66, 94), (64, 64, 16), (2, 2, 2), (130, 258, 1030)])
@pytest.mark.parametrize("layout", ["column-major", "row-major", "row-major, A transposed", "row-major, B transposed",
                                    "row-major, both transposed", "column-major, both transposed"])
def test_real8_dense_path_and_its_exceptions(eng, layout, shape):
    """REAL*8 on plainly laid out operands runs a blocked kernel of its own; the rule of the runtime's
    template that a zero factor of B leaves its term out (osprey/libfi/matrix/xgemmx.h:227) still holds when
    A carries an infinity: the result is what the general kernel gives."""
    import torch
    dev = torch.device("cuda", eng.device)
    M, N, K = shape
    g = torch.Generator().manual_seed(123)
    a = torch.rand((M, K), generator=g, dtype=torch.float64) - 0.5      # mathematical A(i,l)
    b = torch.rand((K, N), generator=g, dtype=torch.float64) - 0.5
    c0 = torch.rand((M, N), generator=g, dtype=torch.float64)

    def run(a_math, b_math):
        if layout == "column-major":       # X(i,j) at i + ld*j: the transposed matrix stored row-major
            A, B, C = a_math.t().contiguous().to(dev), b_math.t().contiguous().to(dev), c0.t().contiguous().to(dev)
            eng.xgemmx("s", M, N, K, 1.5, A, 1, M, B, 1, K, 0.5, C, 1, M)
            return C.t().cpu()
        if layout == "column-major, both transposed":   # A held as its transpose [M][K] rows contiguous, B likewise
            A, B, C = a_math.contiguous().to(dev), b_math.contiguous().to(dev), c0.t().contiguous().to(dev)
            eng.xgemmx("s", M, N, K, 1.5, A, K, 1, B, N, 1, 0.5, C, 1, M)
            return C.t().cpu()
        C = c0.clone().to(dev)
        ta, tb = "A transposed" in layout or "both" in layout, "B transposed" in layout or "both" in layout
        A = (a_math.t().contiguous() if ta else a_math.contiguous()).to(dev)     # [K][M] when transposed
        B = (b_math.t().contiguous() if tb else b_math.contiguous()).to(dev)     # [N][K] when transposed
        a1, a2 = (1, M) if ta else (K, 1)
        b1, b2 = (1, K) if tb else (N, 1)
        eng.xgemmx("s", M, N, K, 1.5, A, a1, a2, B, b1, b2, 0.5, C, N, 1)
        return C.cpu()

    want = 1.5 * (a @ b) + 0.5 * c0
    got = run(a, b)
    assert ((got - want).abs().max() / want.abs().max()).item() <= 1e-12
    # an infinity in A whose partner in B is zero: the term is left out, the row stays finite
    a2, b2 = a.clone(), b.clone()
    a2[M // 3, K // 2] = float("inf")
    b2[K // 2, :] = 0.0
    got2 = run(a2, b2)
    a_fin = a2.clone()
    a_fin[M // 3, K // 2] = 0.0
    want2 = 1.5 * (a_fin @ b2) + 0.5 * c0
    assert torch.isfinite(got2).all()
    assert ((got2 - want2).abs().max() / want2.abs().max()).item() <= 1e-12
