"""GPU: MATMUL of a COMPLEX operand with a REAL or INTEGER one, or with COMPLEX of the other width
— the 26 entry points _MATMUL_C4S4, _MATMUL_S4C4, _MATMUL_C4I1 ... _MATMUL_JC, _MATMUL_C4C and
_MATMUL_CC4 (osprey/libfi/matrix/matmul_c4s4.c, matmul_i1c4.c, matmul_c4c.c, ...).  The reference forms
the real and imaginary parts as separate products of the REAL kernel for the two component kinds,
with the increments of the COMPLEX arrays doubled, and as C' = B'A' where MATRIX_A has the wider
components; the check repeats exactly those calls on the CPU restatement, and compares with a
complex128 product as well."""
import ctypes

import numpy as np
import pytest

import open64_b200 as o
import oracle
from open64_b200._lib import DopeVector
from util import relmax

pytestmark = pytest.mark.gpu
INTS = ["i1", "i2", "i4", "j"]
ORDER = INTS + ["s4", "s"]
COMP = {"c4": "s4", "c": "s"}           # component kind of a COMPLEX kind
DT = {"s": np.float64, "s4": np.float32, "i1": np.int8, "i2": np.int16, "i4": np.int32, "j": np.int64,
      "c4": np.complex64, "c": np.complex128}
UP = {"s": "S", "s4": "S4", "i1": "I1", "i2": "I2", "i4": "I4", "j": "J", "c4": "C4", "c": "C"}
PAIRS = [("c4", "c"), ("c", "c4")]
for _c in ("c4", "c"):
    for _x in INTS + ["s4", "s"]:
        PAIRS += [(_c, _x), (_x, _c)]


def _rand(kind, rng, size):
    if kind in COMP:
        rt = DT[COMP[kind]]
        return (rng.standard_normal(size).astype(rt) + 1j * rng.standard_normal(size).astype(rt)).astype(DT[kind])
    if kind in ("s", "s4"):
        return rng.standard_normal(size).astype(DT[kind])
    return rng.integers(-99, 99, size, dtype=DT[kind])


def _dv(kind, arr, extents, strides, assoc=True):
    code = (DopeVector.TYPE_COMPLEX if kind in COMP else
            DopeVector.TYPE_REAL if kind in ("s", "s4") else DopeVector.TYPE_INTEGER)
    return DopeVector.make(arr.ctypes.data if arr is not None else None, extents, strides,
                           8 * np.dtype(DT[kind]).itemsize, code, assoc)


def _result_kind(ka, kb):
    comps = [COMP.get(k, k) for k in (ka, kb)]
    return "c" if "s" in comps else "c4"


def _parts(kind, arr):
    """The flat arrays the kernel is handed for one operand, and the factor on its increments."""
    if kind in COMP:
        flat = arr.view(DT[COMP[kind]])
        return [flat, flat[1:]], 2
    return [arr], 1


def _ref_product(ka, kb, a, b, m, n, k, inc_a, inc_b):
    """The entry point's kernel calls, repeated on the CPU restatement.  inc_a / inc_b: (inc1, inc2)
    in elements; the result is column-major m x n."""
    kc = _result_kind(ka, kb)
    rt = DT[COMP[kc]]
    c = np.zeros(2 * m * n, rt)
    pa, fa = _parts(ka, a)
    pb, fb = _parts(kb, b)
    a1, a2, b1, b2 = inc_a[0] * fa, inc_a[1] * fa, inc_b[0] * fb, inc_b[1] * fb
    swapped = ORDER.index(COMP.get(ka, ka)) > ORDER.index(COMP.get(kb, kb))

    def mul(alpha, ia, ib, beta, part_c):
        cv = c[part_c:]
        if not swapped:
            oracle.xgemmx(m, n, k, alpha, pa[ia], a1, a2, pb[ib].astype(rt, copy=False), b1, b2, beta, cv, 2, 2 * m)
        else:
            oracle.xgemmx(n, m, k, alpha, pb[ib], b2, b1, pa[ia].astype(rt, copy=False), a2, a1, beta, cv, 2 * m, 2)

    if ka in COMP and kb in COMP:
        mul(1.0, 0, 0, 0.0, 0)
        mul(-1.0, 1, 1, 1.0, 0)
        mul(1.0, 0, 1, 0.0, 1)
        mul(1.0, 1, 0, 1.0, 1)
    else:
        mul(1.0, 0, 0, 0.0, 0)
        mul(1.0, 1 if ka in COMP else 0, 1 if kb in COMP else 0, 0.0, 1)
    return c.view(DT[kc])


def _close(kc, got, want):
    g = np.ascontiguousarray(got, dtype=np.complex128).view(np.float64)   # (re, im) pairs
    w = np.ascontiguousarray(want, dtype=np.complex128).view(np.float64)
    return relmax(g, w) <= (1e-4 if kc == "c4" else 1e-12)


@pytest.mark.parametrize("ka,kb", PAIRS)
def test_matmul_complex_mixed_entry_points(eng, ka, kb):
    name = "_MATMUL_" + UP[ka] + UP[kb]
    fn = getattr(eng.lib, name)
    kc = _result_kind(ka, kb)
    rng = np.random.default_rng(21)
    m, k, n = 37, 29, 41
    a, b = _rand(ka, rng, m * k), _rand(kb, rng, k * n)
    A, B = a.reshape(k, m).T.astype(np.complex128), b.reshape(n, k).T.astype(np.complex128)
    # matrix x matrix, column-major
    c = np.zeros(m * n, DT[kc])
    fn(ctypes.byref(_dv(kc, c, (m, n), (1, m))), ctypes.byref(_dv(ka, a, (m, k), (1, m))),
       ctypes.byref(_dv(kb, b, (k, n), (1, k))))
    assert eng.lib.o64_compat_last_status() == o.OK
    ref = _ref_product(ka, kb, a, b, m, n, k, (1, m), (1, k))
    assert _close(kc, c, ref)
    assert _close(kc, c.reshape(n, m).T, A @ B)
    # matrix x vector and vector x matrix
    x = b[:k].copy()
    y = np.zeros(m, DT[kc])
    fn(ctypes.byref(_dv(kc, y, (m,), (1,))), ctypes.byref(_dv(ka, a, (m, k), (1, m))),
       ctypes.byref(_dv(kb, x, (k,), (1,))))
    assert eng.lib.o64_compat_last_status() == o.OK
    assert _close(kc, y, A @ x.astype(np.complex128))
    xv = a[:k].copy()
    y2 = np.zeros(n, DT[kc])
    fn(ctypes.byref(_dv(kc, y2, (n,), (1,))), ctypes.byref(_dv(ka, xv, (k,), (1,))),
       ctypes.byref(_dv(kb, b, (k, n), (1, k))))
    assert eng.lib.o64_compat_last_status() == o.OK
    assert _close(kc, y2, xv.astype(np.complex128) @ B)
    # a RESULT that is not associated is allocated by the runtime and handed to the caller
    R = _dv(kc, None, (0, 0), (0, 0), assoc=False)
    R.flags1 = 2 << 29
    fn(ctypes.byref(R), ctypes.byref(_dv(ka, a, (m, k), (1, m))), ctypes.byref(_dv(kb, b, (k, n), (1, k))))
    assert eng.lib.o64_compat_last_status() == o.OK and R.ptr and (R.flags0 & 1)
    assert R.dimension[0].extent == m and R.dimension[1].extent == n
    assert R.orig_size == m * n * 8 * np.dtype(DT[kc]).itemsize
    real_t = ctypes.c_float if kc == "c4" else ctypes.c_double
    got = np.ctypeslib.as_array(ctypes.cast(R.ptr, ctypes.POINTER(real_t)), (2 * m * n,)).copy().view(DT[kc])
    assert _close(kc, got, ref)
    ctypes.CDLL(None).free(ctypes.c_void_p(R.ptr))
    # extents that do not conform
    fn(ctypes.byref(_dv(kc, c, (m, n), (1, m))), ctypes.byref(_dv(ka, a, (m, k), (1, m))),
       ctypes.byref(_dv(kb, b, (k + 1, n), (1, k + 1))))
    assert eng.lib.o64_compat_last_status() == o.ERR_CONFORM


@pytest.mark.parametrize("ka,kb", [("c4", "s4"), ("i2", "c"), ("c", "c4"), ("c4", "j")])
def test_matmul_complex_mixed_sections(eng, ka, kb):
    """Array sections: every other row of A, every third column of B, a RESULT embedded in a larger
    array whose other elements must stay as they were."""
    fn = getattr(eng.lib, "_MATMUL_" + UP[ka] + UP[kb])
    kc = _result_kind(ka, kb)
    rng = np.random.default_rng(22)
    m, k, n = 19, 23, 17
    lda, ldb, ldc = 2 * m + 3, k + 2, 2 * m + 1
    a, b = _rand(ka, rng, lda * k), _rand(kb, rng, ldb * 3 * n)
    A = a.reshape(k, lda).T[0:2 * m:2, :].astype(np.complex128)
    B = b.reshape(3 * n, ldb).T[:k, 0:3 * n:3].astype(np.complex128)
    c = _rand(kc, rng, ldc * n)
    before = c.copy()
    fn(ctypes.byref(_dv(kc, c, (m, n), (2, ldc))), ctypes.byref(_dv(ka, a, (m, k), (2, lda))),
       ctypes.byref(_dv(kb, b, (k, n), (1, 3 * ldb))))
    assert eng.lib.o64_compat_last_status() == o.OK
    C = c.reshape(n, ldc).T
    assert _close(kc, C[0:2 * m:2, :], A @ B)
    mask = np.ones((ldc, n), bool)
    mask[0:2 * m:2, :] = False
    assert np.array_equal(C[mask], before.reshape(n, ldc).T[mask])
