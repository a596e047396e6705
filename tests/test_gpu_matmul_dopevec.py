"""GPU: _MATMUL_S4S4, the operator entry point the reference's Fortran front end calls for MATMUL
on REAL*4 arrays (osprey/libfi/matrix/matmul_s4s4.c:66-112), driven through dope vectors and
checked against the CPU restatement of the runtime's strided kernels."""
import ctypes

import numpy as np
import pytest

import open64_b200 as o
import oracle
from open64_b200._lib import DopeVector
from util import TOL_F32, relmax

pytestmark = pytest.mark.gpu


def _dv(arr, extents, strides, assoc=True):
    return DopeVector.real4(arr.ctypes.data if arr is not None else None, extents, strides, assoc)


def test_matrix_matrix_column_major_and_sections(eng):
    rng = np.random.default_rng(1)
    m, k, n = 37, 29, 41
    a = rng.standard_normal(m * k).astype(np.float32)          # Fortran A(m,k), column-major
    b = rng.standard_normal(k * n).astype(np.float32)
    c = np.full(m * n, np.nan, np.float32)
    A, B, C = _dv(a, (m, k), (1, m)), _dv(b, (k, n), (1, k)), _dv(c, (m, n), (1, m))
    eng.lib._MATMUL_S4S4(ctypes.byref(C), ctypes.byref(A), ctypes.byref(B))
    assert eng.lib.o64_compat_last_status() == o.OK
    ref = np.zeros(m * n, np.float32)
    oracle.s4gemmx(m, n, k, 1.0, a, 1, m, b, 1, k, 0.0, ref, 1, m)
    assert relmax(c, ref) <= TOL_F32
    # an array section A(1:m:2, :) and a transposed view of B expressed through strides
    m2 = (m + 1) // 2
    bt = np.ascontiguousarray(b.reshape(n, k).T).ravel()        # storage of B^T: (n,k) column-major
    c2 = np.full(m2 * n, np.nan, np.float32)
    A2 = _dv(a, (m2, k), (2, m))
    B2 = _dv(bt, (k, n), (n, 1))
    C2 = _dv(c2, (m2, n), (1, m2))
    eng.lib._MATMUL_S4S4(ctypes.byref(C2), ctypes.byref(A2), ctypes.byref(B2))
    assert eng.lib.o64_compat_last_status() == o.OK
    ref2 = np.zeros(m2 * n, np.float32)
    oracle.s4gemmx(m2, n, k, 1.0, a, 2, m, bt, n, 1, 0.0, ref2, 1, m2)
    assert relmax(c2, ref2) <= TOL_F32


def test_rank_one_operands(eng):
    rng = np.random.default_rng(2)
    m, k = 45, 33
    a = rng.standard_normal(m * k).astype(np.float32)
    x = rng.standard_normal(k).astype(np.float32)
    x[5] = 0.0
    y = np.full(m, np.nan, np.float32)
    eng.lib._MATMUL_S4S4(ctypes.byref(_dv(y, (m,), (1,))), ctypes.byref(_dv(a, (m, k), (1, m))),
                         ctypes.byref(_dv(x, (k,), (1,))))
    assert eng.lib.o64_compat_last_status() == o.OK
    ref = np.zeros(m, np.float32)
    oracle.s4gemvx(m, k, 1.0, a, 1, m, x, 1, 0.0, ref, 1)
    assert relmax(y, ref) <= TOL_F32
    # vector times matrix: y = x B with x of length m, B(m,k)
    xv = rng.standard_normal(m).astype(np.float32)
    y2 = np.full(k, np.nan, np.float32)
    eng.lib._MATMUL_S4S4(ctypes.byref(_dv(y2, (k,), (1,))), ctypes.byref(_dv(xv, (m,), (1,))),
                         ctypes.byref(_dv(a, (m, k), (1, m))))
    assert eng.lib.o64_compat_last_status() == o.OK
    ref2 = np.zeros(k, np.float32)
    oracle.s4gemvx(k, m, 1.0, a, m, 1, xv, 1, 0.0, ref2, 1)
    assert relmax(y2, ref2) <= TOL_F32


def test_result_is_allocated_when_not_associated(eng):
    rng = np.random.default_rng(3)
    m, k, n = 12, 7, 9
    a = rng.standard_normal(m * k).astype(np.float32)
    b = rng.standard_normal(k * n).astype(np.float32)
    R = _dv(None, (0, 0), (0, 0), assoc=False)
    R.flags1 = 2 << 29
    eng.lib._MATMUL_S4S4(ctypes.byref(R), ctypes.byref(_dv(a, (m, k), (1, m))), ctypes.byref(_dv(b, (k, n), (1, k))))
    assert eng.lib.o64_compat_last_status() == o.OK
    assert R.flags0 & 1 and R.ptr and R.orig_base == R.ptr and R.orig_size == m * n * 32
    assert (R.dimension[0].extent, R.dimension[1].extent) == (m, n)
    assert (R.dimension[0].stride_mult, R.dimension[1].stride_mult) == (1, m)
    got = np.ctypeslib.as_array(ctypes.cast(R.ptr, ctypes.POINTER(ctypes.c_float)), shape=(m * n,)).copy()
    ctypes.CDLL(None).free(ctypes.c_void_p(R.ptr))              # the caller owns the storage
    ref = np.zeros(m * n, np.float32)
    oracle.s4gemmx(m, n, k, 1.0, a, 1, m, b, 1, k, 0.0, ref, 1, m)
    assert relmax(got, ref) <= TOL_F32


def test_rank_and_conformance_errors_are_codes_not_aborts(eng):
    a = np.zeros(12, np.float32)
    v = _dv(a, (3,), (1,))
    mtx = _dv(a, (3, 4), (1, 3))
    eng.lib._MATMUL_S4S4(ctypes.byref(_dv(a, (3,), (1,))), ctypes.byref(v), ctypes.byref(v))
    assert eng.lib.o64_compat_last_status() == o.ERR_RANK        # vector x vector: FESCIRNK
    eng.lib._MATMUL_S4S4(ctypes.byref(_dv(a, (3, 3), (1, 3))), ctypes.byref(mtx), ctypes.byref(mtx))
    assert eng.lib.o64_compat_last_status() == o.ERR_CONFORM     # (3,4) x (3,4): FESCICNF
    eng.lib._MATMUL_S4S4(ctypes.byref(_dv(a, (2,), (1,))), ctypes.byref(mtx), ctypes.byref(_dv(a, (4,), (1,))))
    assert eng.lib.o64_compat_last_status() == o.ERR_CONFORM     # result extent 2 != 3
