"""GPU: the COMPLEX*8 / COMPLEX*16 members of the runtime's MATMUL family — _c4gemmx__ / _cgemmx__
with their conjugation flags (osprey/libfi/matrix/c4gemmx.f, cgemmx.f), the matrix-vector kernels,
the BLAS hooks cgemm_ / zgemm_ and _MATMUL_C4C4 / _MATMUL_CC over dope vectors — against the CPU
restatement.  Gate: max|y - ref| / max|ref| <= 1e-5 (COMPLEX*8), 1e-12 (COMPLEX*16)."""
import ctypes

import numpy as np
import pytest
import torch

import open64_b200 as o
import oracle
from open64_b200._lib import DopeVector

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {np.complex64: 1e-5, np.complex128: 1e-12}


def _cplx(rng, size, dt):
    return (rng.standard_normal(size) + 1j * rng.standard_normal(size)).astype(dt)


def _close(got, want, dt):
    return np.abs(got - want).max() / max(np.abs(want).max(), 1e-30) <= TOL[dt]


@pytest.mark.parametrize("dt", [np.complex64, np.complex128])
@pytest.mark.parametrize("shape", [(1, 1, 1), (19, 13, 17), (64, 64, 64), (130, 70, 33)])
def test_cgemmx_matches_oracle(eng, dt, shape):
    m, n, k = shape
    rng = np.random.default_rng(m + n * 3 + k * 5)
    a, b, c0 = _cplx(rng, m * k, dt), _cplx(rng, k * n, dt), _cplx(rng, m * n, dt)
    for alpha, beta, ca, cb in ((1.0, 0.0, 0, 0), (0.5 - 2j, 1.0, 1, 0), (-1j, 0.25 + 1j, 0, 1), (2.0, -1.0, 1, 1)):
        ref = oracle.cgemmx(m, n, k, alpha, a, 1, m, b, 1, k, beta, c0.copy(), 1, m, ca, cb)
        for where in ("host", "device"):
            ta, tb, tc = (torch.from_numpy(v.copy()) for v in (a, b, c0))
            if where == "device":
                ta, tb, tc = ta.to(DEV), tb.to(DEV), tc.to(DEV)
            eng.cgemmx(m, n, k, alpha, ta, 1, m, tb, 1, k, beta, tc, 1, m, ca, cb)
            assert _close(tc.cpu().numpy(), ref, dt), (where, alpha, beta, ca, cb)
    # transposed operand through the increments, K = 0, alpha = 0 with beta = 1
    ref = oracle.cgemmx(m, n, k, 1.0, a, 1, m, b, n, 1, 0.0, c0.copy(), n, 1)
    tc = torch.from_numpy(c0.copy())
    eng.cgemmx(m, n, k, 1.0, torch.from_numpy(a), 1, m, torch.from_numpy(b), n, 1, 0.0, tc, n, 1)
    assert _close(tc.numpy(), ref, dt)
    tc = torch.from_numpy(c0.copy())
    eng.cgemmx(m, n, 0, 1.0, torch.from_numpy(a), 1, m, torch.from_numpy(b), 1, k, 3.0, tc, 1, m)
    assert not tc.numpy().any()
    tc = torch.from_numpy(c0.copy())
    eng.cgemmx(m, n, k, 0.0, torch.from_numpy(a), 1, m, torch.from_numpy(b), 1, k, 1.0, tc, 1, m)
    assert np.array_equal(tc.numpy(), c0)


@pytest.mark.parametrize("dt", [np.complex64, np.complex128])
def test_cgemvx_and_blas_hooks(eng, dt):
    rng = np.random.default_rng(3)
    m, n, k = 33, 21, 45
    a, x, y0 = _cplx(rng, m * k, dt), _cplx(rng, 2 * k, dt), _cplx(rng, m, dt)
    x[::6] = 0
    for conj in (0, 1):
        ref = oracle.cgemvx(m, k, 0.75 + 1j, a, 1, m, x, 2, 2.0 - 1j, y0.copy(), 1, conj)
        y = torch.from_numpy(y0.copy())
        eng.cgemvx(m, k, 0.75 + 1j, torch.from_numpy(a), 1, m, torch.from_numpy(x), 2, 2.0 - 1j, y, 1, conj)
        assert _close(y.numpy(), ref, dt)
    y = torch.from_numpy(y0.copy())
    eng.cgemvx(m, 0, 1.0, torch.from_numpy(a), 1, m, torch.from_numpy(x), 1, 5.0, y, 1)
    assert not y.numpy().any()
    # BLAS: C = alpha op(A) op(B) + beta C, column-major, 'c' = conjugate transpose
    A, B, C0 = _cplx(rng, (m, k), dt), _cplx(rng, (k, n), dt), _cplx(rng, (m, n), dt)
    ops = {"n": lambda z: z, "t": lambda z: z.T, "c": lambda z: z.conj().T}
    for ta in "ntc":
        for tb in "nc":
            sa = np.asfortranarray(A if ta == "n" else ops[ta](A))      # stored so that op(stored) == A
            sb = np.asfortranarray(B if tb == "n" else ops[tb](B))
            tc = torch.from_numpy(np.asfortranarray(C0).ravel(order="F").copy())
            eng.cgemm(ta, tb, m, n, k, 1.25 - 0.5j, torch.from_numpy(sa.ravel(order="F").copy()), sa.shape[0],
                      torch.from_numpy(sb.ravel(order="F").copy()), sb.shape[0], -0.5j, tc, m)
            want = (1.25 - 0.5j) * (A @ B) + (-0.5j) * C0
            assert _close(tc.numpy().reshape(n, m).T, want.astype(dt), dt), (ta, tb)


def _dv(arr, extents, strides, dt, assoc=True):
    bits = 64 if dt is np.complex64 else 128
    return DopeVector.make(arr.ctypes.data if arr is not None else None, extents, strides, bits, DopeVector.TYPE_COMPLEX, assoc)


@pytest.mark.parametrize("dt,name", [(np.complex64, "_MATMUL_C4C4"), (np.complex128, "_MATMUL_CC")])
def test_matmul_complex_entry_points(eng, dt, name):
    fn = getattr(eng.lib, name)
    rng = np.random.default_rng(9)
    m, k, n = 37, 29, 41
    a, b = _cplx(rng, m * k, dt), _cplx(rng, k * n, dt)
    A, B = a.reshape(k, m).T, b.reshape(n, k).T
    c = np.zeros(m * n, dt)
    fn(ctypes.byref(_dv(c, (m, n), (1, m), dt)), ctypes.byref(_dv(a, (m, k), (1, m), dt)), ctypes.byref(_dv(b, (k, n), (1, k), dt)))
    assert eng.lib.o64_compat_last_status() == o.OK
    assert _close(c.reshape(n, m).T, A @ B, dt)
    x = b[:k].copy()
    y = np.zeros(m, dt)
    fn(ctypes.byref(_dv(y, (m,), (1,), dt)), ctypes.byref(_dv(a, (m, k), (1, m), dt)), ctypes.byref(_dv(x, (k,), (1,), dt)))
    assert eng.lib.o64_compat_last_status() == o.OK and _close(y, A @ x, dt)
    xv = a[:k].copy()
    y2 = np.zeros(n, dt)
    fn(ctypes.byref(_dv(y2, (n,), (1,), dt)), ctypes.byref(_dv(xv, (k,), (1,), dt)), ctypes.byref(_dv(b, (k, n), (1, k), dt)))
    assert eng.lib.o64_compat_last_status() == o.OK and _close(y2, xv @ B, dt)
    R = _dv(None, (0, 0), (0, 0), dt, assoc=False)
    R.flags1 = 2 << 29
    fn(ctypes.byref(R), ctypes.byref(_dv(a, (m, k), (1, m), dt)), ctypes.byref(_dv(b, (k, n), (1, k), dt)))
    assert eng.lib.o64_compat_last_status() == o.OK and R.ptr and R.dimension[1].extent == n
    assert R.orig_size == m * n * (64 if dt is np.complex64 else 128)
    real_t = ctypes.c_float if dt is np.complex64 else ctypes.c_double
    got = np.ctypeslib.as_array(ctypes.cast(R.ptr, ctypes.POINTER(real_t)), (2 * m * n,)).copy().view(dt)
    assert _close(got.reshape(n, m).T, A @ B, dt)
    ctypes.CDLL(None).free(ctypes.c_void_p(R.ptr))
    fn(ctypes.byref(_dv(c, (m, n), (1, m), dt)), ctypes.byref(_dv(a, (m, k), (1, m), dt)), ctypes.byref(_dv(b, (k + 1, n), (1, k + 1), dt)))
    assert eng.lib.o64_compat_last_status() == o.ERR_CONFORM
