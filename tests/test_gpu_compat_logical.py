"""GPU: the LOGICAL members of the runtime's MATMUL family (template osprey/libfi/matrix/lgemmx.h:
C = (beta .AND. C) .OR. (alpha .AND. (A .AND. B, OR-reduced over K)); 1-, 2-, 4- and 8-byte logicals
carried as integers, non-zero is true): the ten strided kernels and the sixteen _MATMUL_L?L? entry
points against the CPU restatement and against numpy.  Exact."""
import ctypes

import numpy as np
import pytest
import torch

import open64_b200 as o
import oracle
from open64_b200._lib import DopeVector

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"l1": np.int8, "l2": np.int16, "l4": np.int32, "l": np.int64}
KINDS = ["l1", "l2", "l4", "l"]
KERNELS = {(a if a == c else a + c): (a, c) for i, a in enumerate(KINDS) for c in KINDS[i:]}


def _logicals(kind, rng, size, density=0.08):
    """Mostly false; the true values are not all 1 (any non-zero value counts)."""
    v = (rng.random(size) < density) * rng.integers(1, 100, size) * rng.choice([-1, 1], size)
    return v.astype(DT[kind])


@pytest.mark.parametrize("kernel", list(KERNELS))
def test_lgemmx_kernels_match_oracle(eng, kernel):
    ka, kc = KERNELS[kernel]
    rng = np.random.default_rng(len(kernel) * 7 + 1)
    for (m, n, k) in ((1, 1, 1), (19, 13, 17), (130, 70, 33)):
        a, b, c0 = _logicals(ka, rng, m * k), _logicals(kc, rng, k * n), _logicals(kc, rng, m * n, 0.3)
        for alpha, beta in ((True, False), (True, True), (False, True), (False, False)):
            ref = oracle.lgemmx(m, n, k, alpha, a, 1, m, b, 1, k, beta, c0.copy(), 1, m)
            for where in ("host", "device"):
                ta, tb, tc = (torch.from_numpy(v.copy()) for v in (a, b, c0))
                if where == "device":
                    ta, tb, tc = ta.to(DEV), tb.to(DEV), tc.to(DEV)
                eng.lgemmx(kernel, m, n, k, alpha, ta, 1, m, tb, 1, k, beta, tc, 1, m)
                if not alpha and beta:
                    assert np.array_equal(tc.cpu().numpy(), c0)     # untouched, also the values other than 1
                else:
                    assert np.array_equal(tc.cpu().numpy(), ref), (where, alpha, beta)
        tc = torch.from_numpy(c0.copy())
        eng.lgemmx(kernel, m, n, 0, True, torch.from_numpy(a), 1, m, torch.from_numpy(b), 1, k, True, tc, 1, m)
        assert not tc.numpy().any()                                   # K = 0 clears C whatever beta says


def _dv(kind, arr, extents, strides, assoc=True):
    return DopeVector.make(arr.ctypes.data if arr is not None else None, extents, strides,
                           8 * np.dtype(DT[kind]).itemsize, DopeVector.TYPE_LOGICAL, assoc)


@pytest.mark.parametrize("ka", KINDS)
@pytest.mark.parametrize("kb", KINDS)
def test_matmul_logical_entry_points(eng, ka, kb):
    up = {"l1": "L1", "l2": "L2", "l4": "L4", "l": "L"}
    kc = KINDS[max(KINDS.index(ka), KINDS.index(kb))]
    fn = getattr(eng.lib, "_MATMUL_" + up[ka] + up[kb])
    rng = np.random.default_rng(11)
    m, k, n = 37, 29, 41
    a, b = _logicals(ka, rng, m * k), _logicals(kb, rng, k * n)
    A, B = a.reshape(k, m).T != 0, b.reshape(n, k).T != 0
    want = (A.astype(np.int64) @ B.astype(np.int64)) > 0
    c = np.full(m * n, 7, DT[kc])
    fn(ctypes.byref(_dv(kc, c, (m, n), (1, m))), ctypes.byref(_dv(ka, a, (m, k), (1, m))), ctypes.byref(_dv(kb, b, (k, n), (1, k))))
    assert eng.lib.o64_compat_last_status() == o.OK
    assert np.array_equal(c.reshape(n, m).T, want.astype(DT[kc]))
    x = b[:k].copy()
    y = np.full(m, 7, DT[kc])
    fn(ctypes.byref(_dv(kc, y, (m,), (1,))), ctypes.byref(_dv(ka, a, (m, k), (1, m))), ctypes.byref(_dv(kb, x, (k,), (1,))))
    assert eng.lib.o64_compat_last_status() == o.OK
    assert np.array_equal(y, ((A.astype(np.int64) @ (x != 0).astype(np.int64)) > 0).astype(DT[kc]))
    xv = a[:k].copy()
    y2 = np.full(n, 7, DT[kc])
    fn(ctypes.byref(_dv(kc, y2, (n,), (1,))), ctypes.byref(_dv(ka, xv, (k,), (1,))), ctypes.byref(_dv(kb, b, (k, n), (1, k))))
    assert eng.lib.o64_compat_last_status() == o.OK
    assert np.array_equal(y2, (((xv != 0).astype(np.int64) @ B.astype(np.int64)) > 0).astype(DT[kc]))
    fn(ctypes.byref(_dv(kc, c, (m, n), (1, m))), ctypes.byref(_dv(ka, a, (m, k), (1, m))), ctypes.byref(_dv(kb, b, (k + 1, n), (1, k + 1))))
    assert eng.lib.o64_compat_last_status() == o.ERR_CONFORM
