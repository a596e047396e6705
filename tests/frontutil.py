"""Operands for the MATMUL entry points: numpy storage + dope vectors in the runtime's layout, and the
expected product computed with numpy in the arithmetic of the result kind."""
import ctypes

import numpy as np

from open64_b200._lib import DopeVector
from oracle import ref_front as rf


class Operand:
    """A rank-1 or rank-2 Fortran array (or array section) of one of the runtime's kinds."""

    def __init__(self, kind, extents, rng, layout="dense"):
        self.kind = kind
        dt, self.type_code, self.bits = rf.KINDS[kind]
        self.dtype = np.dtype(dt)
        self.extents = tuple(extents)
        n1 = extents[0]
        n2 = extents[1] if len(extents) == 2 else 1
        # element strides (inc1 down a column, inc2 across): dense column-major, a padded leading
        # dimension with every second row (a section A(1:2*n1:2, :) of a larger array), or the
        # transposed storage of a row-major array
        if layout == "dense":
            inc1, inc2 = 1, max(n1, 1)
        elif layout == "section":
            inc1, inc2 = 2, 2 * n1 + 3
        elif layout == "transposed":
            inc1, inc2 = max(n2, 1) + 1, 1
        else:
            raise ValueError(layout)
        self.inc = (inc1, inc2)[:len(extents)]
        span = (max(n1, 1) - 1) * inc1 + (max(n2, 1) - 1) * inc2 + 1
        if kind[0] == "L":
            flat = rng.choice(np.array([0, 0, 0, 1, 5, -1]), span).astype(dt)   # any non-zero value is .TRUE.
        elif kind[0] in "IJ":
            flat = rng.integers(-100, 101, span).astype(dt)
        elif kind[0] == "C":
            flat = (rng.standard_normal(span) + 1j * rng.standard_normal(span)).astype(dt)
        else:
            flat = rng.standard_normal(span).astype(dt)
        if span > 3 and kind[0] != "L":
            flat[rng.integers(0, span, max(span // 7, 1))] = 0   # zeros exercise the skip-if-zero branches
        self.storage = flat
        idx = (np.arange(n1)[:, None] * inc1 + np.arange(n2)[None, :] * inc2)
        self.index = idx if len(extents) == 2 else idx[:, 0]

    def values(self):
        return self.storage[self.index]

    def dv(self):
        return DopeVector.make(self.storage.ctypes.data, self.extents, self.inc, self.bits, self.type_code)


class Result:
    """RESULT: associated storage pre-filled with a sentinel, or an unassociated descriptor the
    callee must allocate (matmul.h:222-266)."""

    def __init__(self, kind, extents, associated=True, layout="dense"):
        self.kind = kind
        dt, self.type_code, self.bits = rf.KINDS[kind]
        self.dtype = np.dtype(dt)
        self.extents = tuple(extents)
        self.associated = associated
        n1 = extents[0]
        n2 = extents[1] if len(extents) == 2 else 1
        inc1, inc2 = (1, max(n1, 1)) if layout == "dense" else (3, 3 * n1 + 2)
        self.inc = (inc1, inc2)[:len(extents)]
        span = (max(n1, 1) - 1) * inc1 + (max(n2, 1) - 1) * inc2 + 1
        self.storage = np.full(span, 77, dtype=dt)
        idx = (np.arange(n1)[:, None] * inc1 + np.arange(n2)[None, :] * inc2)
        self.index = idx if len(extents) == 2 else idx[:, 0]
        if associated:
            self.desc = DopeVector.make(self.storage.ctypes.data, self.extents, self.inc, self.bits, self.type_code)
        else:
            self.desc = DopeVector.make(None, (0,) * len(extents), (0,) * len(extents), self.bits, self.type_code,
                                        assoc=False)
            self.desc.orig_base = None

    def values(self):
        """The result as an array of the logical shape; for an allocated RESULT the callee's storage
        is copied out and freed (the caller owns it)."""
        if self.associated:
            return self.storage[self.index].copy()
        d = self.desc
        n = int(np.prod(self.extents)) if self.extents else 0
        if n == 0:
            return np.zeros(self.extents, self.dtype)
        raw = (ctypes.c_ubyte * (n * self.dtype.itemsize)).from_address(d.ptr)
        out = np.frombuffer(bytes(raw), dtype=self.dtype).reshape(self.extents, order="F").copy()
        ctypes.CDLL(None).free(ctypes.c_void_p(d.ptr))
        d.ptr = None
        return out

    def descriptor_words(self):
        """Everything of the descriptor except the two addresses (they differ between two calls that
        each allocate)."""
        d = self.desc
        dims = [(d.dimension[i].low_bound, d.dimension[i].extent, d.dimension[i].stride_mult)
                for i in range(len(self.extents))]
        return (d.el_len, d.flags0, d.flags1, d.type_pad, d.type_bits, d.orig_size, tuple(dims),
                (d.ptr is not None and d.ptr != 0), d.orig_base == d.ptr)


def expected(a, b, res_kind):
    """numpy's product in the arithmetic of the result kind."""
    dt = np.dtype(rf.KINDS[res_kind][0])
    A, B = a.values(), b.values()
    if res_kind[0] == "L":
        return ((A != 0).astype(np.int64) @ (B != 0).astype(np.int64) > 0).astype(dt)
    if res_kind[0] in "IJ":
        return (A.astype(np.int64) @ B.astype(np.int64)).astype(dt)      # wraps like the Fortran kernels
    wide = np.complex128 if res_kind[0] == "C" else np.float64
    return A.astype(wide) @ B.astype(wide)


def shapes_for(case, m, k, n):
    """Extents of A, B and RESULT for 'mm' (matrix x matrix), 'mv' and 'vm'."""
    if case == "mm":
        return (m, k), (k, n), (m, n)
    if case == "mv":
        return (m, k), (k,), (m,)
    return (k,), (k, n), (n,)


def tolerance(res_kind):
    if res_kind[0] in "IJL":
        return 0.0
    return 1e-4 if res_kind in ("S4", "C4") else 1e-12


def close(got, want, res_kind):
    tol = tolerance(res_kind)
    if tol == 0.0:
        return np.array_equal(got, want)
    scale = max(float(np.abs(want).max()) if want.size else 0.0, 1e-30)
    return float(np.abs(got.astype(want.dtype) - want).max() if want.size else 0.0) <= tol * scale
