"""GPU: DOT_PRODUCT over dope vectors (_DOT_<A><B>, osprey/libfi/dotprod) against numpy on the elements
the reference's own _PREDOT (predot@.c, compiled from the reference tree) says the vectors have."""
import ctypes

import numpy as np
import pytest

import open64_b200 as o
from open64_b200._lib import DOT_RESTYPE
from oracle import ref_front as rf

import frontutil as fu

pytestmark = pytest.mark.gpu

NAMES = [n[5:] for n in DOT_RESTYPE]           # "S4S4", "I4J", "L4L", "C4C4", ...


def _predot(a, b):
    """(n, element strides) as the reference parses them; None when oracle/_ref is not built."""
    if not rf.available("oracle"):
        return None
    n, lx, ix, ly, iy = (ctypes.c_long() for _ in range(5))
    A, B = a.dv(), b.dv()
    rf.lib().ref_PREDOT(ctypes.byref(A), ctypes.byref(B), ctypes.byref(n), ctypes.byref(lx), ctypes.byref(ix),
                        ctypes.byref(ly), ctypes.byref(iy))
    assert lx.value == a.storage.ctypes.data and ly.value == b.storage.ctypes.data
    return n.value, ix.value, iy.value


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("n,layout", [(1, "dense"), (1000, "dense"), (4097, "section"), (300000, "dense")])
def test_dot_product(eng, name, n, layout):
    ka, kb = rf.split_kinds(name)
    kr = rf.result_kind(ka, kb)
    rng = np.random.default_rng(n + len(name))
    a, b = fu.Operand(ka, (n,), rng, layout), fu.Operand(kb, (n,), rng, "dense")
    parsed = _predot(a, b)
    if parsed is not None:
        assert parsed == (n, a.inc[0], b.inc[0])
    A, B = a.dv(), b.dv()
    got = getattr(eng.lib, "_DOT_" + name)(ctypes.byref(A), ctypes.byref(B))
    assert eng.lib.o64_compat_last_status() == o.OK
    x, y = a.values(), b.values()
    if kr[0] == "L":
        assert int(got) == int(((x != 0) & (y != 0)).any())
    elif kr[0] in "IJ":
        dt = np.dtype(rf.KINDS[kr][0])
        want = (x.astype(np.int64) * y.astype(np.int64)).sum().astype(dt)     # wraps in the result kind
        assert int(got) == int(want)
    elif kr[0] == "C":
        want = np.vdot(x.astype(np.complex128), y.astype(np.complex128))      # conjugates the first vector
        g = complex(got.re, got.im)
        scale = np.abs(x.astype(np.complex128) * y).sum() + 1e-30
        assert abs(g - want) <= (1e-5 if kr == "C4" else 1e-13) * scale
    else:
        want = (x.astype(np.float64) * y.astype(np.float64)).sum()
        scale = np.abs(x.astype(np.float64) * y).sum() + 1e-30
        assert abs(float(got) - want) <= (1e-5 if kr == "S4" else 1e-13) * scale


def test_empty_and_nonconformable(eng):
    rng = np.random.default_rng(1)
    a0, b = fu.Operand("S4", (0,), rng), fu.Operand("S4", (5,), rng)
    A, B = a0.dv(), b.dv()
    assert eng.lib._DOT_S4S4(ctypes.byref(A), ctypes.byref(B)) == 0.0
    assert eng.lib.o64_compat_last_status() == o.OK
    a9 = fu.Operand("S4", (9,), rng)
    A = a9.dv()
    assert eng.lib._DOT_S4S4(ctypes.byref(A), ctypes.byref(B)) == 0.0
    assert eng.lib.o64_compat_last_status() == o.ERR_CONFORM
    m = fu.Operand("S4", (3, 3), rng)
    M = m.dv()
    eng.lib._DOT_S4S4(ctypes.byref(M), ctypes.byref(B))
    assert eng.lib.o64_compat_last_status() == o.ERR_RANK
