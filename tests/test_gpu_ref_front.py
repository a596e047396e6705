"""GPU: the reference's own C wrappers (osprey/libfi/matrix/matmul_<a><b>.c with _premult of matmul.h,
compiled from the reference tree by oracle/ref_front.mk) driving the ENGINE's strided kernels, beside
the engine's own _MATMUL_<A><B> entry points on the same dope vectors.  Both paths end in the same
CUDA kernels, so results must be bit-identical and the RESULT descriptors equal word for word; a
difference can only come from the engine's restatement of _premult or of a wrapper's operand order.
The rank dispatchers with the BLAS hook bound (F90_MATMUL_BLAS) run in a process of their own."""
import ctypes
import os
import subprocess
import sys
import textwrap
import zlib

import numpy as np
import pytest

import open64_b200 as o
from open64_b200._lib import LIB_PATH
from oracle import ref_front as rf

import frontutil as fu

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def front(eng):
    rf.build()
    if not rf.available("engine"):
        pytest.skip("oracle/_ref is not built and the reference tree is not on this machine")
    return rf


CASES = (("mm", "dense", "dense", True), ("mm", "section", "transposed", False),
         ("mv", "transposed", "section", True), ("vm", "section", "dense", False),
         ("mv", "dense", "dense", False), ("mm", "transposed", "section", True))


@pytest.mark.parametrize("name", rf.ENTRY_POINTS)
def test_engine_entry_point_equals_reference_wrapper(eng, front, name):
    ka, kb = rf.split_kinds(name)
    kr = rf.result_kind(ka, kb)
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    mine = getattr(eng.lib, "_MATMUL_" + name)
    for case, la, lb, assoc in CASES:
        sa, sb, sr = fu.shapes_for(case, 37, 21, 29)
        a, b = fu.Operand(ka, sa, rng, la), fu.Operand(kb, sb, rng, lb)
        r_ref = fu.Result(kr, sr, associated=assoc, layout="strided")
        r_eng = fu.Result(kr, sr, associated=assoc, layout="strided")
        assert rf.call(name, r_ref.desc, a.dv(), b.dv(), backend="engine") == 0
        assert eng.lib.o64_compat_last_status() == o.OK, "the reference wrapper's kernel call failed in the engine"
        A, B = a.dv(), b.dv()
        mine(ctypes.byref(r_eng.desc), ctypes.byref(A), ctypes.byref(B))
        assert eng.lib.o64_compat_last_status() == o.OK
        assert r_ref.descriptor_words() == r_eng.descriptor_words(), f"{name} {case}: RESULT descriptors differ"
        if assoc:
            assert r_ref.storage.tobytes() == r_eng.storage.tobytes(), f"{name} {case} {la}/{lb}"
        got_ref, got_eng = r_ref.values(), r_eng.values()
        assert got_ref.tobytes() == got_eng.tobytes(), f"{name} {case} {la}/{lb}"
        assert fu.close(got_eng, fu.expected(a, b, kr), kr)


def test_error_codes_map_onto_the_runtimes(eng, front):
    c = rf.codes("engine")
    rng = np.random.default_rng(5)
    v, m34 = fu.Operand("S4", (4,), rng), fu.Operand("S4", (3, 4), rng)
    trials = [(fu.Result("S4", (3,)), v, v, "FESCIRNK", o.ERR_RANK),
              (fu.Result("S4", (3, 3)), m34, m34, "FESCICNF", o.ERR_CONFORM),
              (fu.Result("S4", (2,)), m34, v, "FESCICNF", o.ERR_CONFORM)]
    for r, a, b, ref_code, my_code in trials:
        assert rf.call("S4S4", r.desc, a.dv(), b.dv(), backend="engine") == c[ref_code]
        A, B = a.dv(), b.dv()
        eng.lib._MATMUL_S4S4(ctypes.byref(r.desc), ctypes.byref(A), ctypes.byref(B))
        assert eng.lib.o64_compat_last_status() == my_code


def test_dispatchers_reach_the_engine_through_the_blas_hook(eng, front):
    """refdisp_MATMUL_<A><B> (MATMUL_*dispatch.c) -> __f90_open_blas_lib (mmx_dlutil.c, unmodified) ->
    dlsym finds the engine's sgemm_/dgemm_/cgemm_/zgemm_ -> the call of mmx_fort.h:94-95 lands in the
    engine; the result is held against the dispatcher's own dot-product loops (no BLAS bound)."""
    prog = textwrap.dedent(f"""
        import ctypes, os, sys, zlib
        sys.path.insert(0, {ROOT!r}); sys.path.insert(0, os.path.join({ROOT!r}, "tests"))
        import numpy as np
        eng = ctypes.CDLL({LIB_PATH!r}, mode=ctypes.RTLD_GLOBAL)      # what LD_PRELOAD=libo64gemm.so does
        from oracle import ref_front as rf
        import frontutil as fu
        eng.o64_compat_last_status.restype = ctypes.c_int
        for name in rf.DISPATCHED:
            ka, kb = rf.split_kinds(name); kr = rf.result_kind(ka, kb)
            rng = np.random.default_rng(zlib.crc32(name.encode()))
            a, b = fu.Operand(ka, (33, 17), rng, "section"), fu.Operand(kb, (17, 26), rng, "transposed")
            r = fu.Result(kr, (33, 26), associated=False)
            assert rf.call(name, r.desc, a.dv(), b.dv(), backend="engine", dispatched=True) == 0
            assert eng.o64_compat_last_status() == 0, name
            got = r.values()
            assert fu.close(got, fu.expected(a, b, kr), kr), name
        front = rf.lib("engine")
        for n in ("sgemm", "dgemm", "cgemm", "zgemm"):
            p = ctypes.c_void_p.in_dll(front, "__f90_" + n + "_blas").value
            assert p == ctypes.cast(getattr(eng, n + "_"), ctypes.c_void_p).value, n
        print("ok")
    """)
    env = dict(os.environ, F90_MATMUL_BLAS="1")
    r = subprocess.run([sys.executable, "-c", prog], capture_output=True, text=True, env=env, cwd=ROOT)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr
