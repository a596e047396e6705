"""The reference's own C code for the MATMUL boundary, compiled from its sources (oracle/ref_front.mk),
held against the engine's view of the same boundary.  CPU only: the reference's wrappers run here with
the CPU oracle's strided kernels behind them.

What this pins to reference-built code: the layout of the dope vector (o64_dopevec_t vs the compiler's
DopeVectorType), _premult's parsing / allocation / conformance rules as exercised through all 80
wrappers, the operand exchange of the mixed-kind wrappers, the rank dispatchers, and the dlsym hook of
mmx_dlutil.c resolving to the engine's sgemm_ / dgemm_ / cgemm_ / zgemm_.
"""
import ctypes
import os
import subprocess
import sys
import textwrap
import zlib

import numpy as np
import pytest

from open64_b200._lib import DopeVector, LIB_PATH
from oracle import ref_front as rf

import frontutil as fu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def front(built):
    rf.build()
    if not rf.available("oracle"):
        pytest.skip("oracle/_ref is not built and the reference tree is not on this machine")
    return rf


def test_dope_vector_layout_matches_the_compilers(front):
    """Field by field: one field of the real DopeVectorType is set through its bit-field name, the
    same field of o64_dopevec_t through the documented word and bit position; the bytes must agree."""
    assert rf.lib().o64front_dv_sizeof() == ctypes.sizeof(DopeVector) == 216

    def mine(setter):
        d = DopeVector()
        setter(d)
        return bytes(d)

    ones = (1 << 64) - 1
    cases = {
        0: lambda d: setattr(d, "flags0", 1 << 0),            # assoc
        1: lambda d: setattr(d, "flags0", 1 << 1),            # ptr_alloc
        2: lambda d: setattr(d, "flags0", 3 << 2),            # p_or_a
        3: lambda d: setattr(d, "flags0", 1 << 4),            # a_contig
        4: lambda d: setattr(d, "flags1", 7 << 29),           # n_dim
        5: lambda d: setattr(d, "type_bits", 0xff),           # type
        6: lambda d: setattr(d, "type_bits", 1 << 8),         # dpflag
        7: lambda d: setattr(d, "type_bits", 7 << 9),         # kind_or_star
        8: lambda d: setattr(d, "type_bits", 0xfff << 12),    # int_len
        9: lambda d: setattr(d, "type_bits", 0xff << 24),     # dec_len
        10: lambda d: setattr(d, "ptr", ones),
        11: lambda d: setattr(d, "el_len", ones),
        12: lambda d: setattr(d, "orig_base", ones),
        13: lambda d: setattr(d, "orig_size", ones),
        14: lambda d: setattr(d.dimension[1], "low_bound", -1),
        15: lambda d: setattr(d.dimension[1], "extent", -1),
        16: lambda d: setattr(d.dimension[1], "stride_mult", -1),
        17: lambda d: setattr(d.dimension[6], "stride_mult", -1),
    }
    for which, setter in cases.items():
        assert rf.dv_probe(which) == mine(setter), f"field {which} sits elsewhere in the real structure"


def test_error_codes_are_the_runtimes(front):
    c = rf.codes()
    assert c["FESCICNF"] == c["FESCIRNK"] + 1 and c["FENOMEMY"] < c["FESCIRNK"]


@pytest.mark.parametrize("name", rf.ENTRY_POINTS)
def test_reference_wrappers_over_the_oracle_kernels(front, name):
    """Every wrapper, three rank cases, strided and transposed operands, RESULT associated or not:
    reference front half + oracle arithmetic against numpy."""
    ka, kb = rf.split_kinds(name)
    kr = rf.result_kind(ka, kb)
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    for case, la, lb, assoc in (("mm", "dense", "dense", True), ("mm", "section", "transposed", False),
                                ("mv", "transposed", "section", True), ("vm", "section", "dense", False),
                                ("mm", "transposed", "section", True)):
        sa, sb, sr = fu.shapes_for(case, 13, 9, 11)
        a, b = fu.Operand(ka, sa, rng, la), fu.Operand(kb, sb, rng, lb)
        r = fu.Result(kr, sr, associated=assoc, layout="dense" if assoc is False else "strided")
        A, B = a.dv(), b.dv()
        code = rf.call(name, r.desc, A, B)
        assert code == 0, f"{name} {case}: runtime error {code}"
        if not assoc:
            d = r.desc
            assert d.flags0 & 1 and d.ptr and d.orig_base == d.ptr
            n_el = int(np.prod(sr))
            assert d.orig_size == n_el * rf.KINDS[kr][2]
            words = max(rf.KINDS[kr][2] // 32, 1)
            assert d.dimension[0].stride_mult == words and d.dimension[0].extent == sr[0]
            if len(sr) == 2:
                assert d.dimension[1].stride_mult == words * sr[0] and d.dimension[1].extent == sr[1]
        got = r.values()
        assert fu.close(got, fu.expected(a, b, kr), kr), f"{name} {case} {la}/{lb}"
        if assoc:  # nothing outside the RESULT's elements was written
            mask = np.ones(r.storage.size, bool)
            mask[r.index.ravel()] = False
            assert np.all(r.storage[mask] == 77)


def test_rank_and_conformance_errors(front):
    c = rf.codes()
    rng = np.random.default_rng(5)
    v = fu.Operand("S4", (4,), rng)
    m34 = fu.Operand("S4", (3, 4), rng)
    r = fu.Result("S4", (3,))
    assert rf.call("S4S4", r.desc, v.dv(), v.dv()) == c["FESCIRNK"]                      # vector x vector
    assert rf.call("S4S4", fu.Result("S4", (3, 3)).desc, m34.dv(), m34.dv()) == c["FESCICNF"]  # (3,4) x (3,4)
    assert rf.call("S4S4", fu.Result("S4", (2,)).desc, m34.dv(), v.dv()) == c["FESCICNF"]      # result extent
    assert rf.call("I2I4", fu.Result("I4", (3, 3)).desc, fu.Operand("I2", (3, 4), rng).dv(),
                   fu.Operand("I4", (3, 4), rng).dv()) == c["FESCICNF"]


@pytest.mark.parametrize("name", rf.DISPATCHED)
def test_rank_dispatchers_without_a_blas(front, name):
    """MATMUL_<A><B>dispatch.c with no BLAS bound: the dot-product loops of mmx_fort.h."""
    ka, kb = rf.split_kinds(name)
    kr = rf.result_kind(ka, kb)
    rng = np.random.default_rng(11)
    for case in ("mm", "mv", "vm"):
        sa, sb, sr = fu.shapes_for(case, 7, 5, 6)
        a, b = fu.Operand(ka, sa, rng, "section"), fu.Operand(kb, sb, rng, "dense")
        r = fu.Result(kr, sr, associated=False)
        r.desc.flags1 = len(sr) << 29
        assert rf.call(name, r.desc, a.dv(), b.dv(), dispatched=True) == 0
        assert fu.close(r.values(), fu.expected(a, b, kr), kr), f"{name} {case}"
    bad = fu.Result(kr, (3,), associated=False)
    v = fu.Operand(ka, (3,), rng)
    assert rf.call(name, bad.desc, v.dv(), fu.Operand(kb, (3,), rng).dv(), dispatched=True) == rf.codes()["FESCIRNK"]


def test_blas_hook_binds_the_engines_symbols(front):
    """mmx_dlutil.c as the reference ships it: with F90_MATMUL_BLAS set, __f90_open_blas_lib() looks
    sgemm_, dgemm_, cgemm_ and zgemm_ up in the process (dlopen(NULL) + dlsym) before any libblas;
    with libo64gemm.so loaded into the global scope (what LD_PRELOAD does) they must be the engine's.
    A process of its own: the hook resolves once per process."""
    if not rf.available("engine"):
        pytest.skip("libfi_front_engine.so is not built")
    prog = textwrap.dedent(f"""
        import ctypes, os
        eng = ctypes.CDLL({LIB_PATH!r}, mode=ctypes.RTLD_GLOBAL)
        front = ctypes.CDLL({rf._LIBS['engine']!r})
        names = ("sgemm", "dgemm", "cgemm", "zgemm")
        ptr = lambda n: ctypes.c_void_p.in_dll(front, "__f90_" + n + "_blas").value
        assert all(ptr(n) is None for n in names), "bound before the hook ran"
        front.__f90_open_blas_lib()
        if os.environ.get("F90_MATMUL_BLAS"):
            for n in names:
                want = ctypes.cast(getattr(eng, n + "_"), ctypes.c_void_p).value
                assert ptr(n) == want, n + "_ resolved elsewhere"
        else:
            assert all(ptr(n) is None for n in names), "bound although F90_MATMUL_BLAS is unset"
        print("ok")
    """)
    for env_on in (True, False):
        env = dict(os.environ)
        env.pop("F90_MATMUL_BLAS", None)
        if env_on:
            env["F90_MATMUL_BLAS"] = "1"
        r = subprocess.run([sys.executable, "-c", prog], capture_output=True, text=True, env=env, cwd=ROOT)
        assert r.returncode == 0 and r.stdout.strip() == "ok", r.stdout + r.stderr


@pytest.mark.parametrize("name", ["S4S4", "SS", "I1I4", "JI2", "C4S", "LL1"])
def test_zero_sized_result_needs_no_device(front, name):
    """A(0,k) x B(k,n): both the reference wrapper and the engine's entry point return before any
    kernel would run, so the RESULT descriptors can be compared on a machine without a GPU."""
    import open64_b200 as o
    ka, kb = rf.split_kinds(name)
    kr = rf.result_kind(ka, kb)
    rng = np.random.default_rng(3)
    a, b = fu.Operand(ka, (0, 5), rng), fu.Operand(kb, (5, 4), rng)
    r_ref, r_eng = fu.Result(kr, (0, 4), associated=False), fu.Result(kr, (0, 4), associated=False)
    assert rf.call(name, r_ref.desc, a.dv(), b.dv()) == 0
    A, B = a.dv(), b.dv()
    getattr(o.lib(), "_MATMUL_" + name)(ctypes.byref(r_eng.desc), ctypes.byref(A), ctypes.byref(B))
    assert o.lib().o64_compat_last_status() == o.OK
    # all words but the address: with nothing to allocate the reference stores an uninitialised
    # MatrixDimenType.C (matmul.h:252-262 skips the malloc), the engine stores NULL
    assert r_ref.descriptor_words()[:7] == r_eng.descriptor_words()[:7]
    assert not r_eng.desc.ptr


def test_result_without_element_length_gets_the_entry_points_kind(built):
    """An unassociated REAL*8 RESULT whose type word carries no length: the engine sizes it from the
    entry point's result kind and records that length, so strides are read back with the same unit."""
    import open64_b200 as o
    rng = np.random.default_rng(4)
    a, b = fu.Operand("S", (0, 3), rng), fu.Operand("S", (3, 2), rng)
    r = fu.Result("S", (0, 2), associated=False)
    r.desc.type_bits = DopeVector.TYPE_REAL            # int_len = 0
    A, B = a.dv(), b.dv()
    o.lib()._MATMUL_SS(ctypes.byref(r.desc), ctypes.byref(A), ctypes.byref(B))
    assert o.lib().o64_compat_last_status() == o.OK
    assert (r.desc.type_bits >> 12) & 0xfff == 64
    assert r.desc.dimension[0].stride_mult == 2 and r.desc.dimension[1].stride_mult == 0


@pytest.mark.parametrize("kind", ["S4", "S", "C4", "C", "I4", "J", "L4", "L"])
def test_predot_reads_vectors_as_the_engine_does(front, kind):
    """_PREDOT (osprey/libfi/dotprod/predot@.c, compiled from the reference tree): length, addresses
    and element strides of two rank-1 dope vectors built the way the engine's tests build them."""
    rng = np.random.default_rng(2)
    a, b = fu.Operand(kind, (37,), rng, "section"), fu.Operand(kind, (37,), rng, "dense")
    n, lx, ix, ly, iy = (ctypes.c_long() for _ in range(5))
    A, B = a.dv(), b.dv()
    rf.lib().ref_PREDOT(ctypes.byref(A), ctypes.byref(B), ctypes.byref(n), ctypes.byref(lx), ctypes.byref(ix),
                        ctypes.byref(ly), ctypes.byref(iy))
    assert (n.value, ix.value, iy.value) == (37, a.inc[0], b.inc[0])
    assert lx.value == a.storage.ctypes.data and ly.value == b.storage.ctypes.data
