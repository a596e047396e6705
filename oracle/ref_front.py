"""The reference's own C front half of MATMUL, built from its sources into ``oracle/_ref/``.

Test infrastructure only (nothing under ``open64_b200`` imports this).  ``ref_front.mk`` compiles
the unmodified wrappers ``osprey/libfi/matrix/matmul_<a><b>.c`` (``_premult`` of ``matmul.h:135-400``
plus the kernel call), the rank dispatchers ``MATMUL_*dispatch.c`` and the BLAS hook
``mmx_dlutil.c`` where they lie in the reference tree, renames their entry points
(``ref_MATMUL_S4S4``, ``refdisp_MATMUL_S4S4``) and binds the strided kernels they call either to the
CPU oracle (``backend="oracle"``, runs anywhere) or to the engine's Fortran-ABI kernels
(``backend="engine"``, needs a B200).  The reference's arithmetic kernels are Fortran and cannot
be built here, so this pins the boundary (dope vectors, RESULT allocation, conformance errors,
operand exchange of mixed kinds, the ``dlsym`` BLAS hook), not the arithmetic.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_OUT = os.path.join(_HERE, "_ref")
_LIBS = {"oracle": os.path.join(_OUT, "libfi_front_oracle.so"),
         "engine": os.path.join(_OUT, "libfi_front_engine.so")}
REFERENCE_ROOT = os.environ.get("O64_REFERENCE_ROOT", "/root/reference")

# element kinds in the runtime's naming: letter -> (numpy dtype, dope-vector type code, bits)
KINDS = {
    "S4": (np.float32, 3, 32), "S": (np.float64, 3, 64), "C4": (np.complex64, 4, 64), "C": (np.complex128, 4, 128),
    "I1": (np.int8, 2, 8), "I2": (np.int16, 2, 16), "I4": (np.int32, 2, 32), "J": (np.int64, 2, 64),
    "L1": (np.int8, 5, 8), "L2": (np.int16, 5, 16), "L4": (np.int32, 5, 32), "L": (np.int64, 5, 64),
}
ENTRY_POINTS = (
    "S4S4 SS C4C4 CC S4S SS4 "
    "I1I1 I1I2 I1I4 I1J I2I1 I2I2 I2I4 I2J I4I1 I4I2 I4I4 I4J JI1 JI2 JI4 JJ "
    "I1S4 S4I1 I1S SI1 I2S4 S4I2 I2S SI2 I4S4 S4I4 I4S SI4 JS4 S4J JS SJ "
    "C4S4 S4C4 C4S SC4 CS4 S4C CS SC C4C CC4 C4I1 C4I2 C4I4 C4J I1C4 I2C4 I4C4 JC4 CI1 CI2 CI4 CJ I1C I2C I4C JC "
    "L1L1 L1L2 L1L4 L1L L2L1 L2L2 L2L4 L2L L4L1 L4L2 L4L4 L4L LL1 LL2 LL4 LL").split()
DISPATCHED = "S4S4 S4S SS4 SS C4C4 C4C CC4 CC C4S4 S4C4 C4S SC4 CS4 S4C CS SC".split()


def split_kinds(name):
    """'I2S4' -> ('I2', 'S4')."""
    for cut in (2, 1):
        a, b = name[:cut], name[cut:]
        if a in KINDS and b in KINDS:
            return a, b
    raise ValueError(name)


def result_kind(a, b):
    """Kind of MATMUL's result for operand kinds a, b (osprey/crayf90/fe90/intrin.h:4185-4440)."""
    if a[0] == "L":
        return a if KINDS[a][2] >= KINDS[b][2] else b
    cx = a[0] == "C" or b[0] == "C"
    ints = [k for k in (a, b) if k[0] in "IJ"]
    if len(ints) == 2:
        return a if KINDS[a][2] >= KINDS[b][2] else b
    comp_bits = max(32 if k in ("S4", "C4") else 64 for k in (a, b) if k[0] not in "IJ")
    if cx:
        return "C4" if comp_bits == 32 else "C"
    return "S4" if comp_bits == 32 else "S"


def reference_present():
    return os.path.isdir(os.path.join(REFERENCE_ROOT, "osprey", "libfi", "matrix"))


def build(force=False):
    """Runs ref_front.mk when the reference tree is on this machine; otherwise the files built
    earlier (they travel with the repository's other built libraries) are used as they are."""
    if not reference_present():
        return available()
    cmd = ["make", "-s", "-f", os.path.join(_HERE, "ref_front.mk"), f"REF={REFERENCE_ROOT}", "-j8"]
    if force:
        cmd.append("-B")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("ref_front.mk failed:\n" + r.stdout + r.stderr)
    return available()


def available(backend="oracle"):
    return os.path.exists(_LIBS[backend])


_loaded = {}


def lib(backend="oracle"):
    if backend not in _loaded:
        if not available(backend):
            raise RuntimeError(f"{_LIBS[backend]} is not built (make -f oracle/ref_front.mk needs the reference tree)")
        L = ctypes.CDLL(_LIBS[backend])
        L.o64front_call.argtypes = [ctypes.c_void_p] * 4
        L.o64front_call.restype = ctypes.c_int
        L.o64front_code.argtypes = [ctypes.c_int]
        L.o64front_dv_sizeof.restype = ctypes.c_long
        L.o64front_dv_probe.argtypes = [ctypes.c_int, ctypes.c_void_p]
        _loaded[backend] = L
    return _loaded[backend]


def codes(backend="oracle"):
    L = lib(backend)
    return {"FESCIRNK": L.o64front_code(0), "FESCICNF": L.o64front_code(1), "FENOMEMY": L.o64front_code(2)}


def call(name, R, A, B, backend="oracle", dispatched=False):
    """Runs the reference's ``_MATMUL_<name>`` (the wrapper, or the rank dispatcher in front of the
    BLAS hook) on three dope vectors (ctypes structures); returns 0 or the code the runtime would
    have aborted with."""
    L = lib(backend)
    fn = getattr(L, ("refdisp_MATMUL_" if dispatched else "ref_MATMUL_") + name)
    return L.o64front_call(ctypes.cast(fn, ctypes.c_void_p), ctypes.addressof(R), ctypes.addressof(A),
                           ctypes.addressof(B))


def dv_probe(which, backend="oracle"):
    L = lib(backend)
    buf = (ctypes.c_ubyte * L.o64front_dv_sizeof())()
    if L.o64front_dv_probe(which, buf) != 0:
        raise ValueError(which)
    return bytes(buf)
