"""Loads libo64gemm.so (built in-tree by ``open64_b200.build``) and declares its C ABI.

There is no fallback: if the library is missing the import fails with instructions, and every
compute call needs a B200.  Prototypes follow ``include/o64gemm.h``.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# O64_LIBRARY: another build of the same library (the -DO64_TUNING one, for instance)
LIB_PATH = os.environ.get("O64_LIBRARY") or os.path.join(_HERE, "libo64gemm.so")

OK = 0
ERR_RANK, ERR_CONFORM, ERR_NOMEM, ERR_ALIGN, ERR_DTYPE, ERR_TIMEOUT, ERR_CUDA, ERR_NCCL = range(-1, -9, -1)
ACT_NONE, ACT_RELU, ACT_GELU_TANH, ACT_GELU_ERF, ACT_SILU = range(5)
KIND_F32, KIND_BF16, KIND_FP8, KIND_S8 = range(4)
GATHER_NONE, GATHER_ROWMAJOR, GATHER_SLABS, GATHER_PUSH = range(4)
OUT_BF16, OUT_S8, OUT_E4M3 = range(3)
UNIQUE_ID_BYTES = 128
STATIC_SCRATCH_BYTES = 16 << 20

# every symbol include/o64gemm.h declares
EXPORTS = [
    "o64_create", "o64_destroy", "o64_last_status", "o64_set_wait_budget_us", "o64_test_gemm_bf16_withheld", "o64_test_last_tail_split", "o64_test_force_tail_split", "o64_status_string", "o64_version",
    "o64_plan_get", "o64_plan_set", "o64_plan_model", "o64_plan_tune", "o64_plan_tune_clear", "o64_plan_save", "o64_plan_load", "o64_plan_count", "o64_linear_f32", "o64_gemm_bf16", "o64_gemm_bf16_swiglu",
    "o64_gemm_fp8_scaled", "o64_gemm_fp8_scaled_ex", "o64_gemm_fp8_scaled_kn", "o64_gemm_s8_scaled", "o64_gemm_s8s8_s32", "o64_gemm_s8s8_s32_static", "o64_naive_gemm", "o64_comm_unique_id",
    "o64_comm_init", "o64_comm_destroy", "o64_comm_alloc_result", "o64_gemm_s8_sharded_workspace", "o64_gemm_s8_sharded", "o64_gemm_bf16_sharded",
    "sgemm_", "_s4gemmx__", "_s4gemvx__", "_MATMUL_S4S4", "o64_compat_last_status", "o64_compat_handle",
    "dgemm_", "_sgemmx__", "_sgemvx__", "_MATMUL_SS",
    "_i1gemmx__", "_i1i2gemmx__", "_i1i4gemmx__", "_i1jgemmx__", "_i2gemmx__", "_i2i4gemmx__", "_i2jgemmx__",
    "_i4gemmx__", "_i4jgemmx__", "_jgemmx__",
    "_MATMUL_I1I1", "_MATMUL_I1I2", "_MATMUL_I1I4", "_MATMUL_I1J", "_MATMUL_I2I1", "_MATMUL_I2I2", "_MATMUL_I2I4",
    "_MATMUL_I2J", "_MATMUL_I4I1", "_MATMUL_I4I2", "_MATMUL_I4I4", "_MATMUL_I4J", "_MATMUL_JI1", "_MATMUL_JI2",
    "_MATMUL_JI4", "_MATMUL_JJ",
    "_l1gemmx__", "_l1l2gemmx__", "_l1l4gemmx__", "_l1lgemmx__", "_l2gemmx__", "_l2l4gemmx__", "_l2lgemmx__", "_l4gemmx__", "_l4lgemmx__", "_lgemmx__",
    "_MATMUL_L1L1", "_MATMUL_L1L2", "_MATMUL_L1L4", "_MATMUL_L1L", "_MATMUL_L2L1", "_MATMUL_L2L2", "_MATMUL_L2L4", "_MATMUL_L2L",
    "_MATMUL_L4L1", "_MATMUL_L4L2", "_MATMUL_L4L4", "_MATMUL_L4L", "_MATMUL_LL1", "_MATMUL_LL2", "_MATMUL_LL4", "_MATMUL_LL",
    "_c4gemmx__", "_cgemmx__", "_c4gemvx__", "_cgemvx__", "cgemm_", "zgemm_", "_MATMUL_C4C4", "_MATMUL_CC",
    "_s4sgemmx__", "_i1s4gemmx__", "_i2s4gemmx__", "_i4s4gemmx__", "_js4gemmx__", "_i1sgemmx__", "_i2sgemmx__", "_i4sgemmx__", "_jsgemmx__",
    "_MATMUL_S4S", "_MATMUL_SS4", "_MATMUL_I1S4", "_MATMUL_S4I1", "_MATMUL_I1S", "_MATMUL_SI1", "_MATMUL_I2S4", "_MATMUL_S4I2", "_MATMUL_I2S", "_MATMUL_SI2", "_MATMUL_I4S4", "_MATMUL_S4I4", "_MATMUL_I4S", "_MATMUL_SI4", "_MATMUL_JS4", "_MATMUL_S4J", "_MATMUL_JS", "_MATMUL_SJ",
    "_MATMUL_C4S4", "_MATMUL_S4C4", "_MATMUL_C4S", "_MATMUL_SC4", "_MATMUL_CS4", "_MATMUL_S4C", "_MATMUL_CS", "_MATMUL_SC", "_MATMUL_C4C",
    "_MATMUL_CC4", "_MATMUL_C4I1", "_MATMUL_C4I2", "_MATMUL_C4I4", "_MATMUL_C4J", "_MATMUL_I1C4", "_MATMUL_I2C4", "_MATMUL_I4C4", "_MATMUL_JC4",
    "_MATMUL_CI1", "_MATMUL_CI2", "_MATMUL_CI4", "_MATMUL_CJ", "_MATMUL_I1C", "_MATMUL_I2C", "_MATMUL_I4C", "_MATMUL_JC",
    "_DOT_S4S4", "_DOT_SS", "_DOT_S4S", "_DOT_SS4", "_DOT_I4I4", "_DOT_JJ", "_DOT_I4J", "_DOT_JI4", "_DOT_I4S4", "_DOT_S4I4",
    "_DOT_I4S", "_DOT_SI4", "_DOT_JS4", "_DOT_S4J", "_DOT_JS", "_DOT_SJ", "_DOT_L4L4", "_DOT_LL", "_DOT_L4L", "_DOT_LL4",
    "_DOT_C4C4", "_DOT_CC",
]


class Complex8(ctypes.Structure):
    _fields_ = [("re", ctypes.c_float), ("im", ctypes.c_float)]


class Complex16(ctypes.Structure):
    _fields_ = [("re", ctypes.c_double), ("im", ctypes.c_double)]


# result type of each DOT_PRODUCT entry point
DOT_RESTYPE = {
    "_DOT_S4S4": ctypes.c_float, "_DOT_SS": ctypes.c_double, "_DOT_S4S": ctypes.c_double, "_DOT_SS4": ctypes.c_double,
    "_DOT_I4I4": ctypes.c_int32, "_DOT_JJ": ctypes.c_int64, "_DOT_I4J": ctypes.c_int64, "_DOT_JI4": ctypes.c_int64,
    "_DOT_I4S4": ctypes.c_float, "_DOT_S4I4": ctypes.c_float, "_DOT_I4S": ctypes.c_double, "_DOT_SI4": ctypes.c_double,
    "_DOT_JS4": ctypes.c_float, "_DOT_S4J": ctypes.c_float, "_DOT_JS": ctypes.c_double, "_DOT_SJ": ctypes.c_double,
    "_DOT_L4L4": ctypes.c_int32, "_DOT_LL": ctypes.c_int64, "_DOT_L4L": ctypes.c_int64, "_DOT_LL4": ctypes.c_int64,
    "_DOT_C4C4": Complex8, "_DOT_CC": Complex16,
}


class Plan(ctypes.Structure):
    _fields_ = [
        ("kind", ctypes.c_int), ("tile_m", ctypes.c_int), ("tile_n", ctypes.c_int),
        ("tile_k", ctypes.c_int), ("stages", ctypes.c_int), ("cta_group", ctypes.c_int),
        ("group_m", ctypes.c_int), ("raster", ctypes.c_int), ("mma_m", ctypes.c_int),
        ("mma_n", ctypes.c_int), ("mma_k", ctypes.c_int), ("num_ctas", ctypes.c_int),
        ("split_k", ctypes.c_int), ("predicted_ms", ctypes.c_double),
    ]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


class DvDimen(ctypes.Structure):
    _fields_ = [("low_bound", ctypes.c_long), ("extent", ctypes.c_long), ("stride_mult", ctypes.c_long)]


class DopeVector(ctypes.Structure):
    """o64_dopevec_t: the reference's DopeVectorType on x86-64 (osprey/clibinc/cray/dopevec.h:212-334)."""
    _fields_ = [("ptr", ctypes.c_void_p), ("el_len", ctypes.c_ulong), ("flags0", ctypes.c_uint32),
                ("flags1", ctypes.c_uint32), ("type_pad", ctypes.c_uint32), ("type_bits", ctypes.c_uint32),
                ("orig_base", ctypes.c_void_p), ("orig_size", ctypes.c_ulong), ("dimension", DvDimen * 7)]

    TYPE_LOGICAL = 5
    TYPE_INTEGER, TYPE_REAL, TYPE_COMPLEX = 2, 3, 4  # osprey/clibinc/cray/dopevec.h: DVTYPE_INTEGER, _REAL, _COMPLEX

    @classmethod
    def make(cls, ptr, extents, strides, bits=32, type_code=3, assoc=True):
        """An array descriptor: extents and ELEMENT strides per dimension; `bits` is the element
        length (stride_mult is stored in 32-bit words for 64-bit elements, as the runtime expects)."""
        d = cls()
        d.ptr = ptr
        d.el_len = bits
        d.flags0 = 1 if assoc else 0
        d.flags1 = len(extents) << 29
        d.type_bits = type_code | (bits << 12)
        d.orig_base = ptr
        for i, (e, s) in enumerate(zip(extents, strides)):
            d.dimension[i].low_bound = 1
            d.dimension[i].extent = e
            d.dimension[i].stride_mult = s * max(bits // 32, 1)
        return d

    @classmethod
    def real4(cls, ptr, extents, strides, assoc=True):
        """A REAL*4 array descriptor: extents and element strides per dimension."""
        return cls.make(ptr, extents, strides, 32, cls.TYPE_REAL, assoc)


class Epilogue(ctypes.Structure):
    _fields_ = [("bias", ctypes.c_void_p), ("act", ctypes.c_int)]


class O64Error(RuntimeError):
    def __init__(self, status, where=""):
        self.status = status
        msg = lib().o64_status_string(status).decode()
        super().__init__(f"{where}: {msg} ({status})" if where else f"{msg} ({status})")


_lib = None


def lib():
    """The loaded library.  Raises if it has not been built: there is no other code path."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m open64_b200.build` "
            "(nvcc, sm_100a).  open64_b200 has no CPU or eager fallback.")
    L = ctypes.CDLL(LIB_PATH)
    vp, i64, ci, cf = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
    pi, pf = ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_float)
    L.o64_create.argtypes = [ctypes.POINTER(vp), ci]
    L.o64_destroy.argtypes = [vp]
    L.o64_last_status.argtypes = [vp, vp, pi]
    L.o64_status_string.argtypes = [ci]
    L.o64_test_last_tail_split.argtypes = [pi, pi]
    L.o64_test_force_tail_split.argtypes = [ci]
    L.o64_set_wait_budget_us.argtypes = [vp, i64]
    L.o64_test_gemm_bf16_withheld.argtypes = [vp, i64, i64, i64, vp, i64, vp, i64, vp, i64, ci, vp]
    L.o64_status_string.restype = ctypes.c_char_p
    L.o64_version.restype = ctypes.c_char_p
    L.o64_plan_get.argtypes = [vp, ci, i64, i64, i64, ctypes.POINTER(Plan)]
    L.o64_plan_set.argtypes = [vp, ci, ctypes.POINTER(Plan)]
    L.o64_plan_tune.argtypes = [vp, ci, ci, i64, i64, i64, vp, ctypes.POINTER(Plan)]
    L.o64_plan_tune_clear.argtypes = [vp]
    L.o64_plan_save.argtypes = [vp, ctypes.c_char_p]
    L.o64_plan_load.argtypes = [vp, ctypes.c_char_p]
    L.o64_plan_count.argtypes = [vp]
    L.o64_plan_model.argtypes = [ci, ci, i64, i64, i64, ci, ctypes.POINTER(Plan), ctypes.POINTER(Plan)]
    L.o64_linear_f32.argtypes = [vp, i64, i64, i64, vp, i64, vp, i64, vp, vp, i64, ci, vp]
    L.o64_gemm_bf16.argtypes = [vp, i64, i64, i64, vp, i64, vp, i64, ci, vp, i64,
                                ctypes.POINTER(Epilogue), vp]
    L.o64_gemm_bf16_swiglu.argtypes = [vp, i64, i64, i64, vp, i64, vp, vp, i64, vp, i64, vp]
    L.o64_gemm_fp8_scaled.argtypes = [vp, i64, i64, i64, vp, i64, vp, i64, vp, vp, vp, vp, i64, vp]
    L.o64_gemm_s8s8_s32.argtypes = [vp, i64, i64, i64, vp, i64, vp, i64, vp, i64, vp]
    L.o64_gemm_fp8_scaled_ex.argtypes = [vp, i64, i64, i64, vp, i64, vp, i64, vp, vp, vp, ci, vp, i64, ci, vp]
    L.o64_gemm_fp8_scaled_kn.argtypes = [vp, i64, i64, i64, vp, i64, vp, i64, vp, vp, vp, ci, vp, i64, ci, vp]
    L.o64_gemm_s8_scaled.argtypes = [vp, i64, i64, i64, vp, i64, vp, i64, vp, vp, vp, ci, vp, i64, ci, vp]
    L.o64_gemm_s8s8_s32_static.argtypes = [i64, i64, i64, vp, i64, vp, i64, vp, i64, vp]
    L.o64_naive_gemm.argtypes = [vp, ci, i64, i64, i64, vp, i64, vp, i64, ci, vp, vp, vp, ci, vp,
                                 i64, vp]
    L.o64_comm_unique_id.argtypes = [vp]
    L.o64_comm_init.argtypes = [vp, vp, ci, ci]
    L.o64_comm_destroy.argtypes = [vp]
    L.o64_comm_alloc_result.argtypes = [vp, ctypes.c_size_t, ctypes.POINTER(vp)]
    L.o64_gemm_s8_sharded_workspace.argtypes = [i64, i64, ci, ci]
    L.o64_gemm_s8_sharded_workspace.restype = ctypes.c_size_t
    L.o64_gemm_s8_sharded.argtypes = [vp, i64, i64, i64, vp, i64, vp, i64, vp, ci, vp, vp]
    L.o64_gemm_bf16_sharded.argtypes = [vp, i64, i64, i64, vp, i64, vp, i64, vp, ci, ctypes.POINTER(Epilogue), vp]
    L.sgemm_.argtypes = [ctypes.c_char_p, ctypes.c_char_p, pi, pi, pi, pf, vp, pi, vp, pi, pf, vp, pi]
    L.sgemm_.restype = None
    L._s4gemmx__.argtypes = [pi, pi, pi, pf, vp, pi, pi, vp, pi, pi, pf, vp, pi, pi]
    L._s4gemmx__.restype = None
    L._s4gemvx__.argtypes = [pi, pi, pf, vp, pi, pi, vp, pi, pf, vp, pi]
    L._s4gemvx__.restype = None
    L.dgemm_.argtypes = [ctypes.c_char_p, ctypes.c_char_p, pi, pi, pi, vp, vp, pi, vp, pi, vp, vp, pi]
    L.dgemm_.restype = None
    for name in [e for e in EXPORTS if e.endswith("gemmx__") and e != "_s4gemmx__"]:
        getattr(L, name).argtypes = [pi, pi, pi, vp, vp, pi, pi, vp, pi, pi, vp, vp, pi, pi]
        getattr(L, name).restype = None
    L._sgemvx__.argtypes = [pi, pi, vp, vp, pi, pi, vp, pi, vp, vp, pi]
    L._sgemvx__.restype = None
    for name in ("_c4gemmx__", "_cgemmx__"):  # two conjugation flags in front
        getattr(L, name).argtypes = [pi, pi, pi, pi, pi, vp, vp, pi, pi, vp, pi, pi, vp, vp, pi, pi]
    for name in ("_c4gemvx__", "_cgemvx__"):
        getattr(L, name).argtypes = [pi, pi, pi, vp, vp, pi, pi, vp, pi, vp, vp, pi]
        getattr(L, name).restype = None
    for name in ("cgemm_", "zgemm_"):
        getattr(L, name).argtypes = [ctypes.c_char_p, ctypes.c_char_p, pi, pi, pi, vp, vp, pi, vp, pi, vp, vp, pi]
        getattr(L, name).restype = None
    for name in [e for e in EXPORTS if e.startswith("_MATMUL_")]:
        getattr(L, name).argtypes = [ctypes.POINTER(DopeVector)] * 3
        getattr(L, name).restype = None
    for name, rt in DOT_RESTYPE.items():
        getattr(L, name).argtypes = [ctypes.POINTER(DopeVector)] * 2
        getattr(L, name).restype = rt
    L.o64_compat_last_status.restype = ci
    L.o64_compat_handle.restype = vp
    _lib = L
    return L


def check(status, where=""):
    if status != OK:
        raise O64Error(status, where)
