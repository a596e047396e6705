"""ctypes bindings of the CPU oracle (``gemm_ref.c``) over numpy arrays.

Test infrastructure only; the shipped package never imports this module.  bf16 values are
carried as ``uint16`` bit patterns and e4m3 values as ``uint8`` bit patterns.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libo64ref.so")

ACT_NONE, ACT_RELU, ACT_GELU_TANH, ACT_GELU_ERF, ACT_SILU = range(5)

__all__ = [
    "ACT_NONE", "ACT_RELU", "ACT_GELU_TANH", "ACT_GELU_ERF", "ACT_SILU", "build", "lib",
    "linear_f32", "linear_f32_acc64", "gemm_bf16", "swiglu_bf16", "gemm_fp8_scaled",
    "gemm_s8s8_s32", "gemm_s8_scaled", "gemm_fp8_scaled_ex", "s4gemmx", "s4gemvx", "xgemmx", "sgemvx_f64", "cgemmx", "cgemvx", "lgemmx", "internal_mm_f32", "bf16_to_f32", "f32_to_bf16",
    "e4m3_to_f32", "f32_to_e4m3", "num_threads", "set_num_threads",
]


def build(force=False):
    """Compile ``gemm_ref.c`` with the Makefile beside it (gcc, a second or two)."""
    src = os.path.join(_HERE, "gemm_ref.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _c(a, dt):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


L = ctypes.c_long
I = ctypes.c_int
F = ctypes.c_float


def linear_f32(A, B, bias=None, act=ACT_NONE, transB=False, acc64=False):
    """act(A @ B + bias) by the compiler's loop nest; B is [K,N], or [N,K] when transB."""
    A = _c(A, np.float32)
    B = _c(B, np.float32)
    bias = _c(bias, np.float32) if bias is not None else None
    M, K = A.shape
    N = B.shape[0] if transB else B.shape[1]
    assert (B.shape[1] if transB else B.shape[0]) == K
    Y = np.empty((M, N), np.float32)
    fn = lib().o64ref_linear_f32_acc64 if acc64 else lib().o64ref_linear_f32
    fn(L(M), L(N), L(K), _p(A), L(A.shape[1]), _p(B), L(B.shape[1]), I(int(transB)), _p(bias),
       _p(Y), L(N), I(act))
    return Y


def linear_f32_acc64(A, B, bias=None, act=ACT_NONE, transB=False):
    return linear_f32(A, B, bias, act, transB, acc64=True)


def gemm_bf16(A, B, bias=None, act=ACT_NONE, transB=True):
    """fp32 nest on bf16 bit patterns (uint16); returns fp32."""
    A = _c(A, np.uint16)
    B = _c(B, np.uint16)
    bias = _c(bias, np.float32) if bias is not None else None
    M, K = A.shape
    N = B.shape[0] if transB else B.shape[1]
    assert (B.shape[1] if transB else B.shape[0]) == K
    C = np.empty((M, N), np.float32)
    lib().o64ref_gemm_bf16(L(M), L(N), L(K), _p(A), L(K), _p(B), L(B.shape[1]), I(int(transB)),
                           _p(bias), _p(C), L(N), I(act))
    return C


def swiglu_bf16(X, Wg, Wu):
    """bf16(silu(X@Wg) * (X@Wu)); X [M,K], Wg/Wu [K,N]; uint16 in, uint16 out."""
    X = _c(X, np.uint16)
    Wg = _c(Wg, np.uint16)
    Wu = _c(Wu, np.uint16)
    M, K = X.shape
    N = Wg.shape[1]
    assert Wg.shape == Wu.shape == (K, N)
    H = np.empty((M, N), np.uint16)
    lib().o64ref_swiglu_bf16(L(M), L(N), L(K), _p(X), L(K), _p(Wg), _p(Wu), L(N), _p(H), L(N))
    return H


def gemm_fp8_scaled(A8, B8, scaleA=None, scaleB=None, bias=None):
    """(A8*sA) @ (B8*sB)^T + bias in fp32; A8 [M,K], B8 [N,K] as e4m3 bit patterns."""
    A8 = _c(A8, np.uint8)
    B8 = _c(B8, np.uint8)
    M, K = A8.shape
    N = B8.shape[0]
    assert B8.shape[1] == K
    sA = _c(scaleA, np.float32) if scaleA is not None else None
    sB = _c(scaleB, np.float32) if scaleB is not None else None
    bias = _c(bias, np.float32) if bias is not None else None
    C = np.empty((M, N), np.float32)
    lib().o64ref_gemm_fp8_scaled(L(M), L(N), L(K), _p(A8), L(K), _p(B8), L(K), _p(sA), _p(sB),
                                 _p(bias), _p(C), L(N))
    return C


def gemm_s8s8_s32(A, B):
    """A [M,K] int8 times B [N,K]^T int8 -> int32, exact."""
    A = _c(A, np.int8)
    B = _c(B, np.int8)
    M, K = A.shape
    N = B.shape[0]
    assert B.shape[1] == K
    C = np.empty((M, N), np.int32)
    lib().o64ref_gemm_s8s8_s32(L(M), L(N), L(K), _p(A), L(K), _p(B), L(K), _p(C), L(N))
    return C


_OUT_DT = {0: np.float32, 1: np.int8, 2: np.uint8, 3: np.uint16}


def gemm_s8_scaled(A, B, scaleA=None, scaleB=None, bias=None, act=ACT_NONE, out_kind=0):
    """convert(act(float(A @ B^T) * (sA[m] * sB[n]) + bias[n])), int8 operands; out_kind 0 = fp32 value,
    1 = int8 (nearest even, saturating), 3 = bf16 bits."""
    A = _c(A, np.int8)
    B = _c(B, np.int8)
    M, K = A.shape
    N = B.shape[0]
    assert B.shape[1] == K
    sA = _c(scaleA, np.float32) if scaleA is not None else None
    sB = _c(scaleB, np.float32) if scaleB is not None else None
    bias = _c(bias, np.float32) if bias is not None else None
    C = np.empty((M, N), _OUT_DT[out_kind])
    lib().o64ref_gemm_s8_scaled(L(M), L(N), L(K), _p(A), L(K), _p(B), L(K), _p(sA), _p(sB), _p(bias), I(act),
                                I(out_kind), _p(C), L(N))
    return C


def gemm_fp8_scaled_ex(A8, B8, scaleA=None, scaleB=None, bias=None, act=ACT_NONE, out_kind=0):
    """The same tail on the fp32 nest over e4m3 bit patterns; out_kind 0 = fp32 value, 2 = e4m3 bits
    (nearest even, saturating), 3 = bf16 bits."""
    A8 = _c(A8, np.uint8)
    B8 = _c(B8, np.uint8)
    M, K = A8.shape
    N = B8.shape[0]
    assert B8.shape[1] == K
    sA = _c(scaleA, np.float32) if scaleA is not None else None
    sB = _c(scaleB, np.float32) if scaleB is not None else None
    bias = _c(bias, np.float32) if bias is not None else None
    C = np.empty((M, N), _OUT_DT[out_kind])
    lib().o64ref_gemm_fp8_scaled_ex(L(M), L(N), L(K), _p(A8), L(K), _p(B8), L(K), _p(sA), _p(sB), _p(bias), I(act),
                                    I(out_kind), _p(C), L(N))
    return C


def s4gemmx(M, N, K, alpha, A, inc1a, inc2a, B, inc1b, inc2b, beta, C, inc1c, inc2c):
    """The runtime's strided kernel, in place on the flat fp32 array C."""
    assert A.dtype == B.dtype == C.dtype == np.float32 and C.flags.c_contiguous
    lib().o64ref_s4gemmx(I(M), I(N), I(K), F(alpha), _p(np.ascontiguousarray(A)), I(inc1a),
                         I(inc2a), _p(np.ascontiguousarray(B)), I(inc1b), I(inc2b), F(beta),
                         _p(C), I(inc1c), I(inc2c))
    return C


def s4gemvx(M, N, alpha, A, inc1a, inc2a, X, incx, beta, Y, incy):
    assert A.dtype == X.dtype == Y.dtype == np.float32 and Y.flags.c_contiguous
    lib().o64ref_s4gemvx(I(M), I(N), F(alpha), _p(np.ascontiguousarray(A)), I(inc1a), I(inc2a),
                         _p(np.ascontiguousarray(X)), I(incx), F(beta), _p(Y), I(incy))
    return Y


_KIND = {np.dtype(np.int8): "i1", np.dtype(np.int16): "i2", np.dtype(np.int32): "i4", np.dtype(np.int64): "j"}
_UCT = {1: ctypes.c_uint8, 2: ctypes.c_uint16, 4: ctypes.c_uint32, 8: ctypes.c_uint64}


def xgemmx(M, N, K, alpha, A, inc1a, inc2a, B, inc1b, inc2b, beta, C, inc1c, inc2c):
    """The strided kernel for the element kinds of (A, C): the same kind throughout (float32,
    float64, int8 ... int64), an integer pair with A the narrower kind (i1i2gemmx ... i4jgemmx), or a
    REAL result with a narrower real or an integer A (s4sgemmx, i1s4gemmx ... jsgemmx); in place on
    the flat array C; integers wrap in the kind of C."""
    assert B.dtype == C.dtype and C.flags.c_contiguous
    kinds = dict(_KIND)
    kinds[np.dtype(np.float32)] = "s4"
    kinds[np.dtype(np.float64)] = "s"
    ka, kc = kinds[A.dtype], kinds[C.dtype]
    if C.dtype.kind == "f":
        conv = ctypes.c_float if C.dtype == np.float32 else ctypes.c_double
        name = "o64ref_sgemmx_f64" if (ka, kc) == ("s", "s") else "o64ref_%s%sgemmx" % (ka, "" if ka == kc else kc)
    else:
        assert A.dtype.kind == "i" and A.dtype.itemsize <= C.dtype.itemsize
        name = "o64ref_%s%sgemmx" % (ka, "" if ka == kc else kc)
        ct = _UCT[C.dtype.itemsize]
        mask = (1 << (8 * C.dtype.itemsize)) - 1
        conv = lambda v: ct(int(v) & mask)
    getattr(lib(), name)(I(M), I(N), I(K), conv(alpha), _p(np.ascontiguousarray(A)), I(inc1a), I(inc2a),
                         _p(np.ascontiguousarray(B)), I(inc1b), I(inc2b), conv(beta), _p(C), I(inc1c),
                         I(inc2c))
    return C


def sgemvx_f64(M, N, alpha, A, inc1a, inc2a, X, incx, beta, Y, incy):
    assert A.dtype == X.dtype == Y.dtype == np.float64 and Y.flags.c_contiguous
    D = ctypes.c_double
    lib().o64ref_sgemvx_f64(I(M), I(N), D(alpha), _p(np.ascontiguousarray(A)), I(inc1a), I(inc2a),
                            _p(np.ascontiguousarray(X)), I(incx), D(beta), _p(Y), I(incy))
    return Y


def _cpair(z, dt):
    return np.array([complex(z).real, complex(z).imag], dtype=dt)


def cgemmx(M, N, K, alpha, A, inc1a, inc2a, B, inc1b, inc2b, beta, C, inc1c, inc2c, conja=False, conjb=False):
    """The complex strided kernel (complex64: c4gemmx, complex128: cgemmx), in place on the flat
    array C; increments in complex elements."""
    assert A.dtype == B.dtype == C.dtype and C.dtype in (np.complex64, np.complex128) and C.flags.c_contiguous
    single = C.dtype == np.complex64
    rt = np.float32 if single else np.float64
    fn = lib().o64ref_c4gemmx if single else lib().o64ref_cgemmx
    al, be = _cpair(alpha, rt), _cpair(beta, rt)
    fn(I(int(conja)), I(int(conjb)), I(M), I(N), I(K), _p(al), _p(np.ascontiguousarray(A)), I(inc1a), I(inc2a),
       _p(np.ascontiguousarray(B)), I(inc1b), I(inc2b), _p(be), _p(C), I(inc1c), I(inc2c))
    return C


def cgemvx(M, N, alpha, A, inc1a, inc2a, X, incx, beta, Y, incy, conj=False):
    assert A.dtype == X.dtype == Y.dtype and Y.dtype in (np.complex64, np.complex128) and Y.flags.c_contiguous
    single = Y.dtype == np.complex64
    rt = np.float32 if single else np.float64
    fn = lib().o64ref_c4gemvx if single else lib().o64ref_cgemvx
    al, be = _cpair(alpha, rt), _cpair(beta, rt)
    fn(I(int(conj)), I(M), I(N), _p(al), _p(np.ascontiguousarray(A)), I(inc1a), I(inc2a),
       _p(np.ascontiguousarray(X)), I(incx), _p(be), _p(Y), I(incy))
    return Y


def lgemmx(M, N, K, alpha, A, inc1a, inc2a, B, inc1b, inc2b, beta, C, inc1c, inc2c):
    """The LOGICAL strided kernel for the integer carrier kinds of (A, C) (l1gemmx ... l4lgemmx, lgemmx)."""
    assert B.dtype == C.dtype and C.flags.c_contiguous and A.dtype.itemsize <= C.dtype.itemsize
    lk = {1: "l1", 2: "l2", 4: "l4", 8: "l"}
    ka, kc = lk[A.dtype.itemsize], lk[C.dtype.itemsize]
    name = "o64ref_%s%sgemmx" % (ka, "" if ka == kc else kc)
    getattr(lib(), name)(I(M), I(N), I(K), I(int(bool(alpha))), _p(np.ascontiguousarray(A)), I(inc1a), I(inc2a),
                         _p(np.ascontiguousarray(B)), I(inc1b), I(inc2b), I(int(bool(beta))), _p(C), I(inc1c), I(inc2c))
    return C


def internal_mm_f32(A_colmajor, B_colmajor, M, N, K):
    """Dot-product form on contiguous column-major operands; returns column-major R (flat)."""
    A = _c(A_colmajor, np.float32).ravel()
    B = _c(B_colmajor, np.float32).ravel()
    R = np.empty(M * N, np.float32)
    lib().o64ref_internal_mm_f32(I(M), I(N), I(K), _p(A), _p(B), _p(R))
    return R


def bf16_to_f32(a):
    a = _c(a, np.uint16)
    out = np.empty(a.shape, np.float32)
    lib().o64ref_bf16_to_f32(L(a.size), _p(a), _p(out))
    return out


def f32_to_bf16(a):
    a = _c(a, np.float32)
    out = np.empty(a.shape, np.uint16)
    lib().o64ref_f32_to_bf16(L(a.size), _p(a), _p(out))
    return out


def e4m3_to_f32(a):
    a = _c(a, np.uint8)
    out = np.empty(a.shape, np.float32)
    lib().o64ref_e4m3_to_f32(L(a.size), _p(a), _p(out))
    return out


def f32_to_e4m3(a):
    a = _c(a, np.float32)
    out = np.empty(a.shape, np.uint8)
    lib().o64ref_f32_to_e4m3(L(a.size), _p(a), _p(out))
    return out


def num_threads():
    return int(lib().o64ref_num_threads())


def set_num_threads(n):
    """Overrides OMP_NUM_THREADS for the oracle's loops (0 or None: all cores of the host)."""
    lib().o64ref_set_num_threads(I(int(n) if n else (os.cpu_count() or 1)))
    return num_threads()
