"""Host-side harness over the C ABI: torch tensors in, torch tensors out.

torch is plumbing here (device memory, streams, process groups); all arithmetic runs in
libo64gemm.so.  The method names follow the operator surface the engine serves:
``linear`` / ``matmul`` with bias and activation epilogues, the scaled fp8 and int8 products,
and the Fortran-ABI compat calls (``sgemm``, ``s4gemmx``, ``s4gemvx``) that the reference's
runtime binds (osprey/libfi/matrix/matmul_s4s4.c:87-111, mmx_dlutil.c:122-136).
"""
import ctypes

import torch

from . import _lib
from ._lib import (ACT_GELU_ERF, ACT_GELU_TANH, ACT_NONE, ACT_RELU, ACT_SILU, GATHER_NONE,
                   GATHER_ROWMAJOR, GATHER_SLABS, KIND_BF16, KIND_F32, KIND_FP8, KIND_S8, O64Error,
                   Plan, check)

_ACTS = {None: ACT_NONE, "none": ACT_NONE, "relu": ACT_RELU, "gelu_tanh": ACT_GELU_TANH,
         "gelu": ACT_GELU_ERF, "gelu_erf": ACT_GELU_ERF, "silu": ACT_SILU}


def _act(a):
    if isinstance(a, int):
        return a
    return _ACTS[a]


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(t):
    """torch's current stream on t's device as a cudaStream_t (the raw handle: building a
    torch.cuda.Stream object per call costs more than the rest of the wrapper)."""
    if not t.is_cuda:
        return None
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(t.device.index))
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _rowmajor(t, name):
    if t.dim() != 2:
        raise O64Error(_lib.ERR_RANK, f"{name}: rank {t.dim()}")
    if t.stride(1) != 1 and t.shape[1] != 1:
        t = t.contiguous()
    return t


class Engine:
    """One handle on one device.  Not thread-safe; make one per thread or per stream user."""

    def __init__(self, device=0):
        self._h = ctypes.c_void_p()
        self.lib = _lib.lib()
        if isinstance(device, torch.device):
            device = device.index or 0
        self.device = int(device)
        check(self.lib.o64_create(ctypes.byref(self._h), self.device), "o64_create")

    def close(self):
        if self._h:
            self.lib.o64_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- plans -------------------------------------------------------------------------
    def plan_get(self, kind, M, N, K):
        p = Plan()
        check(self.lib.o64_plan_get(self._h, kind, M, N, K, ctypes.byref(p)), "o64_plan_get")
        return p.as_dict()

    def plan_set(self, kind, **fields):
        if not fields:
            check(self.lib.o64_plan_set(self._h, kind, None), "o64_plan_set")
            return
        p = Plan()
        for k, v in fields.items():
            setattr(p, k, v)
        check(self.lib.o64_plan_set(self._h, kind, ctypes.byref(p)), "o64_plan_set")

    def plan_tune(self, kind, M, N, K, swiglu=False):
        """Times every kernel shape for these extents on scratch operands and keeps the fastest for
        later calls of the same shape; returns it (predicted_ms holds the measured time)."""
        p = Plan()
        s = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        check(self.lib.o64_plan_tune(self._h, kind, 1 if swiglu else 0, M, N, K, s, ctypes.byref(p)), "o64_plan_tune")
        return p.as_dict()

    def plan_save(self, path):
        check(self.lib.o64_plan_save(self._h, str(path).encode()), "o64_plan_save")

    def plan_load(self, path):
        """Merges measured plans from a file; returns how many plans the handle holds afterwards."""
        check(self.lib.o64_plan_load(self._h, str(path).encode()), "o64_plan_load")
        return self.lib.o64_plan_count(self._h)

    def plan_tune_clear(self):
        check(self.lib.o64_plan_tune_clear(self._h), "o64_plan_tune_clear")

    def last_status(self, stream=None):
        """Synchronises and returns (status, detail); status is 0 or ERR_TIMEOUT."""
        detail = ctypes.c_int(0)
        s = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream) if stream is None else stream
        st = self.lib.o64_last_status(self._h, s, ctypes.byref(detail))
        return st, detail.value

    def last_tail_split(self):
        """(tiles, pairs) of the K split the last CTA-pair launch chose for its last wave; (0, 0) = none."""
        t, p = ctypes.c_int(0), ctypes.c_int(0)
        check(self.lib.o64_test_last_tail_split(ctypes.byref(t), ctypes.byref(p)), "o64_test_last_tail_split")
        return t.value, p.value

    def force_tail_split(self, mode):
        """Test hook, process-wide: 1 = always cut a partly filled last wave along K, 0 = never, -1 = model."""
        check(self.lib.o64_test_force_tail_split(int(mode)), "o64_test_force_tail_split")

    def set_wait_budget_us(self, microseconds):
        """Budget of the kernels' bounded waits for later calls (0 = the default, two seconds)."""
        check(self.lib.o64_set_wait_budget_us(self._h, int(microseconds)), "o64_set_wait_budget_us")

    def test_gemm_bf16_withheld(self, A, B, withhold_kblock, out=None):
        """The failure-path hook: a bf16 GEMM (B [N,K]) whose loader leaves out one K block, so the
        kernel's waits run out of the wait budget.  Returns the (undefined) result buffer; read
        last_status() afterwards."""
        M, K = A.shape
        N = B.shape[0]
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
        check(self.lib.o64_test_gemm_bf16_withheld(self._h, M, N, K, _ptr(A), A.stride(0), _ptr(B), B.stride(0),
                                                   _ptr(out), out.stride(0), int(withhold_kblock), _stream(A)),
              "o64_test_gemm_bf16_withheld")
        return out

    # ---- native layer ------------------------------------------------------------------
    def linear_f32(self, A, B, bias=None, act="none", out=None):
        """act(A @ B + bias), fp32; A [M,K], B [K,N]."""
        A = _rowmajor(A, "A")
        B = _rowmajor(B, "B")
        M, K = A.shape
        if B.shape[0] != K:
            raise O64Error(_lib.ERR_CONFORM, "linear_f32")
        N = B.shape[1]
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=A.device)
        check(self.lib.o64_linear_f32(self._h, M, N, K, _ptr(A), A.stride(0), _ptr(B), B.stride(0),
                                      _ptr(bias), _ptr(out), out.stride(0), _act(act), _stream(A)),
              "o64_linear_f32")
        return out

    def gemm_bf16(self, A, B, transB=True, bias=None, act="none", out=None):
        """act(A @ op(B) + bias); A [M,K] bf16; B [N,K] when transB else [K,N]; bf16 result."""
        A = _rowmajor(A, "A")
        B = _rowmajor(B, "B")
        M, K = A.shape
        N = B.shape[0] if transB else B.shape[1]
        if (B.shape[1] if transB else B.shape[0]) != K:
            raise O64Error(_lib.ERR_CONFORM, "gemm_bf16")
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
        epi = _lib.Epilogue(_ptr(bias), _act(act))
        check(self.lib.o64_gemm_bf16(self._h, M, N, K, _ptr(A), A.stride(0), _ptr(B), B.stride(0),
                                     1 if transB else 0, _ptr(out), out.stride(0), ctypes.byref(epi),
                                     _stream(A)), "o64_gemm_bf16")
        return out

    def swiglu(self, X, Wg, Wu, out=None):
        """bf16(silu(X @ Wg) * (X @ Wu)); X [M,K], Wg/Wu [K,N] with one leading dimension."""
        X = _rowmajor(X, "X")
        Wg = _rowmajor(Wg, "Wg")
        Wu = _rowmajor(Wu, "Wu")
        M, K = X.shape
        if Wg.shape != Wu.shape or Wg.shape[0] != K or Wg.stride(0) != Wu.stride(0):
            raise O64Error(_lib.ERR_CONFORM, "swiglu")
        N = Wg.shape[1]
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=X.device)
        check(self.lib.o64_gemm_bf16_swiglu(self._h, M, N, K, _ptr(X), X.stride(0), _ptr(Wg), _ptr(Wu),
                                            Wg.stride(0), _ptr(out), out.stride(0), _stream(X)),
              "o64_gemm_bf16_swiglu")
        return out

    def mlp_swiglu(self, X, Wg, Wu, Wd, h=None, out=None):
        """(silu(X Wg) * (X Wu)) Wd with the SiLU-multiply fused into the first GEMM."""
        h = self.swiglu(X, Wg, Wu, out=h)
        return self.gemm_bf16(h, Wd, transB=False, out=out)

    def gemm_fp8_scaled(self, A8, B8, scaleA=None, scaleB=None, bias=None, out=None):
        """bf16((A8 @ B8^T) * sA[m] * sB[n] + bias[n]); A8 [M,K], B8 [N,K] e4m3."""
        A8 = _rowmajor(A8, "A8")
        B8 = _rowmajor(B8, "B8")
        M, K = A8.shape
        N = B8.shape[0]
        if B8.shape[1] != K:
            raise O64Error(_lib.ERR_CONFORM, "gemm_fp8_scaled")
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=A8.device)
        check(self.lib.o64_gemm_fp8_scaled(self._h, M, N, K, _ptr(A8), A8.stride(0), _ptr(B8),
                                           B8.stride(0), _ptr(scaleA), _ptr(scaleB), _ptr(bias),
                                           _ptr(out), out.stride(0), _stream(A8)), "o64_gemm_fp8_scaled")
        return out

    def gemm_fp8_scaled_ex(self, A8, B8, scaleA=None, scaleB=None, bias=None, act="none", out_kind=_lib.OUT_BF16, out=None):
        """convert(act((A8 @ B8^T) * sA[m] * sB[n] + bias[n])): bf16, or e4m3 again (saturating, nearest even)."""
        M, K = A8.shape
        N = B8.shape[0]
        if B8.shape[1] != K:
            raise O64Error(_lib.ERR_CONFORM, "gemm_fp8_scaled_ex")
        if out is None:
            out = torch.empty((M, N), dtype=torch.float8_e4m3fn if out_kind == _lib.OUT_E4M3 else torch.bfloat16,
                              device=A8.device)
        check(self.lib.o64_gemm_fp8_scaled_ex(self._h, M, N, K, _ptr(A8), A8.stride(0), _ptr(B8), B8.stride(0),
                                              _ptr(scaleA), _ptr(scaleB), _ptr(bias), _act(act), _ptr(out),
                                              out.stride(0), out_kind, _stream(A8)), "o64_gemm_fp8_scaled_ex")
        return out

    def gemm_fp8_scaled_kn(self, A8, B8_kn, scaleA=None, scaleB=None, bias=None, act="none", out_kind=_lib.OUT_BF16, out=None):
        """gemm_fp8_scaled_ex with the weight stored [K,N] (N contiguous); transposed into scratch per call."""
        M, K = A8.shape
        N = B8_kn.shape[1]
        if B8_kn.shape[0] != K:
            raise O64Error(_lib.ERR_CONFORM, "gemm_fp8_scaled_kn")
        if out is None:
            out = torch.empty((M, N), dtype=torch.float8_e4m3fn if out_kind == _lib.OUT_E4M3 else torch.bfloat16,
                              device=A8.device)
        check(self.lib.o64_gemm_fp8_scaled_kn(self._h, M, N, K, _ptr(A8), A8.stride(0), _ptr(B8_kn), B8_kn.stride(0),
                                              _ptr(scaleA), _ptr(scaleB), _ptr(bias), _act(act), _ptr(out),
                                              out.stride(0), out_kind, _stream(A8)), "o64_gemm_fp8_scaled_kn")
        return out

    def gemm_s8_scaled(self, A, B, scaleA=None, scaleB=None, bias=None, act="none", out_kind=_lib.OUT_BF16, out=None):
        """convert(act(float(A @ B^T) * sA[m] * sB[n] + bias[n])), int8 operands: bf16, or int8 again
        (saturating, nearest even)."""
        M, K = A.shape
        N = B.shape[0]
        if B.shape[1] != K:
            raise O64Error(_lib.ERR_CONFORM, "gemm_s8_scaled")
        if out is None:
            out = torch.empty((M, N), dtype=torch.int8 if out_kind == _lib.OUT_S8 else torch.bfloat16, device=A.device)
        check(self.lib.o64_gemm_s8_scaled(self._h, M, N, K, _ptr(A), A.stride(0), _ptr(B), B.stride(0), _ptr(scaleA),
                                          _ptr(scaleB), _ptr(bias), _act(act), _ptr(out), out.stride(0), out_kind,
                                          _stream(A)), "o64_gemm_s8_scaled")
        return out

    def gemm_s8(self, A, B, out=None):
        """A [M,K] int8 times B [N,K]^T int8 -> int32, exact."""
        A = _rowmajor(A, "A")
        B = _rowmajor(B, "B")
        M, K = A.shape
        N = B.shape[0]
        if B.shape[1] != K:
            raise O64Error(_lib.ERR_CONFORM, "gemm_s8")
        if out is None:
            out = torch.empty((M, N), dtype=torch.int32, device=A.device)
        check(self.lib.o64_gemm_s8s8_s32(self._h, M, N, K, _ptr(A), A.stride(0), _ptr(B), B.stride(0),
                                         _ptr(out), out.stride(0), _stream(A)), "o64_gemm_s8s8_s32")
        return out

    @staticmethod
    def gemm_s8_static(A, B, out=None):
        """The int8 product through the entry point that allocates nothing: no handle, scratch in
        a static device array (see include/o64gemm.h).  Device tensors only."""
        lib = _lib.lib()
        M, K = A.shape
        N = B.shape[0]
        if B.shape[1] != K:
            raise O64Error(_lib.ERR_CONFORM, "gemm_s8_static")
        if out is None:
            out = torch.empty((M, N), dtype=torch.int32, device=A.device)
        check(lib.o64_gemm_s8s8_s32_static(M, N, K, _ptr(A), A.stride(0), _ptr(B), B.stride(0), _ptr(out),
                                           out.stride(0), _stream(A)), "o64_gemm_s8s8_s32_static")
        return out

    def naive(self, kind, A, B, transB=True, scaleA=None, scaleB=None, bias=None, act="none"):
        """One-thread-per-output device reference; fp32 result (int32 for KIND_S8)."""
        M, K = A.shape
        N = B.shape[0] if transB else B.shape[1]
        out = torch.empty((M, N), dtype=torch.int32 if kind == KIND_S8 else torch.float32,
                          device=A.device)
        check(self.lib.o64_naive_gemm(self._h, kind, M, N, K, _ptr(A), A.stride(0), _ptr(B), B.stride(0),
                                      1 if transB else 0, _ptr(scaleA), _ptr(scaleB), _ptr(bias),
                                      _act(act), _ptr(out), out.stride(0), _stream(A)), "o64_naive_gemm")
        return out

    # ---- multi-GPU ---------------------------------------------------------------------
    def comm_init_from_process_group(self, group=None):
        """Binds an NCCL communicator over the ranks of a torch.distributed group: rank 0
        makes the id, the group's broadcast carries the bytes."""
        import torch.distributed as dist
        from .sharded import broadcast_unique_id
        rank = dist.get_rank(group)
        world = dist.get_world_size(group)

        def make_id():
            buf = (ctypes.c_char * _lib.UNIQUE_ID_BYTES)()
            check(self.lib.o64_comm_unique_id(buf), "o64_comm_unique_id")
            return bytes(buf)

        idb = broadcast_unique_id(make_id, group)
        check(self.lib.o64_comm_init(self._h, ctypes.create_string_buffer(idb, _lib.UNIQUE_ID_BYTES),
                                     rank, world), "o64_comm_init")
        return rank, world

    def alloc_result(self, M, N, dtype=torch.int32):
        """A [M,N] result buffer that every rank of the bound communicator can store into (the
        target of GATHER_PUSH).  Collective; the engine owns the memory."""

        class _Ext:
            pass

        nbytes = M * N * torch.empty((), dtype=dtype).element_size()
        ptr = ctypes.c_void_p()
        check(self.lib.o64_comm_alloc_result(self._h, nbytes, ctypes.byref(ptr)), "o64_comm_alloc_result")
        ext = _Ext()
        ext.__cuda_array_interface__ = {"shape": (M, N), "typestr": "<i4" if dtype == torch.int32 else "<u2",
                                        "data": (ptr.value, False), "version": 2, "strides": None}
        t = torch.as_tensor(ext, device=torch.device("cuda", self.device))
        return t if dtype == torch.int32 else t.view(dtype)

    def gemm_s8_sharded(self, A, B_slab, N, gather=GATHER_ROWMAJOR, out=None, workspace=None):
        """Column-sharded int8 GEMM: this rank owns B_slab [N/g, K]; `out` is the full [M,N]
        int32 (row-major, or slab-major [g][M][N/g] for GATHER_SLABS)."""
        M, K = A.shape
        if out is None:
            out = torch.empty((M, N), dtype=torch.int32, device=A.device)
        check(self.lib.o64_gemm_s8_sharded(self._h, M, N, K, _ptr(A), A.stride(0), _ptr(B_slab),
                                           B_slab.stride(0), _ptr(out), gather, _ptr(workspace),
                                           _stream(A)), "o64_gemm_s8_sharded")
        return out

    def gemm_bf16_sharded(self, A, B_slab, N, gather=GATHER_NONE, bias=None, act="none", out=None):
        """Column-sharded bf16 linear: this rank owns B_slab [N/g, K]; `bias` is the full [N] vector.
        `out` is the full [M,N] bf16 result (row-major; slab-major [g][M][N/g] for GATHER_SLABS;
        from alloc_result(..., dtype=torch.bfloat16) for GATHER_PUSH)."""
        M, K = A.shape
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
        ep = _lib.Epilogue(_ptr(bias), _act(act))
        check(self.lib.o64_gemm_bf16_sharded(self._h, M, N, K, _ptr(A), A.stride(0), _ptr(B_slab), B_slab.stride(0),
                                             _ptr(out), gather, ctypes.byref(ep), _stream(A)), "o64_gemm_bf16_sharded")
        return out

    # ---- compat layer (Fortran ABI, synchronous) -----------------------------------------
    def sgemm(self, transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc):
        ci, cf = ctypes.c_int, ctypes.c_float
        self.lib.sgemm_(transa.encode(), transb.encode(), ctypes.byref(ci(m)), ctypes.byref(ci(n)),
                        ctypes.byref(ci(k)), ctypes.byref(cf(alpha)), _ptr(a), ctypes.byref(ci(lda)),
                        _ptr(b), ctypes.byref(ci(ldb)), ctypes.byref(cf(beta)), _ptr(c),
                        ctypes.byref(ci(ldc)))
        check(self.lib.o64_compat_last_status(), "sgemm_")
        return c

    def s4gemmx(self, m, n, k, alpha, a, inc1a, inc2a, b, inc1b, inc2b, beta, c, inc1c, inc2c):
        ci, cf = ctypes.c_int, ctypes.c_float
        r = lambda v: ctypes.byref(ci(v))
        self.lib._s4gemmx__(r(m), r(n), r(k), ctypes.byref(cf(alpha)), _ptr(a), r(inc1a), r(inc2a),
                            _ptr(b), r(inc1b), r(inc2b), ctypes.byref(cf(beta)), _ptr(c), r(inc1c),
                            r(inc2c))
        check(self.lib.o64_compat_last_status(), "_s4gemmx__")
        return c

    def s4gemvx(self, m, n, alpha, a, incca, incra, x, incx, beta, y, incy):
        ci, cf = ctypes.c_int, ctypes.c_float
        r = lambda v: ctypes.byref(ci(v))
        self.lib._s4gemvx__(r(m), r(n), ctypes.byref(cf(alpha)), _ptr(a), r(incca), r(incra), _ptr(x),
                            r(incx), ctypes.byref(cf(beta)), _ptr(y), r(incy))
        check(self.lib.o64_compat_last_status(), "_s4gemvx__")
        return y

    _CTYPES = {"s4": ctypes.c_float, "s": ctypes.c_double, "i1": ctypes.c_int8, "i2": ctypes.c_int16,
               "i4": ctypes.c_int32, "j": ctypes.c_int64}

    def xgemmx(self, kind, m, n, k, alpha, a, inc1a, inc2a, b, inc1b, inc2b, beta, c, inc1c, inc2c):
        """The strided kernel `_<kind>gemmx__` of the runtime, in place on c.  kind: "s4", "s", "i1",
        "i2", "i4", "j", or a mixed pair "i1i2" ... "i4j", "s4s", "i1s4" ... "js4", "i1s" ... "js" (A of the
        first kind; B, C, alpha, beta of the second)."""
        name = "_%sgemmx__" % kind
        ckind = kind
        if kind not in self._CTYPES:  # a pair such as "i1i4", "js4", "s4s": the kind of B and C comes last
            ckind = next(sfx for sfx in ("s4", "i1", "i2", "i4", "s", "j") if kind.endswith(sfx) and kind[:-len(sfx)] in self._CTYPES)
        ct = self._CTYPES[ckind]
        r = lambda v: ctypes.byref(ctypes.c_int(v))
        getattr(self.lib, name)(r(m), r(n), r(k), ctypes.byref(ct(alpha)), _ptr(a), r(inc1a), r(inc2a),
                                _ptr(b), r(inc1b), r(inc2b), ctypes.byref(ct(beta)), _ptr(c), r(inc1c),
                                r(inc2c))
        check(self.lib.o64_compat_last_status(), name)
        return c

    def sgemvx(self, m, n, alpha, a, incca, incra, x, incx, beta, y, incy):
        """_sgemvx__: the REAL*8 matrix-vector kernel."""
        cd = ctypes.c_double
        r = lambda v: ctypes.byref(ctypes.c_int(v))
        self.lib._sgemvx__(r(m), r(n), ctypes.byref(cd(alpha)), _ptr(a), r(incca), r(incra), _ptr(x),
                           r(incx), ctypes.byref(cd(beta)), _ptr(y), r(incy))
        check(self.lib.o64_compat_last_status(), "_sgemvx__")
        return y

    def dgemm(self, transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc):
        ci, cd = ctypes.c_int, ctypes.c_double
        self.lib.dgemm_(transa.encode(), transb.encode(), ctypes.byref(ci(m)), ctypes.byref(ci(n)),
                        ctypes.byref(ci(k)), ctypes.byref(cd(alpha)), _ptr(a), ctypes.byref(ci(lda)),
                        _ptr(b), ctypes.byref(ci(ldb)), ctypes.byref(cd(beta)), _ptr(c),
                        ctypes.byref(ci(ldc)))
        check(self.lib.o64_compat_last_status(), "dgemm_")
        return c

    def cgemmx(self, m, n, k, alpha, a, inc1a, inc2a, b, inc1b, inc2b, beta, c, inc1c, inc2c, conja=False, conjb=False):
        """_c4gemmx__ / _cgemmx__ (by c's dtype: complex64 / complex128), in place on c; increments in
        complex elements."""
        single = c.dtype == torch.complex64
        fn = self.lib._c4gemmx__ if single else self.lib._cgemmx__
        ct = ctypes.c_float if single else ctypes.c_double
        r = lambda v: ctypes.byref(ctypes.c_int(int(v)))
        cx = lambda z: (ct * 2)(complex(z).real, complex(z).imag)
        al, be = cx(alpha), cx(beta)
        fn(r(conja), r(conjb), r(m), r(n), r(k), ctypes.cast(al, ctypes.c_void_p), _ptr(a), r(inc1a), r(inc2a),
           _ptr(b), r(inc1b), r(inc2b), ctypes.cast(be, ctypes.c_void_p), _ptr(c), r(inc1c), r(inc2c))
        check(self.lib.o64_compat_last_status(), "_cgemmx__")
        return c

    def cgemvx(self, m, n, alpha, a, incca, incra, x, incx, beta, y, incy, conj=False):
        """_c4gemvx__ / _cgemvx__ by y's dtype, in place on y."""
        single = y.dtype == torch.complex64
        fn = self.lib._c4gemvx__ if single else self.lib._cgemvx__
        ct = ctypes.c_float if single else ctypes.c_double
        r = lambda v: ctypes.byref(ctypes.c_int(int(v)))
        cx = lambda z: (ct * 2)(complex(z).real, complex(z).imag)
        al, be = cx(alpha), cx(beta)
        fn(r(conj), r(m), r(n), ctypes.cast(al, ctypes.c_void_p), _ptr(a), r(incca), r(incra), _ptr(x), r(incx),
           ctypes.cast(be, ctypes.c_void_p), _ptr(y), r(incy))
        check(self.lib.o64_compat_last_status(), "_cgemvx__")
        return y

    def cgemm(self, transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc):
        """cgemm_ / zgemm_ by c's dtype (column-major BLAS)."""
        single = c.dtype == torch.complex64
        fn = self.lib.cgemm_ if single else self.lib.zgemm_
        ct = ctypes.c_float if single else ctypes.c_double
        r = lambda v: ctypes.byref(ctypes.c_int(int(v)))
        cx = lambda z: (ct * 2)(complex(z).real, complex(z).imag)
        al, be = cx(alpha), cx(beta)
        fn(transa.encode(), transb.encode(), r(m), r(n), r(k), ctypes.cast(al, ctypes.c_void_p), _ptr(a), r(lda),
           _ptr(b), r(ldb), ctypes.cast(be, ctypes.c_void_p), _ptr(c), r(ldc))
        check(self.lib.o64_compat_last_status(), "cgemm_")
        return c

    _LTYPES = {"l1": ctypes.c_int8, "l2": ctypes.c_int16, "l4": ctypes.c_int32, "l": ctypes.c_int64}

    def lgemmx(self, kind, m, n, k, alpha, a, inc1a, inc2a, b, inc1b, inc2b, beta, c, inc1c, inc2c):
        """The LOGICAL strided kernel `_<kind>gemmx__`: kind "l1", "l2", "l4", "l" or a pair "l1l2" ... "l4l"
        (A of the first kind; B, C, alpha, beta of the second); logicals are integer tensors, non-zero is true."""
        ckind = kind if kind in self._LTYPES else next(sfx for sfx in ("l1", "l2", "l4", "l")
                                                        if kind.endswith(sfx) and kind[:-len(sfx)] in self._LTYPES)
        ct = self._LTYPES[ckind]
        r = lambda v: ctypes.byref(ctypes.c_int(v))
        getattr(self.lib, "_%sgemmx__" % kind)(r(m), r(n), r(k), ctypes.byref(ct(1 if alpha else 0)), _ptr(a), r(inc1a),
                                               r(inc2a), _ptr(b), r(inc1b), r(inc2b), ctypes.byref(ct(1 if beta else 0)),
                                               _ptr(c), r(inc1c), r(inc2c))
        check(self.lib.o64_compat_last_status(), "_%sgemmx__" % kind)
        return c
