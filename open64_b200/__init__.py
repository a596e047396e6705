"""open64_b200 — a B200 (sm_100a) dense GEMM / fused-linear engine behind the matrix-multiply
boundary of the Open64 compiler's runtime.  All arithmetic runs in libo64gemm.so (hand-written
CUDA: TMA, tcgen05.mma, tensor memory); this package is the ctypes harness over its C ABI.

Build the library first:  python -m open64_b200.build
"""
from ._lib import (ACT_GELU_ERF, ACT_GELU_TANH, ACT_NONE, ACT_RELU, ACT_SILU, ERR_ALIGN,  # noqa: F401
                   ERR_CONFORM, ERR_CUDA, ERR_DTYPE, ERR_NCCL, ERR_NOMEM, ERR_RANK, ERR_TIMEOUT,
                   EXPORTS, GATHER_NONE, GATHER_PUSH, GATHER_ROWMAJOR, GATHER_SLABS, KIND_BF16, KIND_F32, KIND_FP8,
                   KIND_S8, LIB_PATH, OK, OUT_BF16, OUT_E4M3, OUT_S8, O64Error, Plan, lib)
from .engine import Engine  # noqa: F401
from . import workloads  # noqa: F401
