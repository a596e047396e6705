"""CPU oracle for the GEMM path: a ctypes view of ``oracle/gemm_ref.c``.

Test infrastructure only.  Nothing under ``open64_b200`` imports this package; only the
tests, the smoke check and the benchmark's CPU-baseline leg do.  Parity is UNPINNED: the
reference holds no golden vectors for a matrix product (see the header of ``gemm_ref.c``).
"""
from .ref import *  # noqa: F401,F403
