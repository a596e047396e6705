"""GPU: the int8 GEMM entry point that allocates nothing (o64_gemm_s8s8_s32_static).

Some callers run with a fixed device-memory plan: everything on the device was handed out up
front, or the call sits in a section where cudaMalloc (which synchronises the device and can fail)
is not allowed.  For them the library keeps its scratch in a static device array.  These tests
call that entry point through the C ABI, twice in a row per case (the array keeps the previous
call's contents), and require the result to be bit-identical to the handle-based entry point.

Collected last on purpose: a run that stops at the first failure has then already run every other
test.  The tests make no assumption about what ran before them in the process.
"""
import ctypes

import numpy as np
import pytest
import torch

import open64_b200 as o
import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("shape", [(300, 520, 400),      # aligned pitch: operands used in place
                                   (130, 72, 200),       # 200-byte rows: both operands are copied
                                   (1024, 2048, 1000)])  # several tiles per CTA, copied operands
def test_static_scratch_matches_handle_path_twice(eng, shape):
    M, N, K = shape
    A, B = o.workloads.c5_int8(M, N, K, seed=M + 2 * N + K)
    Ad, Bd = A.to(DEV), B.to(DEV)
    expected = eng.gemm_s8(Ad, Bd)                        # the existing entry point
    torch.cuda.synchronize()
    assert np.array_equal(expected.cpu().numpy(), oracle.gemm_s8s8_s32(A.numpy(), B.numpy()))
    lib = o.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):
        C = torch.full((M, N), -7, dtype=torch.int32, device=DEV)
        rc = lib.o64_gemm_s8s8_s32_static(M, N, K, _ptr(Ad), Ad.stride(0), _ptr(Bd), Bd.stride(0),
                                          _ptr(C), C.stride(0), stream)
        assert rc == o.OK, (call, rc)
        torch.cuda.synchronize()
        assert torch.equal(C, expected), f"call {call} differs from the handle-based result"
    # a different problem in between must not leak into the next call either
    A2, B2 = o.workloads.c5_int8(64, 40, 56, seed=1)
    o.Engine.gemm_s8_static(A2.to(DEV), B2.to(DEV))
    C = o.Engine.gemm_s8_static(Ad, Bd)
    assert torch.equal(C, expected)


def test_misaligned_base_pointer_is_copied(eng):
    M, N, K = 96, 64, 128
    A, B = o.workloads.c5_int8(M, N, K, seed=5)
    flat = torch.zeros(M * K + 3, dtype=torch.int8, device=DEV)
    flat[3:] = A.to(DEV).reshape(-1)
    Aoff = flat[3:].view(M, K)                            # base address off by 3 bytes
    expected = eng.gemm_s8(A.to(DEV), B.to(DEV))
    for _ in range(2):
        assert torch.equal(o.Engine.gemm_s8_static(Aoff, B.to(DEV)), expected)


def test_rejections(built):
    lib = o.lib()
    A = torch.zeros((64, 64), dtype=torch.int8, device=DEV)
    C = torch.zeros((64, 64), dtype=torch.int32, device=DEV)
    f = lib.o64_gemm_s8s8_s32_static
    assert f(64, 64, 64, _ptr(A), 64, _ptr(A), 64, _ptr(C), 64, None) == o.OK
    assert f(64, 64, 64, _ptr(A), 32, _ptr(A), 64, _ptr(C), 64, None) == o.ERR_CONFORM
    assert f(-1, 64, 64, _ptr(A), 64, _ptr(A), 64, _ptr(C), 64, None) == o.ERR_RANK
    assert f(64, 64, 64, None, 64, _ptr(A), 64, _ptr(C), 64, None) == o.ERR_RANK
    host = torch.zeros((64, 64), dtype=torch.int8)
    assert f(64, 64, 64, _ptr(host), 64, _ptr(A), 64, _ptr(C), 64, None) == o.ERR_RANK   # would need staging
    # padded copies beyond the static array: 40000 x 500 -> 40000 x 512 bytes = 19.5 MiB > 16 MiB
    big = torch.zeros((40000, 500), dtype=torch.int8, device=DEV)
    Cb = torch.zeros((40000, 64), dtype=torch.int32, device=DEV)
    Bb = torch.zeros((64, 500), dtype=torch.int8, device=DEV)
    assert 40000 * 512 > o._lib.STATIC_SCRATCH_BYTES
    assert f(40000, 64, 500, _ptr(big), 500, _ptr(Bb), 500, _ptr(Cb), 64, None) == o.ERR_NOMEM
    torch.cuda.synchronize()


def test_no_device_memory_is_taken(eng):
    """The property the entry point exists for: after the first call on the device (which resolves the
    static array's address) a call whose operands need padded copies leaves the device's free memory
    exactly where it was."""
    A, B = o.workloads.c5_int8(130, 72, 200, seed=9)
    Ad, Bd = A.to(DEV), B.to(DEV)
    C = torch.empty((130, 72), dtype=torch.int32, device=DEV)
    o.Engine.gemm_s8_static(Ad, Bd, out=C)               # warm-up: set-up and module load are behind us
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        o.Engine.gemm_s8_static(Ad, Bd, out=C)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert np.array_equal(C.cpu().numpy(), oracle.gemm_s8s8_s32(A.numpy(), B.numpy()))
