"""GPU, two devices in ONE process: per-device kernel set-up (the dynamic shared-memory limit and the
cluster occupancy are properties of a device, not of the process), and the refusal of operands that
live on another GPU.  Skipped on a one-GPU machine."""
import numpy as np
import pytest
import torch

import open64_b200 as o
import oracle
from util import TOL_LOWP, bits16, relmax

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def two(built):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs in one process")
    e0, e1 = o.Engine(0), o.Engine(1)
    yield e0, e1
    e0.close()
    e1.close()


def test_each_device_gets_its_own_kernel_setup(two):
    ref_cache = {}
    for pin in (dict(cta_group=1, tile_m=128, tile_n=256, split_k=1), dict(cta_group=2, tile_m=256, tile_n=256),
                dict(cta_group=2, tile_m=512, tile_n=256), dict(split_k=-2, tile_n=256)):
        M = 64 if pin.get("split_k", 0) < 0 else 512
        A, B = o.workloads.c2_gemm_bf16(M, 512, 512)
        ref = ref_cache.setdefault(M, oracle.gemm_bf16(bits16(A), bits16(B)))
        for eng in two:                      # device 0 first: the second device must not inherit its set-up
            dev = torch.device("cuda", eng.device)
            eng.plan_set(o.KIND_BF16, **pin)
            with torch.cuda.device(dev):
                c = eng.gemm_bf16(A.to(dev), B.to(dev), transB=True).float().cpu().numpy()
            eng.plan_set(o.KIND_BF16)
            assert eng.last_status() == (o.OK, 0)
            assert relmax(c, ref) <= TOL_LOWP, f"device {eng.device}, pin {pin}"


def test_static_entry_point_on_the_second_device(two):
    A, B = o.workloads.c5_int8(130, 72, 200)
    want = oracle.gemm_s8s8_s32(A.numpy(), B.numpy())
    with torch.cuda.device(1):
        dev = torch.device("cuda", 1)
        c = o.Engine.gemm_s8_static(A.to(dev), B.to(dev))
        torch.cuda.synchronize()
    assert np.array_equal(c.cpu().numpy(), want)


def test_operands_of_another_gpu_are_refused(two):
    e0, _ = two
    A, B = o.workloads.c2_gemm_bf16(128, 128, 128)
    a0, b1 = A.to("cuda:0"), B.to("cuda:1")
    out0 = torch.empty((128, 128), dtype=torch.bfloat16, device="cuda:0")
    with pytest.raises(o.O64Error) as e:
        e0.gemm_bf16(a0, b1, transB=True, out=out0)
    assert e.value.status == o.ERR_RANK
    A8, B8 = o.workloads.c5_int8(64, 64, 64)
    with torch.cuda.device(0):
        with pytest.raises(o.O64Error) as e:
            o.Engine.gemm_s8_static(A8.to("cuda:0"), B8.to("cuda:1"),
                                    out=torch.empty((64, 64), dtype=torch.int32, device="cuda:0"))
    assert e.value.status == o.ERR_RANK
