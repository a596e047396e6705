"""CPU: the C-ABI library loads without a GPU and exports every symbol its header declares."""
import ctypes
import os
import re

import pytest

import open64_b200 as o

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "o64gemm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"^\s*(?:const\s+)?(?:int|void|size_t|char|float|double|int32_t|int64_t|o64_complex8_t|o64_complex16_t|o64_handle_t)"
                       r"\s*\*?\s*(\w+)\s*\(", text, flags=re.M)
    return sorted(set(names))


def test_header_and_library_agree(built):
    declared = header_functions()
    assert len(declared) >= 20
    lib = o.lib()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in o64gemm.h but not exported"
    assert sorted(o.EXPORTS) == declared


def test_no_compute_without_gpu_is_an_error_not_a_fallback(built):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = ctypes.c_void_p()
    assert o.lib().o64_create(ctypes.byref(h), 0) == o.ERR_CUDA
    assert not h
    with pytest.raises(o.O64Error):
        o.Engine(0)


def test_status_strings(built):
    lib = o.lib()
    seen = set()
    for code in range(0, -9, -1):
        s = lib.o64_status_string(code).decode()
        assert s and s != "unknown status"
        seen.add(s)
    assert len(seen) == 9
    assert lib.o64_status_string(-99).decode() == "unknown status"
    assert b"sm_100a" in lib.o64_version()


def test_null_arguments_are_rejected(built):
    lib = o.lib()
    assert lib.o64_create(None, 0) == o.ERR_RANK
    assert lib.o64_destroy(None) == o.ERR_RANK
    assert lib.o64_plan_get(None, 1, 1, 1, 1, None) == o.ERR_RANK
    assert lib.o64_comm_unique_id(None) == o.ERR_RANK
    assert lib.o64_gemm_s8_sharded_workspace(128, 256, 2, o.GATHER_ROWMAJOR) == 128 * 256 * 4
    assert lib.o64_gemm_s8_sharded_workspace(128, 256, 2, o.GATHER_SLABS) == 0


def test_product_never_touches_the_oracle():
    """The shipped package and its sources may not import, link or name the CPU oracle."""
    pkg = os.path.join(ROOT, "open64_b200")
    for base, _, files in os.walk(pkg):
        if os.path.basename(base) == "build":
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(base, f)).read()
                assert "oracle" not in text and "o64ref" not in text, f"{f} refers to the oracle"
