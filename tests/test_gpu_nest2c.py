"""GPU: a C program whose loop nests were rewritten by o64nest, linked against libo64gemm.so, gives
the same results as the untouched program compiled by gcc: fp32 within 1e-4 of the largest
magnitude, REAL*8 within 1e-12, the integer kinds bit for bit."""
import os
import subprocess

import numpy as np
import pytest

from util import TOL_F32, relmax

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOOL = os.path.join(ROOT, "open64_b200", "nest2c", "o64nest")
SRC = os.path.join(ROOT, "tests", "nests", "layers.c")
LIBDIR = os.path.join(ROOT, "open64_b200")


def test_rewritten_program_matches_the_original(built, tmp_path):
    ref_exe, new_exe = tmp_path / "ref", tmp_path / "new"
    new_src = tmp_path / "layers_o64.c"
    subprocess.run(["gcc", "-O2", "-ffp-contract=off", SRC, "-o", str(ref_exe), "-lm"], check=True)
    subprocess.run([TOOL, SRC, "-o", str(new_src)], check=True)
    subprocess.run(["gcc", "-O2", str(new_src), "-I", os.path.join(ROOT, "include"), "-o", str(new_exe),
                    "-L", LIBDIR, "-lo64gemm", f"-Wl,-rpath,{LIBDIR}", "-lm"], check=True)
    ref_out, new_out = tmp_path / "ref.bin", tmp_path / "new.bin"
    subprocess.run([str(ref_exe), str(ref_out)], check=True, timeout=120)
    r = subprocess.run([str(new_exe), str(new_out)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    a, b = open(ref_out, "rb").read(), open(new_out, "rb").read()
    assert len(a) == len(b)
    MM, NN = 192, 160
    off = 0

    def take(buf, dtype, count):
        nonlocal off
        v = np.frombuffer(buf, dtype=dtype, count=count, offset=off)
        return v

    layout = [("fused linear", np.float32, MM * NN), ("plain product", np.float32, MM * NN),
              ("REAL*8 in place", np.float64, 100 * 80), ("int times transposed", np.int32, 64 * 48),
              ("int64", np.int64, 40 * 56), ("flattened", np.float32, MM * NN)]
    for name, dt, count in layout:
        x, y = take(a, dt, count), take(b, dt, count)
        off += count * np.dtype(dt).itemsize
        assert np.abs(x).max() > 0, name
        if dt is np.float32:
            assert relmax(y, x) <= TOL_F32, name
        elif dt is np.float64:
            assert relmax(y, x) <= 1e-12, name
        else:
            assert np.array_equal(x, y), name
    assert off == len(a)


def test_rewritten_tiled_program_matches_the_original(built, tmp_path):
    """tests/nests/tiled.c: nests already blocked by the reference's loop-nest optimiser (and fused
    linears with GELU / SiLU tails) run through the engine give what gcc's code for the nests gives."""
    src = os.path.join(ROOT, "tests", "nests", "tiled.c")
    ref_exe, new_exe = tmp_path / "ref", tmp_path / "new"
    new_src = tmp_path / "tiled_o64.c"
    subprocess.run(["gcc", "-O2", "-ffp-contract=off", src, "-o", str(ref_exe), "-lm"], check=True)
    subprocess.run([TOOL, src, "-o", str(new_src)], check=True)
    subprocess.run(["gcc", "-O2", str(new_src), "-I", os.path.join(ROOT, "include"), "-o", str(new_exe),
                    "-L", LIBDIR, "-lo64gemm", f"-Wl,-rpath,{LIBDIR}", "-lm"], check=True)
    ref_out, new_out = tmp_path / "ref.bin", tmp_path / "new.bin"
    subprocess.run([str(ref_exe), str(ref_out)], check=True, timeout=120)
    r = subprocess.run([str(new_exe), str(new_out)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    a, b = open(ref_out, "rb").read(), open(new_out, "rb").read()
    assert len(a) == len(b)
    off = 0
    layout = [("blocked i, k", np.float32, 300 * 260), ("blocked i, j, k interchanged", np.float32, 300 * 260),
              ("blocked by hand", np.float32, 300 * 260), ("REAL*8 accumulating", np.float64, 90 * 50),
              ("int accumulating", np.int32, 40 * 56), ("SiLU", np.float32, 300 * 260),
              ("GELU tanh", np.float32, 300 * 260), ("GELU erf", np.float32, 300 * 260)]
    for name, dt, count in layout:
        x = np.frombuffer(a, dtype=dt, count=count, offset=off)
        y = np.frombuffer(b, dtype=dt, count=count, offset=off)
        off += count * np.dtype(dt).itemsize
        assert np.abs(x).max() > 0, name
        if dt is np.float32:
            assert relmax(y, x) <= TOL_F32, name
        elif dt is np.float64:
            assert relmax(y, x) <= 1e-12, name
        else:
            assert np.array_equal(x, y), name
    assert off == len(a)


def test_rewritten_sections_program_matches_the_original(built, tmp_path):
    """tests/nests/sections.c: product nests over sections of arrays (loops that do not start at zero);
    the elements outside the sections keep their values, the triangular nest runs as gcc compiled it."""
    src = os.path.join(ROOT, "tests", "nests", "sections.c")
    ref_exe, new_exe = tmp_path / "ref", tmp_path / "new"
    new_src = tmp_path / "sections_o64.c"
    subprocess.run(["gcc", "-O2", "-ffp-contract=off", src, "-o", str(ref_exe), "-lm"], check=True)
    subprocess.run([TOOL, src, "-o", str(new_src)], check=True)
    subprocess.run(["gcc", "-O2", "-ffp-contract=off", str(new_src), "-I", os.path.join(ROOT, "include"), "-o", str(new_exe),
                    "-L", LIBDIR, "-lo64gemm", f"-Wl,-rpath,{LIBDIR}", "-lm"], check=True)
    ref_out, new_out = tmp_path / "ref.bin", tmp_path / "new.bin"
    subprocess.run([str(ref_exe), str(ref_out)], check=True, timeout=120)
    r = subprocess.run([str(new_exe), str(new_out)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    a, b = open(ref_out, "rb").read(), open(new_out, "rb").read()
    assert len(a) == len(b)
    off = 0
    layout = [("section of the fused linear", np.float32, 140 * 96), ("REAL*8 flattened section", np.float64, 50 * 20),
              ("integer section", np.int32, 40 * 56), ("triangle (untouched nest)", np.float32, 140 * 96)]
    for name, dt, count in layout:
        x = np.frombuffer(a, dtype=dt, count=count, offset=off)
        y = np.frombuffer(b, dtype=dt, count=count, offset=off)
        off += count * np.dtype(dt).itemsize
        assert np.abs(x).max() > 0, name
        if dt is np.float32:
            assert relmax(y, x) <= TOL_F32, name
        elif dt is np.float64:
            assert relmax(y, x) <= 1e-12, name
        else:
            assert np.array_equal(x, y), name
    assert off == len(a)
    # outside the section nothing was written: the fill values are still there
    y = np.frombuffer(b, dtype=np.float32, count=140 * 96).reshape(140, 96)
    assert (y[:2] == -5.0).all() and (y[:, :3] == -5.0).all() and (y[:, 95:] == -5.0).all()
