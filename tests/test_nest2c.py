"""CPU: o64nest, the source rewriter that turns GEMM-shaped loop nests (as the reference prints
them back to C, osprey/be/whirl2c/wn2c.cxx:4078-4118) into calls of the engine."""
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOOL = os.path.join(ROOT, "open64_b200", "nest2c", "o64nest")
SRC = os.path.join(ROOT, "tests", "nests", "layers.c")


def rewrite(text):
    r = subprocess.run([TOOL], input=text, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    n = int(re.search(r"(\d+) nest", r.stderr).group(1))
    return r.stdout, n


def test_every_product_nest_of_the_fixture_is_replaced(built, tmp_path):
    out, n = rewrite(open(SRC).read())
    assert n == 6
    # the fused linear: bias and ReLU in the call, extents from the inclusive bounds, the loops'
    # blocking-size pragmas as a plan (i loop: tile_m and the L2 group; j loop: tile_n)
    # (pitches are the declared inner extents, spelled as in the declaration)
    assert ("o64_linear_f32(o64nest_handle(), 192, 160, 224, &A[0][0], KK, &B[0][0], NN, bias, &Y[0][0], NN, "
            "O64_ACT_RELU, NULL)") in out
    assert "o64_plan.tile_m = 32;" in out and "o64_plan.tile_n = 64;" in out and "o64_plan.group_m = 4;" in out
    assert "o64_linear_f32(o64nest_handle(), MM, NN, KK, &A[0][0], KK, &B[0][0], NN, NULL, &Yplain[0][0], NN, O64_ACT_NONE" in out
    # other kinds and layouts go to the runtime's strided kernels; a transposed operand swaps its increments
    assert "_sgemmx__(&o64_m, &o64_n, &o64_k" in out and "o64_m = 100, o64_n = 80, o64_k = 60" in out
    assert "_i4gemmx__(" in out and "o64_b1 = 1, o64_b2 = 32" in out
    assert "_jgemmx__(" in out
    assert "o64_linear_f32(o64nest_handle(), m, n, kk, &X[0], kk, &W[0], n, NULL, &O[0], n, O64_ACT_NONE" in out
    # the nest that is not a product is untouched, and so is everything around the nests
    assert "Y[i][j] = Y[i][j] + A[i][k] + B[k][j];" in out
    assert "static unsigned rng_state = 12345u;" in out and "for (int j = 0; j < NN; j++) bias[j] = frand();" in out
    # what comes out is C that compiles against the public header
    path = tmp_path / "layers_out.c"
    path.write_text(out)
    r = subprocess.run(["gcc", "-fsyntax-only", "-Wall", "-Werror=implicit-function-declaration",
                        "-I", os.path.join(ROOT, "include"), str(path)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


NOT_RECOGNISED = [
    # a first value in terms of another loop's variable: not a rectangle
    "float A[8][8],B[8][8],C[8][8];\nvoid f(){for(int i=0;i<8;i++)for(int j=i;j<8;j++){C[i][j]=0;for(int k=0;k<8;k++)C[i][j]+=A[i][k]*B[k][j];}}",
    # a bound in terms of another loop's variable
    "float A[8][8],B[8][8],C[8][8];\nvoid f(){for(int i=0;i<8;i++)for(int j=0;j<8;j++){C[i][j]=0;for(int k=0;k<=j;k++)C[i][j]+=A[i][k]*B[k][j];}}",
    # step of two
    "float A[8][8],B[8][8],C[8][8];\nvoid f(){for(int i=0;i<8;i+=2)for(int j=0;j<8;j++){C[i][j]=0;for(int k=0;k<8;k++)C[i][j]+=A[i][k]*B[k][j];}}",
    # accumulator not zeroed
    "float A[8][8],B[8][8],C[8][8];\nvoid f(){for(int i=0;i<8;i++)for(int j=0;j<8;j++){C[i][j]=1;for(int k=0;k<8;k++)C[i][j]+=A[i][k]*B[k][j];}}",
    # the output is also an operand
    "float A[8][8],C[8][8];\nvoid f(){for(int i=0;i<8;i++)for(int j=0;j<8;j++){C[i][j]=0;for(int k=0;k<8;k++)C[i][j]+=A[i][k]*C[k][j];}}",
    # mixed element types
    "float A[8][8];double B[8][8];float C[8][8];\nvoid f(){for(int i=0;i<8;i++)for(int j=0;j<8;j++){C[i][j]=0;for(int k=0;k<8;k++)C[i][j]+=A[i][k]*B[k][j];}}",
    # subscripts that are not a matrix product (both operands indexed by i and k)
    "float A[8][8],B[8][8],C[8][8];\nvoid f(){for(int i=0;i<8;i++)for(int j=0;j<8;j++){C[i][j]=0;for(int k=0;k<8;k++)C[i][j]+=A[i][k]*B[i][k];}}",
    # a tail the engine has no epilogue for, on a kind that only has the plain product
    "double A[8][8],B[8][8],C[8][8],b[8];\nvoid f(){for(int i=0;i<8;i++)for(int j=0;j<8;j++){double s=0;for(int k=0;k<8;k++)s+=A[i][k]*B[k][j];C[i][j]=s+b[j];}}",
    # undeclared arrays: the pitch is unknown
    "void f(){for(int i=0;i<8;i++)for(int j=0;j<8;j++){C[i][j]=0;for(int k=0;k<8;k++)C[i][j]+=A[i][k]*B[k][j];}}",
]


@pytest.mark.parametrize("text", NOT_RECOGNISED)
def test_nests_outside_the_pattern_pass_through_unchanged(built, text):
    out, n = rewrite(text)
    assert n == 0 and out == text


def test_whirl2c_spellings(built):
    text = ("_IEEE32 A[512LL][512LL];\n_IEEE32 B[512LL][512LL];\n_IEEE32 Y[512LL][512LL];\n_IEEE32 bias[512LL];\n"
            "void layer() {\n  _INT32 i; _INT32 j; _INT32 k; _IEEE32 acc;\n"
            "  for(i = 0; i <= 511; i = i + 1)\n  {\n    for(j = 0; j <= 511; j = j + 1)\n    {\n      acc = 0.0F;\n"
            "      for(k = 0; k <= 511; k = k + 1)\n      {\n        acc = acc + (A[i][k] * B[k][j]);\n      }\n"
            "      Y[i][j] = _MAX(acc + bias[j], 0.0F);\n    }\n  }\n}\n")
    out, n = rewrite(text)
    assert n == 1
    assert "o64_linear_f32(o64nest_handle(), 512, 512, 512, &A[0][0], 512, &B[0][0], 512, bias, &Y[0][0], 512, O64_ACT_RELU, NULL)" in out
    # x > 0 ? x : 0 is the same tail
    out2, n2 = rewrite(text.replace("_MAX(acc + bias[j], 0.0F)", "(acc + bias[j]) > 0.0F ? (acc + bias[j]) : 0.0F"))
    assert n2 == 1 and "O64_ACT_RELU" in out2


TILED = os.path.join(ROOT, "tests", "nests", "tiled.c")


def test_nests_the_reference_has_already_tiled(built, tmp_path):
    """Strip loops + blocked loops with min() bounds, in any order, become one accumulating call of the
    strided kernel; the strip sizes travel as plan pins; GELU / SiLU tails fuse into the linear."""
    out, n = rewrite(open(TILED).read())
    assert n == 8
    assert "blocked 64 x - x 16 (i x j x k)" in out
    assert "blocked 100 x 32 x 64 (i x j x k, j outside i)" in out and "o64_plan.raster = 1;" in out
    assert "blocked - x - x 40" in out
    assert "o64_plan.tile_m = 64;" in out and "o64_plan.tile_k = 16;" in out
    assert "o64_plan_set(o64_compat_handle(), O64_KIND_F32, &o64_plan)" in out
    # beta = 1, whole extents recovered from the strip loops' bounds
    assert out.count("&o64_one, (float *)&C") == 3 and "o64_m = 300, o64_n = 260, o64_k = 200" in out
    assert "_sgemmx__(&o64_m, &o64_n, &o64_k, &o64_one" in out and "o64_m = 90, o64_n = 50, o64_k = 70" in out
    assert "_i4gemmx__(" in out and "o64_m = 40, o64_n = 56, o64_k = 24" in out
    # the zeroing nests in front stay
    assert out.count("C1[i][j] = 0.0F;") == 1 and "C3[i][j] = 0;" in out
    for act in ("O64_ACT_SILU", "O64_ACT_GELU_TANH", "O64_ACT_GELU_ERF"):
        assert out.count(act + ", NULL)") == 1
    assert "&A[0][0], 200, &B[0][0], 260, bias, &G1[0][0], 260, O64_ACT_SILU" in out
    # the nest whose blocked loop overruns its strip is not a tiling of a product: untouched
    assert "for (int i = it; i < it + 64; i++)" in out
    path = tmp_path / "tiled_out.c"
    path.write_text(out)
    r = subprocess.run(["gcc", "-fsyntax-only", "-Werror=implicit-function-declaration", "-I", os.path.join(ROOT, "include"),
                        str(path)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


@pytest.mark.parametrize("text", [
    # the blocked loop's bound is not strip + block - 1
    "float A[8][8],B[8][8],C[8][8];\nvoid f(){for(int t=0;t<8;t+=4)for(int i=t;i<t+2;i++)for(int j=0;j<8;j++)for(int k=0;k<8;k++)C[i][j]+=A[i][k]*B[k][j];}",
    # the minimum is taken against another bound than the strip loop's
    "float A[8][8],B[8][8],C[8][8];\nvoid f(){for(int t=0;t<8;t+=4)for(int i=t;i<(t+4<6?t+4:6);i++)for(int j=0;j<8;j++)for(int k=0;k<8;k++)C[i][j]+=A[i][k]*B[k][j];}",
    # a second statement in the innermost body
    "float A[8][8],B[8][8],C[8][8];\nvoid f(){for(int i=0;i<8;i++)for(int j=0;j<8;j++)for(int k=0;k<8;k++){C[i][j]+=A[i][k]*B[k][j];A[i][k]=0;}}",
    # an activation the engine does not have
    "float A[8][8],B[8][8],C[8][8];\nvoid f(){for(int i=0;i<8;i++)for(int j=0;j<8;j++){float s=0;for(int k=0;k<8;k++)s+=A[i][k]*B[k][j];C[i][j]=tanhf(s);}}",
])
def test_near_misses_of_the_tiled_form_pass_through(built, text):
    out, n = rewrite(text)
    assert n == 0 and out == text


def test_a_loop_around_a_product_nest_stays(built):
    """A stepping loop whose variable no inner loop starts from is no strip loop: it stays, and the
    accumulating nest inside it is replaced (and so runs once per iteration, as before)."""
    text = ("float A[8][8],B[8][8],C[8][8];\nvoid f(){for(int t=0;t<8;t+=4)for(int i=0;i<8;i++)for(int j=0;j<8;j++)"
            "for(int k=0;k<8;k++)C[i][j]+=A[i][k]*B[k][j];}")
    out, n = rewrite(text)
    assert n == 1 and "for(int t=0;t<8;t+=4){" in out and "_s4gemmx__(" in out


def test_nests_over_sections_of_arrays(built, tmp_path):
    """Loops that do not start at zero: the operands' first elements and the extents follow the first values."""
    out, n = rewrite(open(os.path.join(ROOT, "tests", "nests", "sections.c")).read())
    assert n == 3
    assert ("o64_linear_f32(o64nest_handle(), (M - (2)), (((N - 2) + 1) - (3)), (K - (1)), &A[2][1], K, &B[1][3], N, "
            "&bias[3], &Y[2][3], N, O64_ACT_RELU, NULL)") in out
    assert "&P[(lo) * (30) + ((lo + 1))]" in out and "&Q[((lo + 1)) * (20) + 4]" in out and "&R[(lo) * (20) + 4]" in out
    assert "o64_m = ((hi) - (lo))" in out or "o64_m = (hi - (lo))" in out
    assert "&Ai[5][2]" in out and "&Bi[2][7]" in out and "&Ci[5][7]" in out and "o64_m = 35, o64_n = 44, o64_k = 21" in out
    # the triangular nest is still there
    assert "for (j = i; j < N; j++)" in out and "T[i][j] = acc;" in out
    path = tmp_path / "sections_out.c"
    path.write_text(out)
    r = subprocess.run(["gcc", "-fsyntax-only", "-Wall", "-Werror=implicit-function-declaration",
                        "-I", os.path.join(ROOT, "include"), str(path)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
