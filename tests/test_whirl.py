"""CPU: o64whirl, the matcher over WHIRL dumps (the ASCII form the reference's ir_b2a prints).  The
dumps are derived by hand from lower_mm_matmul (osprey/be/vho/f90_lower.cxx:5116-5178) and the ASCII
writer's format (osprey/common/com/ir_reader.cxx:976-1560) by tests/whirl/make_dumps.py."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOOL = os.path.join(ROOT, "open64_b200", "whirl", "o64whirl")
DUMPS = os.path.join(ROOT, "tests", "whirl")


def run(path_or_text, stdin=False):
    r = subprocess.run([TOOL, "-" if stdin else path_or_text], input=path_or_text if stdin else None,
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    recs = [json.loads(line) for line in r.stdout.splitlines() if line.startswith("{\"function\"")]
    return recs, r.stdout, r.stderr


def test_fixtures_are_what_the_script_writes(built, tmp_path):
    names = ("matmul_f90.whirl.txt", "linear_relu.whirl.txt", "matmul_intrinsic.whirl.txt")
    for name in names:
        assert os.path.exists(os.path.join(DUMPS, name))
    before = {n: open(os.path.join(DUMPS, n)).read() for n in names}
    subprocess.run([sys.executable, os.path.join(DUMPS, "make_dumps.py")], check=True)
    for n, text in before.items():
        assert open(os.path.join(DUMPS, n)).read() == text


def test_fortran_matmul_nests(built):
    recs, out, err = run(os.path.join(DUMPS, "matmul_f90.whirl.txt"))
    assert "3 nests recognised" in err
    by = {r["function"]: r for r in recs}
    assert set(by) == {"mm_const_", "mm_dummy_", "mm_int_bt_"}          # not_mm_ multiplies A by itself
    c = by["mm_const_"]
    # column-major A(300,200), B(200,260), C(300,260): element (i,l) of A at i + 300 l, and so on
    assert (c["kind"], c["m"], c["n"], c["k"]) == ("s4", "300", "260", "200")
    assert (c["A"]["inc1"], c["A"]["inc2"], c["B"]["inc1"], c["B"]["inc2"], c["C"]["inc1"], c["C"]["inc2"]) == \
        ("1", "300", "1", "200", "1", "300")
    d = by["mm_dummy_"]
    assert (d["kind"], d["m"], d["n"], d["k"]) == ("s", "m", "n", "kk") and d["A"]["inc2"] == "m" and d["B"]["inc2"] == "kk"
    t = by["mm_int_bt_"]
    assert t["kind"] == "i4" and (t["B"]["inc1"], t["B"]["inc2"]) == ("260", "1")   # the transposed operand
    assert "_s4gemmx__(&m_, &n_, &k_, &one, a_, &a1, &a2, b_, &b1, &b2, &zero, c_, &c1, &c2);" in out
    assert "_sgemmx__(" in out and "_i4gemmx__(" in out


def test_fused_linear_with_bias_and_relu(built):
    recs, out, _ = run(os.path.join(DUMPS, "linear_relu.whirl.txt"))
    assert len(recs) == 1
    r = recs[0]
    assert (r["m"], r["n"], r["k"], r["bias"], r["relu"]) == ("192", "160", "224", "bias", True)
    assert "o64_linear_f32(h, 192, 160, 224, A, 224, B, 160, bias, Y, 160, O64_ACT_RELU, stream);" in out


def test_damaged_and_foreign_input(built):
    text = open(os.path.join(DUMPS, "linear_relu.whirl.txt")).read()
    # a loop that does not start at zero is not create_doloop's loop
    recs, _, _ = run(text.replace("   I4INTCONST 0 (0x0)\n  I4STID 74", "   I4INTCONST 1 (0x1)\n  I4STID 74", 1), stdin=True)
    assert recs == []
    # a step of two
    recs, _, _ = run(text.replace("    I4INTCONST 1 (0x1)\n   I4ADD\n  I4STID 74", "    I4INTCONST 2 (0x2)\n   I4ADD\n  I4STID 74", 1), stdin=True)
    assert recs == []
    # a truncated file and plain prose do no harm
    recs, _, err = run(text[: len(text) // 2], stdin=True)
    assert recs == [] and "0 nests" in err
    recs, _, err = run("this is not WHIRL\n BLOCK\n", stdin=True)
    assert recs == []


def test_matmul_still_an_intrinsic(built):
    """The WHIRL the lowering pass receives: MATMUL as an INTRINSIC_OP over two PARMs.  The tool names the
    operands and the runtime entry point that takes their dope vectors."""
    recs, out, err = run(os.path.join(DUMPS, "matmul_intrinsic.whirl.txt"))
    assert "0 nests recognised, 2 MATMUL intrinsics" in err
    by = {r["function"]: r for r in recs}
    assert set(by) == {"mm_intrinsic_", "mm_intrinsic_r8_"}            # mm_in_place_ writes over its operand
    assert by["mm_intrinsic_"] == {"function": "mm_intrinsic_", "intrinsic": "MATMUL", "kind": "S4", "A": "a_", "B": "b_", "C": "c_"}
    assert by["mm_intrinsic_r8_"]["kind"] == "S"
    assert "_MATMUL_S4S4(&c__dope, &a__dope, &b__dope);" in out and "_MATMUL_SS(&r__dope, &p__dope, &q__dope);" in out
