"""Writes the WHIRL dumps under tests/whirl/ (run from the repository root: python tests/whirl/make_dumps.py).

No front end of the reference can be built here, so the dumps are derived by hand from the two sides that
fix them: the nest lower_mm_matmul builds (osprey/be/vho/f90_lower.cxx:5116-5178, loops as create_doloop
makes them, :4027-4092, nested by create_doloop_nest, :4095-4115) and the format the reference's ASCII
writer prints WHIRL in (ir_put_wn / ir_put_stmt, osprey/common/com/ir_reader.cxx:976-1560: operands above
their operator, one more space of indent per level; DO_LOOP with INIT / COMP / INCR / BODY markers; BLOCK
closed by END_BLOCK; symbols as <level,index,name>, types as T<index,name,align>, pregs named after '#').
Fortran arrays arrive with their subscripts reversed (the last WHIRL dimension is the first Fortran one).
"""
import os

HERE = os.path.dirname(os.path.abspath(__file__))

TY = {"F4": "T<10,.predef_F4,4>", "F8": "T<11,.predef_F8,8>", "I4": "T<4,.predef_I4,4>", "I8": "T<5,.predef_I8,8>"}
PREG = {"F4": "<1,6,.preg_F4>", "F8": "<1,7,.preg_F8>", "I4": "<1,4,.preg_I4>", "I8": "<1,5,.preg_I8>"}
ESIZE = {"F4": 4, "F8": 8, "I4": 4, "I8": 8}


class W:
    def __init__(self):
        self.lines = []

    def put(self, indent, text):
        self.lines.append(" " * indent + text)


def ldid_preg(w, d, ty, num, name):
    w.put(d, f"{ty}{ty}LDID {num} {PREG[ty]} {TY[ty]} # {name}")


def intconst(w, d, v):
    w.put(d, f"I4INTCONST {v} (0x{v:x})")


def count(w, d, c):
    """A trip count: a constant, or a dummy argument loaded through its address."""
    if isinstance(c, int):
        intconst(w, d, c)
    else:
        w.put(d, f"I4I4LDID 0 <2,{c[1]},{c[0]}> {TY['I4']}")


def do_loop(w, d, num, name, cnt, body):
    """create_doloop: index from 0 while index <= count - 1, step 1."""
    w.put(d, "DO_LOOP")
    w.put(d + 1, f"IDNAME {num} {PREG['I4']}")
    w.put(d, "INIT")
    intconst(w, d + 2, 0)
    w.put(d + 1, f"I4STID {num} {PREG['I4']} {TY['I4']} # {name}")
    w.put(d, "COMP")
    ldid_preg(w, d + 2, "I4", num, name)
    count(w, d + 3, cnt)
    intconst(w, d + 3, 1)
    w.put(d + 2, "I4SUB")
    w.put(d + 1, "I4I4LE")
    w.put(d, "INCR")
    ldid_preg(w, d + 3, "I4", num, name)
    intconst(w, d + 3, 1)
    w.put(d + 2, "I4ADD")
    w.put(d + 1, f"I4STID {num} {PREG['I4']} {TY['I4']} # {name}")
    w.put(d, "BODY")
    w.put(d + 1, "BLOCK")
    body(d + 1)
    w.put(d + 1, "END_BLOCK")


def array(w, d, ty, sym, dims, idx):
    """U8ARRAY ndim esize: base, the extents, the subscripts (slowest dimension first)."""
    w.put(d + 1, f"U8LDA 0 <1,{sym[1]},{sym[0]}> T<{60 + sym[1]},anon_ptr.,8>")
    for c in dims:
        count(w, d + 1, c)
    for num, name in idx:
        ldid_preg(w, d + 1, "I4", num, name)
    w.put(d, f"U8ARRAY {len(dims)} {ESIZE[ty]}")


def iload(w, d, ty, sym, dims, idx):
    array(w, d + 1, ty, sym, dims, idx)
    w.put(d, f"{ty}{ty}ILOAD 0 {TY[ty]} T<{60 + sym[1]},anon_ptr.,8>")


def matmul_nest(w, d, ty, A, B, R, m, n, k, a_sub, b_sub, r_sub="ji", bias=None, relu=False):
    """The two result loops around lower_mm_matmul's accumulation.  A, B, R: (name, symbol index, dims).
    a_sub / b_sub / r_sub: which of 'i', 'j', 'k' subscripts the slower and the faster dimension; the
    loop of the result's faster subscript is the inner one (Fortran R(i,j): r_sub 'ji', i inner)."""
    L1, L0, LK, ACC = (74, "@f90li_1_1"), (75, "@f90li_0_1"), (76, "@f90_mmidx_2"), (77, "@f90mm_3")
    var = {r_sub[0]: L1, r_sub[1]: L0, "k": LK}
    outer_count, inner_count = (n, m) if r_sub == "ji" else (m, n)

    def inner(dk):
        ldid_preg(w, dk + 2, ty, ACC[0], ACC[1])
        iload(w, dk + 3, ty, A[:2], A[2], [var[a_sub[0]], var[a_sub[1]]])
        iload(w, dk + 3, ty, B[:2], B[2], [var[b_sub[0]], var[b_sub[1]]])
        w.put(dk + 2, f"{ty}MPY")
        w.put(dk + 1, f"{ty}ADD")
        w.put(dk, f"{ty}STID {ACC[0]} {PREG[ty]} {TY[ty]} # {ACC[1]}")

    def body0(d0):
        if ty in ("F4", "F8"):
            w.put(d0 + 1, f"{ty}CONST <1,20,0.000000000000>")
        else:
            intconst(w, d0 + 1, 0)
        w.put(d0, f"{ty}STID {ACC[0]} {PREG[ty]} {TY[ty]} # {ACC[1]}")
        do_loop(w, d0, LK[0], LK[1], k, inner)
        # the store of the result element, with the optional tail max(acc + bias(i), 0)
        if bias:
            ldid_preg(w, d0 + (3 if relu else 2), ty, ACC[0], ACC[1])
            dd = d0 + (3 if relu else 2)
            w.put(dd + 2, f"U8LDA 0 <1,{bias[1]},{bias[0]}> T<{60 + bias[1]},anon_ptr.,8>")
            count(w, dd + 2, bias[2])
            ldid_preg(w, dd + 2, "I4", *var["j"])
            w.put(dd + 1, f"U8ARRAY 1 {ESIZE[ty]}")
            w.put(dd, f"{ty}{ty}ILOAD 0 {TY[ty]} T<{60 + bias[1]},anon_ptr.,8>")
            w.put(dd - 1, f"{ty}ADD")
            if relu:
                w.put(d0 + 2, f"{ty}CONST <1,20,0.000000000000>")
                w.put(d0 + 1, f"{ty}MAX")
        else:
            ldid_preg(w, d0 + 1, ty, ACC[0], ACC[1])
        array(w, d0 + 1, ty, R[:2], R[2], [var[r_sub[0]], var[r_sub[1]]])
        w.put(d0, f"{ty}ISTORE 0 T<{60 + R[1]},anon_ptr.,8>")

    do_loop(w, d, L1[0], L1[1], outer_count, lambda d1: do_loop(w, d1, L0[0], L0[1], inner_count, body0))


def function(w, name, body):
    w.put(0, f" LOC 1 1")
    w.put(0, f"FUNC_ENTRY <1,51,{name}>")
    w.put(0, "BODY")
    w.put(1, "BLOCK")
    w.put(1, "END_BLOCK")
    w.put(1, "BLOCK")
    w.put(1, "END_BLOCK")
    w.put(1, "BLOCK")
    w.put(1, "PRAGMA 0 120 <null-st> 0 (0x0) # PREAMBLE_END")
    body(1)
    w.put(1, "RETURN")
    w.put(1, "END_BLOCK")


def matmul_intrinsic(w, d, ty, A, B, R):
    """R = MATMUL(A, B) as the front end leaves it for the lowering pass (fei_matmul, osprey/crayf90/sgi/
    cwh_intrin.cxx:1168-1201): INTRINSIC_OP INTRN_MATMUL over two value PARMs, wrapped in an ARRAYEXP and
    stored through the result's section.  The operands' own subtrees (whole-array sections: ARRSECTION over
    LDA with one TRIPLET per dimension, loaded and wrapped in ARRAYEXP) are schematic: the node kinds and
    their order follow the WHIRL definitions of those operators (kids of ARRSECTION: base, extents,
    subscripts; kids of TRIPLET: first value, stride, count; kids of ARRAYEXP: value, extents), the
    intrinsic's number is a placeholder."""
    def section(dd, X):
        name, idx, dims = X
        w.put(dd + 1, f"U8LDA 0 <1,{idx},{name}> T<{60 + idx},anon_ptr.,8>")
        for e in dims:
            intconst(w, dd + 1, e)
        for e in dims:
            intconst(w, dd + 2, 0)
            intconst(w, dd + 2, 1)
            intconst(w, dd + 2, e)
            w.put(dd + 1, "I4TRIPLET")
        w.put(dd, f"U8ARRSECTION {len(dims)} {ESIZE[ty]}")

    def operand(dd, X):
        section(dd + 3, X)
        w.put(dd + 2, f"{ty}{ty}ILOAD 0 {TY[ty]} T<{60 + X[1]},anon_ptr.,8>")
        for e in X[2]:
            intconst(w, dd + 2, e)
        w.put(dd + 1, f"{ty}ARRAYEXP {len(X[2]) + 1}")
        w.put(dd, f"{ty}PARM 2 {TY[ty]} #  by_value")

    operand(d + 3, A)
    operand(d + 3, B)
    w.put(d + 2, f"{ty}INTRINSIC_OP 2 <0,MATMUL> 0")
    for e in R[2]:
        intconst(w, d + 2, e)
    w.put(d + 1, f"{ty}ARRAYEXP {len(R[2]) + 1}")
    section(d + 1, R)
    w.put(d, f"{ty}ISTORE 0 T<{60 + R[1]},anon_ptr.,8>")


def main():
    # MATMUL still as an intrinsic (the WHIRL the lowering pass receives)
    w = W()
    function(w, "mm_intrinsic_", lambda d: matmul_intrinsic(
        w, d, "F4", ("a_", 41, [200, 300]), ("b_", 42, [260, 200]), ("c_", 43, [260, 300])))
    function(w, "mm_intrinsic_r8_", lambda d: matmul_intrinsic(
        w, d, "F8", ("p_", 44, [70, 90]), ("q_", 45, [50, 70]), ("r_", 46, [50, 90])))
    # the result is also an operand: A = MATMUL(A, B) needs a temporary, the entry point cannot be bound as is
    function(w, "mm_in_place_", lambda d: matmul_intrinsic(
        w, d, "F4", ("a_", 41, [200, 200]), ("b_", 42, [200, 200]), ("a_", 41, [200, 200])))
    with open(os.path.join(HERE, "matmul_intrinsic.whirl.txt"), "w") as f:
        f.write("\n".join(w.lines) + "\n")
    w = W()
    # C = MATMUL(A, B), REAL*4, constant extents: A(300,200), B(200,260), C(300,260); WHIRL dims reversed
    function(w, "mm_const_", lambda d: matmul_nest(
        w, d, "F4", ("a_", 41, [200, 300]), ("b_", 42, [260, 200]), ("c_", 43, [260, 300]), 300, 260, 200, "ki", "jk"))
    # REAL*8 with extents that are dummy arguments (loaded, not constant)
    M, N, K = ("m", 3), ("n", 4), ("kk", 5)
    function(w, "mm_dummy_", lambda d: matmul_nest(
        w, d, "F8", ("a", 6, [K, M]), ("b", 7, [N, K]), ("r", 8, [N, M]), M, N, K, "ki", "jk"))
    # INTEGER*4, B given transposed (MATMUL(A, TRANSPOSE(BT)) lowered to subscripts): BT(260,200)
    function(w, "mm_int_bt_", lambda d: matmul_nest(
        w, d, "I4", ("ia_", 44, [200, 300]), ("ibt_", 45, [200, 260]), ("ic_", 46, [260, 300]), 300, 260, 200, "ki", "kj"))
    # a nest that only looks like one: the accumulation multiplies A by itself with the same subscripts
    function(w, "not_mm_", lambda d: matmul_nest(
        w, d, "F4", ("a_", 41, [200, 300]), ("a_", 41, [200, 300]), ("c_", 43, [260, 300]), 300, 260, 200, "ki", "ki"))
    with open(os.path.join(HERE, "matmul_f90.whirl.txt"), "w") as f:
        f.write("\n".join(w.lines) + "\n")
    # the C-style fused linear: row-major Y[i][j] = max(acc + bias[j], 0); here R's inner subscript is j
    w = W()
    function(w, "linear_relu", lambda d: matmul_nest(
        w, d, "F4", ("A", 51, [192, 224]), ("B", 52, [224, 160]), ("Y", 53, [192, 160]), 192, 160, 224, "ik", "kj",
        r_sub="ij", bias=("bias", 54, 160), relu=True))
    with open(os.path.join(HERE, "linear_relu.whirl.txt"), "w") as f:
        f.write("\n".join(w.lines) + "\n")


if __name__ == "__main__":
    main()
