// o64nest: rewrites GEMM-shaped loop nests in C source into calls of the GEMM engine.
//
// The reference compiler can print its intermediate form back as C (whirl2c: a DO_LOOP becomes
// `for(i = lb; i <= ub; i = i + 1)`, osprey/be/whirl2c/wn2c.cxx:4078-4118).  This tool is the
// other half of that seam: it reads such C (or hand-written C of the same shape), finds the
// nest the reference builds for a matrix product (osprey/be/vho/f90_lower.cxx:5149-5169: an
// accumulator zeroed, one inner loop over K, acc = acc + a*b) with an optional bias / ReLU tail,
// and replaces it by one call into libo64gemm.so.  Everything else is copied through.
//
// Recognised (any spacing, redundant parentheses, `x = x + 1` / `x++` / `x += 1` steps, `<` or
// `<=` bounds, any lower bound that does not depend on the loop's own variable):
//
//     for (i ...)  for (j ...) { acc = 0; for (k ...) acc = acc + A[i][k] * B[k][j];
//                                Y[i][j] = acc;  |  acc + bias[j];  |  max(acc + bias[j], 0); }
//     for (i ...)  for (j ...) { C[i][j] = 0; for (k ...) C[i][j] = C[i][j] + A[i][k] * B[k][j]; }
//
// with 2-D subscripts on arrays declared in the same file (`float A[512][512]`, parameters
// `float A[][512]`, `float (*A)[512]`) or flattened subscripts `A[i*lda + k]`.
//   float, plain layout, any tail      -> o64_linear_f32 (bias and ReLU fused)
//   float / double / int / long long,
//   any layout (transposed operands),
//   no tail                            -> _s4gemmx__ / _sgemmx__ / _i4gemmx__ / _jgemmx__ (strides)
//
// Loop pragmas of the reference (osprey/common/com/wn_pragmas.h:143-151, applied per loop in
// osprey/be/lno/ff_pragmas.cxx:279-300) in front of a loop of the nest:
//   #pragma blocking size (n1[, n2])  on the i loop: tile_m = n1, L2 group = n2 / n1 tiles
//                                     on the j loop: tile_n = n1;  on the k loop: tile_k = n1
//   #pragma interchange (j, i, ...)   raster: N fastest
// become an o64_plan_set call in front of the product (the engine rejects sizes it has no
// kernel for; the emitted code then falls back to the automatic plan).
//
// Tails: besides max(x, 0) the elementwise functions the reference lowers through its exp / tanh
// intrinsics (osprey/common/com/intrn_entry.def:915,1346): x / (1 + expf(-x)) (SiLU),
// 0.5 x (1 + tanhf(0.79788456 (x + 0.044715 x^3))) and 0.5 x (1 + erff(0.70710678 x)) (GELU), on
// x = acc or acc + bias[j], written inline or through one temporary (t = acc + bias[j]; Y = f(t);).
//
// Nests the reference has ALREADY tiled are recognised too.  After scalar expansion and distribution the
// accumulation is a perfect nest around  C[i][j] = C[i][j] + A[i][k] * B[k][j]  (snl_test.cxx:1036-1040);
// cache blocking (SNL_INV_Cache_Block, osprey/be/lno/snl_inv.cxx:639-887) then puts strip loops
// `for (it = 0; it <= ub; it = it + B)` outside and rewrites the blocked loop as
// `for (i = it; i <= _I4MIN(it + (B - 1), ub); i = i + 1)` (snl_inv.cxx:774-805; whirl2c prints OPR_MIN
// as _I4MIN, osprey/be/whirl2c/wn2c.cxx:658), in any loop order.  Such a nest - any permutation of the
// three element loops, any subset of them strip-mined - becomes ONE accumulating call of the strided
// kernel (beta = 1: the zeroing nest in front stays as it is), and the strip sizes it was blocked with
// are handed on as plan pins of the fp32 kernel (o64_plan_set on o64_compat_handle()).
//
//   o64nest input.c [-o output.c]       ("-" or no input: stdin; no -o: stdout)
//   exit status: 0, also when nothing was recognised (the count goes to stderr); 2 on usage errors
#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

namespace {

// ------------------------------------------------------------------------------------------
// tokens
// ------------------------------------------------------------------------------------------
struct Tok {
    enum Kind { Id, Num, Punct, Pragma, End } kind;
    std::string text;
    size_t begin, end;  // byte range in the source
};

std::vector<Tok> tokenize(const std::string &s) {
    std::vector<Tok> out;
    size_t i = 0;
    const size_t n = s.size();
    bool line_start = true;
    while (i < n) {
        const char c = s[i];
        if (c == '\n') {
            line_start = true;
            ++i;
        } else if (isspace((unsigned char)c)) {
            ++i;
        } else if (c == '/' && i + 1 < n && s[i + 1] == '/') {
            while (i < n && s[i] != '\n') ++i;
        } else if (c == '/' && i + 1 < n && s[i + 1] == '*') {
            i += 2;
            while (i + 1 < n && !(s[i] == '*' && s[i + 1] == '/')) ++i;
            i = i + 2 <= n ? i + 2 : n;
        } else if (c == '#' && line_start) {
            const size_t b = i;
            while (i < n && s[i] != '\n') {
                if (s[i] == '\\' && i + 1 < n && s[i + 1] == '\n') ++i;
                ++i;
            }
            std::string text = s.substr(b, i - b);
            out.push_back({text.find("pragma") != std::string::npos ? Tok::Pragma : Tok::Punct, text, b, i});
            if (out.back().kind == Tok::Punct) out.back().text = "#";  // other directives: opaque
        } else if (c == '"' || c == '\'') {
            const size_t b = i++;
            while (i < n && s[i] != c) {
                if (s[i] == '\\') ++i;
                ++i;
            }
            ++i;
            out.push_back({Tok::Punct, "\"", b, i});
            line_start = false;
        } else if (isalpha((unsigned char)c) || c == '_') {
            const size_t b = i;
            while (i < n && (isalnum((unsigned char)s[i]) || s[i] == '_')) ++i;
            out.push_back({Tok::Id, s.substr(b, i - b), b, i});
            line_start = false;
        } else if (isdigit((unsigned char)c) || (c == '.' && i + 1 < n && isdigit((unsigned char)s[i + 1]))) {
            const size_t b = i;
            while (i < n && (isalnum((unsigned char)s[i]) || s[i] == '.' ||
                             ((s[i] == '+' || s[i] == '-') && (s[i - 1] == 'e' || s[i - 1] == 'E'))))
                ++i;
            out.push_back({Tok::Num, s.substr(b, i - b), b, i});
            line_start = false;
        } else {
            static const char *two[] = {"<=", ">=", "==", "!=", "++", "--", "+=", "-=", "*=", "&&", "||", "->"};
            std::string p(1, c);
            for (const char *t : two)
                if (i + 1 < n && s[i] == t[0] && s[i + 1] == t[1]) p = t;
            out.push_back({Tok::Punct, p, i, i + p.size()});
            i += p.size();
            line_start = false;
        }
    }
    out.push_back({Tok::End, "", n, n});
    return out;
}

// ------------------------------------------------------------------------------------------
// expressions
// ------------------------------------------------------------------------------------------
struct Expr;
typedef std::shared_ptr<Expr> ExprP;
struct Expr {
    enum Kind { Num, Id, Index, Bin, Neg, Call, Cond } kind;
    std::string text;          // Num / Id: spelling; Bin: operator; Call: callee
    std::vector<ExprP> kids;   // Index: base, subscript; Bin: lhs, rhs; Cond: test, then, else
};

ExprP mk(Expr::Kind k, const std::string &t, std::vector<ExprP> kids = {}) {
    auto e = std::make_shared<Expr>();
    e->kind = k;
    e->text = t;
    e->kids = std::move(kids);
    return e;
}

struct Parser {
    const std::vector<Tok> &t;
    size_t p;
    bool ok = true;
    Parser(const std::vector<Tok> &toks, size_t pos) : t(toks), p(pos) {}
    bool is(const char *s) const { return t[p].kind == Tok::Punct && t[p].text == s; }
    bool accept(const char *s) {
        if (is(s)) {
            ++p;
            return true;
        }
        return false;
    }
    void expect(const char *s) {
        if (!accept(s)) ok = false;
    }

    ExprP primary() {
        if (!ok) return nullptr;
        ExprP e;
        if (accept("(")) {
            // a cast such as (float) or (_IEEE32): skip it
            if (t[p].kind == Tok::Id && t[p + 1].kind == Tok::Punct && t[p + 1].text == ")" && is_type(t[p].text)) {
                p += 2;
                return unary();
            }
            e = ternary();
            expect(")");
        } else if (t[p].kind == Tok::Num) {
            e = mk(Expr::Num, t[p++].text);
        } else if (t[p].kind == Tok::Id) {
            e = mk(Expr::Id, t[p++].text);
            if (accept("(")) {
                std::vector<ExprP> args;
                if (!is(")")) {
                    do args.push_back(ternary());
                    while (accept(","));
                }
                expect(")");
                e = mk(Expr::Call, e->text, args);
            }
        } else {
            ok = false;
            return nullptr;
        }
        while (ok && accept("[")) {
            ExprP sub = ternary();
            expect("]");
            e = mk(Expr::Index, "", {e, sub});
        }
        return e;
    }
    ExprP unary() {
        if (accept("-")) return mk(Expr::Neg, "-", {unary()});
        if (accept("+")) return unary();
        return primary();
    }
    ExprP mul() {
        ExprP e = unary();
        while (ok && (is("*") || is("/"))) {
            std::string op = t[p++].text;
            e = mk(Expr::Bin, op, {e, unary()});
        }
        return e;
    }
    ExprP add() {
        ExprP e = mul();
        while (ok && (is("+") || is("-"))) {
            std::string op = t[p++].text;
            e = mk(Expr::Bin, op, {e, mul()});
        }
        return e;
    }
    ExprP rel() {
        ExprP e = add();
        while (ok && (is("<") || is(">") || is("<=") || is(">="))) {
            std::string op = t[p++].text;
            e = mk(Expr::Bin, op, {e, add()});
        }
        return e;
    }
    ExprP ternary() {
        ExprP e = rel();
        if (ok && accept("?")) {
            ExprP a = ternary();
            expect(":");
            ExprP b = ternary();
            e = mk(Expr::Cond, "?", {e, a, b});
        }
        return e;
    }
    static bool is_type(const std::string &s) {
        static const char *names[] = {"float", "double", "int", "long", "_IEEE32", "_IEEE64", "_INT32", "_INT64"};
        for (const char *n : names)
            if (s == n) return true;
        return false;
    }
};

std::string str(const ExprP &e) {
    if (!e) return "?";
    switch (e->kind) {
    case Expr::Num:
    case Expr::Id: return e->text;
    case Expr::Index: return str(e->kids[0]) + "[" + str(e->kids[1]) + "]";
    case Expr::Bin: return "(" + str(e->kids[0]) + " " + e->text + " " + str(e->kids[1]) + ")";
    case Expr::Neg: return "(-" + str(e->kids[0]) + ")";
    case Expr::Call: {
        std::string s = e->text + "(";
        for (size_t i = 0; i < e->kids.size(); ++i) s += (i ? ", " : "") + str(e->kids[i]);
        return s + ")";
    }
    case Expr::Cond: return "(" + str(e->kids[0]) + " ? " + str(e->kids[1]) + " : " + str(e->kids[2]) + ")";
    }
    return "?";
}

bool is_id(const ExprP &e, const std::string &name) { return e && e->kind == Expr::Id && e->text == name; }
bool is_zero(const ExprP &e) {
    if (!e || e->kind != Expr::Num) return false;
    return atof(e->text.c_str()) == 0.0 && e->text.find_first_of("123456789") == std::string::npos;
}
bool is_one(const ExprP &e) { return e && e->kind == Expr::Num && atoll(e->text.c_str()) == 1 && atof(e->text.c_str()) == 1.0; }
bool same(const ExprP &a, const ExprP &b) { return str(a) == str(b); }
bool mentions(const ExprP &e, const std::string &v) {
    if (!e) return false;
    if (e->kind == Expr::Id) return e->text == v;
    for (const ExprP &k : e->kids)
        if (mentions(k, v)) return true;
    return false;
}

// ------------------------------------------------------------------------------------------
// declarations: element type and row pitch of 2-D arrays
// ------------------------------------------------------------------------------------------
struct ArrayDecl {
    std::string type;  // "f32", "f64", "i32", "i64"
    std::string ld;    // inner extent as written; empty for pointers / 1-D arrays
};

std::string type_code(const std::vector<std::string> &words) {
    int longs = 0;
    bool f = false, d = false, i = false;
    for (const std::string &w : words) {
        if (w == "float" || w == "_IEEE32") f = true;
        else if (w == "double" || w == "_IEEE64") d = true;
        else if (w == "int" || w == "_INT32") i = true;
        else if (w == "long") ++longs;
        else if (w == "_INT64") longs = 2;
    }
    if (f) return "f32";
    if (d) return "f64";
    if (longs >= 1) return "i64";  // LP64: long and long long are 64 bits
    if (i) return "i32";
    return "";
}

std::map<std::string, ArrayDecl> scan_decls(const std::vector<Tok> &t) {
    std::map<std::string, ArrayDecl> out;
    for (size_t p = 0; p + 1 < t.size(); ++p) {
        if (t[p].kind != Tok::Id || !Parser::is_type(t[p].text)) continue;
        std::vector<std::string> words;
        size_t q = p;
        while (t[q].kind == Tok::Id && (Parser::is_type(t[q].text) || t[q].text == "const" || t[q].text == "unsigned" ||
                                        t[q].text == "signed" || t[q].text == "restrict" || t[q].text == "__restrict__" ||
                                        t[q].text == "static"))
            words.push_back(t[q++].text);
        const std::string type = type_code(words);
        if (type.empty()) continue;
        // declarators separated by commas, up to ';' ')' '{' or '='
        while (true) {
            bool ptr_to_array = false;
            while (t[q].kind == Tok::Punct && (t[q].text == "*" || t[q].text == "(")) {
                if (t[q].text == "(") ptr_to_array = true;
                ++q;
            }
            while (t[q].kind == Tok::Id && (t[q].text == "const" || t[q].text == "restrict" || t[q].text == "__restrict__")) ++q;
            if (t[q].kind != Tok::Id) break;
            const std::string name = t[q++].text;
            if (ptr_to_array && t[q].kind == Tok::Punct && t[q].text == ")") ++q;
            std::vector<std::string> dims;
            while (t[q].kind == Tok::Punct && t[q].text == "[") {
                size_t r = q + 1;
                std::string d;
                int depth = 1;
                while (t[r].kind != Tok::End) {
                    if (t[r].kind == Tok::Punct && t[r].text == "[") ++depth;
                    if (t[r].kind == Tok::Punct && t[r].text == "]" && --depth == 0) break;
                    d += t[r++].text;
                }
                dims.push_back(d);
                q = r + 1;
            }
            ArrayDecl a;
            a.type = type;
            if (ptr_to_array && dims.size() == 1) a.ld = dims[0];      // T (*A)[LD]
            else if (dims.size() == 2) a.ld = dims[1];                 // T A[..][LD]
            out[name] = a;
            if (t[q].kind == Tok::Punct && t[q].text == ",") {
                // in a parameter list the next declarator starts with a type again: let the outer scan find it
                if (t[q + 1].kind == Tok::Id && Parser::is_type(t[q + 1].text)) break;
                if (t[q + 1].kind == Tok::Id && t[q + 1].text == "const") break;
                ++q;
                continue;
            }
            break;
        }
    }
    return out;
}

std::string strip_suffix(const std::string &num) {  // 512LL -> 512
    size_t e = num.size();
    while (e > 0 && (num[e - 1] == 'L' || num[e - 1] == 'l' || num[e - 1] == 'U' || num[e - 1] == 'u')) --e;
    return num.substr(0, e);
}

// ------------------------------------------------------------------------------------------
// loops and the nest
// ------------------------------------------------------------------------------------------
struct Loop {
    std::string var;
    ExprP lb;         // first value (0 in the nest the reference builds; a section's first index otherwise)
    ExprP ub;         // exclusive bound when !inclusive
    bool inclusive = false;
    std::vector<std::string> pragmas;  // in front of this loop
    size_t body;      // first token of the body
};

void take_pragmas(const std::vector<Tok> &t, size_t &p, std::vector<std::string> *out) {
    while (t[p].kind == Tok::Pragma) out->push_back(t[p++].text);
}

// for ( v = lb ; v < ub ; step ), lb free of v   -- leaves p on the first token of the body
bool parse_for(const std::vector<Tok> &t, size_t &p, Loop *L) {
    if (!(t[p].kind == Tok::Id && t[p].text == "for")) return false;
    Parser ps(t, p + 1);
    ps.expect("(");
    if (ps.t[ps.p].kind == Tok::Id && Parser::is_type(ps.t[ps.p].text)) ++ps.p;  // for (int i = ...
    if (ps.t[ps.p].kind != Tok::Id) return false;
    L->var = ps.t[ps.p++].text;
    ps.expect("=");
    ExprP lb = ps.ternary();
    ps.expect(";");
    ExprP test = ps.ternary();
    ps.expect(";");
    if (!ps.ok || !lb || mentions(lb, L->var) || !test || test->kind != Expr::Bin || !is_id(test->kids[0], L->var)) return false;
    L->lb = lb;
    if (test->text == "<=") L->inclusive = true;
    else if (test->text != "<") return false;
    L->ub = test->kids[1];
    if (mentions(L->ub, L->var)) return false;
    // step
    if (ps.accept("++") || ps.accept("--")) {
        if (ps.t[ps.p - 1].text != "++" || !(ps.t[ps.p].kind == Tok::Id && ps.t[ps.p].text == L->var)) return false;
        ++ps.p;
    } else {
        if (!(ps.t[ps.p].kind == Tok::Id && ps.t[ps.p].text == L->var)) return false;
        ++ps.p;
        if (ps.accept("++")) {
        } else if (ps.accept("+=")) {
            if (!is_one(ps.ternary())) return false;
        } else if (ps.accept("=")) {
            ExprP e = ps.ternary();
            if (!e || e->kind != Expr::Bin || e->text != "+") return false;
            const bool a = is_id(e->kids[0], L->var) && is_one(e->kids[1]);
            const bool b = is_id(e->kids[1], L->var) && is_one(e->kids[0]);
            if (!a && !b) return false;
        } else {
            return false;
        }
    }
    ps.expect(")");
    if (!ps.ok) return false;
    p = ps.p;
    L->body = p;
    return true;
}


// A DO loop in the shapes whirl2c prints: for (v = lb; v <= ub; v = v + step) with a constant step.
struct GLoop {
    std::string var;
    ExprP lb, ub;
    bool inclusive = false;
    long long step = 1;
    std::vector<std::string> pragmas;
};

bool const_int(const ExprP &e, long long *v) {
    if (!e) return false;
    if (e->kind == Expr::Num && e->text.find_first_of(".eE") == std::string::npos) {
        *v = atoll(strip_suffix(e->text).c_str());
        return true;
    }
    long long a, b;
    if (e->kind == Expr::Bin && const_int(e->kids[0], &a) && const_int(e->kids[1], &b)) {
        if (e->text == "+") *v = a + b;
        else if (e->text == "-") *v = a - b;
        else if (e->text == "*") *v = a * b;
        else return false;
        return true;
    }
    return false;
}

bool parse_for_general(const std::vector<Tok> &t, size_t &p, GLoop *L) {
    if (!(t[p].kind == Tok::Id && t[p].text == "for")) return false;
    Parser ps(t, p + 1);
    ps.expect("(");
    if (ps.t[ps.p].kind == Tok::Id && Parser::is_type(ps.t[ps.p].text)) ++ps.p;
    if (ps.t[ps.p].kind != Tok::Id) return false;
    L->var = ps.t[ps.p++].text;
    ps.expect("=");
    L->lb = ps.ternary();
    ps.expect(";");
    ExprP test = ps.ternary();
    ps.expect(";");
    if (!ps.ok || !L->lb || !test || test->kind != Expr::Bin || !is_id(test->kids[0], L->var)) return false;
    if (test->text == "<=") L->inclusive = true;
    else if (test->text != "<") return false;
    L->ub = test->kids[1];
    if (mentions(L->ub, L->var) || mentions(L->lb, L->var)) return false;
    if (!(ps.t[ps.p].kind == Tok::Id && ps.t[ps.p].text == L->var)) {
        if (ps.accept("++") && ps.t[ps.p].kind == Tok::Id && ps.t[ps.p].text == L->var) {
            ++ps.p;
            L->step = 1;
        } else {
            return false;
        }
    } else {
        ++ps.p;
        if (ps.accept("++")) {
            L->step = 1;
        } else if (ps.accept("+=")) {
            if (!const_int(ps.ternary(), &L->step)) return false;
        } else if (ps.accept("=")) {
            ExprP e = ps.ternary();
            if (!e || e->kind != Expr::Bin || e->text != "+") return false;
            if (is_id(e->kids[0], L->var) && const_int(e->kids[1], &L->step)) {
            } else if (is_id(e->kids[1], L->var) && const_int(e->kids[0], &L->step)) {
            } else {
                return false;
            }
        } else {
            return false;
        }
    }
    ps.expect(")");
    if (!ps.ok || L->step < 1) return false;
    p = ps.p;
    return true;
}

// min(a, b) in the spellings it is printed in; false if e is no minimum
bool split_min(const ExprP &e, ExprP *a, ExprP *b) {
    if (!e) return false;
    if (e->kind == Expr::Call && e->kids.size() == 2) {
        static const char *names[] = {"_I4MIN", "_I8MIN", "_U4MIN", "_U8MIN", "min", "MIN", "_MIN"};
        for (const char *n : names)
            if (e->text == n) {
                *a = e->kids[0];
                *b = e->kids[1];
                return true;
            }
    }
    if (e->kind == Expr::Cond && e->kids[0]->kind == Expr::Bin && (e->kids[0]->text == "<" || e->kids[0]->text == "<=") &&
        same(e->kids[0]->kids[0], e->kids[1]) && same(e->kids[0]->kids[1], e->kids[2])) {
        *a = e->kids[1];
        *b = e->kids[2];
        return true;
    }
    return false;
}

// e == var + c (either order) or var: the constant
bool var_plus_const(const ExprP &e, const std::string &var, long long *c) {
    if (is_id(e, var)) {
        *c = 0;
        return true;
    }
    if (e && e->kind == Expr::Bin && e->text == "+") {
        if (is_id(e->kids[0], var) && const_int(e->kids[1], c)) return true;
        if (is_id(e->kids[1], var) && const_int(e->kids[0], c)) return true;
    }
    return false;
}

// One operand of the product: X[r][c] or X[r*LD + c]; on success name, row / column loop
// variables and the pitch.
struct Ref {
    std::string name, row, col, ld;
    ExprP whole;
};

bool affine2(const ExprP &e, const std::vector<std::string> &vars, std::string *row, std::string *col, std::string *ld) {
    // e == v1 * LD + v2  (any order, LD free of loop variables)
    if (!e || e->kind != Expr::Bin || e->text != "+") return false;
    for (int swap = 0; swap < 2; ++swap) {
        const ExprP &a = e->kids[swap], &b = e->kids[1 - swap];
        if (b->kind != Expr::Id) continue;
        if (a->kind != Expr::Bin || a->text != "*") continue;
        for (int s2 = 0; s2 < 2; ++s2) {
            const ExprP &v = a->kids[s2], &l = a->kids[1 - s2];
            if (v->kind != Expr::Id) continue;
            bool v_is_var = false, b_is_var = false, l_free = true;
            for (const std::string &x : vars) {
                v_is_var |= v->text == x;
                b_is_var |= b->text == x;
                l_free &= !mentions(l, x);
            }
            if (v_is_var && b_is_var && l_free && v->text != b->text) {
                *row = v->text;
                *col = b->text;
                *ld = l->kind == Expr::Num ? strip_suffix(l->text) : str(l);
                return true;
            }
        }
    }
    return false;
}

bool parse_ref(const ExprP &e, const std::vector<std::string> &vars, const std::map<std::string, ArrayDecl> &decls, Ref *r) {
    if (!e || e->kind != Expr::Index) return false;
    r->whole = e;
    const ExprP &base = e->kids[0];
    if (base->kind == Expr::Index && base->kids[0]->kind == Expr::Id) {  // X[r][c]
        r->name = base->kids[0]->text;
        if (base->kids[1]->kind != Expr::Id || e->kids[1]->kind != Expr::Id) return false;
        r->row = base->kids[1]->text;
        r->col = e->kids[1]->text;
        auto it = decls.find(r->name);
        if (it == decls.end() || it->second.ld.empty()) return false;
        r->ld = strip_suffix(it->second.ld);
        return r->row != r->col;
    }
    if (base->kind == Expr::Id) {  // X[r*LD + c]
        r->name = base->text;
        return affine2(e->kids[1], vars, &r->row, &r->col, &r->ld);
    }
    return false;
}

// statement: lhs = rhs ;   or   lhs += rhs ;
struct Assign {
    ExprP lhs, rhs;
    bool plus_equals = false;
};
bool parse_assign(const std::vector<Tok> &t, size_t &p, Assign *a) {
    Parser ps(t, p);
    // `float acc = 0;` declares and initialises the accumulator in one statement
    while (ps.t[ps.p].kind == Tok::Id && (Parser::is_type(ps.t[ps.p].text) || ps.t[ps.p].text == "register")) ++ps.p;
    a->lhs = ps.primary();
    if (!ps.ok || !a->lhs) return false;
    if (ps.accept("+=")) a->plus_equals = true;
    else if (!ps.accept("=")) return false;
    a->rhs = ps.ternary();
    ps.expect(";");
    if (!ps.ok) return false;
    p = ps.p;
    return true;
}

struct Nest {
    Loop li, lj, lk;
    Ref a, b, c;
    std::string type;      // element type of C
    std::string bias;      // name of the bias vector (indexed by j), or empty
    bool relu = false;
    int act = 0;           // 0 none, 1 ReLU, 2 GELU (tanh), 3 GELU (erf), 4 SiLU
    bool tail = false;     // bias or an activation present
    size_t tok_begin, tok_end;  // tokens [begin, end) to replace (pragmas in front included)
};

// x, or max(x, 0) in its spellings; returns the inner expression
ExprP strip_relu(const ExprP &e, bool *relu) {
    *relu = false;
    if (e && e->kind == Expr::Call && e->kids.size() == 2 &&
        (e->text == "max" || e->text == "MAX" || e->text == "_MAX" || e->text == "fmaxf" || e->text == "fmax")) {
        for (int s = 0; s < 2; ++s)
            if (is_zero(e->kids[s])) {
                *relu = true;
                return e->kids[1 - s];
            }
    }
    if (e && e->kind == Expr::Cond && e->kids[0]->kind == Expr::Bin) {  // x > 0 ? x : 0
        const ExprP &test = e->kids[0];
        if ((test->text == ">" || test->text == ">=") && is_zero(test->kids[1]) && same(test->kids[0], e->kids[1]) &&
            is_zero(e->kids[2])) {
            *relu = true;
            return e->kids[1];
        }
    }
    return e;
}


// ---- the elementwise tails ---------------------------------------------------------------------
void flatten_product(const ExprP &e, std::vector<ExprP> *out) {
    if (e && e->kind == Expr::Bin && e->text == "*") {
        flatten_product(e->kids[0], out);
        flatten_product(e->kids[1], out);
    } else {
        out->push_back(e);
    }
}
bool num_near(const ExprP &e, double v, double tol) {
    if (!e || e->kind != Expr::Num) return false;
    const double x = atof(e->text.c_str());
    return x > v - tol && x < v + tol;
}
bool call_named(const ExprP &e, std::initializer_list<const char *> names, size_t nargs) {
    if (!e || e->kind != Expr::Call || e->kids.size() != nargs) return false;
    for (const char *n : names)
        if (e->text == n) return true;
    return false;
}
// 1 + f  in either order: f
ExprP one_plus(const ExprP &e) {
    if (!e || e->kind != Expr::Bin || e->text != "+") return nullptr;
    if (num_near(e->kids[0], 1.0, 1e-9)) return e->kids[1];
    if (num_near(e->kids[1], 1.0, 1e-9)) return e->kids[0];
    return nullptr;
}
// x / (1 + exp(-x)): x
ExprP match_silu(const ExprP &e) {
    if (!e || e->kind != Expr::Bin || e->text != "/") return nullptr;
    const ExprP ex = one_plus(e->kids[1]);
    if (!call_named(ex, {"expf", "exp", "_F4EXP", "__expf"}, 1)) return nullptr;
    const ExprP &arg = ex->kids[0];
    if (!arg || arg->kind != Expr::Neg || !same(arg->kids[0], e->kids[0])) return nullptr;
    return e->kids[0];
}
// 0.5 * x * (1 + tanh(c1 * (x + c2 * x * x * x)))  or  0.5 * x * (1 + erf(x * c)): x and which
ExprP match_gelu(const ExprP &e, int *which) {
    std::vector<ExprP> f;
    flatten_product(e, &f);
    if (f.size() != 3) return nullptr;
    ExprP half, x, bracket;
    for (const ExprP &g : f) {
        if (!half && num_near(g, 0.5, 1e-9)) half = g;
        else if (!bracket && one_plus(g)) bracket = g;
        else if (!x) x = g;
    }
    if (!half || !x || !bracket) return nullptr;
    const ExprP fn = one_plus(bracket);
    if (call_named(fn, {"erff", "erf", "_F4ERF"}, 1)) {
        std::vector<ExprP> a;
        flatten_product(fn->kids[0], &a);
        if (a.size() == 2 && ((same(a[0], x) && num_near(a[1], 0.70710678, 1e-5)) || (same(a[1], x) && num_near(a[0], 0.70710678, 1e-5)))) {
            *which = 3;
            return x;
        }
        const ExprP &q = fn->kids[0];
        if (q->kind == Expr::Bin && q->text == "/" && same(q->kids[0], x) && num_near(q->kids[1], 1.41421356, 1e-5)) {
            *which = 3;
            return x;
        }
        return nullptr;
    }
    if (call_named(fn, {"tanhf", "tanh", "_F4TANH"}, 1)) {
        std::vector<ExprP> a;
        flatten_product(fn->kids[0], &a);
        if (a.size() != 2) return nullptr;
        ExprP sum = num_near(a[0], 0.7978845608, 1e-5) ? a[1] : (num_near(a[1], 0.7978845608, 1e-5) ? a[0] : nullptr);
        if (!sum || sum->kind != Expr::Bin || sum->text != "+") return nullptr;
        for (int sw = 0; sw < 2; ++sw) {
            if (!same(sum->kids[sw], x)) continue;
            std::vector<ExprP> c;
            flatten_product(sum->kids[1 - sw], &c);
            int xs = 0, cs = 0;
            for (const ExprP &g : c) {
                if (same(g, x)) ++xs;
                else if (num_near(g, 0.044715, 1e-6)) ++cs;
                else return nullptr;
            }
            if (xs == 3 && cs == 1) {
                *which = 2;
                return x;
            }
        }
    }
    return nullptr;
}
// the activation around x, if any: returns x and sets *act (0 none, 1 ReLU, 2 / 3 GELU, 4 SiLU)
ExprP strip_activation(const ExprP &e, int *act) {
    bool relu = false;
    ExprP v = strip_relu(e, &relu);
    if (relu) {
        *act = 1;
        return v;
    }
    if (ExprP x = match_silu(e)) {
        *act = 4;
        return x;
    }
    int which = 0;
    if (ExprP x = match_gelu(e, &which)) {
        *act = which;
        return x;
    }
    *act = 0;
    return e;
}

bool open_block(const std::vector<Tok> &t, size_t &p) {
    if (t[p].kind == Tok::Punct && t[p].text == "{") {
        ++p;
        return true;
    }
    return false;
}
bool close_block(const std::vector<Tok> &t, size_t &p, bool braced) {
    if (!braced) return true;
    if (t[p].kind == Tok::Punct && t[p].text == "}") {
        ++p;
        return true;
    }
    return false;
}

bool match_nest(const std::vector<Tok> &t, size_t start, const std::map<std::string, ArrayDecl> &decls, Nest *n) {
    size_t p = start;
    n->tok_begin = start;
    take_pragmas(t, p, &n->li.pragmas);
    if (!parse_for(t, p, &n->li)) return false;
    const bool bi = open_block(t, p);
    take_pragmas(t, p, &n->lj.pragmas);
    if (!parse_for(t, p, &n->lj)) return false;
    const bool bj = open_block(t, p);
    if (!bj) return false;  // the j body holds at least two statements
    Assign init;
    if (!parse_assign(t, p, &init) || init.plus_equals || !is_zero(init.rhs)) return false;
    take_pragmas(t, p, &n->lk.pragmas);
    if (!parse_for(t, p, &n->lk)) return false;
    const bool bk = open_block(t, p);
    Assign upd;
    if (!parse_assign(t, p, &upd)) return false;
    if (!close_block(t, p, bk)) return false;
    if (!same(upd.lhs, init.lhs)) return false;
    // acc = acc + a*b  |  acc = a*b + acc  |  acc += a*b
    ExprP prod = upd.rhs;
    if (!upd.plus_equals) {
        if (!prod || prod->kind != Expr::Bin || prod->text != "+") return false;
        if (same(prod->kids[0], init.lhs)) prod = prod->kids[1];
        else if (same(prod->kids[1], init.lhs)) prod = prod->kids[0];
        else return false;
    }
    if (!prod || prod->kind != Expr::Bin || prod->text != "*") return false;
    const std::vector<std::string> vars = {n->li.var, n->lj.var, n->lk.var};
    if (vars[0] == vars[1] || vars[0] == vars[2] || vars[1] == vars[2]) return false;
    // a rectangular iteration space only: no bound of one loop in terms of another loop's variable
    for (const Loop *L : {&n->li, &n->lj, &n->lk})
        for (const std::string &v : vars)
            if (mentions(L->lb, v) || mentions(L->ub, v)) return false;
    Ref r0, r1;
    if (!parse_ref(prod->kids[0], vars, decls, &r0) || !parse_ref(prod->kids[1], vars, decls, &r1)) return false;
    auto uses = [](const Ref &r, const std::string &x, const std::string &y) {
        return (r.row == x && r.col == y) || (r.row == y && r.col == x);
    };
    if (uses(r0, vars[0], vars[2]) && uses(r1, vars[2], vars[1])) {
        n->a = r0;
        n->b = r1;
    } else if (uses(r1, vars[0], vars[2]) && uses(r0, vars[2], vars[1])) {
        n->a = r1;
        n->b = r0;
    } else {
        return false;
    }
    // the store
    ExprP out_ref;
    if (init.lhs->kind == Expr::Id) {  // scalar accumulator: one more statement stores it
        Assign st;
        if (!parse_assign(t, p, &st) || st.plus_equals) return false;
        // x = acc or acc + bias[j]; sets n->bias
        auto pre_activation = [&](ExprP v) {
            if (v && v->kind == Expr::Bin && v->text == "+") {
                for (int s = 0; s < 2; ++s) {
                    const ExprP &x = v->kids[s], &y = v->kids[1 - s];
                    if (same(x, init.lhs) && y->kind == Expr::Index && y->kids[0]->kind == Expr::Id &&
                        is_id(y->kids[1], vars[1])) {
                        n->bias = y->kids[0]->text;
                        return true;
                    }
                }
            }
            return same(v, init.lhs);
        };
        ExprP temp;  // t = acc + bias[j];  in front of  Y = f(t);
        if (st.lhs->kind == Expr::Id && !same(st.lhs, init.lhs)) {
            if (!pre_activation(st.rhs)) return false;
            temp = st.lhs;
            if (!parse_assign(t, p, &st) || st.plus_equals) return false;
        }
        out_ref = st.lhs;
        ExprP v = strip_activation(st.rhs, &n->act);
        n->relu = n->act == 1;
        if (temp) {
            if (!same(v, temp)) return false;
        } else if (!pre_activation(v)) {
            return false;
        }
    } else {
        out_ref = init.lhs;  // C[i][j] accumulated in place
    }
    if (!parse_ref(out_ref, vars, decls, &n->c) || !uses(n->c, vars[0], vars[1])) return false;
    if (!close_block(t, p, bj) || !close_block(t, p, bi)) return false;
    n->tail = n->act != 0 || !n->bias.empty();
    // element types: all three arrays of one kind
    auto type_of = [&](const std::string &name) {
        auto it = decls.find(name);
        return it == decls.end() ? std::string() : it->second.type;
    };
    n->type = type_of(n->c.name);
    if (n->type.empty() || type_of(n->a.name) != n->type || type_of(n->b.name) != n->type) return false;
    if (!n->bias.empty() && type_of(n->bias) != n->type) return false;
    if (n->c.name == n->a.name || n->c.name == n->b.name) return false;  // the nest would read its own output
    // a bias / ReLU tail exists only fused into the fp32 linear on plainly laid out operands
    const bool plain = n->a.row == vars[0] && n->a.col == vars[2] && n->b.row == vars[2] && n->b.col == vars[1] &&
                       n->c.row == vars[0] && n->c.col == vars[1];
    if (n->tail && !(n->type == "f32" && plain)) return false;
    n->tok_end = p;
    return true;
}


// ------------------------------------------------------------------------------------------
// a nest the reference has already tiled: strip loops outside, blocked element loops inside, the
// accumulation statement as the only statement
// ------------------------------------------------------------------------------------------
struct TiledNest {
    GLoop li, lj, lk;              // the element loops, by role
    long long bi = 0, bj = 0, bk = 0;  // strip sizes (0: that loop was not blocked)
    bool j_outer_of_i = false;     // the j strip (or loop) encloses the i one: the reference interchanged
    Ref a, b, c;
    std::string type;
    size_t tok_begin, tok_end;
};

bool match_tiled(const std::vector<Tok> &t, size_t start, const std::map<std::string, ArrayDecl> &decls, TiledNest *n) {
    size_t p = start;
    n->tok_begin = start;
    std::vector<GLoop> loops;
    std::vector<bool> braced;
    while (true) {
        GLoop L;
        take_pragmas(t, p, &L.pragmas);
        if (!parse_for_general(t, p, &L)) break;
        loops.push_back(L);
        braced.push_back(open_block(t, p));
        if (loops.size() > 9) return false;
    }
    if (loops.size() < 3) return false;
    Assign upd;
    if (!parse_assign(t, p, &upd)) return false;
    for (size_t i = loops.size(); i-- > 0;)
        if (!close_block(t, p, braced[i])) return false;
    // strip loops step by the block size from 0; element loops step by 1
    std::vector<const GLoop *> strips, elems;
    for (const GLoop &L : loops) (L.step > 1 ? strips : elems).push_back(&L);
    if (elems.size() != 3) return false;
    for (const GLoop *S : strips)
        if (!is_zero(S->lb)) return false;
    // the statement: C = C + A * B  |  C = A * B + C  |  C += A * B
    ExprP prod = upd.rhs;
    if (!upd.plus_equals) {
        if (!prod || prod->kind != Expr::Bin || prod->text != "+") return false;
        if (same(prod->kids[0], upd.lhs)) prod = prod->kids[1];
        else if (same(prod->kids[1], upd.lhs)) prod = prod->kids[0];
        else return false;
    }
    if (!prod || prod->kind != Expr::Bin || prod->text != "*") return false;
    const std::vector<std::string> vars = {elems[0]->var, elems[1]->var, elems[2]->var};
    if (vars[0] == vars[1] || vars[0] == vars[2] || vars[1] == vars[2]) return false;
    Ref r0, r1, rc;
    if (!parse_ref(prod->kids[0], vars, decls, &r0) || !parse_ref(prod->kids[1], vars, decls, &r1) ||
        !parse_ref(upd.lhs, vars, decls, &rc))
        return false;
    // roles: C is indexed by (i, j); k is the variable C does not use; A uses (i, k), B uses (k, j)
    auto has = [](const Ref &r, const std::string &v) { return r.row == v || r.col == v; };
    std::string vk;
    for (const std::string &v : vars)
        if (!has(rc, v)) vk = v;
    if (vk.empty()) return false;
    // i is the variable that walks C's rows, j the one that walks its columns
    const std::string vi = rc.row, vj = rc.col;
    if (vi == vk || vj == vk || vi == vj) return false;
    const Ref *ra = nullptr, *rb = nullptr;
    for (int sw = 0; sw < 2 && !ra; ++sw) {
        const Ref &x = sw ? r1 : r0, &y = sw ? r0 : r1;
        if (has(x, vi) && has(x, vk) && has(y, vk) && has(y, vj)) ra = &x, rb = &y;
    }
    if (!ra) return false;
    n->a = *ra, n->b = *rb, n->c = rc;
    // element loops by role; each is either whole (lb 0, plain bound) or blocked (lb = strip variable,
    // bound = min(strip + B - 1, ub) or strip + B - 1 when the block divides the extent)
    size_t order_i = 0, order_j = 0;
    for (const GLoop *E : elems) {
        GLoop whole = *E;
        long long blk = 0;
        size_t depth = 0;
        for (size_t d = 0; d < loops.size(); ++d)
            if (&loops[d] == E) depth = d;
        if (!is_zero(E->lb)) {
            if (E->lb->kind != Expr::Id) return false;
            const GLoop *S = nullptr;
            for (const GLoop *cand : strips)
                if (cand->var == E->lb->text) S = cand;
            if (!S) return false;
            for (size_t d = 0; d < loops.size(); ++d)
                if (&loops[d] == S) {
                    if (d > depth) return false;  // a strip loop encloses its element loop
                    depth = d;
                }
            blk = S->step;
            ExprP x, y, bound = E->ub;
            long long c = 0;
            const long long want = E->inclusive ? blk - 1 : blk;
            if (split_min(bound, &x, &y)) {
                ExprP rest;
                if (var_plus_const(x, S->var, &c) && c == want) rest = y;
                else if (var_plus_const(y, S->var, &c) && c == want) rest = x;
                else return false;
                if (!same(rest, S->ub) || E->inclusive != S->inclusive) return false;  // the strip's own bound
            } else if (!(var_plus_const(bound, S->var, &c) && c == want)) {
                return false;
            }
            whole.lb = S->lb;
            whole.ub = S->ub;
            whole.inclusive = S->inclusive;
        }
        if (E->var == vi) n->li = whole, n->bi = blk, order_i = depth;
        else if (E->var == vj) n->lj = whole, n->bj = blk, order_j = depth;
        else n->lk = whole, n->bk = blk;
    }
    // every strip loop must belong to one of the element loops
    size_t used = (n->bi ? 1 : 0) + (n->bj ? 1 : 0) + (n->bk ? 1 : 0);
    if (used != strips.size()) return false;
    n->j_outer_of_i = order_j < order_i;
    auto type_of = [&](const std::string &name) {
        auto it = decls.find(name);
        return it == decls.end() ? std::string() : it->second.type;
    };
    n->type = type_of(n->c.name);
    if (n->type.empty() || type_of(n->a.name) != n->type || type_of(n->b.name) != n->type) return false;
    if (n->c.name == n->a.name || n->c.name == n->b.name) return false;
    // only nests that need this matcher: the plain untiled form with a zeroed accumulator is match_nest's
    n->tok_end = p;
    return true;
}

std::string extent_of(const ExprP &ub, bool inclusive) {
    long long v;
    if (const_int(ub, &v)) return std::to_string(inclusive ? v + 1 : v);
    return inclusive ? "(" + str(ub) + " + 1)" : str(ub);
}

std::string emit_tiled(const TiledNest &n, const std::string &indent) {
    const std::string M = extent_of(n.li.ub, n.li.inclusive), N = extent_of(n.lj.ub, n.lj.inclusive),
                      K = extent_of(n.lk.ub, n.lk.inclusive);
    std::ostringstream o;
    const std::string in2 = indent + "    ";
    const char *fn = n.type == "f32" ? "_s4gemmx__" : n.type == "f64" ? "_sgemmx__" : n.type == "i32" ? "_i4gemmx__" : "_jgemmx__";
    const char *ct = n.type == "f32" ? "float" : n.type == "f64" ? "double" : n.type == "i32" ? "int32_t" : "int64_t";
    auto base = [](const Ref &r) { return "&" + str(r.whole->kids[0]->kind == Expr::Index ? r.whole->kids[0]->kids[0] : r.whole->kids[0]) +
                                          (r.whole->kids[0]->kind == Expr::Index ? "[0][0]" : "[0]"); };
    auto incs = [&](const Ref &r, const std::string &rowvar, std::string *i1, std::string *i2) {
        if (r.row == rowvar) {
            *i1 = r.ld;
            *i2 = "1";
        } else {
            *i1 = "1";
            *i2 = r.ld;
        }
    };
    std::string a1, a2, b1, b2, c1, c2;
    incs(n.a, n.li.var, &a1, &a2);
    incs(n.b, n.lk.var, &b1, &b2);
    incs(n.c, n.li.var, &c1, &c2);
    o << "{\n";
    o << in2 << "/* o64nest: " << n.c.name << "(" << M << " x " << N << ") += " << n.a.name << " * " << n.b.name << " over " << K
      << "; the nest was blocked " << (n.bi ? std::to_string(n.bi) : std::string("-")) << " x "
      << (n.bj ? std::to_string(n.bj) : std::string("-")) << " x " << (n.bk ? std::to_string(n.bk) : std::string("-"))
      << " (i x j x k" << (n.j_outer_of_i ? ", j outside i" : "") << ") */\n";
    const bool pinned = n.type == "f32" && (n.bi || n.bj || n.bk || n.j_outer_of_i);
    if (pinned) {
        // the strip sizes of the cache blocking become the tile of the fp32 kernel where it has one of that size
        o << in2 << "o64_plan_t o64_plan;\n" << in2 << "memset(&o64_plan, 0, sizeof(o64_plan));\n";
        if (n.bi) o << in2 << "o64_plan.tile_m = " << n.bi << ";\n";
        if (n.bj) o << in2 << "o64_plan.tile_n = " << n.bj << ";\n";
        if (n.bk) o << in2 << "o64_plan.tile_k = " << n.bk << ";\n";
        if (n.j_outer_of_i) o << in2 << "o64_plan.raster = 1;\n";
        o << in2 << "if (o64_plan_set(o64_compat_handle(), O64_KIND_F32, &o64_plan) != O64_OK)\n"
          << in2 << "    o64_plan_set(o64_compat_handle(), O64_KIND_F32, NULL);  /* no kernel of that size: automatic plan */\n";
    }
    o << in2 << "const int o64_m = " << M << ", o64_n = " << N << ", o64_k = " << K << ";\n";
    o << in2 << "const int o64_a1 = " << a1 << ", o64_a2 = " << a2 << ", o64_b1 = " << b1 << ", o64_b2 = " << b2
      << ", o64_c1 = " << c1 << ", o64_c2 = " << c2 << ";\n";
    o << in2 << "const " << ct << " o64_one = 1;  /* beta = 1: the nest accumulates into " << n.c.name << " */\n";
    o << in2 << fn << "(&o64_m, &o64_n, &o64_k, &o64_one, (const " << ct << " *)" << base(n.a) << ", &o64_a1, &o64_a2, (const "
      << ct << " *)" << base(n.b) << ", &o64_b1, &o64_b2, &o64_one, (" << ct << " *)" << base(n.c) << ", &o64_c1, &o64_c2);\n";
    o << in2 << "o64nest_check(o64_compat_last_status(), \"" << fn << "\");\n";
    if (pinned) o << in2 << "o64_plan_set(o64_compat_handle(), O64_KIND_F32, NULL);\n";
    o << indent << "}";
    return o.str();
}

std::string extent(const Loop &L) {
    long long lo = 0, hi = 0;
    const bool lo_const = const_int(L.lb, &lo), hi_const = const_int(L.ub, &hi);
    if (lo_const && hi_const) return std::to_string((L.inclusive ? hi + 1 : hi) - lo);
    std::string e = L.inclusive ? "(" + str(L.ub) + " + 1)" : str(L.ub);
    if (lo_const && lo == 0) return e;
    return "(" + e + " - (" + str(L.lb) + "))";
}

bool pragma_ints(const std::string &text, const char *name, std::vector<long long> *vals, std::vector<std::string> *ids) {
    std::string low;
    for (char c : text) low += (char)tolower((unsigned char)c);
    size_t at = low.find(name);
    if (at == std::string::npos) return false;
    at = low.find('(', at);
    if (at == std::string::npos) return false;
    const size_t end = low.find(')', at);
    std::string inner = text.substr(at + 1, end == std::string::npos ? std::string::npos : end - at - 1);
    std::stringstream ss(inner);
    std::string item;
    while (std::getline(ss, item, ',')) {
        size_t b = item.find_first_not_of(" \t"), e = item.find_last_not_of(" \t");
        if (b == std::string::npos) continue;
        item = item.substr(b, e - b + 1);
        if (isdigit((unsigned char)item[0]) || item[0] == '-') vals->push_back(atoll(item.c_str()));
        else ids->push_back(item);
    }
    return true;
}

std::string emit(const Nest &n, const std::string &indent) {
    const std::string M = extent(n.li), N = extent(n.lj), K = extent(n.lk);
    std::ostringstream o;
    const std::string in2 = indent + "    ";
    o << "{\n";
    o << in2 << "/* o64nest: " << n.c.name << "(" << M << " x " << N << ") = " << n.a.name << " * " << n.b.name
      << " over " << K << (n.bias.empty() ? "" : " + " + n.bias)
      << (n.act == 1 ? ", max(., 0)" : n.act == 2 ? ", GELU (tanh)" : n.act == 3 ? ", GELU (erf)" : n.act == 4 ? ", SiLU" : "") << " */\n";
    // plan pins from the loops' pragmas
    long long tile_m = 0, tile_n = 0, tile_k = 0, group = 0, raster = 0;
    std::string ignored;
    auto scan = [&](const Loop &L, int which) {
        for (const std::string &pr : L.pragmas) {
            std::vector<long long> v;
            std::vector<std::string> ids;
            if (pragma_ints(pr, "blocking size", &v, &ids) && !v.empty()) {
                if (which == 0) {
                    tile_m = v[0];
                    if (v.size() > 1 && v[0] > 0) group = v[1] / v[0];
                } else if (which == 1) {
                    tile_n = v[0];
                } else {
                    tile_k = v[0];
                }
            } else if (pragma_ints(pr, "interchange", &v, &ids) && !ids.empty()) {
                raster = ids[0] == n.lj.var ? 1 : 0;
            } else {
                ignored += " " + pr;
            }
        }
    };
    scan(n.li, 0);
    scan(n.lj, 1);
    scan(n.lk, 2);
    const bool plain = n.a.row == n.li.var && n.a.col == n.lk.var && n.b.row == n.lk.var && n.b.col == n.lj.var &&
                       n.c.row == n.li.var && n.c.col == n.lj.var;
    // the element the loops touch first: every index variable at its loop's first value
    auto first_of = [&](const std::string &var) {
        const Loop &L = var == n.li.var ? n.li : (var == n.lj.var ? n.lj : n.lk);
        long long v;
        return const_int(L.lb, &v) ? std::to_string(v) : "(" + str(L.lb) + ")";
    };
    auto base = [&](const Ref &r) {
        const bool two_d = r.whole->kids[0]->kind == Expr::Index;
        const std::string name = str(two_d ? r.whole->kids[0]->kids[0] : r.whole->kids[0]);
        const std::string r0 = first_of(r.row), c0 = first_of(r.col);
        if (two_d) return "&" + name + "[" + r0 + "][" + c0 + "]";
        if (r0 == "0" && c0 == "0") return "&" + name + "[0]";
        return "&" + name + "[" + r0 + " * (" + r.ld + ") + " + c0 + "]";
    };
    const std::string bias_arg = n.bias.empty() ? "NULL" : (first_of(n.lj.var) == "0" ? n.bias : "&" + n.bias + "[" + first_of(n.lj.var) + "]");
    static const char *act_names[] = {"O64_ACT_NONE", "O64_ACT_RELU", "O64_ACT_GELU_TANH", "O64_ACT_GELU_ERF", "O64_ACT_SILU"};
    if (n.type == "f32" && plain) {
        const bool pinned = tile_m || tile_n || tile_k || group || raster;
        if (pinned) {
            o << in2 << "o64_plan_t o64_plan;\n" << in2 << "memset(&o64_plan, 0, sizeof(o64_plan));\n";
            if (tile_m) o << in2 << "o64_plan.tile_m = " << tile_m << ";\n";
            if (tile_n) o << in2 << "o64_plan.tile_n = " << tile_n << ";\n";
            if (tile_k) o << in2 << "o64_plan.tile_k = " << tile_k << ";\n";
            if (group) o << in2 << "o64_plan.group_m = " << group << ";\n";
            if (raster) o << in2 << "o64_plan.raster = 1;\n";
            o << in2 << "if (o64_plan_set(o64nest_handle(), O64_KIND_F32, &o64_plan) != O64_OK)\n"
              << in2 << "    o64_plan_set(o64nest_handle(), O64_KIND_F32, NULL);  /* no kernel of that size: automatic plan */\n";
        }
        o << in2 << "o64nest_check(o64_linear_f32(o64nest_handle(), " << M << ", " << N << ", " << K << ", " << base(n.a)
          << ", " << n.a.ld << ", " << base(n.b) << ", " << n.b.ld << ", " << bias_arg << ", "
          << base(n.c) << ", " << n.c.ld << ", " << act_names[n.act] << ", NULL), \"o64_linear_f32\");\n";
        if (pinned) o << in2 << "o64_plan_set(o64nest_handle(), O64_KIND_F32, NULL);\n";
    } else {
        // the strided kernels of the runtime: element (r, c) of X at X[inc1*r + inc2*c]
        const char *fn = n.type == "f32" ? "_s4gemmx__" : n.type == "f64" ? "_sgemmx__" : n.type == "i32" ? "_i4gemmx__" : "_jgemmx__";
        const char *ct = n.type == "f32" ? "float" : n.type == "f64" ? "double" : n.type == "i32" ? "int32_t" : "int64_t";
        auto incs = [&](const Ref &r, const std::string &rowvar, std::string *i1, std::string *i2) {
            // inc1: step of the first index of the mathematical operand, inc2: of the second
            if (r.row == rowvar) {
                *i1 = r.ld;
                *i2 = "1";
            } else {
                *i1 = "1";
                *i2 = r.ld;
            }
        };
        std::string a1, a2, b1, b2, c1, c2;
        incs(n.a, n.li.var, &a1, &a2);
        incs(n.b, n.lk.var, &b1, &b2);
        incs(n.c, n.li.var, &c1, &c2);
        o << in2 << "const int o64_m = " << M << ", o64_n = " << N << ", o64_k = " << K << ";\n";
        o << in2 << "const int o64_a1 = " << a1 << ", o64_a2 = " << a2 << ", o64_b1 = " << b1 << ", o64_b2 = " << b2
          << ", o64_c1 = " << c1 << ", o64_c2 = " << c2 << ";\n";
        o << in2 << "const " << ct << " o64_one = 1, o64_zero = 0;\n";
        o << in2 << fn << "(&o64_m, &o64_n, &o64_k, &o64_one, (const " << ct << " *)" << base(n.a) << ", &o64_a1, &o64_a2, (const "
          << ct << " *)" << base(n.b) << ", &o64_b1, &o64_b2, &o64_zero, (" << ct << " *)" << base(n.c) << ", &o64_c1, &o64_c2);\n";
        o << in2 << "o64nest_check(o64_compat_last_status(), \"" << fn << "\");\n";
    }
    if (!ignored.empty()) o << in2 << "/* pragmas without a counterpart here:" << ignored << " */\n";
    o << indent << "}";
    return o.str();
}

const char *kPrelude =
    "/* added by o64nest */\n"
    "#include <stdint.h>\n#include <stdio.h>\n#include <stdlib.h>\n#include <string.h>\n#include \"o64gemm.h\"\n"
    "static o64_handle_t o64nest_handle(void) {\n"
    "    static o64_handle_t h;\n"
    "    if (!h && o64_create(&h, 0) != O64_OK) {\n"
    "        fprintf(stderr, \"o64nest: cannot open the GEMM engine\\n\");\n"
    "        abort();\n"
    "    }\n"
    "    return h;\n"
    "}\n"
    "static void o64nest_check(int rc, const char *what) {\n"
    "    if (rc != O64_OK) {  /* the runtime this replaces aborts on rank / conformance / memory errors */\n"
    "        fprintf(stderr, \"%s: %s\\n\", what, o64_status_string(rc));\n"
    "        abort();\n"
    "    }\n"
    "}\n\n";

}  // namespace

int main(int argc, char **argv) {
    std::string in_path = "-", out_path;
    for (int i = 1; i < argc; ++i) {
        if (!strcmp(argv[i], "-o") && i + 1 < argc) out_path = argv[++i];
        else if (argv[i][0] == '-' && argv[i][1]) {
            fprintf(stderr, "usage: o64nest [input.c] [-o output.c]\n");
            return 2;
        } else in_path = argv[i];
    }
    std::string src;
    if (in_path == "-") {
        std::stringstream ss;
        ss << std::cin.rdbuf();
        src = ss.str();
    } else {
        std::ifstream f(in_path);
        if (!f) {
            fprintf(stderr, "o64nest: cannot read %s\n", in_path.c_str());
            return 2;
        }
        std::stringstream ss;
        ss << f.rdbuf();
        src = ss.str();
    }
    const std::vector<Tok> toks = tokenize(src);
    const auto decls = scan_decls(toks);
    std::string out;
    size_t copied = 0;
    int found = 0;
    for (size_t p = 0; p < toks.size();) {
        const bool starts = toks[p].kind == Tok::Pragma || (toks[p].kind == Tok::Id && toks[p].text == "for");
        Nest n;
        TiledNest tn;
        if (starts && !match_nest(toks, p, decls, &n) && match_tiled(toks, p, decls, &tn)) {
            const size_t b = toks[tn.tok_begin].begin, e = toks[tn.tok_end - 1].end;
            size_t first_for = tn.tok_begin;
            while (toks[first_for].kind == Tok::Pragma) ++first_for;
            const size_t fb = toks[first_for].begin;
            size_t line = src.rfind('\n', fb);
            line = line == std::string::npos ? 0 : line + 1;
            std::string indent = src.substr(line, fb - line);
            if (indent.find_first_not_of(" \t") != std::string::npos) indent.clear();
            out += src.substr(copied, b - copied);
            if (first_for != tn.tok_begin) out += indent;
            out += emit_tiled(tn, indent);
            copied = e;
            p = tn.tok_end;
            ++found;
            continue;
        }
        if (starts && match_nest(toks, p, decls, &n)) {
            const size_t b = toks[n.tok_begin].begin, e = toks[n.tok_end - 1].end;
            size_t first_for = n.tok_begin;
            while (toks[first_for].kind == Tok::Pragma) ++first_for;
            const size_t fb = toks[first_for].begin;
            size_t line = src.rfind('\n', fb);
            line = line == std::string::npos ? 0 : line + 1;
            std::string indent = src.substr(line, fb - line);
            if (indent.find_first_not_of(" \t") != std::string::npos) indent.clear();
            out += src.substr(copied, b - copied);
            if (first_for != n.tok_begin) out += indent;  // the nest began with a pragma in column 0
            out += emit(n, indent);
            copied = e;
            p = n.tok_end;
            ++found;
            continue;
        } else {
            ++p;
        }
    }
    out += src.substr(copied);
    if (found) out = kPrelude + out;
    fprintf(stderr, "o64nest: %d nest%s replaced\n", found, found == 1 ? "" : "s");
    if (out_path.empty()) {
        fputs(out.c_str(), stdout);
    } else {
        std::ofstream f(out_path);
        f << out;
    }
    return 0;
}
