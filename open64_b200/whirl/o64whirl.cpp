// o64whirl: finds the loop nest the reference builds for MATMUL in a WHIRL dump and prints the engine
// call that replaces it.
//
// Input: WHIRL as the reference's own tools print it in ASCII (ir_b2a; writer ir_put_wn / ir_put_stmt,
// osprey/common/com/ir_reader.cxx:976-1560): one node per line, indented by depth; expressions and
// simple statements with the children first and the operator last, structured statements first with
// markers (DO_LOOP ... INIT / COMP / INCR / BODY, BLOCK ... END_BLOCK).  The binary .B file needs the
// reference's reader and symbol tables (osprey/common/com/ir_bread.cxx:1497-1584) and a front end to
// produce it; neither can be built without the reference's toolchain, so this tool starts from the dump.
//
// Recognised: the nest of lower_mm_matmul (osprey/be/vho/f90_lower.cxx:5116-5178) inside the two result
// loops of create_doloop_nest (:4095-4115), every loop in create_doloop's form (:4027-4092: index from
// 0, test  index <= count - 1, step 1):
//
//     DO_LOOP v1 { DO_LOOP v0 {  STID acc = 0
//                                DO_LOOP vk { STID acc = ADD(LDID acc, MPY(ILOAD(ARRAY A ..), ILOAD(ARRAY B ..))) }
//                                ISTORE  ARRAY R(..) = LDID acc            -- or MAX(ADD(LDID acc, ILOAD bias), 0)
//     } }
//
// with rank-2 ARRAY nodes whose subscripts are the loop indices (in either order: a transposed operand
// only exchanges its increments).  For each nest: one line of JSON (function, element kind, extents,
// arrays with their increments, tail) and the C call on the runtime's strided kernel (or the fused
// fp32 linear when the layout is plain and a bias / ReLU tail is present).  Also recognised: MATMUL
// before the lowering pass has expanded it (an INTRINSIC_OP, see match_intrinsic below).
//
//   o64whirl dump.txt            exit status 0 (the number of nests goes to stderr), 2 on usage errors
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

namespace {

struct Node;
typedef std::shared_ptr<Node> NodeP;
struct Node {
    std::string op;              // "I4I4LDID", "DO_LOOP", "BLOCK", ...
    std::string rest;            // the remainder of the line
    int indent = 0;
    std::vector<NodeP> kids;     // expressions / simple statements: operands; BLOCK: statements
    NodeP index, init, comp, incr, body;  // DO_LOOP
};

struct Line {
    int indent;
    std::string op, rest;
};

std::vector<Line> read_lines(std::istream &in) {
    std::vector<Line> out;
    std::string s;
    while (std::getline(in, s)) {
        size_t i = 0;
        while (i < s.size() && s[i] == ' ') ++i;
        if (i == s.size()) continue;
        size_t j = i;
        while (j < s.size() && s[j] != ' ') ++j;
        Line l;
        l.indent = (int)i;
        l.op = s.substr(i, j - i);
        l.rest = j < s.size() ? s.substr(j + 1) : "";
        if (l.op == "LOC") continue;  // source positions between statements
        out.push_back(l);
    }
    return out;
}

bool is_marker(const std::string &op) {
    return op == "INIT" || op == "COMP" || op == "INCR" || op == "BODY" || op == "END_BLOCK" || op == "THEN" ||
           op == "ELSE" || op == "END_IF";
}

struct Reader {
    const std::vector<Line> &l;
    size_t p = 0;
    explicit Reader(const std::vector<Line> &lines) : l(lines) {}
    bool at(const char *op, int indent) const { return p < l.size() && l[p].op == op && l[p].indent == indent; }

    // children first, operator last: consumes lines up to and including the one at `indent`
    NodeP postfix(int indent) {
        std::vector<NodeP> pending;
        while (p < l.size()) {
            const Line &ln = l[p];
            if (ln.indent < indent || is_marker(ln.op)) return nullptr;
            auto n = std::make_shared<Node>();
            n->op = ln.op, n->rest = ln.rest, n->indent = ln.indent;
            size_t first = pending.size();
            while (first > 0 && pending[first - 1]->indent == ln.indent + 1) --first;
            n->kids.assign(pending.begin() + first, pending.end());
            pending.resize(first);
            ++p;
            if (ln.indent == indent) return pending.empty() ? n : nullptr;
            pending.push_back(n);
        }
        return nullptr;
    }

    NodeP block(int indent) {  // at "BLOCK"
        if (!at("BLOCK", indent)) return nullptr;
        auto b = std::make_shared<Node>();
        b->op = "BLOCK", b->indent = indent;
        ++p;
        while (p < l.size() && !at("END_BLOCK", indent)) {
            NodeP s = statement(indent);
            if (!s) return nullptr;
            b->kids.push_back(s);
        }
        if (!at("END_BLOCK", indent)) return nullptr;
        ++p;
        return b;
    }

    NodeP statement(int indent) {
        if (at("DO_LOOP", indent)) {
            auto d = std::make_shared<Node>();
            d->op = "DO_LOOP", d->rest = l[p].rest, d->indent = indent;
            ++p;
            d->index = postfix(indent + 1);
            if (!d->index || !at("INIT", indent)) return nullptr;
            ++p;
            d->init = postfix(indent + 1);
            if (!d->init || !at("COMP", indent)) return nullptr;
            ++p;
            d->comp = postfix(indent + 1);
            if (!d->comp || !at("INCR", indent)) return nullptr;
            ++p;
            d->incr = postfix(indent + 1);
            if (!d->incr) return nullptr;
            while (p < l.size() && !at("BODY", indent)) {  // optional LOOP_INFO with its own operands
                if (l[p].indent < indent) return nullptr;
                ++p;
            }
            if (!at("BODY", indent)) return nullptr;
            ++p;
            d->body = block(indent + 1);
            return d->body ? d : nullptr;
        }
        if (at("BLOCK", indent)) return block(indent);
        if (at("IF", indent) || at("WHILE_DO", indent) || at("DO_WHILE", indent) || at("REGION", indent)) {
            // other structured statements: kept opaque, skipped up to the next line at this depth that
            // closes them (END_IF) or, for the loops, their BODY block
            auto o = std::make_shared<Node>();
            o->op = l[p].op, o->indent = indent;
            const bool is_if = o->op == "IF";
            ++p;
            while (p < l.size()) {
                if (l[p].indent == indent && (is_if ? l[p].op == "END_IF" : l[p].op == "END_BLOCK")) break;
                if (l[p].indent < indent) return nullptr;
                ++p;
            }
            if (is_if && p < l.size()) ++p;
            return o;
        }
        return postfix(indent);
    }
};

// ---- pieces of a line -------------------------------------------------------------------------
// "<1,4,.preg_I4>" -> name; the preg's own name follows "# "
std::string sym_name(const std::string &rest) {
    const size_t a = rest.find('<');
    if (a == std::string::npos) return "";
    const size_t b = rest.find('>', a);
    if (b == std::string::npos) return "";
    const std::string inner = rest.substr(a + 1, b - a - 1);
    const size_t c = inner.rfind(',');
    return c == std::string::npos ? inner : inner.substr(c + 1);
}
std::string preg_or_sym(const Node &n) {  // identity of what an LDID / STID / IDNAME names
    const size_t h = n.rest.find("# ");
    std::string key = std::to_string(atoll(n.rest.c_str())) + ":" + sym_name(n.rest);
    (void)h;
    return key;
}
std::string display_name(const Node &n) {
    const size_t h = n.rest.find("# ");
    if (h != std::string::npos) return n.rest.substr(h + 2);
    return sym_name(n.rest);
}
bool ends_with(const std::string &s, const char *suffix) {
    const size_t n = strlen(suffix);
    return s.size() >= n && s.compare(s.size() - n, n, suffix) == 0;
}
bool int_const(const NodeP &n, long long *v) {
    if (!n || !ends_with(n->op, "INTCONST")) return false;
    *v = atoll(n->rest.c_str());
    return true;
}
bool is_zero_const(const NodeP &n) {
    long long v;
    if (int_const(n, &v)) return v == 0;
    if (n && ends_with(n->op, "CONST") && n->kids.empty()) {  // F4CONST <1,20,0.000000>
        const std::string name = sym_name(n->rest);
        return !name.empty() && atof(name.c_str()) == 0.0 && name.find_first_of("123456789") == std::string::npos;
    }
    return false;
}

// ---- create_doloop's loop ---------------------------------------------------------------------
struct LoopInfo {
    std::string var;       // identity of the index
    std::string count;     // trip count as text (a constant, or the name a count is loaded from)
    NodeP body;
};

std::string count_text(const NodeP &n) {
    long long v;
    if (int_const(n, &v)) return std::to_string(v);
    if (n && ends_with(n->op, "LDID")) return display_name(*n);
    if (n && ends_with(n->op, "CVT") && n->kids.size() == 1) return count_text(n->kids[0]);
    return "";
}

bool loop_info(const NodeP &d, LoopInfo *out) {
    if (!d || d->op != "DO_LOOP" || !d->index || d->index->op != "IDNAME") return false;
    out->var = preg_or_sym(*d->index);
    // INIT: STID var = 0
    if (!ends_with(d->init->op, "STID") || preg_or_sym(*d->init) != out->var || d->init->kids.size() != 1 ||
        !is_zero_const(d->init->kids[0]))
        return false;
    // COMP: LE(LDID var, SUB(count, 1))  or  LE(LDID var, constant)
    const NodeP &c = d->comp;
    if (!ends_with(c->op, "LE") || c->kids.size() != 2 || !ends_with(c->kids[0]->op, "LDID") ||
        preg_or_sym(*c->kids[0]) != out->var)
        return false;
    const NodeP &ub = c->kids[1];
    long long v, one;
    if (int_const(ub, &v)) {
        out->count = std::to_string(v + 1);
    } else if (ends_with(ub->op, "SUB") && ub->kids.size() == 2 && int_const(ub->kids[1], &one) && one == 1) {
        out->count = count_text(ub->kids[0]);
        if (out->count.empty()) return false;
    } else {
        return false;
    }
    // INCR: STID var = ADD(LDID var, 1)
    const NodeP &s = d->incr;
    if (!ends_with(s->op, "STID") || preg_or_sym(*s) != out->var || s->kids.size() != 1) return false;
    const NodeP &a = s->kids[0];
    if (!ends_with(a->op, "ADD") || a->kids.size() != 2) return false;
    const bool fwd = ends_with(a->kids[0]->op, "LDID") && preg_or_sym(*a->kids[0]) == out->var && int_const(a->kids[1], &one) && one == 1;
    const bool rev = ends_with(a->kids[1]->op, "LDID") && preg_or_sym(*a->kids[1]) == out->var && int_const(a->kids[0], &one) && one == 1;
    if (!fwd && !rev) return false;
    out->body = d->body;
    return true;
}

// ---- ILOAD(ARRAY(base, d0, d1, x0, x1)) -----------------------------------------------------------
struct ArrayRef {
    std::string name;
    std::string dim1;          // extent of the faster dimension: the pitch in elements
    std::string idx0, idx1;    // loop variables subscripting the slower / the faster dimension
    long long esize = 0;
};

bool array_ref(const NodeP &addr, ArrayRef *r) {
    if (!addr || !ends_with(addr->op, "ARRAY") || addr->kids.size() != 5) return false;
    int ndim = 0;
    long long esize = 0;
    if (sscanf(addr->rest.c_str(), "%d %lld", &ndim, &esize) != 2 || ndim != 2) return false;
    r->esize = esize;
    const NodeP &base = addr->kids[0];
    if (!(ends_with(base->op, "LDA") || ends_with(base->op, "LDID"))) return false;
    r->name = display_name(*base);
    r->dim1 = count_text(addr->kids[2]);
    if (r->dim1.empty()) return false;
    for (int i = 0; i < 2; ++i) {
        NodeP x = addr->kids[3 + i];
        if (ends_with(x->op, "CVT") && x->kids.size() == 1) x = x->kids[0];
        if (!ends_with(x->op, "LDID")) return false;
        (i ? r->idx1 : r->idx0) = preg_or_sym(*x);
    }
    return r->idx0 != r->idx1;
}
bool load_of_array(const NodeP &n, ArrayRef *r) { return n && ends_with(n->op, "ILOAD") && n->kids.size() == 1 && array_ref(n->kids[0], r); }

// increment of loop variable v in r (in elements); "" if v does not subscript r
std::string inc_of(const ArrayRef &r, const std::string &v) {
    if (r.idx1 == v) return "1";
    if (r.idx0 == v) return r.dim1;
    return "";
}

struct Match {
    std::string kind;   // s4, s, i4, j
    std::string m, n, k;
    ArrayRef a, b, c;
    std::string vi, vj, vk;
    std::string bias;
    bool relu = false;
};

bool elem_kind(const std::string &op, std::string *kind) {  // by the result type letters of the opcode
    if (op.compare(0, 2, "F4") == 0) *kind = "s4";
    else if (op.compare(0, 2, "F8") == 0) *kind = "s";
    else if (op.compare(0, 2, "I4") == 0) *kind = "i4";
    else if (op.compare(0, 2, "I8") == 0) *kind = "j";
    else return false;
    return true;
}

bool match_nest(const NodeP &outer, Match *m) {
    LoopInfo l1, l0, lk;
    if (!loop_info(outer, &l1) || l1.body->kids.size() != 1 || !loop_info(l1.body->kids[0], &l0)) return false;
    const std::vector<NodeP> &st = l0.body->kids;
    if (st.size() != 3) return false;
    // STID acc = 0
    if (!ends_with(st[0]->op, "STID") || st[0]->kids.size() != 1 || !is_zero_const(st[0]->kids[0])) return false;
    const std::string acc = preg_or_sym(*st[0]);
    if (!loop_info(st[1], &lk) || lk.body->kids.size() != 1) return false;
    // STID acc = ADD(LDID acc, MPY(x, y))
    const NodeP &upd = lk.body->kids[0];
    if (!ends_with(upd->op, "STID") || preg_or_sym(*upd) != acc || upd->kids.size() != 1) return false;
    const NodeP &add = upd->kids[0];
    if (!ends_with(add->op, "ADD") || add->kids.size() != 2) return false;
    NodeP mpy;
    for (int s = 0; s < 2; ++s)
        if (ends_with(add->kids[s]->op, "LDID") && preg_or_sym(*add->kids[s]) == acc) mpy = add->kids[1 - s];
    if (!mpy || !ends_with(mpy->op, "MPY") || mpy->kids.size() != 2) return false;
    if (!elem_kind(mpy->op, &m->kind)) return false;
    ArrayRef x, y;
    if (!load_of_array(mpy->kids[0], &x) || !load_of_array(mpy->kids[1], &y)) return false;
    // ISTORE: kids = value, address
    const NodeP &store = st[2];
    if (!ends_with(store->op, "ISTORE") || store->kids.size() != 2 || !array_ref(store->kids[1], &m->c)) return false;
    NodeP val = store->kids[0];
    if (ends_with(val->op, "MAX") && val->kids.size() == 2) {
        for (int s = 0; s < 2; ++s)
            if (is_zero_const(val->kids[s])) {
                m->relu = true;
                val = val->kids[1 - s];
                break;
            }
        if (!m->relu) return false;
    }
    if (ends_with(val->op, "ADD") && val->kids.size() == 2) {
        for (int s = 0; s < 2; ++s) {
            const NodeP &p = val->kids[s], &q = val->kids[1 - s];
            if (ends_with(p->op, "LDID") && preg_or_sym(*p) == acc && ends_with(q->op, "ILOAD") && q->kids.size() == 1 &&
                ends_with(q->kids[0]->op, "ARRAY") && q->kids[0]->kids.size() == 3) {
                m->bias = display_name(*q->kids[0]->kids[0]);
                val = p;
                break;
            }
        }
    }
    if (!ends_with(val->op, "LDID") || preg_or_sym(*val) != acc) return false;
    // roles: k is the inner loop; i walks C and the operand that also holds k ... as in the nest's source
    m->vk = lk.var;
    const std::string r0 = l0.var, r1 = l1.var;
    if (inc_of(m->c, r0).empty() || inc_of(m->c, r1).empty() || !inc_of(m->c, m->vk).empty()) return false;
    for (int s = 0; s < 2; ++s) {
        const ArrayRef &p = s ? y : x, &q = s ? x : y;
        for (int t = 0; t < 2; ++t) {
            const std::string &vi = t ? r1 : r0, &vj = t ? r0 : r1;
            if (!inc_of(p, vi).empty() && !inc_of(p, m->vk).empty() && !inc_of(q, m->vk).empty() && !inc_of(q, vj).empty() &&
                m->a.name.empty()) {
                m->a = p, m->b = q, m->vi = vi, m->vj = vj;
            }
        }
    }
    if (m->a.name.empty()) return false;
    m->m = m->vi == l0.var ? l0.count : l1.count;
    m->n = m->vj == l0.var ? l0.count : l1.count;
    m->k = lk.count;
    return true;
}

// ---- MATMUL before it is expanded --------------------------------------------------------------
// Ahead of the F90 lowering pass the product is still one node: the front end builds an INTRINSIC_OP
// INTRN_MATMUL with two value PARMs under an ARRAYEXP (fei_matmul, osprey/crayf90/sgi/cwh_intrin.cxx:
// 1168-1201) and the statement stores that array expression; lower_mm_matmul later turns it into the
// nest above (osprey/be/vho/f90_lower.cxx:5330-5337).  Printed by ir_put_wn as
// "<type>INTRINSIC_OP 2 <number,MATMUL> ..." (osprey/common/com/ir_reader.cxx:1089-1096).  What is
// reported: the element kind from the opcode, and the first variable named under each operand and under
// the store's address - enough to bind the runtime's entry point _MATMUL_<K><K> on the arrays' dope
// vectors, the call the front end emits when it does not expand the intrinsic in line.
struct IntrinsicMatch {
    std::string kind, a, b, c;
};

const Node *first_variable(const Node &n) {
    if ((ends_with(n.op, "LDA") || ends_with(n.op, "LDID")) && !sym_name(n.rest).empty() &&
        sym_name(n.rest).compare(0, 6, ".preg_") != 0)
        return &n;
    for (const NodeP &k : n.kids)
        if (const Node *f = first_variable(*k)) return f;
    return nullptr;
}

const Node *find_matmul_op(const Node &n) {
    if (ends_with(n.op, "INTRINSIC_OP") && n.rest.find(",MATMUL>") != std::string::npos) return &n;
    for (const NodeP &k : n.kids)
        if (const Node *f = find_matmul_op(*k)) return f;
    return nullptr;
}

bool match_intrinsic(const NodeP &stmt, IntrinsicMatch *m) {
    if (!stmt || stmt->kids.empty()) return false;
    const bool istore = ends_with(stmt->op, "ISTORE") || ends_with(stmt->op, "MSTORE");
    const bool stid = ends_with(stmt->op, "STID");
    if (!istore && !stid) return false;
    const Node *op = find_matmul_op(*stmt->kids[0]);  // the stored value
    if (!op || op->kids.size() != 2) return false;
    for (const NodeP &k : op->kids)
        if (!ends_with(k->op, "PARM")) return false;
    const std::string t = op->op.substr(0, op->op.size() - strlen("INTRINSIC_OP"));
    if (t == "F4") m->kind = "S4";
    else if (t == "F8") m->kind = "S";
    else if (t == "I4") m->kind = "I4";
    else if (t == "I8") m->kind = "J";
    else if (t == "I2") m->kind = "I2";
    else if (t == "I1") m->kind = "I1";
    else if (t == "C4") m->kind = "C4";
    else if (t == "C8") m->kind = "C";
    else return false;
    const Node *a = first_variable(*op->kids[0]), *b = first_variable(*op->kids[1]);
    const Node *c = istore ? (stmt->kids.size() >= 2 ? first_variable(*stmt->kids[1]) : nullptr) : stmt.get();
    if (!a || !b || !c) return false;
    m->a = sym_name(a->rest), m->b = sym_name(b->rest), m->c = sym_name(c->rest);
    return !(m->c == m->a || m->c == m->b);  // the runtime's entry point may not write over an operand
}

void find_intrinsics(const NodeP &n, std::vector<IntrinsicMatch> *out) {
    if (!n) return;
    if (n->op == "DO_LOOP") {
        find_intrinsics(n->body, out);
        return;
    }
    if (n->op == "BLOCK") {
        for (const NodeP &k : n->kids) find_intrinsics(k, out);
        return;
    }
    IntrinsicMatch m;
    if (match_intrinsic(n, &m)) out->push_back(m);
}

void print(const IntrinsicMatch &m, const std::string &func) {
    printf("{\"function\": \"%s\", \"intrinsic\": \"MATMUL\", \"kind\": \"%s\", \"A\": \"%s\", \"B\": \"%s\", \"C\": \"%s\"}\n",
           func.c_str(), m.kind.c_str(), m.a.c_str(), m.b.c_str(), m.c.c_str());
    printf("    _MATMUL_%s%s(&%s_dope, &%s_dope, &%s_dope);   /* RESULT, MATRIX_A, MATRIX_B: the arrays' dope vectors */\n",
           m.kind.c_str(), m.kind.c_str(), m.c.c_str(), m.a.c_str(), m.b.c_str());
}

void find(const NodeP &n, std::vector<Match> *out) {
    if (!n) return;
    if (n->op == "DO_LOOP") {
        Match m;
        if (match_nest(n, &m)) {
            out->push_back(m);
            return;
        }
        find(n->body, out);
        return;
    }
    for (const NodeP &k : n->kids) find(k, out);
}

void print(const Match &m, const std::string &func) {
    const std::string a1 = inc_of(m.a, m.vi), a2 = inc_of(m.a, m.vk), b1 = inc_of(m.b, m.vk), b2 = inc_of(m.b, m.vj),
                      c1 = inc_of(m.c, m.vi), c2 = inc_of(m.c, m.vj);
    printf("{\"function\": \"%s\", \"kind\": \"%s\", \"m\": \"%s\", \"n\": \"%s\", \"k\": \"%s\", "
           "\"A\": {\"array\": \"%s\", \"inc1\": \"%s\", \"inc2\": \"%s\"}, \"B\": {\"array\": \"%s\", \"inc1\": \"%s\", \"inc2\": \"%s\"}, "
           "\"C\": {\"array\": \"%s\", \"inc1\": \"%s\", \"inc2\": \"%s\"}, \"bias\": \"%s\", \"relu\": %s}\n",
           func.c_str(), m.kind.c_str(), m.m.c_str(), m.n.c_str(), m.k.c_str(), m.a.name.c_str(), a1.c_str(), a2.c_str(),
           m.b.name.c_str(), b1.c_str(), b2.c_str(), m.c.name.c_str(), c1.c_str(), c2.c_str(), m.bias.c_str(),
           m.relu ? "true" : "false");
    const bool plain = a2 == "1" && b2 == "1" && c2 == "1";
    if (m.kind == "s4" && plain && (m.relu || !m.bias.empty())) {
        printf("    { /* %s = %s%s * %s%s */\n", m.c.name.c_str(), m.relu ? "max(" : "", m.a.name.c_str(), m.b.name.c_str(),
               m.bias.empty() ? (m.relu ? ", 0)" : "") : (m.relu ? " + bias, 0)" : " + bias"));
        printf("      o64_linear_f32(h, %s, %s, %s, %s, %s, %s, %s, %s, %s, %s, %s, stream);\n    }\n", m.m.c_str(), m.n.c_str(),
               m.k.c_str(), m.a.name.c_str(), a1.c_str(), m.b.name.c_str(), b1.c_str(), m.bias.empty() ? "NULL" : m.bias.c_str(),
               m.c.name.c_str(), c1.c_str(), m.relu ? "O64_ACT_RELU" : "O64_ACT_NONE");
    } else if (!m.relu && m.bias.empty()) {
        const char *ct = m.kind == "s4" ? "float" : m.kind == "s" ? "double" : m.kind == "i4" ? "int32_t" : "int64_t";
        printf("    { const int m_ = %s, n_ = %s, k_ = %s, a1 = %s, a2 = %s, b1 = %s, b2 = %s, c1 = %s, c2 = %s;\n", m.m.c_str(),
               m.n.c_str(), m.k.c_str(), a1.c_str(), a2.c_str(), b1.c_str(), b2.c_str(), c1.c_str(), c2.c_str());
        printf("      const %s one = 1, zero = 0;\n", ct);
        printf("      _%sgemmx__(&m_, &n_, &k_, &one, %s, &a1, &a2, %s, &b1, &b2, &zero, %s, &c1, &c2);\n    }\n", m.kind.c_str(),
               m.a.name.c_str(), m.b.name.c_str(), m.c.name.c_str());
    } else {
        printf("    /* a tail on a kind or layout with no fused kernel: the nest stays */\n");
    }
}

}  // namespace

int main(int argc, char **argv) {
    if (argc != 2) {
        fprintf(stderr, "usage: o64whirl dump.txt   (WHIRL printed by ir_b2a; - for stdin)\n");
        return 2;
    }
    std::vector<Line> lines;
    if (!strcmp(argv[1], "-")) {
        lines = read_lines(std::cin);
    } else {
        std::ifstream f(argv[1]);
        if (!f) {
            fprintf(stderr, "o64whirl: cannot read %s\n", argv[1]);
            return 2;
        }
        lines = read_lines(f);
    }
    // every FUNC_ENTRY: its last BLOCK is the body; structured statements are parsed, anything this
    // reader does not understand ends the function's scan (nothing is guessed)
    int found = 0, intrinsics = 0;
    Reader r(lines);
    std::string func = "?";
    while (r.p < lines.size()) {
        const Line &ln = lines[r.p];
        if (ln.op == "FUNC_ENTRY") {
            const size_t a = ln.rest.rfind(',');
            const size_t b = ln.rest.rfind('>');
            if (a != std::string::npos && b != std::string::npos && b > a) func = ln.rest.substr(a + 1, b - a - 1);
            ++r.p;
        } else if (ln.op == "BLOCK") {
            const size_t save = r.p;
            NodeP b = r.block(ln.indent);
            if (!b) {
                r.p = save + 1;
                continue;
            }
            std::vector<Match> ms;
            find(b, &ms);
            for (const Match &m : ms) print(m, func);
            found += (int)ms.size();
            std::vector<IntrinsicMatch> is;
            find_intrinsics(b, &is);
            for (const IntrinsicMatch &m : is) print(m, func);
            intrinsics += (int)is.size();
        } else {
            ++r.p;
        }
    }
    fprintf(stderr, "o64whirl: %d nest%s recognised", found, found == 1 ? "" : "s");
    if (intrinsics) fprintf(stderr, ", %d MATMUL intrinsic%s", intrinsics, intrinsics == 1 ? "" : "s");
    fprintf(stderr, "\n");
    return 0;
}
