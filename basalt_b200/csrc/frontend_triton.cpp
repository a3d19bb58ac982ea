// Triton source -> tile-level BIR; see frontend_triton.hpp.
//
// Three stages in one file: a tokenizer and parser for the Python subset `@triton.jit` kernels are
// written in; an abstract interpreter that runs the kernel body at compile time over symbolic tile
// values (every Python variable is bound to a node of an expression DAG that knows its shape and
// element type; `for ... in range(...)` with compile-time bounds is unrolled symbolically); and a
// code generator that is triggered by each `tl.store`:
//
//   * a store whose value does not involve `tl.dot` becomes a loop over the tile's lanes,
//     `for (l = tid.x; l < lanes; l += bdim.x)`, whose body instantiates the expression DAG at
//     that lane.  Masked loads and stores are real branches, never a select over an unconditional
//     access (the reference's rule, crates/basalt-sema/src/triton_lower.rs:59-73).  Under the CPU
//     oracle's launch (one thread per program) the loop walks every lane, which is exactly the
//     reference's one-thread-per-program model; on the GPU the CTA's threads share the lanes and
//     neighbouring threads touch neighbouring addresses.
//   * a store whose value is a chain of `tl.dot` (optionally plus a loaded tile, optionally cast)
//     becomes ONE `mma`: the pointer tiles of the operands are analysed as affine functions of the
//     tile indices (constant strides, a run-time base), consecutive K slabs of an unrolled loop are
//     merged, and the op gets the full K extent with explicit leading dimensions.  The reference
//     lowers `tl.dot` to a scalar triple loop because its back ends refuse `mma`
//     (triton_lower.rs:9-31); this back end has real lowerings for it, up to TMA + tcgen05.
//     With a zero accumulator the association is the same as `mma`'s (sum first, addend after).
//
// The kernel ABI is the reference's (triton_lower.rs:517-551): parameters in source order, pointers
// as ptr.global, every scalar as i64, a `tl.constexpr` parameter with a literal default dropped.
#include "frontend_triton.hpp"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <climits>
#include <cstring>
#include <functional>
#include <memory>
#include <set>
#include <sstream>
#include <vector>

namespace basalt {
namespace {

struct Fail {
    std::string code, msg;
};
[[noreturn]] void fail(const char* code, int line, const std::string& msg) { throw Fail{code, "line " + std::to_string(line) + ": " + msg}; }

// ---------------------------------------------------------------------------------------------
// Tokens
// ---------------------------------------------------------------------------------------------
enum class Tk : uint8_t { Name, Int, Float, Str, Op, Newline, Indent, Dedent, Eof };
struct Token {
    Tk k = Tk::Eof;
    std::string s;
    int64_t i = 0;
    double f = 0;
    int line = 0;
};

std::vector<Token> tokenize(const char* src, size_t len) {
    std::vector<Token> out;
    std::vector<int> indents{0};
    const char *p = src, *end = src + len;
    int line = 1, depth = 0;
    bool at_line_start = true;
    auto push = [&](Tk k, std::string s = "") {
        Token t;
        t.k = k;
        t.s = std::move(s);
        t.line = line;
        out.push_back(t);
    };
    while (p < end) {
        if (at_line_start && depth == 0) {
            int col = 0;
            const char* q = p;
            while (q < end && (*q == ' ' || *q == '\t')) { col += *q == '\t' ? 8 - col % 8 : 1; q++; }
            if (q >= end) break;
            if (*q == '\n' || *q == '\r' || *q == '#') {   // blank or comment-only line
                while (q < end && *q != '\n') q++;
                if (q < end) q++;
                line++;
                p = q;
                continue;
            }
            if (col > indents.back()) { indents.push_back(col); push(Tk::Indent); }
            else {
                while (col < indents.back()) { indents.pop_back(); push(Tk::Dedent); }
                if (col != indents.back()) fail("E201", line, "inconsistent indentation");
            }
            p = q;
            at_line_start = false;
        }
        char c = *p;
        if (c == '\n') {
            if (depth == 0) { push(Tk::Newline); at_line_start = true; }
            line++;
            p++;
            continue;
        }
        if (c == ' ' || c == '\t' || c == '\r') { p++; continue; }
        if (c == '\\' && p + 1 < end && p[1] == '\n') { p += 2; line++; continue; }
        if (c == '#') { while (p < end && *p != '\n') p++; continue; }
        if (isalpha((unsigned char)c) || c == '_') {
            const char* s = p;
            while (p < end && (isalnum((unsigned char)*p) || *p == '_')) p++;
            push(Tk::Name, std::string(s, p));
            continue;
        }
        if (isdigit((unsigned char)c) || (c == '.' && p + 1 < end && isdigit((unsigned char)p[1]))) {
            const char* s = p;
            bool flt = false;
            if (c == '0' && p + 1 < end && (p[1] == 'x' || p[1] == 'X')) { p += 2; while (p < end && isxdigit((unsigned char)*p)) p++; }
            else {
                while (p < end && (isdigit((unsigned char)*p) || *p == '_')) p++;
                if (p < end && *p == '.') { flt = true; p++; while (p < end && isdigit((unsigned char)*p)) p++; }
                if (p < end && (*p == 'e' || *p == 'E')) {
                    const char* q = p + 1;
                    if (q < end && (*q == '+' || *q == '-')) q++;
                    if (q < end && isdigit((unsigned char)*q)) { flt = true; p = q; while (p < end && isdigit((unsigned char)*p)) p++; }
                }
            }
            std::string body(s, p);
            body.erase(std::remove(body.begin(), body.end(), '_'), body.end());
            Token t;
            t.line = line;
            if (flt) { t.k = Tk::Float; t.f = strtod(body.c_str(), nullptr); }
            else { t.k = Tk::Int; t.i = (int64_t)strtoull(body.c_str(), nullptr, 0); }
            out.push_back(t);
            continue;
        }
        if (c == '"' || c == '\'') {
            int start = line;
            bool triple = p + 2 < end && p[1] == c && p[2] == c;
            p += triple ? 3 : 1;
            std::string body;
            for (;;) {
                if (p >= end) fail("E202", start, "unterminated string literal");
                if (triple ? (p + 2 < end && p[0] == c && p[1] == c && p[2] == c) : *p == c) { p += triple ? 3 : 1; break; }
                if (*p == '\n') { if (!triple) fail("E202", start, "unterminated string literal"); line++; }
                if (*p == '\\' && p + 1 < end) { body += p[1]; p += 2; continue; }
                body += *p++;
            }
            Token t;
            t.k = Tk::Str;
            t.s = body;
            t.line = start;
            out.push_back(t);
            continue;
        }
        static const char* const ops2[] = {"**", "//", "<=", ">=", "==", "!=", "+=", "-=", "*=", "/=", "->", "<<", ">>"};
        bool matched = false;
        for (const char* o : ops2)
            if (p + 1 < end && p[0] == o[0] && p[1] == o[1]) { push(Tk::Op, o); p += 2; matched = true; break; }
        if (matched) continue;
        if (strchr("+-*/%<>=()[]{},:.@&|~^", c)) {
            if (c == '(' || c == '[' || c == '{') depth++;
            if (c == ')' || c == ']' || c == '}') depth = depth > 0 ? depth - 1 : 0;
            push(Tk::Op, std::string(1, c));
            p++;
            continue;
        }
        fail("E200", line, std::string("unexpected character `") + c + "`");
    }
    if (!out.empty() && out.back().k != Tk::Newline) push(Tk::Newline);
    while (indents.size() > 1) { indents.pop_back(); push(Tk::Dedent); }
    push(Tk::Eof);
    return out;
}

// ---------------------------------------------------------------------------------------------
// AST
// ---------------------------------------------------------------------------------------------
struct Expr;
using EP = std::shared_ptr<Expr>;
struct Expr {
    enum K { Name, Int, Float, Str, Attr, Call, Bin, Cmp, Unary, Subscript, Tuple, NoneLit, SliceAll, BoolLit } k = Name;
    std::string s;   // name, attribute, operator
    int64_t i = 0;
    double f = 0;
    EP a, b;
    std::vector<EP> args;
    std::vector<std::pair<std::string, EP>> kwargs;
    int line = 0;
};
struct Stmt {
    enum K { Assign, AugAssign, ExprStmt, For, If, Return, Pass } k = Pass;
    std::string target, op;
    EP value, cond;
    std::vector<EP> range_args;
    std::vector<Stmt> body, orelse;
    int line = 0;
};
struct Param {
    std::string name;
    bool is_constexpr = false;
    EP def;
};
struct Kernel {
    std::string name;
    std::vector<Param> params;
    std::vector<Stmt> body;
    int line = 0;
};

class Parser {
public:
    explicit Parser(std::vector<Token> t) : t_(std::move(t)) {}
    std::vector<Kernel> run() {
        std::vector<Kernel> ks;
        while (tok().k != Tk::Eof) {
            if (is_op("@")) {
                bool jit = false;
                while (is_op("@")) {
                    i_++;
                    std::string dotted = name();
                    while (eat_op(".")) dotted += "." + name();
                    if (is_op("(")) skip_parens();
                    if (dotted == "triton.jit" || dotted == "jit" || dotted == "tl.jit") jit = true;
                    need(Tk::Newline);
                }
                if (!is_name("def")) fail("E201", tok().line, "expected `def` after a decorator");
                if (jit) ks.push_back(def());
                else skip_statement();
            } else skip_statement();
        }
        return ks;
    }

private:
    std::vector<Token> t_;
    size_t i_ = 0;
    const Token& tok() const { return t_[i_]; }
    bool is_op(const char* s) const { return tok().k == Tk::Op && tok().s == s; }
    bool is_name(const char* s) const { return tok().k == Tk::Name && tok().s == s; }
    bool eat_op(const char* s) { if (is_op(s)) { i_++; return true; } return false; }
    bool eat_name(const char* s) { if (is_name(s)) { i_++; return true; } return false; }
    void need_op(const char* s) { if (!eat_op(s)) fail("E201", tok().line, std::string("expected `") + s + "`, found `" + show() + "`"); }
    void need(Tk k) { if (tok().k != k) fail("E201", tok().line, "unexpected `" + show() + "`"); i_++; }
    std::string show() const {
        switch (tok().k) {
            case Tk::Newline: return "end of line";
            case Tk::Indent: return "indent";
            case Tk::Dedent: return "dedent";
            case Tk::Eof: return "end of file";
            case Tk::Int: return std::to_string(tok().i);
            case Tk::Float: return std::to_string(tok().f);
            default: return tok().s;
        }
    }
    std::string name() {
        if (tok().k != Tk::Name) fail("E201", tok().line, "expected a name, found `" + show() + "`");
        return t_[i_++].s;
    }
    void skip_parens() {
        int depth = 0;
        do {
            if (tok().k == Tk::Eof) fail("E202", tok().line, "unterminated bracket");
            if (is_op("(") || is_op("[") || is_op("{")) depth++;
            if (is_op(")") || is_op("]") || is_op("}")) depth--;
            i_++;
        } while (depth > 0);
    }
    // anything that is not a kernel: skip the logical line and, if it opens a block, the block
    void skip_statement() {
        while (tok().k != Tk::Newline && tok().k != Tk::Eof) i_++;
        if (tok().k == Tk::Newline) i_++;
        if (tok().k == Tk::Indent) {
            int depth = 0;
            do {
                if (tok().k == Tk::Indent) depth++;
                if (tok().k == Tk::Dedent) depth--;
                if (tok().k == Tk::Eof) return;
                i_++;
            } while (depth > 0);
        }
    }

    Kernel def() {
        Kernel k;
        k.line = tok().line;
        i_++;   // def
        k.name = name();
        need_op("(");
        while (!is_op(")")) {
            if (is_op("*") || is_op("**")) fail("E304", tok().line, "variadic parameters are outside the subset");
            Param p;
            p.name = name();
            if (eat_op(":")) {
                EP ann = expr();
                std::string text = dotted(ann);
                if (text == "tl.constexpr" || text == "constexpr" || text == "triton.language.constexpr") p.is_constexpr = true;
            }
            if (eat_op("=")) p.def = expr();
            k.params.push_back(p);
            if (!eat_op(",")) break;
        }
        need_op(")");
        if (eat_op("->")) expr();
        need_op(":");
        k.body = block();
        return k;
    }
    static std::string dotted(const EP& e) {
        if (!e) return "";
        if (e->k == Expr::Name) return e->s;
        if (e->k == Expr::Attr) return dotted(e->a) + "." + e->s;
        if (e->k == Expr::Str) return e->s;
        return "?";
    }

    std::vector<Stmt> block() {
        std::vector<Stmt> body;
        if (tok().k != Tk::Newline) {   // `if x: stmt` on one line
            body.push_back(simple());
            return body;
        }
        need(Tk::Newline);
        need(Tk::Indent);
        while (tok().k != Tk::Dedent && tok().k != Tk::Eof) statement(&body);
        if (tok().k == Tk::Dedent) i_++;
        return body;
    }

    void statement(std::vector<Stmt>* out) {
        int line = tok().line;
        if (eat_name("for")) {
            Stmt s;
            s.k = Stmt::For;
            s.line = line;
            s.target = name();
            if (!eat_name("in")) fail("E201", tok().line, "expected `in`");
            EP it = expr();
            std::string callee = it->k == Expr::Call ? dotted(it->a) : "";
            if (callee != "range" && callee != "tl.range" && callee != "tl.static_range") fail("E304", line, "only `for ... in range(...)` loops are in the subset");
            s.range_args = it->args;
            need_op(":");
            s.body = block();
            out->push_back(s);
            return;
        }
        if (eat_name("if")) {
            Stmt s;
            s.k = Stmt::If;
            s.line = line;
            s.cond = expr();
            need_op(":");
            s.body = block();
            if (eat_name("else")) { need_op(":"); s.orelse = block(); }
            else if (is_name("elif")) fail("E304", tok().line, "`elif` is outside the subset");
            out->push_back(s);
            return;
        }
        for (const char* k : {"while", "with", "try", "def", "class", "lambda", "import", "from", "global", "assert", "raise", "del"})
            if (is_name(k)) fail("E304", line, std::string("`") + k + "` is outside the subset");
        out->push_back(simple());
        if (tok().k == Tk::Newline) i_++;
        else if (tok().k != Tk::Dedent && tok().k != Tk::Eof) fail("E201", tok().line, "unexpected `" + show() + "`");
    }

    Stmt simple() {
        Stmt s;
        s.line = tok().line;
        if (eat_name("pass")) { s.k = Stmt::Pass; return s; }
        if (eat_name("return")) {
            s.k = Stmt::Return;
            if (tok().k != Tk::Newline) s.value = expr();
            return s;
        }
        EP e = expr();
        if (is_op("=")) {
            i_++;
            if (e->k != Expr::Name) fail("E304", s.line, "only plain names can be assigned to");
            s.k = Stmt::Assign;
            s.target = e->s;
            s.value = expr();
            return s;
        }
        for (const char* o : {"+=", "-=", "*=", "/="}) {
            if (!is_op(o)) continue;
            i_++;
            if (e->k != Expr::Name) fail("E304", s.line, "only plain names can be assigned to");
            s.k = Stmt::AugAssign;
            s.target = e->s;
            s.op = std::string(1, o[0]);
            s.value = expr();
            return s;
        }
        s.k = Stmt::ExprStmt;
        s.value = e;
        return s;
    }

    EP mk(Expr::K k, int line) {
        EP e = std::make_shared<Expr>();
        e->k = k;
        e->line = line;
        return e;
    }
    EP expr() {
        EP e = or_expr();
        if (is_name("if")) fail("E304", tok().line, "conditional expressions are outside the subset (use tl.where)");
        return e;
    }
    EP or_expr() {
        EP l = and_expr();
        while (is_name("or")) { int ln = tok().line; i_++; EP r = and_expr(); EP b = mk(Expr::Bin, ln); b->s = "or"; b->a = l; b->b = r; l = b; }
        return l;
    }
    EP and_expr() {
        EP l = not_expr();
        while (is_name("and")) { int ln = tok().line; i_++; EP r = not_expr(); EP b = mk(Expr::Bin, ln); b->s = "and"; b->a = l; b->b = r; l = b; }
        return l;
    }
    EP not_expr() {
        if (is_name("not")) { int ln = tok().line; i_++; EP u = mk(Expr::Unary, ln); u->s = "not"; u->a = not_expr(); return u; }
        return comparison();
    }
    EP comparison() {
        EP l = bin_level(0);
        for (const char* o : {"<", ">", "<=", ">=", "==", "!="}) {
            if (!is_op(o)) continue;
            int ln = tok().line;
            i_++;
            EP c = mk(Expr::Cmp, ln);
            c->s = o;
            c->a = l;
            c->b = bin_level(0);
            for (const char* o2 : {"<", ">", "<=", ">=", "==", "!="}) if (is_op(o2)) fail("E304", tok().line, "chained comparisons are outside the subset");
            return c;
        }
        if (is_name("is") || is_name("in")) fail("E304", tok().line, "`is` / `in` are outside the subset");
        return l;
    }
    // levels: 0 |, 1 ^, 2 &, 3 << >>, 4 + -, 5 * / // %
    EP bin_level(int level) {
        static const std::vector<std::vector<std::string>> ops = {{"|"}, {"^"}, {"&"}, {"<<", ">>"}, {"+", "-"}, {"*", "/", "//", "%", "@"}};
        if (level == (int)ops.size()) return unary();
        EP l = bin_level(level + 1);
        for (;;) {
            bool found = false;
            for (auto& o : ops[level]) {
                if (!is_op(o.c_str())) continue;
                int ln = tok().line;
                i_++;
                EP r = bin_level(level + 1);
                EP b = mk(Expr::Bin, ln);
                b->s = o;
                b->a = l;
                b->b = r;
                l = b;
                found = true;
                break;
            }
            if (!found) return l;
        }
    }
    EP unary() {
        int ln = tok().line;
        if (eat_op("-")) { EP u = mk(Expr::Unary, ln); u->s = "-"; u->a = unary(); return u; }
        if (eat_op("+")) return unary();
        if (eat_op("~")) { EP u = mk(Expr::Unary, ln); u->s = "~"; u->a = unary(); return u; }
        EP e = postfix();
        if (is_op("**")) fail("E304", tok().line, "`**` is outside the subset");
        return e;
    }
    EP postfix() {
        EP e = atom();
        for (;;) {
            int ln = tok().line;
            if (eat_op(".")) { EP a = mk(Expr::Attr, ln); a->s = name(); a->a = e; e = a; continue; }
            if (eat_op("(")) {
                EP c = mk(Expr::Call, ln);
                c->a = e;
                while (!is_op(")")) {
                    if (is_op("*") || is_op("**")) fail("E304", tok().line, "argument unpacking is outside the subset");
                    if (tok().k == Tk::Name && t_[i_ + 1].k == Tk::Op && t_[i_ + 1].s == "=") {
                        std::string kw = name();
                        i_++;
                        c->kwargs.push_back({kw, expr()});
                    } else c->args.push_back(expr());
                    if (!eat_op(",")) break;
                }
                need_op(")");
                e = c;
                continue;
            }
            if (eat_op("[")) {
                EP s = mk(Expr::Subscript, ln);
                s->a = e;
                while (!is_op("]")) {
                    if (eat_op(":")) {
                        if (!is_op(",") && !is_op("]")) fail("E307", tok().line, "partial slices are outside the subset");
                        s->args.push_back(mk(Expr::SliceAll, ln));
                    } else {
                        EP idx = expr();
                        if (is_op(":")) fail("E307", tok().line, "partial slices are outside the subset");
                        s->args.push_back(idx);
                    }
                    if (!eat_op(",")) break;
                }
                need_op("]");
                e = s;
                continue;
            }
            return e;
        }
    }
    EP atom() {
        int ln = tok().line;
        if (tok().k == Tk::Int) { EP e = mk(Expr::Int, ln); e->i = t_[i_++].i; return e; }
        if (tok().k == Tk::Float) { EP e = mk(Expr::Float, ln); e->f = t_[i_++].f; return e; }
        if (tok().k == Tk::Str) { EP e = mk(Expr::Str, ln); e->s = t_[i_++].s; return e; }
        if (tok().k == Tk::Name) {
            std::string n = t_[i_++].s;
            if (n == "None") return mk(Expr::NoneLit, ln);
            if (n == "True" || n == "False") { EP e = mk(Expr::BoolLit, ln); e->i = n == "True"; return e; }
            if (n == "lambda") fail("E304", ln, "`lambda` is outside the subset");
            EP e = mk(Expr::Name, ln);
            e->s = n;
            return e;
        }
        if (eat_op("(")) {
            if (eat_op(")")) return mk(Expr::Tuple, ln);
            EP first = expr();
            if (is_op(",")) {
                EP t = mk(Expr::Tuple, ln);
                t->args.push_back(first);
                while (eat_op(",")) { if (is_op(")")) break; t->args.push_back(expr()); }
                need_op(")");
                return t;
            }
            need_op(")");
            return first;
        }
        if (eat_op("[")) {
            EP t = mk(Expr::Tuple, ln);
            while (!is_op("]")) { t->args.push_back(expr()); if (!eat_op(",")) break; }
            need_op("]");
            return t;
        }
        fail("E201", ln, "expected an expression, found `" + show() + "`");
    }
};

// ---------------------------------------------------------------------------------------------
// Symbolic tile values
// ---------------------------------------------------------------------------------------------
enum class El : uint8_t { I1, I32, I64, F16, F32, F64 };
Scalar scalar_of(El e) {
    switch (e) {
        case El::I1: return Scalar::I1;
        case El::I32: return Scalar::I32;
        case El::I64: return Scalar::I64;
        case El::F16: return Scalar::F16;
        case El::F32: return Scalar::F32;
        default: return Scalar::F64;
    }
}
bool is_flt(El e) { return e >= El::F16; }

struct Dim {
    int64_t n = 1;
    int sym = -1;   // >= 0: the extent is the run-time value of this BIR parameter
    bool operator==(const Dim& o) const { return n == o.n && sym == o.sym; }
    bool is_one() const { return sym < 0 && n == 1; }
};

struct Node;
using NP = std::shared_ptr<Node>;
struct Node {
    enum K { CInt, CFlt, PScalar, PPtr, Pid, NProg, Arange, Bin, Cmp, Neg, Not, Expand, Load, Dot, Zeros, Cast, Where, Reduce } k = CInt;
    El el = El::I64;
    bool is_ptr = false;
    El pointee = El::F32;
    std::vector<Dim> shape;
    std::vector<NP> in;   // Load: ptr, mask?, other?   Dot: a, b, acc   Where: c, a, b
    int64_t iv = 0;       // CInt; Arange lo; Expand axis; Pid axis
    double fv = 0;
    int param = -1;       // BIR parameter index
    std::string op;
    bool has_mask = false, has_other = false;
    int line = 0;
    size_t rank() const { return shape.size(); }
};

struct Value {
    enum K { Tile, Tuple, DType, None } k = None;
    NP n;
    std::vector<int64_t> tup;
    El dt = El::F32;
};

// ---------------------------------------------------------------------------------------------
// Compiler for one kernel
// ---------------------------------------------------------------------------------------------
class KernelCompiler {
public:
    KernelCompiler(const Kernel& k, const TritonOptions& o, Module* m, const std::vector<Kernel>* all = nullptr) : k_(k), opt_(o), m_(m), all_(all) {}

    // Names of the @triton.jit functions this one calls (by plain name): those are helpers, inlined at the call.
    static void callees(const std::vector<Stmt>& body, const std::vector<Kernel>& all, std::set<std::string>* out) {
        for (auto& s : body) {
            callees_in(s.value, all, out);
            callees_in(s.cond, all, out);
            for (auto& a : s.range_args) callees_in(a, all, out);
            callees(s.body, all, out);
            callees(s.orelse, all, out);
        }
    }

    Function run() {
        classify_params();
        f_.name = k_.name;
        f_.is_kernel = true;
        f_.ret = Ty::v();
        cur_ = new_block();
        exec(k_.body);
        if (!closed_[cur_]) ret();
        canonicalize(f_);
        return std::move(f_);
    }

private:
    const Kernel& k_;
    const TritonOptions& opt_;
    Module* m_;
    const std::vector<Kernel>* all_;   // every @triton.jit function of the source, for calls between them
    int depth_ = 0;                    // nesting of inlined calls
    Value ret_value_;                  // what the innermost inlined call returned
    int shared_cells_ = 0;
    Function f_;
    std::map<std::string, Value> env_;
    uint32_t cur_ = 0;
    std::vector<bool> closed_;
    bool returned_ = false;

    static void callees_in(const EP& e, const std::vector<Kernel>& all, std::set<std::string>* out) {
        if (!e) return;
        if (e->k == Expr::Call && e->a && e->a->k == Expr::Name)
            for (auto& g : all) if (g.name == e->a->s) out->insert(g.name);
        callees_in(e->a, all, out);
        callees_in(e->b, all, out);
        for (auto& a : e->args) callees_in(a, all, out);
        for (auto& kw : e->kwargs) callees_in(kw.second, all, out);
    }
    const Kernel* jit_function(const std::string& name) const {
        if (!all_) return nullptr;
        for (auto& g : *all_) if (g.name == name) return &g;
        return nullptr;
    }
    // Which parameters of a helper are used as pointers (in its own body, or passed on to a helper that does).
    std::set<std::string> pointer_params_of(const Kernel& g, int depth) {
        std::set<std::string> names;
        if (depth > 8) return names;
        std::vector<const Stmt*> assigns;
        pointer_positions(g.body, &names, &assigns, depth + 1);
        for (bool grew = true; grew;) {
            grew = false;
            for (const Stmt* s : assigns) {
                if (!names.count(s->target)) continue;
                std::set<std::string> more;
                additive_names(s->value, &more);
                for (auto& m : more) if (names.insert(m).second) grew = true;
            }
        }
        return names;
    }

    // ---- parameters ----
    static void additive_names(const EP& e, std::set<std::string>* out) {
        if (!e) return;
        if (e->k == Expr::Name) out->insert(e->s);
        else if (e->k == Expr::Bin && (e->s == "+" || e->s == "-")) { additive_names(e->a, out); additive_names(e->b, out); }
        else if (e->k == Expr::Subscript) additive_names(e->a, out);
    }
    void pointer_positions(const std::vector<Stmt>& body, std::set<std::string>* names, std::vector<const Stmt*>* assigns, int depth = 0) {
        for (auto& s : body) {
            if (s.k == Stmt::For || s.k == Stmt::If) { pointer_positions(s.body, names, assigns, depth); pointer_positions(s.orelse, names, assigns, depth); }
            if (s.k == Stmt::Assign || s.k == Stmt::AugAssign) assigns->push_back(&s);
            if (s.value) find_calls(s.value, names, depth);
        }
    }
    void find_calls(const EP& e, std::set<std::string>* names, int depth = 0) {
        if (!e) return;
        if (e->k == Expr::Call) {
            std::string callee = dotted(e->a);
            const bool memory = callee == "tl.load" || callee == "tl.store" || callee.rfind("tl.atomic_", 0) == 0;
            if (memory && !e->args.empty()) additive_names(e->args[0], names);
            for (auto& kw : e->kwargs) if (memory && (kw.first == "pointer" || kw.first == "ptr")) additive_names(kw.second, names);
            if (const Kernel* g = jit_function(callee)) {   // an argument bound to a helper's pointer parameter is a pointer here too
                std::set<std::string> ptrs = pointer_params_of(*g, depth);
                for (size_t i = 0; i < e->args.size() && i < g->params.size(); i++)
                    if (ptrs.count(g->params[i].name)) additive_names(e->args[i], names);
                for (auto& kw : e->kwargs) if (ptrs.count(kw.first)) additive_names(kw.second, names);
            }
        }
        find_calls(e->a, names, depth);
        find_calls(e->b, names, depth);
        for (auto& a : e->args) find_calls(a, names, depth);
        for (auto& kw : e->kwargs) find_calls(kw.second, names, depth);
    }
    // A call of another @triton.jit function of the same source: its body runs here, in a scope of its own,
    // with the arguments bound to its parameters; `return` hands a value back.
    Value call_jit(const Kernel& g, const EP& e) {
        const int line = e->line;
        if (depth_ >= 16) fail("E304", line, "calls between @triton.jit functions nest more than 16 deep (recursion has no lowering)");
        if (e->args.size() > g.params.size()) fail("E300", line, "`" + g.name + "` takes " + std::to_string(g.params.size()) + " arguments");
        std::map<std::string, Value> scope;
        for (size_t i = 0; i < e->args.size(); i++) scope[g.params[i].name] = eval(e->args[i]);
        for (auto& kw : e->kwargs) {
            bool known = false;
            for (auto& p : g.params) known |= p.name == kw.first;
            if (!known) fail("E300", line, "`" + g.name + "` has no parameter `" + kw.first + "`");
            if (scope.count(kw.first)) fail("E300", line, "`" + kw.first + "` is given twice");
            scope[kw.first] = eval(kw.second);
        }
        for (auto& p : g.params) {
            if (scope.count(p.name)) continue;
            if (!p.def) fail("E300", line, "`" + g.name + "` needs an argument for `" + p.name + "`");
            scope[p.name] = eval(p.def);
        }
        std::swap(env_, scope);
        const bool was_returned = returned_;
        Value was_value = ret_value_;
        returned_ = false;
        ret_value_ = Value();
        depth_++;
        exec(g.body);
        depth_--;
        Value out = ret_value_;
        std::swap(env_, scope);
        returned_ = was_returned;
        ret_value_ = was_value;
        return out;
    }
    static std::string dotted(const EP& e) {
        if (!e) return "";
        if (e->k == Expr::Name) return e->s;
        if (e->k == Expr::Attr) return dotted(e->a) + "." + e->s;
        return "?";
    }

    void classify_params() {
        std::set<std::string> ptr_names;
        std::vector<const Stmt*> assigns;
        pointer_positions(k_.body, &ptr_names, &assigns);
        for (bool grew = true; grew;) {   // a name assigned from an additive expression passes pointer-ness on
            grew = false;
            for (const Stmt* s : assigns) {
                if (!ptr_names.count(s->target)) continue;
                std::set<std::string> more;
                additive_names(s->value, &more);
                for (auto& m : more) if (ptr_names.insert(m).second) grew = true;
            }
        }
        for (auto& p : k_.params) {
            if (env_.count(p.name)) fail("E302", k_.line, "parameter `" + p.name + "` is named twice");
            Value v;
            v.k = Value::Tile;
            v.n = std::make_shared<Node>();
            v.n->line = k_.line;
            if (p.is_constexpr) {
                int64_t val = 0;
                bool have = false, in_abi = true;
                if (p.def) {
                    if (p.def->k == Expr::Int) { val = p.def->i; have = true; in_abi = false; }
                    else if (p.def->k == Expr::BoolLit) { val = p.def->i; have = true; in_abi = false; }
                    else if (p.def->k == Expr::Unary && p.def->s == "-" && p.def->a->k == Expr::Int) { val = -p.def->a->i; have = true; in_abi = false; }
                    else fail("E304", k_.line, "the default of constexpr `" + p.name + "` must be an integer literal");
                }
                auto it = opt_.constexprs.find(p.name);
                if (it != opt_.constexprs.end()) { val = it->second; have = true; }
                if (in_abi) { v.n->param = (int)f_.params.size(); f_.params.push_back(Ty::s(Scalar::I64)); }
                if (have) { v.n->k = Node::CInt; v.n->iv = val; v.n->param = -1; }
                else v.n->k = Node::PScalar;   // left symbolic: its run-time value is the extent
                v.n->el = El::I64;
            } else if (opt_.pointee.count(p.name) || ptr_names.count(p.name)) {
                v.n->k = Node::PPtr;
                v.n->is_ptr = true;
                auto it = opt_.pointee.find(p.name);
                Scalar sc = it == opt_.pointee.end() ? Scalar::F32 : it->second;
                v.n->pointee = sc == Scalar::F16 ? El::F16 : sc == Scalar::F64 ? El::F64 : sc == Scalar::I64 ? El::I64 : sc == Scalar::I32 ? El::I32 : El::F32;
                if (sc != Scalar::F16 && sc != Scalar::F32 && sc != Scalar::F64 && sc != Scalar::I64 && sc != Scalar::I32)
                    fail("E300", k_.line, "pointee type of `" + p.name + "` must be f16, f32, f64, i32 or i64");
                v.n->param = (int)f_.params.size();
                f_.params.push_back(Ty::p(Space::Global));
            } else {
                v.n->k = Node::PScalar;
                v.n->el = El::I64;
                v.n->param = (int)f_.params.size();
                f_.params.push_back(Ty::s(Scalar::I64));
            }
            env_[p.name] = v;
        }
    }

    // ---- node constructors ----
    NP node(Node::K k, int line) {
        NP n = std::make_shared<Node>();
        n->k = k;
        n->line = line;
        return n;
    }
    NP cint(int64_t v, int line) { NP n = node(Node::CInt, line); n->iv = v; n->el = El::I64; return n; }
    NP cflt(double v, int line) { NP n = node(Node::CFlt, line); n->fv = v; n->el = El::F32; return n; }

    static bool ceval(const NP& n, int64_t* out) {
        if (!n || n->rank() != 0 || n->is_ptr) return false;
        if (n->k == Node::CInt) { *out = n->iv; return true; }
        if (n->k == Node::Neg) { int64_t a; if (!ceval(n->in[0], &a)) return false; *out = -a; return true; }
        if (n->k == Node::Bin && n->el == El::I64) {
            int64_t a, b;
            if (!ceval(n->in[0], &a) || !ceval(n->in[1], &b)) return false;
            if (n->op == "+") *out = a + b;
            else if (n->op == "-") *out = a - b;
            else if (n->op == "*") *out = a * b;
            else if (n->op == "//" || n->op == "/") { if (b == 0) return false; int64_t q = a / b; if ((a % b != 0) && ((a < 0) != (b < 0))) q--; *out = q; }
            else if (n->op == "%") { if (b == 0) return false; int64_t r = a % b; if (r != 0 && ((r < 0) != (b < 0))) r += b; *out = r; }
            else if (n->op == "&") *out = a & b;
            else if (n->op == "|") *out = a | b;
            else if (n->op == "^") *out = a ^ b;
            else if (n->op == "<<") *out = a << (b & 63);
            else if (n->op == ">>") *out = a >> (b & 63);
            else if (n->op == "min") *out = std::min(a, b);
            else if (n->op == "max") *out = std::max(a, b);
            else return false;
            return true;
        }
        return false;
    }

    std::vector<Dim> broadcast(const NP& a, const NP& b, int line) {
        if (a->rank() == 0) return b->shape;
        if (b->rank() == 0) return a->shape;
        if (a->rank() != b->rank()) fail("E305", line, "tile ranks differ: " + shape_text(a->shape) + " and " + shape_text(b->shape));
        std::vector<Dim> out;
        for (size_t i = 0; i < a->rank(); i++) {
            if (a->shape[i] == b->shape[i]) out.push_back(a->shape[i]);
            else if (a->shape[i].is_one()) out.push_back(b->shape[i]);
            else if (b->shape[i].is_one()) out.push_back(a->shape[i]);
            else fail("E305", line, "tile shapes do not broadcast: " + shape_text(a->shape) + " and " + shape_text(b->shape));
        }
        return out;
    }
    static std::string shape_text(const std::vector<Dim>& s) {
        std::string t = "[";
        for (size_t i = 0; i < s.size(); i++) t += (i ? ", " : "") + (s[i].sym >= 0 ? "%arg" + std::to_string(s[i].sym) : std::to_string(s[i].n));
        return t + "]";
    }

    NP convert(NP n, El to, int line) {
        if (n->is_ptr) fail("E300", line, "a pointer is used as a number");
        if (n->el == to) return n;
        if (n->k == Node::CInt && n->rank() == 0 && is_flt(to)) { NP c = cflt((double)n->iv, line); c->el = to; return c; }
        if (n->k == Node::CInt && n->rank() == 0 && n->el == El::I64 && to == El::I32) { NP c = cint((int64_t)(int32_t)n->iv, line); c->el = El::I32; return c; }
        if (n->k == Node::CFlt && n->rank() == 0 && is_flt(to)) { NP c = cflt(n->fv, line); c->el = to; return c; }
        NP c = node(Node::Cast, line);
        c->el = to;
        c->shape = n->shape;
        c->in = {n};
        return c;
    }

    NP binary(const std::string& op, NP a, NP b, int line) {
        bool logic = op == "&" || op == "|" || op == "^";
        if (a->is_ptr || b->is_ptr) {
            if (op != "+" && op != "-") fail("E300", line, "only + and - apply to pointers");
            if (a->is_ptr && b->is_ptr) fail("E300", line, "two pointers cannot be added");
            if (b->is_ptr) { if (op == "-") fail("E300", line, "a pointer cannot be subtracted from a number"); std::swap(a, b); }
            if (is_flt(b->el)) fail("E300", line, "a pointer offset must be an integer");
            NP n = node(Node::Bin, line);
            n->op = op;
            n->is_ptr = true;
            n->pointee = a->pointee;
            n->shape = broadcast(a, b, line);
            n->in = {a, convert(b, El::I64, line)};
            return n;
        }
        El el;
        if (logic && a->el == El::I1 && b->el == El::I1) el = El::I1;
        else if (is_flt(a->el) || is_flt(b->el)) {
            if (logic || op == "<<" || op == ">>") fail("E300", line, "`" + op + "` needs integer operands");
            el = std::max(is_flt(a->el) ? a->el : El::F16, is_flt(b->el) ? b->el : El::F16);
            // a Python float literal adopts the tile's float type (Triton's weak typing of literals)
            if (a->k == Node::CFlt && a->rank() == 0 && is_flt(b->el)) el = b->el;
            if (b->k == Node::CFlt && b->rank() == 0 && is_flt(a->el)) el = a->el;
            if (op == "/" && !is_flt(a->el) && !is_flt(b->el)) el = El::F32;
        } else if (op == "/") el = El::F32;   // true division of integers
        else {
            // 32-bit data stays 32 bits wide (and wraps there) against itself and against integer literals
            auto is32 = [](const NP& n) { return n->el == El::I32; };
            auto lit = [](const NP& n) { return n->k == Node::CInt && n->rank() == 0 && n->iv >= INT32_MIN && n->iv <= INT32_MAX; };
            el = (is32(a) && (is32(b) || lit(b))) || (is32(b) && lit(a)) ? El::I32 : El::I64;
        }
        if (el == El::F16 && op != "min" && op != "max") fail("E304", line, "arithmetic on float16 tiles is outside the subset; convert with .to(tl.float32)");
        NP n = node(Node::Bin, line);
        n->op = op;
        n->el = el;
        n->shape = broadcast(a, b, line);
        n->in = {convert(a, el, line), convert(b, el, line)};
        int64_t folded;
        if (el == El::I64 && ceval(n, &folded)) return cint(folded, line);
        return n;
    }

    // ---- expression evaluation ----
    NP tile(const Value& v, int line, const char* what) {
        if (v.k != Value::Tile) fail("E300", line, std::string(what) + " must be a number or a tile");
        return v.n;
    }
    int64_t const_of(const NP& n, int line, const char* what) {
        int64_t v;
        if (!ceval(n, &v)) fail("E306", line, std::string(what) + " must be a compile-time constant");
        return v;
    }
    const EP* kwarg(const EP& call, const char* name) {
        for (auto& kw : call->kwargs) if (kw.first == name) return &kw.second;
        return nullptr;
    }
    EP arg_or_kw(const EP& call, size_t pos, const char* name) {
        if (pos < call->args.size()) return call->args[pos];
        if (const EP* k = kwarg(call, name)) return *k;
        return nullptr;
    }

    Value eval(const EP& e) {
        Value v;
        switch (e->k) {
            case Expr::Int: v.k = Value::Tile; v.n = cint(e->i, e->line); return v;
            case Expr::Float: v.k = Value::Tile; v.n = cflt(e->f, e->line); return v;
            case Expr::BoolLit: { v.k = Value::Tile; v.n = cint(e->i, e->line); v.n->el = El::I1; return v; }
            case Expr::NoneLit: v.k = Value::None; return v;
            case Expr::Str: fail("E304", e->line, "string values are outside the subset");
            case Expr::SliceAll: fail("E201", e->line, "`:` outside a subscript");
            case Expr::Name: {
                auto it = env_.find(e->s);
                if (it == env_.end()) fail("E301", e->line, "`" + e->s + "` is not defined");
                return it->second;
            }
            case Expr::Attr: {
                std::string d = dotted(e);
                static const struct { const char* n; El el; } dts[] = {{"tl.float16", El::F16}, {"tl.float32", El::F32}, {"tl.float64", El::F64}, {"tl.int64", El::I64},
                                                                        {"tl.int32", El::I32}, {"tl.int1", El::I1}};
                for (auto& t : dts) if (d == t.n) { v.k = Value::DType; v.dt = t.el; return v; }
                if (d == "tl.bfloat16") fail("E304", e->line, "bfloat16 has no BIR type");
                fail("E301", e->line, "`" + d + "` is not known");
            }
            case Expr::Tuple: {
                v.k = Value::Tuple;
                for (auto& a : e->args) v.tup.push_back(const_of(tile(eval(a), a->line, "a tuple entry"), a->line, "a tuple entry"));
                return v;
            }
            case Expr::Unary: {
                NP a = tile(eval(e->a), e->line, "the operand");
                v.k = Value::Tile;
                if (e->s == "-") {
                    if (a->is_ptr) fail("E300", e->line, "a pointer cannot be negated");
                    int64_t c;
                    if (ceval(a, &c)) { v.n = cint(-c, e->line); return v; }
                    if (a->k == Node::CFlt && a->rank() == 0) { v.n = cflt(-a->fv, e->line); v.n->el = a->el; return v; }
                    NP n = node(Node::Neg, e->line);
                    n->el = a->el == El::I1 ? El::I64 : a->el;
                    n->shape = a->shape;
                    n->in = {convert(a, n->el, e->line)};
                    if (a->k == Node::CInt) { v.n = cint(-a->iv, e->line); v.n->el = a->el; return v; }
                    v.n = n;
                    return v;
                }
                if (e->s == "~" || e->s == "not") {
                    if (a->el != El::I1) fail("E304", e->line, "`" + e->s + "` of a value that is not a mask is outside the subset");
                    NP n = node(Node::Not, e->line);
                    n->el = El::I1;
                    n->shape = a->shape;
                    n->in = {a};
                    v.n = n;
                    return v;
                }
                fail("E304", e->line, "unary `" + e->s + "` is outside the subset");
            }
            case Expr::Bin: {
                if (e->s == "@") fail("E307", e->line, "the `@` operator is outside the subset; use tl.dot");
                NP a = tile(eval(e->a), e->line, "the left operand"), b = tile(eval(e->b), e->line, "the right operand");
                std::string op = e->s == "and" ? "&" : e->s == "or" ? "|" : e->s;
                if ((e->s == "and" || e->s == "or") && (a->el != El::I1 || b->el != El::I1)) fail("E304", e->line, "`and` / `or` of values that are not masks are outside the subset");
                v.k = Value::Tile;
                v.n = binary(op, a, b, e->line);
                return v;
            }
            case Expr::Cmp: {
                NP a = tile(eval(e->a), e->line, "the left operand"), b = tile(eval(e->b), e->line, "the right operand");
                if (a->is_ptr || b->is_ptr) fail("E304", e->line, "pointer comparisons are outside the subset");
                El el = (is_flt(a->el) || is_flt(b->el)) ? std::max(is_flt(a->el) ? a->el : El::F32, is_flt(b->el) ? b->el : El::F32)
                        : (a->el == El::I32 && (b->el == El::I32 || b->k == Node::CInt)) || (b->el == El::I32 && a->k == Node::CInt) ? El::I32 : El::I64;
                NP n = node(Node::Cmp, e->line);
                n->op = e->s;
                n->el = El::I1;
                n->shape = broadcast(a, b, e->line);
                n->in = {convert(a, el, e->line), convert(b, el, e->line)};
                v.k = Value::Tile;
                v.n = n;
                return v;
            }
            case Expr::Subscript: {
                NP a = tile(eval(e->a), e->line, "the subscripted value");
                if (a->rank() != 1 || e->args.size() != 2) fail("E307", e->line, "only x[:, None] and x[None, :] on a rank-1 tile are in the subset");
                bool first_all = e->args[0]->k == Expr::SliceAll, second_all = e->args[1]->k == Expr::SliceAll;
                bool first_none = e->args[0]->k == Expr::NoneLit, second_none = e->args[1]->k == Expr::NoneLit;
                if (!((first_all && second_none) || (first_none && second_all))) fail("E307", e->line, "only x[:, None] and x[None, :] are in the subset");
                NP n = node(Node::Expand, e->line);
                n->el = a->el;
                n->is_ptr = a->is_ptr;
                n->pointee = a->pointee;
                n->iv = first_all ? 1 : 0;   // the axis that was inserted
                Dim one;
                n->shape = first_all ? std::vector<Dim>{a->shape[0], one} : std::vector<Dim>{one, a->shape[0]};
                n->in = {a};
                v.k = Value::Tile;
                v.n = n;
                return v;
            }
            case Expr::Call: return call(e);
        }
        fail("E304", e->line, "expression outside the subset");
    }

    Value call(const EP& e) {
        Value v;
        v.k = Value::Tile;
        int line = e->line;
        // method calls: x.to(dtype)
        if (e->a->k == Expr::Attr && e->a->s == "to" && dotted(e->a).rfind("tl.", 0) != 0) {
            NP x = tile(eval(e->a->a), line, "the converted value");
            EP dt = arg_or_kw(e, 0, "dtype");
            if (!dt) fail("E300", line, ".to() needs a dtype");
            Value d = eval(dt);
            if (d.k != Value::DType) fail("E300", line, ".to() needs a dtype");
            v.n = convert(x, d.dt, line);
            return v;
        }
        std::string callee = dotted(e->a);
        if (const Kernel* g = jit_function(callee)) return call_jit(*g, e);
        if (callee == "tl.program_id" || callee == "tl.num_programs") {
            EP ax = arg_or_kw(e, 0, "axis");
            int64_t axis = ax ? const_of(tile(eval(ax), line, "axis"), line, "the axis") : 0;
            if (axis < 0 || axis > 2) fail("E300", line, "the axis must be 0, 1 or 2");
            NP n = node(callee == "tl.program_id" ? Node::Pid : Node::NProg, line);
            n->iv = axis;
            n->el = El::I64;
            v.n = n;
            return v;
        }
        if (callee == "tl.arange") {
            EP lo = arg_or_kw(e, 0, "start"), hi = arg_or_kw(e, 1, "end");
            if (!lo || !hi) fail("E300", line, "tl.arange takes a start and an end");
            int64_t l = const_of(tile(eval(lo), line, "start"), line, "the start of tl.arange");
            NP h = tile(eval(hi), line, "end");
            NP n = node(Node::Arange, line);
            n->el = El::I64;
            n->iv = l;
            Dim d;
            int64_t hv;
            if (ceval(h, &hv)) {
                if (hv <= l) fail("E300", line, "tl.arange needs end > start");
                d.n = hv - l;
            } else if (h->k == Node::PScalar && h->rank() == 0 && l == 0) d.sym = h->param;   // a constexpr left symbolic
            else fail("E306", line, "the end of tl.arange must be a compile-time constant or a bare constexpr parameter");
            n->shape = {d};
            v.n = n;
            return v;
        }
        if (callee == "tl.zeros" || callee == "tl.full") {
            EP sh = arg_or_kw(e, 0, "shape");
            EP dt = callee == "tl.zeros" ? arg_or_kw(e, 1, "dtype") : arg_or_kw(e, 2, "dtype");
            if (!sh) fail("E300", line, callee + " needs a shape");
            Value s = eval(sh);
            std::vector<int64_t> dims;
            if (s.k == Value::Tuple) dims = s.tup;
            else if (s.k == Value::Tile) dims = {const_of(s.n, line, "the shape")};
            else fail("E300", line, callee + " needs a shape");
            if (dims.empty() || dims.size() > 2) fail("E307", line, "tiles of rank 1 and 2 only");
            El el = El::F32;
            if (dt) { Value d = eval(dt); if (d.k != Value::DType) fail("E300", line, "dtype expected"); el = d.dt; }
            NP n = node(Node::Zeros, line);
            n->el = el;
            for (int64_t x : dims) { if (x <= 0) fail("E300", line, "tile extents must be positive"); Dim d; d.n = x; n->shape.push_back(d); }
            if (callee == "tl.full") {
                EP val = arg_or_kw(e, 1, "value");
                if (!val) fail("E300", line, "tl.full needs a value");
                NP c = tile(eval(val), line, "value");
                if (c->rank() != 0) fail("E300", line, "tl.full needs a scalar value");
                n->in = {convert(c, el, line)};
            }
            v.n = n;
            return v;
        }
        if (callee == "tl.load") {
            EP p = arg_or_kw(e, 0, "pointer"), m = arg_or_kw(e, 1, "mask"), o = arg_or_kw(e, 2, "other");
            if (!p) fail("E300", line, "tl.load needs a pointer");
            NP ptr = tile(eval(p), line, "pointer");
            if (!ptr->is_ptr) fail("E300", line, "tl.load of a value that is not a pointer");
            NP n = node(Node::Load, line);
            n->el = ptr->pointee;
            n->shape = ptr->shape;
            n->in = {ptr};
            if (m && m->k != Expr::NoneLit) {
                NP mask = tile(eval(m), line, "mask");
                if (mask->el != El::I1) fail("E300", line, "a mask must be a comparison result");
                if (!(broadcast(ptr, mask, line) == ptr->shape)) fail("E305", line, "the mask is larger than the pointer tile");
                n->has_mask = true;
                n->in.push_back(mask);
                if (o && o->k != Expr::NoneLit) {
                    NP other = tile(eval(o), line, "other");
                    if (!(broadcast(ptr, other, line) == ptr->shape)) fail("E305", line, "`other` is larger than the pointer tile");
                    n->has_other = true;
                    n->in.push_back(convert(other, n->el, line));
                }
            }
            v.n = n;
            return v;
        }
        if (callee == "tl.store") {
            EP p = arg_or_kw(e, 0, "pointer"), val = arg_or_kw(e, 1, "value"), m = arg_or_kw(e, 2, "mask");
            if (!p || !val) fail("E300", line, "tl.store needs a pointer and a value");
            NP ptr = tile(eval(p), line, "pointer"), x = tile(eval(val), line, "value"), mask;
            if (!ptr->is_ptr) fail("E300", line, "tl.store to a value that is not a pointer");
            if (m && m->k != Expr::NoneLit) {
                mask = tile(eval(m), line, "mask");
                if (mask->el != El::I1) fail("E300", line, "a mask must be a comparison result");
            }
            store(ptr, x, mask, line);
            v.k = Value::None;
            return v;
        }
        if (callee == "tl.dot") {
            EP a = arg_or_kw(e, 0, "input"), b = arg_or_kw(e, 1, "other"), c = arg_or_kw(e, 2, "acc");
            if (!a || !b) fail("E300", line, "tl.dot takes two tiles");
            NP x = tile(eval(a), line, "input"), y = tile(eval(b), line, "other");
            if (x->rank() != 2 || y->rank() != 2) fail("E305", line, "tl.dot needs two rank-2 tiles");
            for (auto& d : {x->shape[0], x->shape[1], y->shape[0], y->shape[1]}) if (d.sym >= 0) fail("E306", line, "tl.dot extents must be compile-time constants");
            if (x->shape[1].n != y->shape[0].n) fail("E305", line, "tl.dot inner extents differ: " + shape_text(x->shape) + " and " + shape_text(y->shape));
            if (x->el != y->el || !is_flt(x->el)) fail("E300", line, "tl.dot operands must have the same floating-point type");
            NP n = node(Node::Dot, line);
            n->el = El::F32;
            n->shape = {x->shape[0], y->shape[1]};
            NP acc;
            if (c && c->k != Expr::NoneLit) {
                acc = tile(eval(c), line, "acc");
                if (acc->rank() != 2 || !(acc->shape == n->shape) || acc->el != El::F32) fail("E305", line, "the tl.dot accumulator must be a float32 tile of the result's shape");
            }
            n->in = {x, y, acc};
            v.n = n;
            return v;
        }
        if (callee == "tl.where") {
            if (e->args.size() != 3) fail("E300", line, "tl.where takes three arguments");
            NP c = tile(eval(e->args[0]), line, "condition"), a = tile(eval(e->args[1]), line, "x"), b = tile(eval(e->args[2]), line, "y");
            if (c->el != El::I1) fail("E300", line, "the condition of tl.where must be a mask");
            if (a->is_ptr || b->is_ptr) fail("E304", line, "tl.where over pointers is outside the subset");
            El el = (is_flt(a->el) || is_flt(b->el)) ? std::max(is_flt(a->el) ? a->el : El::F16, is_flt(b->el) ? b->el : El::F16) : std::max(a->el, b->el);
            if (a->k == Node::CFlt && is_flt(b->el)) el = b->el;
            if (b->k == Node::CFlt && is_flt(a->el)) el = a->el;
            NP n = node(Node::Where, line);
            n->el = el;
            NP ab = node(Node::Zeros, line);
            ab->shape = broadcast(a, b, line);
            n->shape = broadcast(c, ab, line);
            n->in = {c, convert(a, el, line), convert(b, el, line)};
            v.n = n;
            return v;
        }
        if (callee == "tl.maximum" || callee == "tl.minimum" || callee == "min" || callee == "max") {
            if (e->args.size() != 2) fail("E300", line, callee + " takes two arguments");
            NP a = tile(eval(e->args[0]), line, "x"), b = tile(eval(e->args[1]), line, "y");
            v.n = binary(callee.find("max") != std::string::npos ? "max" : "min", a, b, line);
            return v;
        }
        if (callee == "tl.cdiv") {
            if (e->args.size() != 2) fail("E300", line, "tl.cdiv takes two arguments");
            NP a = tile(eval(e->args[0]), line, "x"), b = tile(eval(e->args[1]), line, "y");
            v.n = binary("//", binary("+", a, binary("-", b, cint(1, line), line), line), b, line);
            return v;
        }
        if (callee == "tl.multiple_of" || callee == "tl.max_contiguous" || callee == "tl.max_constancy") {
            if (e->args.empty()) fail("E300", line, callee + " takes a value");
            return eval(e->args[0]);   // compiler hints: the value itself
        }
        if (callee == "tl.sum" || callee == "tl.max" || callee == "tl.min") {
            EP in = arg_or_kw(e, 0, "input"), ax = arg_or_kw(e, 1, "axis");
            if (!in) fail("E300", line, callee + " takes a tile");
            NP x = tile(eval(in), line, "input");
            if (x->rank() != 1) fail("E307", line, "reductions of rank-1 tiles only");
            if (ax && ax->k != Expr::NoneLit && const_of(tile(eval(ax), line, "axis"), line, "the axis") != 0) fail("E300", line, "a rank-1 tile has only axis 0");
            if (x->is_ptr || x->el == El::I1 || x->el == El::F16 || x->el == El::F64 || x->el == El::I64)
                fail("E304", line, "reductions of int32 and float32 tiles only");
            NP n = node(Node::Reduce, line);
            n->op = callee.substr(3);
            n->el = x->el;
            n->in = {x};
            v.n = n;
            return v;
        }
        if (callee == "tl.atomic_add" || callee == "tl.atomic_max" || callee == "tl.atomic_min") {
            EP p = arg_or_kw(e, 0, "pointer"), val = arg_or_kw(e, 1, "val"), m = arg_or_kw(e, 2, "mask");
            if (!p || !val) fail("E300", line, callee + " needs a pointer and a value");
            NP ptr = tile(eval(p), line, "pointer"), x = tile(eval(val), line, "value"), mask;
            if (!ptr->is_ptr) fail("E300", line, callee + " on a value that is not a pointer");
            if (m && m->k != Expr::NoneLit) {
                mask = tile(eval(m), line, "mask");
                if (mask->el != El::I1) fail("E300", line, "a mask must be a comparison result");
            }
            atomic(callee.substr(10), ptr, x, mask, line);
            v.k = Value::None;     // the old value is not modelled
            return v;
        }
        for (const char* k : {"tl.argmax", "tl.argmin", "tl.reshape", "tl.trans", "tl.view", "tl.broadcast_to", "tl.expand_dims", "tl.cumsum", "tl.sort", "tl.join",
                              "tl.split", "tl.permute", "tl.make_block_ptr", "tl.advance", "tl.atomic_cas", "tl.atomic_xchg", "tl.atomic_and", "tl.atomic_or", "tl.atomic_xor"})
            if (callee == k) fail("E307", line, "`" + callee + "` is a tile construct this lowering does not model");
        for (const char* k : {"tl.exp", "tl.log", "tl.sqrt", "tl.sin", "tl.cos", "tl.sigmoid", "tl.softmax", "tl.abs", "tl.rand", "tl.randn", "tl.fma", "tl.exp2", "tl.log2", "tl.rsqrt",
                              "tl.device_print", "tl.static_print", "tl.static_assert", "tl.device_assert", "print"})
            if (callee == k) fail("E304", line, "`" + callee + "` has no BIR lowering");
        fail("E301", line, "`" + callee + "` is not a known function");
    }

    // ---- statements (abstract interpretation) ----
    void exec(const std::vector<Stmt>& body) {
        for (auto& s : body) {
            if (returned_) return;
            switch (s.k) {
                case Stmt::Pass: break;
                case Stmt::Return:
                    if (depth_ > 0) {   // inside an inlined helper: the value goes back to the call
                        if (s.value && s.value->k == Expr::Tuple) fail("E307", s.line, "a helper that returns several values is not modelled");
                        ret_value_ = s.value && s.value->k != Expr::NoneLit ? eval(s.value) : Value();
                    } else if (s.value && s.value->k != Expr::NoneLit) fail("E300", s.line, "a kernel returns nothing");
                    returned_ = true;
                    break;
                case Stmt::ExprStmt:
                    if (s.value->k == Expr::Str) break;   // docstring
                    eval(s.value);
                    break;
                case Stmt::Assign: env_[s.target] = eval(s.value); break;
                case Stmt::AugAssign: {
                    auto it = env_.find(s.target);
                    if (it == env_.end()) fail("E301", s.line, "`" + s.target + "` is not defined");
                    NP a = tile(it->second, s.line, "the target"), b = tile(eval(s.value), s.line, "the operand");
                    Value v;
                    v.k = Value::Tile;
                    v.n = binary(s.op, a, b, s.line);
                    env_[s.target] = v;
                    break;
                }
                case Stmt::For: {
                    std::vector<int64_t> r;
                    for (auto& a : s.range_args) r.push_back(const_of(tile(eval(a), s.line, "a range bound"), s.line, "a range bound"));
                    if (r.empty() || r.size() > 3) fail("E300", s.line, "range takes one to three arguments");
                    int64_t lo = r.size() == 1 ? 0 : r[0], hi = r.size() == 1 ? r[0] : r[1], step = r.size() == 3 ? r[2] : 1;
                    if (step <= 0) fail("E304", s.line, "range steps must be positive");
                    if ((hi - lo + step - 1) / step > 65536) fail("E304", s.line, "the loop is too long to unroll");
                    for (int64_t i = lo; i < hi && !returned_; i += step) {
                        Value v;
                        v.k = Value::Tile;
                        v.n = cint(i, s.line);
                        env_[s.target] = v;
                        exec(s.body);
                    }
                    break;
                }
                case Stmt::If: {
                    NP c = tile(eval(s.cond), s.line, "the condition");
                    int64_t cv;
                    if (c->rank() != 0) fail("E300", s.line, "the condition of `if` must be a scalar");
                    if (c->k == Node::CInt) cv = c->iv;
                    else if (!ceval(c, &cv)) fail("E304", s.line, "`if` on a run-time value is outside the subset (use masks)");
                    exec(cv ? s.body : s.orelse);
                    break;
                }
            }
        }
    }

    // ---- BIR emission ----
    uint32_t new_block() {
        f_.blocks.emplace_back();
        closed_.push_back(false);
        return (uint32_t)f_.blocks.size() - 1;
    }
    Val push(const Inst& in) {
        uint32_t id = (uint32_t)f_.insts.size();
        f_.insts.push_back(in);
        f_.blocks[cur_].insts.push_back(id);
        return Val::V(id);
    }
    void br(uint32_t to) {
        Term& t = f_.blocks[cur_].term;
        t.kind = Term::Br;
        t.t = to;
        closed_[cur_] = true;
    }
    void condbr(Val c, uint32_t tb, uint32_t fb) {
        Term& t = f_.blocks[cur_].term;
        t.kind = Term::CondBr;
        t.has_val = true;
        t.val = c;
        t.t = tb;
        t.f = fb;
        closed_[cur_] = true;
    }
    void ret() {
        Term& t = f_.blocks[cur_].term;
        t.kind = Term::Ret;
        t.has_val = false;
        closed_[cur_] = true;
    }
    static const Ty I64() { return Ty::s(Scalar::I64); }
    Val ci(Ty ty, int64_t v) { Inst in; in.op = Opc::ConstI; in.ty = ty; in.imm = v; return push(in); }
    Val cf(Ty ty, double v) { Inst in; in.op = Opc::ConstF; in.ty = ty; in.fimm = v; return push(in); }
    Val bin(BinOp op, Ty ty, Val a, Val b) { Inst in; in.op = Opc::Bin; in.sub = (uint8_t)op; in.ty = ty; in.ops = {a, b}; return push(in); }
    Val icmp(ICmp p, Ty operand, Val a, Val b) { Inst in; in.op = Opc::ICmp; in.sub = (uint8_t)p; in.ty = Ty::s(Scalar::I1); in.aux = operand; in.ops = {a, b}; return push(in); }
    Val fcmp(FCmp p, Ty operand, Val a, Val b) { Inst in; in.op = Opc::FCmp; in.sub = (uint8_t)p; in.ty = Ty::s(Scalar::I1); in.aux = operand; in.ops = {a, b}; return push(in); }
    Val select(Ty ty, Val c, Val a, Val b) { Inst in; in.op = Opc::Select; in.ty = ty; in.ops = {c, a, b}; return push(in); }
    Val cast(CastOp op, Ty to, Ty from, Val v) { Inst in; in.op = Opc::Cast; in.sub = (uint8_t)op; in.ty = to; in.aux = from; in.ops = {v}; return push(in); }
    Val index(unsigned sub) { Inst in; in.op = Opc::Index; in.sub = (uint8_t)sub; in.ty = I64(); return push(in); }
    Val phi(Ty ty, std::vector<std::pair<uint32_t, Val>> arms) {
        Inst in;
        in.op = Opc::Phi;
        in.ty = ty;
        for (auto& a : arms) { in.phi_blocks.push_back(a.first); in.ops.push_back(a.second); }
        return push(in);
    }

    // Instantiates a node at tile position (i, j); `idx` holds one i64 value per axis of the
    // consumer's shape (rank 1: {i}; rank 2: {i, j}).  Values are memoised per scope, and a scope
    // ends with the branch it was opened for, so a cached value always dominates its reuse.
    struct Scope { std::map<std::pair<const Node*, std::pair<uint32_t, uint32_t>>, Val> memo; };
    std::vector<Scope> scopes_;
    static uint32_t key_of(Val v) { return (v.param ? 0x80000000u : 0u) | v.idx; }

    std::vector<Val> child_idx(const NP& child, const std::vector<Val>& idx) const {
        // same-rank children (or scalars) take the consumer's indices; an axis of extent 1 is read at 0 in gen()
        if (child->rank() == 0) return {};
        return idx;
    }

    Val gen(const NP& n, const std::vector<Val>& idx) {
        if (n->rank() > idx.size()) fail("E305", n->line, "a rank-" + std::to_string(n->rank()) + " tile is used where rank " + std::to_string(idx.size()) + " is stored");
        std::pair<uint32_t, uint32_t> ik{n->rank() > 0 ? key_of(idx[0]) : 0xffffffffu, n->rank() > 1 ? key_of(idx[1]) : 0xffffffffu};
        auto key = std::make_pair((const Node*)n.get(), ik);
        for (auto s = scopes_.rbegin(); s != scopes_.rend(); ++s) {
            auto it = s->memo.find(key);
            if (it != s->memo.end()) return it->second;
        }
        Val v = gen_uncached(n, idx);
        scopes_.back().memo[key] = v;
        return v;
    }

    Val gen_uncached(const NP& n, const std::vector<Val>& idx) {
        const Ty ty = n->is_ptr ? Ty::p(Space::Global) : Ty::s(scalar_of(n->el));
        switch (n->k) {
            case Node::CInt: return ci(ty, n->iv);
            case Node::CFlt: return cf(ty, n->el == El::F32 ? (double)(float)n->fv : n->fv);
            case Node::PScalar: case Node::PPtr: return Val::P((uint32_t)n->param);
            case Node::Pid: return index(3 + (unsigned)n->iv);
            case Node::NProg: return index(9 + (unsigned)n->iv);
            case Node::Arange: {
                Val i = n->shape[0].is_one() ? ci(I64(), 0) : idx[0];
                return n->iv ? bin(BinOp::Add, I64(), i, ci(I64(), n->iv)) : i;
            }
            case Node::Expand: {
                // the child is rank 1; its axis is the one that was not inserted
                Val i = idx[n->iv == 1 ? 0 : 1];
                if (n->in[0]->shape[0].is_one()) i = ci(I64(), 0);
                return gen(n->in[0], {i});
            }
            case Node::Zeros: return n->in.empty() ? (is_flt(n->el) ? cf(ty, 0.0) : ci(ty, 0)) : gen(n->in[0], {});
            case Node::Neg: {
                Val a = gen(n->in[0], sub_idx(n->in[0], idx));
                return is_flt(n->el) ? bin(BinOp::FSub, ty, cf(ty, 0.0), a) : bin(BinOp::Sub, ty, ci(ty, 0), a);
            }
            case Node::Not: {
                Val a = gen(n->in[0], sub_idx(n->in[0], idx));
                return bin(BinOp::Xor, ty, a, ci(ty, 1));
            }
            case Node::Cast: {
                const NP& c = n->in[0];
                Val a = gen(c, sub_idx(c, idx));
                Ty from = Ty::s(scalar_of(c->el));
                if (is_flt(c->el) && is_flt(n->el)) return cast(n->el > c->el ? CastOp::FPExt : CastOp::FPTrunc, ty, from, a);
                if (is_flt(n->el)) {
                    if (c->el == El::I1) return cast(CastOp::UIToFP, ty, I64(), cast(CastOp::ZExt, I64(), from, a));
                    return cast(CastOp::SIToFP, ty, from, a);
                }
                if (is_flt(c->el)) {
                    if (n->el == El::I1) return fcmp(FCmp::One, from, a, cf(from, 0.0));
                    return cast(CastOp::FPToSI, ty, from, a);
                }
                if (n->el == El::I1) return icmp(ICmp::Ne, from, a, ci(from, 0));
                if (c->el == El::I1) return cast(CastOp::ZExt, ty, from, a);
                return cast(n->el > c->el ? CastOp::SExt : CastOp::Trunc, ty, from, a);   // i32 <-> i64
            }
            case Node::Cmp: {
                const NP &x = n->in[0], &y = n->in[1];
                Val a = gen(x, sub_idx(x, idx)), b = gen(y, sub_idx(y, idx));
                Ty ot = Ty::s(scalar_of(x->el));
                const std::string& o = n->op;
                if (is_flt(x->el)) return fcmp(o == "<" ? FCmp::Olt : o == ">" ? FCmp::Ogt : o == "<=" ? FCmp::Ole : o == ">=" ? FCmp::Oge : o == "==" ? FCmp::Oeq : FCmp::One, ot, a, b);
                return icmp(o == "<" ? ICmp::Slt : o == ">" ? ICmp::Sgt : o == "<=" ? ICmp::Sle : o == ">=" ? ICmp::Sge : o == "==" ? ICmp::Eq : ICmp::Ne, ot, a, b);
            }
            case Node::Where: {
                Val c = gen(n->in[0], sub_idx(n->in[0], idx)), a = gen(n->in[1], sub_idx(n->in[1], idx)), b = gen(n->in[2], sub_idx(n->in[2], idx));
                return select(ty, c, a, b);
            }
            case Node::Bin: {
                const NP &x = n->in[0], &y = n->in[1];
                Val a = gen(x, sub_idx(x, idx)), b = gen(y, sub_idx(y, idx));
                const std::string& o = n->op;
                if (n->is_ptr) {
                    Val off = bin(BinOp::Mul, I64(), b, ci(I64(), scalar_bytes(scalar_of(n->pointee))));
                    if (o == "-") off = bin(BinOp::Sub, I64(), ci(I64(), 0), off);
                    return bin(BinOp::Add, ty, a, off);
                }
                if (o == "min" || o == "max") {
                    Val c = is_flt(n->el) ? fcmp(o == "min" ? FCmp::Olt : FCmp::Ogt, ty, a, b) : icmp(o == "min" ? ICmp::Slt : ICmp::Sgt, ty, a, b);
                    return select(ty, c, a, b);
                }
                if (is_flt(n->el)) {
                    if (o == "+") return bin(BinOp::FAdd, ty, a, b);
                    if (o == "-") return bin(BinOp::FSub, ty, a, b);
                    if (o == "*") return bin(BinOp::FMul, ty, a, b);
                    if (o == "/") return bin(BinOp::FDiv, ty, a, b);
                    fail("E304", n->line, "`" + o + "` on floating-point tiles is outside the subset");
                }
                if (o == "+") return bin(BinOp::Add, ty, a, b);
                if (o == "-") return bin(BinOp::Sub, ty, a, b);
                if (o == "*") return bin(BinOp::Mul, ty, a, b);
                if (o == "&") return bin(BinOp::And, ty, a, b);
                if (o == "|") return bin(BinOp::Or, ty, a, b);
                if (o == "^") return bin(BinOp::Xor, ty, a, b);
                if (o == "<<") return bin(BinOp::Shl, ty, a, b);
                if (o == ">>") return bin(BinOp::AShr, ty, a, b);
                if (o == "//" || o == "%") {
                    // Python floors; BIR division truncates.  They agree for non-negative operands,
                    // which is what index arithmetic uses; a constant positive divisor is required.
                    int64_t d;
                    if (!ceval(y, &d) || d <= 0) fail("E304", n->line, "`" + o + "` needs a positive compile-time divisor");
                    return bin(o == "//" ? BinOp::Div : BinOp::Rem, ty, a, b);
                }
                fail("E304", n->line, "`" + o + "` is outside the subset");
            }
            case Node::Load: {
                const NP& p = n->in[0];
                Ty vt = Ty::s(scalar_of(n->el));
                auto do_load = [&]() {
                    Val addr = gen(p, sub_idx(p, idx));
                    Inst in;
                    in.op = Opc::Load;
                    in.ty = vt;
                    in.space = Space::Global;
                    in.align = scalar_bytes(vt.sc);
                    in.ops = {addr};
                    return push(in);
                };
                const bool guarded = lane_ && lane_->guarded;
                if (!n->has_mask && !guarded) return do_load();
                Val m;
                if (n->has_mask) {
                    m = gen(n->in[1], sub_idx(n->in[1], idx));
                    if (guarded) m = bin(BinOp::And, Ty::s(Scalar::I1), m, lane_->guard);   // a lane past the tile loads nothing
                } else m = lane_->guard;
                Val other = n->has_other ? gen(n->in[2], sub_idx(n->in[2], idx)) : (is_flt(n->el) ? cf(vt, 0.0) : ci(vt, 0));
                uint32_t from = cur_, tb = new_block(), mb = new_block();
                condbr(m, tb, mb);
                cur_ = tb;
                scopes_.emplace_back();
                Val lv = do_load();
                scopes_.pop_back();
                uint32_t t_end = cur_;
                br(mb);
                cur_ = mb;
                return phi(vt, {{from, other}, {t_end, lv}});
            }
            case Node::Dot: fail("E307", n->line, "a tl.dot result can only be stored (optionally plus a loaded tile, optionally converted)");
            case Node::Reduce: fail("E307", n->line, "a reduction result can only be the value of tl.atomic_add / tl.atomic_max / tl.atomic_min on a scalar pointer");
        }
        fail("E304", n->line, "node outside the subset");
    }
    std::vector<Val> sub_idx(const NP& child, const std::vector<Val>& idx) {
        if (child->rank() == 0) return {};
        std::vector<Val> out = idx;
        for (size_t a = 0; a < child->rank() && a < out.size(); a++)
            if (child->shape[a].is_one()) out[a] = zero();
        return out;
    }
    Val zero() { return ci(I64(), 0); }

    bool has_dot(const NP& n, std::set<const Node*>* seen) const {
        if (!n || !seen->insert(n.get()).second) return false;
        if (n->k == Node::Dot) return true;
        for (auto& c : n->in) if (has_dot(c, seen)) return true;
        return false;
    }

    // ---- lane loops ----
    // One lane of an unrolled iteration: its tile indices and, for every lane but the first, the
    // predicate "this lane exists" (l + u * bdim.x < lanes), which guards its loads and its effects.
    struct Lane {
        std::vector<Val> idx;
        bool guarded = false;
        Val guard;
    };
    const Lane* lane_ = nullptr;   // the lane gen() is instantiating for, so that loads can honour its guard
    static constexpr int kUnroll = 4;

    // for (l = tid.x; l < lanes; l += kUnroll * bdim.x): lanes l, l + bdim.x, ... of one iteration are
    // instantiated together -- first `values` for every lane (its loads), then `effects` for every lane
    // -- so that a thread has kUnroll independent loads in flight and neighbouring threads still touch
    // neighbouring addresses.  `carried` values ride along as phis; `fold` combines a lane's values into them.
    void lane_loop(const std::vector<Dim>& shape, int line, const std::function<std::vector<Val>(const Lane&)>& values,
                   const std::function<void(const Lane&, const std::vector<Val>&)>& effects, std::vector<Val>* carried = nullptr,
                   const std::function<std::vector<Val>(const Lane&, const std::vector<Val>&, const std::vector<Val>&)>* fold = nullptr) {
        scopes_.emplace_back();
        Val lanes;
        if (shape.empty()) lanes = ci(I64(), 1);
        else if (shape.size() == 1) lanes = shape[0].sym >= 0 ? Val::P((uint32_t)shape[0].sym) : ci(I64(), shape[0].n);
        else {
            if (shape[0].sym >= 0 || shape[1].sym >= 0) fail("E306", line, "rank-2 tiles need compile-time extents");
            lanes = ci(I64(), shape[0].n * shape[1].n);
        }
        // a reduction has one load per lane, so it takes twice the lanes per iteration to keep as many bytes in flight
        const int unroll = shape.empty() ? 1 : (fold ? 2 * kUnroll : kUnroll);
        Val tid = index(0), stride = index(6);
        uint32_t pre = cur_, head = new_block(), bodyb = new_block(), done = new_block();
        br(head);
        cur_ = head;
        Inst ph;   // the second incoming value is patched in once the latch exists
        ph.op = Opc::Phi;
        ph.ty = I64();
        ph.ops = {tid};
        ph.phi_blocks = {pre};
        Val l = push(ph);
        std::vector<Val> acc;
        if (carried)
            for (Val init : *carried) {
                Inst pa;
                pa.op = Opc::Phi;
                pa.ty = f_.val_ty(init);
                pa.ops = {init};
                pa.phi_blocks = {pre};
                acc.push_back(push(pa));
            }
        condbr(icmp(ICmp::Slt, I64(), l, lanes), bodyb, done);
        cur_ = bodyb;
        scopes_.emplace_back();
        std::vector<Lane> ls((size_t)unroll);
        Val lu = l;
        for (int u = 0; u < unroll; u++) {
            if (u) {
                lu = bin(BinOp::Add, I64(), lu, stride);
                ls[u].guarded = true;
                ls[u].guard = icmp(ICmp::Slt, I64(), lu, lanes);
            }
            if (shape.size() == 1) ls[u].idx = {lu};
            else if (shape.size() == 2) {
                Val n1 = ci(I64(), shape[1].n);
                ls[u].idx = {bin(BinOp::Div, I64(), lu, n1), bin(BinOp::Rem, I64(), lu, n1)};
            }
        }
        std::vector<std::vector<Val>> vals((size_t)unroll);
        for (int u = 0; u < unroll; u++) { lane_ = &ls[u]; vals[u] = values(ls[u]); }
        std::vector<Val> cur_acc = acc;
        for (int u = 0; u < unroll; u++) {
            lane_ = &ls[u];
            if (fold) cur_acc = (*fold)(ls[u], vals[u], cur_acc);
            else effects(ls[u], vals[u]);
        }
        lane_ = nullptr;
        Val next = bin(BinOp::Add, I64(), lu, stride);
        uint32_t latch_end = cur_;
        br(head);
        f_.insts[l.idx].ops.push_back(next);
        f_.insts[l.idx].phi_blocks.push_back(latch_end);
        for (size_t k = 0; k < acc.size(); k++) {
            f_.insts[acc[k].idx].ops.push_back(cur_acc[k]);
            f_.insts[acc[k].idx].phi_blocks.push_back(latch_end);
        }
        scopes_.pop_back();
        scopes_.pop_back();
        cur_ = done;
        if (carried) *carried = acc;   // the values the loop leaves with: the head's phis
    }

    // the predicate under which a lane's side effect happens: its mask and its guard, whichever exist
    bool lane_condition(const Lane& lane, const NP& mask, Val* out) {
        bool have = false;
        if (mask) { *out = gen(mask, sub_idx(mask, lane.idx)); have = true; }
        if (lane.guarded) { *out = have ? bin(BinOp::And, Ty::s(Scalar::I1), *out, lane.guard) : lane.guard; have = true; }
        return have;
    }
    void under(bool have, Val cond, const std::function<void()>& emit) {
        if (!have) { emit(); return; }
        uint32_t tb = new_block(), after = new_block();
        condbr(cond, tb, after);
        cur_ = tb;
        scopes_.emplace_back();
        emit();
        scopes_.pop_back();
        br(after);
        cur_ = after;
    }

    void store(const NP& ptr, const NP& value, const NP& mask, int line) {
        std::vector<Dim> shape = broadcast(ptr, value, line);
        if (!(shape == ptr->shape)) fail("E305", line, "the stored value is larger than the pointer tile");
        std::set<const Node*> seen;
        if (has_dot(value, &seen)) { store_dot(ptr, value, mask, line); return; }
        El el = ptr->pointee;
        NP val = convert(value, el, line);
        if (mask && !(broadcast(ptr, mask, line) == ptr->shape)) fail("E305", line, "the mask is larger than the pointer tile");
        lane_loop(shape, line,
                  [&](const Lane& lane) { return std::vector<Val>{gen(val, sub_idx(val, lane.idx))}; },
                  [&](const Lane& lane, const std::vector<Val>& v) {
                      Val cond;
                      bool have = lane_condition(lane, mask, &cond);
                      under(have, cond, [&]() {
                          Inst st;
                          st.op = Opc::Store;
                          st.ty = Ty::v();
                          st.aux = Ty::s(scalar_of(el));
                          st.space = Space::Global;
                          st.align = scalar_bytes(scalar_of(el));
                          st.ops = {gen(ptr, sub_idx(ptr, lane.idx)), v[0]};
                          push(st);
                      });
                  });
    }

    // ---- atomics and CTA-wide reductions ----
    // tl.atomic_<op>(ptr, tile): one atomic per lane of the tile.  tl.atomic_<op>(scalar_ptr, tl.<red>(x)):
    // every thread folds the lanes it walks, a warp combines its 32 partial results (warp.reduce for
    // int32, an xor butterfly of shuffles for float32), lane 0 of every warp parks the warp's value in
    // shared memory, the first warp combines those after a barrier, and thread 0 issues the program's
    // one atomic.  The CTA must be whole warps, which Triton's num_warps guarantees.
    void atomic(const std::string& op, const NP& ptr, const NP& value, const NP& mask, int line) {
        AtomOp aop = op == "add" ? AtomOp::Add : op == "max" ? AtomOp::Max : AtomOp::Min;
        El el = ptr->pointee;
        if (el != El::I32 && el != El::F32 && el != El::I64) fail("E304", line, "atomics on int32, int64 and float32 only");
        if (value->k == Node::Reduce) {
            if (ptr->rank() != 0 || mask) fail("E307", line, "a reduction result goes to a scalar pointer, unmasked");
            if (value->op != (op == "add" ? "sum" : op)) fail("E307", line, "tl.atomic_" + op + " of tl." + value->op + " is not one reduction");
            if (value->el != el) fail("E300", line, "the reduced tile and the target have different element types");
            reduce_to_atomic(aop, ptr, value->in[0], line);
            return;
        }
        std::vector<Dim> shape = broadcast(ptr, value, line);
        if (!(shape == ptr->shape)) fail("E305", line, "the value is larger than the pointer tile");
        NP val = convert(value, el, line);
        lane_loop(shape, line,
                  [&](const Lane& lane) { return std::vector<Val>{gen(val, sub_idx(val, lane.idx))}; },
                  [&](const Lane& lane, const std::vector<Val>& v) {
                      Val cond;
                      bool have = lane_condition(lane, mask, &cond);
                      under(have, cond, [&]() {
                          Inst at;
                          at.op = Opc::Atomic;
                          at.sub = (uint8_t)aop;
                          at.ty = Ty::s(scalar_of(el));
                          at.space = Space::Global;
                          at.ops = {gen(ptr, sub_idx(ptr, lane.idx)), v[0]};
                          push(at);
                      });
                  });
    }

    Val combine(AtomOp op, El el, Val a, Val b) {
        Ty t = Ty::s(scalar_of(el));
        if (op == AtomOp::Add) return bin(is_flt(el) ? BinOp::FAdd : BinOp::Add, t, a, b);
        Val c = is_flt(el) ? fcmp(op == AtomOp::Max ? FCmp::Ogt : FCmp::Olt, t, a, b) : icmp(op == AtomOp::Max ? ICmp::Sgt : ICmp::Slt, t, a, b);
        return select(t, c, a, b);
    }

    // The per-thread fold of a reduction whose tile is `tl.load(p + pid * B + tl.arange(0, B), mask = offs < n)` over
    // int32: the program's lanes are B consecutive words, so a thread reads them as 16-byte vectors (four in flight,
    // lanes 4j .. 4j+3 for j = tid, tid + bdim, ...) instead of one masked word per lane -- integer max, min and
    // wrapping add do not depend on the order of the fold.  The number of lanes the mask lets through is computed
    // once per program (the mask is an upper bound on a unit-stride index, so they are a prefix); what is left
    // after the vectors, and everything when the program's first word is not 16-byte aligned, goes through a scalar
    // loop; the masked-off lanes contribute `other` (0 when absent, as in the lane-by-lane form) once.
    // Returns false, having emitted nothing, when the tile is not of that shape.
    bool fold_contiguous_i32(AtomOp op, const NP& x, Val identity, Val* acc_io) {
        if (x->k != Node::Load || x->rank() != 1 || x->el != El::I32) return false;
        const NP& p = x->in[0];
        Aff ap = affine(p);
        if (!ap.ok || ap.ci != 1 || !ap.ptr) return false;
        NP lhs, rhs;
        int64_t other = 0;
        if (x->has_mask) {
            const NP& m = x->in[1];
            if (m->k != Node::Cmp || m->op != "<" || m->in[0]->rank() != 1 || m->in[1]->rank() != 0 || m->in[0]->el != El::I64 || m->in[1]->el != El::I64) return false;
            Aff al = affine(m->in[0]);
            if (!al.ok || al.ci != 1) return false;
            lhs = m->in[0]; rhs = m->in[1];
            if (x->has_other && (x->in[2]->rank() != 0 || !ceval(x->in[2], &other))) return false;
            if (op == AtomOp::Add && other != 0) return false;   // a sum would need `other` once per masked-off lane
        }
        const Ty t = Ty::s(Scalar::I32), pg = Ty::p(Space::Global), v4 = Ty::vec(Scalar::I32, 4), i1 = Ty::s(Scalar::I1);
        scopes_.emplace_back();
        Val zero = ci(I64(), 0);
        Val lanes = x->shape[0].sym >= 0 ? Val::P((uint32_t)x->shape[0].sym) : ci(I64(), x->shape[0].n);
        Val p0 = gen(p, sub_idx(p, {zero}));
        Val cnt = lanes;
        if (x->has_mask) {
            Val rem = bin(BinOp::Sub, I64(), gen(rhs, {}), gen(lhs, sub_idx(lhs, {zero})));
            rem = select(I64(), icmp(ICmp::Slt, I64(), rem, zero), zero, rem);
            cnt = select(I64(), icmp(ICmp::Slt, I64(), rem, lanes), rem, lanes);
        }
        Val aligned = icmp(ICmp::Eq, I64(), bin(BinOp::And, I64(), cast(CastOp::Bitcast, I64(), pg, p0), ci(I64(), 15)), zero);
        Val nv = select(I64(), aligned, bin(BinOp::AShr, I64(), cnt, ci(I64(), 2)), zero);
        Val tid = index(0), stride = index(6);
        // ---- vectors: four per iteration, every load unconditional (a vector past the end re-reads the last one
        // and its fold is dropped), so that the four are in flight together
        uint32_t pre = cur_, vhead = new_block(), vbody = new_block(), vdone = new_block();
        br(vhead);
        cur_ = vhead;
        Inst pj; pj.op = Opc::Phi; pj.ty = I64(); pj.ops = {tid}; pj.phi_blocks = {pre};
        Val j = push(pj);
        Inst pa; pa.op = Opc::Phi; pa.ty = t; pa.ops = {*acc_io}; pa.phi_blocks = {pre};
        Val acc = push(pa);
        condbr(icmp(ICmp::Slt, I64(), j, nv), vbody, vdone);
        cur_ = vbody;
        Val last = bin(BinOp::Sub, I64(), nv, ci(I64(), 1));
        Val ju = j, cur = acc;
        std::vector<Val> vecs, guards;
        for (int u = 0; u < 4; u++) {
            if (u) ju = bin(BinOp::Add, I64(), ju, stride);
            Val g = u ? icmp(ICmp::Slt, I64(), ju, nv) : Val();
            Val jc = u ? select(I64(), g, ju, last) : ju;
            Inst ld; ld.op = Opc::Load; ld.ty = v4; ld.space = Space::Global; ld.align = 16;
            ld.ops = {bin(BinOp::Add, pg, p0, bin(BinOp::Mul, I64(), jc, ci(I64(), 16)))};
            vecs.push_back(push(ld));
            guards.push_back(g);
        }
        for (int u = 0; u < 4; u++) {
            Val e[4];
            for (unsigned l = 0; l < 4; l++) { Inst ex; ex.op = Opc::VecExtract; ex.ty = t; ex.sub = (uint8_t)l; ex.ops = {vecs[u]}; e[l] = push(ex); }
            Val m4 = combine(op, El::I32, combine(op, El::I32, e[0], e[1]), combine(op, El::I32, e[2], e[3]));
            Val folded = combine(op, El::I32, cur, m4);
            cur = u ? select(t, guards[u], folded, cur) : folded;
        }
        Val jnext = bin(BinOp::Add, I64(), ju, stride);
        uint32_t vend = cur_;
        br(vhead);
        f_.insts[j.idx].ops.push_back(jnext); f_.insts[j.idx].phi_blocks.push_back(vend);
        f_.insts[acc.idx].ops.push_back(cur); f_.insts[acc.idx].phi_blocks.push_back(vend);
        // ---- what the vectors left: lanes 4 nv .. cnt-1, one word per trip
        cur_ = vdone;
        Val l0 = bin(BinOp::Add, I64(), bin(BinOp::Shl, I64(), nv, ci(I64(), 2)), tid);
        uint32_t spre = cur_, shead = new_block(), sbody = new_block(), sdone = new_block();
        br(shead);
        cur_ = shead;
        Inst pl; pl.op = Opc::Phi; pl.ty = I64(); pl.ops = {l0}; pl.phi_blocks = {spre};
        Val l = push(pl);
        Inst ps2; ps2.op = Opc::Phi; ps2.ty = t; ps2.ops = {acc}; ps2.phi_blocks = {spre};
        Val sacc = push(ps2);
        condbr(icmp(ICmp::Slt, I64(), l, cnt), sbody, sdone);
        cur_ = sbody;
        Inst ld; ld.op = Opc::Load; ld.ty = t; ld.space = Space::Global; ld.align = 4;
        ld.ops = {bin(BinOp::Add, pg, p0, bin(BinOp::Mul, I64(), l, ci(I64(), 4)))};
        Val w = push(ld);
        Val snext_acc = combine(op, El::I32, sacc, w);
        Val lnext = bin(BinOp::Add, I64(), l, stride);
        uint32_t send = cur_;
        br(shead);
        f_.insts[l.idx].ops.push_back(lnext); f_.insts[l.idx].phi_blocks.push_back(send);
        f_.insts[sacc.idx].ops.push_back(snext_acc); f_.insts[sacc.idx].phi_blocks.push_back(send);
        cur_ = sdone;
        Val out = sacc;
        if (x->has_mask && op != AtomOp::Add) {   // max and min are idempotent: the masked-off lanes' value counts once
            Val some_off = icmp(ICmp::Slt, I64(), cnt, lanes);
            out = select(t, some_off, combine(op, El::I32, sacc, ci(t, other)), sacc);
        }
        (void)identity; (void)i1;
        scopes_.pop_back();
        *acc_io = out;
        return true;
    }

    void reduce_to_atomic(AtomOp op, const NP& ptr, const NP& x, int line) {
        El el = x->el;
        Ty t = Ty::s(scalar_of(el));
        scopes_.emplace_back();
        Val identity;
        if (op == AtomOp::Add) identity = is_flt(el) ? cf(t, 0.0) : ci(t, 0);
        else if (is_flt(el)) identity = cf(t, op == AtomOp::Max ? -INFINITY : INFINITY);
        else identity = ci(t, op == AtomOp::Max ? (int64_t)INT32_MIN : (int64_t)INT32_MAX);
        std::vector<Val> carried = {identity};
        std::function<std::vector<Val>(const Lane&, const std::vector<Val>&, const std::vector<Val>&)> fold =
            [&](const Lane& lane, const std::vector<Val>& v, const std::vector<Val>& acc) {
                Val folded = combine(op, el, v[0], acc[0]);
                if (lane.guarded) folded = select(t, lane.guard, folded, acc[0]);   // a lane past the tile contributes nothing
                return std::vector<Val>{folded};
            };
        if (!fold_contiguous_i32(op, x, identity, &carried[0]))
            lane_loop(x->shape, line, [&](const Lane& lane) { return std::vector<Val>{gen(x, sub_idx(x, lane.idx))}; }, nullptr, &carried, &fold);
        // warp step, then the warps of the CTA through shared memory, then one atomic per program
        auto warp_combine = [&](Val v) {
            if (el == El::I32) {
                Inst wr;
                wr.op = Opc::WarpReduce;
                wr.sub = (uint8_t)(op == AtomOp::Add ? RedOp::Add : op == AtomOp::Max ? RedOp::Max : RedOp::Min);
                wr.ty = t;
                wr.ops = {v};
                return push(wr);
            }
            for (int m = 16; m >= 1; m >>= 1) {
                Inst sh;
                sh.op = Opc::Shuffle;
                sh.sub = (uint8_t)Shfl::Xor;
                sh.ty = t;
                sh.ops = {v, ci(Ty::s(Scalar::I32), m)};
                Val other = push(sh);
                v = combine(op, el, other, v);
            }
            return v;
        };
        Val warp = warp_combine(carried[0]);
        SharedObj so;   // one word per warp of the CTA (at most 32)
        so.key = ((int64_t)m_->funcs.size() << 32) + 65536 * (int64_t)shared_cells_++;
        so.bytes = 128;
        so.align = 16;
        m_->shared_objs.push_back(so);
        const Ty ps = Ty::p(Space::Shared);
        Val tid = index(0), c31 = ci(I64(), 31), c5 = ci(I64(), 5), c4 = ci(I64(), 4), zero64 = ci(I64(), 0);
        Val lane = bin(BinOp::And, I64(), tid, c31), wid = bin(BinOp::LShr, I64(), tid, c5);
        under(true, icmp(ICmp::Eq, I64(), lane, zero64), [&]() {
            Inst st;
            st.op = Opc::Store;
            st.ty = Ty::v();
            st.aux = t;
            st.space = Space::Shared;
            st.align = 4;
            st.ops = {bin(BinOp::Add, ps, ci(ps, so.key), bin(BinOp::Mul, I64(), wid, c4)), warp};
            push(st);
        });
        Inst bar;
        bar.op = Opc::Barrier;
        bar.ty = Ty::v();
        push(bar);
        under(true, icmp(ICmp::Slt, I64(), tid, ci(I64(), 32)), [&]() {
            Val warps = bin(BinOp::LShr, I64(), bin(BinOp::Add, I64(), index(6), c31), c5);
            Val have = icmp(ICmp::Slt, I64(), tid, warps);
            uint32_t from = cur_, lb = new_block(), mb = new_block();
            condbr(have, lb, mb);
            cur_ = lb;
            Inst ld;
            ld.op = Opc::Load;
            ld.ty = t;
            ld.space = Space::Shared;
            ld.align = 4;
            ld.ops = {bin(BinOp::Add, ps, ci(ps, so.key), bin(BinOp::Mul, I64(), tid, c4))};
            Val part = push(ld);
            uint32_t l_end = cur_;
            br(mb);
            cur_ = mb;
            Val v = phi(t, {{from, identity}, {l_end, part}});
            Val all = warp_combine(v);
            under(true, icmp(ICmp::Eq, I64(), tid, zero64), [&]() {
                Inst at;
                at.op = Opc::Atomic;
                at.sub = (uint8_t)op;
                at.ty = t;
                at.space = Space::Global;
                at.ops = {gen(ptr, {}), all};
                push(at);
            });
        });
        scopes_.pop_back();
    }

    // ---- tl.dot -> mma ----
    // value = base + ci * i + cj * j (in elements) with constant ci, cj; c0 collects the constant
    // part of the base, `rest` the run-time scalar terms (compared by identity).
    struct Aff {
        bool ok = false;
        int64_t ci = 0, cj = 0, c0 = 0;
        std::map<const Node*, int64_t> rest;   // run-time scalar terms of the base, each with its constant coefficient
        const Node* ptr = nullptr;
        void add_rest(const std::map<const Node*, int64_t>& o, int64_t s) {
            for (auto& kv : o) { rest[kv.first] += s * kv.second; if (rest[kv.first] == 0) rest.erase(kv.first); }
        }
    };
    Aff affine(const NP& n) {
        Aff r;
        if (n->rank() == 0) {
            r.ok = true;
            int64_t c;
            if (ceval(n, &c)) r.c0 = c;
            else if (n->k == Node::PPtr) r.ptr = n.get();
            else if (n->k == Node::Bin && !n->is_ptr && (n->op == "+" || n->op == "-")) {
                Aff a = affine(n->in[0]), b = affine(n->in[1]);
                int64_t sg = n->op == "+" ? 1 : -1;
                r.c0 = a.c0 + sg * b.c0;
                r.rest = a.rest;
                r.add_rest(b.rest, sg);
            } else if (n->k == Node::Bin && n->is_ptr && n->op == "+") {
                Aff a = affine(n->in[0]), b = affine(n->in[1]);
                r = a;
                r.c0 += b.c0;
                r.add_rest(b.rest, 1);
            } else if (n->k == Node::Bin && !n->is_ptr && n->op == "*" && (ceval(n->in[0], &c) || ceval(n->in[1], &c))) {
                int64_t k = 0;
                Aff t = ceval(n->in[1], &k) ? affine(n->in[0]) : (ceval(n->in[0], &k), affine(n->in[1]));
                r.c0 = t.c0 * k;
                r.add_rest(t.rest, k);
            } else r.rest[n.get()] = 1;
            return r;
        }
        switch (n->k) {
            case Node::Arange: r.ok = true; r.ci = n->shape[0].is_one() ? 0 : 1; r.c0 = n->iv; return r;
            case Node::Expand: {
                Aff a = affine(n->in[0]);
                if (!a.ok) return r;
                r = a;
                if (n->iv == 1) { r.ci = a.ci; r.cj = 0; } else { r.cj = a.ci; r.ci = 0; }
                return r;
            }
            case Node::Bin: {
                Aff a = affine(n->in[0]), b = affine(n->in[1]);
                if (!a.ok || !b.ok) return r;
                if (n->op == "+" || n->op == "-") {
                    int64_t sg = n->op == "+" ? 1 : -1;
                    if (sg < 0 && b.ptr) return r;
                    r.ok = true;
                    r.ci = a.ci + sg * b.ci; r.cj = a.cj + sg * b.cj; r.c0 = a.c0 + sg * b.c0;
                    r.rest = a.rest;
                    r.add_rest(b.rest, sg);
                    r.ptr = a.ptr ? a.ptr : b.ptr;
                    return r;
                }
                if (n->op == "*") {
                    int64_t k;
                    const Aff* t = nullptr;
                    if (ceval(n->in[1], &k)) t = &a;
                    else if (ceval(n->in[0], &k)) t = &b;
                    else return r;   // a run-time scalar times a tile index: the stride is not a constant
                    if (t->ptr) return r;
                    r.ok = true;
                    r.ci = t->ci * k; r.cj = t->cj * k; r.c0 = t->c0 * k;
                    r.add_rest(t->rest, k);
                    return r;
                }
                return r;
            }
            default: return r;
        }
    }

    struct Slab { NP a_ptr, b_ptr; int64_t k; int line; };

    void store_dot(const NP& ptr, NP value, const NP& mask, int line) {
        if (mask) fail("E307", line, "a masked store of a tl.dot result is outside the subset (tile extents must divide the matrix)");
        El out_el = ptr->pointee;
        if (value->k == Node::Cast && is_flt(value->el)) value = value->in[0];
        NP dotv = value, addend;
        std::vector<Slab> slabs;   // the accumulator chain in program order (k ascending)
        if (!flatten_sum(value, &slabs)) {
            slabs.clear();
            bool ok = false;
            if (value->k == Node::Bin && value->op == "+" && value->el == El::F32) {
                for (int side = 0; side < 2 && !ok; side++) {
                    std::vector<Slab> tmp;
                    if (value->in[1 - side]->k == Node::Load && flatten_sum(value->in[side], &tmp) && !tmp.empty()) {
                        dotv = value->in[side];
                        addend = value->in[1 - side];
                        slabs = tmp;
                        ok = true;
                    }
                }
            }
            if (!ok) fail("E307", line, "the stored value must be tl.dot results accumulated from tl.zeros over unmasked tl.load tiles, optionally plus one loaded tile");
        }
        if (slabs.empty()) fail("E307", line, "no tl.dot found in the stored value");
        const int64_t M = dotv->shape[0].n, N = dotv->shape[1].n;
        Aff a0 = affine(slabs[0].a_ptr), b0 = affine(slabs[0].b_ptr), d0 = affine(ptr);
        if (!a0.ok || !b0.ok || !d0.ok || !a0.ptr || !b0.ptr || !d0.ptr) fail("E307", line, "tl.dot operand and result pointers must be tiles with constant strides");
        bool a_col, b_col;
        int64_t lda, ldb;
        if (a0.cj == 1) { a_col = false; lda = a0.ci; } else if (a0.ci == 1) { a_col = true; lda = a0.cj; } else fail("E307", line, "the A tile has no unit stride");
        if (b0.cj == 1) { b_col = false; ldb = b0.ci; } else if (b0.ci == 1) { b_col = true; ldb = b0.cj; } else fail("E307", line, "the B tile has no unit stride");
        if (d0.cj != 1) fail("E307", line, "the result tile must be row-major");
        const int64_t a_kstride = a_col ? lda : 1, b_kstride = b_col ? 1 : ldb;   // elements per step of k
        int64_t K = 0;
        for (size_t t = 0; t < slabs.size(); t++) {
            Aff at = affine(slabs[t].a_ptr), bt = affine(slabs[t].b_ptr);
            if (!at.ok || !bt.ok || at.ci != a0.ci || at.cj != a0.cj || bt.ci != b0.ci || bt.cj != b0.cj || at.rest != a0.rest || bt.rest != b0.rest || at.ptr != a0.ptr || bt.ptr != b0.ptr)
                fail("E307", slabs[t].line, "the K slabs of the tl.dot chain do not share one operand layout");
            if (at.c0 - a0.c0 != K * a_kstride || bt.c0 - b0.c0 != K * b_kstride) fail("E307", slabs[t].line, "the K slabs of the tl.dot chain are not consecutive");
            K += slabs[t].k;
        }
        El in_el = static_cast<const Node*>(a0.ptr)->pointee;
        if (static_cast<const Node*>(b0.ptr)->pointee != in_el) fail("E300", line, "tl.dot operands have different element types");
        Inst mm;
        mm.op = Opc::Mma;
        mm.ty = Ty::v();
        mm.in_dt = scalar_of(in_el);
        mm.acc_dt = Scalar::F32;
        mm.out_dt = scalar_of(out_el);
        mm.has_out = out_el != El::F32;
        if (out_el != El::F32 && out_el != El::F16) fail("E300", line, "a tl.dot result is stored as float32 or float16");
        mm.a_col = a_col;
        mm.b_col = b_col;
        mm.m = (uint32_t)M;
        mm.n = (uint32_t)N;
        mm.k = (uint32_t)K;
        mm.has_ld = true;
        mm.ld[0] = lda;
        mm.ld[1] = ldb;
        mm.ld[3] = d0.ci;
        scopes_.emplace_back();
        std::vector<Val> origin = {zero(), zero()};
        Val pa = gen(slabs[0].a_ptr, sub_idx(slabs[0].a_ptr, origin)), pb = gen(slabs[0].b_ptr, sub_idx(slabs[0].b_ptr, origin)), pd = gen(ptr, sub_idx(ptr, origin));
        Val pc;
        if (addend) {
            if (addend->k != Node::Load || addend->has_mask) fail("E307", line, "the tile added to a tl.dot result must be an unmasked tl.load");
            Aff c0 = affine(addend->in[0]);
            if (!c0.ok || !c0.ptr || c0.cj != 1) fail("E307", line, "the added tile must be row-major with a constant stride");
            if (addend->el != El::F32 && !(addend->el == out_el)) fail("E300", line, "the added tile must be float32");
            if (addend->in[0]->pointee != out_el) fail("E307", line, "the added tile and the result must have the same element type");
            mm.ld[2] = c0.ci;
            pc = gen(addend->in[0], sub_idx(addend->in[0], origin));
        } else {
            mm.ld[2] = d0.ci;
            pc = ci(Ty::p(Space::Global), 0);
        }
        mm.ops = {pa, pb, pc, pd};
        push(mm);
        scopes_.pop_back();
    }

    // Collects, in program order, the K slabs of an accumulation that starts from tl.zeros:
    // tl.dot(a, b, acc) chains and `acc + tl.dot(a, b)` sums (what `acc += tl.dot(a, b)` unrolls to).
    bool flatten_sum(const NP& n, std::vector<Slab>* out) {
        if (!n) return true;
        if (n->k == Node::Zeros && n->in.empty()) return true;
        if (n->k == Node::Dot) {
            const NP &a = n->in[0], &b = n->in[1];
            if (a->k != Node::Load || b->k != Node::Load || a->has_mask || b->has_mask) return false;
            if (!flatten_sum(n->in[2], out)) return false;
            out->push_back(Slab{a->in[0], b->in[0], a->shape[1].n, n->line});
            return true;
        }
        if (n->k == Node::Bin && n->op == "+" && n->el == El::F32) return flatten_sum(n->in[0], out) && flatten_sum(n->in[1], out);
        return false;
    }
};

}  // namespace

bool parse_triton_bindings(const char* text, TritonOptions* out, std::string* why) {
    if (!text) return true;
    std::istringstream ss(text);
    std::string item;
    while (ss >> item) {
        size_t eq = item.find('=');
        if (eq == std::string::npos || eq == 0 || eq + 1 >= item.size()) { if (why) *why = "expected name=value, found `" + item + "`"; return false; }
        std::string name = item.substr(0, eq), val = item.substr(eq + 1);
        if (val[0] == '*') {
            Scalar sc;
            std::string t = val.substr(1);
            if (t == "fp16") t = "f16";
            if (t == "fp32") t = "f32";
            if (t == "fp64") t = "f64";
            if (!parse_scalar(t, &sc)) { if (why) *why = "unknown element type `" + val + "`"; return false; }
            out->pointee[name] = sc;
        } else {
            char* endp = nullptr;
            long long v = strtoll(val.c_str(), &endp, 0);
            if (!endp || *endp) { if (why) *why = "`" + val + "` is not an integer"; return false; }
            out->constexprs[name] = v;
        }
    }
    return true;
}

bool compile_triton(const char* src, size_t len, const TritonOptions& opts, Module* out, Diag* d) {
    try {
        Parser p(tokenize(src, len));
        std::vector<Kernel> kernels = p.run();
        if (kernels.empty()) fail("E201", 1, "no @triton.jit function found");
        Module m;
        m.shared_mem_bytes = 0;
        auto nw = opts.constexprs.find("num_warps");
        if (nw != opts.constexprs.end()) {   // Triton's launch-time num_warps: the CTA size the kernel is compiled for
            if (nw->second < 1 || nw->second > 32) fail("E300", 1, "num_warps must be between 1 and 32");
            m.has_launch_bounds = true;
            m.max_threads = (uint32_t)(32 * nw->second);
            auto mb = opts.constexprs.find("min_blocks");
            m.min_blocks = mb == opts.constexprs.end() ? 1 : (uint32_t)mb->second;
        }
        // A @triton.jit function that another one calls is a helper: it is inlined at its calls and is no entry.
        std::set<std::string> helpers;
        for (size_t i = 0; i < kernels.size(); i++)
            for (size_t j = 0; j < i; j++) if (kernels[i].name == kernels[j].name) fail("E302", kernels[i].line, "`" + kernels[i].name + "` is defined twice");
        for (auto& k : kernels) {
            std::set<std::string> called;
            KernelCompiler::callees(k.body, kernels, &called);
            called.erase(k.name);      // a function that calls itself is refused where the call is met
            helpers.insert(called.begin(), called.end());
        }
        if (helpers.size() == kernels.size()) fail("E304", kernels[0].line, "every @triton.jit function is called by another one: no kernel is left");
        for (auto& k : kernels) {
            if (helpers.count(k.name)) continue;
            KernelCompiler kc(k, opts, &m, &kernels);
            Function f = kc.run();
            m.funcs.push_back(std::move(f));
        }
        std::string why;
        if (!verify_module(m, &why)) {
            if (d) { d->code = "E304"; d->arg = "internal: lowering produced an invalid module: " + why; }
            return false;
        }
        *out = std::move(m);
        return true;
    } catch (const Fail& f) {
        if (d) { d->code = f.code; d->arg = f.msg; }
        return false;
    }
}

}  // namespace basalt
