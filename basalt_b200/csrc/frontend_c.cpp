// CUDA-C subset -> slot-form BIR; see frontend_c.hpp.
//
// One pass: a recursive-descent parser that type-checks and emits BIR as it goes, so there is no
// AST.  The language accepted is what device kernels are written in: functions with
// __global__/__device__ qualifiers, scalar and pointer parameters, scalar locals, __shared__
// arrays with constant extents, if/for/while/do, the C expression operators with the usual
// arithmetic conversions, threadIdx/blockIdx/blockDim/gridDim, __syncthreads, warp shuffles and
// votes (with or without the _sync mask), atomics, min/max, object- and function-like #define, #if/#ifdef groups.  Anything else is
// refused with E304 rather than guessed at.
//
// Differences from the reference's lowering (crates/basalt-sema/src/lower.rs), each deliberate:
//   * a comparison yields an i1 that is widened to int only where arithmetic needs it (C++ bool),
//     so `if (i < n)` branches on the icmp itself; the reference widens and re-compares
//     (lower.rs:1894-1910);
//   * a __shared__ array records its byte size in a `shared_obj` module line, so the backend can
//     allocate it (the reference's 8-byte cells cannot hold an array, crates/basalt-ptx/src/emit.rs:630-660);
//   * atomics take their address space and value type from the pointer operand; the reference
//     hard-wires `i32` and `global` (lower.rs:2613-2640), which makes shared-memory atomics
//     inexpressible;
//   * `__launch_bounds__(t[, b])` on a kernel becomes the module's launch_bounds line;
//   * intrinsics give source access to BIR's tile op: `__basalt_mma_f32(m,n,k,a,b,c,d[,lda,ldb,ldc,ldd])`,
//     `__basalt_mma_f16(...)` (f16 operands, f32 accumulate, f16 result) and `__basalt_mma_f16_nt(...)`
//     (the same with B stored transposed, [n x k]).
#include "frontend_c.hpp"

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace basalt {
namespace {

struct Fail {
    std::string code, msg;
};

enum class Tk : uint8_t { Ident, Int, Float, Punct, Str, Eof };
struct Token {
    Tk k = Tk::Eof;
    std::string s;
    uint64_t u = 0;
    double f = 0;
    bool uns = false, lng = false, f32 = false, hex = false;
    int line = 0;
};

[[noreturn]] void fail(const char* code, int line, const std::string& msg) { throw Fail{code, "line " + std::to_string(line) + ": " + msg}; }

// ---------------------------------------------------------------------------------------------
// Lexer with object-like macros.
// ---------------------------------------------------------------------------------------------
class Lexer {
public:
    Lexer(const char* s, size_t n) : p_(s), end_(s + n) {}
    std::vector<Token> run() {
        std::vector<Token> out;
        bool line_start = true;
        for (;;) {
            skip_space(&line_start);
            if (p_ >= end_) break;
            if (*p_ == '#' && line_start) { directive(); continue; }
            line_start = false;
            if (!active()) {   // inside a conditional group that is not taken: the text is skipped, line by line
                while (p_ < end_ && *p_ != '\n') p_++;
                continue;
            }
            Token t = next();
            if (t.k == Tk::Ident) expand_into(t, &out, 0);
            else out.push_back(t);
        }
        if (!conds_.empty()) fail("E202", line_, "unterminated #if");
        Token e;
        e.k = Tk::Eof;
        e.line = line_;
        out.push_back(e);
        return out;
    }

private:
    const char *p_, *end_;
    int line_ = 1;
    struct FnMacro {
        std::vector<std::string> params;
        std::vector<Token> body;
    };
    std::map<std::string, std::vector<Token>> macros_;
    std::map<std::string, FnMacro> fn_macros_;
    // #if / #ifdef / #ifndef nesting: whether the group is being taken, whether one of its branches has been
    struct Cond { bool taking, taken, parent_active; };
    std::vector<Cond> conds_;
    bool active() const { return conds_.empty() || conds_.back().taking; }
    bool defined(const std::string& n) const { return macros_.count(n) || fn_macros_.count(n); }
    // the controlling expression of #if / #elif: an integer literal, NAME (its value if it is a literal macro),
    // defined(NAME) / defined NAME, with a leading `!`
    bool condition(std::string e, int line) {
        size_t i = 0;
        auto space = [&]() { while (i < e.size() && isspace((unsigned char)e[i])) i++; };
        auto word = [&]() { size_t b = i; while (i < e.size() && (isalnum((unsigned char)e[i]) || e[i] == '_')) i++; return e.substr(b, i - b); };
        bool neg = false;
        for (space(); i < e.size() && e[i] == '!'; space()) { neg = !neg; i++; }
        bool v = false;
        if (i < e.size() && isdigit((unsigned char)e[i])) {
            char* endp = nullptr;
            v = strtoll(e.c_str() + i, &endp, 0) != 0;
            i = (size_t)(endp - e.c_str());
            while (i < e.size() && strchr("uUlL", e[i])) i++;
        } else if (i < e.size() && (isalpha((unsigned char)e[i]) || e[i] == '_')) {
            std::string w = word();
            if (w == "defined") {
                space();
                const bool paren = i < e.size() && e[i] == '(';
                if (paren) { i++; space(); }
                std::string n = word();
                if (n.empty()) fail("E201", line, "defined needs a name");
                if (paren) { space(); if (i >= e.size() || e[i] != ')') fail("E201", line, "`)` expected after defined(" + n); i++; }
                v = defined(n);
            } else {
                auto it = macros_.find(w);   // an undefined name counts as 0
                v = it != macros_.end() && it->second.size() == 1 && it->second[0].k == Tk::Int && it->second[0].u != 0;
            }
        } else fail("E304", line, "this #if expression is outside the subset (a literal, a name or defined(NAME), with `!`)");
        space();
        if (i < e.size()) fail("E304", line, "this #if expression is outside the subset (a literal, a name or defined(NAME), with `!`)");
        return neg ? !v : v;
    }

    // Appends what the identifier `t` stands for: itself, the tokens of an object-like macro, or, when it names
    // a function-like macro and a `(` follows, the macro's body with each parameter replaced by the tokens of
    // its argument (arguments are expanded as they are read; a name not followed by `(` stays a name, as in C).
    void expand_into(const Token& t, std::vector<Token>* out, int depth) {
        auto obj = macros_.find(t.s);
        if (obj != macros_.end()) {
            for (Token m : obj->second) { m.line = t.line; out->push_back(m); }
            return;
        }
        auto fn = fn_macros_.find(t.s);
        if (fn == fn_macros_.end()) { out->push_back(t); return; }
        bool line_start = false;
        skip_space(&line_start);
        if (p_ >= end_ || *p_ != '(') { out->push_back(t); return; }
        if (depth > 32) fail("E304", t.line, "macro calls nest too deeply");
        p_++;
        std::vector<std::vector<Token>> args(1);
        for (int parens = 0;;) {
            skip_space(&line_start);
            if (p_ >= end_) fail("E202", t.line, "unterminated call of macro `" + t.s + "`");
            Token a = next();
            if (a.k == Tk::Punct && a.s == "(") parens++;
            else if (a.k == Tk::Punct && a.s == ")") { if (parens == 0) break; parens--; }
            else if (a.k == Tk::Punct && a.s == "," && parens == 0) { args.emplace_back(); continue; }
            if (a.k == Tk::Ident) expand_into(a, &args.back(), depth + 1);
            else args.back().push_back(a);
        }
        const FnMacro& m = fn->second;
        if (m.params.empty() && args.size() == 1 && args[0].empty()) args.clear();
        if (args.size() != m.params.size())
            fail("E300", t.line, "macro `" + t.s + "` takes " + std::to_string(m.params.size()) + " argument(s), " + std::to_string(args.size()) + " given");
        for (const Token& b : m.body) {
            size_t which = m.params.size();
            if (b.k == Tk::Ident) for (size_t i = 0; i < m.params.size(); i++) if (m.params[i] == b.s) which = i;
            if (which == m.params.size()) { Token c = b; c.line = t.line; out->push_back(c); }
            else for (Token c : args[which]) { c.line = t.line; out->push_back(c); }
        }
    }

    void skip_space(bool* line_start) {
        while (p_ < end_) {
            if (*p_ == '\n') { line_++; p_++; *line_start = true; }
            else if (*p_ == ' ' || *p_ == '\t' || *p_ == '\r' || *p_ == '\f' || *p_ == '\v') p_++;
            else if (*p_ == '\\' && p_ + 1 < end_ && p_[1] == '\n') { p_ += 2; line_++; }
            else if (*p_ == '/' && p_ + 1 < end_ && p_[1] == '/') { while (p_ < end_ && *p_ != '\n') p_++; }
            else if (*p_ == '/' && p_ + 1 < end_ && p_[1] == '*') {
                int start = line_;
                p_ += 2;
                for (;;) {
                    if (p_ + 1 >= end_) fail("E202", start, "unterminated comment");
                    if (*p_ == '*' && p_[1] == '/') { p_ += 2; break; }
                    if (*p_ == '\n') line_++;
                    p_++;
                }
            } else break;
        }
    }

    void directive() {
        int line = line_;
        p_++;
        std::string text;
        while (p_ < end_ && *p_ != '\n') {
            if (*p_ == '\\' && p_ + 1 < end_ && p_[1] == '\n') { p_ += 2; line_++; text += ' '; continue; }
            text += *p_++;
        }
        size_t i = 0;
        while (i < text.size() && isspace((unsigned char)text[i])) i++;
        size_t j = i;
        while (j < text.size() && isalpha((unsigned char)text[j])) j++;
        std::string name = text.substr(i, j - i);
        const std::string rest = text.substr(j);
        if (name == "ifdef" || name == "ifndef" || name == "if") {
            const bool parent = active();
            bool take = false;
            if (parent) {
                if (name == "if") take = condition(rest, line);
                else {
                    std::string n = rest;
                    while (!n.empty() && isspace((unsigned char)n.front())) n.erase(n.begin());
                    while (!n.empty() && isspace((unsigned char)n.back())) n.pop_back();
                    if (n.empty()) fail("E201", line, "#" + name + " needs a name");
                    take = defined(n) == (name == "ifdef");
                }
            }
            conds_.push_back({take, take, parent});
            return;
        }
        if (name == "elif" || name == "else" || name == "endif") {
            if (conds_.empty()) fail("E201", line, "#" + name + " without #if");
            Cond& c = conds_.back();
            if (name == "endif") { conds_.pop_back(); return; }
            const bool take = c.parent_active && !c.taken && (name == "else" || condition(rest, line));
            c.taking = take;
            c.taken = c.taken || take;
            return;
        }
        if (!active()) return;
        if (name == "include" || name == "pragma" || name.empty()) return;
        if (name == "undef") {
            std::string n = rest;
            while (!n.empty() && isspace((unsigned char)n.front())) n.erase(n.begin());
            while (!n.empty() && isspace((unsigned char)n.back())) n.pop_back();
            macros_.erase(n);
            fn_macros_.erase(n);
            return;
        }
        if (name == "error") fail("E304", line, "#error" + rest);
        if (name != "define") fail("E304", line, "preprocessor directive `#" + name + "` is outside the subset");
        while (j < text.size() && isspace((unsigned char)text[j])) j++;
        size_t k = j;
        while (k < text.size() && (isalnum((unsigned char)text[k]) || text[k] == '_')) k++;
        std::string macro = text.substr(j, k - j);
        if (macro.empty()) fail("E201", line, "#define without a name");
        FnMacro fm;
        const bool function_like = k < text.size() && text[k] == '(';
        if (function_like) {   // the parameter list follows the name with no space in between
            size_t q = k + 1;
            for (;;) {
                while (q < text.size() && isspace((unsigned char)text[q])) q++;
                if (q < text.size() && text[q] == ')') { q++; break; }
                size_t r = q;
                while (r < text.size() && (isalnum((unsigned char)text[r]) || text[r] == '_')) r++;
                if (r == q) fail(text.compare(q, 3, "...") == 0 ? "E304" : "E201", line, "#define " + macro + ": a parameter list of plain names is expected");
                fm.params.push_back(text.substr(q, r - q));
                q = r;
                while (q < text.size() && isspace((unsigned char)text[q])) q++;
                if (q < text.size() && text[q] == ',') { q++; continue; }
                if (q < text.size() && text[q] == ')') { q++; break; }
                fail("E201", line, "#define " + macro + ": `,` or `)` expected in the parameter list");
            }
            k = q;
        }
        std::string body = text.substr(k);
        Lexer sub(body.data(), body.size());
        sub.macros_ = macros_;
        sub.fn_macros_ = fn_macros_;
        for (auto& prm : fm.params) { sub.macros_.erase(prm); sub.fn_macros_.erase(prm); }   // a parameter hides a macro of its name
        sub.line_ = line;
        std::vector<Token> toks = sub.run();
        toks.pop_back();
        if (function_like) { fm.body = toks; fn_macros_[macro] = fm; macros_.erase(macro); }
        else { macros_[macro] = toks; fn_macros_.erase(macro); }
    }

    Token next() {
        Token t;
        t.line = line_;
        char c = *p_;
        if (isalpha((unsigned char)c) || c == '_') {
            const char* s = p_;
            while (p_ < end_ && (isalnum((unsigned char)*p_) || *p_ == '_')) p_++;
            t.k = Tk::Ident;
            t.s.assign(s, p_);
            return t;
        }
        if (isdigit((unsigned char)c) || (c == '.' && p_ + 1 < end_ && isdigit((unsigned char)p_[1]))) return number();
        if (c == '"') {
            const char* s = ++p_;
            while (p_ < end_ && *p_ != '"' && *p_ != '\n') p_++;
            if (p_ >= end_ || *p_ != '"') fail("E202", line_, "unterminated string literal");
            t.k = Tk::Str;
            t.s.assign(s, p_);
            p_++;
            return t;
        }
        static const char* const kPunct[] = {"<<=", ">>=", "...", "++", "--", "->", "<<", ">>", "<=", ">=", "==", "!=", "&&", "||", "+=", "-=",
                                             "*=",  "/=",  "%=",  "&=", "|=", "^=", "::"};
        for (const char* q : kPunct) {
            size_t n = strlen(q);
            if ((size_t)(end_ - p_) >= n && !strncmp(p_, q, n)) {
                t.k = Tk::Punct;
                t.s = q;
                p_ += n;
                return t;
            }
        }
        if (strchr("+-*/%&|^~!<>=?:;,.()[]{}", c)) {
            t.k = Tk::Punct;
            t.s = std::string(1, c);
            p_++;
            return t;
        }
        fail("E200", line_, std::string("unexpected character `") + c + "`");
    }

    Token number() {
        Token t;
        t.line = line_;
        const char* s = p_;
        bool is_float = false;
        if (*p_ == '0' && p_ + 1 < end_ && (p_[1] == 'x' || p_[1] == 'X')) {
            p_ += 2;
            t.hex = true;
            while (p_ < end_ && isxdigit((unsigned char)*p_)) p_++;
        } else {
            while (p_ < end_ && isdigit((unsigned char)*p_)) p_++;
            if (p_ < end_ && *p_ == '.') { is_float = true; p_++; while (p_ < end_ && isdigit((unsigned char)*p_)) p_++; }
            if (p_ < end_ && (*p_ == 'e' || *p_ == 'E')) {
                const char* q = p_ + 1;
                if (q < end_ && (*q == '+' || *q == '-')) q++;
                if (q < end_ && isdigit((unsigned char)*q)) { is_float = true; p_ = q; while (p_ < end_ && isdigit((unsigned char)*p_)) p_++; }
            }
        }
        std::string body(s, p_);
        if (is_float || (!t.hex && p_ < end_ && (*p_ == 'f' || *p_ == 'F'))) {
            t.k = Tk::Float;
            t.f = strtod(body.c_str(), nullptr);
            if (p_ < end_ && (*p_ == 'f' || *p_ == 'F')) { t.f32 = true; p_++; }
            else if (p_ < end_ && (*p_ == 'l' || *p_ == 'L')) p_++;
        } else {
            t.k = Tk::Int;
            t.u = strtoull(body.c_str(), nullptr, 0);
            while (p_ < end_ && strchr("uUlL", *p_)) {
                if (*p_ == 'u' || *p_ == 'U') t.uns = true; else t.lng = true;
                p_++;
            }
        }
        if (p_ < end_ && (isalnum((unsigned char)*p_) || *p_ == '_')) fail("E200", line_, "malformed number `" + std::string(s, p_ + 1) + "`");
        return t;
    }
};

// ---------------------------------------------------------------------------------------------
// Types and values.
// ---------------------------------------------------------------------------------------------
enum class B : uint8_t { Void, Bool, Char, UChar, Short, UShort, Int, UInt, Long, ULong, Half, Float, Double };

struct CT {
    B b = B::Int;
    int ptr = 0;               // pointer depth: 0 or 1
    bool cnst = false;         // scalar: the object is const; pointer: the pointee is const
    Space psp = Space::Global; // pointer: the space it points into
    std::vector<int> dims;     // array extents, outermost first
    bool is_ptr() const { return ptr > 0 && dims.empty(); }
    bool is_arr() const { return !dims.empty(); }
    bool is_scalar() const { return ptr == 0 && dims.empty(); }
};

bool is_int(B b) { return b >= B::Bool && b <= B::ULong; }
bool is_flt(B b) { return b >= B::Half; }
bool is_signed(B b) { return b == B::Char || b == B::Short || b == B::Int || b == B::Long; }
unsigned size_of(B b) {
    switch (b) {
        case B::Void: return 1;
        case B::Bool: case B::Char: case B::UChar: return 1;
        case B::Short: case B::UShort: case B::Half: return 2;
        case B::Int: case B::UInt: case B::Float: return 4;
        default: return 8;
    }
}
Scalar scalar_of(B b) {
    switch (b) {
        case B::Bool: return Scalar::I1;
        case B::Char: case B::UChar: return Scalar::I8;
        case B::Short: case B::UShort: return Scalar::I16;
        case B::Int: case B::UInt: return Scalar::I32;
        case B::Long: case B::ULong: return Scalar::I64;
        case B::Half: return Scalar::F16;
        case B::Float: return Scalar::F32;
        case B::Double: return Scalar::F64;
        default: return Scalar::I32;
    }
}
CT scalar_ct(B b) { CT t; t.b = b; return t; }
const char* base_name(B b) {
    static const char* const n[] = {"void", "bool", "char", "unsigned char", "short", "unsigned short", "int", "unsigned", "long", "unsigned long", "__half", "float", "double"};
    return n[(int)b];
}

// An expression result: an lvalue (address of a cell in `sp`) or an rvalue.
struct Ex {
    bool lv = false;
    Val v;
    CT ty;
    Space sp = Space::Local;
    bool is_void = false;
};

struct Local {
    int64_t key;   // slot address constant
    CT ty;
    Space sp;
};

struct FuncSig {
    CT ret;
    bool ret_void = false;
    std::vector<CT> params;
    bool is_kernel = false, defined = false;
};

struct DeclSpec {
    CT base;
    bool base_void = false;
    bool q_global = false, q_device = false, q_host = false, q_shared = false, q_constant = false;
    bool has_lb = false;
    uint32_t lb_threads = 0, lb_blocks = 0;
    int line = 0;
};

// ---------------------------------------------------------------------------------------------
// Parser + lowering.
// ---------------------------------------------------------------------------------------------
class Compiler {
public:
    Compiler(std::vector<Token> toks, Module* m) : t_(std::move(toks)), m_(m) {}

    void run() {
        m_->shared_mem_bytes = 0;
        while (!at_eof()) top_level();
        bool any_kernel = false;
        for (auto& f : m_->funcs) any_kernel |= f.is_kernel;
        (void)any_kernel;
    }

private:
    std::vector<Token> t_;
    size_t i_ = 0;
    Module* m_;
    std::map<std::string, FuncSig> sigs_;

    // per-function state
    Function* f_ = nullptr;
    FuncSig* sig_ = nullptr;
    uint32_t cur_ = 0;
    std::vector<bool> closed_;
    std::vector<std::map<std::string, Local>> scopes_;
    int64_t next_slot_ = 0;
    struct Loop { uint32_t brk, cont; };
    std::vector<Loop> loops_;

    // ---- token helpers ----
    const Token& tok() const { return t_[i_]; }
    const Token& peek(size_t n = 1) const { return t_[std::min(i_ + n, t_.size() - 1)]; }
    bool at_eof() const { return tok().k == Tk::Eof; }
    bool is_p(const char* s) const { return tok().k == Tk::Punct && tok().s == s; }
    bool is_id(const char* s) const { return tok().k == Tk::Ident && tok().s == s; }
    bool eat_p(const char* s) { if (is_p(s)) { i_++; return true; } return false; }
    bool eat_id(const char* s) { if (is_id(s)) { i_++; return true; } return false; }
    void need_p(const char* s) {
        if (!eat_p(s)) fail("E201", tok().line, std::string("expected `") + s + "`, found `" + show(tok()) + "`");
    }
    static std::string show(const Token& t) {
        if (t.k == Tk::Eof) return "end of file";
        if (t.k == Tk::Int) return std::to_string(t.u);
        if (t.k == Tk::Float) return std::to_string(t.f);
        return t.s;
    }
    std::string need_ident() {
        if (tok().k != Tk::Ident) fail("E201", tok().line, "expected an identifier, found `" + show(tok()) + "`");
        return t_[i_++].s;
    }

    // ---- emission helpers ----
    uint32_t new_block() {
        f_->blocks.emplace_back();
        closed_.push_back(false);
        return (uint32_t)f_->blocks.size() - 1;
    }
    void at(uint32_t b) { cur_ = b; }
    void open_if_closed() { if (closed_[cur_]) cur_ = new_block(); }   // code after return/break: a dead block
    Val push(const Inst& in) {
        open_if_closed();
        uint32_t id = (uint32_t)f_->insts.size();
        f_->insts.push_back(in);
        f_->blocks[cur_].insts.push_back(id);
        return Val::V(id);
    }
    void br(uint32_t to) {
        if (closed_[cur_]) return;
        Term& t = f_->blocks[cur_].term;
        t.kind = Term::Br;
        t.t = to;
        closed_[cur_] = true;
    }
    void condbr(Val c, uint32_t tb, uint32_t fb) {
        open_if_closed();
        Term& t = f_->blocks[cur_].term;
        t.kind = Term::CondBr;
        t.has_val = true;
        t.val = c;
        t.t = tb;
        t.f = fb;
        closed_[cur_] = true;
    }
    void ret(bool has, Val v) {
        open_if_closed();
        Term& t = f_->blocks[cur_].term;
        t.kind = Term::Ret;
        t.has_val = has;
        t.val = v;
        closed_[cur_] = true;
    }
    Val ci(Ty ty, int64_t v) {
        Inst in;
        in.op = Opc::ConstI;
        in.ty = ty;
        if (ty.is_sc(Scalar::I32)) v = (int64_t)(int32_t)(uint32_t)v;
        if (ty.is_sc(Scalar::I16)) v = (int64_t)(int16_t)(uint16_t)v;
        if (ty.is_sc(Scalar::I8)) v = (int64_t)(int8_t)(uint8_t)v;
        if (ty.is_sc(Scalar::I1)) v &= 1;
        in.imm = v;
        return push(in);
    }
    Val cf(Ty ty, double v) {
        Inst in;
        in.op = Opc::ConstF;
        in.ty = ty;
        in.fimm = v;
        return push(in);
    }
    Val bin(BinOp op, Ty ty, Val a, Val b) {
        Inst in;
        in.op = Opc::Bin;
        in.sub = (uint8_t)op;
        in.ty = ty;
        in.ops = {a, b};
        return push(in);
    }
    Val cast(CastOp op, Ty to, Ty from, Val v) {
        Inst in;
        in.op = Opc::Cast;
        in.sub = (uint8_t)op;
        in.ty = to;
        in.aux = from;
        in.ops = {v};
        return push(in);
    }
    Val icmp(ICmp p, Ty operand, Val a, Val b) {
        Inst in;
        in.op = Opc::ICmp;
        in.sub = (uint8_t)p;
        in.ty = Ty::s(Scalar::I1);
        in.aux = operand;
        in.ops = {a, b};
        return push(in);
    }
    Val fcmp(FCmp p, Ty operand, Val a, Val b) {
        Inst in;
        in.op = Opc::FCmp;
        in.sub = (uint8_t)p;
        in.ty = Ty::s(Scalar::I1);
        in.aux = operand;
        in.ops = {a, b};
        return push(in);
    }
    Val select(Ty ty, Val c, Val a, Val b) {
        Inst in;
        in.op = Opc::Select;
        in.ty = ty;
        in.ops = {c, a, b};
        return push(in);
    }
    Val load(Ty ty, Space sp, Val addr, bool vol = false) {
        Inst in;
        in.op = Opc::Load;
        in.ty = ty;
        in.space = sp;
        in.align = ty.is_ptr() ? 8 : scalar_bytes(ty.sc);
        in.vol = vol;
        in.ops = {addr};
        return push(in);
    }
    void store(Ty ty, Space sp, Val addr, Val v) {
        Inst in;
        in.op = Opc::Store;
        in.ty = Ty::v();
        in.aux = ty;
        in.space = sp;
        in.align = ty.is_ptr() ? 8 : scalar_bytes(ty.sc);
        in.ops = {addr, v};
        push(in);
    }
    Val phi(Ty ty, std::vector<std::pair<uint32_t, Val>> arms) {
        Inst in;
        in.op = Opc::Phi;
        in.ty = ty;
        for (auto& a : arms) { in.phi_blocks.push_back(a.first); in.ops.push_back(a.second); }
        return push(in);
    }

    // ---- types ----
    static Ty vty(const CT& t, Space arr_space = Space::Local) {
        if (t.is_arr()) return Ty::p(arr_space);
        if (t.ptr) return Ty::p(t.psp);
        return Ty::s(scalar_of(t.b));
    }
    static int64_t elem_bytes(const CT& t) {   // size of what a pointer/array element step covers
        if (t.is_arr()) {
            int64_t n = t.ptr ? 8 : size_of(t.b);
            for (size_t i = 1; i < t.dims.size(); i++) n *= t.dims[i];
            return n;
        }
        return size_of(t.b);
    }
    static int64_t total_bytes(const CT& t) {
        int64_t n = t.ptr ? 8 : size_of(t.b);
        for (int d : t.dims) n *= d;
        return n;
    }
    static std::string show(const CT& t) {
        std::string s = (t.cnst ? std::string("const ") : std::string()) + base_name(t.b);
        for (int i = 0; i < t.ptr; i++) s += "*";
        for (int d : t.dims) s += "[" + std::to_string(d) + "]";
        return s;
    }

    bool type_start(const Token& t) const {
        if (t.k != Tk::Ident) return false;
        static const char* const kw[] = {"const", "volatile", "static", "inline", "__forceinline__", "__inline__", "__noinline__", "extern", "__global__", "__device__",
                                         "__host__", "__shared__", "__constant__", "__launch_bounds__", "unsigned", "signed", "int", "long", "short", "char",
                                         "float", "double", "void", "bool", "size_t", "int32_t", "uint32_t", "int64_t", "uint64_t", "int8_t", "uint8_t", "int16_t", "uint16_t",
                                         "__half", "half", "__restrict__"};
        for (const char* k : kw) if (t.s == k) return true;
        return false;
    }

    DeclSpec decl_spec() {
        DeclSpec d;
        d.line = tok().line;
        bool uns = false, sgn = false, have = false, is_const = false;
        int longs = 0;
        B b = B::Int;
        for (;;) {
            if (tok().k != Tk::Ident) break;
            const std::string& s = tok().s;
            if (s == "const") is_const = true;
            else if (s == "volatile" || s == "static" || s == "inline" || s == "__forceinline__" || s == "__inline__" || s == "__noinline__" || s == "__restrict__") {}
            else if (s == "extern") {
                if (peek().k == Tk::Str) i_++;   // extern "C"
            }
            else if (s == "__global__") d.q_global = true;
            else if (s == "__device__") d.q_device = true;
            else if (s == "__host__") d.q_host = true;
            else if (s == "__shared__") d.q_shared = true;
            else if (s == "__constant__") d.q_constant = true;
            else if (s == "__launch_bounds__") {
                i_++;
                need_p("(");
                d.has_lb = true;
                d.lb_threads = (uint32_t)const_int();
                if (eat_p(",")) d.lb_blocks = (uint32_t)const_int();
                if (eat_p(",")) (void)const_int();
                if (!is_p(")")) fail("E201", tok().line, "expected `)` after __launch_bounds__ arguments");
            }
            else if (s == "unsigned") { uns = true; have = true; }
            else if (s == "signed") { sgn = true; have = true; }
            else if (s == "int") { have = true; }
            else if (s == "long") { longs++; have = true; }
            else if (s == "short") { b = B::Short; have = true; }
            else if (s == "char") { b = B::Char; have = true; }
            else if (s == "float") { b = B::Float; have = true; }
            else if (s == "double") { b = B::Double; have = true; }
            else if (s == "void") { b = B::Void; have = true; }
            else if (s == "bool") { b = B::Bool; have = true; }
            else if (s == "size_t" || s == "uint64_t") { b = B::ULong; have = true; }
            else if (s == "int64_t") { b = B::Long; have = true; }
            else if (s == "int32_t") { b = B::Int; have = true; }
            else if (s == "uint32_t") { b = B::UInt; have = true; }
            else if (s == "int16_t") { b = B::Short; have = true; }
            else if (s == "uint16_t") { b = B::UShort; have = true; }
            else if (s == "int8_t") { b = B::Char; have = true; }
            else if (s == "uint8_t") { b = B::UChar; have = true; }
            else if (s == "__half" || s == "half") { b = B::Half; have = true; }
            else break;
            i_++;
        }
        if (!have) fail("E201", d.line, "expected a type, found `" + show(tok()) + "`");
        if (longs) b = B::Long;
        if (uns) {
            if (b == B::Int) b = B::UInt; else if (b == B::Long) b = B::ULong; else if (b == B::Short) b = B::UShort; else if (b == B::Char) b = B::UChar;
            else fail("E300", d.line, std::string("`unsigned ") + base_name(b) + "` is not a type");
        }
        (void)sgn;
        if ((int)d.q_global + (int)(d.q_device || d.q_host) > 1 && d.q_global)
            fail("E303", d.line, "__global__ cannot be combined with __device__ or __host__");
        d.base.b = b;
        d.base.cnst = is_const;
        d.base_void = b == B::Void;
        return d;
    }

    // `*`s, qualifiers, name, array extents.  `name` may be empty for an abstract declarator.
    CT declarator(const DeclSpec& d, std::string* name, bool allow_abstract) {
        CT t = d.base;
        while (eat_p("*")) {
            t.ptr++;
            for (;;) {
                if (eat_id("const") || eat_id("__restrict__") || eat_id("restrict") || eat_id("volatile")) continue;
                break;
            }
        }
        if (t.ptr > 1) fail("E304", tok().line, "pointers to pointers are outside the subset");
        if (t.ptr == 0 && eat_p("&")) fail("E304", tok().line, "references are outside the subset");
        if (tok().k == Tk::Ident && !type_start(tok())) *name = t_[i_++].s;
        else if (!allow_abstract) fail("E201", tok().line, "expected a name, found `" + show(tok()) + "`");
        while (eat_p("[")) {
            if (is_p("]")) fail("E304", tok().line, "arrays need a constant extent");
            int64_t n = const_int();
            if (n <= 0 || n > (1 << 24)) fail("E300", tok().line, "array extent out of range");
            t.dims.push_back((int)n);
            need_p("]");
        }
        return t;
    }

    // Integer constant expression: literals, + - * / % << >> and parentheses, sizeof(type).
    int64_t const_int(int minprec = 0) {
        int64_t v = const_unary();
        for (;;) {
            static const struct { const char* s; int prec; } ops[] = {{"*", 10}, {"/", 10}, {"%", 10}, {"+", 9}, {"-", 9}, {"<<", 8}, {">>", 8}};
            int prec = -1;
            std::string op;
            for (auto& o : ops) if (is_p(o.s)) { prec = o.prec; op = o.s; }
            if (prec < 0 || prec < minprec) return v;
            int line = tok().line;
            i_++;
            int64_t r = const_int(prec + 1);
            if ((op == "/" || op == "%") && r == 0) fail("E300", line, "division by zero in a constant expression");
            if (op == "*") v *= r; else if (op == "/") v /= r; else if (op == "%") v %= r; else if (op == "+") v += r; else if (op == "-") v -= r;
            else if (op == "<<") v <<= (r & 63); else v >>= (r & 63);
        }
    }
    int64_t const_unary() {
        if (eat_p("-")) return -const_unary();
        if (eat_p("+")) return const_unary();
        if (eat_p("(")) { int64_t v = const_int(); need_p(")"); return v; }
        if (tok().k == Tk::Int) return (int64_t)t_[i_++].u;
        if (is_id("sizeof")) {
            i_++;
            need_p("(");
            DeclSpec d = decl_spec();
            std::string nm;
            CT t = declarator(d, &nm, true);
            need_p(")");
            return t.ptr ? 8 : total_bytes(t);
        }
        fail("E300", tok().line, "expected an integer constant expression, found `" + show(tok()) + "`");
    }

    // ---- top level ----
    void top_level() {
        if (eat_p(";")) return;
        for (const char* k : {"struct", "union", "enum", "typedef", "template", "class", "namespace", "using"})
            if (is_id(k)) fail("E304", tok().line, std::string("`") + k + "` is outside the subset");
        DeclSpec d = decl_spec();
        std::string name;
        CT t = declarator(d, &name, false);
        if (!is_p("(")) fail("E304", d.line, "file-scope variable `" + name + "` (global storage is outside the subset)");
        if (t.is_arr()) fail("E300", d.line, "a function cannot return an array");
        i_++;
        FuncSig sig;
        sig.ret = t;
        sig.ret_void = d.base_void && t.ptr == 0;
        sig.is_kernel = d.q_global;
        std::vector<std::string> names;
        if (is_id("void") && peek().k == Tk::Punct && peek().s == ")") i_++;
        if (!is_p(")")) {
            for (;;) {
                DeclSpec pd = decl_spec();
                std::string pn;
                CT pt = declarator(pd, &pn, true);
                if (pd.base_void && pt.ptr == 0) fail("E300", pd.line, "parameter of type void");
                if (pt.is_arr()) {   // T p[] style parameters decay; extents are dropped
                    if (pt.ptr) fail("E304", pd.line, "arrays of pointers are outside the subset");
                    pt.dims.clear();
                    pt.ptr = 1;
                }
                sig.params.push_back(pt);
                names.push_back(pn);
                if (eat_p(",")) continue;
                break;
            }
        }
        need_p(")");
        if (sig.is_kernel && !sig.ret_void) fail("E303", d.line, "a __global__ function must return void");
        auto it = sigs_.find(name);
        if (it != sigs_.end()) {
            if (it->second.params.size() != sig.params.size() || it->second.is_kernel != sig.is_kernel)
                fail("E302", d.line, "`" + name + "` redeclared with a different signature");
        }
        if (eat_p(";")) {
            if (it == sigs_.end()) sigs_[name] = sig;
            return;
        }
        if (it != sigs_.end() && it->second.defined) fail("E302", d.line, "`" + name + "` is defined twice");
        sig.defined = true;
        sigs_[name] = sig;
        if (d.has_lb) {
            if (!sig.is_kernel) fail("E303", d.line, "__launch_bounds__ on a function that is not __global__");
            m_->has_launch_bounds = true;
            m_->max_threads = d.lb_threads;
            m_->min_blocks = d.lb_blocks;
        }
        if (!is_p("{")) fail("E201", tok().line, "expected `{` or `;` after the parameter list");
        function_body(name, names);
    }

    void function_body(const std::string& name, const std::vector<std::string>& names) {
        m_->funcs.emplace_back();
        f_ = &m_->funcs.back();
        sig_ = &sigs_[name];
        f_->name = name;
        f_->is_kernel = sig_->is_kernel;
        f_->ret = sig_->ret_void ? Ty::v() : vty(sig_->ret);
        for (auto& p : sig_->params) f_->params.push_back(vty(p));
        closed_.clear();
        scopes_.clear();
        loops_.clear();
        next_slot_ = 0;
        cur_ = new_block();
        scopes_.emplace_back();
        for (size_t i = 0; i < names.size(); i++) {
            if (names[i].empty()) continue;
            if (scopes_.back().count(names[i])) fail("E302", tok().line, "parameter `" + names[i] + "` is named twice");
            Local l{(next_slot_++) * 65536, sig_->params[i], Space::Param};
            Val addr = ci(Ty::p(Space::Param), l.key);
            store(vty(l.ty), Space::Param, addr, Val::P((uint32_t)i));
            scopes_.back()[names[i]] = l;
        }
        block_stmt();
        if (!closed_[cur_]) {
            if (sig_->ret_void) ret(false, Val());
            else {
                Ty rt = f_->ret;
                Val z = rt.is_float() ? cf(rt, 0.0) : ci(rt, 0);
                ret(true, z);
            }
        }
        canonicalize(*f_);
        f_ = nullptr;
    }

    // ---- statements ----
    void block_stmt() {
        need_p("{");
        scopes_.emplace_back();
        while (!is_p("}")) {
            if (at_eof()) fail("E202", tok().line, "unterminated block");
            statement();
        }
        i_++;
        scopes_.pop_back();
    }

    void statement() {
        if (is_p("{")) { block_stmt(); return; }
        if (eat_p(";")) return;
        int line = tok().line;
        if (eat_id("if")) {
            need_p("(");
            Val c = to_bool(rval(expr()), line);
            need_p(")");
            uint32_t tb = new_block(), fb = new_block(), mb = new_block();
            condbr(c, tb, fb);
            at(tb);
            scoped_statement();
            br(mb);
            at(fb);
            if (eat_id("else")) scoped_statement();
            br(mb);
            at(mb);
            return;
        }
        if (eat_id("while")) {
            need_p("(");
            uint32_t cb = new_block(), bb = new_block(), xb = new_block();
            br(cb);
            at(cb);
            Val c = to_bool(rval(expr()), line);
            need_p(")");
            condbr(c, bb, xb);
            at(bb);
            loops_.push_back({xb, cb});
            scoped_statement();
            loops_.pop_back();
            br(cb);
            at(xb);
            return;
        }
        if (eat_id("do")) {
            uint32_t bb = new_block(), cb = new_block(), xb = new_block();
            br(bb);
            at(bb);
            loops_.push_back({xb, cb});
            scoped_statement();
            loops_.pop_back();
            br(cb);
            at(cb);
            if (!eat_id("while")) fail("E201", tok().line, "expected `while` after a do body");
            need_p("(");
            Val c = to_bool(rval(expr()), line);
            need_p(")");
            need_p(";");
            condbr(c, bb, xb);
            at(xb);
            return;
        }
        if (eat_id("for")) {
            need_p("(");
            scopes_.emplace_back();
            if (!eat_p(";")) {
                if (type_start(tok())) declaration();
                else { expr(); need_p(";"); }
            }
            uint32_t cb = new_block(), bb = new_block(), sb = new_block(), xb = new_block();
            br(cb);
            at(cb);
            if (is_p(";")) br(bb);
            else {
                Val c = to_bool(rval(expr()), line);
                condbr(c, bb, xb);
            }
            need_p(";");
            size_t step_at = i_;
            skip_to_close_paren();
            at(bb);
            loops_.push_back({xb, sb});
            scoped_statement();
            loops_.pop_back();
            br(sb);
            size_t after = i_;
            at(sb);
            i_ = step_at;
            if (!is_p(")")) expr();
            need_p(")");
            i_ = after;
            br(cb);
            at(xb);
            scopes_.pop_back();
            return;
        }
        if (eat_id("return")) {
            if (sig_->ret_void) {
                if (!is_p(";")) fail("E300", line, "a void function cannot return a value");
                need_p(";");
                ret(false, Val());
            } else {
                if (is_p(";")) fail("E300", line, "missing return value");
                Ex v = convert(rval(expr()), sig_->ret, line);
                need_p(";");
                ret(true, v.v);
            }
            return;
        }
        if (eat_id("switch")) {
            // The dispatch block is filled in after the body, when every label is known: the scrutinee is evaluated
            // before it, the body starts in an unreachable block (code before the first label never runs), a label
            // opens a new block that the code before it falls into, `break` leaves for the block after the switch and
            // `continue` still belongs to the enclosing loop.
            need_p("(");
            Ex sv = rval(expr());
            if (!sv.ty.is_scalar() || !is_int(sv.ty.b)) fail("E300", line, "the value a `switch` selects on must be an integer");
            sv = convert(sv, scalar_ct(promote(sv.ty.b)), line);
            need_p(")");
            if (!is_p("{")) fail("E304", line, "a `switch` body must be a block");
            i_++;
            const uint32_t dispatch = new_block(), after = new_block(), before_first_label = new_block();
            br(dispatch);
            at(before_first_label);
            loops_.push_back({after, loops_.empty() ? UINT32_MAX : loops_.back().cont});
            scopes_.emplace_back();
            std::vector<std::pair<int64_t, uint32_t>> cases;
            bool has_default = false;
            uint32_t default_block = after;
            while (!is_p("}")) {
                if (at_eof()) fail("E202", line, "unterminated `switch`");
                const int label_line = tok().line;
                if (eat_id("case") || is_id("default")) {
                    const bool is_default = is_id("default");
                    int64_t value = 0;
                    if (is_default) i_++;
                    else value = const_int();
                    need_p(":");
                    const uint32_t lb = new_block();
                    br(lb);   // the code above falls through into the label
                    at(lb);
                    if (is_default) {
                        if (has_default) fail("E302", label_line, "a second `default` label");
                        has_default = true;
                        default_block = lb;
                    } else {
                        if (size_of(sv.ty.b) == 4) value = (int64_t)(int32_t)value;
                        for (auto& c : cases) if (c.first == value) fail("E302", label_line, "the case value " + std::to_string(value) + " appears twice");
                        cases.push_back({value, lb});
                    }
                    continue;
                }
                statement();
            }
            i_++;
            scopes_.pop_back();
            loops_.pop_back();
            br(after);
            at(dispatch);
            Term& t = f_->blocks[cur_].term;
            t.kind = Term::Switch;
            t.has_val = true;
            t.val = sv.v;
            t.t = default_block;
            t.cases = cases;
            closed_[cur_] = true;
            at(after);
            return;
        }
        if (eat_id("break")) {
            if (loops_.empty()) fail("E201", line, "`break` outside a loop or switch");
            need_p(";");
            br(loops_.back().brk);
            return;
        }
        if (eat_id("continue")) {
            if (loops_.empty() || loops_.back().cont == UINT32_MAX) fail("E201", line, "`continue` outside a loop");
            need_p(";");
            br(loops_.back().cont);
            return;
        }
        if (is_id("case") || is_id("default")) fail("E201", line, "`" + tok().s + "` outside a switch");
        if (is_id("goto") || is_id("struct") || is_id("union") || is_id("enum") || is_id("typedef") || is_id("template") || is_id("asm"))
            fail("E304", line, "`" + tok().s + "` is outside the subset");
        if (type_start(tok())) { declaration(); return; }
        expr();
        need_p(";");
    }

    void scoped_statement() {
        scopes_.emplace_back();
        statement();
        scopes_.pop_back();
    }

    void skip_to_close_paren() {
        int depth = 0;
        for (;;) {
            if (at_eof()) fail("E202", tok().line, "unterminated `for (`");
            if (is_p("(")) depth++;
            else if (is_p(")")) { if (depth == 0) { i_++; return; } depth--; }
            i_++;
        }
    }

    void declaration() {
        DeclSpec d = decl_spec();
        if (d.q_global || d.q_device || d.q_host) fail("E303", d.line, "execution-space qualifier on a local declaration");
        if (d.q_constant) fail("E304", d.line, "__constant__ variables are outside the subset");
        for (;;) {
            std::string name;
            CT t = declarator(d, &name, false);
            if (d.base_void && t.ptr == 0) fail("E300", d.line, "variable `" + name + "` declared void");
            if (scopes_.back().count(name)) fail("E302", d.line, "`" + name + "` is already declared in this scope");
            Local l;
            l.ty = t;
            l.sp = d.q_shared ? Space::Shared : Space::Local;
            if (t.is_arr() && !d.q_shared) fail("E304", d.line, "local arrays are outside the subset (only __shared__ arrays)");
            if (t.is_arr() && t.ptr) fail("E304", d.line, "arrays of pointers are outside the subset");
            l.key = (next_slot_++) * 65536;
            if (d.q_shared) {
                SharedObj so;
                so.key = l.key + shared_key_base();
                l.key = so.key;
                so.bytes = (uint32_t)total_bytes(t);
                so.align = t.is_arr() ? 16 : (t.ptr ? 8 : size_of(t.b));
                m_->shared_objs.push_back(so);
                if (is_p("=")) fail("E300", d.line, "a __shared__ variable cannot have an initialiser");
            }
            if (eat_p("=")) {
                if (is_p("{")) fail("E304", d.line, "brace initialisers are outside the subset");
                Ex v = convert(rval(assign()), unqual(t), d.line);
                if (t.ptr) l.ty.psp = v.ty.psp;   // a pointer local points into whatever space its initialiser does
                Val addr = ci(Ty::p(l.sp), l.key);
                store(vty(l.ty), l.sp, addr, v.v);
            }
            scopes_.back()[name] = l;
            if (eat_p(",")) continue;
            break;
        }
        need_p(";");
    }

    // Shared cells of different functions of one module must not collide: offset by function index.
    int64_t shared_key_base() const { return (int64_t)(m_->funcs.size() - 1) * (int64_t(1) << 32); }

    static CT unqual(CT t) { if (!t.ptr) t.cnst = false; return t; }

    // ---- expressions ----
    Ex rval(Ex e) {
        if (e.is_void) return e;
        if (!e.lv) return e;
        Ex r;
        r.ty = e.ty;
        if (e.ty.is_arr()) {   // decay to a pointer to the first element
            CT p;
            p.b = e.ty.b;
            p.dims.assign(e.ty.dims.begin() + 1, e.ty.dims.end());
            if (!p.dims.empty()) {   // pointer to a sub-array: keep as an array lvalue-like address
                r.ty = e.ty;
                r.v = e.v;
                r.sp = e.sp;
                r.lv = false;
                return r;
            }
            p.ptr = 1;
            p.psp = e.sp;
            p.cnst = e.ty.cnst;
            r.ty = p;
            r.v = e.v;
            return r;
        }
        r.v = load(vty(e.ty), e.sp, e.v);
        if (!r.ty.ptr) r.ty.cnst = false;
        return r;
    }

    void need_value(const Ex& e, int line) {
        if (e.is_void) fail("E300", line, "a void value is used");
    }

    Val to_bool(Ex e, int line) {
        need_value(e, line);
        if (e.ty.is_arr()) fail("E300", line, "an array is used as a condition");
        if (e.ty.ptr) return icmp(ICmp::Ne, vty(e.ty), e.v, ci(vty(e.ty), 0));
        if (e.ty.b == B::Bool) return e.v;
        Ty t = vty(e.ty);
        if (is_flt(e.ty.b)) return fcmp(FCmp::One, t, e.v, cf(t, 0.0));
        return icmp(ICmp::Ne, t, e.v, ci(t, 0));
    }

    static int rank(B b) {
        switch (b) {
            case B::Bool: return 0;
            case B::Char: case B::UChar: return 1;
            case B::Short: case B::UShort: return 2;
            case B::Int: return 3;
            case B::UInt: return 4;
            case B::Long: return 5;
            case B::ULong: return 6;
            case B::Half: return 7;
            case B::Float: return 8;
            case B::Double: return 9;
            default: return -1;
        }
    }
    static B promote(B b) { return rank(b) < 3 ? B::Int : b; }
    static B common(B a, B b) {
        a = promote(a);
        b = promote(b);
        return rank(a) >= rank(b) ? a : b;
    }

    Ex convert(Ex e, const CT& to, int line) {
        need_value(e, line);
        if (to.is_arr()) fail("E300", line, "cannot convert to an array type");
        if (e.ty.is_arr()) fail("E304", line, "multi-dimensional array values are outside the subset");
        Ex r;
        r.ty = to;
        if (to.ptr) {
            if (e.ty.ptr) {
                if (e.ty.b != to.b && to.b != B::Void && e.ty.b != B::Void) fail("E300", line, "cannot convert `" + show(e.ty) + "` to `" + show(to) + "`");
                if (e.ty.cnst && !to.cnst) fail("E308", line, "conversion drops const from `" + show(e.ty) + "`");
                r.v = e.v;
                r.ty.psp = e.ty.psp;
                return r;
            }
            if (is_int(e.ty.b)) {   // only the null pointer constant
                const Inst& in = f_->insts[e.v.idx];
                if (!e.v.param && in.op == Opc::ConstI && in.imm == 0) { r.v = ci(vty(to), 0); return r; }
            }
            fail("E300", line, "cannot convert `" + show(e.ty) + "` to `" + show(to) + "`");
        }
        if (e.ty.ptr) fail("E300", line, "cannot convert `" + show(e.ty) + "` to `" + show(to) + "`");
        B from = e.ty.b, tb = to.b;
        if (tb == B::Void) fail("E300", line, "cannot convert to void");
        r.ty.cnst = false;
        if (from == tb) { r.v = e.v; return r; }
        Ty ft = Ty::s(scalar_of(from)), tt = Ty::s(scalar_of(tb));
        if (tb == B::Bool) { r.v = to_bool(e, line); return r; }
        if (is_int(from) && is_int(tb)) {
            unsigned fs = scalar_bits(ft.sc), ts = scalar_bits(tt.sc);
            if (from == B::Bool) r.v = cast(CastOp::ZExt, tt, ft, e.v);
            else if (fs == ts) r.v = e.v;
            else if (fs < ts) r.v = cast(is_signed(from) ? CastOp::SExt : CastOp::ZExt, tt, ft, e.v);
            else r.v = cast(CastOp::Trunc, tt, ft, e.v);
            return r;
        }
        if (is_int(from) && is_flt(tb)) {
            Val v = e.v;
            Ty st = ft;
            if (scalar_bits(ft.sc) < 32) {   // widen narrow integers first
                st = Ty::s(Scalar::I32);
                v = cast(from == B::Bool || !is_signed(from) ? CastOp::ZExt : CastOp::SExt, st, ft, v);
            }
            r.v = cast(is_signed(from) ? CastOp::SIToFP : CastOp::UIToFP, tt, st, v);
            return r;
        }
        if (is_flt(from) && is_int(tb)) {
            Ty it = scalar_bits(tt.sc) < 32 ? Ty::s(Scalar::I32) : tt;
            Val v = cast(is_signed(tb) ? CastOp::FPToSI : CastOp::FPToUI, it, ft, e.v);
            if (it != tt) v = cast(CastOp::Trunc, tt, it, v);
            r.v = v;
            return r;
        }
        r.v = cast(rank(tb) > rank(from) ? CastOp::FPExt : CastOp::FPTrunc, tt, ft, e.v);
        return r;
    }

    Ex expr() {
        Ex e = assign();
        while (eat_p(",")) e = assign();
        return e;
    }

    Ex assign() {
        int line = tok().line;
        Ex l = ternary();
        static const struct { const char* s; const char* op; } kOps[] = {{"=", ""}, {"+=", "+"}, {"-=", "-"}, {"*=", "*"}, {"/=", "/"}, {"%=", "%"},
                                                                       {"&=", "&"}, {"|=", "|"}, {"^=", "^"}, {"<<=", "<<"}, {">>=", ">>"}};
        for (auto& o : kOps) {
            if (!is_p(o.s)) continue;
            i_++;
            check_assignable(l, line);
            Ex r = rval(assign());
            if (*o.op) r = arith(o.op, rval(l), r, line);
            Ex v = convert(r, unqual(l.ty), line);
            store(vty(l.ty), l.sp, l.v, v.v);
            v.lv = false;
            return v;
        }
        return l;
    }

    void check_assignable(const Ex& l, int line) {
        if (!l.lv || l.ty.is_arr()) fail("E300", line, "the left side of an assignment is not assignable");
        if (l.ty.cnst && !l.ty.ptr) fail("E308", line, "assignment to a const object");
    }

    Ex ternary() {
        int line = tok().line;
        Ex c = binary(1);
        if (!is_p("?")) return c;
        i_++;
        Val cv = to_bool(rval(c), line);
        uint32_t tb = new_block(), fb = new_block(), mb = new_block();
        condbr(cv, tb, fb);
        at(tb);
        Ex a = rval(expr());
        uint32_t a_end = cur_;
        if (!eat_p(":")) fail("E201", tok().line, "expected `:` in a conditional expression");
        at(fb);
        Ex b = rval(ternary());
        need_value(a, line);
        need_value(b, line);
        CT ty;
        if (a.ty.ptr || b.ty.ptr) ty = a.ty.ptr ? a.ty : b.ty;
        else ty = scalar_ct(common(a.ty.b, b.ty.b));
        b = convert(b, ty, line);
        uint32_t b_end = cur_;
        br(mb);
        at(a_end);
        a = convert(a, ty, line);
        a_end = cur_;
        br(mb);
        at(mb);
        Ex r;
        r.ty = ty;
        r.v = phi(vty(ty), {{a_end, a.v}, {b_end, b.v}});
        return r;
    }

    static int prec_of(const Token& t) {
        if (t.k != Tk::Punct) return -1;
        static const struct { const char* s; int p; } tab[] = {{"||", 1}, {"&&", 2}, {"|", 3}, {"^", 4}, {"&", 5}, {"==", 6}, {"!=", 6}, {"<", 7}, {">", 7}, {"<=", 7},
                                                               {">=", 7}, {"<<", 8}, {">>", 8}, {"+", 9}, {"-", 9}, {"*", 10}, {"/", 10}, {"%", 10}};
        for (auto& e : tab) if (t.s == e.s) return e.p;
        return -1;
    }

    Ex binary(int minprec) {
        Ex l = unary();
        for (;;) {
            int p = prec_of(tok());
            if (p < 0 || p < minprec) return l;
            std::string op = tok().s;
            int line = tok().line;
            i_++;
            if (op == "&&" || op == "||") {
                Val lv = to_bool(rval(l), line);
                uint32_t l_end = cur_;
                uint32_t rb = new_block(), mb = new_block();
                if (op == "&&") condbr(lv, rb, mb); else condbr(lv, mb, rb);
                l_end = cur_;
                at(rb);
                Val rv = to_bool(rval(binary(p + 1)), line);
                uint32_t r_end = cur_;
                br(mb);
                at(mb);
                // the short-circuit arm contributes the constant the operator is known to yield
                Ex r;
                r.ty = scalar_ct(B::Bool);
                Inst k;
                k.op = Opc::ConstI;
                k.ty = Ty::s(Scalar::I1);
                k.imm = op == "||" ? 1 : 0;
                // constants must dominate the phi: place it in the left operand's block
                uint32_t kid = (uint32_t)f_->insts.size();
                f_->insts.push_back(k);
                f_->blocks[l_end].insts.push_back(kid);
                r.v = phi(Ty::s(Scalar::I1), {{l_end, Val::V(kid)}, {r_end, rv}});
                l = r;
                continue;
            }
            l = rval(l);   // left operand is read before the right one is evaluated
            Ex r = rval(binary(p + 1));
            l = arith(op.c_str(), l, r, line);
        }
    }

    // Pointer + integer, in bytes: widen, scale, add (crates/basalt-sema/src/lower.rs:1736-1787).
    Val ptr_add(const Ex& p, Ex idx, int64_t esz, bool negate, int line) {
        if (idx.ty.ptr || !is_int(idx.ty.b)) fail("E300", line, "pointer offset must be an integer");
        Ty i64t = Ty::s(Scalar::I64);
        B ib = idx.ty.b;
        Ex w = idx;
        if (size_of(ib) != 8 || ib == B::Bool) w.v = cast(is_signed(ib) ? CastOp::SExt : CastOp::ZExt, i64t, Ty::s(scalar_of(ib)), idx.v);
        Val off = bin(BinOp::Mul, i64t, w.v, ci(i64t, esz));
        if (negate) off = bin(BinOp::Sub, i64t, ci(i64t, 0), off);
        Ty pt = p.ty.is_arr() ? Ty::p(p.sp) : vty(p.ty);
        return bin(BinOp::Add, pt, p.v, off);
    }

    Ex arith(const char* op, Ex a, Ex b, int line) {
        need_value(a, line);
        need_value(b, line);
        std::string o = op;
        if (a.ty.is_arr() || b.ty.is_arr()) fail("E304", line, "arithmetic on multi-dimensional arrays is outside the subset");
        // pointer arithmetic
        if (a.ty.ptr || b.ty.ptr) {
            if ((o == "+" || o == "-") && a.ty.ptr && !b.ty.ptr) {
                if (a.ty.b == B::Void) fail("E300", line, "arithmetic on a void pointer");
                Ex r;
                r.ty = a.ty;
                r.v = ptr_add(a, b, size_of(a.ty.b), o == "-", line);
                return r;
            }
            if (o == "+" && b.ty.ptr && !a.ty.ptr) return arith("+", b, a, line);
            if (o == "-" && a.ty.ptr && b.ty.ptr) {
                Ty i64t = Ty::s(Scalar::I64);
                Val x = cast(CastOp::Bitcast, i64t, vty(a.ty), a.v), y = cast(CastOp::Bitcast, i64t, vty(b.ty), b.v);
                Ex r;
                r.ty = scalar_ct(B::Long);
                r.v = bin(BinOp::Div, i64t, bin(BinOp::Sub, i64t, x, y), ci(i64t, size_of(a.ty.b)));
                return r;
            }
            if ((o == "==" || o == "!=" || o == "<" || o == ">" || o == "<=" || o == ">=") ) {
                CT pt = a.ty.ptr ? a.ty : b.ty;
                a = convert(a, pt, line);
                b = convert(b, pt, line);
                Ex r;
                r.ty = scalar_ct(B::Bool);
                ICmp p = o == "==" ? ICmp::Eq : o == "!=" ? ICmp::Ne : o == "<" ? ICmp::Ult : o == ">" ? ICmp::Ugt : o == "<=" ? ICmp::Ule : ICmp::Uge;
                r.v = icmp(p, vty(pt), a.v, b.v);
                return r;
            }
            fail("E300", line, "invalid operands to `" + o + "`: `" + show(a.ty) + "` and `" + show(b.ty) + "`");
        }
        if (a.ty.b == B::Half || b.ty.b == B::Half) fail("E304", line, "arithmetic on __half is outside the subset; convert with __half2float");
        bool shift = o == "<<" || o == ">>";
        B cb = shift ? promote(a.ty.b) : common(a.ty.b, b.ty.b);
        CT ct = scalar_ct(cb);
        a = convert(a, ct, line);
        b = convert(b, shift ? scalar_ct(cb) : ct, line);
        Ty t = vty(ct);
        Ex r;
        bool flt = is_flt(cb), sgn = is_signed(cb);
        if (o == "==" || o == "!=" || o == "<" || o == ">" || o == "<=" || o == ">=") {
            r.ty = scalar_ct(B::Bool);
            if (flt) {
                FCmp p = o == "==" ? FCmp::Oeq : o == "!=" ? FCmp::One : o == "<" ? FCmp::Olt : o == ">" ? FCmp::Ogt : o == "<=" ? FCmp::Ole : FCmp::Oge;
                r.v = fcmp(p, t, a.v, b.v);
            } else {
                ICmp p = o == "==" ? ICmp::Eq : o == "!=" ? ICmp::Ne
                       : o == "<" ? (sgn ? ICmp::Slt : ICmp::Ult) : o == ">" ? (sgn ? ICmp::Sgt : ICmp::Ugt)
                       : o == "<=" ? (sgn ? ICmp::Sle : ICmp::Ule) : (sgn ? ICmp::Sge : ICmp::Uge);
                r.v = icmp(p, t, a.v, b.v);
            }
            return r;
        }
        r.ty = ct;
        if (flt) {
            BinOp bo;
            if (o == "+") bo = BinOp::FAdd; else if (o == "-") bo = BinOp::FSub; else if (o == "*") bo = BinOp::FMul; else if (o == "/") bo = BinOp::FDiv;
            else fail("E300", line, "invalid operands to `" + o + "`: floating-point values");
            r.v = bin(bo, t, a.v, b.v);
            return r;
        }
        BinOp bo;
        if (o == "+") bo = BinOp::Add;
        else if (o == "-") bo = BinOp::Sub;
        else if (o == "*") bo = BinOp::Mul;
        else if (o == "/" || o == "%") {
            if (!sgn) return unsigned_divrem(o == "/", a, b, t, ct, line);
            bo = o == "/" ? BinOp::Div : BinOp::Rem;
        }
        else if (o == "&") bo = BinOp::And;
        else if (o == "|") bo = BinOp::Or;
        else if (o == "^") bo = BinOp::Xor;
        else if (o == "<<") bo = BinOp::Shl;
        else if (o == ">>") bo = sgn ? BinOp::AShr : BinOp::LShr;
        else fail("E201", line, "unknown operator `" + o + "`");
        r.v = bin(bo, t, a.v, b.v);
        return r;
    }

    // BIR division is signed (crates/basalt-x86/src/oracle.rs:1546-1610).  An unsigned divide by a power-of-two
    // constant is a shift or a mask; any other 32-bit one is done in 64 bits, where both operands, zero-extended,
    // are non-negative and the signed quotient and remainder are the unsigned ones.  A 64-bit unsigned divide by
    // anything else has no such widening and is refused.
    Ex unsigned_divrem(bool is_div, const Ex& a, const Ex& b, Ty t, const CT& ct, int line) {
        Ex r;
        r.ty = ct;
        const Inst* k = b.v.param ? nullptr : &f_->insts[b.v.idx];
        if (k && k->op == Opc::ConstI) {
            uint64_t d = (uint64_t)k->imm;
            if (scalar_bits(t.sc) == 32) d &= 0xffffffffu;
            if (d != 0 && !(d & (d - 1))) {
                int sh = 0;
                while ((d >> sh) != 1) sh++;
                r.v = is_div ? bin(BinOp::LShr, t, a.v, ci(t, sh)) : bin(BinOp::And, t, a.v, ci(t, (int64_t)(d - 1)));
                return r;
            }
        }
        if (scalar_bits(t.sc) != 32) fail("E304", line, "64-bit unsigned division by anything but a power-of-two constant is outside the subset (BIR division is signed)");
        const Ty wide = Ty::s(Scalar::I64);
        Val q = bin(is_div ? BinOp::Div : BinOp::Rem, wide, cast(CastOp::ZExt, wide, t, a.v), cast(CastOp::ZExt, wide, t, b.v));
        r.v = cast(CastOp::Trunc, t, wide, q);
        return r;
    }

    Ex unary() {
        int line = tok().line;
        if (eat_p("-")) {
            Ex e = rval(unary());
            need_value(e, line);
            if (e.ty.ptr || e.ty.is_arr()) fail("E300", line, "unary minus on a pointer");
            if (e.ty.b == B::Half) fail("E304", line, "arithmetic on __half is outside the subset");
            e = convert(e, scalar_ct(promote(e.ty.b)), line);
            Ty t = vty(e.ty);
            // 0 - x, as the reference lowers it (crates/basalt-sema/src/lower.rs:1931-1939)
            e.v = is_flt(e.ty.b) ? bin(BinOp::FSub, t, cf(t, 0.0), e.v) : bin(BinOp::Sub, t, ci(t, 0), e.v);
            return e;
        }
        if (eat_p("+")) {
            Ex e = rval(unary());
            need_value(e, line);
            if (!e.ty.ptr) e = convert(e, scalar_ct(promote(e.ty.b)), line);
            return e;
        }
        if (eat_p("!")) {
            Ex e = rval(unary());
            Val b = to_bool(e, line);
            Ex r;
            r.ty = scalar_ct(B::Bool);
            r.v = bin(BinOp::Xor, Ty::s(Scalar::I1), b, ci(Ty::s(Scalar::I1), 1));
            return r;
        }
        if (eat_p("~")) {
            Ex e = rval(unary());
            need_value(e, line);
            if (e.ty.ptr || !is_int(e.ty.b)) fail("E300", line, "`~` needs an integer operand");
            e = convert(e, scalar_ct(promote(e.ty.b)), line);
            Ty t = vty(e.ty);
            e.v = bin(BinOp::Xor, t, e.v, ci(t, -1));
            return e;
        }
        if (eat_p("*")) {
            Ex e = rval(unary());
            need_value(e, line);
            if (!e.ty.ptr) fail("E300", line, "`*` needs a pointer operand");
            if (e.ty.b == B::Void) fail("E300", line, "dereference of a void pointer");
            Ex r;
            r.lv = true;
            r.v = e.v;
            r.ty = scalar_ct(e.ty.b);
            r.ty.cnst = e.ty.cnst;
            r.sp = e.ty.psp;
            return r;
        }
        if (eat_p("&")) {
            Ex e = unary();
            if (!e.lv) fail("E300", line, "`&` needs an lvalue");
            if (e.ty.is_arr() || e.ty.ptr) fail("E304", line, "address of an array or pointer object is outside the subset");
            if (e.sp == Space::Local || e.sp == Space::Param) fail("E304", line, "address of a local variable is outside the subset");
            Ex r;
            r.ty = e.ty;
            r.ty.ptr = 1;
            r.ty.psp = e.sp;
            r.v = e.v;
            return r;
        }
        if (is_p("++") || is_p("--")) {
            bool inc = is_p("++");
            i_++;
            Ex l = unary();
            check_assignable(l, line);
            return step(l, inc, true, line);
        }
        if (is_id("sizeof")) {
            Ex r;
            r.ty = scalar_ct(B::ULong);
            r.v = ci(Ty::s(Scalar::I64), const_unary());
            return r;
        }
        if (is_p("(") && type_start(peek())) {   // cast
            i_++;
            DeclSpec d = decl_spec();
            std::string nm;
            CT to = declarator(d, &nm, true);
            need_p(")");
            Ex e = rval(unary());
            if (d.base_void && to.ptr == 0) { Ex r; r.is_void = true; return r; }
            if (to.ptr && e.ty.ptr) {   // pointer casts reinterpret the pointee
                Ex r;
                r.ty = to;
                r.ty.psp = e.ty.psp;
                r.v = e.v;
                return r;
            }
            return convert(e, to, line);
        }
        return postfix();
    }

    Ex step(Ex l, bool inc, bool prefix, int line) {
        Ex old = rval(l);
        Ex one;
        one.ty = scalar_ct(B::Int);
        one.v = ci(Ty::s(Scalar::I32), 1);
        Ex nv = arith(inc ? "+" : "-", old, one, line);
        Ex st = convert(nv, unqual(l.ty), line);
        store(vty(l.ty), l.sp, l.v, st.v);
        return prefix ? st : old;
    }

    Ex postfix() {
        Ex e = primary();
        for (;;) {
            int line = tok().line;
            if (eat_p("[")) {
                Ex idx = rval(expr());
                need_p("]");
                need_value(idx, line);
                Ex base = e.lv && e.ty.is_arr() ? e : rval(e);
                if (base.ty.is_arr()) {
                    Ex r;
                    r.lv = true;
                    r.sp = base.sp;
                    r.v = ptr_add(base, idx, elem_bytes(base.ty), false, line);
                    r.ty = base.ty;
                    r.ty.dims.erase(r.ty.dims.begin());
                    e = r;
                    continue;
                }
                if (!base.ty.ptr) fail("E300", line, "subscript of a value that is neither a pointer nor an array");
                if (base.ty.b == B::Void) fail("E300", line, "subscript of a void pointer");
                Ex r;
                r.lv = true;
                r.sp = base.ty.psp;
                r.v = ptr_add(base, idx, size_of(base.ty.b), false, line);
                r.ty = scalar_ct(base.ty.b);
                r.ty.cnst = base.ty.cnst;
                e = r;
                continue;
            }
            if (is_p("++") || is_p("--")) {
                bool inc = is_p("++");
                i_++;
                check_assignable(e, line);
                e = step(e, inc, false, line);
                continue;
            }
            if (is_p(".") || is_p("->")) fail("E304", line, "member access is outside the subset");
            return e;
        }
    }

    Ex index_value(unsigned sub) {
        Inst in;
        in.op = Opc::Index;
        in.sub = (uint8_t)sub;
        in.ty = Ty::s(Scalar::I32);
        Ex r;
        r.ty = scalar_ct(B::UInt);
        r.v = push(in);
        return r;
    }

    Ex primary() {
        int line = tok().line;
        if (eat_p("(")) {
            Ex e = expr();
            need_p(")");
            return e;
        }
        if (tok().k == Tk::Int) {
            const Token& t = t_[i_++];
            B b;
            if (t.lng) b = t.uns ? B::ULong : B::Long;
            else if (t.uns) b = t.u <= 0xffffffffull ? B::UInt : B::ULong;
            else if (t.u <= 0x7fffffffull) b = B::Int;
            else if (t.hex && t.u <= 0xffffffffull) b = B::UInt;
            else b = t.u <= 0x7fffffffffffffffull ? B::Long : B::ULong;
            Ex r;
            r.ty = scalar_ct(b);
            r.v = ci(vty(r.ty), (int64_t)t.u);
            return r;
        }
        if (tok().k == Tk::Float) {
            const Token& t = t_[i_++];
            Ex r;
            r.ty = scalar_ct(t.f32 ? B::Float : B::Double);
            r.v = cf(vty(r.ty), t.f32 ? (double)(float)t.f : t.f);
            return r;
        }
        if (tok().k != Tk::Ident) fail("E201", line, "expected an expression, found `" + show(tok()) + "`");
        std::string name = t_[i_++].s;
        if (name == "true" || name == "false") {
            Ex r;
            r.ty = scalar_ct(B::Bool);
            r.v = ci(Ty::s(Scalar::I1), name == "true");
            return r;
        }
        if (name == "warpSize") {
            Ex r;
            r.ty = scalar_ct(B::Int);
            r.v = ci(Ty::s(Scalar::I32), 32);
            return r;
        }
        static const char* const kDims[] = {"threadIdx", "blockIdx", "blockDim", "gridDim"};
        for (unsigned g = 0; g < 4; g++) {
            if (name != kDims[g]) continue;
            need_p(".");
            std::string c = need_ident();
            if (c != "x" && c != "y" && c != "z") fail("E301", line, "`" + name + "` has no member `" + c + "`");
            return index_value(g * 3 + (unsigned)(c[0] - 'x'));
        }
        if (is_p("(")) return call(name, line);
        for (size_t s = scopes_.size(); s-- > 0;) {
            auto it = scopes_[s].find(name);
            if (it == scopes_[s].end()) continue;
            Ex r;
            r.lv = true;
            r.ty = it->second.ty;
            r.sp = it->second.sp;
            r.v = ci(Ty::p(r.sp), it->second.key);
            return r;
        }
        fail("E301", line, "`" + name + "` is not declared");
    }

    std::vector<Ex> args(int line) {
        std::vector<Ex> a;
        need_p("(");
        if (!is_p(")")) {
            for (;;) {
                a.push_back(rval(assign()));
                need_value(a.back(), line);
                if (eat_p(",")) continue;
                break;
            }
        }
        need_p(")");
        return a;
    }

    static void need_argc(const std::string& name, const std::vector<Ex>& a, size_t lo, size_t hi, int line) {
        if (a.size() < lo || a.size() > hi) fail("E300", line, "`" + name + "` takes " + std::to_string(lo) + (hi != lo ? " to " + std::to_string(hi) : "") + " arguments");
    }

    Ex call(const std::string& name, int line) {
        // ---- builtins ----
        if (name == "__syncthreads") {
            std::vector<Ex> a = args(line);
            need_argc(name, a, 0, 0, line);
            Inst in;
            in.op = Opc::Barrier;
            in.ty = Ty::v();
            push(in);
            Ex r;
            r.is_void = true;
            return r;
        }
        static const struct { const char* base; Shfl k; } kSh[] = {{"__shfl", Shfl::Idx}, {"__shfl_up", Shfl::Up}, {"__shfl_down", Shfl::Down}, {"__shfl_xor", Shfl::Xor}};
        for (auto& s : kSh) {
            bool sync = name == std::string(s.base) + "_sync";
            if (!sync && name != s.base) continue;
            std::vector<Ex> a = args(line);
            size_t o = sync ? 1 : 0;
            need_argc(name, a, o + 2, o + 3, line);
            if (sync) require_full_mask(a[0], name, line);
            if (a.size() == o + 3) require_const(a[o + 2], 32, name + " width", line);
            Ex v = a[o];
            if (v.ty.ptr || size_of(v.ty.b) > 4 || v.ty.b == B::Half) fail("E304", line, name + " of a value that is not 32 bits wide is outside the subset");
            if (size_of(v.ty.b) < 4) v = convert(v, scalar_ct(B::Int), line);
            Ex lane = convert(a[o + 1], scalar_ct(B::Int), line);
            Inst in;
            in.op = Opc::Shuffle;
            in.sub = (uint8_t)s.k;
            in.ty = vty(v.ty);
            in.ops = {v.v, lane.v};
            Ex r;
            r.ty = v.ty;
            r.v = push(in);
            return r;
        }
        static const struct { const char* base; Opc op; } kVote[] = {{"__ballot", Opc::Ballot}, {"__any", Opc::VoteAny}, {"__all", Opc::VoteAll}};
        for (auto& s : kVote) {
            bool sync = name == std::string(s.base) + "_sync";
            if (!sync && name != s.base) continue;
            std::vector<Ex> a = args(line);
            size_t o = sync ? 1 : 0;
            need_argc(name, a, o + 1, o + 1, line);
            if (sync) require_full_mask(a[0], name, line);
            Ex p = convert(a[o], scalar_ct(B::Int), line);   // the reference's typing: i32 in, i32 out (lower.rs:2601-2611)
            Inst in;
            in.op = s.op;
            in.ty = Ty::s(Scalar::I32);
            in.ops = {p.v};
            Ex r;
            r.ty = scalar_ct(s.op == Opc::Ballot ? B::UInt : B::Int);
            r.v = push(in);
            return r;
        }
        static const struct { const char* n; AtomOp op; } kAt[] = {{"atomicAdd", AtomOp::Add}, {"atomicSub", AtomOp::Sub}, {"atomicExch", AtomOp::Exch}, {"atomicMin", AtomOp::Min},
                                                                   {"atomicMax", AtomOp::Max}, {"atomicAnd", AtomOp::And}, {"atomicOr", AtomOp::Or}, {"atomicXor", AtomOp::Xor}};
        for (auto& s : kAt) {
            if (name != s.n) continue;
            std::vector<Ex> a = args(line);
            need_argc(name, a, 2, 2, line);
            if (!a[0].ty.ptr) fail("E300", line, name + " needs a pointer as its first argument");
            if (a[0].ty.cnst) fail("E308", line, name + " through a pointer to const");
            B eb = a[0].ty.b;
            bool ok = eb == B::Int || eb == B::UInt || eb == B::Long || eb == B::ULong || ((eb == B::Float || eb == B::Double) && (s.op == AtomOp::Add || s.op == AtomOp::Exch || s.op == AtomOp::Min || s.op == AtomOp::Max));
            if (!ok) fail("E304", line, name + " on `" + show(a[0].ty) + "` is outside the subset");
            if ((s.op == AtomOp::Min || s.op == AtomOp::Max) && (eb == B::UInt || eb == B::ULong))
                fail("E304", line, name + " on an unsigned type is outside the subset (BIR integer min/max are signed)");
            Ex v = convert(a[1], scalar_ct(eb), line);
            Inst in;
            in.op = Opc::Atomic;
            in.sub = (uint8_t)s.op;
            in.ty = Ty::s(scalar_of(eb));
            in.space = a[0].ty.psp;
            in.ops = {a[0].v, v.v};
            Ex r;
            r.ty = scalar_ct(eb);
            r.v = push(in);
            return r;
        }
        if (name == "atomicCAS") {
            std::vector<Ex> a = args(line);
            need_argc(name, a, 3, 3, line);
            if (!a[0].ty.ptr || !(a[0].ty.b == B::Int || a[0].ty.b == B::UInt || a[0].ty.b == B::Long || a[0].ty.b == B::ULong))
                fail("E304", line, "atomicCAS needs a pointer to a 32- or 64-bit integer");
            if (a[0].ty.cnst) fail("E308", line, "atomicCAS through a pointer to const");
            B eb = a[0].ty.b;
            Ex c = convert(a[1], scalar_ct(eb), line), v = convert(a[2], scalar_ct(eb), line);
            Inst in;
            in.op = Opc::AtomicCas;
            in.ty = Ty::s(scalar_of(eb));
            in.space = a[0].ty.psp;
            in.ops = {a[0].v, c.v, v.v};
            Ex r;
            r.ty = scalar_ct(eb);
            r.v = push(in);
            return r;
        }
        if (name == "min" || name == "max" || name == "fminf" || name == "fmaxf") {
            std::vector<Ex> a = args(line);
            need_argc(name, a, 2, 2, line);
            if (a[0].ty.ptr || a[1].ty.ptr) fail("E300", line, name + " of pointers");
            B cb = name[0] == 'f' ? B::Float : common(a[0].ty.b, a[1].ty.b);
            if (cb == B::Half) fail("E304", line, name + " on __half is outside the subset");
            CT ct = scalar_ct(cb);
            Ex x = convert(a[0], ct, line), y = convert(a[1], ct, line);
            bool is_min = name == "min" || name == "fminf";
            Ty t = vty(ct);
            Val c = is_flt(cb) ? fcmp(is_min ? FCmp::Olt : FCmp::Ogt, t, x.v, y.v)
                               : icmp(is_signed(cb) ? (is_min ? ICmp::Slt : ICmp::Sgt) : (is_min ? ICmp::Ult : ICmp::Ugt), t, x.v, y.v);
            Ex r;
            r.ty = ct;
            r.v = select(t, c, x.v, y.v);
            return r;
        }
        if (name == "abs" || name == "fabsf") {
            std::vector<Ex> a = args(line);
            need_argc(name, a, 1, 1, line);
            CT ct = scalar_ct(name == "abs" ? (is_flt(a[0].ty.b) ? a[0].ty.b : promote(a[0].ty.b)) : B::Float);
            if (a[0].ty.ptr || ct.b == B::Half) fail("E300", line, name + " needs an arithmetic operand");
            Ex x = convert(a[0], ct, line);
            Ty t = vty(ct);
            Ex r;
            r.ty = ct;
            if (is_flt(ct.b)) {
                Val neg = bin(BinOp::FSub, t, cf(t, 0.0), x.v);
                r.v = select(t, fcmp(FCmp::Olt, t, x.v, cf(t, 0.0)), neg, x.v);
            } else {
                Val neg = bin(BinOp::Sub, t, ci(t, 0), x.v);
                r.v = select(t, icmp(ICmp::Slt, t, x.v, ci(t, 0)), neg, x.v);
            }
            return r;
        }
        if (name == "__half2float" || name == "__float2half" || name == "__float2half_rn") {
            std::vector<Ex> a = args(line);
            need_argc(name, a, 1, 1, line);
            bool widen = name == "__half2float";
            Ex x = convert(a[0], scalar_ct(widen ? B::Half : B::Float), line);
            Ex r;
            r.ty = scalar_ct(widen ? B::Float : B::Half);
            r.v = cast(widen ? CastOp::FPExt : CastOp::FPTrunc, vty(r.ty), vty(x.ty), x.v);
            return r;
        }
        if (name == "__basalt_mma_f32" || name == "__basalt_mma_f16" || name == "__basalt_mma_f16_nt") return mma_intrinsic(name, line);
        static const char* const kKnown[] = {"sqrtf", "sqrt", "expf", "exp", "logf", "log", "sinf", "cosf", "powf", "fmaf", "__fmaf_rn", "rsqrtf", "printf", "__ldg",
                                             "cudaMalloc", "cudaMemcpy", "cudaFree", "cudaDeviceSynchronize", "__syncwarp", "__popc", "__clz"};
        for (const char* k : kKnown) if (name == k) fail("E304", line, "`" + name + "` has no BIR lowering");

        // ---- user functions ----
        auto it = sigs_.find(name);
        if (it == sigs_.end()) fail("E301", line, "function `" + name + "` is not declared");
        const FuncSig& sg = it->second;
        if (sg.is_kernel) fail("E303", line, "a __global__ function cannot be called from device code");
        std::vector<Ex> a = args(line);
        if (a.size() != sg.params.size()) fail("E300", line, "`" + name + "` takes " + std::to_string(sg.params.size()) + " arguments");
        Inst in;
        in.op = Opc::Call;
        in.callee = name;
        in.ty = sg.ret_void ? Ty::v() : vty(sg.ret);
        for (size_t i = 0; i < a.size(); i++) in.ops.push_back(convert(a[i], sg.params[i], line).v);
        Ex r;
        Val v = push(in);
        if (sg.ret_void) r.is_void = true;
        else { r.ty = sg.ret; r.v = v; }
        return r;
    }

    void require_full_mask(const Ex& m, const std::string& name, int line) { require_const(m, 0xffffffffll, name + " mask", line, true); }
    void require_const(const Ex& e, int64_t want, const std::string& what, int line, bool low32 = false) {
        const Inst* k = e.v.param ? nullptr : &f_->insts[e.v.idx];
        bool ok = k && k->op == Opc::ConstI && (low32 ? ((uint64_t)k->imm & 0xffffffffull) == (uint64_t)want : k->imm == want);
        if (!ok) fail("E304", line, what + " must be the constant " + (low32 ? std::string("0xffffffff") : std::to_string(want)) + " (BIR shuffles and votes are full-warp)");
    }

    // __basalt_mma_f32(m, n, k, a, b, c, d [, lda, ldb, ldc, ldd]): D = C + A*B on row-major tiles; c may
    // be 0 for D = A*B.  The _f16 form takes __half operands, accumulates in f32, writes __half.
    Ex mma_intrinsic(const std::string& name, int line) {
        bool f16 = name != "__basalt_mma_f32";
        need_p("(");
        Inst in;
        in.op = Opc::Mma;
        in.ty = Ty::v();
        in.m = (uint32_t)const_int(); need_p(",");
        in.n = (uint32_t)const_int(); need_p(",");
        in.k = (uint32_t)const_int(); need_p(",");
        if (!in.m || !in.n || !in.k) fail("E300", line, "mma extents must be positive");
        in.in_dt = f16 ? Scalar::F16 : Scalar::F32;
        in.acc_dt = Scalar::F32;
        in.out_dt = f16 ? Scalar::F16 : Scalar::F32;
        in.has_out = f16;
        in.b_col = name == "__basalt_mma_f16_nt";   // B stored [n x k]
        B want = f16 ? B::Half : B::Float;
        for (int j = 0; j < 4; j++) {
            Ex p = rval(assign());
            need_value(p, line);
            if (j == 2 && !p.ty.ptr) p = convert(p, ptr_ct(want), line);   // literal 0
            if (!p.ty.ptr || p.ty.b != want) fail("E300", line, name + " operand " + std::to_string(j + 1) + " must be a `" + base_name(want) + "*`");
            if (j == 3 && p.ty.cnst) fail("E308", line, name + " writes through a pointer to const");
            Val v = p.v;
            if (p.ty.psp != Space::Global && j != 2) {}
            in.ops.push_back(v);
            if (j < 3) need_p(",");
        }
        if (eat_p(",")) {
            in.has_ld = true;
            for (int j = 0; j < 4; j++) {
                in.ld[j] = const_int();
                if (j < 3) need_p(",");
            }
        }
        need_p(")");
        push(in);
        Ex r;
        r.is_void = true;
        return r;
    }
    static CT ptr_ct(B b) { CT t; t.b = b; t.ptr = 1; return t; }
};

}  // namespace

bool compile_cuda_c(const char* src, size_t len, Module* out, Diag* d) {
    try {
        Lexer lx(src, len);
        Module m;
        Compiler c(lx.run(), &m);
        c.run();
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
