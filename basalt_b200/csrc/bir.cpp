// BIR text parser / printer / verifier. Grammar: see bir.hpp (reference:
// crates/basalt-bir/src/lib.rs:21-68, parse.rs, print.rs).
#include "bir.hpp"

#include <charconv>
#include <cmath>
#include <cstring>
#include <map>

namespace basalt {

static const char* kScalar[] = {"i1", "i8", "i16", "i32", "i64", "f16", "f32", "f64"};
static const char* kSpace[] = {"global", "shared", "constant", "local", "param"};
static const char* kBin[] = {"add", "sub", "mul", "div", "rem", "fadd", "fsub", "fmul",
                             "fdiv", "frem", "and", "or", "xor", "shl", "lshr", "ashr"};
static const char* kICmp[] = {"eq", "ne", "slt", "sle", "sgt", "sge", "ult", "ule", "ugt", "uge"};
static const char* kFCmp[] = {"oeq", "one", "olt", "ole", "ogt", "oge", "ord", "uno"};
static const char* kCast[] = {"trunc", "zext", "sext", "fptrunc", "fpext",
                              "fptosi", "fptoui", "sitofp", "uitofp", "bitcast"};
static const char* kShfl[] = {"shuffle.idx", "shuffle.up", "shuffle.down", "shuffle.xor"};
static const char* kAtom[] = {"atomic.add", "atomic.sub", "atomic.exch", "atomic.min",
                              "atomic.max", "atomic.and", "atomic.or", "atomic.xor"};
static const char* kIndex[] = {"tid.x", "tid.y", "tid.z", "bid.x", "bid.y", "bid.z",
                               "bdim.x", "bdim.y", "bdim.z", "gdim.x", "gdim.y", "gdim.z"};
static const char* kRed[] = {"warp.reduce.max", "warp.reduce.min", "warp.reduce.add",
                             "warp.reduce.and", "warp.reduce.or", "warp.reduce.xor"};

const char* scalar_text(Scalar s) { return kScalar[(int)s]; }
const char* space_text(Space s) { return kSpace[(int)s]; }
const char* binop_text(BinOp o) { return kBin[(int)o]; }
const char* icmp_text(ICmp o) { return kICmp[(int)o]; }
const char* fcmp_text(FCmp o) { return kFCmp[(int)o]; }
const char* cast_text(CastOp o) { return kCast[(int)o]; }
const char* shfl_text(Shfl o) { return kShfl[(int)o]; }
const char* atom_text(AtomOp o) { return kAtom[(int)o]; }
const char* index_text(unsigned sub) { return kIndex[sub]; }
const char* redop_text(RedOp o) { return kRed[(int)o]; }

unsigned scalar_bits(Scalar s) {
    static const unsigned b[] = {1, 8, 16, 32, 64, 16, 32, 64};
    return b[(int)s];
}
unsigned scalar_bytes(Scalar s) { return s == Scalar::I1 ? 1 : scalar_bits(s) / 8; }

template <size_t N>
static int find_in(const char* const (&tab)[N], const std::string& w) {
    for (size_t i = 0; i < N; i++)
        if (w == tab[i]) return (int)i;
    return -1;
}

bool parse_scalar(const std::string& w, Scalar* out) {
    int i = find_in(kScalar, w);
    if (i < 0) return false;
    *out = (Scalar)i;
    return true;
}

std::string ty_text(Ty t) {
    switch (t.kind) {
        case Ty::Void: return "void";
        case Ty::Sc: return scalar_text(t.sc);
        case Ty::Ptr: return std::string("ptr.") + space_text(t.sp);
        case Ty::Vec: return "v" + std::to_string((unsigned)t.lanes) + scalar_text(t.sc);
    }
    return "?";
}

bool parse_ty(const std::string& w, Ty* out) {
    if (w == "void") { *out = Ty::v(); return true; }
    Scalar s;
    if (parse_scalar(w, &s)) { *out = Ty::s(s); return true; }
    if (w.rfind("ptr.", 0) == 0) {
        int i = find_in(kSpace, w.substr(4));
        if (i < 0) return false;
        *out = Ty::p((Space)i);
        return true;
    }
    if (w.size() > 2 && w[0] == 'v' && isdigit((unsigned char)w[1])) {
        size_t i = 1;
        unsigned lanes = 0;
        while (i < w.size() && isdigit((unsigned char)w[i])) {
            lanes = lanes * 10 + (unsigned)(w[i] - '0');
            if (lanes > 255) return false;
            i++;
        }
        if (!parse_scalar(w.substr(i), &s)) return false;
        *out = Ty::vec(s, (uint8_t)lanes);
        return true;
    }
    return false;
}

// ---- lexer ---------------------------------------------------------------------------------
namespace {
enum class Tk { Word, LParen, RParen, LBrace, RBrace, LBracket, RBracket, Comma, Colon, Eq, Arrow, Eof };
struct Token {
    Tk t;
    std::string w;
    size_t line;
};
bool word_char(char c) { return isalnum((unsigned char)c) || c == '_' || c == '.' || c == '@' || c == '%' || c == '-' || c == '+'; }

std::vector<Token> lex(const char* s, size_t n) {
    std::vector<Token> out;
    size_t line = 1, i = 0;
    auto push = [&](Tk t) { out.push_back(Token{t, "", line}); };
    while (i < n) {
        char c = s[i];
        if (c == '\n') { line++; i++; continue; }
        if (isspace((unsigned char)c)) { i++; continue; }
        switch (c) {
            case '(': push(Tk::LParen); i++; continue;
            case ')': push(Tk::RParen); i++; continue;
            case '{': push(Tk::LBrace); i++; continue;
            case '}': push(Tk::RBrace); i++; continue;
            case '[': push(Tk::LBracket); i++; continue;
            case ']': push(Tk::RBracket); i++; continue;
            case ',': push(Tk::Comma); i++; continue;
            case ':': push(Tk::Colon); i++; continue;
            case '=': push(Tk::Eq); i++; continue;
            default: break;
        }
        if (c == '-' && i + 1 < n && s[i + 1] == '>') { push(Tk::Arrow); i += 2; continue; }
        size_t st = i;
        while (i < n && word_char(s[i])) i++;
        if (i == st) { i++; continue; }   // unknown punctuation: skipped, the parser reports the damage
        out.push_back(Token{Tk::Word, std::string(s + st, i - st), line});
    }
    out.push_back(Token{Tk::Eof, "", out.empty() ? line : out.back().line});
    return out;
}

struct Parser {
    std::vector<Token> toks;
    size_t pos = 0;
    ParseError err;
    bool failed = false;

    const Token& cur() const { return toks[pos]; }
    void bump() { if (pos + 1 < toks.size()) pos++; }
    bool fail(const std::string& m) {
        if (!failed) { failed = true; err.line = cur().line; err.msg = m; }
        return false;
    }
    bool is(Tk t) const { return cur().t == t; }
    bool peek_word(const char* w) const { return cur().t == Tk::Word && cur().w == w; }
    bool expect(Tk t, const char* what) {
        if (!is(t)) return fail(std::string("expected ") + what);
        bump();
        return true;
    }
    bool kw(const char* w) {
        if (!peek_word(w)) return fail(std::string("expected `") + w + "`");
        bump();
        return true;
    }
    bool word(std::string* out) {
        if (!is(Tk::Word)) return fail("expected a word");
        *out = cur().w;
        bump();
        return true;
    }
    bool ty(Ty* out) {
        std::string w;
        if (!word(&w)) return false;
        if (!parse_ty(w, out)) return fail("unknown type `" + w + "`");
        return true;
    }
    bool scalar(Scalar* out) {
        std::string w;
        if (!word(&w)) return false;
        if (!parse_scalar(w, out)) return fail("unknown scalar type `" + w + "`");
        return true;
    }
    bool val(Val* out) {
        std::string w;
        if (!word(&w)) return false;
        if (w.rfind("%arg", 0) == 0 && w.size() > 4) {
            uint32_t n = 0;
            auto r = std::from_chars(w.data() + 4, w.data() + w.size(), n);
            if (r.ec == std::errc() && r.ptr == w.data() + w.size()) { *out = Val::P(n); return true; }
        } else if (w.size() > 1 && w[0] == '%') {
            uint32_t n = 0;
            auto r = std::from_chars(w.data() + 1, w.data() + w.size(), n);
            if (r.ec == std::errc() && r.ptr == w.data() + w.size()) { *out = Val::V(n); return true; }
        }
        return fail("expected a value reference, found `" + w + "`");
    }
    bool block_id(uint32_t* out) {
        std::string w;
        if (!word(&w)) return false;
        if (w.size() > 2 && w[0] == 'b' && w[1] == 'b') {
            auto r = std::from_chars(w.data() + 2, w.data() + w.size(), *out);
            if (r.ec == std::errc() && r.ptr == w.data() + w.size()) return true;
        }
        return fail("expected a block label, found `" + w + "`");
    }
    bool u32(uint32_t* out) {
        std::string w;
        if (!word(&w)) return false;
        auto r = std::from_chars(w.data(), w.data() + w.size(), *out);
        if (r.ec != std::errc() || r.ptr != w.data() + w.size()) return fail("expected an integer, found `" + w + "`");
        return true;
    }
    bool i64(int64_t* out) {
        std::string w;
        if (!word(&w)) return false;
        const char* b = w.data();
        if (*b == '+') b++;
        auto r = std::from_chars(b, w.data() + w.size(), *out);
        if (r.ec != std::errc() || r.ptr != w.data() + w.size()) return fail("expected an integer, found `" + w + "`");
        return true;
    }
    bool f64(double* out) {
        std::string w;
        if (!word(&w)) return false;
        if (w == "inf" || w == "+inf" || w == "infinity") { *out = INFINITY; return true; }
        if (w == "-inf" || w == "-infinity") { *out = -INFINITY; return true; }
        if (w == "NaN" || w == "nan") { *out = NAN; return true; }
        const char* b = w.data();
        if (*b == '+') b++;
        auto r = std::from_chars(b, w.data() + w.size(), *out);
        if (r.ec != std::errc() || r.ptr != w.data() + w.size()) return fail("expected a float, found `" + w + "`");
        return true;
    }
    bool space(Space* out) {
        Ty t;
        size_t save_line = cur().line;
        if (!ty(&t)) return false;
        if (!t.is_ptr()) { failed = true; err.line = save_line; err.msg = "expected a pointer type"; return false; }
        *out = t.sp;
        return true;
    }
    bool val_list(std::vector<Val>* out) {
        if (!expect(Tk::LBracket, "`[`")) return false;
        if (!is(Tk::RBracket)) {
            for (;;) {
                Val v;
                if (!val(&v)) return false;
                out->push_back(v);
                if (is(Tk::Comma)) { bump(); continue; }
                break;
            }
        }
        return expect(Tk::RBracket, "`]`");
    }
    bool vals(Inst& in, int n) {
        for (int i = 0; i < n; i++) {
            if (i && !expect(Tk::Comma, "`,`")) return false;
            Val v;
            if (!val(&v)) return false;
            in.ops.push_back(v);
        }
        return true;
    }

    bool parse_op(const std::string& w, Inst& in) {
        int i;
        if ((i = find_in(kBin, w)) >= 0) { in.op = Opc::Bin; in.sub = (uint8_t)i; return ty(&in.ty) && vals(in, 2); }
        if ((i = find_in(kCast, w)) >= 0) { in.op = Opc::Cast; in.sub = (uint8_t)i; return ty(&in.ty) && ty(&in.aux) && vals(in, 1); }
        if ((i = find_in(kShfl, w)) >= 0) { in.op = Opc::Shuffle; in.sub = (uint8_t)i; return ty(&in.ty) && vals(in, 2); }
        if ((i = find_in(kAtom, w)) >= 0) { in.op = Opc::Atomic; in.sub = (uint8_t)i; return ty(&in.ty) && space(&in.space) && vals(in, 2); }
        if ((i = find_in(kIndex, w)) >= 0) { in.op = Opc::Index; in.sub = (uint8_t)i; return ty(&in.ty); }
        if ((i = find_in(kRed, w)) >= 0) { in.op = Opc::WarpReduce; in.sub = (uint8_t)i; return ty(&in.ty) && vals(in, 1); }
        if (w == "const.i") { in.op = Opc::ConstI; return ty(&in.ty) && i64(&in.imm); }
        if (w == "const.f") { in.op = Opc::ConstF; return ty(&in.ty) && f64(&in.fimm); }
        if (w == "icmp" || w == "fcmp") {
            std::string p;
            if (!word(&p)) return false;
            int pi = w == "icmp" ? find_in(kICmp, p) : find_in(kFCmp, p);
            if (pi < 0) return fail("unknown " + w + " predicate `" + p + "`");
            in.op = w == "icmp" ? Opc::ICmp : Opc::FCmp;
            in.sub = (uint8_t)pi;
            in.ty = Ty::s(Scalar::I1);
            return ty(&in.aux) && vals(in, 2);
        }
        if (w == "select") { in.op = Opc::Select; return ty(&in.ty) && vals(in, 3); }
        if (w == "load" || w == "store") {
            bool st = w == "store";
            in.op = st ? Opc::Store : Opc::Load;
            Ty t;
            if (!ty(&t) || !space(&in.space)) return false;
            if (st) { in.aux = t; in.ty = Ty::v(); } else in.ty = t;
            if (!vals(in, st ? 2 : 1)) return false;
            if (!expect(Tk::Comma, "`,`") || !kw("align") || !u32(&in.align)) return false;
            if (is(Tk::Comma)) { bump(); if (!kw("volatile")) return false; in.vol = true; }
            return true;
        }
        if (w == "phi") {
            in.op = Opc::Phi;
            if (!ty(&in.ty) || !expect(Tk::LBracket, "`[`")) return false;
            if (!is(Tk::RBracket)) {
                for (;;) {
                    uint32_t bb;
                    Val v;
                    if (!block_id(&bb) || !expect(Tk::Arrow, "`->`") || !val(&v)) return false;
                    in.phi_blocks.push_back(bb);
                    in.ops.push_back(v);
                    if (is(Tk::Comma)) { bump(); continue; }
                    break;
                }
            }
            return expect(Tk::RBracket, "`]`");
        }
        if (w == "barrier") { in.op = Opc::Barrier; in.ty = Ty::v(); return true; }
        if (w == "ballot" || w == "vote.any" || w == "vote.all") {
            in.op = w == "ballot" ? Opc::Ballot : w == "vote.any" ? Opc::VoteAny : Opc::VoteAll;
            return ty(&in.ty) && vals(in, 1);
        }
        if (w == "atomic.cas") { in.op = Opc::AtomicCas; return ty(&in.ty) && space(&in.space) && vals(in, 3); }
        if (w == "mma") {
            in.op = Opc::Mma;
            in.ty = Ty::v();
            std::string la, lb;
            if (!scalar(&in.in_dt) || !scalar(&in.acc_dt) || !word(&la) || !word(&lb)) return false;
            if ((la != "row" && la != "col") || (lb != "row" && lb != "col")) return fail("unknown mma layout");
            in.a_col = la == "col";
            in.b_col = lb == "col";
            if (!kw("m") || !u32(&in.m) || !kw("n") || !u32(&in.n) || !kw("k") || !u32(&in.k)) return false;
            if (peek_word("ld")) {
                bump();
                in.has_ld = true;
                for (int j = 0; j < 4; j++) if (!i64(&in.ld[j])) return false;
            }
            in.out_dt = in.acc_dt;
            if (peek_word("out")) { bump(); in.has_out = true; if (!scalar(&in.out_dt)) return false; }
            return vals(in, 4);
        }
        if (w == "kernel.launch") {
            in.op = Opc::KernelLaunch;
            in.ty = Ty::v();
            std::string nm;
            if (!word(&nm)) return false;
            if (nm.empty() || nm[0] != '@') return fail("expected `@name`");
            in.callee = nm.substr(1);
            if (!kw("grid") || !vals(in, 3) || !kw("block")) return false;
            for (int j = 0; j < 3; j++) {
                if (j && !expect(Tk::Comma, "`,`")) return false;
                Val v;
                if (!val(&v)) return false;
                in.ops.push_back(v);
            }
            Val v;
            if (!kw("shared") || !val(&v)) return false;
            in.ops.push_back(v);
            if (!kw("stream") || !val(&v)) return false;
            in.ops.push_back(v);
            return val_list(&in.ops);
        }
        if (w == "cuda.malloc") { in.op = Opc::CudaMalloc; return ty(&in.ty) && vals(in, 1); }
        if (w == "cuda.memcpy") { in.op = Opc::CudaMemcpy; in.ty = Ty::v(); return vals(in, 4); }
        if (w == "cuda.free") { in.op = Opc::CudaFree; in.ty = Ty::v(); return vals(in, 1); }
        if (w == "cuda.device_sync") { in.op = Opc::CudaSync; in.ty = Ty::v(); return true; }
        if (w == "call") {
            in.op = Opc::Call;
            std::string nm;
            if (!ty(&in.ty) || !word(&nm)) return false;
            if (nm.empty() || nm[0] != '@') return fail("expected `@name`");
            in.callee = nm.substr(1);
            return val_list(&in.ops);
        }
        if (w == "vec.extract") {
            in.op = Opc::VecExtract;
            uint32_t lane;
            if (!ty(&in.ty) || !vals(in, 1) || !expect(Tk::Comma, "`,`") || !u32(&lane)) return false;
            in.sub = (uint8_t)lane;
            return true;
        }
        if (w == "vec.build") { in.op = Opc::VecBuild; return ty(&in.ty) && val_list(&in.ops); }
        return fail("unknown opcode `" + w + "`");
    }

    bool parse_term(Term& t) {
        std::string w;
        if (!word(&w)) return false;
        if (w == "br") { t.kind = Term::Br; return block_id(&t.t); }
        if (w == "condbr") {
            t.kind = Term::CondBr;
            t.has_val = true;
            return val(&t.val) && expect(Tk::Comma, "`,`") && block_id(&t.t) && expect(Tk::Comma, "`,`") && block_id(&t.f);
        }
        if (w == "switch") {
            t.kind = Term::Switch;
            t.has_val = true;
            if (!val(&t.val) || !expect(Tk::Comma, "`,`") || !kw("default") || !block_id(&t.t) || !expect(Tk::LBracket, "`[`")) return false;
            if (!is(Tk::RBracket)) {
                for (;;) {
                    int64_t cv;
                    uint32_t bb;
                    if (!i64(&cv) || !expect(Tk::Arrow, "`->`") || !block_id(&bb)) return false;
                    t.cases.push_back({cv, bb});
                    if (is(Tk::Comma)) { bump(); continue; }
                    break;
                }
            }
            return expect(Tk::RBracket, "`]`");
        }
        if (w == "ret") {
            t.kind = Term::Ret;
            if (is(Tk::Word) && !cur().w.empty() && cur().w[0] == '%') { t.has_val = true; return val(&t.val); }
            return true;
        }
        return fail("expected a terminator, found `" + w + "`");
    }

    bool parse_func(Function& f) {
        f.is_kernel = true;
        if (peek_word("host")) { bump(); f.is_kernel = false; }
        std::string nm;
        if (!kw("func") || !word(&nm)) return false;
        if (nm.size() < 2 || nm[0] != '@') return fail("expected `@name`, found `" + nm + "`");
        f.name = nm.substr(1);
        if (!expect(Tk::LParen, "`(`")) return false;
        if (!is(Tk::RParen)) {
            for (;;) {
                Ty t;
                if (!ty(&t)) return false;
                f.params.push_back(t);
                if (is(Tk::Comma)) { bump(); continue; }
                break;
            }
        }
        if (!expect(Tk::RParen, "`)`") || !expect(Tk::Arrow, "`->`") || !ty(&f.ret) || !expect(Tk::LBrace, "`{`")) return false;
        while (!is(Tk::RBrace)) {
            uint32_t bb;
            if (!block_id(&bb)) return false;
            if (bb != f.blocks.size()) return fail("block label bb" + std::to_string(bb) + " out of order, expected bb" + std::to_string(f.blocks.size()));
            if (!expect(Tk::Colon, "`:`")) return false;
            Block blk;
            for (;;) {
                if (!is(Tk::Word)) return fail("unexpected end of input inside a block");
                const std::string& w = cur().w;
                if (w == "br" || w == "condbr" || w == "switch" || w == "ret") break;
                bool prefix = w[0] == '%' && pos + 1 < toks.size() && toks[pos + 1].t == Tk::Eq;
                uint32_t id = (uint32_t)f.insts.size();
                if (prefix) {
                    uint32_t n = 0;
                    auto r = std::from_chars(w.data() + 1, w.data() + w.size(), n);
                    if (r.ec != std::errc() || r.ptr != w.data() + w.size()) return fail("bad value name `" + w + "`");
                    if (n != id) return fail("value %" + std::to_string(n) + " out of order, expected %" + std::to_string(id));
                    bump();
                    bump();
                }
                std::string opw;
                if (!word(&opw)) return false;
                Inst in;
                if (!parse_op(opw, in)) return false;
                if (prefix != in.has_result())
                    return fail("`" + opw + "` " + (in.has_result() ? "produces" : "does not produce") + " a result but " + (prefix ? "one was named" : "none was named"));
                f.insts.push_back(std::move(in));
                blk.insts.push_back(id);
            }
            if (!parse_term(blk.term)) return false;
            f.blocks.push_back(std::move(blk));
        }
        return expect(Tk::RBrace, "`}`");
    }

    bool parse_mod(Module& m) {
        if (!kw("module") || !expect(Tk::LBrace, "`{`")) return false;
        if (peek_word("launch_bounds")) {
            bump();
            m.has_launch_bounds = true;
            if (!kw("max_threads") || !expect(Tk::Eq, "`=`") || !u32(&m.max_threads)) return false;
            if (!kw("min_blocks") || !expect(Tk::Eq, "`=`") || !u32(&m.min_blocks)) return false;
        }
        if (!kw("shared_mem_bytes") || !u32(&m.shared_mem_bytes) || !kw("target_dtypes")) return false;
        while (is(Tk::Word)) {
            Scalar s;
            if (!parse_scalar(cur().w, &s)) break;
            m.target_dtypes.push_back(s);
            bump();
        }
        while (peek_word("shared_obj")) {
            bump();
            SharedObj so;
            if (!i64(&so.key) || !kw("bytes") || !u32(&so.bytes) || !kw("align") || !u32(&so.align)) return false;
            m.shared_objs.push_back(so);
        }
        while (peek_word("func") || peek_word("host")) {
            Function f;
            if (!parse_func(f)) return false;
            m.funcs.push_back(std::move(f));
        }
        if (!expect(Tk::RBrace, "`}`")) return false;
        if (!is(Tk::Eof)) return fail("trailing input after the module");
        return true;
    }
};
}  // namespace

bool parse_module(const char* src, size_t len, Module* out, ParseError* err) {
    Parser p;
    p.toks = lex(src, len);
    Module m;
    if (!p.parse_mod(m)) {
        if (err) *err = p.err;
        return false;
    }
    *out = std::move(m);
    return true;
}

// ---- printer -------------------------------------------------------------------------------
static std::string val_text(Val v) { return (v.param ? "%arg" : "%") + std::to_string(v.idx); }

// Shortest decimal that parses back to the same double, never in exponent form: what Rust's `{}`
// prints for an f64 (crates/basalt-bir/src/print.rs:88-90).
static std::string f64_text(double d) {
    if (std::isnan(d)) return "NaN";
    if (std::isinf(d)) return d < 0 ? "-inf" : "inf";
    char buf[1100];
    auto r = std::to_chars(buf, buf + sizeof buf, d, std::chars_format::fixed);
    return std::string(buf, r.ptr);
}

static void print_inst(std::string& o, const Inst& in) {
    auto v = [&](size_t i) { return val_text(in.ops[i]); };
    auto list = [&](size_t from) {
        o += "[";
        for (size_t i = from; i < in.ops.size(); i++) { if (i > from) o += ", "; o += v(i); }
        o += "]";
    };
    std::string ty = ty_text(in.ty);
    switch (in.op) {
        case Opc::ConstI: o += "const.i " + ty + " " + std::to_string(in.imm); break;
        case Opc::ConstF: o += "const.f " + ty + " " + f64_text(in.fimm); break;
        case Opc::Bin: o += std::string(kBin[in.sub]) + " " + ty + " " + v(0) + ", " + v(1); break;
        case Opc::ICmp: o += std::string("icmp ") + kICmp[in.sub] + " " + ty_text(in.aux) + " " + v(0) + ", " + v(1); break;
        case Opc::FCmp: o += std::string("fcmp ") + kFCmp[in.sub] + " " + ty_text(in.aux) + " " + v(0) + ", " + v(1); break;
        case Opc::Select: o += "select " + ty + " " + v(0) + ", " + v(1) + ", " + v(2); break;
        case Opc::Cast: o += std::string(kCast[in.sub]) + " " + ty + " " + ty_text(in.aux) + " " + v(0); break;
        case Opc::Load:
            o += "load " + ty + " ptr." + space_text(in.space) + " " + v(0) + ", align " + std::to_string(in.align);
            if (in.vol) o += ", volatile";
            break;
        case Opc::Store:
            o += "store " + ty_text(in.aux) + " ptr." + space_text(in.space) + " " + v(0) + ", " + v(1) + ", align " + std::to_string(in.align);
            if (in.vol) o += ", volatile";
            break;
        case Opc::Phi:
            o += "phi " + ty + " [";
            for (size_t i = 0; i < in.ops.size(); i++) {
                if (i) o += ", ";
                o += "bb" + std::to_string(in.phi_blocks[i]) + " -> " + v(i);
            }
            o += "]";
            break;
        case Opc::Index: o += std::string(kIndex[in.sub]) + " " + ty; break;
        case Opc::Barrier: o += "barrier"; break;
        case Opc::Shuffle: o += std::string(kShfl[in.sub]) + " " + ty + " " + v(0) + ", " + v(1); break;
        case Opc::Ballot: o += "ballot " + ty + " " + v(0); break;
        case Opc::VoteAny: o += "vote.any " + ty + " " + v(0); break;
        case Opc::VoteAll: o += "vote.all " + ty + " " + v(0); break;
        case Opc::Atomic: o += std::string(kAtom[in.sub]) + " " + ty + " ptr." + space_text(in.space) + " " + v(0) + ", " + v(1); break;
        case Opc::AtomicCas: o += "atomic.cas " + ty + " ptr." + space_text(in.space) + " " + v(0) + ", " + v(1) + ", " + v(2); break;
        case Opc::Mma:
            o += std::string("mma ") + scalar_text(in.in_dt) + " " + scalar_text(in.acc_dt) + " " + (in.a_col ? "col" : "row") + " " + (in.b_col ? "col" : "row") +
                 " m " + std::to_string(in.m) + " n " + std::to_string(in.n) + " k " + std::to_string(in.k);
            if (in.has_ld) for (int j = 0; j < 4; j++) o += (j ? " " : " ld ") + std::to_string(in.ld[j]);
            if (in.has_out) o += std::string(" out ") + scalar_text(in.out_dt);
            o += " " + v(0) + ", " + v(1) + ", " + v(2) + ", " + v(3);
            break;
        case Opc::KernelLaunch:
            o += "kernel.launch @" + in.callee + " grid " + v(0) + ", " + v(1) + ", " + v(2) + " block " + v(3) + ", " + v(4) + ", " + v(5) + " shared " + v(6) + " stream " + v(7) + " ";
            list(8);
            break;
        case Opc::CudaMalloc: o += "cuda.malloc " + ty + " " + v(0); break;
        case Opc::CudaMemcpy: o += "cuda.memcpy " + v(0) + ", " + v(1) + ", " + v(2) + ", " + v(3); break;
        case Opc::CudaFree: o += "cuda.free " + v(0); break;
        case Opc::CudaSync: o += "cuda.device_sync"; break;
        case Opc::Call: o += "call " + ty + " @" + in.callee + " "; list(0); break;
        case Opc::VecExtract: o += "vec.extract " + ty + " " + v(0) + ", " + std::to_string((unsigned)in.sub); break;
        case Opc::VecBuild: o += "vec.build " + ty + " "; list(0); break;
        case Opc::WarpReduce: o += std::string(kRed[in.sub]) + " " + ty + " " + v(0); break;
    }
}

std::string print_module(const Module& m) {
    std::string o = "module {\n";
    if (m.has_launch_bounds)
        o += "  launch_bounds max_threads=" + std::to_string(m.max_threads) + " min_blocks=" + std::to_string(m.min_blocks) + "\n";
    o += "  shared_mem_bytes " + std::to_string(m.shared_mem_bytes) + "\n  target_dtypes";
    for (Scalar s : m.target_dtypes) o += std::string(" ") + scalar_text(s);
    o += "\n";
    for (auto& so : m.shared_objs)
        o += "  shared_obj " + std::to_string(so.key) + " bytes " + std::to_string(so.bytes) + " align " + std::to_string(so.align) + "\n";
    for (auto& f : m.funcs) {
        o += "\n  ";
        if (!f.is_kernel) o += "host ";
        o += "func @" + f.name + "(";
        for (size_t i = 0; i < f.params.size(); i++) { if (i) o += ", "; o += ty_text(f.params[i]); }
        o += ") -> " + ty_text(f.ret) + " {\n";
        for (size_t b = 0; b < f.blocks.size(); b++) {
            o += "  bb" + std::to_string(b) + ":\n";
            for (uint32_t id : f.blocks[b].insts) {
                o += "    ";
                if (f.insts[id].has_result()) o += "%" + std::to_string(id) + " = ";
                print_inst(o, f.insts[id]);
                o += "\n";
            }
            const Term& t = f.blocks[b].term;
            o += "    ";
            switch (t.kind) {
                case Term::Br: o += "br bb" + std::to_string(t.t); break;
                case Term::CondBr: o += "condbr " + val_text(t.val) + ", bb" + std::to_string(t.t) + ", bb" + std::to_string(t.f); break;
                case Term::Switch:
                    o += "switch " + val_text(t.val) + ", default bb" + std::to_string(t.t) + " [";
                    for (size_t i = 0; i < t.cases.size(); i++) {
                        if (i) o += ", ";
                        o += std::to_string(t.cases[i].first) + " -> bb" + std::to_string(t.cases[i].second);
                    }
                    o += "]";
                    break;
                case Term::Ret: o += t.has_val ? "ret " + val_text(t.val) : "ret"; break;
            }
            o += "\n";
        }
        o += "  }\n";
    }
    o += "}\n";
    return o;
}

// ---- verifier ------------------------------------------------------------------------------
bool verify_module(const Module& m, std::string* why) {
    auto bad = [&](const Function& f, const std::string& s) {
        if (why) *why = "@" + f.name + ": " + s;
        return false;
    };
    for (auto& f : m.funcs) {
        if (f.blocks.empty()) return bad(f, "function has no blocks");
        std::vector<char> listed(f.insts.size(), 0);
        for (auto& b : f.blocks)
            for (uint32_t id : b.insts) {
                if (id >= f.insts.size()) return bad(f, "block lists an instruction outside the arena");
                if (listed[id]) return bad(f, "instruction %" + std::to_string(id) + " is listed twice");
                listed[id] = 1;
            }
        auto ok_val = [&](Val v) { return v.param ? v.idx < f.params.size() : (v.idx < f.insts.size() && f.insts[v.idx].has_result()); };
        for (size_t i = 0; i < f.insts.size(); i++) {
            const Inst& in = f.insts[i];
            for (Val v : in.ops)
                if (!ok_val(v)) return bad(f, "%" + std::to_string(i) + " uses an undefined value");
            if (in.op == Opc::Phi) {
                if (in.phi_blocks.size() != in.ops.size()) return bad(f, "phi arity mismatch");
                for (uint32_t b : in.phi_blocks)
                    if (b >= f.blocks.size()) return bad(f, "phi names a missing block");
            }
            if (in.op == Opc::VecExtract) {
                Ty vt = f.val_ty(in.ops[0]);
                if (!vt.is_vec() || in.sub >= vt.lanes) return bad(f, "vec.extract lane out of range");
            }
            if (in.op == Opc::VecBuild && (!in.ty.is_vec() || in.ops.size() != in.ty.lanes)) return bad(f, "vec.build arity mismatch");
        }
        for (auto& b : f.blocks) {
            const Term& t = b.term;
            if (t.has_val && !ok_val(t.val)) return bad(f, "terminator uses an undefined value");
            if (t.kind != Term::Ret && t.t >= f.blocks.size()) return bad(f, "branch to a missing block");
            if (t.kind == Term::CondBr && t.f >= f.blocks.size()) return bad(f, "branch to a missing block");
            for (auto& c : t.cases)
                if (c.second >= f.blocks.size()) return bad(f, "switch case names a missing block");
        }
    }
    return true;
}

void canonicalize(Function& f) {
    std::vector<uint32_t> remap(f.insts.size(), UINT32_MAX);
    std::vector<Inst> arena;
    arena.reserve(f.insts.size());
    for (auto& b : f.blocks)
        for (uint32_t& id : b.insts) {
            remap[id] = (uint32_t)arena.size();
            arena.push_back(std::move(f.insts[id]));
            id = remap[id];
        }
    auto fix = [&](Val& v) { if (!v.param) v.idx = remap[v.idx]; };
    for (auto& in : arena) for (Val& v : in.ops) fix(v);
    for (auto& b : f.blocks) if (b.term.has_val) fix(b.term.val);
    f.insts = std::move(arena);
}

}  // namespace basalt
