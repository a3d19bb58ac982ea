// Generic BIR -> PTX lowering for sm_100a.
//
// Follows the reference emitter's contract op by op (crates/basalt-ptx/src/emit.rs:810-1892):
// the same mnemonic families, signed div/rem and atomic min/max, full-mask `.sync` warp
// collectives, phi resolution by moves on the incoming edge.  Differences, all deliberate:
//   * `.version 8.7 / .target sm_100a` instead of 8.0 / sm_70 (emit.rs:1956-1960);
//   * f32/f64 add, sub and mul carry an explicit `.rn` so ptxas never contracts them into an
//     fma: the CPU oracle multiplies and adds separately (crates/basalt-x86/src/oracle.rs:1530-1543)
//     and float known-answer fixtures are compared bit for bit;
//   * i8/i16 values are kept sign-extended in their 32-bit register (the reference re-extends at
//     each use, emit.rs:966-986); shift counts are masked as x86 does so results match the oracle;
//   * f16 is lowered (load/store/convert natively, arithmetic through f32 with one rounding);
//   * an atomic whose result is unused becomes `red`; `warp.reduce` becomes `redux.sync`;
//   * a sized `shared_obj` becomes a real `.shared` array; unsized synthetic addresses keep the
//     reference's 8-byte cell (emit.rs:630-660, 1929-1934);
//   * phi moves go through temporaries when one phi of a block feeds another (swap problem).
#include "emit.hpp"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <set>

namespace basalt {
namespace {

enum Cls { P, R, RD, F, FD, H, NCLS };
const char* kClsPrefix[NCLS] = {"%p", "%r", "%rd", "%f", "%fd", "%h"};
const char* kClsDecl[NCLS] = {".pred", ".b32", ".b64", ".f32", ".f64", ".b16"};

Cls cls_of(Scalar s) {
    switch (s) {
        case Scalar::I1: return P;
        case Scalar::I8: case Scalar::I16: case Scalar::I32: return R;
        case Scalar::I64: return RD;
        case Scalar::F16: return H;
        case Scalar::F32: return F;
        case Scalar::F64: return FD;
    }
    return R;
}

uint16_t f64_to_f16_bits(double d) {
    uint64_t b;
    memcpy(&b, &d, 8);
    uint16_t sign = (uint16_t)((b >> 48) & 0x8000u);
    int exp = (int)((b >> 52) & 0x7ff);
    uint64_t man = b & 0xFFFFFFFFFFFFFull;
    if (exp == 0x7ff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
    if (exp == 0 && man == 0) return sign;
    int e = exp - 1023;
    uint64_t sig = man | (1ull << 52);
    int shift = e < -14 ? 28 - e : 42;
    if (shift > 63) return sign;
    uint64_t q = sig >> shift, rem = sig & ((1ull << shift) - 1), half = 1ull << (shift - 1);
    if (rem > half || (rem == half && (q & 1))) q++;
    uint32_t out = e < -14 ? (uint32_t)q : (uint32_t)(((uint32_t)(e + 14) << 10) + q);
    if (out >= 0x7c00u) out = 0x7c00u;
    return (uint16_t)(sign | out);
}

std::string hex32(uint32_t v) { char b[16]; snprintf(b, sizeof b, "%08X", v); return b; }
std::string hex64(uint64_t v) { char b[24]; snprintf(b, sizeof b, "%016llX", (unsigned long long)v); return b; }

const char* space_word(Space s) {
    switch (s) {
        case Space::Global: return "global";
        case Space::Shared: return "shared";
        case Space::Constant: return "local";   // synthetic cells only; see LocalSlots in the reference
        case Space::Local: return "local";
        case Space::Param: return "local";
    }
    return "global";
}

struct FnEmitter {
    const Module& mod;
    const Function& f;
    std::vector<std::string> body, decls, plan, extra_params, module_decls;
    int counts[NCLS] = {0, 0, 0, 0, 0, 0};
    std::map<uint32_t, std::vector<std::string>> regs;    // inst id -> registers (one per lane)
    std::vector<std::vector<std::string>> param_regs;
    std::map<std::pair<int, int64_t>, std::string> cells; // (space, key) -> symbol
    std::vector<uint32_t> uses;
    int label_n = 0, mma_n = 0;
    unsigned maxntid = 0, cluster = 0, tmem_cols = 0;
    bool pair_twin = false;   // emitting `<name>__pair`: the mma must take the two-SM lowering
    int est_regs = 0, budget = 0;   // the register-budget pass's figures for this body (set by run)
    bool capped = false;            // run emitted .maxnreg
    Diag diag;
    bool failed = false;

    FnEmitter(const Module& m, const Function& fn, bool pair = false) : mod(m), f(fn), pair_twin(pair) {}

    std::string fresh(Cls c) { return kClsPrefix[c] + std::to_string(counts[c]++); }
    void line(const std::string& s) { body.push_back("\t" + s); }
    void label(const std::string& s) { body.push_back(s + ":"); }
    std::string fresh_label(const char* stem) { return "$" + std::string(stem) + "_" + std::to_string(label_n++); }
    bool fail(const char* code, const std::string& why) {
        if (!failed) { failed = true; diag.code = code; diag.arg = why; }
        return false;
    }

    Cls cls(Ty t) const {
        if (t.is_ptr()) return RD;
        return cls_of(t.sc);
    }
    std::vector<std::string> alloc(Ty t) {
        std::vector<std::string> out;
        int n = t.is_vec() ? t.lanes : 1;
        for (int i = 0; i < n; i++) out.push_back(fresh(cls(t)));
        return out;
    }
    const std::vector<std::string>& vregs(Val v) {
        if (v.param) return param_regs[v.idx];
        auto it = regs.find(v.idx);
        if (it != regs.end()) return it->second;
        const Inst& in = f.insts[v.idx];
        if (in.op == Opc::VecExtract) {
            std::vector<std::string> r{vregs(in.ops[0])[in.sub]};
            return regs[v.idx] = r;
        }
        if (in.op == Opc::VecBuild) {
            std::vector<std::string> r;
            for (Val o : in.ops) r.push_back(vregs(o)[0]);
            return regs[v.idx] = r;
        }
        return regs[v.idx] = alloc(in.ty);
    }
    const std::string& reg(Val v) { return vregs(v)[0]; }
    Ty ty(Val v) const { return f.val_ty(v); }

    std::string cell_symbol(Space sp, int64_t key) {
        auto k = std::make_pair((int)sp, key);
        auto it = cells.find(k);
        if (it != cells.end()) return it->second;
        std::string sym;
        if (sp == Space::Shared) {
            uint32_t bytes = 8, align = 8;
            for (auto& so : mod.shared_objs) if (so.key == key) { bytes = so.bytes; align = so.align ? so.align : 8; }
            sym = "__shared_" + std::to_string(cells.size());
            decls.push_back("\t.shared .align " + std::to_string(align) + " .b8 " + sym + "[" + std::to_string(bytes) + "];");
        } else {
            sym = "__local_" + std::to_string(cells.size());
            decls.push_back("\t.local .align 8 .b8 " + sym + "[8];");
        }
        return cells[k] = sym;
    }

    // ---- parameters ------------------------------------------------------------------------
    std::string param_name(size_t i) const { return f.name + "_param_" + std::to_string(i); }
    std::string param_decl(size_t i) const {
        Ty t = f.params[i];
        std::string n = param_name(i);
        if (t.is_ptr()) return ".param .u64 " + n;
        if (t.is_vec()) {
            unsigned bytes = t.lanes * scalar_bytes(t.sc);
            return ".param .align " + std::to_string(bytes > 16 ? 16 : bytes) + " .b8 " + n + "[" + std::to_string(bytes) + "]";
        }
        switch (t.sc) {
            case Scalar::I1: case Scalar::I8: return ".param .u8 " + n;
            case Scalar::I16: return ".param .u16 " + n;
            case Scalar::I32: return ".param .u32 " + n;
            case Scalar::I64: return ".param .u64 " + n;
            case Scalar::F16: return ".param .b16 " + n;
            case Scalar::F32: return ".param .f32 " + n;
            case Scalar::F64: return ".param .f64 " + n;
        }
        return "";
    }
    void load_scalar_param(Scalar s, const std::string& dst, const std::string& addr) {
        switch (s) {
            case Scalar::I1: {
                std::string t = fresh(R);
                line("ld.param.u8 " + t + ", [" + addr + "];");
                line("setp.ne.u32 " + dst + ", " + t + ", 0;");
                break;
            }
            case Scalar::I8: line("ld.param.s8 " + dst + ", [" + addr + "];"); break;
            case Scalar::I16: line("ld.param.s16 " + dst + ", [" + addr + "];"); break;
            case Scalar::I32: line("ld.param.u32 " + dst + ", [" + addr + "];"); break;
            case Scalar::I64: line("ld.param.u64 " + dst + ", [" + addr + "];"); break;
            case Scalar::F16: line("ld.param.b16 " + dst + ", [" + addr + "];"); break;
            case Scalar::F32: line("ld.param.f32 " + dst + ", [" + addr + "];"); break;
            case Scalar::F64: line("ld.param.f64 " + dst + ", [" + addr + "];"); break;
        }
    }
    void emit_param_loads() {
        for (size_t i = 0; i < f.params.size(); i++) {
            Ty t = f.params[i];
            param_regs.push_back(alloc(t));
            if (t.is_ptr()) line("ld.param.u64 " + param_regs[i][0] + ", [" + param_name(i) + "];");
            else if (t.is_vec())
                for (unsigned l = 0; l < t.lanes; l++) load_scalar_param(t.sc, param_regs[i][l], param_name(i) + "+" + std::to_string(l * scalar_bytes(t.sc)));
            else load_scalar_param(t.sc, param_regs[i][0], param_name(i));
        }
    }

    // ---- helpers ---------------------------------------------------------------------------
    // Re-establishes the "sign-extended in 32 bits" invariant of an i8/i16 value held in `r`.
    void canon(Scalar s, const std::string& r) {
        if (s == Scalar::I8) line("bfe.s32 " + r + ", " + r + ", 0, 8;");
        else if (s == Scalar::I16) line("bfe.s32 " + r + ", " + r + ", 0, 16;");
    }
    // Zero-extended copy of a narrow value (for unsigned compares, lshr, zext, uitofp).
    std::string zx(Scalar s, const std::string& r) {
        if (s != Scalar::I8 && s != Scalar::I16) return r;
        std::string t = fresh(R);
        line("and.b32 " + t + ", " + r + ", " + (s == Scalar::I8 ? "255" : "65535") + ";");
        return t;
    }
    std::string as_pred(Val v) {   // i1 -> predicate; any other integer -> (v != 0)
        Ty t = ty(v);
        if (t.is_sc(Scalar::I1)) return reg(v);
        std::string p = fresh(P);
        if (cls(t) == RD) line("setp.ne.u64 " + p + ", " + reg(v) + ", 0;");
        else line("setp.ne.u32 " + p + ", " + reg(v) + ", 0;");
        return p;
    }
    std::string f16_to_f32(const std::string& h) { std::string t = fresh(F); line("cvt.f32.f16 " + t + ", " + h + ";"); return t; }

    // ---- per-op lowering -------------------------------------------------------------------
    void lower_const_i(uint32_t id, const Inst& in) {
        const std::string& d = reg(Val::V(id));
        if (in.ty.is_ptr()) {
            if (in.ty.sp == Space::Global) line("mov.u64 " + d + ", " + std::to_string(in.imm) + ";");
            else line("mov.u64 " + d + ", " + cell_symbol(in.ty.sp, in.imm) + ";");
            return;
        }
        switch (in.ty.sc) {
            case Scalar::I1: line("setp.ne.u32 " + d + ", " + std::to_string(in.imm & 1) + ", 0;"); break;
            case Scalar::I8: line("mov.u32 " + d + ", " + std::to_string((int32_t)(int8_t)in.imm) + ";"); break;
            case Scalar::I16: line("mov.u32 " + d + ", " + std::to_string((int32_t)(int16_t)in.imm) + ";"); break;
            case Scalar::I32: line("mov.u32 " + d + ", " + std::to_string((int32_t)in.imm) + ";"); break;
            case Scalar::I64: line("mov.u64 " + d + ", " + std::to_string(in.imm) + ";"); break;
            default: fail("E091", "const.i on a float type");
        }
    }
    void lower_const_f(uint32_t id, const Inst& in) {
        const std::string& d = reg(Val::V(id));
        if (in.ty.is_sc(Scalar::F32)) { float v = (float)in.fimm; uint32_t b; memcpy(&b, &v, 4); line("mov.f32 " + d + ", 0f" + hex32(b) + ";"); }
        else if (in.ty.is_sc(Scalar::F64)) { uint64_t b; memcpy(&b, &in.fimm, 8); line("mov.f64 " + d + ", 0d" + hex64(b) + ";"); }
        else if (in.ty.is_sc(Scalar::F16)) line("mov.b16 " + d + ", " + std::to_string(f64_to_f16_bits(in.fimm)) + ";");
        else fail("E091", "const.f on a non-float type");
    }

    void bin_scalar(BinOp op, Scalar s, const std::string& d, const std::string& a, const std::string& b) {
        Cls c = cls_of(s);
        if (c == P) {
            const char* m = op == BinOp::And ? "and" : op == BinOp::Or ? "or" : "xor";
            line(std::string(m) + ".pred " + d + ", " + a + ", " + b + ";");
            return;
        }
        if (c == F || c == FD || c == H) {
            if (c == H) {   // widen, operate in f32, round once
                std::string x = f16_to_f32(a), y = f16_to_f32(b), r = fresh(F);
                bin_scalar(op, Scalar::F32, r, x, y);
                line("cvt.rn.f16.f32 " + d + ", " + r + ";");
                return;
            }
            std::string t = c == F ? "f32" : "f64";
            switch (op) {
                case BinOp::FAdd: line("add.rn." + t + " " + d + ", " + a + ", " + b + ";"); return;
                case BinOp::FSub: line("sub.rn." + t + " " + d + ", " + a + ", " + b + ";"); return;
                case BinOp::FMul: line("mul.rn." + t + " " + d + ", " + a + ", " + b + ";"); return;
                case BinOp::FDiv: line("div.rn." + t + " " + d + ", " + a + ", " + b + ";"); return;
                case BinOp::FRem: {   // a - trunc(a/b)*b, each step rounded (oracle.rs:1618-1627)
                    std::string q = fresh(c), tr = fresh(c), pr = fresh(c);
                    line("div.rn." + t + " " + q + ", " + a + ", " + b + ";");
                    line("cvt.rzi." + t + "." + t + " " + tr + ", " + q + ";");
                    line("mul.rn." + t + " " + pr + ", " + tr + ", " + b + ";");
                    line("sub.rn." + t + " " + d + ", " + a + ", " + pr + ";");
                    return;
                }
                default: fail("E090", "integer operator on a float type"); return;
            }
        }
        bool w64 = c == RD;
        std::string sfx = w64 ? "64" : "32";
        auto shift_count = [&]() {   // x86 masks the count in cl; 32-bit register in PTX either way
            std::string cnt = fresh(R);
            if (w64) { line("cvt.u32.u64 " + cnt + ", " + b + ";"); line("and.b32 " + cnt + ", " + cnt + ", 63;"); }
            else line("and.b32 " + cnt + ", " + b + ", 31;");
            return cnt;
        };
        switch (op) {
            case BinOp::Add: line("add.s" + sfx + " " + d + ", " + a + ", " + b + ";"); break;
            case BinOp::Sub: line("sub.s" + sfx + " " + d + ", " + a + ", " + b + ";"); break;
            case BinOp::Mul: line("mul.lo.s" + sfx + " " + d + ", " + a + ", " + b + ";"); break;
            case BinOp::Div: line("div.s" + sfx + " " + d + ", " + a + ", " + b + ";"); break;
            case BinOp::Rem: line("rem.s" + sfx + " " + d + ", " + a + ", " + b + ";"); break;
            case BinOp::And: line("and.b" + sfx + " " + d + ", " + a + ", " + b + ";"); return;
            case BinOp::Or: line("or.b" + sfx + " " + d + ", " + a + ", " + b + ";"); return;
            case BinOp::Xor: line("xor.b" + sfx + " " + d + ", " + a + ", " + b + ";"); return;
            case BinOp::Shl: line("shl.b" + sfx + " " + d + ", " + a + ", " + shift_count() + ";"); break;
            case BinOp::LShr: line("shr.u" + sfx + " " + d + ", " + zx(s, a) + ", " + shift_count() + ";"); break;
            case BinOp::AShr: line("shr.s" + sfx + " " + d + ", " + a + ", " + shift_count() + ";"); return;
            default: fail("E090", "float operator on an integer type"); return;
        }
        canon(s, d);
    }
    void lower_bin(uint32_t id, const Inst& in) {
        BinOp op = (BinOp)in.sub;
        if (in.ty.is_ptr()) {   // pointer arithmetic shares the 64-bit class (emit.rs:1055-1083)
            bin_scalar(op, Scalar::I64, reg(Val::V(id)), reg(in.ops[0]), reg(in.ops[1]));
            return;
        }
        auto& d = vregs(Val::V(id));
        auto& a = vregs(in.ops[0]);
        auto& b = vregs(in.ops[1]);
        // A 32- or 64-bit multiply by a constant power of two is a shift.  ptxas keeps `mul.lo` as a multiply-add pipe
        // instruction (three of them for a 64-bit product); in a kernel that is bound by that pipe -- the helper chain --
        // the index arithmetic of the vectorised loop then takes 4 % of it (32.7 -> 34.0 T int-op/s with shifts).
        if (op == BinOp::Mul && (in.ty.sc == Scalar::I32 || in.ty.sc == Scalar::I64)) {
            for (int k = 0; k < 2; k++) {
                const Val c = in.ops[k];
                if (c.param || f.insts[c.idx].op != Opc::ConstI) continue;
                const uint64_t v = in.ty.sc == Scalar::I32 ? (uint64_t)(uint32_t)f.insts[c.idx].imm : (uint64_t)f.insts[c.idx].imm;
                if (v < 2 || (v & (v - 1)) != 0) continue;
                int sh = 0;
                while ((v >> sh) != 1) sh++;
                auto& x = k == 0 ? b : a;
                for (size_t l = 0; l < d.size(); l++)
                    line(std::string("shl.b") + (in.ty.sc == Scalar::I64 ? "64 " : "32 ") + d[l] + ", " + x[l] + ", " + std::to_string(sh) + ";");
                return;
            }
        }
        for (size_t l = 0; l < d.size(); l++) bin_scalar(op, in.ty.sc, d[l], a[l], b[l]);
    }

    void lower_icmp(uint32_t id, const Inst& in) {
        ICmp p = (ICmp)in.sub;
        const std::string& d = reg(Val::V(id));
        static const char* sfx[] = {"eq", "ne", "lt", "le", "gt", "ge", "lt", "le", "gt", "ge"};
        bool is_signed = p <= ICmp::Sge;
        Ty ot = in.aux;
        if (ot.is_sc(Scalar::I1)) {
            if (p == ICmp::Ne) line("xor.pred " + d + ", " + reg(in.ops[0]) + ", " + reg(in.ops[1]) + ";");
            else if (p == ICmp::Eq) { line("xor.pred " + d + ", " + reg(in.ops[0]) + ", " + reg(in.ops[1]) + ";"); line("not.pred " + d + ", " + d + ";"); }
            else fail("E091", "ordered compare of predicates");
            return;
        }
        if (ot.is_ptr() || ot.is_sc(Scalar::I64)) {
            bool sg = is_signed && !ot.is_ptr() && p != ICmp::Eq && p != ICmp::Ne;
            line(std::string("setp.") + sfx[(int)p] + (sg ? ".s64 " : ".u64 ") + d + ", " + reg(in.ops[0]) + ", " + reg(in.ops[1]) + ";");
            return;
        }
        std::string a = reg(in.ops[0]), b = reg(in.ops[1]);
        if (!is_signed) { a = zx(ot.sc, a); b = zx(ot.sc, b); }
        line(std::string("setp.") + sfx[(int)p] + (is_signed ? ".s32 " : ".u32 ") + d + ", " + a + ", " + b + ";");
    }
    void lower_fcmp(uint32_t id, const Inst& in) {
        static const char* sfx[] = {"eq", "ne", "lt", "le", "gt", "ge", "num", "nan"};
        std::string a = reg(in.ops[0]), b = reg(in.ops[1]), t = "f32";
        if (in.aux.is_sc(Scalar::F16)) { a = f16_to_f32(a); b = f16_to_f32(b); }
        else if (in.aux.is_sc(Scalar::F64)) t = "f64";
        line(std::string("setp.") + sfx[in.sub] + "." + t + " " + reg(Val::V(id)) + ", " + a + ", " + b + ";");
    }
    void lower_select(uint32_t id, const Inst& in) {
        std::string c = as_pred(in.ops[0]);
        auto& d = vregs(Val::V(id));
        auto& a = vregs(in.ops[1]);
        auto& b = vregs(in.ops[2]);
        Cls k = cls(in.ty);
        for (size_t l = 0; l < d.size(); l++) {
            if (k == P) {
                std::string t1 = fresh(P), t2 = fresh(P), nc = fresh(P);
                line("and.pred " + t1 + ", " + c + ", " + a[l] + ";");
                line("not.pred " + nc + ", " + c + ";");
                line("and.pred " + t2 + ", " + nc + ", " + b[l] + ";");
                line("or.pred " + d[l] + ", " + t1 + ", " + t2 + ";");
            } else {
                const char* t = k == R ? "b32" : k == RD ? "b64" : k == F ? "f32" : k == FD ? "f64" : "b16";
                line(std::string("selp.") + t + " " + d[l] + ", " + a[l] + ", " + b[l] + ", " + c + ";");
            }
        }
    }

    void cast_scalar(CastOp op, Scalar ds, bool dptr, Scalar ss, bool sptr, const std::string& d, const std::string& a) {
        Cls dc = dptr ? RD : cls_of(ds), sc = sptr ? RD : cls_of(ss);
        auto fty = [](Cls c) { return c == F ? "f32" : c == FD ? "f64" : "f16"; };
        switch (op) {
            case CastOp::Trunc: {
                std::string lo = a;
                if (sc == RD && dc != RD) { lo = fresh(R); line("cvt.u32.u64 " + lo + ", " + a + ";"); }
                if (dc == P) {
                    std::string t = fresh(R);
                    line("and.b32 " + t + ", " + lo + ", 1;");
                    line("setp.ne.u32 " + d + ", " + t + ", 0;");
                } else if (dc == RD) line("mov.u64 " + d + ", " + a + ";");
                else { line("mov.u32 " + d + ", " + lo + ";"); canon(ds, d); }
                return;
            }
            case CastOp::ZExt: {
                if (sc == P) { line(std::string(dc == RD ? "selp.u64 " : "selp.u32 ") + d + ", 1, 0, " + a + ";"); return; }
                if (sc == RD) { line("mov.u64 " + d + ", " + a + ";"); return; }
                std::string z = zx(ss, a);
                if (dc == RD) line("cvt.u64.u32 " + d + ", " + z + ";");
                else { line("mov.u32 " + d + ", " + z + ";"); canon(ds, d); }
                return;
            }
            case CastOp::SExt: {
                if (sc == P) { line(std::string(dc == RD ? "selp.s64 " : "selp.s32 ") + d + ", -1, 0, " + a + ";"); return; }
                if (sc == RD) { line("mov.u64 " + d + ", " + a + ";"); return; }
                if (dc == RD) line("cvt.s64.s32 " + d + ", " + a + ";");
                else line("mov.u32 " + d + ", " + a + ";");
                return;
            }
            case CastOp::FPTrunc: case CastOp::FPExt:
                if (dc == sc) { line(std::string("mov.") + (dc == H ? "b16" : fty(dc)) + " " + d + ", " + a + ";"); return; }
                line(std::string("cvt.") + (op == CastOp::FPTrunc ? "rn." : "") + fty(dc) + "." + fty(sc) + " " + d + ", " + a + ";");
                return;
            case CastOp::FPToSI: case CastOp::FPToUI: {
                const char* su = op == CastOp::FPToSI ? "s" : "u";
                if (dc == RD) { line(std::string("cvt.rzi.") + su + "64." + fty(sc) + " " + d + ", " + a + ";"); return; }
                std::string t = dc == P ? fresh(R) : d;
                line(std::string("cvt.rzi.") + su + "32." + fty(sc) + " " + t + ", " + a + ";");
                if (dc == P) { line("and.b32 " + t + ", " + t + ", 1;"); line("setp.ne.u32 " + d + ", " + t + ", 0;"); }
                else canon(ds, d);
                return;
            }
            case CastOp::SIToFP: case CastOp::UIToFP: {
                bool sg = op == CastOp::SIToFP;
                std::string src = a;
                const char* st = sc == RD ? (sg ? "s64" : "u64") : (sg ? "s32" : "u32");
                if (sc == P) { src = fresh(R); line(std::string(sg ? "selp.s32 " : "selp.u32 ") + src + (sg ? ", -1, 0, " : ", 1, 0, ") + a + ";"); }
                else if (!sg) src = zx(ss, a);
                line(std::string("cvt.rn.") + fty(dc) + "." + st + " " + d + ", " + src + ";");
                return;
            }
            case CastOp::Bitcast:
                if (dc == sc) {
                    const char* t = dc == R ? "b32" : dc == RD ? "b64" : dc == F ? "f32" : dc == FD ? "f64" : "b16";
                    line(std::string("mov.") + t + " " + d + ", " + a + ";");
                } else if ((dc == F && sc == R) || (dc == R && sc == F)) line("mov.b32 " + d + ", " + a + ";");
                else if ((dc == FD && sc == RD) || (dc == RD && sc == FD)) line("mov.b64 " + d + ", " + a + ";");
                else if (dc == H && sc == R) line("cvt.u16.u32 " + d + ", " + a + ";");
                else if (dc == R && sc == H) { line("cvt.u32.u16 " + d + ", " + a + ";"); canon(Scalar::I16, d); }
                else fail("E091", "bitcast between types of different size");
                return;
        }
    }
    void lower_cast(uint32_t id, const Inst& in) {
        auto& d = vregs(Val::V(id));
        auto& a = vregs(in.ops[0]);
        for (size_t l = 0; l < d.size(); l++)
            cast_scalar((CastOp)in.sub, in.ty.sc, in.ty.is_ptr(), in.aux.sc, in.aux.is_ptr(), d[l], a[l]);
    }

    static const char* mem_ty(Scalar s, bool ptr) {
        if (ptr) return "u64";
        switch (s) {
            case Scalar::I1: return "u8";
            case Scalar::I8: return "s8";
            case Scalar::I16: return "s16";
            case Scalar::I32: return "u32";
            case Scalar::I64: return "u64";
            case Scalar::F16: return "b16";
            case Scalar::F32: return "f32";
            case Scalar::F64: return "f64";
        }
        return "u32";
    }
    void lower_load(uint32_t id, const Inst& in) {
        auto& d = vregs(Val::V(id));
        std::string addr = reg(in.ops[0]);
        std::string pre = std::string("ld.") + (in.vol ? "volatile." : "") + space_word(in.space) + ".";
        Ty t = in.ty;
        if (t.is_vec() && t.sc != Scalar::I1 && (t.lanes == 2 || (t.lanes == 4 && scalar_bytes(t.sc) <= 4)) && in.align >= t.lanes * scalar_bytes(t.sc)) {
            std::string list;
            for (size_t l = 0; l < d.size(); l++) list += (l ? ", " : "") + d[l];
            line(pre + "v" + std::to_string((int)t.lanes) + "." + mem_ty(t.sc, false) + " {" + list + "}, [" + addr + "];");
            return;
        }
        for (size_t l = 0; l < d.size(); l++) {
            std::string at = "[" + addr + (l ? "+" + std::to_string(l * scalar_bytes(t.sc)) : "") + "]";
            if (!t.is_ptr() && t.sc == Scalar::I1) {
                std::string tmp = fresh(R);
                line(pre + "u8 " + tmp + ", " + at + ";");
                line("setp.ne.u32 " + d[l] + ", " + tmp + ", 0;");
            } else line(pre + mem_ty(t.sc, t.is_ptr()) + " " + d[l] + ", " + at + ";");
        }
    }
    void lower_store(const Inst& in) {
        auto& v = vregs(in.ops[1]);
        std::string addr = reg(in.ops[0]);
        std::string pre = std::string("st.") + (in.vol ? "volatile." : "") + space_word(in.space) + ".";
        Ty t = in.aux;
        auto sty = [&](Scalar s, bool ptr) -> std::string {
            if (ptr) return "u64";
            switch (s) { case Scalar::I1: case Scalar::I8: return "u8"; case Scalar::I16: return "u16"; default: return mem_ty(s, false); }
        };
        if (t.is_vec() && t.sc != Scalar::I1 && (t.lanes == 2 || (t.lanes == 4 && scalar_bytes(t.sc) <= 4)) && in.align >= t.lanes * scalar_bytes(t.sc)) {
            std::string list;
            for (size_t l = 0; l < v.size(); l++) list += (l ? ", " : "") + v[l];
            line(pre + "v" + std::to_string((int)t.lanes) + "." + sty(t.sc, false) + " [" + addr + "], {" + list + "};");
            return;
        }
        for (size_t l = 0; l < v.size(); l++) {
            std::string at = "[" + addr + (l ? "+" + std::to_string(l * scalar_bytes(t.sc)) : "") + "]";
            std::string src = v[l];
            if (!t.is_ptr() && t.sc == Scalar::I1) { src = fresh(R); line("selp.u32 " + src + ", 1, 0, " + v[l] + ";"); }
            line(pre + sty(t.sc, t.is_ptr()) + " " + at + ", " + src + ";");
        }
    }

    void lower_index(uint32_t id, const Inst& in) {
        static const char* sreg[] = {"%tid.x", "%tid.y", "%tid.z", "%ctaid.x", "%ctaid.y", "%ctaid.z",
                                     "%ntid.x", "%ntid.y", "%ntid.z", "%nctaid.x", "%nctaid.y", "%nctaid.z"};
        const std::string& d = reg(Val::V(id));
        if (cls(in.ty) == RD) {
            std::string t = fresh(R);
            line(std::string("mov.u32 ") + t + ", " + sreg[in.sub] + ";");
            line("cvt.u64.u32 " + d + ", " + t + ";");
        } else if (cls(in.ty) == R) {
            line(std::string("mov.u32 ") + d + ", " + sreg[in.sub] + ";");
            canon(in.ty.sc, d);
        } else fail("E091", "index intrinsic with a non-integer type");
    }

    void lower_shuffle(uint32_t id, const Inst& in) {
        static const char* mode[] = {"idx", "up", "down", "bfly"};
        const char* clamp = (Shfl)in.sub == Shfl::Up ? "0x0" : "0x1f";
        const std::string& d = reg(Val::V(id));
        std::string lane = reg(in.ops[1]);
        if (cls(ty(in.ops[1])) == RD) { std::string t = fresh(R); line("cvt.u32.u64 " + t + ", " + lane + ";"); lane = t; }
        std::string op = std::string("shfl.sync.") + mode[in.sub] + ".b32 ";
        Cls c = cls(in.ty);
        if (c == R || c == F) {
            line(op + d + ", " + reg(in.ops[0]) + ", " + lane + ", " + clamp + ", 0xffffffff;");
            if (c == R) canon(in.ty.sc, d);
        } else if (c == RD || c == FD) {   // split in two halves (emit.rs:1506-1543)
            std::string lo = fresh(R), hi = fresh(R);
            line("mov.b64 {" + lo + ", " + hi + "}, " + reg(in.ops[0]) + ";");
            line(op + lo + ", " + lo + ", " + lane + ", " + clamp + ", 0xffffffff;");
            line(op + hi + ", " + hi + ", " + lane + ", " + clamp + ", 0xffffffff;");
            line("mov.b64 " + d + ", {" + lo + ", " + hi + "};");
        } else fail("E091", "shuffle of this type is not implemented");
    }
    void lower_vote(uint32_t id, const Inst& in) {
        std::string p = as_pred(in.ops[0]);
        const std::string& d = reg(Val::V(id));
        if (in.op == Opc::Ballot) {
            if (cls(in.ty) == RD) { std::string t = fresh(R); line("vote.sync.ballot.b32 " + t + ", " + p + ", 0xffffffff;"); line("cvt.u64.u32 " + d + ", " + t + ";"); }
            else line("vote.sync.ballot.b32 " + d + ", " + p + ", 0xffffffff;");
            return;
        }
        const char* m = in.op == Opc::VoteAny ? "any" : "all";
        if (in.ty.is_sc(Scalar::I1)) { line(std::string("vote.sync.") + m + ".pred " + d + ", " + p + ", 0xffffffff;"); return; }
        std::string q = fresh(P);
        line(std::string("vote.sync.") + m + ".pred " + q + ", " + p + ", 0xffffffff;");
        line(std::string(cls(in.ty) == RD ? "selp.u64 " : "selp.u32 ") + d + ", 1, 0, " + q + ";");
    }

    void lower_atomic(uint32_t id, const Inst& in) {
        AtomOp op = (AtomOp)in.sub;
        if (in.space != Space::Global && in.space != Space::Shared) { fail("E092", "atomics exist on global and shared memory only"); return; }
        std::string sp = space_word(in.space), addr = "[" + reg(in.ops[0]) + "]", v = reg(in.ops[1]);
        Cls c = cls(in.ty);
        bool w64 = c == RD || c == FD, flt = c == F || c == FD, unused = uses[id] == 0;
        std::string d = reg(Val::V(id));
        if (flt && (op == AtomOp::Min || op == AtomOp::Max)) {   // CAS retry loop (emit.rs:1700-1796)
            std::string ib = w64 ? "b64" : "b32", ft = w64 ? "f64" : "f32";
            Cls ic = w64 ? RD : R;
            std::string old = fresh(ic), assumed = fresh(ic), cand = fresh(c), curf = fresh(c), candb = fresh(ic), p = fresh(P);
            std::string loop = fresh_label("atomic_fminmax_loop");
            line("ld." + sp + "." + ib + " " + old + ", " + addr + ";");
            label(loop);
            line("mov." + ib + " " + assumed + ", " + old + ";");
            line("mov." + ib + " " + curf + ", " + assumed + ";");
            line(std::string(op == AtomOp::Min ? "min." : "max.") + ft + " " + cand + ", " + curf + ", " + v + ";");
            line("mov." + ib + " " + candb + ", " + cand + ";");
            line("atom." + sp + ".cas." + ib + " " + old + ", " + addr + ", " + assumed + ", " + candb + ";");
            line("setp.ne." + ib + " " + p + ", " + old + ", " + assumed + ";");
            line("@" + p + " bra " + loop + ";");
            line("mov." + ib + " " + d + ", " + old + ";");
            return;
        }
        std::string t, m;
        switch (op) {
            case AtomOp::Add: m = "add"; t = flt ? (w64 ? "f64" : "f32") : (w64 ? "u64" : "u32"); break;
            case AtomOp::Sub: {
                m = "add";
                std::string n = fresh(c);
                if (flt) { t = w64 ? "f64" : "f32"; line("neg." + t + " " + n + ", " + v + ";"); }
                else { t = w64 ? "u64" : "u32"; line(std::string("neg.s") + (w64 ? "64 " : "32 ") + n + ", " + v + ";"); }
                v = n;
                break;
            }
            case AtomOp::Exch: m = "exch"; t = w64 ? "b64" : "b32"; unused = false; break;
            case AtomOp::Min: m = "min"; t = w64 ? "s64" : "s32"; break;
            case AtomOp::Max: m = "max"; t = w64 ? "s64" : "s32"; break;
            case AtomOp::And: m = "and"; t = w64 ? "b64" : "b32"; break;
            case AtomOp::Or: m = "or"; t = w64 ? "b64" : "b32"; break;
            case AtomOp::Xor: m = "xor"; t = w64 ? "b64" : "b32"; break;
        }
        if (unused) line("red." + sp + "." + m + "." + t + " " + addr + ", " + v + ";");
        else line("atom." + sp + "." + m + "." + t + " " + d + ", " + addr + ", " + v + ";");
    }
    void lower_cas(uint32_t id, const Inst& in) {
        if (in.space != Space::Global && in.space != Space::Shared) { fail("E092", "atomics exist on global and shared memory only"); return; }
        Cls c = cls(in.ty);
        bool w64 = c == RD || c == FD;
        std::string ib = w64 ? "b64" : "b32";
        line(std::string("atom.") + space_word(in.space) + ".cas." + ib + " " + reg(Val::V(id)) + ", [" + reg(in.ops[0]) + "], " + reg(in.ops[1]) + ", " + reg(in.ops[2]) + ";");
    }
    void lower_warp_reduce(uint32_t id, const Inst& in) {
        static const char* m[] = {"max.s32", "min.s32", "add.s32", "and.b32", "or.b32", "xor.b32"};
        line(std::string("redux.sync.") + m[in.sub] + " " + reg(Val::V(id)) + ", " + reg(in.ops[0]) + ", 0xffffffff;");
    }

    // The pointer parameter a value is derived from through pointer additions, or -1.
    int base_param(Val v) const {
        for (int depth = 0; depth < 64; depth++) {
            if (v.param) return f.params[v.idx].is_ptr() ? (int)v.idx : -1;
            const Inst& d = f.insts[v.idx];
            if (d.op != Opc::Bin || (BinOp)d.sub != BinOp::Add || !d.ty.is_ptr()) return -1;
            if (f.val_ty(d.ops[0]).is_ptr()) v = d.ops[0];
            else if (f.val_ty(d.ops[1]).is_ptr()) v = d.ops[1];
            else return -1;
        }
        return -1;
    }

    // value = parameter (or none) + c0 + cx*bid.x + cy*bid.y, when the value is such a function.
    struct Aff {
        bool ok = false;
        int param = -1;
        long long c0 = 0, cx = 0, cy = 0;
    };
    Aff affine(Val v, int depth = 0) const {
        Aff r;
        if (depth > 64) return r;
        if (v.param) {
            r.ok = f.params[v.idx].is_ptr();
            r.param = (int)v.idx;
            return r;
        }
        const Inst& d = f.insts[v.idx];
        if (d.ty.is_vec()) return r;
        switch (d.op) {
            case Opc::ConstI:
                if (d.ty.is_ptr() && d.ty.sp != Space::Global) return r;
                r.ok = true;
                r.c0 = d.imm;
                return r;
            case Opc::Index:
                r.ok = d.sub == 3 || d.sub == 4;
                r.cx = d.sub == 3;
                r.cy = d.sub == 4;
                return r;
            case Opc::Cast: {
                CastOp c = (CastOp)d.sub;
                if (c != CastOp::SExt && c != CastOp::ZExt && c != CastOp::Trunc && c != CastOp::Bitcast) return r;
                if (d.aux.is_float() || d.ty.is_float()) return r;
                return affine(d.ops[0], depth + 1);
            }
            case Opc::Bin: {
                BinOp b = (BinOp)d.sub;
                Aff x = affine(d.ops[0], depth + 1), y = affine(d.ops[1], depth + 1);
                if (!x.ok || !y.ok) return r;
                if (b == BinOp::Add || b == BinOp::Sub) {
                    if (x.param >= 0 && y.param >= 0) return r;
                    if (b == BinOp::Sub && y.param >= 0) return r;
                    long long sgn = b == BinOp::Add ? 1 : -1;
                    r.ok = true;
                    r.param = x.param >= 0 ? x.param : y.param;
                    r.c0 = x.c0 + sgn * y.c0; r.cx = x.cx + sgn * y.cx; r.cy = x.cy + sgn * y.cy;
                    return r;
                }
                if (b == BinOp::Mul || b == BinOp::Shl) {
                    if (x.param >= 0 || y.param >= 0) return r;
                    bool yc = y.cx == 0 && y.cy == 0, xc = x.cx == 0 && x.cy == 0;
                    if (b == BinOp::Shl) {
                        if (!yc || y.c0 < 0 || y.c0 > 40) return r;
                        r.ok = true; r.c0 = x.c0 << y.c0; r.cx = x.cx << y.c0; r.cy = x.cy << y.c0;
                        return r;
                    }
                    if (!yc && !xc) return r;
                    const Aff& k = yc ? y : x;
                    const Aff& t = yc ? x : y;
                    r.ok = true; r.c0 = t.c0 * k.c0; r.cx = t.cx * k.c0; r.cy = t.cy * k.c0;
                    return r;
                }
                return r;
            }
            default: return r;
        }
    }

    // `mma` as a CTA-collective op: every thread of the CTA reaches it, the tile product is
    // computed once.  This generic form spreads the m*n outputs over the CTA's threads and
    // follows the oracle's arithmetic exactly: acc = 0; acc = acc + a*b (two roundings);
    // D = C + acc (oracle.rs:2178-2337).  Shapes the fast paths cover never get here.
    void lower_mma(const Inst& in) {
        MmaSite site;
        site.inst = &in;
        site.a = reg(in.ops[0]); site.b = reg(in.ops[1]); site.c = reg(in.ops[2]); site.d = reg(in.ops[3]);
        site.sa = ty(in.ops[0]).sp; site.sb = ty(in.ops[1]).sp; site.sc = ty(in.ops[2]).sp; site.sd = ty(in.ops[3]).sp;
        const Inst* cd = in.ops[2].param ? nullptr : &f.insts[in.ops[2].idx];
        site.c_is_null = cd && cd->op == Opc::ConstI && cd->ty.is_ptr() && cd->ty.sp == Space::Global && cd->imm == 0;
        site.uid = mma_n++;
        site.kernel = f.name;
        site.nparams = (unsigned)f.params.size();
        site.max_threads = mod.has_launch_bounds ? mod.max_threads : 0;
        size_t n_mma = 0;
        for (auto& b : f.blocks) for (uint32_t id : b.insts) n_mma += f.insts[id].op == Opc::Mma;
        site.sole_mma = n_mma == 1;
        site.a_param = base_param(in.ops[0]);
        site.b_param = base_param(in.ops[1]);
        if (site.a_param >= 0) site.a_base = param_regs[site.a_param][0];
        if (site.b_param >= 0) site.b_base = param_regs[site.b_param][0];
        Aff fa = affine(in.ops[0]), fb = affine(in.ops[1]), fd = affine(in.ops[3]);
        site.affine = fa.ok && fb.ok && fd.ok && fa.param >= 0 && fb.param >= 0 && fd.param >= 0;
        site.a_c0 = fa.c0; site.a_cx = fa.cx; site.a_cy = fa.cy;
        site.b_c0 = fb.c0; site.b_cx = fb.cx; site.b_cy = fb.cy;
        site.d_c0 = fd.c0; site.d_cx = fd.cx; site.d_cy = fd.cy;
        site.d_param = fd.param;
        if (site.affine) { site.a_param = fa.param; site.b_param = fb.param; site.a_base = param_regs[fa.param][0]; site.b_base = param_regs[fb.param][0]; site.d_base = param_regs[fd.param][0]; }
        site.pure_kernel = f.blocks.size() == 1 && f.blocks[0].term.kind == Term::Ret;
        for (uint32_t id : f.blocks[0].insts) {
            Opc o = f.insts[id].op;
            if (o != Opc::Mma && o != Opc::ConstI && o != Opc::Index && o != Opc::Bin && o != Opc::Cast) site.pure_kernel = false;
        }
        site.maxntid = &maxntid;
        site.extra_params = &extra_params;
        site.module_decls = &module_decls;
        site.pair_twin = pair_twin;
        site.cluster = &cluster;
        site.tmem_cols = &tmem_cols;
        if (emit_mma_fast(site, &decls, &body, &plan)) return;
        if (pair_twin) { fail("E099", "internal: the two-SM twin of " + f.name + " has no lowering"); return; }

        const int64_t lda = in.has_ld && in.ld[0] ? in.ld[0] : (in.a_col ? in.m : in.k);
        const int64_t ldb = in.has_ld && in.ld[1] ? in.ld[1] : (in.b_col ? in.k : in.n);
        const int64_t ldc = in.has_ld && in.ld[2] ? in.ld[2] : in.n;
        const int64_t ldd = in.has_ld && in.ld[3] ? in.ld[3] : in.n;
        const bool flt = in.acc_dt >= Scalar::F16;
        const unsigned isz = scalar_bytes(in.in_dt), asz = scalar_bytes(in.acc_dt), osz = scalar_bytes(in.out_dt);
        std::string tid = fresh(R), nt = fresh(R), t1 = fresh(R), t2 = fresh(R), e = fresh(R), i = fresh(R), j = fresh(R), kk = fresh(R);
        std::string p = fresh(P), q = fresh(P), pa = fresh(RD), pb = fresh(RD), pc = fresh(RD), off = fresh(RD);
        std::string l_e = fresh_label("mma_e"), l_eend = fresh_label("mma_e_end"), l_k = fresh_label("mma_k"), l_kend = fresh_label("mma_k_end");
        Cls ac = cls_of(in.acc_dt);
        std::string acc = fresh(ac), av = fresh(ac), bv = fresh(ac), pr = fresh(ac), cv = fresh(ac);
        line("bar.sync 0;");
        line("mov.u32 " + tid + ", %tid.x;"); line("mov.u32 " + nt + ", %ntid.x;");
        line("mov.u32 " + t1 + ", %tid.y;"); line("mad.lo.u32 " + tid + ", " + t1 + ", " + nt + ", " + tid + ";");
        line("mov.u32 " + t2 + ", %ntid.y;"); line("mul.lo.u32 " + nt + ", " + nt + ", " + t2 + ";");
        line("mov.u32 " + t1 + ", %tid.z;"); line("mad.lo.u32 " + tid + ", " + t1 + ", " + nt + ", " + tid + ";");
        line("mov.u32 " + t2 + ", %ntid.z;"); line("mul.lo.u32 " + nt + ", " + nt + ", " + t2 + ";");
        line("mov.u32 " + e + ", " + tid + ";");
        label(l_e);
        line("setp.ge.u32 " + p + ", " + e + ", " + std::to_string((uint64_t)in.m * in.n) + ";");
        line("@" + p + " bra " + l_eend + ";");
        line("div.u32 " + i + ", " + e + ", " + std::to_string(in.n) + ";");
        line("rem.u32 " + j + ", " + e + ", " + std::to_string(in.n) + ";");
        line(flt ? std::string(ac == FD ? "mov.f64 " : "mov.f32 ") + acc + (ac == FD ? ", 0d0000000000000000;" : ", 0f00000000;") : "mov.u32 " + acc + ", 0;");
        line("mov.u32 " + kk + ", 0;");
        label(l_k);
        line("setp.ge.u32 " + q + ", " + kk + ", " + std::to_string(in.k) + ";");
        line("@" + q + " bra " + l_kend + ";");
        // element addresses: row-major X[r,c] at r*ld + c; col-major at c*ld + r
        auto elem_addr = [&](const std::string& dst, const std::string& base, const std::string& r, const std::string& c, int64_t ld, bool col, unsigned esz) {
            std::string lin = fresh(RD), w = fresh(RD);
            line("cvt.u64.u32 " + lin + ", " + (col ? c : r) + ";");
            line("mul.lo.u64 " + lin + ", " + lin + ", " + std::to_string(ld) + ";");
            line("cvt.u64.u32 " + w + ", " + (col ? r : c) + ";");
            line("add.u64 " + lin + ", " + lin + ", " + w + ";");
            line("mad.lo.u64 " + dst + ", " + lin + ", " + std::to_string(esz) + ", " + base + ";");
        };
        auto load_elem = [&](const std::string& dst, Space sp, const std::string& addr, Scalar st, Scalar want) {
            if (st == want || (st == Scalar::I32 && want == Scalar::I32)) { line(std::string("ld.") + space_word(sp) + "." + mem_ty(st, false) + " " + dst + ", [" + addr + "];"); return; }
            if (st == Scalar::F16) { std::string h = fresh(H); line(std::string("ld.") + space_word(sp) + ".b16 " + h + ", [" + addr + "];"); line("cvt.f32.f16 " + dst + ", " + h + ";"); return; }
            // narrower integer inputs are sign-extended by the load (movsx in the oracle)
            line(std::string("ld.") + space_word(sp) + "." + mem_ty(st, false) + " " + dst + ", [" + addr + "];");
        };
        elem_addr(pa, site.a, i, kk, lda, in.a_col, isz);
        elem_addr(pb, site.b, kk, j, ldb, in.b_col, isz);
        load_elem(av, site.sa, pa, in.in_dt, in.acc_dt);
        load_elem(bv, site.sb, pb, in.in_dt, in.acc_dt);
        if (flt) {
            std::string t = ac == FD ? "f64" : "f32";
            line("mul.rn." + t + " " + pr + ", " + av + ", " + bv + ";");
            line("add.rn." + t + " " + acc + ", " + acc + ", " + pr + ";");
        } else {
            line("mul.lo.s32 " + pr + ", " + av + ", " + bv + ";");
            line("add.s32 " + acc + ", " + acc + ", " + pr + ";");
        }
        line("add.u32 " + kk + ", " + kk + ", 1;");
        line("bra " + l_k + ";");
        label(l_kend);
        if (!site.c_is_null) {
            elem_addr(pc, site.c, i, j, ldc, false, asz);
            load_elem(cv, site.sc, pc, in.acc_dt, in.acc_dt);
            if (flt) line(std::string("add.rn.") + (ac == FD ? "f64 " : "f32 ") + cv + ", " + cv + ", " + acc + ";");
            else line("add.s32 " + cv + ", " + cv + ", " + acc + ";");
        } else line(std::string(ac == FD ? "mov.f64 " : ac == F ? "mov.f32 " : "mov.u32 ") + cv + ", " + acc + ";");
        elem_addr(off, site.d, i, j, ldd, false, osz);
        if (in.out_dt == Scalar::F16 && in.acc_dt == Scalar::F32) {
            std::string h = fresh(H);
            line("cvt.rn.f16.f32 " + h + ", " + cv + ";");
            line(std::string("st.") + space_word(site.sd) + ".b16 [" + off + "], " + h + ";");
        } else {
            std::string st = in.acc_dt == Scalar::I8 ? "u8" : in.acc_dt == Scalar::I16 ? "u16" : mem_ty(in.acc_dt, false);
            line(std::string("st.") + space_word(site.sd) + "." + st + " [" + off + "], " + cv + ";");
        }
        line("add.u32 " + e + ", " + e + ", " + nt + ";");
        line("bra " + l_e + ";");
        label(l_eend);
        line("bar.sync 0;");
    }

    void lower_inst(uint32_t id) {
        const Inst& in = f.insts[id];
        switch (in.op) {
            case Opc::ConstI: lower_const_i(id, in); break;
            case Opc::ConstF: lower_const_f(id, in); break;
            case Opc::Bin: lower_bin(id, in); break;
            case Opc::ICmp: lower_icmp(id, in); break;
            case Opc::FCmp: lower_fcmp(id, in); break;
            case Opc::Select: lower_select(id, in); break;
            case Opc::Cast: lower_cast(id, in); break;
            case Opc::Load: lower_load(id, in); break;
            case Opc::Store: lower_store(in); break;
            case Opc::Phi: vregs(Val::V(id)); break;   // written on the incoming edges
            case Opc::Index: lower_index(id, in); break;
            case Opc::Barrier: line("bar.sync 0;"); break;
            case Opc::Shuffle: lower_shuffle(id, in); break;
            case Opc::Ballot: case Opc::VoteAny: case Opc::VoteAll: lower_vote(id, in); break;
            case Opc::Atomic: lower_atomic(id, in); break;
            case Opc::AtomicCas: lower_cas(id, in); break;
            case Opc::Mma: lower_mma(in); break;
            case Opc::VecExtract: case Opc::VecBuild: vregs(Val::V(id)); break;   // register aliases
            case Opc::WarpReduce: lower_warp_reduce(id, in); break;
            default: fail("E090", "operation has no device lowering"); break;
        }
    }

    // ---- phis and terminators --------------------------------------------------------------
    void mov_same(Ty t, const std::string& d, const std::string& s) {
        Cls c = cls(t);
        const char* w = c == P ? "pred" : c == R ? "b32" : c == RD ? "b64" : c == F ? "f32" : c == FD ? "f64" : "b16";
        line(std::string("mov.") + w + " " + d + ", " + s + ";");
    }
    bool edge_has_phis(uint32_t to) const {
        for (uint32_t id : f.blocks[to].insts) if (f.insts[id].op == Opc::Phi) return true;
        return false;
    }
    void emit_phi_copies(uint32_t from, uint32_t to) {
        std::vector<std::pair<uint32_t, Val>> copies;
        std::set<uint32_t> phis;
        for (uint32_t id : f.blocks[to].insts) {
            const Inst& in = f.insts[id];
            if (in.op != Opc::Phi) continue;
            phis.insert(id);
            for (size_t k = 0; k < in.ops.size(); k++) if (in.phi_blocks[k] == from) { copies.push_back({id, in.ops[k]}); break; }
        }
        bool staged = false;
        for (auto& c : copies) if (!c.second.param && phis.count(c.second.idx) && c.second.idx != c.first) staged = true;
        if (!staged) {
            for (auto& c : copies) {
                auto& d = vregs(Val::V(c.first));
                auto& s = vregs(c.second);
                for (size_t l = 0; l < d.size(); l++) if (d[l] != s[l]) mov_same(f.insts[c.first].ty, d[l], s[l]);
            }
            return;
        }
        std::vector<std::vector<std::string>> tmp;
        for (auto& c : copies) {
            tmp.push_back(alloc(f.insts[c.first].ty));
            auto& s = vregs(c.second);
            for (size_t l = 0; l < s.size(); l++) mov_same(f.insts[c.first].ty, tmp.back()[l], s[l]);
        }
        for (size_t k = 0; k < copies.size(); k++) {
            auto& d = vregs(Val::V(copies[k].first));
            for (size_t l = 0; l < d.size(); l++) mov_same(f.insts[copies[k].first].ty, d[l], tmp[k][l]);
        }
    }
    std::string blk(uint32_t b) const { return "$L" + std::to_string(b); }
    void goto_block(uint32_t from, uint32_t to) {
        emit_phi_copies(from, to);
        line("bra " + blk(to) + ";");
    }
    void lower_term(uint32_t from, const Term& t) {
        switch (t.kind) {
            case Term::Br: goto_block(from, t.t); break;
            case Term::CondBr: {
                std::string p = as_pred(t.val);
                if (!edge_has_phis(t.t) && !edge_has_phis(t.f)) {
                    line("@" + p + " bra " + blk(t.t) + ";");
                    line("bra " + blk(t.f) + ";");
                    break;
                }
                std::string taken = fresh_label("condbr_true");
                line("@" + p + " bra " + taken + ";");
                goto_block(from, t.f);
                label(taken);
                goto_block(from, t.t);
                break;
            }
            case Term::Switch: {
                Ty st = ty(t.val);
                bool w64 = cls(st) == RD;
                std::string p = fresh(P);
                for (auto& c : t.cases) {
                    std::string cv = w64 ? std::to_string(c.first) : std::to_string((int32_t)(st.is_sc(Scalar::I8) ? (int8_t)c.first : st.is_sc(Scalar::I16) ? (int16_t)c.first : (int32_t)c.first));
                    line(std::string("setp.eq.") + (w64 ? "s64 " : "s32 ") + p + ", " + reg(t.val) + ", " + cv + ";");
                    if (edge_has_phis(c.second)) {
                        std::string skip = fresh_label("switch_skip");
                        line("@!" + p + " bra " + skip + ";");
                        goto_block(from, c.second);
                        label(skip);
                    } else line("@" + p + " bra " + blk(c.second) + ";");
                }
                goto_block(from, t.t);
                break;
            }
            case Term::Ret: line("ret;"); break;   // a kernel entry drops any value (emit.rs:1884-1890)
        }
    }

    bool run(std::string* out) {
        uses.assign(f.insts.size(), 0);
        for (auto& b : f.blocks) {
            for (uint32_t id : b.insts) for (Val v : f.insts[id].ops) if (!v.param) uses[v.idx]++;
            if (b.term.has_val && !b.term.val.param) uses[b.term.val.idx]++;
        }
        emit_param_loads();
        // Programmatic dependent launch: the next kernel on the stream may be set up while this grid runs, and this grid --
        // when it is itself launched that way -- touches memory only once the grids before it have completed and their
        // writes are visible.  Both are no-ops under an ordinary launch.
        line("griddepcontrol.launch_dependents;");
        line("griddepcontrol.wait;");
        for (uint32_t b = 0; b < f.blocks.size(); b++) {
            label(blk(b));
            for (uint32_t id : f.blocks[b].insts) { lower_inst(id); if (failed) return false; }
            lower_term(b, f.blocks[b].term);
            if (failed) return false;
        }
        std::string o = ".visible .entry " + f.name + "(";
        std::vector<std::string> pd;
        for (size_t i = 0; i < f.params.size(); i++) pd.push_back(param_decl(i));
        for (auto& e : extra_params) pd.push_back(e);
        for (size_t i = 0; i < pd.size(); i++) o += (i ? ",\n\t" : "\n\t") + pd[i];
        o += pd.empty() ? ")\n" : "\n)\n";
        if (mod.has_launch_bounds) {
            o += ".maxntid " + std::to_string(maxntid ? maxntid : mod.max_threads) + ", 1, 1\n";
            if (mod.min_blocks) o += ".minnctapersm " + std::to_string(maxntid ? 1u : mod.min_blocks) + "\n";
        }
        if (cluster) o += ".reqnctapercluster " + std::to_string(cluster) + ", 1, 1\n";
        // The tensor-memory budget beside the register budget: an SM has 512 columns, and every CTA resident on it
        // allocates its own (a CTA that cannot get them would wait inside tcgen05.alloc for one that never leaves).
        const unsigned resident_ctas = maxntid ? 1u : (mod.min_blocks ? mod.min_blocks : 1u);
        if (tmem_cols * resident_ctas > 512) {
            fail("E099", "internal: " + std::to_string(resident_ctas) + " resident CTAs x " + std::to_string(tmem_cols) + " tensor-memory columns exceed the SM's 512");
            return false;
        }
        // the register-budget pass: pressure of this body against the budget the launch bounds imply
        std::vector<std::string> all_decls;
        for (int c = 0; c < NCLS; c++)
            if (counts[c]) all_decls.push_back(std::string("\t.reg ") + kClsDecl[c] + " " + kClsPrefix[c] + "<" + std::to_string(counts[c]) + ">;");
        for (auto& d : decls) all_decls.push_back(d);
        est_regs = ptx_register_pressure(all_decls, body);
        const unsigned threads = maxntid ? maxntid : (mod.has_launch_bounds ? mod.max_threads : 0);
        budget = register_budget(threads, maxntid ? 1u : mod.min_blocks);
        // Launch bounds without a CTA count: the default residency is this backend's choice, so a body that
        // overshoots its budget by a quarter at most is held to it (ptxas then trades a few registers for the
        // residency); a larger overshoot is left alone rather than spilled.
        if (mod.has_launch_bounds && !mod.min_blocks && !maxntid && est_regs > budget && 4 * est_regs <= 5 * budget) {
            o += ".maxnreg " + std::to_string(budget) + "\n";
            capped = true;
        }
        o += "{\n";
        for (int c = 0; c < NCLS; c++)
            if (counts[c]) o += std::string("\t.reg ") + kClsDecl[c] + " " + kClsPrefix[c] + "<" + std::to_string(counts[c]) + ">;\n";
        for (auto& d : decls) o += d + "\n";
        for (auto& l : body) o += l + "\n";
        o += "}\n";
        *out = o;
        return true;
    }
};

}  // namespace

bool emit_ptx(const Module& in, const EmitOptions& opts, EmitResult* out, Diag* d) {
    if (!check_module(in, d)) return false;
    Module m = in;
    out->reports.clear();
    // The vectorisers pick the largest unroll whose body, lowered by this emitter, stays inside the budget.
    const int budget = opts.reg_budget > 0 ? opts.reg_budget : register_budget(m.has_launch_bounds ? m.max_threads : 0, m.min_blocks);
    PressureFn measure = [](const Module& mm, const Function& fn) {
        FnEmitter fe(mm, fn);
        std::string ignored;
        return fe.run(&ignored) ? fe.est_regs : (1 << 20);
    };
    optimize_module(m, opts.opt_level, budget, opts.max_unroll, measure, &out->reports);
    std::string why;
    if (!verify_module(m, &why)) {
        if (d) { d->code = "E400"; d->arg = "internal: optimised module failed verification: " + why; }
        return false;
    }
    if (opts.want_bir) out->bir = print_module(m);
    std::string text = "//\n// Generated by basalt-b200 (nvidia-ptx-sm100)\n//\n.version 8.7\n.target sm_100a\n.address_size 64\n\n";
    std::string bodies;
    std::vector<std::string> module_decls;
    for (size_t i = 0; i < m.funcs.size(); i++) {
        const Function& f = m.funcs[i];
        const OptReport& r = out->reports[i];
        FnEmitter fe(m, f);
        std::string fn_text;
        if (!fe.run(&fn_text)) {
            if (d) *d = fe.diag;
            return false;
        }
        text += "// kernel " + f.name + ": est_regs=" + std::to_string(fe.est_regs) + " budget=" + std::to_string(fe.budget) + (fe.capped ? " maxnreg" : "") +
                (fe.tmem_cols ? " tmem_cols=" + std::to_string(fe.tmem_cols) : "");
        if (r.elementwise) text += " elementwise";
        if (r.reduction) text += " reduction";
        if (r.vec_lanes) text += " lanes=" + std::to_string(r.vec_lanes) + " unroll=" + std::to_string(r.unroll);
        if (r.warp_reduces) text += " warp_reduces=" + std::to_string(r.warp_reduces);
        text += "\n";
        if (!r.coarse_of.empty())
        {
            // elements a thread should handle: one trip of the vectorised loop for a streaming body (many short CTAs stream
            // fastest), four trips when the body is arithmetic-heavy (the 32-level helper chain: 31 to 33 T int-op/s on 2 to
            // 8 waves, 22 on 128 -- there the per-CTA set-up is no longer hidden behind memory)
            size_t arithmetic = 0;
            for (auto& in : f.insts) arithmetic += in.op == Opc::Bin;
            const int trips = arithmetic > 256 ? 4 : 1;
            text += "//!basalt.plan " + r.coarse_of + " coarse=" + f.name + " params=" + std::to_string(f.params.size() - 1) + " per_thread=" +
                    std::to_string(std::max(1, r.vec_lanes) * std::max(1, r.unroll) * trips) + " pdl=1\n";
        }
        for (auto& p : fe.plan) text += p + "\n";
        // a kernel with no other launch plan still says that it begins with griddepcontrol.wait (a coarse twin's line,
        // which comes later and carries the same key, replaces this one)
        if (fe.plan.empty() && r.coarse_of.empty() && f.is_kernel) text += "//!basalt.plan " + f.name + " pdl=1\n";
        for (auto& md : fe.module_decls)
            if (std::find(module_decls.begin(), module_decls.end(), md) == module_decls.end()) module_decls.push_back(md);
        bodies += fn_text + "\n";
        // A plan that names a `pair=` entry asks for the same function once more, lowered for pairs of SMs.
        for (auto& p : fe.plan) {
            size_t at = p.find(" pair=");
            if (at == std::string::npos) continue;
            Function twin = f;
            twin.name = p.substr(at + 6, p.find(' ', at + 6) == std::string::npos ? std::string::npos : p.find(' ', at + 6) - (at + 6));
            FnEmitter fe2(m, twin, true);
            std::string twin_text;
            if (!fe2.run(&twin_text)) {
                if (d) *d = fe2.diag;
                return false;
            }
            for (auto& md : fe2.module_decls)
                if (std::find(module_decls.begin(), module_decls.end(), md) == module_decls.end()) module_decls.push_back(md);
            text += "// kernel " + twin.name + ": est_regs=" + std::to_string(fe2.est_regs) + " budget=" + std::to_string(fe2.budget) +
                    (fe2.tmem_cols ? " tmem_cols=" + std::to_string(fe2.tmem_cols) : "") + "\n";
            bodies += twin_text + "\n";
        }
    }
    text += "\n";
    for (auto& md : module_decls) text += md + "\n";
    out->ptx = text + bodies;
    return true;
}

}  // namespace basalt
