// TEST INFRASTRUCTURE, not product code: a restatement of the reference's x86-64 register-allocating
// CPU back end ("x86-regalloc", crates/basalt-x86/src/regalloc.rs with the allocator of
// crates/basalt-passes/src/regalloc.rs and the encoder's instruction set of
// crates/basalt-x86/src/enc.rs), so that the timed CPU baseline is the code shape the reference's
// own CPU launch path executes, not a C loop that gcc optimised.  Only the tests and the CPU legs of
// the benchmark use it.  It is linked with the BIR parser and construct_ssa of the library under
// test (the same text format and the same first pass the reference's emit runs, regalloc.rs:110-116);
// everything after that -- liveness, linear scan, instruction selection, encoding -- is in this file.
//
// What is restated (file:line in the reference):
//  * the refusal surface (regalloc.rs:132-207): one kernel function, no vectors or f16 (E091), no
//    warp collectives, mma, calls or host ops (E090), SysV register arguments only (E093);
//  * the launch model (regalloc.rs:413-500): the function takes the kernel's parameters plus a trailing
//    int64 nthreads, and runs the body once per thread in a native loop whose counter lives in r11;
//    tid.x is r11, bdim.x is nthreads, every other index is 0 / extent 1; barrier is a nop; atomics
//    are plain load-compute-store (regalloc.rs:1129-1216);
//  * the register budget (regalloc.rs:17-45): rsi, rdi, r8, r9 and xmm3..xmm7 are the allocator's
//    pools, rax, rcx, rdx, r10 and xmm0..xmm2 are scratch for the instruction templates;
//  * linear scan over one conservative interval per value (passes regalloc.rs:1-60, 255-525): block
//    liveness with phi operands used at the end of the predecessor, intervals sorted by (start, value),
//    an interval that ends at p keeps its register through p, spill whichever of {new, furthest active}
//    ends later, one slot per spilled value;
//  * parameters staged to the frame on entry and re-placed at the top of every iteration
//    (regalloc.rs:436-470); phis resolved in the predecessor through one staging slot per phi
//    (regalloc.rs:1238-1279); select and conditional branches as real branches;
//  * the instruction templates of every op (regalloc.rs:675-1345), including the two-path
//    unsigned<->float conversions and the software frem.
// Differences, all deliberate: the code is placed in executable memory and called directly instead of
// being wrapped in an ELF object and linked against a C driver; a `shared_obj` line sizes the frame
// cell of a shared array (the reference gives every synthetic cell 8 bytes) and such a cell starts
// zeroed, the rule of the other two CPU oracles; register-to-register float moves copy the whole xmm
// register.
#include <sys/mman.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <set>
#include <string>
#include <tuple>
#include <vector>

#include "../basalt_b200/csrc/bir.hpp"
#include "../basalt_b200/csrc/passes.hpp"

using namespace basalt;

namespace {

// ---------------------------------------------------------------------------------------------------
// Encoder
// ---------------------------------------------------------------------------------------------------
enum Reg : uint8_t { RAX = 0, RCX = 1, RDX = 2, RBX = 3, RSP = 4, RBP = 5, RSI = 6, RDI = 7, R8 = 8, R9 = 9, R10 = 10, R11 = 11 };
enum class W : uint8_t { B1 = 1, B2 = 2, B4 = 4, B8 = 8 };
enum CC : uint8_t { CC_B = 2, CC_AE = 3, CC_E = 4, CC_NE = 5, CC_BE = 6, CC_A = 7, CC_S = 8, CC_P = 10, CC_NP = 11, CC_L = 12, CC_GE = 13, CC_LE = 14, CC_G = 15 };
enum class Alu : uint8_t { Add = 0, Or = 1, And = 4, Sub = 5, Xor = 6, Cmp = 7 };
enum class Shift : uint8_t { Shl = 4, Shr = 5, Sar = 7 };
enum class Sse : uint8_t { Add = 0x58, Mul = 0x59, Sub = 0x5C, Div = 0x5E };

struct Rm {
    enum Kind : uint8_t { Direct, RbpDisp, IndBase } kind;
    uint8_t reg;
    int32_t disp;
    static Rm direct(uint8_t r) { return Rm{Direct, r, 0}; }
    static Rm rbp(int32_t d) { return Rm{RbpDisp, RBP, d}; }
    static Rm ind(uint8_t base) { return Rm{IndBase, base, 0}; }
};

class Enc {
public:
    std::vector<uint8_t> code;

    void label(const std::string& name) { labels_[name] = code.size(); }
    void jmp(const std::string& target) { byte(0xE9); fixup(target); }
    void jcc(uint8_t cc, const std::string& target) { byte(0x0F); byte(0x80 + cc); fixup(target); }
    void setcc(uint8_t cc, uint8_t dst) { inst(0, false, true, {0x0F, (uint8_t)(0x90 + cc)}, 0, Rm::direct(dst)); }
    void ret() { byte(0xC3); }
    void nop() { byte(0x90); }
    void rep_stosq() { bytes({0xF3, 0x48, 0xAB}); }   // rcx quadwords of rax at [rdi]
    void push(uint8_t r) { if (r >= 8) byte(0x41); byte(0x50 + (r & 7)); }
    void pop(uint8_t r) { if (r >= 8) byte(0x41); byte(0x58 + (r & 7)); }
    void mov_rbp_rsp() { bytes({0x48, 0x89, 0xE5}); }
    void mov_rsp_rbp() { bytes({0x48, 0x89, 0xEC}); }
    void sub_rsp(int32_t imm) { bytes({0x48, 0x81, 0xEC}); imm32(imm); }

    // mov between a register and a register / frame slot / [base]
    void load(W w, uint8_t dst, Rm src) { gp(w, w == W::B1 ? 0x8A : 0x8B, dst, src); }
    void store(W w, Rm dst, uint8_t src) { gp(w, w == W::B1 ? 0x88 : 0x89, src, dst); }
    void mov_rr(W w, uint8_t dst, uint8_t src) { store(w, Rm::direct(dst), src); }
    void movabs(uint8_t dst, int64_t imm) {
        byte(0x48 | (dst >= 8 ? 1 : 0));
        byte(0xB8 + (dst & 7));
        for (int i = 0; i < 8; i++) byte((uint8_t)((uint64_t)imm >> (8 * i)));
    }
    void mov_imm32(W w, uint8_t dst, int32_t imm) {
        if (w == W::B8) { inst(0, true, false, {0xC7}, 0, Rm::direct(dst)); imm32(imm); return; }
        if (dst >= 8) byte(0x41);
        byte(0xB8 + (dst & 7));
        imm32(imm);
    }
    void lea_rbp(uint8_t dst, int32_t disp) { inst(0, true, false, {0x8D}, dst, Rm::rbp(disp)); }
    void alu_rr(Alu op, W w, uint8_t dst, uint8_t src) { gp(w, (uint8_t)((uint8_t)op * 8 + (w == W::B1 ? 0 : 1)), src, Rm::direct(dst)); }
    void alu_imm32(Alu op, W w, uint8_t dst, int32_t imm) {   // 32- and 64-bit forms only
        inst(0, w == W::B8, false, {0x81}, (uint8_t)op, Rm::direct(dst));
        imm32(imm);
    }
    void imul_rr(W w, uint8_t dst, uint8_t src) { inst(w == W::B2 ? 0x66 : 0, w == W::B8, false, {0x0F, 0xAF}, dst, Rm::direct(src)); }
    void sign_extend_acc(W w) {   // cwd / cdq / cqo
        if (w == W::B2) byte(0x66);
        if (w == W::B8) byte(0x48);
        byte(0x99);
    }
    void idiv(W w, uint8_t divisor) { inst(w == W::B2 ? 0x66 : 0, w == W::B8, false, {0xF7}, 7, Rm::direct(divisor)); }
    void shift_cl(Shift k, W w, uint8_t dst) { gp(w, w == W::B1 ? 0xD2 : 0xD3, (uint8_t)k, Rm::direct(dst)); }
    void shift_1(Shift k, W w, uint8_t dst) { gp(w, w == W::B1 ? 0xD0 : 0xD1, (uint8_t)k, Rm::direct(dst)); }
    void test_rr(W w, uint8_t r) { gp(w, w == W::B1 ? 0x84 : 0x85, r, Rm::direct(r)); }
    void movzx(W dw, W sw, uint8_t dst, Rm src) {
        inst(dw == W::B2 ? 0x66 : 0, dw == W::B8, sw == W::B1, {0x0F, (uint8_t)(sw == W::B1 ? 0xB6 : 0xB7)}, dst, src);
    }
    void movsx(W dw, W sw, uint8_t dst, Rm src) {
        if (sw == W::B4) { inst(0, true, false, {0x63}, dst, src); return; }
        inst(dw == W::B2 ? 0x66 : 0, dw == W::B8, sw == W::B1, {0x0F, (uint8_t)(sw == W::B1 ? 0xBE : 0xBF)}, dst, src);
    }
    // SSE scalar
    void fload(bool f64, uint8_t dst, Rm src) { inst(f64 ? 0xF2 : 0xF3, false, false, {0x0F, 0x10}, dst, src); }
    void fstore(bool f64, Rm dst, uint8_t src) { inst(f64 ? 0xF2 : 0xF3, false, false, {0x0F, 0x11}, src, dst); }
    void fmove(uint8_t dst, uint8_t src) { inst(0, false, false, {0x0F, 0x28}, dst, Rm::direct(src)); }
    void farith(Sse op, bool f64, uint8_t dst, uint8_t src) { inst(f64 ? 0xF2 : 0xF3, false, false, {0x0F, (uint8_t)op}, dst, Rm::direct(src)); }
    void ucomi(bool f64, uint8_t a, uint8_t b) { inst(f64 ? 0x66 : 0, false, false, {0x0F, 0x2E}, a, Rm::direct(b)); }
    void cvtss2sd(uint8_t dst, uint8_t src) { inst(0xF3, false, false, {0x0F, 0x5A}, dst, Rm::direct(src)); }
    void cvtsd2ss(uint8_t dst, uint8_t src) { inst(0xF2, false, false, {0x0F, 0x5A}, dst, Rm::direct(src)); }
    void cvtt_to_si(bool f64, W w, uint8_t dst_gpr, uint8_t src_xmm) { inst(f64 ? 0xF2 : 0xF3, w == W::B8, false, {0x0F, 0x2C}, dst_gpr, Rm::direct(src_xmm)); }
    void cvt_si_to(bool f64, W w, uint8_t dst_xmm, uint8_t src_gpr) { inst(f64 ? 0xF2 : 0xF3, w == W::B8, false, {0x0F, 0x2A}, dst_xmm, Rm::direct(src_gpr)); }
    void gpr_to_xmm(W w, uint8_t dst_xmm, uint8_t src_gpr) { inst(0x66, w == W::B8, false, {0x0F, 0x6E}, dst_xmm, Rm::direct(src_gpr)); }
    void xmm_to_gpr(W w, uint8_t dst_gpr, uint8_t src_xmm) { inst(0x66, w == W::B8, false, {0x0F, 0x7E}, src_xmm, Rm::direct(dst_gpr)); }

    bool finish(std::string* why) {
        for (auto& f : fixups_) {
            auto it = labels_.find(f.second);
            if (it == labels_.end()) { *why = "undefined label " + f.second; return false; }
            int64_t rel = (int64_t)it->second - (int64_t)(f.first + 4);
            for (int i = 0; i < 4; i++) code[f.first + i] = (uint8_t)((uint32_t)rel >> (8 * i));
        }
        return true;
    }

private:
    std::map<std::string, size_t> labels_;
    std::vector<std::pair<size_t, std::string>> fixups_;

    void byte(uint8_t b) { code.push_back(b); }
    void bytes(std::initializer_list<uint8_t> bs) { for (uint8_t b : bs) code.push_back(b); }
    void imm32(int32_t v) { for (int i = 0; i < 4; i++) byte((uint8_t)((uint32_t)v >> (8 * i))); }
    void fixup(const std::string& target) { fixups_.push_back({code.size(), target}); imm32(0); }

    // [prefix] [REX] opcode modrm [disp].  `byte_regs`: an operand is an 8-bit register, so sil/dil
    // need a REX prefix to be addressable.
    void inst(uint8_t prefix, bool rex_w, bool byte_regs, std::initializer_list<uint8_t> opcode, uint8_t reg, Rm rm) {
        if (prefix) byte(prefix);
        uint8_t rex = 0x40 | (rex_w ? 8 : 0) | (reg >= 8 ? 4 : 0) | (rm.reg >= 8 ? 1 : 0);
        bool need = rex != 0x40 || (byte_regs && ((reg >= 4 && reg < 8) || (rm.kind == Rm::Direct && rm.reg >= 4 && rm.reg < 8)));
        if (need) byte(rex);
        for (uint8_t b : opcode) byte(b);
        switch (rm.kind) {
            case Rm::Direct: byte(0xC0 | ((reg & 7) << 3) | (rm.reg & 7)); break;
            case Rm::RbpDisp: byte(0x80 | ((reg & 7) << 3) | 5); imm32(rm.disp); break;
            case Rm::IndBase:
                if ((rm.reg & 7) == 4) { byte(0x00 | ((reg & 7) << 3) | 4); byte(0x24); }            // rsp / r12: SIB
                else if ((rm.reg & 7) == 5) { byte(0x40 | ((reg & 7) << 3) | 5); byte(0); }          // rbp / r13: disp8 0
                else byte(0x00 | ((reg & 7) << 3) | (rm.reg & 7));
                break;
        }
    }
    void gp(W w, uint8_t opcode, uint8_t reg, Rm rm) { inst(w == W::B2 ? 0x66 : 0, w == W::B8, w == W::B1, {opcode}, reg, rm); }
};

// ---------------------------------------------------------------------------------------------------
// Linear-scan allocation
// ---------------------------------------------------------------------------------------------------
struct ValueId {
    bool inst;       // false: parameter (orders before every instruction result)
    uint32_t idx;
    bool operator<(const ValueId& o) const { return std::tie(inst, idx) < std::tie(o.inst, o.idx); }
    bool operator==(const ValueId& o) const { return inst == o.inst && idx == o.idx; }
};
ValueId vid(Val v) { return ValueId{!v.param, v.idx}; }

struct Location {
    bool is_float = false, spill = false;
    uint32_t idx = 0;
};

struct Allocation {
    std::map<ValueId, Location> loc;
    uint32_t int_spills = 0, float_spills = 0;
};

bool float_class(Ty t) { return t.kind == Ty::Sc && t.sc >= Scalar::F16; }

std::vector<uint32_t> successors(const Term& t) {
    switch (t.kind) {
        case Term::Br: return {t.t};
        case Term::CondBr: return {t.t, t.f};
        case Term::Switch: {
            std::vector<uint32_t> out{t.t};
            for (auto& c : t.cases) out.push_back(c.second);
            return out;
        }
        case Term::Ret: return {};
    }
    return {};
}

Allocation allocate(const Function& f, uint32_t int_regs, uint32_t float_regs) {
    size_t nb = f.blocks.size();
    std::vector<uint32_t> inst_block(f.insts.size(), 0), inst_pos(f.insts.size(), 0);
    std::vector<size_t> bstart(nb), bterm(nb);
    size_t pos = 0;
    for (size_t b = 0; b < nb; b++) {
        bstart[b] = pos;
        for (uint32_t id : f.blocks[b].insts) { inst_block[id] = (uint32_t)b; inst_pos[id] = (uint32_t)pos++; }
        bterm[b] = pos++;
    }
    auto def_block = [&](ValueId v) { return v.inst ? inst_block[v.idx] : 0u; };

    std::vector<std::set<ValueId>> defs(nb), uses(nb), live_in(nb), live_out(nb);
    std::map<ValueId, size_t> last_use;
    auto use_at = [&](ValueId v, size_t p) { auto it = last_use.find(v); if (it == last_use.end() || it->second < p) last_use[v] = p; };
    for (uint32_t p = 0; p < f.params.size(); p++) defs[0].insert(ValueId{false, p});
    for (size_t b = 0; b < nb; b++) {
        for (uint32_t id : f.blocks[b].insts) {
            const Inst& in = f.insts[id];
            if (in.has_result()) defs[b].insert(ValueId{true, id});
            if (in.op == Opc::Phi) {
                for (size_t i = 0; i < in.ops.size(); i++) {
                    uint32_t pred = in.phi_blocks[i];
                    ValueId v = vid(in.ops[i]);
                    if (def_block(v) != pred) uses[pred].insert(v);
                    use_at(v, bterm[pred]);
                }
            } else {
                for (Val o : in.ops) {
                    ValueId v = vid(o);
                    if (def_block(v) != b) uses[b].insert(v);
                    use_at(v, inst_pos[id]);
                }
            }
        }
        const Term& t = f.blocks[b].term;
        if (t.has_val) {
            ValueId v = vid(t.val);
            if (def_block(v) != b) uses[b].insert(v);
            use_at(v, bterm[b]);
        }
    }
    for (bool changed = true; changed;) {
        changed = false;
        for (size_t b = 0; b < nb; b++) {
            std::set<ValueId> out, in = uses[b];
            for (uint32_t s : successors(f.blocks[b].term)) out.insert(live_in[s].begin(), live_in[s].end());
            for (auto& v : out) if (!defs[b].count(v)) in.insert(v);
            if (in != live_in[b] || out != live_out[b]) changed = true;
            live_in[b] = std::move(in);
            live_out[b] = std::move(out);
        }
    }

    struct Interval { size_t start, end; ValueId v; bool is_float; };
    std::vector<Interval> ivs;
    auto add_value = [&](ValueId v, Ty ty, size_t def_pos) {
        size_t start = def_pos, end = def_pos;
        auto it = last_use.find(v);
        if (it != last_use.end()) end = std::max(end, it->second);
        for (size_t b = 0; b < nb; b++) {
            if (live_in[b].count(v)) { start = std::min(start, bstart[b]); end = std::max(end, bstart[b]); }
            if (live_out[b].count(v)) { start = std::min(start, bterm[b]); end = std::max(end, bterm[b]); }
        }
        ivs.push_back({start, end, v, float_class(ty)});
    };
    for (uint32_t p = 0; p < f.params.size(); p++) add_value(ValueId{false, p}, f.params[p], 0);
    for (uint32_t i = 0; i < f.insts.size(); i++) if (f.insts[i].has_result()) add_value(ValueId{true, i}, f.insts[i].ty, inst_pos[i]);
    std::sort(ivs.begin(), ivs.end(), [](const Interval& a, const Interval& b) { return std::tie(a.start, a.v) < std::tie(b.start, b.v); });

    struct ClassState {
        std::vector<bool> taken;
        std::vector<std::tuple<size_t, ValueId, uint32_t>> active;   // (end, value, register), kept sorted
        uint32_t spills = 0;
    } st[2];
    st[0].taken.assign(int_regs, false);
    st[1].taken.assign(float_regs, false);
    Allocation out;
    for (const Interval& iv : ivs) {
        ClassState& s = st[iv.is_float ? 1 : 0];
        // an interval that ends exactly where the new one starts still holds its register
        for (size_t i = 0; i < s.active.size();) {
            if (std::get<0>(s.active[i]) < iv.start) { s.taken[std::get<2>(s.active[i])] = false; s.active.erase(s.active.begin() + i); }
            else i++;
        }
        auto take = [&](uint32_t r) {
            s.taken[r] = true;
            s.active.push_back({iv.end, iv.v, r});
            std::sort(s.active.begin(), s.active.end());
            out.loc[iv.v] = Location{iv.is_float, false, r};
        };
        auto free_it = std::find(s.taken.begin(), s.taken.end(), false);
        if (free_it != s.taken.end()) { take((uint32_t)(free_it - s.taken.begin())); continue; }
        if (!s.active.empty() && std::get<0>(s.active.back()) > iv.end) {
            auto [end, victim, r] = s.active.back();
            (void)end;
            s.active.pop_back();
            out.loc[victim] = Location{iv.is_float, true, s.spills++};
            take(r);
        } else {
            out.loc[iv.v] = Location{iv.is_float, true, s.spills++};
        }
    }
    out.int_spills = st[0].spills;
    out.float_spills = st[1].spills;
    return out;
}

// ---------------------------------------------------------------------------------------------------
// Checks
// ---------------------------------------------------------------------------------------------------
const uint8_t kIntPool[4] = {RSI, RDI, R8, R9};
const uint8_t kFloatPool[5] = {3, 4, 5, 6, 7};
const uint8_t kIntArgs[6] = {RDI, RSI, RDX, RCX, R8, R9};

bool is_f16(Ty t) { return t.kind == Ty::Sc && t.sc == Scalar::F16; }
bool is_fp(Ty t) { return t.kind == Ty::Sc && (t.sc == Scalar::F32 || t.sc == Scalar::F64); }
bool is_f64(Ty t) { return t.kind == Ty::Sc && t.sc == Scalar::F64; }
W width_of(Ty t) {
    if (t.kind == Ty::Ptr) return W::B8;
    switch (t.sc) {
        case Scalar::I1: case Scalar::I8: return W::B1;
        case Scalar::I16: return W::B2;
        case Scalar::I32: case Scalar::F32: return W::B4;
        default: return W::B8;
    }
}
bool local_like(Space s) { return s != Space::Global; }

struct ArgLoc { bool sse; uint8_t reg; };
bool classify_params(const std::vector<Ty>& params, std::vector<ArgLoc>* locs, ArgLoc* nthreads) {
    size_t ni = 0, ns = 0;
    for (Ty t : params) {
        if (is_fp(t)) { if (ns >= 8) return false; locs->push_back({true, (uint8_t)ns++}); }
        else { if (ni >= 6) return false; locs->push_back({false, kIntArgs[ni++]}); }
    }
    if (ni >= 6) return false;
    *nthreads = {false, kIntArgs[ni]};
    return true;
}

bool refuse(Diag* d, const char* code, const char* arg) { d->code = code; d->arg = arg; return false; }

bool check(const Module& m, Diag* d) {
    if (m.funcs.size() != 1) return refuse(d, "E093", "multi-function module: one symbol per object");
    const Function& f = m.funcs[0];
    if (!f.is_kernel) return refuse(d, "E093", "host/non-kernel function compilation is not implemented");
    if (f.ret.is_vec()) return refuse(d, "E091", "vector-typed return value");
    for (Ty t : f.params) if (t.is_vec()) return refuse(d, "E091", "vector-typed parameter");
    if (is_f16(f.ret)) return refuse(d, "E091", "f16 return value needs F16C");
    for (Ty t : f.params) if (is_f16(t)) return refuse(d, "E091", "f16 parameter needs F16C");
    std::vector<ArgLoc> locs;
    ArgLoc nt;
    if (!classify_params(f.params, &locs, &nt))
        return refuse(d, "E093", "argument classes overflow SysV's 6 integer / 8 SSE registers (incl. trailing nthreads)");
    for (const Inst& in : f.insts) {
        if (in.ty.is_vec()) return refuse(d, "E091", "vector-typed instruction result");
        if (is_f16(in.ty)) return refuse(d, "E091", "f16 arithmetic needs F16C");
        switch (in.op) {
            case Opc::Shuffle: case Opc::Ballot: case Opc::VoteAny: case Opc::VoteAll: case Opc::WarpReduce:
                return refuse(d, "E090", "warp-collective op has no meaning under one-thread-at-a-time execution");
            case Opc::Cast: case Opc::FCmp:
                if (is_f16(in.aux)) return refuse(d, "E091", "f16 operand needs F16C");
                break;
            case Opc::Store:
                if (is_f16(in.aux)) return refuse(d, "E091", "f16 store needs F16C");
                if (in.aux.is_vec()) return refuse(d, "E091", "vector-typed store");
                break;
            case Opc::Mma: return refuse(d, "E090", "mma has no lowering in the regalloc-based x86-64 backend");
            case Opc::KernelLaunch: case Opc::CudaMalloc: case Opc::CudaMemcpy: case Opc::CudaFree: case Opc::CudaSync:
                return refuse(d, "E090", "kernel launch / CUDA Runtime API calls are sema-only");
            case Opc::Call: return refuse(d, "E090", "function calls have no lowering in the regalloc-based x86-64 backend");
            case Opc::VecExtract: case Opc::VecBuild: return refuse(d, "E091", "vector op");
            default: break;
        }
    }
    return true;
}

// ---------------------------------------------------------------------------------------------------
// Code generation
// ---------------------------------------------------------------------------------------------------
struct Frame {
    std::vector<int32_t> param_stage, int_spill, float_spill;
    int32_t nthreads_home = 0, retval_home = 0;
    std::map<uint32_t, int32_t> phi_stage;
    std::map<std::pair<int, int64_t>, int32_t> cell;   // (space, key) -> displacement of a local-like cell
    std::vector<std::pair<int32_t, int32_t>> zeroed;   // (displacement, bytes) of the cells a shared_obj line sizes
    int32_t size = 0;
};

struct OpLoc { bool mem; uint8_t reg; int32_t disp; };

class CodeGen {
public:
    CodeGen(const Module& m, const Function& f, const Allocation& a) : m_(m), f_(f), alloc_(a) {}
    Enc enc;

    bool run(std::string* why) {
        std::vector<ArgLoc> plocs;
        ArgLoc nthreads;
        classify_params(f_.params, &plocs, &nthreads);
        build_frame();
        for (size_t b = 0; b < f_.blocks.size(); b++)
            for (uint32_t id : f_.blocks[b].insts) {
                const Inst& in = f_.insts[id];
                if (in.op == Opc::Phi)
                    for (size_t i = 0; i < in.ops.size(); i++) phi_copies_[{in.phi_blocks[i], (uint32_t)b}].push_back({id, in.ops[i]});
            }

        enc.push(RBP);
        enc.mov_rbp_rsp();
        enc.sub_rsp(frame_.size);
        for (size_t i = 0; i < plocs.size(); i++) {
            Ty ty = f_.params[i];
            if (plocs[i].sse) enc.fstore(is_f64(ty), Rm::rbp(frame_.param_stage[i]), plocs[i].reg);
            else enc.store(width_of(ty), Rm::rbp(frame_.param_stage[i]), plocs[i].reg);
        }
        enc.store(W::B8, Rm::rbp(frame_.nthreads_home), nthreads.reg);
        // the argument registers are free now: clear the cells of sized shared arrays
        for (auto& z : frame_.zeroed) {
            enc.lea_rbp(RDI, z.first);
            enc.mov_imm32(W::B4, RCX, z.second / 8);
            enc.mov_imm32(W::B4, RAX, 0);
            enc.rep_stosq();
        }
        enc.mov_imm32(W::B8, R11, 0);

        enc.label("__loop_check");
        enc.load(W::B8, RAX, Rm::rbp(frame_.nthreads_home));
        enc.alu_rr(Alu::Cmp, W::B8, R11, RAX);
        enc.jcc(CC_GE, "__loop_end");
        place_params();
        for (size_t b = 0; b < f_.blocks.size(); b++) {
            enc.label(block_label((uint32_t)b));
            for (uint32_t id : f_.blocks[b].insts) lower(id);
            lower_term((uint32_t)b, f_.blocks[b].term);
        }
        enc.label("__loop_incr");
        enc.alu_imm32(Alu::Add, W::B8, R11, 1);
        enc.jmp("__loop_check");

        enc.label("__loop_end");
        if (!f_.ret.is_void()) {
            if (is_fp(f_.ret)) enc.fload(is_f64(f_.ret), 0, Rm::rbp(frame_.retval_home));
            else enc.load(width_of(f_.ret), RAX, Rm::rbp(frame_.retval_home));
        }
        enc.mov_rsp_rbp();
        enc.pop(RBP);
        enc.ret();
        return enc.finish(why);
    }

private:
    const Module& m_;
    const Function& f_;
    const Allocation& alloc_;
    Frame frame_;
    uint32_t labels_ = 0;
    std::map<std::pair<uint32_t, uint32_t>, std::vector<std::pair<uint32_t, Val>>> phi_copies_;

    static std::string block_label(uint32_t b) { return "bb" + std::to_string(b); }
    std::string fresh(const char* what) { return std::string("__") + what + "_" + std::to_string(++labels_); }

    void build_frame() {
        int32_t off = 0;
        auto slot = [&]() { off += 8; return -off; };
        for (size_t i = 0; i < f_.params.size(); i++) frame_.param_stage.push_back(slot());
        frame_.nthreads_home = slot();
        if (!f_.ret.is_void()) frame_.retval_home = slot();
        for (uint32_t i = 0; i < alloc_.int_spills; i++) frame_.int_spill.push_back(slot());
        for (uint32_t i = 0; i < alloc_.float_spills; i++) frame_.float_spill.push_back(slot());
        for (uint32_t i = 0; i < f_.insts.size(); i++) if (f_.insts[i].op == Opc::Phi) frame_.phi_stage[i] = slot();
        for (const Inst& in : f_.insts) {
            if (in.op != Opc::ConstI || !in.ty.is_ptr() || !local_like(in.ty.sp)) continue;
            std::pair<int, int64_t> key{(int)in.ty.sp, in.imm};
            if (frame_.cell.count(key)) continue;
            int32_t bytes = 8, align = 8;
            bool sized = false;
            if (in.ty.sp == Space::Shared)
                for (auto& so : m_.shared_objs)
                    if (so.key == in.imm) { bytes = (int32_t)((so.bytes + 7) & ~7u); align = std::max<int32_t>(8, std::min<uint32_t>(so.align, 16)); sized = true; }
            off += bytes;
            off = (off + align - 1) & ~(align - 1);
            frame_.cell[key] = -off;
            if (sized) frame_.zeroed.push_back({-off, bytes});
        }
        frame_.size = (off + 15) & ~15;
    }

    OpLoc loc_of(ValueId v) const {
        const Location& l = alloc_.loc.at(v);
        if (l.is_float) return l.spill ? OpLoc{true, 0, frame_.float_spill[l.idx]} : OpLoc{false, kFloatPool[l.idx], 0};
        return l.spill ? OpLoc{true, 0, frame_.int_spill[l.idx]} : OpLoc{false, kIntPool[l.idx], 0};
    }
    Rm rm_of(const OpLoc& l) const { return l.mem ? Rm::rbp(l.disp) : Rm::direct(l.reg); }

    // operand reads
    void load_gpr(Val v, uint8_t dst, W w) {
        OpLoc l = loc_of(vid(v));
        if (l.mem) enc.load(w, dst, Rm::rbp(l.disp));
        else if (l.reg != dst) enc.mov_rr(w, dst, l.reg);
    }
    void load_gpr_zx(Val v, uint8_t dst, W dw, W sw) {
        OpLoc l = loc_of(vid(v));
        if (sw == W::B1 || sw == W::B2) enc.movzx(dw, sw, dst, rm_of(l));
        else if (l.mem) enc.load(sw, dst, Rm::rbp(l.disp));
        else enc.mov_rr(sw, dst, l.reg);     // a 32-bit write clears the upper half
    }
    void load_gpr_sx(Val v, uint8_t dst, W dw, W sw) {
        OpLoc l = loc_of(vid(v));
        if (sw == W::B1 || sw == W::B2) enc.movsx(dw, sw, dst, rm_of(l));
        else if (sw == W::B4) enc.movsx(W::B8, W::B4, dst, rm_of(l));
        else if (l.mem) enc.load(W::B8, dst, Rm::rbp(l.disp));
        else enc.mov_rr(W::B8, dst, l.reg);
    }
    void load_xmm(Val v, uint8_t dst, bool f64) {
        OpLoc l = loc_of(vid(v));
        if (l.mem) enc.fload(f64, dst, Rm::rbp(l.disp));
        else if (l.reg != dst) enc.fmove(dst, l.reg);
    }
    // result placement
    void place_gpr(ValueId v, uint8_t src, W w) {
        OpLoc l = loc_of(v);
        if (l.mem) enc.store(w, Rm::rbp(l.disp), src);
        else if (l.reg != src) enc.mov_rr(w, l.reg, src);
    }
    void place_gpr(uint32_t id, uint8_t src, W w) { place_gpr(ValueId{true, id}, src, w); }
    void place_xmm(ValueId v, uint8_t src, bool f64) {
        OpLoc l = loc_of(v);
        if (l.mem) enc.fstore(f64, Rm::rbp(l.disp), src);
        else if (l.reg != src) enc.fmove(l.reg, src);
    }
    void place_xmm(uint32_t id, uint8_t src, bool f64) { place_xmm(ValueId{true, id}, src, f64); }
    void copy_value(Val v, uint32_t id, Ty ty) {
        if (is_fp(ty)) { load_xmm(v, 0, is_f64(ty)); place_xmm(id, 0, is_f64(ty)); }
        else { load_gpr(v, RAX, width_of(ty)); place_gpr(id, RAX, width_of(ty)); }
    }
    void place_params() {
        for (uint32_t i = 0; i < f_.params.size(); i++) {
            Ty ty = f_.params[i];
            if (is_fp(ty)) { enc.fload(is_f64(ty), 0, Rm::rbp(frame_.param_stage[i])); place_xmm(ValueId{false, i}, 0, is_f64(ty)); }
            else { enc.load(width_of(ty), RAX, Rm::rbp(frame_.param_stage[i])); place_gpr(ValueId{false, i}, RAX, width_of(ty)); }
        }
    }

    void lower(uint32_t id) {
        const Inst& in = f_.insts[id];
        Ty ty = in.ty;
        switch (in.op) {
            case Opc::ConstI:
                if (ty.is_ptr() && local_like(ty.sp)) {
                    enc.lea_rbp(RAX, frame_.cell.at({(int)ty.sp, in.imm}));
                    place_gpr(id, RAX, W::B8);
                } else {
                    enc.movabs(RAX, in.imm);
                    place_gpr(id, RAX, width_of(ty));
                }
                break;
            case Opc::ConstF:
                if (is_f64(ty)) {
                    int64_t bits;
                    std::memcpy(&bits, &in.fimm, 8);
                    enc.movabs(RAX, bits);
                    enc.gpr_to_xmm(W::B8, 0, RAX);
                    place_xmm(id, 0, true);
                } else {
                    float fv = (float)in.fimm;
                    int32_t bits;
                    std::memcpy(&bits, &fv, 4);
                    enc.mov_imm32(W::B4, RAX, bits);
                    enc.gpr_to_xmm(W::B4, 0, RAX);
                    place_xmm(id, 0, false);
                }
                break;
            case Opc::Bin: lower_bin(id, (BinOp)in.sub, in.ops[0], in.ops[1], ty); break;
            case Opc::ICmp: {
                W w = width_of(in.aux);
                load_gpr(in.ops[0], RAX, w);
                load_gpr(in.ops[1], RCX, w);
                enc.alu_rr(Alu::Cmp, w, RAX, RCX);
                static const uint8_t cc[] = {CC_E, CC_NE, CC_L, CC_LE, CC_G, CC_GE, CC_B, CC_BE, CC_A, CC_AE};
                enc.setcc(cc[in.sub], RAX);
                place_gpr(id, RAX, W::B1);
                break;
            }
            case Opc::FCmp: lower_fcmp(id, (FCmp)in.sub, in.aux, in.ops[0], in.ops[1]); break;
            case Opc::Select: {
                load_gpr(in.ops[0], RAX, W::B1);
                enc.test_rr(W::B1, RAX);
                std::string other = fresh("select_false"), end = fresh("select_end");
                enc.jcc(CC_E, other);
                copy_value(in.ops[1], id, ty);
                enc.jmp(end);
                enc.label(other);
                copy_value(in.ops[2], id, ty);
                enc.label(end);
                break;
            }
            case Opc::Cast: lower_cast(id, (CastOp)in.sub, in.aux, in.ops[0], ty); break;
            case Opc::Load:
                load_gpr(in.ops[0], R10, W::B8);
                if (is_fp(ty)) { enc.fload(is_f64(ty), 0, Rm::ind(R10)); place_xmm(id, 0, is_f64(ty)); }
                else { enc.load(width_of(ty), RAX, Rm::ind(R10)); place_gpr(id, RAX, width_of(ty)); }
                break;
            case Opc::Store:
                load_gpr(in.ops[0], R10, W::B8);
                if (is_fp(in.aux)) { load_xmm(in.ops[1], 0, is_f64(in.aux)); enc.fstore(is_f64(in.aux), Rm::ind(R10), 0); }
                else { load_gpr(in.ops[1], RAX, width_of(in.aux)); enc.store(width_of(in.aux), Rm::ind(R10), RAX); }
                break;
            case Opc::Phi: break;   // every predecessor writes the phi's location before it jumps
            case Opc::Index:
                if (in.sub == 0) place_gpr(id, R11, width_of(ty));                                  // tid.x: the loop counter
                else if (in.sub == 6) { enc.load(W::B8, RAX, Rm::rbp(frame_.nthreads_home)); place_gpr(id, RAX, width_of(ty)); }   // bdim.x
                else { enc.movabs(RAX, in.sub < 6 ? 0 : 1); place_gpr(id, RAX, width_of(ty)); }   // other tid/bid = 0, other extents = 1
                break;
            case Opc::Barrier: enc.nop(); break;
            case Opc::Atomic: lower_atomic(id, (AtomOp)in.sub, in.ops[0], in.ops[1], ty); break;
            case Opc::AtomicCas: {
                W w = width_of(ty);
                load_gpr(in.ops[0], R10, W::B8);
                enc.load(w, RAX, Rm::ind(R10));
                load_gpr(in.ops[1], RCX, w);
                enc.alu_rr(Alu::Cmp, w, RAX, RCX);
                std::string mismatch = fresh("cas_mismatch");
                enc.jcc(CC_NE, mismatch);
                load_gpr(in.ops[2], RDX, w);
                enc.store(w, Rm::ind(R10), RDX);
                enc.label(mismatch);
                place_gpr(id, RAX, w);
                break;
            }
            default: break;   // refused by check()
        }
    }

    void lower_bin(uint32_t id, BinOp op, Val a, Val b, Ty ty) {
        if (is_fp(ty)) {
            bool f64 = is_f64(ty);
            load_xmm(a, 0, f64);
            load_xmm(b, 1, f64);
            switch (op) {
                case BinOp::FAdd: enc.farith(Sse::Add, f64, 0, 1); break;
                case BinOp::FSub: enc.farith(Sse::Sub, f64, 0, 1); break;
                case BinOp::FMul: enc.farith(Sse::Mul, f64, 0, 1); break;
                case BinOp::FDiv: enc.farith(Sse::Div, f64, 0, 1); break;
                default:   // frem: a - trunc(a / b) * b
                    enc.fmove(2, 0);
                    enc.farith(Sse::Div, f64, 0, 1);
                    enc.cvtt_to_si(f64, W::B8, RAX, 0);
                    enc.cvt_si_to(f64, W::B8, 0, RAX);
                    enc.farith(Sse::Mul, f64, 0, 1);
                    enc.fmove(1, 2);
                    enc.farith(Sse::Sub, f64, 1, 0);
                    enc.fmove(0, 1);
                    break;
            }
            place_xmm(id, 0, f64);
            return;
        }
        W w = width_of(ty);
        switch (op) {
            case BinOp::Add: case BinOp::Sub: case BinOp::And: case BinOp::Or: case BinOp::Xor: {
                load_gpr(a, RAX, w);
                load_gpr(b, RCX, w);
                Alu alu = op == BinOp::Add ? Alu::Add : op == BinOp::Sub ? Alu::Sub : op == BinOp::And ? Alu::And : op == BinOp::Or ? Alu::Or : Alu::Xor;
                enc.alu_rr(alu, w, RAX, RCX);
                place_gpr(id, RAX, w);
                break;
            }
            case BinOp::Mul:
                if (w == W::B1) {
                    load_gpr_zx(a, RAX, W::B4, W::B1);
                    load_gpr_zx(b, RCX, W::B4, W::B1);
                    enc.imul_rr(W::B4, RAX, RCX);
                } else {
                    load_gpr(a, RAX, w);
                    load_gpr(b, RCX, w);
                    enc.imul_rr(w, RAX, RCX);
                }
                place_gpr(id, RAX, w);
                break;
            case BinOp::Div: case BinOp::Rem: {
                W dw = w == W::B1 ? W::B4 : w;
                if (w == W::B1) { load_gpr_sx(a, RAX, W::B4, W::B1); load_gpr_sx(b, R10, W::B4, W::B1); }
                else { load_gpr(a, RAX, w); load_gpr(b, R10, w); }
                enc.sign_extend_acc(dw);
                enc.idiv(dw, R10);
                place_gpr(id, op == BinOp::Div ? RAX : RDX, w);
                break;
            }
            case BinOp::Shl: case BinOp::LShr: case BinOp::AShr:
                load_gpr(a, RAX, w);
                load_gpr(b, RCX, w);
                enc.shift_cl(op == BinOp::Shl ? Shift::Shl : op == BinOp::LShr ? Shift::Shr : Shift::Sar, w, RAX);
                place_gpr(id, RAX, w);
                break;
            default: break;
        }
    }

    // ucomis sets ZF, PF, CF: unordered = all three; a > b none; a < b CF; a == b ZF.
    void lower_fcmp(uint32_t id, FCmp pred, Ty cty, Val a, Val b) {
        bool f64 = is_f64(cty);
        load_xmm(a, 0, f64);
        load_xmm(b, 1, f64);
        enc.ucomi(f64, 0, 1);
        auto both = [&](uint8_t c1, uint8_t c2) { enc.setcc(c1, RAX); enc.setcc(c2, RCX); enc.alu_rr(Alu::And, W::B1, RAX, RCX); };
        switch (pred) {
            case FCmp::Ogt: enc.setcc(CC_A, RAX); break;
            case FCmp::Oge: enc.setcc(CC_AE, RAX); break;
            case FCmp::Ord: enc.setcc(CC_NP, RAX); break;
            case FCmp::Uno: enc.setcc(CC_P, RAX); break;
            case FCmp::Olt: both(CC_B, CC_NE); break;     // unordered also sets ZF
            case FCmp::Ole: both(CC_BE, CC_NP); break;
            case FCmp::Oeq: both(CC_E, CC_NP); break;
            case FCmp::One: both(CC_NE, CC_NP); break;
        }
        place_gpr(id, RAX, W::B1);
    }

    void lower_cast(uint32_t id, CastOp op, Ty sty, Val v, Ty dty) {
        switch (op) {
            case CastOp::Trunc: load_gpr(v, RAX, width_of(dty)); place_gpr(id, RAX, width_of(dty)); break;
            case CastOp::ZExt: load_gpr_zx(v, RAX, width_of(dty), width_of(sty)); place_gpr(id, RAX, width_of(dty)); break;
            case CastOp::SExt: load_gpr_sx(v, RAX, width_of(dty), width_of(sty)); place_gpr(id, RAX, width_of(dty)); break;
            case CastOp::FPTrunc: load_xmm(v, 0, true); enc.cvtsd2ss(0, 0); place_xmm(id, 0, false); break;
            case CastOp::FPExt: load_xmm(v, 0, false); enc.cvtss2sd(0, 0); place_xmm(id, 0, true); break;
            case CastOp::FPToSI:
                load_xmm(v, 0, is_f64(sty));
                enc.cvtt_to_si(is_f64(sty), width_of(dty) == W::B8 ? W::B8 : W::B4, RAX, 0);
                place_gpr(id, RAX, width_of(dty));
                break;
            case CastOp::FPToUI: {
                bool f64 = is_f64(sty);
                load_xmm(v, 0, f64);
                if (width_of(dty) != W::B8) { enc.cvtt_to_si(f64, W::B8, RAX, 0); place_gpr(id, RAX, width_of(dty)); break; }
                // values of 2^63 and above: convert v - 2^63 and set the top bit
                int64_t two63;
                if (f64) { double dv = 9223372036854775808.0; std::memcpy(&two63, &dv, 8); }
                else { float fv = 9223372036854775808.0f; uint32_t b; std::memcpy(&b, &fv, 4); two63 = b; }
                enc.movabs(RCX, two63);
                enc.gpr_to_xmm(f64 ? W::B8 : W::B4, 1, RCX);
                enc.ucomi(f64, 0, 1);
                std::string hi = fresh("fptoui_hi"), done = fresh("fptoui_done");
                enc.jcc(CC_AE, hi);
                enc.cvtt_to_si(f64, W::B8, RAX, 0);
                enc.jmp(done);
                enc.label(hi);
                enc.farith(Sse::Sub, f64, 0, 1);
                enc.cvtt_to_si(f64, W::B8, RAX, 0);
                enc.movabs(RCX, INT64_MIN);
                enc.alu_rr(Alu::Xor, W::B8, RAX, RCX);
                enc.label(done);
                place_gpr(id, RAX, W::B8);
                break;
            }
            case CastOp::SIToFP: {
                W sw = width_of(sty);
                if (sw == W::B1 || sw == W::B2) load_gpr_sx(v, RAX, W::B4, sw);
                else load_gpr(v, RAX, sw);
                enc.cvt_si_to(is_f64(dty), sw == W::B8 ? W::B8 : W::B4, 0, RAX);
                place_xmm(id, 0, is_f64(dty));
                break;
            }
            case CastOp::UIToFP: {
                bool f64 = is_f64(dty);
                W sw = width_of(sty);
                if (sw != W::B8) {
                    if (sw == W::B4) load_gpr(v, RAX, W::B4);
                    else load_gpr_zx(v, RAX, W::B8, sw);
                    enc.cvt_si_to(f64, W::B8, 0, RAX);
                    place_xmm(id, 0, f64);
                    break;
                }
                // top bit set: halve with the lost bit or-ed back in (round to odd), convert, double
                load_gpr(v, RAX, W::B8);
                enc.test_rr(W::B8, RAX);
                std::string hi = fresh("uitofp_hi"), done = fresh("uitofp_done");
                enc.jcc(CC_S, hi);
                enc.cvt_si_to(f64, W::B8, 0, RAX);
                enc.jmp(done);
                enc.label(hi);
                enc.mov_rr(W::B8, RCX, RAX);
                enc.alu_imm32(Alu::And, W::B8, RCX, 1);
                enc.shift_1(Shift::Shr, W::B8, RAX);
                enc.alu_rr(Alu::Or, W::B8, RAX, RCX);
                enc.cvt_si_to(f64, W::B8, 0, RAX);
                enc.farith(Sse::Add, f64, 0, 0);
                enc.label(done);
                place_xmm(id, 0, f64);
                break;
            }
            case CastOp::Bitcast: {
                bool sf = is_fp(sty), df = is_fp(dty);
                W w = width_of(dty);
                if (!sf && df) { load_gpr(v, RAX, w); enc.gpr_to_xmm(w, 0, RAX); place_xmm(id, 0, w == W::B8); }
                else if (sf && !df) { load_xmm(v, 0, is_f64(sty)); enc.xmm_to_gpr(w, RAX, 0); place_gpr(id, RAX, w); }
                else if (sf) { load_xmm(v, 0, is_f64(sty)); place_xmm(id, 0, is_f64(dty)); }
                else { load_gpr(v, RAX, w); place_gpr(id, RAX, w); }
                break;
            }
        }
    }

    // One thread runs at a time, so an atomic is load, compute, store; the old value is the result.
    void lower_atomic(uint32_t id, AtomOp op, Val ptr, Val val, Ty ty) {
        load_gpr(ptr, R10, W::B8);
        if (is_fp(ty)) {
            bool f64 = is_f64(ty);
            enc.fload(f64, 0, Rm::ind(R10));
            enc.fmove(2, 0);
            load_xmm(val, 1, f64);
            switch (op) {
                case AtomOp::Add: enc.farith(Sse::Add, f64, 0, 1); break;
                case AtomOp::Sub: enc.farith(Sse::Sub, f64, 0, 1); break;
                case AtomOp::Exch: enc.fmove(0, 1); break;
                case AtomOp::Min: case AtomOp::Max: {
                    enc.ucomi(f64, 0, 1);
                    std::string skip = fresh("atomic_minmax_skip");
                    enc.jcc(op == AtomOp::Min ? CC_BE : CC_AE, skip);
                    enc.fmove(0, 1);
                    enc.label(skip);
                    break;
                }
                default: {
                    W w = f64 ? W::B8 : W::B4;
                    enc.xmm_to_gpr(w, RAX, 0);
                    enc.xmm_to_gpr(w, RCX, 1);
                    enc.alu_rr(op == AtomOp::And ? Alu::And : op == AtomOp::Or ? Alu::Or : Alu::Xor, w, RAX, RCX);
                    enc.gpr_to_xmm(w, 0, RAX);
                    break;
                }
            }
            enc.fstore(f64, Rm::ind(R10), 0);
            if (!ty.is_void()) place_xmm(id, 2, f64);
            return;
        }
        W w = width_of(ty);
        enc.load(w, RAX, Rm::ind(R10));
        enc.mov_rr(w, RDX, RAX);
        load_gpr(val, RCX, w);
        switch (op) {
            case AtomOp::Add: enc.alu_rr(Alu::Add, w, RAX, RCX); break;
            case AtomOp::Sub: enc.alu_rr(Alu::Sub, w, RAX, RCX); break;
            case AtomOp::And: enc.alu_rr(Alu::And, w, RAX, RCX); break;
            case AtomOp::Or: enc.alu_rr(Alu::Or, w, RAX, RCX); break;
            case AtomOp::Xor: enc.alu_rr(Alu::Xor, w, RAX, RCX); break;
            case AtomOp::Exch: enc.mov_rr(w, RAX, RCX); break;
            case AtomOp::Min: case AtomOp::Max: {
                enc.alu_rr(Alu::Cmp, w, RAX, RCX);
                std::string skip = fresh("atomic_minmax_skip");
                enc.jcc(op == AtomOp::Min ? CC_LE : CC_GE, skip);
                enc.mov_rr(w, RAX, RCX);
                enc.label(skip);
                break;
            }
        }
        enc.store(w, Rm::ind(R10), RAX);
        place_gpr(id, RDX, w);
    }

    // Stage every incoming value first, then move the staged values into the phis' own locations:
    // two phis of one block may sit in each other's source registers.
    void emit_phi_copies(uint32_t from, uint32_t to) {
        auto it = phi_copies_.find({from, to});
        if (it == phi_copies_.end()) return;
        for (auto& c : it->second) {
            Ty ty = f_.insts[c.first].ty;
            int32_t stage = frame_.phi_stage.at(c.first);
            if (is_fp(ty)) { load_xmm(c.second, 0, is_f64(ty)); enc.fstore(is_f64(ty), Rm::rbp(stage), 0); }
            else { load_gpr(c.second, RAX, width_of(ty)); enc.store(width_of(ty), Rm::rbp(stage), RAX); }
        }
        for (auto& c : it->second) {
            Ty ty = f_.insts[c.first].ty;
            int32_t stage = frame_.phi_stage.at(c.first);
            if (is_fp(ty)) { enc.fload(is_f64(ty), 0, Rm::rbp(stage)); place_xmm(c.first, 0, is_f64(ty)); }
            else { enc.load(width_of(ty), RAX, Rm::rbp(stage)); place_gpr(c.first, RAX, width_of(ty)); }
        }
    }

    void lower_term(uint32_t from, const Term& t) {
        switch (t.kind) {
            case Term::Br:
                emit_phi_copies(from, t.t);
                enc.jmp(block_label(t.t));
                break;
            case Term::CondBr: {
                load_gpr(t.val, RAX, W::B1);
                enc.test_rr(W::B1, RAX);
                std::string other = fresh("condbr_false");
                enc.jcc(CC_E, other);
                emit_phi_copies(from, t.t);
                enc.jmp(block_label(t.t));
                enc.label(other);
                emit_phi_copies(from, t.f);
                enc.jmp(block_label(t.f));
                break;
            }
            case Term::Switch: {
                W w = width_of(f_.val_ty(t.val));
                load_gpr(t.val, RAX, w);
                for (auto& c : t.cases) {
                    enc.movabs(RCX, c.first);
                    enc.alu_rr(Alu::Cmp, w, RAX, RCX);
                    std::string skip = fresh("switch_skip");
                    enc.jcc(CC_NE, skip);
                    emit_phi_copies(from, c.second);
                    enc.jmp(block_label(c.second));
                    enc.label(skip);
                }
                emit_phi_copies(from, t.t);
                enc.jmp(block_label(t.t));
                break;
            }
            case Term::Ret:
                if (t.has_val) {
                    if (is_fp(f_.ret)) { load_xmm(t.val, 0, is_f64(f_.ret)); enc.fstore(is_f64(f_.ret), Rm::rbp(frame_.retval_home), 0); }
                    else { load_gpr(t.val, RAX, width_of(f_.ret)); enc.store(width_of(f_.ret), Rm::rbp(frame_.retval_home), RAX); }
                }
                enc.jmp("__loop_incr");
                break;
        }
    }
};

struct Kernel {
    std::vector<uint8_t> code;
    void* exec = nullptr;
    size_t mapped = 0;
    std::string signature, name;
    uint32_t int_spills = 0, float_spills = 0, frame_mem_ops = 0;
};

void set_msg(char* buf, size_t n, const std::string& s) {
    if (!buf || !n) return;
    std::snprintf(buf, n, "%s", s.c_str());
}

}  // namespace

#define ORX_API extern "C" __attribute__((visibility("default")))

// Compiles one BIR module.  0 = ok, 1 = refused (code8 holds the E-code), 2 = could not map executable memory.
ORX_API int orx_compile(const char* bir, size_t len, void** out, char* code8, char* msg, size_t msglen) {
    Module m;
    ParseError pe;
    if (!parse_module(bir, len, &m, &pe)) { std::snprintf(code8, 8, "E400"); set_msg(msg, msglen, pe.text()); return 1; }
    std::string why;
    if (!verify_module(m, &why)) { std::snprintf(code8, 8, "E400"); set_msg(msg, msglen, why); return 1; }
    Diag d;
    if (!check(m, &d)) { std::snprintf(code8, 8, "%s", d.code.c_str()); set_msg(msg, msglen, d.arg); return 1; }
    Function& f = m.funcs[0];
    construct_ssa(f);
    canonicalize(f);
    Allocation a = allocate(f, 4, 5);
    CodeGen cg(m, f, a);
    if (!cg.run(&why)) { std::snprintf(code8, 8, "E099"); set_msg(msg, msglen, why); return 1; }
    Kernel* k = new Kernel;
    k->code = std::move(cg.enc.code);
    k->name = f.name;
    k->int_spills = a.int_spills;
    k->float_spills = a.float_spills;
    for (Ty t : f.params) k->signature += ty_text(t) + " ";
    k->signature += "-> " + ty_text(f.ret);
    k->mapped = (k->code.size() + 4095) & ~(size_t)4095;
    void* p = mmap(nullptr, k->mapped, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
    if (p == MAP_FAILED) { delete k; set_msg(msg, msglen, "mmap failed"); return 2; }
    std::memcpy(p, k->code.data(), k->code.size());
    if (mprotect(p, k->mapped, PROT_READ | PROT_EXEC) != 0) { munmap(p, k->mapped); delete k; set_msg(msg, msglen, "mprotect(PROT_EXEC) failed"); return 2; }
    k->exec = p;
    *out = k;
    return 0;
}

ORX_API void* orx_entry(void* k) { return ((Kernel*)k)->exec; }
ORX_API size_t orx_code(void* k, const uint8_t** bytes) { *bytes = ((Kernel*)k)->code.data(); return ((Kernel*)k)->code.size(); }
ORX_API const char* orx_signature(void* k) { return ((Kernel*)k)->signature.c_str(); }
ORX_API const char* orx_name(void* k) { return ((Kernel*)k)->name.c_str(); }
ORX_API void orx_spills(void* k, uint32_t* ints, uint32_t* floats) { *ints = ((Kernel*)k)->int_spills; *floats = ((Kernel*)k)->float_spills; }
ORX_API void orx_free(void* k) {
    Kernel* kk = (Kernel*)k;
    if (kk->exec) munmap(kk->exec, kk->mapped);
    delete kk;
}
