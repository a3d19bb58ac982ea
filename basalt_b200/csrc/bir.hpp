// BIR data model, text parser and printer for the sm_100a backend.
//
// BIR is the reference compiler's typed-SSA IR; its textual form is a first-class input of the
// reference CLI (crates/basalt-cli/src/main.rs:517-520) and round-trips exactly
// (crates/basalt-bir/src/lib.rs:10-13).  Because this backend is not written in Rust, a module
// crosses the Backend boundary as that text.  The grammar accepted and printed here is the
// reference's (crates/basalt-bir/src/lib.rs:21-68 plus the call / kernel.launch / cuda.* forms of
// crates/basalt-bir/src/print.rs:200-259), with these optional additions that a reference-printed
// file never contains:
//   * `shared_obj <K> bytes <n> align <a>` lines after `target_dtypes`: the byte size of the
//     storage cell that the synthetic address `const.i ptr.shared K` names (the reference backs
//     every such cell with 8 bytes, crates/basalt-ptx/src/emit.rs:630-660, so it cannot hold an
//     array);
//   * `mma ... k <k> [ld <lda> <ldb> <ldc> <ldd>] [out <ty>] a, b, c, d`: explicit leading
//     dimensions (elements; 0 = the operand's own extent as in the reference) and a result type
//     narrower than the accumulator;
//   * `vec.extract <ty> <vec>, <lane>` / `vec.build <vty> [v0, ...]` / `warp.reduce.<op> <ty> <v>`:
//     produced only by this backend's own BIR-to-BIR passes, printable so that the optimised module
//     can be dumped and run through the CPU oracle interpreter.
#pragma once
#include <cstdint>
#include <string>
#include <utility>
#include <vector>

namespace basalt {

enum class Scalar : uint8_t { I1, I8, I16, I32, I64, F16, F32, F64 };
enum class Space : uint8_t { Global, Shared, Constant, Local, Param };

struct Ty {
    enum Kind : uint8_t { Void, Sc, Ptr, Vec } kind = Void;
    Scalar sc = Scalar::I32;
    Space sp = Space::Global;
    uint8_t lanes = 0;
    static Ty v() { return Ty{}; }
    static Ty s(Scalar s) { Ty t; t.kind = Sc; t.sc = s; return t; }
    static Ty p(Space s) { Ty t; t.kind = Ptr; t.sp = s; return t; }
    static Ty vec(Scalar s, uint8_t n) { Ty t; t.kind = Vec; t.sc = s; t.lanes = n; return t; }
    bool operator==(const Ty& o) const {
        if (kind != o.kind) return false;
        switch (kind) {
            case Void: return true;
            case Sc: return sc == o.sc;
            case Ptr: return sp == o.sp;
            case Vec: return sc == o.sc && lanes == o.lanes;
        }
        return false;
    }
    bool operator!=(const Ty& o) const { return !(*this == o); }
    bool is_void() const { return kind == Void; }
    bool is_ptr() const { return kind == Ptr; }
    bool is_vec() const { return kind == Vec; }
    bool is_sc(Scalar s) const { return kind == Sc && sc == s; }
    bool is_float() const { return (kind == Sc || kind == Vec) && sc >= Scalar::F16; }
    bool has_f16() const { return (kind == Sc || kind == Vec) && sc == Scalar::F16; }
};

const char* scalar_text(Scalar s);
const char* space_text(Space s);
unsigned scalar_bytes(Scalar s);
unsigned scalar_bits(Scalar s);
std::string ty_text(Ty t);
bool parse_ty(const std::string& w, Ty* out);
bool parse_scalar(const std::string& w, Scalar* out);

struct Val {
    bool param = false;
    uint32_t idx = 0;
    static Val P(uint32_t i) { Val v; v.param = true; v.idx = i; return v; }
    static Val V(uint32_t i) { Val v; v.param = false; v.idx = i; return v; }
    bool operator==(const Val& o) const { return param == o.param && idx == o.idx; }
    bool operator!=(const Val& o) const { return !(*this == o); }
};

enum class Opc : uint8_t {
    ConstI, ConstF, Bin, ICmp, FCmp, Select, Cast, Load, Store, Phi, Index, Barrier, Shuffle, Ballot,
    VoteAny, VoteAll, Atomic, AtomicCas, Mma, KernelLaunch, CudaMalloc, CudaMemcpy, CudaFree, CudaSync,
    Call,
    // backend-pass products (see the file header)
    VecExtract, VecBuild, WarpReduce
};
enum class BinOp : uint8_t { Add, Sub, Mul, Div, Rem, FAdd, FSub, FMul, FDiv, FRem, And, Or, Xor, Shl, LShr, AShr };
enum class ICmp : uint8_t { Eq, Ne, Slt, Sle, Sgt, Sge, Ult, Ule, Ugt, Uge };
enum class FCmp : uint8_t { Oeq, One, Olt, Ole, Ogt, Oge, Ord, Uno };
enum class CastOp : uint8_t { Trunc, ZExt, SExt, FPTrunc, FPExt, FPToSI, FPToUI, SIToFP, UIToFP, Bitcast };
enum class Shfl : uint8_t { Idx, Up, Down, Xor };
enum class AtomOp : uint8_t { Add, Sub, Exch, Min, Max, And, Or, Xor };
// Index sub-op: 0..11 = tid.x,y,z, bid.x,y,z, bdim.x,y,z, gdim.x,y,z
enum class RedOp : uint8_t { Max, Min, Add, And, Or, Xor };

const char* binop_text(BinOp);
const char* icmp_text(ICmp);
const char* fcmp_text(FCmp);
const char* cast_text(CastOp);
const char* shfl_text(Shfl);
const char* atom_text(AtomOp);
const char* index_text(unsigned sub);
const char* redop_text(RedOp);

struct Inst {
    Opc op = Opc::ConstI;
    Ty ty;               // result type; Void for store / barrier / mma / void calls / host ops
    uint8_t sub = 0;     // BinOp, ICmp, FCmp, CastOp, Shfl, AtomOp, index selector, RedOp, or lane
    Ty aux;              // icmp/fcmp operand type, cast source type, store value type
    Space space = Space::Global;   // load / store / atomic address space
    uint32_t align = 0;
    bool vol = false;
    int64_t imm = 0;     // const.i
    double fimm = 0;     // const.f
    std::vector<Val> ops;
    std::vector<uint32_t> phi_blocks;   // phi: predecessor of ops[i]
    // mma
    uint32_t m = 0, n = 0, k = 0;
    Scalar in_dt = Scalar::F32, acc_dt = Scalar::F32, out_dt = Scalar::F32;
    bool a_col = false, b_col = false, has_ld = false, has_out = false;
    int64_t ld[4] = {0, 0, 0, 0};
    // call / kernel.launch
    std::string callee;
    bool has_result() const { return !ty.is_void(); }
};

struct Term {
    enum Kind : uint8_t { Br, CondBr, Switch, Ret } kind = Ret;
    bool has_val = false;   // condbr / switch scrutinee / ret value
    Val val;
    uint32_t t = 0, f = 0;  // br target / condbr true,false / switch default in t
    std::vector<std::pair<int64_t, uint32_t>> cases;
};

struct Block {
    std::vector<uint32_t> insts;
    Term term;
};

struct Function {
    std::string name;
    bool is_kernel = true;
    std::vector<Ty> params;
    Ty ret;
    std::vector<Block> blocks;
    std::vector<Inst> insts;   // arena; %N is the arena index
    Ty val_ty(Val v) const { return v.param ? params[v.idx] : insts[v.idx].ty; }
};

struct SharedObj {
    int64_t key = 0;
    uint32_t bytes = 0, align = 0;
};

struct Module {
    std::vector<Function> funcs;
    bool has_launch_bounds = false;
    uint32_t max_threads = 0, min_blocks = 0;
    uint32_t shared_mem_bytes = 0;
    std::vector<Scalar> target_dtypes;
    std::vector<SharedObj> shared_objs;
    const Function* find(const std::string& name) const {
        for (auto& f : funcs) if (f.name == name) return &f;
        return nullptr;
    }
};

struct ParseError {
    size_t line = 0;
    std::string msg;
    std::string text() const { return "line " + std::to_string(line) + ": " + msg; }
};

// Parses BIR text. Enforces the reference parser's numbering rule: a `%N =` prefix and a `bbN:`
// label must name the arena index about to be assigned (crates/basalt-bir/src/parse.rs:423-499).
bool parse_module(const char* src, size_t len, Module* out, ParseError* err);
// Prints a module; parse(print(m)) == m and print is deterministic.
std::string print_module(const Module& m);
// Structural checks the parser cannot make: operand ids in range, phi arity, branch targets.
bool verify_module(const Module& m, std::string* why);
// Rewrites each function's arena into print order (blocks in order, instructions in block order),
// dropping instructions no block lists, so that the module prints with valid numbering.
void canonicalize(Function& f);

}  // namespace basalt
