// BIR -> sm_100a PTX text. The role of `impl Backend for Ptx` in the reference
// (crates/basalt-ptx/src/emit.rs:1973-1994): check, (here: optimise,) lower, return text.
#pragma once
#include <string>
#include <vector>

#include "bir.hpp"
#include "passes.hpp"

namespace basalt {

struct EmitOptions {
    int opt_level = 2;      // 0 = the reference's one-to-one lowering, >0 = run the BIR passes
    int reg_budget = 0;     // 32-bit registers per thread the vectorisers may plan for; 0 = from the module's launch bounds (register_budget)
    int max_unroll = 4;     // cap on the vectorisers' unroll factor
    bool want_bir = false;  // also return the optimised BIR text
};

struct EmitResult {
    std::string ptx;
    std::string bir;   // optimised module, when requested
    std::vector<OptReport> reports;
};

// Registers per thread that keep `ctas_per_sm` CTAs of `threads_per_cta` threads resident on an SM of 65 536
// registers (0 = the defaults: 256 threads, the reference's launch geometry; as many CTAs as give 1024 resident
// threads, which is what a streaming kernel needs to saturate HBM), rounded down to the allocation unit of eight.
int register_budget(unsigned threads_per_cta, unsigned ctas_per_sm);
// Maximum number of 32-bit registers live at one point of an emitted function body: live intervals over the
// linearised PTX (`decls`: its .reg declarations, `body`: its statements and labels), extended across loop back
// edges -- steps 1-3 of the reference's linear-scan allocator (crates/basalt-passes/src/regalloc.rs:5-33) applied
// to virtual PTX registers.  ptxas lands between this figure and two thirds of it on the benchmark kernels.
int ptx_register_pressure(const std::vector<std::string>& decls, const std::vector<std::string>& body);

// Deterministic: the same (module, options) always yields the same bytes.
bool emit_ptx(const Module& m, const EmitOptions& opts, EmitResult* out, Diag* d);

// Lowerings of `mma` that use the whole CTA; defined in emit_mma.cpp. `lines` receives PTX
// statements, `decls` register/shared declarations. Returns false when the op's shape is not one
// the fast paths cover (the caller then emits the generic loop nest).
struct MmaSite {
    const Inst* inst;
    std::string a, b, c, d;       // 64-bit registers holding the four operand addresses
    Space sa, sb, sc, sd;         // their address spaces
    bool c_is_null;               // operand c is the literal null pointer: D = A*B
    int uid;                      // unique per function, for labels and symbols
    std::string kernel;           // entry name
    unsigned nparams;             // number of BIR parameters of the entry
    unsigned max_threads;         // the module's launch_bounds max_threads, 0 when absent
    bool sole_mma;                // the function's only mma
    int a_param, b_param;         // parameter each operand pointer is derived from by pointer adds, or -1
    std::string a_base, b_base;   // registers holding those parameters
    // Operand pointers as affine functions of the block index: pointer = parameter + c0 + cx*bid.x + cy*bid.y.
    // Valid when `affine` is set; then a/b/d derive from parameters a_param/b_param/d_param.
    bool affine;
    long long a_c0, a_cx, a_cy, b_c0, b_cx, b_cy, d_c0, d_cx, d_cy;
    int d_param;
    std::string d_base;
    bool pure_kernel;             // one block, nothing but index arithmetic, this mma and `ret`
    unsigned* maxntid;            // the entry's .maxntid, which a lowering may raise
    std::vector<std::string>* extra_params;   // receives .param declarations appended to the entry
    std::vector<std::string>* module_decls;   // receives module-scope declarations
    bool pair_twin = false;       // this is the `<name>__pair` twin of an entry: take the two-SM (cta_group::2) lowering or fail
    unsigned* cluster = nullptr;  // the entry's .reqnctapercluster x extent, which a lowering may set
    unsigned* tmem_cols = nullptr;   // tensor-memory columns the lowering allocates per CTA (an SM has 512)
};
bool emit_mma_fast(const MmaSite& site, std::vector<std::string>* decls, std::vector<std::string>* lines,
                   std::vector<std::string>* plan);

}  // namespace basalt
