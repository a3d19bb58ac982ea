// Module checks and BIR-to-BIR passes of the sm_100a backend.
//
// The reference PTX backend does no optimisation at all: one virtual register per SSA value,
// scalar accesses, one element per thread (crates/basalt-ptx/src/emit.rs:10-18, 1400-1474).  The
// passes here are where the Blackwell lowering differs: helper calls are inlined (the reference
// refuses `call`, emit.rs:503-509), one-element-per-thread kernels are rewritten to 128-bit
// accesses, strided reduction loops likewise, and shuffle butterflies become warp reductions.
// Every pass is BIR in, BIR out, so its result can be printed and run through the CPU oracle
// interpreter in the tests.
#pragma once
#include <functional>
#include <string>

#include "bir.hpp"

namespace basalt {

// A refusal: one of the reference's stable E-codes (crates/basalt-diag/src/ecode.rs:148-181) plus
// a human-readable argument.
struct Diag {
    std::string code;
    std::string arg;
};

// The refusal surface shared by `supports` and `emit`, mirroring check_module of the reference
// (crates/basalt-ptx/src/emit.rs:520-546) with these deliberate differences: f16, `mma` and `call`
// are accepted (they have real lowerings here), so a non-kernel function is accepted when a kernel
// reaches it through calls; the call-graph rules are the reference oracle's
// (crates/basalt-x86/src/oracle.rs:172-176): a cycle is E094, an unreachable helper E095, calling a
// kernel E093.  Host ops stay E090.
bool check_module(const Module& m, Diag* d);

// Promotes promotable local/param slots to SSA values and phis (the reference's construct_ssa,
// crates/basalt-passes/src/ssa.rs), so that slot-form BIR straight from the front end is accepted.
void construct_ssa(Function& f);
// Inlines every call (the graph is acyclic after check_module) and drops the helper functions.
void inline_calls(Module& m);
// Merges straight-line block chains, removes unreachable blocks.
void simplify_cfg(Function& f);
// Removes instructions without side effects whose results are unused.
void dce(Function& f);
// Evaluates instructions whose operands are constants, with the CPU oracle's arithmetic, applies
// integer identities, and turns a conditional branch on a constant into a branch (the reference's
// constant_fold, crates/basalt-passes/src/constfold.rs).  Returns the number of rewrites.
int fold_constants(Function& f);
// Replaces a pure instruction by an identical one that dominates it.  Returns the number removed.
int eliminate_common_subexpressions(Function& f);
// Moves pure instructions whose operands do not change inside a natural loop to the loop's preheader
// (the reference's licm, crates/basalt-passes/src/licm.rs); never a division, never a load.  Returns
// the number moved.
int hoist_loop_invariants(Function& f);

struct OptReport {
    bool elementwise = false;   // one-element-per-thread kernel rewritten to vector accesses
    bool reduction = false;     // strided reduction loop rewritten to vector accesses
    int warp_reduces = 0;       // shuffle butterflies replaced by warp.reduce
    int vec_lanes = 0;
    int unroll = 0;
    int est_regs = 0;           // liveness-based estimate of 32-bit registers per thread
    std::string coarse_of;      // set on a `<name>__coarse` variant: the kernel it stands in for
};

// Rewrites a kernel of the shape `i = bid.x*bdim.x + tid.x; if (i < n) { body(i) }`, whose body
// touches global memory only at `param + i*esz`, into a grid-stride loop over 16-byte vectors with
// a scalar tail and an unaligned fallback.  The set of elements processed is exactly the set the
// original processes under the same launch: [0, min(n, gdim.x*bdim.x)).  `coarse_out` receives a
// second entry, `<name>__coarse`, with one more i64 parameter: the thread count of the launch the
// caller asked for.  The runtime launches it with one wave of resident CTAs instead, so each thread
// loops over many vectors with several loads in flight; the elements processed are the same.
bool vectorize_elementwise(Function& f, int unroll, OptReport* rep, Function* coarse_out = nullptr);
// Rewrites `for (i = g; i < n; i += gdim.x*bdim.x) acc = op(acc, x[i])` (op = signed max/min, add,
// and, or, xor on i32) into the same loop over 16-byte vectors plus a scalar tail loop.
bool vectorize_reduction_loop(Function& f, int unroll, OptReport* rep);
// Replaces a five-step shuffle.xor butterfly (masks 16,8,4,2,1 in any order) combining with an
// i32 max/min/add/and/or/xor by one warp.reduce; every lane receives the same value either way.
int fuse_warp_reductions(Function& f);

// Backward liveness over the CFG; returns the peak number of simultaneously live 32-bit register
// units (64-bit values count 2, predicates 0), the quantity the register-budget pass bounds.
int estimate_registers(const Function& f);

// Runs the whole pipeline on a checked module: inline, simplify, fuse warp reductions, then the
// vectorisers with the largest unroll whose register estimate stays inside `reg_budget`.
// `measure(module, function)` returns the register pressure of the function as it would be emitted (the emitter
// passes ptx_register_pressure of its own lowering); when empty, the BIR-level estimate_registers is used.
using PressureFn = std::function<int(const Module&, const Function&)>;
void optimize_module(Module& m, int opt_level, int reg_budget, int max_unroll, const PressureFn& measure, std::vector<OptReport>* reports);

}  // namespace basalt
