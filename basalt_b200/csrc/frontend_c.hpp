// CUDA-C subset -> BIR.  The role of the reference's C front end plus sema lowering
// (crates/basalt-frontend-c/src/{lex,parse}.rs, crates/basalt-sema/src/{checker,lower}.rs) for the
// part of the language device kernels are written in.
//
// The BIR produced is the slot form the reference's sema layer produces
// (crates/basalt-sema/src/lower.rs:882-898, 992-1063): every parameter and local lives in a
// synthetic storage cell `const.i ptr.<space> slot*65536` read and written with load/store, so
// that construct_ssa promotes it afterwards exactly as it does for reference-produced modules.
#pragma once
#include <cstddef>

#include "bir.hpp"
#include "passes.hpp"

namespace basalt {

// Compiles one translation unit.  On failure returns false and sets `d` to one of the reference's
// front-end codes (crates/basalt-diag/src/ecode.rs:148-181): E200 lexical, E201 syntax, E202
// unterminated comment, E300 type error, E301 undefined name, E302 redefinition, E303 qualifier
// misuse, E304 a construct outside the subset, E308 write through const.
bool compile_cuda_c(const char* src, size_t len, Module* out, Diag* d);

}  // namespace basalt
