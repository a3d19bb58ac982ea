// Triton source -> tile-level BIR.  The role of the reference's Triton lane
// (crates/basalt-frontend-triton/src/parse.rs, crates/basalt-sema/src/{triton_check,triton_lower}.rs),
// re-thought for a GPU: a program is a CTA, `tl.dot` is BIR's CTA-collective `mma`, elementwise
// tile code is a loop over lanes strided by the CTA's thread count.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <string>

#include "bir.hpp"
#include "passes.hpp"

namespace basalt {

struct TritonOptions {
    // Compile-time values for `tl.constexpr` parameters that have no literal default.  Such a
    // parameter stays in the kernel's signature as an i64 (the reference's ABI,
    // crates/basalt-sema/src/triton_lower.rs:517-551); its run-time value is not read.
    std::map<std::string, int64_t> constexprs;
    // Element type behind a pointer parameter; f32 when absent (Triton signatures carry no dtype,
    // and the reference assumes 4-byte elements, triton_lower.rs:72-84).
    std::map<std::string, Scalar> pointee;
};

// Parses "K=5 BLOCK=1024 a_ptr=*f16 b_ptr=*f16" into options; returns false on a malformed item.
bool parse_triton_bindings(const char* text, TritonOptions* out, std::string* why);

// Compiles every `@triton.jit` function of the source.  Refusals carry the reference's codes
// (crates/basalt-diag/src/ecode.rs:148-181): E200/E201/E202 lexical and syntax, E300 type, E301
// undefined name, E304 construct outside the subset, E305 tile shapes that do not broadcast,
// E306 a tile extent that is not a compile-time constant where one is needed, E307 a tile
// construct this lowering does not model.
bool compile_triton(const char* src, size_t len, const TritonOptions& opts, Module* out, Diag* d);

}  // namespace basalt
