// extern "C" Backend entry points declared in include/basalt_b200.h.
#include <cstdlib>
#include <cstring>
#include <string>

#include "../../include/basalt_b200.h"
#include "emit.hpp"
#include "frontend_c.hpp"
#include "frontend_triton.hpp"

using namespace basalt;

static void fill_diag(basalt_diag* out, const std::string& code, const std::string& msg) {
    if (!out) return;
    memset(out, 0, sizeof *out);
    strncpy(out->code, code.c_str(), sizeof out->code - 1);
    strncpy(out->message, msg.c_str(), sizeof out->message - 1);
}

static char* dup_out(const std::string& s, size_t* len) {
    char* p = (char*)malloc(s.size() + 1);
    if (!p) return nullptr;
    memcpy(p, s.data(), s.size());
    p[s.size()] = 0;
    if (len) *len = s.size();
    return p;
}

static bool parse_or_diag(const char* bir, size_t len, Module* m, basalt_diag* d) {
    ParseError pe;
    if (!bir) { fill_diag(d, "E400", "null input"); return false; }
    if (!parse_module(bir, len, m, &pe)) { fill_diag(d, "E400", pe.text()); return false; }
    std::string why;
    if (!verify_module(*m, &why)) { fill_diag(d, "E400", why); return false; }
    return true;
}

static bool opts_ok(const basalt_emit_opts* o, EmitOptions* e, basalt_diag* d) {
    if (!o) return true;
    // "sm_100a", optionally followed by tuning keys: "sm_100a,max_unroll=2,regs=48"
    if (o->target_variant && *o->target_variant) {
        std::string v = o->target_variant;
        size_t comma = v.find(',');
        if (v.substr(0, comma) != "sm_100a") {
            fill_diag(d, "E093", std::string("unknown target variant: ") + o->target_variant);
            return false;
        }
        while (comma != std::string::npos) {
            size_t next = v.find(',', comma + 1);
            std::string kv = v.substr(comma + 1, next == std::string::npos ? std::string::npos : next - comma - 1);
            size_t eq = kv.find('=');
            int val = eq == std::string::npos ? 0 : atoi(kv.c_str() + eq + 1);
            std::string key = kv.substr(0, eq);
            if (key == "max_unroll" && val >= 1) e->max_unroll = val;
            else if (key == "regs" && val >= 16 && val <= 255) e->reg_budget = val;
            else {
                fill_diag(d, "E093", std::string("unknown target variant: ") + o->target_variant);
                return false;
            }
            comma = next;
        }
    }
    e->opt_level = o->opt_level < 0 ? 0 : o->opt_level;
    return true;
}

extern "C" {

const char* basalt_b200_name(void) { return "nvidia-ptx-sm100"; }

int basalt_b200_supports(const char* bir, size_t len, char ecode_out[8]) {
    Module m;
    basalt_diag d;
    if (ecode_out) memset(ecode_out, 0, 8);
    if (!parse_or_diag(bir, len, &m, &d)) {
        if (ecode_out) strncpy(ecode_out, "E400", 7);
        return -1;
    }
    Diag dg;
    if (!check_module(m, &dg)) {
        if (ecode_out) strncpy(ecode_out, dg.code.c_str(), 7);
        return 0;
    }
    return 1;
}

int basalt_b200_emit(const char* bir, size_t len, const basalt_emit_opts* opts, char** ptx_out, size_t* ptx_len, basalt_diag* diag_out) {
    if (ptx_out) *ptx_out = nullptr;
    Module m;
    EmitOptions eo;
    if (!parse_or_diag(bir, len, &m, diag_out) || !opts_ok(opts, &eo, diag_out)) return 1;
    EmitResult r;
    Diag d;
    if (!emit_ptx(m, eo, &r, &d)) { fill_diag(diag_out, d.code, d.arg); return 1; }
    if (ptx_out) *ptx_out = dup_out(r.ptx, ptx_len);
    return 0;
}

int basalt_b200_optimize(const char* bir, size_t len, const basalt_emit_opts* opts, char** bir_out, size_t* bir_len, basalt_diag* diag_out) {
    if (bir_out) *bir_out = nullptr;
    Module m;
    EmitOptions eo;
    if (!parse_or_diag(bir, len, &m, diag_out) || !opts_ok(opts, &eo, diag_out)) return 1;
    eo.want_bir = true;
    EmitResult r;
    Diag d;
    if (!emit_ptx(m, eo, &r, &d)) { fill_diag(diag_out, d.code, d.arg); return 1; }
    if (bir_out) *bir_out = dup_out(r.bir, bir_len);
    return 0;
}

int basalt_b200_roundtrip(const char* bir, size_t len, char** bir_out, size_t* bir_len, basalt_diag* diag_out) {
    if (bir_out) *bir_out = nullptr;
    Module m;
    if (!parse_or_diag(bir, len, &m, diag_out)) return 1;
    if (bir_out) *bir_out = dup_out(print_module(m), bir_len);
    return 0;
}

int basalt_b200_compile_cuda(const char* src, size_t len, char** bir_out, size_t* bir_len, basalt_diag* diag_out) {
    if (bir_out) *bir_out = nullptr;
    if (!src) { fill_diag(diag_out, "E500", "null input"); return 1; }
    Module m;
    Diag dg;
    if (!compile_cuda_c(src, len, &m, &dg)) { fill_diag(diag_out, dg.code, dg.arg); return 1; }
    if (bir_out) *bir_out = dup_out(print_module(m), bir_len);
    return 0;
}

int basalt_b200_compile_triton(const char* src, size_t len, const char* bindings, char** bir_out, size_t* bir_len, basalt_diag* diag_out) {
    if (bir_out) *bir_out = nullptr;
    if (!src) { fill_diag(diag_out, "E500", "null input"); return 1; }
    TritonOptions opts;
    std::string why;
    if (!parse_triton_bindings(bindings, &opts, &why)) { fill_diag(diag_out, "E102", "invalid bindings: " + why); return 1; }
    Module m;
    Diag dg;
    if (!compile_triton(src, len, opts, &m, &dg)) { fill_diag(diag_out, dg.code, dg.arg); return 1; }
    if (bir_out) *bir_out = dup_out(print_module(m), bir_len);
    return 0;
}

void basalt_b200_free(void* p) { free(p); }

}  // extern "C"
