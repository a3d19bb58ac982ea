// basalt-b200: the `basalt --nvidia-ptx <file> [-o out.ptx]` arm of the reference CLI
// (crates/basalt-cli/src/main.rs:511-559) for the sm_100a backend.  Reads BIR text (.bir) or a
// CUDA-C source in the supported subset (.cu), writes PTX to stdout or to the -o path
// (main.rs:553-558); a refusal prints "<E-code>: <message>" on stderr and exits 1, as the reference
// renders a Diag (main.rs:894-900).  `--emit-bir file.cu` stops after the front end, like the
// reference's flag of that name (main.rs:286-327).  A `.py` input is a Triton source (the reference's
// `--triton` lane, main.rs:329-372); `--bind "K=5 a_ptr=*f16 num_warps=4"` gives it constexpr values,
// pointee types and the CTA size.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>

#include "../../include/basalt_b200.h"

static int usage() {
    std::cerr << "usage: basalt-b200 --nvidia-ptx <file.bir> [-o <out.ptx>] [-O0|-O2]\n"
                 "       basalt-b200 --nvidia-ptx <file.cu>  [-o <out.ptx>] [-O0|-O2]\n"
                 "       basalt-b200 --nvidia-ptx <file.py>  [--bind \"K=5 a_ptr=*f16 num_warps=4\"] [-o <out.ptx>]\n"
                 "       basalt-b200 --emit-bir <file.cu|file.py> (front end only)\n"
                 "       basalt-b200 --ir <file.bir|file.cu> (print the module as the backend lowers it)\n";
    return 2;
}

int main(int argc, char** argv) {
    std::string mode, in, out, bind;
    basalt_emit_opts opts{nullptr, 2, nullptr, 0};
    for (int i = 1; i < argc; i++) {
        std::string a = argv[i];
        if (a == "--nvidia-ptx" || a == "--ir" || a == "--emit-bir") {
            if (!mode.empty()) { std::cerr << "E103: conflicting flags: " << mode << " and " << a << "\n"; return 1; }
            mode = a;
        } else if (a == "-o") {
            if (i + 1 >= argc) { std::cerr << "E101: missing argument for flag: -o\n"; return 1; }
            out = argv[++i];
        } else if (a == "--bind") {
            if (i + 1 >= argc) { std::cerr << "E101: missing argument for flag: --bind\n"; return 1; }
            bind = argv[++i];
        } else if (a == "-O0") opts.opt_level = 0;
        else if (a == "-O2") opts.opt_level = 2;
        else if (!a.empty() && a[0] == '-') { std::cerr << "E100: unknown flag: " << a << "\n"; return 1; }
        else in = a;
    }
    if (mode.empty() || in.empty()) return usage();
    const bool is_bir = in.size() >= 4 && in.substr(in.size() - 4) == ".bir";
    const bool is_py = in.size() >= 3 && in.substr(in.size() - 3) == ".py";
    const bool is_cu = (in.size() >= 3 && in.substr(in.size() - 3) == ".cu") || is_py;
    if (!is_bir && !is_cu) { std::cerr << "E102: invalid argument for flag " << mode << ": input must be .bir, .cu or .py\n"; return 1; }
    if (mode == "--emit-bir" && !is_cu) { std::cerr << "E102: invalid argument for flag --emit-bir: input must be .cu or .py\n"; return 1; }
    std::ifstream f(in, std::ios::binary);
    if (!f) { std::cerr << "E500: I/O error reading " << in << ": cannot open\n"; return 1; }
    std::stringstream ss;
    ss << f.rdbuf();
    std::string text = ss.str();
    char* result = nullptr;
    size_t len = 0;
    basalt_diag d;
    if (is_cu) {
        char* bir = nullptr;
        size_t blen = 0;
        int frc = is_py ? basalt_b200_compile_triton(text.data(), text.size(), bind.empty() ? nullptr : bind.c_str(), &bir, &blen, &d)
                        : basalt_b200_compile_cuda(text.data(), text.size(), &bir, &blen, &d);
        if (frc != 0) { std::cerr << d.code << ": " << d.message << "\n"; return 1; }
        text.assign(bir, blen);
        basalt_b200_free(bir);
        if (mode == "--emit-bir") {
            if (out.empty()) std::cout << text;
            else {
                std::ofstream o(out, std::ios::binary);
                if (!o) { std::cerr << "E500: I/O error reading " << out << ": cannot open for writing\n"; return 1; }
                o << text;
            }
            return 0;
        }
    }
    int rc = mode == "--ir" ? basalt_b200_optimize(text.data(), text.size(), &opts, &result, &len, &d)
                            : basalt_b200_emit(text.data(), text.size(), &opts, &result, &len, &d);
    if (rc != 0) { std::cerr << d.code << ": " << d.message << "\n"; return 1; }
    if (out.empty()) std::cout.write(result, (std::streamsize)len);
    else {
        std::ofstream o(out, std::ios::binary);
        if (!o) { std::cerr << "E500: I/O error reading " << out << ": cannot open for writing\n"; basalt_b200_free(result); return 1; }
        o.write(result, (std::streamsize)len);
    }
    basalt_b200_free(result);
    return 0;
}
