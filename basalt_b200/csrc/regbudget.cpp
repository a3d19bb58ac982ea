// The register-budget pass of the sm_100a backend, on PTX text.
//
// The reference leaves registers to ptxas entirely: its emitter declares one virtual register per
// SSA value and a linear-scan allocator exists only for its CPU back ends
// (crates/basalt-passes/src/regalloc.rs:5-33: liveness, intervals, linear scan over a fixed pool).
// On a GPU the pool is not fixed: the registers a thread uses decide how many CTAs an SM can hold
// (65 536 registers per SM), so the backend plans against a budget
//
//     budget = 65 536 / (threads per CTA x CTAs per SM it wants resident)
//
// and needs to know, before the driver's JIT has run, roughly how many registers a body will take.
// `ptx_register_pressure` answers that for one emitted function: the same steps 1-3 of the
// reference's allocator (live intervals over a linearised body, extended across loop back edges),
// then, instead of assigning a pool, the maximum number of 32-bit registers live at one point.
// The vectorisers choose the largest unroll whose body stays inside the budget, the emitter prints
// the figure in the kernel's header comment, and asks for `.maxnreg` when a small overshoot would
// otherwise cost the occupancy the launch bounds ask for.
#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <functional>
#include <map>
#include <string>
#include <vector>

#include "emit.hpp"

namespace basalt {

namespace {

struct Interval {
    int first = -1, last = -1, width = 0;
};

// `.reg .b32 %r<12>;` / `.reg .b64 %a, %b, %c<4>;` -> name -> width in 32-bit registers
void parse_reg_decl(const std::string& line, std::map<std::string, int>* width, std::map<std::string, std::pair<int, int>>* families) {
    size_t at = line.find(".reg");
    if (at == std::string::npos) return;
    size_t ty = line.find('.', at + 4);
    if (ty == std::string::npos) return;
    size_t ty_end = ty + 1;
    while (ty_end < line.size() && (isalnum((unsigned char)line[ty_end]) || line[ty_end] == '_')) ty_end++;
    const std::string t = line.substr(ty + 1, ty_end - ty - 1);
    int w = 1;
    if (t == "pred") w = 0;
    else if (t == "b64" || t == "u64" || t == "s64" || t == "f64") w = 2;
    else if (t == "b128") w = 4;
    size_t i = ty_end;
    while (i < line.size()) {
        while (i < line.size() && line[i] != '%') i++;
        if (i >= line.size()) break;
        size_t j = i + 1;
        while (j < line.size() && (isalnum((unsigned char)line[j]) || line[j] == '_')) j++;
        std::string name = line.substr(i, j - i);
        if (j < line.size() && line[j] == '<') {
            int n = atoi(line.c_str() + j + 1);
            (*families)[name] = {n, w};
        } else (*width)[name] = w;
        i = j;
    }
}

}  // namespace

int ptx_register_pressure(const std::vector<std::string>& decls, const std::vector<std::string>& body) {
    std::map<std::string, int> width;                        // singly declared names
    std::map<std::string, std::pair<int, int>> families;     // %r<N>: prefix -> (count, width)
    for (auto& d : decls) parse_reg_decl(d, &width, &families);
    std::map<std::string, Interval> iv;
    std::map<std::string, int> label_at;
    std::vector<std::pair<int, std::string>> branches;       // (line, target label)
    auto width_of = [&](const std::string& name) -> int {
        auto it = width.find(name);
        if (it != width.end()) return it->second;
        // %r17 -> family %r
        size_t e = name.size();
        while (e > 1 && isdigit((unsigned char)name[e - 1])) e--;
        if (e == name.size()) return -1;
        auto f = families.find(name.substr(0, e));
        if (f == families.end()) return -1;
        return atoi(name.c_str() + e) < f->second.first ? f->second.second : -1;
    };
    // A register whose one definition is `mov <reg>, <numeric immediate>` costs nothing: ptxas folds the
    // immediate into the instructions that use it.
    std::map<std::string, int> imm_defs, other_mentions;
    std::vector<std::pair<std::string, std::string>> copies;
    for (auto& s : body) {
        size_t b = s.find_first_not_of(" \t");
        if (b == std::string::npos) continue;
        bool imm_mov = false;
        std::string dst;
        if (s.compare(b, 4, "mov.") == 0) {
            size_t r = s.find('%', b), comma = s.find(',', b), semi = s.find(';', b);
            if (r != std::string::npos && comma != std::string::npos && semi != std::string::npos && r < comma) {
                size_t v = s.find_first_not_of(" \t", comma + 1);
                if (v != std::string::npos && (isdigit((unsigned char)s[v]) || s[v] == '-')) {
                    imm_mov = true;
                    size_t j = r + 1;
                    while (j < s.size() && (isalnum((unsigned char)s[j]) || s[j] == '_')) j++;
                    dst = s.substr(r, j - r);
                }
            }
        }
        if (imm_mov) imm_defs[dst]++;
        else if (s.compare(b, 5, "mov.b") == 0) {   // mov.b32 %a, %b;
            size_t r = s.find('%', b), comma = s.find(',', b);
            if (r != std::string::npos && comma != std::string::npos && r < comma) {
                size_t v = s.find_first_not_of(" \t", comma + 1);
                if (v != std::string::npos && s[v] == '%') {
                    size_t j = r + 1, k = v + 1;
                    while (j < s.size() && (isalnum((unsigned char)s[j]) || s[j] == '_')) j++;
                    while (k < s.size() && (isalnum((unsigned char)s[k]) || s[k] == '_')) k++;
                    if (k < s.size() && s[k] == ';') copies.push_back({s.substr(r, j - r), s.substr(v, k - v)});
                }
            }
        }
    }
    for (int ln = 0; ln < (int)body.size(); ln++) {
        const std::string& s = body[ln];
        size_t b = s.find_first_not_of(" \t");
        if (b == std::string::npos || s.compare(b, 2, "//") == 0) continue;
        size_t colon = s.find(':');
        if (colon != std::string::npos && s.find(';') == std::string::npos && s.find(' ', b) == std::string::npos) {   // `$label:`
            label_at[s.substr(b, colon - b)] = ln;
            continue;
        }
        size_t br = s.find("bra");
        if (br != std::string::npos && (br == b || s[br - 1] == ' ' || s[br - 1] == '\t')) {
            size_t t = s.find_first_not_of(" \t", br + 3 + (s.compare(br, 7, "bra.uni") == 0 ? 4 : 0));
            size_t e = s.find(';', t);
            if (t != std::string::npos && e != std::string::npos) branches.push_back({ln, s.substr(t, e - t)});
        }
        for (size_t i = b; i < s.size(); i++) {
            if (s[i] != '%') continue;
            size_t j = i + 1;
            while (j < s.size() && (isalnum((unsigned char)s[j]) || s[j] == '_')) j++;
            std::string name = s.substr(i, j - i);
            i = j - 1;
            int w = width_of(name);
            if (w <= 0) continue;                            // special registers, predicates
            if (j < s.size() && s[j] == ',' && s.compare(b, 4, "mov.") != 0 && i == s.find('%', b)) other_mentions[name]++;   // defined by another instruction too
            Interval& x = iv[name];
            if (x.first < 0) { x.first = ln; x.width = w; }
            x.last = ln;
        }
    }
    // A value that enters a loop from before it and is named inside it lives until the back edge.
    std::vector<std::pair<int, int>> loops;
    for (auto& bz : branches) {
        auto it = label_at.find(bz.second);
        if (it != label_at.end() && it->second < bz.first) loops.push_back({it->second, bz.first});
    }
    for (bool changed = true; changed;) {
        changed = false;
        for (auto& kv : iv) {
            Interval& x = kv.second;
            for (auto& lp : loops)
                if (x.first < lp.first && x.last >= lp.first && x.last < lp.second) { x.last = lp.second; changed = true; }
        }
    }
    // Registers joined by register-to-register moves (the copies that implement phis) are counted once where
    // their intervals overlap: ptxas coalesces such copies.
    std::map<std::string, std::string> parent;
    std::function<std::string(const std::string&)> find = [&](const std::string& n) -> std::string {
        auto it = parent.find(n);
        if (it == parent.end() || it->second == n) return n;
        std::string r = find(it->second);
        parent[n] = r;
        return r;
    };
    for (auto& c : copies) {
        std::string a = find(c.first), b2 = find(c.second);
        if (a != b2) parent[a] = b2;
    }
    std::map<std::string, std::vector<const Interval*>> groups;
    for (auto& kv : iv) {
        auto im = imm_defs.find(kv.first);
        if (im != imm_defs.end() && im->second == 1 && !other_mentions.count(kv.first)) continue;
        groups[find(kv.first)].push_back(&kv.second);
    }
    std::vector<int> delta(body.size() + 2, 0);
    for (auto& g : groups) {
        std::vector<const Interval*>& m = g.second;
        std::sort(m.begin(), m.end(), [](const Interval* a, const Interval* b2) { return a->first < b2->first; });
        int lo = m[0]->first, hi = m[0]->last, w = m[0]->width;
        for (size_t i = 1; i < m.size(); i++) {
            if (m[i]->first <= hi + 1) hi = std::max(hi, m[i]->last);
            else { delta[lo] += w; delta[hi + 1] -= w; lo = m[i]->first; hi = m[i]->last; }
            w = std::max(w, m[i]->width);
        }
        delta[lo] += w;
        delta[hi + 1] -= w;
    }
    int cur = 0, peak = 0;
    for (size_t i = 0; i < delta.size(); i++) { cur += delta[i]; peak = std::max(peak, cur); }
    return peak + 4;   // what ptxas keeps for itself (stack pointer, scratch for address arithmetic and predicates)
}

int register_budget(unsigned threads_per_cta, unsigned ctas_per_sm) {
    if (threads_per_cta == 0) threads_per_cta = 256;          // the reference's launch geometry (ptx_gpu_proof.rs:138)
    if (ctas_per_sm == 0) ctas_per_sm = std::max(1u, 1024u / threads_per_cta);   // half of the SM's 2048 thread slots: what a streaming kernel needs to saturate HBM
    unsigned per_thread = 65536u / (threads_per_cta * ctas_per_sm);
    per_thread &= ~7u;                                        // registers are allocated in units of eight
    return (int)std::min(255u, std::max(16u, per_thread));
}

}  // namespace basalt
