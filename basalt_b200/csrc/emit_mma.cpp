// CTA-wide lowerings of `mma` for sm_100a.
//
// In this backend `mma` is a CTA-collective tile operation (every thread of the CTA reaches it,
// the product is computed once), so a kernel whose CTA computes one output tile is a few address
// computations and one `mma` over strided tiles of the full matrices.  Two shapes get a dedicated
// lowering; everything else takes the generic loop nest in emit.cpp.
//
//  * f32 x f32 -> f32, 128x128 tile, 256 threads: register-tiled FFMA.  K slabs of 16 are staged
//    through a double-buffered shared-memory tile pair (A transposed so that a thread's four rows
//    are one 16-byte read); each thread owns 8x8 outputs as four 4x4 quadrants; per K step it
//    issues 4 ld.shared.v4 for 64 fma.rn.f32; the next slab's global loads are in flight while the
//    current one is multiplied.  The same design as the hand-written comparator kernel
//    (kernels/sgemm.cu).
//  * f16 x f16 -> f32 accumulate -> f16, 128x128 tile, 128 threads: TMA + tcgen05.  One thread
//    issues cp.async.bulk.tensor loads of 64-deep K slabs into a ring of 128-byte-swizzled shared
//    stages, one thread issues tcgen05.mma (M128 N128 K16) from shared-memory matrix descriptors
//    into a TMEM accumulator, mbarriers (tcgen05.commit) hand stages back; all four warps drain the
//    accumulator with tcgen05.ld, convert and store.  The tensor maps are kernel parameters the
//    launch runtime appends (the `//!basalt.plan` line says how to build them).  Every mbarrier
//    wait is bounded by %globaltimer; a wait that gives up sets the kernel's status word, the
//    kernel stops issuing copies, still frees its TMEM and returns.
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include "emit.hpp"

namespace basalt {
namespace {

struct Out {
    std::vector<std::string>* lines;
    void operator()(const char* fmt, ...) {
        char buf[1024];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        lines->push_back(std::string("\t") + buf);
    }
    void label(const std::string& l) { lines->push_back(l + ":"); }
};

bool sgemm_ffma(const MmaSite& s, std::vector<std::string>* decls, std::vector<std::string>* lines, std::vector<std::string>* plan) {
    const Inst& in = *s.inst;
    if (in.in_dt != Scalar::F32 || in.acc_dt != Scalar::F32 || in.out_dt != Scalar::F32 || in.a_col || in.b_col) return false;
    if (in.m != 128 || in.n != 128 || in.k % 16 != 0 || !s.c_is_null || !in.has_ld) return false;
    if (s.sa != Space::Global || s.sb != Space::Global || s.sd != Space::Global || s.max_threads != 256) return false;
    const long long lda = in.ld[0] ? in.ld[0] : in.k, ldb = in.ld[1] ? in.ld[1] : in.n, ldd = in.ld[3] ? in.ld[3] : in.n;
    if (lda % 4 || ldb % 4 || ldd % 4 || lda * 4 >= (1ll << 31) || ldb * 4 >= (1ll << 31) || ldd * 4 >= (1ll << 31)) return false;
    const int u = s.uid, nk = (int)(in.k / 16);
    // Tail-wave form: when the kernel is nothing but this op on a tiled grid (operand pointers are the
    // parameters plus constant multiples of the block indices), the CTA decodes its tile from a linear
    // index instead, so that the launch runtime can issue whole tiles first and have the tiles of a sparse
    // last wave worked off by stream units: CTA full + u takes K slabs [u * per, (u + 1) * per) of the tail
    // tiles' slabs laid end to end, segment by segment (a segment ends with its tile); the segments of a tile
    // are summed in unit order by the one that finishes last (see kernels/sgemm.cu for the same scheme in CUDA).
    const bool tail = s.affine && s.pure_kernel && s.sole_mma && s.extra_params && s.a_c0 == 0 && s.a_cx == 0 && s.a_cy == 128 * lda * 4 && s.b_c0 == 0 &&
                      s.b_cy == 0 && s.b_cx == 512 && s.d_c0 == 0 && s.d_cx == 512 && s.d_cy == 128 * ldd * 4 && in.k < (1u << 30);
    // The generator also has a 128-thread form in which a thread owns 16 x 8 outputs (four groups of four rows, 32
    // apart): six 16-byte fragment loads per 64 packed FMAs instead of eight.  It needs 254 registers, so only eight
    // warps are resident per SM, and measures 58.1 TFLOP/s at 4096^3 against 59.3 for the 256-thread form: kept off.
    const bool wide = false;
    const int NT = wide ? 128 : 256, RG = wide ? 4 : 2, SP = 128 / RG;   // threads, row groups per thread, rows between groups
    char nm[64];
    auto R = [&](const char* stem, int i = -1) {
        if (i < 0) snprintf(nm, sizeof nm, "%%mm%d_%s", u, stem);
        else snprintf(nm, sizeof nm, "%%mm%d_%s%d", u, stem, i);
        return std::string(nm);
    };
    char d[256];
    snprintf(d, sizeof d, "\t.reg .f32 %%mm%d_fa<%d>, %%mm%d_st<%d>;", u, 4 * RG, u, 8 * RG);
    decls->push_back(d);
    // accumulators as packed pairs (columns 2p, 2p+1 of the thread's row i in acc2[4i+p]), the eight A values of a
    // K step duplicated into both halves of a 64-bit register, the eight B values as four pairs
    snprintf(d, sizeof d, "\t.reg .b64 %%mm%d_acc2_<%d>, %%mm%d_ad<%d>, %%mm%d_bp<4>;", u, 16 * RG, u, 4 * RG, u);
    decls->push_back(d);
    snprintf(d, sizeof d, "\t.reg .b32 %%mm%d_asq<4>, %%mm%d_xq<4>;", u, u);
    decls->push_back(d);
    snprintf(d, sizeof d, "\t.reg .b32 %%mm%d_tid, %%mm%d_tx, %%mm%d_ty, %%mm%d_t, %%mm%d_arow, %%mm%d_acol, %%mm%d_brow, %%mm%d_bcol, %%mm%d_asst, %%mm%d_bsst, %%mm%d_asrd, %%mm%d_bsrd, %%mm%d_as, %%mm%d_bs, %%mm%d_kb, %%mm%d_kb1, %%mm%d_off, %%mm%d_x, %%mm%d_y;",
             u, u, u, u, u, u, u, u, u, u, u, u, u, u, u, u, u, u, u);
    decls->push_back(d);
    snprintf(d, sizeof d, "\t.reg .b64 %%mm%d_ag, %%mm%d_ag2, %%mm%d_bg, %%mm%d_bg2, %%mm%d_w, %%mm%d_c;", u, u, u, u, u, u);
    decls->push_back(d);
    snprintf(d, sizeof d, "\t.reg .pred %%mm%d_more, %%mm%d_bad;", u, u);
    decls->push_back(d);
    if (tail) {
        snprintf(d, sizeof d, "\t.reg .b32 %%mm%d_cid, %%mm%d_full, %%mm%d_per, %%mm%d_tile, %%mm%d_k0, %%mm%d_it0, %%mm%d_it1, %%mm%d_lgx, %%mm%d_bx, %%mm%d_by, %%mm%d_uf, %%mm%d_kbeg, %%mm%d_nk, %%mm%d_tt, %%mm%d_tk, %%mm%d_p;",
                 u, u, u, u, u, u, u, u, u, u, u, u, u, u, u, u);
        decls->push_back(d);
        snprintf(d, sizeof d, "\t.reg .b64 %%mm%d_ta, %%mm%d_tb, %%mm%d_td, %%mm%d_ws, %%mm%d_tkp, %%mm%d_pp;", u, u, u, u, u, u);
        decls->push_back(d);
        snprintf(d, sizeof d, "\t.reg .pred %%mm%d_whole, %%mm%d_one, %%mm%d_t0, %%mm%d_notlast, %%mm%d_pl;", u, u, u, u, u);
        decls->push_back(d);
        snprintf(d, sizeof d, "\t.shared .align 4 .b8 __mm%d_tks[4];", u);
        decls->push_back(d);
        s.extra_params->push_back(".param .u32 " + s.kernel + "_lgrid_x");
        s.extra_params->push_back(".param .u32 " + s.kernel + "_lgrid_y");
        s.extra_params->push_back(".param .u32 " + s.kernel + "_full_tiles");
        s.extra_params->push_back(".param .u32 " + s.kernel + "_per");
        s.extra_params->push_back(".param .u64 " + s.kernel + "_workspace");
        s.extra_params->push_back(".param .u64 " + s.kernel + "_tickets");
        // the fused gather: the result matrix's base address on up to seven peers, and how many are set
        s.extra_params->push_back(".param .align 8 .b8 " + s.kernel + "_peers[56]");
        s.extra_params->push_back(".param .u32 " + s.kernel + "_npeers");
        snprintf(d, sizeof d, "\t.reg .b32 %%mm%d_np, %%mm%d_pi;", u, u);
        decls->push_back(d);
        snprintf(d, sizeof d, "\t.reg .b64 %%mm%d_pb, %%mm%d_pz, %%mm%d_pq;", u, u, u);
        decls->push_back(d);
        snprintf(d, sizeof d, "\t.reg .pred %%mm%d_pk, %%mm%d_mc;", u, u);
        decls->push_back(d);
    }
    snprintf(d, sizeof d, "\t.shared .align 16 .b8 __mm%d_as[16384];", u);
    decls->push_back(d);
    snprintf(d, sizeof d, "\t.shared .align 16 .b8 __mm%d_bs[16384];", u);
    decls->push_back(d);
    std::string l_loop = "$mm" + std::to_string(u) + "_loop", l_done = "$mm" + std::to_string(u) + "_done", l_skip = "$mm" + std::to_string(u) + "_skip";
    std::string l_next = "$mm" + std::to_string(u) + "_next";
    Out o{lines};
    const std::string tid = R("tid"), tx = R("tx"), ty = R("ty"), t = R("t"), arow = R("arow"), acol = R("acol"), brow = R("brow"), bcol = R("bcol");
    const std::string asst = R("asst"), bsst = R("bsst"), asrd = R("asrd"), bsrd = R("bsrd"), as = R("as"), bs = R("bs"), kb = R("kb"), kb1 = R("kb1"), off = R("off");
    const std::string x = R("x"), y = R("y"), ag = R("ag"), ag2 = R("ag2"), bg = R("bg"), bg2 = R("bg2"), w = R("w"), cp = R("c"), more = R("more"), bad = R("bad");
    auto acc2 = [&](int i) { return R("acc2_", i); };
    auto st = [&](int i) { return R("st", i); };
    auto fa = [&](int i) { return R("fa", i); };
    auto ad = [&](int i) { return R("ad", i); };
    auto bp = [&](int i) { return R("bp", i); };

    o("// mma f32 128x128x%u: register-tiled FFMA, lda=%lld ldb=%lld ldd=%lld", in.k, lda, ldb, ldd);
    o("mov.u32 %s, %%ntid.x;", t.c_str());
    o("setp.ne.u32 %s, %s, %d;", bad.c_str(), t.c_str(), NT);
    o("@%s bra %s;", bad.c_str(), l_skip.c_str());   // wrong block size: leave the output untouched rather than misbehave
    o("mov.u32 %s, %%tid.x;", tid.c_str());
    o("and.b32 %s, %s, 15;", tx.c_str(), tid.c_str());
    o("shr.u32 %s, %s, 4;", ty.c_str(), tid.c_str());
    o("shr.u32 %s, %s, 2;", arow.c_str(), tid.c_str());
    o("and.b32 %s, %s, 3;", t.c_str(), tid.c_str());
    o("shl.b32 %s, %s, 2;", acol.c_str(), t.c_str());
    o("shr.u32 %s, %s, 5;", brow.c_str(), tid.c_str());
    o("and.b32 %s, %s, 31;", t.c_str(), tid.c_str());
    o("shl.b32 %s, %s, 2;", bcol.c_str(), t.c_str());
    std::string abase = s.a, bbase = s.b, dbase = s.d;
    if (tail) {
        const std::string cid = R("cid"), full = R("full"), per = R("per"), tile = R("tile"), k0 = R("k0"), it0 = R("it0"), it1 = R("it1"), lgx = R("lgx"), bx = R("bx"), by = R("by");
        const std::string kbeg = R("kbeg"), nkr = R("nk"), whole = R("whole"), ta = R("ta"), tb = R("tb"), td = R("td");
        std::string l_top = "$mm" + std::to_string(u) + "_top", l_have = "$mm" + std::to_string(u) + "_have";
        o("ld.param.u32 %s, [%s_lgrid_x];", lgx.c_str(), s.kernel.c_str());
        o("ld.param.u32 %s, [%s_full_tiles];", full.c_str(), s.kernel.c_str());
        o("ld.param.u32 %s, [%s_per];", per.c_str(), s.kernel.c_str());
        o("mov.u32 %s, %%ctaid.x;", cid.c_str());
        // it1 != 0 marks a stream unit with slabs [it0, it1) of the tail tiles still to do
        o("mov.u32 %s, 0;", it0.c_str());
        o("mov.u32 %s, 0;", it1.c_str());
        o("mov.u32 %s, %s;", tile.c_str(), cid.c_str());
        o("mov.u32 %s, 0;", k0.c_str());
        o("mov.u32 %s, %d;", nkr.c_str(), nk);
        o("setp.lt.u32 %s, %s, %s;", whole.c_str(), cid.c_str(), full.c_str());
        o("@%s bra %s;", whole.c_str(), l_top.c_str());
        o("ld.param.u32 %s, [%s_lgrid_y];", t.c_str(), s.kernel.c_str());
        o("mul.lo.u32 %s, %s, %s;", t.c_str(), t.c_str(), lgx.c_str());
        o("sub.u32 %s, %s, %s;", t.c_str(), t.c_str(), full.c_str());
        o("mul.lo.u32 %s, %s, %d;", t.c_str(), t.c_str(), nk);               // slabs of all tail tiles
        o("sub.u32 %s, %s, %s;", it0.c_str(), cid.c_str(), full.c_str());
        o("mul.lo.u32 %s, %s, %s;", it0.c_str(), it0.c_str(), per.c_str());
        o("add.u32 %s, %s, %s;", it1.c_str(), it0.c_str(), per.c_str());
        o("min.u32 %s, %s, %s;", it1.c_str(), it1.c_str(), t.c_str());
        o("setp.ge.u32 %s, %s, %s;", whole.c_str(), it0.c_str(), it1.c_str());
        o("@%s bra %s;", whole.c_str(), l_skip.c_str());                    // a unit past the end of the slabs
        o.label(l_top);
        o("setp.eq.u32 %s, %s, 0;", whole.c_str(), it1.c_str());
        o("@%s bra %s;", whole.c_str(), l_have.c_str());
        // the next segment of this unit: the rest of its range, up to the end of the tile it falls in
        o("div.u32 %s, %s, %d;", tile.c_str(), it0.c_str(), nk);
        o("rem.u32 %s, %s, %d;", k0.c_str(), it0.c_str(), nk);
        o("add.u32 %s, %s, %s;", tile.c_str(), tile.c_str(), full.c_str());
        o("mov.u32 %s, %d;", nkr.c_str(), nk);
        o("sub.u32 %s, %s, %s;", nkr.c_str(), nkr.c_str(), k0.c_str());
        o("sub.u32 %s, %s, %s;", t.c_str(), it1.c_str(), it0.c_str());
        o("min.u32 %s, %s, %s;", nkr.c_str(), nkr.c_str(), t.c_str());
        o("add.u32 %s, %s, %s;", it0.c_str(), it0.c_str(), nkr.c_str());
        o.label(l_have);
        o("div.u32 %s, %s, %s;", by.c_str(), tile.c_str(), lgx.c_str());
        o("rem.u32 %s, %s, %s;", bx.c_str(), tile.c_str(), lgx.c_str());
        o("shl.b32 %s, %s, 4;", kbeg.c_str(), k0.c_str());
        // tile pointers: A + by*128*lda*4 + kbeg*4 ; B + bx*512 + kbeg*ldb*4 ; D + by*128*ldd*4 + bx*512
        o("mul.wide.u32 %s, %s, %lld;", w.c_str(), by.c_str(), 128 * lda * 4);
        o("add.u64 %s, %s, %s;", ta.c_str(), s.a_base.c_str(), w.c_str());
        o("mul.wide.u32 %s, %s, 4;", w.c_str(), kbeg.c_str());
        o("add.u64 %s, %s, %s;", ta.c_str(), ta.c_str(), w.c_str());
        o("mul.wide.u32 %s, %s, 512;", w.c_str(), bx.c_str());
        o("add.u64 %s, %s, %s;", tb.c_str(), s.b_base.c_str(), w.c_str());
        o("add.u64 %s, %s, %s;", td.c_str(), s.d_base.c_str(), w.c_str());
        o("mul.wide.u32 %s, %s, %lld;", w.c_str(), kbeg.c_str(), ldb * 4);
        o("add.u64 %s, %s, %s;", tb.c_str(), tb.c_str(), w.c_str());
        o("mul.wide.u32 %s, %s, %lld;", w.c_str(), by.c_str(), 128 * ldd * 4);
        o("add.u64 %s, %s, %s;", td.c_str(), td.c_str(), w.c_str());
        abase = ta; bbase = tb; dbase = td;
    }
    o("mul.wide.u32 %s, %s, %lld;", w.c_str(), arow.c_str(), lda * 4);
    o("add.u64 %s, %s, %s;", ag.c_str(), abase.c_str(), w.c_str());
    o("mul.wide.u32 %s, %s, 4;", w.c_str(), acol.c_str());
    o("add.u64 %s, %s, %s;", ag.c_str(), ag.c_str(), w.c_str());
    o("mul.wide.u32 %s, %s, %lld;", w.c_str(), brow.c_str(), ldb * 4);
    o("add.u64 %s, %s, %s;", bg.c_str(), bbase.c_str(), w.c_str());
    o("mul.wide.u32 %s, %s, 4;", w.c_str(), bcol.c_str());
    o("add.u64 %s, %s, %s;", bg.c_str(), bg.c_str(), w.c_str());
    o("mov.u64 %s, __mm%d_as;", w.c_str(), u);
    o("cvt.u32.u64 %s, %s;", as.c_str(), w.c_str());
    o("mov.u64 %s, __mm%d_bs;", w.c_str(), u);
    o("cvt.u32.u64 %s, %s;", bs.c_str(), w.c_str());
    // The A slab is stored transposed, As[k][m]; column m of row k lives at m ^ 8 * ((k >> 2) & 3), so that the four
    // threads that stage the same row of A (k = 0-3, 4-7, 8-11, 12-15) hit different banks.  A thread's fragment is four
    // consecutive m starting at a multiple of 4, which the swizzle keeps together.
    o("and.b32 %s, %s, 3;", t.c_str(), tid.c_str());
    o("shl.b32 %s, %s, 3;", t.c_str(), t.c_str());
    o("xor.b32 %s, %s, %s;", x.c_str(), arow.c_str(), t.c_str());
    o("mad.lo.u32 %s, %s, 512, %s;", t.c_str(), acol.c_str(), as.c_str());
    o("mad.lo.u32 %s, %s, 4, %s;", asst.c_str(), x.c_str(), t.c_str());
    o("mad.lo.u32 %s, %s, 512, %s;", t.c_str(), brow.c_str(), bs.c_str());
    o("mad.lo.u32 %s, %s, 4, %s;", bsst.c_str(), bcol.c_str(), t.c_str());
    o("mad.lo.u32 %s, %s, 16, %s;", asrd.c_str(), ty.c_str(), as.c_str());
    o("shl.b32 %s, %s, 4;", t.c_str(), ty.c_str());
    for (int q = 0; q < 4; q++) {
        o("xor.b32 %s, %s, %d;", x.c_str(), t.c_str(), q * 32);
        o("add.u32 %s, %s, %s;", R("asq", q).c_str(), as.c_str(), x.c_str());
    }
    o("mad.lo.u32 %s, %s, 16, %s;", bsrd.c_str(), tx.c_str(), bs.c_str());
    for (int i = 0; i < 16 * RG; i++) o("mov.b64 %s, 0;", acc2(i).c_str());
    auto fetch = [&](const char* pred) {
        // rows arow + SP*h of the A slab and rows brow + (NT/32)*h of the B slab, one 16-byte load each
        for (int h = 0; h < RG; h++)
            o("%sld.global.v4.f32 {%s, %s, %s, %s}, [%s+%lld];", pred, st(4 * h).c_str(), st(4 * h + 1).c_str(), st(4 * h + 2).c_str(), st(4 * h + 3).c_str(), ag.c_str(),
              (long long)h * SP * lda * 4);
        for (int h = 0; h < RG; h++)
            o("%sld.global.v4.f32 {%s, %s, %s, %s}, [%s+%lld];", pred, st(4 * RG + 4 * h).c_str(), st(4 * RG + 4 * h + 1).c_str(), st(4 * RG + 4 * h + 2).c_str(),
              st(4 * RG + 4 * h + 3).c_str(), bg.c_str(), (long long)h * (NT / 32) * ldb * 4);
    };
    auto stash = [&]() {   // into the buffer at byte offset `off`
        o("add.u32 %s, %s, %s;", x.c_str(), asst.c_str(), off.c_str());
        for (int c = 0; c < 4; c++)
            for (int h = 0; h < RG; h++) o("st.shared.f32 [%s+%d], %s;", x.c_str(), c * 512 + h * SP * 4, st(4 * h + c).c_str());
        o("add.u32 %s, %s, %s;", y.c_str(), bsst.c_str(), off.c_str());
        for (int h = 0; h < RG; h++)
            o("st.shared.v4.f32 [%s+%d], {%s, %s, %s, %s};", y.c_str(), h * (NT / 32) * 512, st(4 * RG + 4 * h).c_str(), st(4 * RG + 4 * h + 1).c_str(),
              st(4 * RG + 4 * h + 2).c_str(), st(4 * RG + 4 * h + 3).c_str());
    };
    o("mov.u32 %s, 0;", off.c_str());
    o("mov.u32 %s, 0;", kb.c_str());
    fetch("");
    stash();
    o("bar.sync 0;");
    o.label(l_loop);
    o("add.u32 %s, %s, 1;", kb1.c_str(), kb.c_str());
    if (tail) o("setp.lt.u32 %s, %s, %s;", more.c_str(), kb1.c_str(), R("nk").c_str());
    else o("setp.lt.u32 %s, %s, %d;", more.c_str(), kb1.c_str(), nk);
    o("add.u64 %s, %s, 64;", ag.c_str(), ag.c_str());
    o("add.u64 %s, %s, %lld;", bg.c_str(), bg.c_str(), 16 * ldb * 4);
    fetch(("@" + more + " ").c_str());
    for (int q = 0; q < 4; q++) o("add.u32 %s, %s, %s;", R("xq", q).c_str(), R("asq", q).c_str(), off.c_str());
    o("add.u32 %s, %s, %s;", y.c_str(), bsrd.c_str(), off.c_str());
    // Packed FP32: fma.rn.f32x2 does two IEEE fused multiply-adds per instruction (the same bits as two
    // fma.rn.f32), so a K step is 32 FMA instructions plus 8 register pairings instead of 64 FMAs.
    for (int k = 0; k < 16; k++) {
        for (int g = 0; g < RG; g++)
            o("ld.shared.v4.f32 {%s, %s, %s, %s}, [%s+%d];", fa(4 * g).c_str(), fa(4 * g + 1).c_str(), fa(4 * g + 2).c_str(), fa(4 * g + 3).c_str(), R("xq", k >> 2).c_str(),
              k * 512 + g * SP * 4);
        o("ld.shared.v2.b64 {%s, %s}, [%s+%d];", bp(0).c_str(), bp(1).c_str(), y.c_str(), k * 512);
        o("ld.shared.v2.b64 {%s, %s}, [%s+%d];", bp(2).c_str(), bp(3).c_str(), y.c_str(), k * 512 + 256);
        for (int i = 0; i < 4 * RG; i++) o("mov.b64 %s, {%s, %s};", ad(i).c_str(), fa(i).c_str(), fa(i).c_str());
        for (int i = 0; i < 4 * RG; i++)
            for (int q = 0; q < 4; q++) o("fma.rn.f32x2 %s, %s, %s, %s;", acc2(i * 4 + q).c_str(), ad(i).c_str(), bp(q).c_str(), acc2(i * 4 + q).c_str());
    }
    o("@!%s bra %s;", more.c_str(), l_done.c_str());
    o("xor.b32 %s, %s, 8192;", off.c_str(), off.c_str());
    stash();
    o("bar.sync 0;");
    o("mov.u32 %s, %s;", kb.c_str(), kb1.c_str());
    o("bra %s;", l_loop.c_str());
    o.label(l_done);
    if (tail) {
        const std::string k0 = R("k0"), per = R("per"), cid = R("cid"), uf = R("uf"), tile = R("tile"), full = R("full"), tt = R("tt"), tk = R("tk"), pv = R("p");
        const std::string ws = R("ws"), tkp = R("tkp"), pp = R("pp"), one = R("one"), t0 = R("t0"), notlast = R("notlast"), pl = R("pl");
        std::string l_store = "$mm" + std::to_string(u) + "_store", l_sum = "$mm" + std::to_string(u) + "_sum";
        o("setp.eq.u32 %s, %s, %d;", one.c_str(), R("nk").c_str(), nk);
        o("@%s bra %s;", one.c_str(), l_store.c_str());                     // a whole tile
        // A segment that is not a whole tile leaves its partial sums in the workspace, [slot][128][128]: slot 2u + 1
        // when it starts the tile (then it is the last segment of unit u), slot 2u otherwise (then it is the first).
        o("ld.param.u64 %s, [%s_workspace];", ws.c_str(), s.kernel.c_str());
        o("ld.param.u64 %s, [%s_tickets];", tkp.c_str(), s.kernel.c_str());
        o("sub.u32 %s, %s, %s;", tt.c_str(), tile.c_str(), full.c_str());
        o("mul.wide.u32 %s, %s, 4;", w.c_str(), tt.c_str());
        o("add.u64 %s, %s, %s;", tkp.c_str(), tkp.c_str(), w.c_str());
        o("mul.wide.u32 %s, %s, 2048;", w.c_str(), ty.c_str());             // row ty*4, 512 bytes per row
        o("add.u64 %s, %s, %s;", ws.c_str(), ws.c_str(), w.c_str());
        o("mul.wide.u32 %s, %s, 16;", w.c_str(), tx.c_str());
        o("add.u64 %s, %s, %s;", ws.c_str(), ws.c_str(), w.c_str());       // + this thread's position inside a slot
        o("sub.u32 %s, %s, %s;", t.c_str(), cid.c_str(), full.c_str());
        o("shl.b32 %s, %s, 1;", t.c_str(), t.c_str());
        o("setp.eq.u32 %s, %s, 0;", pl.c_str(), k0.c_str());
        o("@%s add.u32 %s, %s, 1;", pl.c_str(), t.c_str(), t.c_str());
        o("mul.wide.u32 %s, %s, 65536;", w.c_str(), t.c_str());
        o("add.u64 %s, %s, %s;", pp.c_str(), ws.c_str(), w.c_str());
        for (int i = 0; i < 4 * RG; i++) {
            int off = ((i & 3) + (i >> 2) * SP) * 512;
            o("st.global.v2.b64 [%s+%d], {%s, %s};", pp.c_str(), off, acc2(i * 4).c_str(), acc2(i * 4 + 1).c_str());
            o("st.global.v2.b64 [%s+%d], {%s, %s};", pp.c_str(), off + 256, acc2(i * 4 + 2).c_str(), acc2(i * 4 + 3).c_str());
        }
        o("membar.gl;");
        o("bar.sync 0;");
        o("setp.eq.u32 %s, %s, 0;", t0.c_str(), tid.c_str());
        o("mov.u64 %s, __mm%d_tks;", w.c_str(), u);
        o("cvt.u32.u64 %s, %s;", x.c_str(), w.c_str());
        o("@%s atom.global.add.u32 %s, [%s], 1;", t0.c_str(), tk.c_str(), tkp.c_str());
        o("@%s st.shared.u32 [%s], %s;", t0.c_str(), x.c_str(), tk.c_str());
        o("bar.sync 0;");
        o("ld.shared.u32 %s, [%s];", tk.c_str(), x.c_str());
        // the units that hold a segment of this tile: uf = tt * nk / per starts it, every later one up to
        // ((tt + 1) * nk - 1) / per begins inside it
        o("mul.lo.u32 %s, %s, %d;", t.c_str(), tt.c_str(), nk);
        o("div.u32 %s, %s, %s;", uf.c_str(), t.c_str(), per.c_str());
        o("add.u32 %s, %s, %d;", t.c_str(), t.c_str(), nk - 1);
        o("div.u32 %s, %s, %s;", tt.c_str(), t.c_str(), per.c_str());       // tt now holds the last unit
        o("sub.u32 %s, %s, %s;", t.c_str(), tt.c_str(), uf.c_str());
        o("setp.ne.u32 %s, %s, %s;", notlast.c_str(), tk.c_str(), t.c_str());
        o("@%s bra %s;", notlast.c_str(), l_next.c_str());                  // another segment finishes this tile
        o("membar.gl;");
        // the last segment to arrive adds every segment in unit order, so the bits do not depend on who was last
        for (int i = 0; i < 16 * RG; i++) o("mov.b64 %s, 0;", acc2(i).c_str());
        o("mov.u32 %s, %s;", pv.c_str(), uf.c_str());
        o.label(l_sum);
        o("shl.b32 %s, %s, 1;", t.c_str(), pv.c_str());
        o("setp.eq.u32 %s, %s, %s;", pl.c_str(), pv.c_str(), uf.c_str());
        o("@%s add.u32 %s, %s, 1;", pl.c_str(), t.c_str(), t.c_str());
        o("mul.wide.u32 %s, %s, 65536;", w.c_str(), t.c_str());
        o("add.u64 %s, %s, %s;", pp.c_str(), ws.c_str(), w.c_str());
        for (int i = 0; i < 4 * RG; i++) {
            int off = ((i & 3) + (i >> 2) * SP) * 512;
            o("ld.global.cg.v2.b64 {%s, %s}, [%s+%d];", bp(0).c_str(), bp(1).c_str(), pp.c_str(), off);
            o("ld.global.cg.v2.b64 {%s, %s}, [%s+%d];", bp(2).c_str(), bp(3).c_str(), pp.c_str(), off + 256);
            for (int j = 0; j < 4; j++) o("add.rn.f32x2 %s, %s, %s;", acc2(i * 4 + j).c_str(), acc2(i * 4 + j).c_str(), bp(j).c_str());
        }
        o("add.u32 %s, %s, 1;", pv.c_str(), pv.c_str());
        o("setp.le.u32 %s, %s, %s;", pl.c_str(), pv.c_str(), tt.c_str());
        o("@%s bra %s;", pl.c_str(), l_sum.c_str());
        o("@%s st.global.u32 [%s], 0;", t0.c_str(), tkp.c_str());           // the ticket is back at zero for the next launch
        o.label(l_store);
    }
    // rows ty*4 + (i&3) + (i>>2)*64, columns tx*4 and tx*4 + 64
    o("shl.b32 %s, %s, 2;", t.c_str(), ty.c_str());
    o("mul.wide.u32 %s, %s, %lld;", w.c_str(), t.c_str(), ldd * 4);
    o("add.u64 %s, %s, %s;", cp.c_str(), dbase.c_str(), w.c_str());
    o("mul.wide.u32 %s, %s, 16;", w.c_str(), tx.c_str());
    o("add.u64 %s, %s, %s;", cp.c_str(), cp.c_str(), w.c_str());
    for (int i = 0; i < 4 * RG; i++) {
        long long rowoff = ((i & 3) + (i >> 2) * SP) * ldd * 4;
        o("st.global.v2.b64 [%s+%lld], {%s, %s};", cp.c_str(), rowoff, acc2(i * 4).c_str(), acc2(i * 4 + 1).c_str());
        o("st.global.v2.b64 [%s+%lld], {%s, %s};", cp.c_str(), rowoff + 256, acc2(i * 4 + 2).c_str(), acc2(i * 4 + 3).c_str());
    }
    if (tail) {
        // the fused gather: the finished tile goes to the same offset behind every peer's base address (256
        // contiguous bytes per row and warp instruction), then a system-scope fence before the CTA can end
        const std::string np = R("np"), pi = R("pi"), pb = R("pb"), pz = R("pz"), pq = R("pq"), pk = R("pk");
        std::string l_peer = "$mm" + std::to_string(u) + "_peer";
        o("ld.param.u32 %s, [%s_npeers];", np.c_str(), s.kernel.c_str());
        o("setp.eq.u32 %s, %s, 0;", pk.c_str(), np.c_str());
        o("@%s bra %s;", pk.c_str(), l_next.c_str());
        // bit 31 of the count: the first table entry is the result's address in an NVLink multicast mapping of the whole
        // group, and the tile leaves with one multimem.st per 16 bytes
        o("setp.ge.u32 %s, %s, 0x80000000;", R("mc").c_str(), np.c_str());
        o("and.b32 %s, %s, 0x7fffffff;", np.c_str(), np.c_str());
        o("sub.u64 %s, %s, %s;", pq.c_str(), cp.c_str(), s.d_base.c_str());
        o("mov.u32 %s, 0;", pi.c_str());
        o("mov.b64 %s, %s_peers;", pb.c_str(), s.kernel.c_str());
        o.label(l_peer);
        o("ld.param.u64 %s, [%s];", pz.c_str(), pb.c_str());
        o("add.u64 %s, %s, %s;", pz.c_str(), pz.c_str(), pq.c_str());
        o("@%s bra %s;", R("mc").c_str(), ("$mm" + std::to_string(u) + "_mcast").c_str());
        for (int i = 0; i < 4 * RG; i++) {
            long long rowoff = ((i & 3) + (i >> 2) * SP) * ldd * 4;
            o("st.global.v2.b64 [%s+%lld], {%s, %s};", pz.c_str(), rowoff, acc2(i * 4).c_str(), acc2(i * 4 + 1).c_str());
            o("st.global.v2.b64 [%s+%lld], {%s, %s};", pz.c_str(), rowoff + 256, acc2(i * 4 + 2).c_str(), acc2(i * 4 + 3).c_str());
        }
        o("add.u64 %s, %s, 8;", pb.c_str(), pb.c_str());
        o("add.u32 %s, %s, 1;", pi.c_str(), pi.c_str());
        o("setp.lt.u32 %s, %s, %s;", pk.c_str(), pi.c_str(), np.c_str());
        o("@%s bra %s;", pk.c_str(), l_peer.c_str());
        o("bra %s;", ("$mm" + std::to_string(u) + "_sent").c_str());
        o.label("$mm" + std::to_string(u) + "_mcast");
        for (int i = 0; i < 4 * RG; i++) {
            long long rowoff = ((i & 3) + (i >> 2) * SP) * ldd * 4;
            for (int h = 0; h < 2; h++) {   // the accumulator pairs as four f32 lanes
                o("mov.b64 {%s, %s}, %s;", fa(0).c_str(), fa(1).c_str(), acc2(i * 4 + 2 * h).c_str());
                o("mov.b64 {%s, %s}, %s;", fa(2).c_str(), fa(3).c_str(), acc2(i * 4 + 2 * h + 1).c_str());
                o("multimem.st.weak.global.v4.f32 [%s+%lld], {%s, %s, %s, %s};", pz.c_str(), rowoff + 256 * h, fa(0).c_str(), fa(1).c_str(), fa(2).c_str(), fa(3).c_str());
            }
        }
        o.label("$mm" + std::to_string(u) + "_sent");
        // One thread fences for the CTA: the barrier orders every thread's peer stores before it, and the fence is
        // cumulative.  A system-scope fence in each of the 256 threads measured 1 % slower at four GPUs.
        o("setp.eq.u32 %s, %s, 0;", pk.c_str(), tid.c_str());
        o("bar.sync 0;");
        o("@%s fence.acq_rel.sys;", pk.c_str());
        // a stream unit with slabs left goes on to its next segment, once no warp still reads this one's slabs
        o.label(l_next);
        o("setp.ge.u32 %s, %s, %s;", pk.c_str(), R("it0").c_str(), R("it1").c_str());
        o("@%s bra %s;", pk.c_str(), l_skip.c_str());
        o("bar.sync 0;");
        o("bra %s;", ("$mm" + std::to_string(u) + "_top").c_str());
    }
    o.label(l_skip);
    o("bar.sync 0;");
    char pl[256];
    if (wide && s.maxntid) *s.maxntid = (unsigned)NT;
    if (tail) snprintf(pl, sizeof pl, "//!basalt.plan %s logical_block=256,1,1 block=%d,1,1 params=%u tail=%u gather=%d", s.kernel.c_str(), NT, s.nparams, in.k, s.d_param);
    else snprintf(pl, sizeof pl, "//!basalt.plan %s block=256,1,1 params=%u", s.kernel.c_str(), s.nparams);
    plan->push_back(pl);
    return true;
}

bool matmul_tcgen05(const MmaSite& s, std::vector<std::string>* decls, std::vector<std::string>* lines, std::vector<std::string>* plan) {
    const Inst& in = *s.inst;
    if (in.in_dt != Scalar::F16 || in.acc_dt != Scalar::F32 || in.out_dt != Scalar::F16 || in.a_col) return false;
    if (in.m != 128 || in.n != 128 || in.k % 64 != 0 || !s.c_is_null || !in.has_ld || !s.sole_mma) return false;
    if (s.sa != Space::Global || s.sb != Space::Global || s.sd != Space::Global || s.max_threads != 128) return false;
    if (s.a_param < 0 || s.b_param < 0 || !s.extra_params || !s.module_decls) return false;
    const bool b_nk = in.b_col;   // B stored [N x K]: K-major like A; otherwise [K x N]: MN-major
    const long long lda = in.ld[0] ? in.ld[0] : in.k, ldb = in.ld[1] ? in.ld[1] : (b_nk ? in.k : in.n), ldd = in.ld[3] ? in.ld[3] : in.n;
    if (lda % 8 || ldb % 8 || ldd % 8) return false;   // 16-byte rows for TMA and for the 16-byte stores
    const int u = s.uid, num_kb = (int)(in.k / 64), STAGES = 3, STAGE_BYTES = 32768;
    const unsigned smem = STAGES * STAGE_BYTES + 1024;
    const std::string P = "%mt" + std::to_string(u) + "_";
    auto r = [&](const char* n) { return P + n; };
    char d[512];
    snprintf(d, sizeof d, "\t.reg .b32 %stid, %swarp, %slane, %st, %stiles, %sbars, %sfull, %sempty, %saccb, %sslot, %sgu, %stmem, %sok, %skb, %ss, %sph, %spar, %sadst, %sbdst, %sm0, %sn0, %sx, %sit, %sg, %sidesc, %slb, %sh<8>, %sv<16>;",
             P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(),
             P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str());
    decls->push_back(d);
    snprintf(d, sizeof d, "\t.reg .b64 %sw, %soff, %srow, %scol, %sda, %sdb, %st0, %snow, %sdt, %scrow, %sstatus, %sma, %smb;", P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(),
             P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str());
    decls->push_back(d);
    snprintf(d, sizeof d, "\t.reg .pred %sp, %sq, %sprod, %smma, %sw1, %sacc, %sdone;", P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str(), P.c_str());
    decls->push_back(d);
    snprintf(d, sizeof d, "\t.shared .align 8 .b8 __mt%d_bars[%d];", u, 8 * (2 * STAGES + 1));
    decls->push_back(d);
    snprintf(d, sizeof d, "\t.shared .align 4 .b8 __mt%d_misc[8];", u);   // [0]: TMEM base column, [4]: a wait gave up
    decls->push_back(d);
    s.module_decls->push_back(".extern .shared .align 1024 .b8 __basalt_dyn_smem[];");
    const std::string ta = s.kernel + "_tmap_a", tb = s.kernel + "_tmap_b", stp = s.kernel + "_status";
    s.extra_params->push_back(".param .align 64 .b8 " + ta + "[128]");
    s.extra_params->push_back(".param .align 64 .b8 " + tb + "[128]");
    s.extra_params->push_back(".param .u64 " + stp);
    const std::string L = "$mt" + std::to_string(u) + "_";
    Out o{lines};
    int wait_n = 0;
    // Bounded wait on the mbarrier at shared address `bar` for phase parity `par`; on give-up
    // clears %ok and jumps to `fail`.
    auto wait = [&](const std::string& bar, const std::string& par, const std::string& fail) {
        std::string lw = L + "w" + std::to_string(wait_n) + "_loop", ld = L + "w" + std::to_string(wait_n) + "_done", lf = L + "w" + std::to_string(wait_n) + "_fail",
                    lt = L + "w" + std::to_string(wait_n) + "_t";
        wait_n++;
        o("mov.u64 %s, 0;", r("t0").c_str());
        o("mov.u32 %s, 0;", r("it").c_str());
        o.label(lw);
        o("mbarrier.try_wait.parity.shared::cta.b64 %s, [%s], %s;", r("done").c_str(), bar.c_str(), par.c_str());
        o("@%s bra %s;", r("done").c_str(), ld.c_str());
        o("ld.volatile.shared.u32 %s, [%s];", r("g").c_str(), r("gu").c_str());
        o("setp.ne.u32 %s, %s, 0;", r("q").c_str(), r("g").c_str());
        o("@%s bra %s;", r("q").c_str(), lf.c_str());
        o("add.u32 %s, %s, 1;", r("it").c_str(), r("it").c_str());
        o("and.b32 %s, %s, 63;", r("g").c_str(), r("it").c_str());
        o("setp.ne.u32 %s, %s, 0;", r("q").c_str(), r("g").c_str());
        o("@%s bra %s;", r("q").c_str(), lw.c_str());
        o("mov.u64 %s, %%globaltimer;", r("now").c_str());
        o("setp.ne.u64 %s, %s, 0;", r("q").c_str(), r("t0").c_str());
        o("@%s bra %s;", r("q").c_str(), lt.c_str());
        o("mov.u64 %s, %s;", r("t0").c_str(), r("now").c_str());
        o("bra %s;", lw.c_str());
        o.label(lt);
        o("sub.u64 %s, %s, %s;", r("dt").c_str(), r("now").c_str(), r("t0").c_str());
        o("setp.lt.u64 %s, %s, 200000000;", r("q").c_str(), r("dt").c_str());   // 200 ms
        o("@%s bra %s;", r("q").c_str(), lw.c_str());
        o("st.volatile.shared.u32 [%s], 1;", r("gu").c_str());
        o.label(lf);
        o("mov.u32 %s, 0;", r("ok").c_str());
        o("bra %s;", fail.c_str());
        o.label(ld);
    };

    o("// mma f16->f32->f16 128x128x%u: TMA + tcgen05, %s B, lda=%lld ldb=%lld ldd=%lld", in.k, b_nk ? "K-major" : "MN-major", lda, ldb, ldd);
    o("mov.u32 %s, %%ntid.x;", r("t").c_str());
    o("setp.ne.u32 %s, %s, 128;", r("p").c_str(), r("t").c_str());
    o("@%s bra %sskip;", r("p").c_str(), L.c_str());
    o("ld.param.u64 %s, [%s];", r("status").c_str(), stp.c_str());
    o("ld.volatile.global.u32 %s, [%s];", r("t").c_str(), r("status").c_str());
    o("setp.ne.u32 %s, %s, 0;", r("p").c_str(), r("t").c_str());
    o("@%s bra %sskip;", r("p").c_str(), L.c_str());   // an earlier CTA gave up: do not pile on
    o("mov.b64 %s, %s;", r("ma").c_str(), ta.c_str());   // generic addresses of the two tensor-map parameters
    o("cvta.param.u64 %s, %s;", r("ma").c_str(), r("ma").c_str());
    o("mov.b64 %s, %s;", r("mb").c_str(), tb.c_str());
    o("cvta.param.u64 %s, %s;", r("mb").c_str(), r("mb").c_str());
    o("mov.u32 %s, %%tid.x;", r("tid").c_str());
    o("shr.u32 %s, %s, 5;", r("warp").c_str(), r("tid").c_str());
    o("and.b32 %s, %s, 31;", r("lane").c_str(), r("tid").c_str());
    o("mov.u64 %s, __basalt_dyn_smem;", r("w").c_str());
    o("cvt.u32.u64 %s, %s;", r("tiles").c_str(), r("w").c_str());
    o("add.u32 %s, %s, 1023;", r("tiles").c_str(), r("tiles").c_str());
    o("and.b32 %s, %s, 0xFFFFFC00;", r("tiles").c_str(), r("tiles").c_str());
    o("mov.u64 %s, __mt%d_bars;", r("w").c_str(), u);
    o("cvt.u32.u64 %s, %s;", r("bars").c_str(), r("w").c_str());
    o("add.u32 %s, %s, %d;", r("accb").c_str(), r("bars").c_str(), 16 * STAGES);
    o("mov.u64 %s, __mt%d_misc;", r("w").c_str(), u);
    o("cvt.u32.u64 %s, %s;", r("slot").c_str(), r("w").c_str());
    o("add.u32 %s, %s, 4;", r("gu").c_str(), r("slot").c_str());
    // tile coordinates from the operand pointers: offset from the matrix base, split by the row pitch
    o("sub.u64 %s, %s, %s;", r("off").c_str(), s.a.c_str(), s.a_base.c_str());
    o("div.u64 %s, %s, %lld;", r("row").c_str(), r("off").c_str(), lda * 2);
    o("cvt.u32.u64 %s, %s;", r("m0").c_str(), r("row").c_str());
    o("sub.u64 %s, %s, %s;", r("off").c_str(), s.b.c_str(), s.b_base.c_str());
    if (b_nk) {
        o("div.u64 %s, %s, %lld;", r("row").c_str(), r("off").c_str(), ldb * 2);
        o("cvt.u32.u64 %s, %s;", r("n0").c_str(), r("row").c_str());
    } else {
        o("shr.u64 %s, %s, 1;", r("col").c_str(), r("off").c_str());
        o("cvt.u32.u64 %s, %s;", r("n0").c_str(), r("col").c_str());   // the B tile pointer sits in row 0
    }
    o("setp.ne.u32 %s, %s, 0;", r("p").c_str(), r("tid").c_str());
    o("@%s bra %sinit_done;", r("p").c_str(), L.c_str());
    o("st.volatile.shared.u32 [%s], 0;", r("gu").c_str());
    for (int i = 0; i < 2 * STAGES + 1; i++) o("mbarrier.init.shared::cta.b64 [%s+%d], 1;", r("bars").c_str(), 8 * i);
    o("fence.mbarrier_init.release.cluster;");
    o("fence.proxy.async.shared::cta;");
    o.label(L + "init_done");
    o("setp.eq.u32 %s, %s, 1;", r("w1").c_str(), r("warp").c_str());
    o("@!%s bra %salloc_done;", r("w1").c_str(), L.c_str());
    if (s.tmem_cols) *s.tmem_cols = 128;
    o("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%s], 128;", r("slot").c_str());
    o("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    o.label(L + "alloc_done");
    o("tcgen05.fence::before_thread_sync;");
    o("bar.sync 0;");
    o("tcgen05.fence::after_thread_sync;");
    o("ld.shared.u32 %s, [%s];", r("tmem").c_str(), r("slot").c_str());
    o("mov.u32 %s, 1;", r("ok").c_str());
    o("setp.eq.u32 %s, %s, 0;", r("p").c_str(), r("lane").c_str());
    o("setp.eq.u32 %s, %s, 0;", r("q").c_str(), r("warp").c_str());
    o("and.pred %s, %s, %s;", r("prod").c_str(), r("p").c_str(), r("q").c_str());
    o("and.pred %s, %s, %s;", r("mma").c_str(), r("p").c_str(), r("w1").c_str());
    o("@%s bra %sproducer;", r("prod").c_str(), L.c_str());
    o("@%s bra %sissuer;", r("mma").c_str(), L.c_str());
    o("bra %sjoin;", L.c_str());

    // ---- TMA producer: one thread ----
    o.label(L + "producer");
    o("mov.u32 %s, 0;", r("kb").c_str());
    o("mov.u32 %s, 0;", r("s").c_str());
    o("mov.u32 %s, 0;", r("ph").c_str());
    o.label(L + "p_loop");
    o("mad.lo.u32 %s, %s, 8, %s;", r("full").c_str(), r("s").c_str(), r("bars").c_str());
    o("add.u32 %s, %s, %d;", r("empty").c_str(), r("full").c_str(), 8 * STAGES);
    o("xor.b32 %s, %s, 1;", r("par").c_str(), r("ph").c_str());   // a fresh barrier passes a wait on parity 1
    wait(r("empty"), r("par"), L + "join");
    o("mad.lo.u32 %s, %s, %d, %s;", r("adst").c_str(), r("s").c_str(), STAGE_BYTES, r("tiles").c_str());
    o("add.u32 %s, %s, 16384;", r("bdst").c_str(), r("adst").c_str());
    o("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%s], %d;", r("full").c_str(), STAGE_BYTES);
    o("shl.b32 %s, %s, 6;", r("x").c_str(), r("kb").c_str());   // k coordinate of this slab
    o("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%s], [%s, {%s, %s}], [%s];", r("adst").c_str(), r("ma").c_str(), r("x").c_str(),
      r("m0").c_str(), r("full").c_str());
    if (b_nk) {
        o("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%s], [%s, {%s, %s}], [%s];", r("bdst").c_str(), r("mb").c_str(), r("x").c_str(),
          r("n0").c_str(), r("full").c_str());
    } else {
        o("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%s], [%s, {%s, %s}], [%s];", r("bdst").c_str(), r("mb").c_str(), r("n0").c_str(),
          r("x").c_str(), r("full").c_str());
        o("add.u32 %s, %s, 8192;", r("bdst").c_str(), r("bdst").c_str());
        o("add.u32 %s, %s, 64;", r("t").c_str(), r("n0").c_str());
        o("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%s], [%s, {%s, %s}], [%s];", r("bdst").c_str(), r("mb").c_str(), r("t").c_str(),
          r("x").c_str(), r("full").c_str());
    }
    o("add.u32 %s, %s, 1;", r("s").c_str(), r("s").c_str());
    o("setp.eq.u32 %s, %s, %d;", r("p").c_str(), r("s").c_str(), STAGES);
    o("@%s mov.u32 %s, 0;", r("p").c_str(), r("s").c_str());
    o("@%s xor.b32 %s, %s, 1;", r("p").c_str(), r("ph").c_str(), r("ph").c_str());
    o("add.u32 %s, %s, 1;", r("kb").c_str(), r("kb").c_str());
    o("setp.lt.u32 %s, %s, %d;", r("p").c_str(), r("kb").c_str(), num_kb);
    o("@%s bra %sp_loop;", r("p").c_str(), L.c_str());
    o("bra %sjoin;", L.c_str());

    // ---- MMA issuer: one thread ----
    // Instruction descriptor: D f32 (bits 4-5 = 1), A and B f16 (0), B major-ness in bit 16, N/8 in
    // bits 17-22, M/16 in bits 24-28.  Matrix descriptors: address/16 in bits 0-13, leading offset/16
    // in 16-29, stride offset/16 in 32-45, version 1 in 46-47, 128-byte swizzle (2) in 61-63.
    const unsigned idesc = (1u << 4) | ((b_nk ? 0u : 1u) << 16) | (16u << 17) | (8u << 24);
    const unsigned long long desc_a_hi = (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
    const unsigned long long desc_b_hi = b_nk ? desc_a_hi : ((512ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61));
    o.label(L + "issuer");
    o("mov.u32 %s, 0;", r("kb").c_str());
    o("mov.u32 %s, 0;", r("s").c_str());
    o("mov.u32 %s, 0;", r("ph").c_str());
    o("mov.u32 %s, %u;", r("idesc").c_str(), idesc);
    o.label(L + "m_loop");
    o("mad.lo.u32 %s, %s, 8, %s;", r("full").c_str(), r("s").c_str(), r("bars").c_str());
    o("add.u32 %s, %s, %d;", r("empty").c_str(), r("full").c_str(), 8 * STAGES);
    wait(r("full"), r("ph"), L + "m_end");
    o("tcgen05.fence::after_thread_sync;");
    o("mad.lo.u32 %s, %s, %d, %s;", r("adst").c_str(), r("s").c_str(), STAGE_BYTES, r("tiles").c_str());
    o("add.u32 %s, %s, 16384;", r("bdst").c_str(), r("adst").c_str());
    for (int k = 0; k < 4; k++) {
        // K-major: a K step of 16 halves is 32 bytes along the 128-byte row; MN-major B: 16 k rows = 2048 bytes
        o("add.u32 %s, %s, %d;", r("x").c_str(), r("adst").c_str(), k * 32);
        o("shr.u32 %s, %s, 4;", r("x").c_str(), r("x").c_str());
        o("and.b32 %s, %s, 0x3FFF;", r("x").c_str(), r("x").c_str());
        o("cvt.u64.u32 %s, %s;", r("da").c_str(), r("x").c_str());
        o("or.b64 %s, %s, 0x%llX;", r("da").c_str(), r("da").c_str(), desc_a_hi);
        o("add.u32 %s, %s, %d;", r("x").c_str(), r("bdst").c_str(), b_nk ? k * 32 : k * 2048);
        o("shr.u32 %s, %s, 4;", r("x").c_str(), r("x").c_str());
        o("and.b32 %s, %s, 0x3FFF;", r("x").c_str(), r("x").c_str());
        o("cvt.u64.u32 %s, %s;", r("db").c_str(), r("x").c_str());
        o("or.b64 %s, %s, 0x%llX;", r("db").c_str(), r("db").c_str(), desc_b_hi);
        if (k == 0) o("setp.ne.u32 %s, %s, 0;", r("acc").c_str(), r("kb").c_str());   // the very first MMA overwrites the accumulator
        else o("setp.ne.u32 %s, %s, 0;", r("acc").c_str(), r("idesc").c_str());   // always true
        o("tcgen05.mma.cta_group::1.kind::f16 [%s], %s, %s, %s, %s;", r("tmem").c_str(), r("da").c_str(), r("db").c_str(), r("idesc").c_str(), r("acc").c_str());
    }
    o("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%s];", r("empty").c_str());
    o("add.u32 %s, %s, 1;", r("s").c_str(), r("s").c_str());
    o("setp.eq.u32 %s, %s, %d;", r("p").c_str(), r("s").c_str(), STAGES);
    o("@%s mov.u32 %s, 0;", r("p").c_str(), r("s").c_str());
    o("@%s xor.b32 %s, %s, 1;", r("p").c_str(), r("ph").c_str(), r("ph").c_str());
    o("add.u32 %s, %s, 1;", r("kb").c_str(), r("kb").c_str());
    o("setp.lt.u32 %s, %s, %d;", r("p").c_str(), r("kb").c_str(), num_kb);
    o("@%s bra %sm_loop;", r("p").c_str(), L.c_str());
    o.label(L + "m_end");
    o("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%s];", r("accb").c_str());

    // ---- epilogue: all four warps ----
    o.label(L + "join");
    o("bar.warp.sync 0xffffffff;");
    o("mov.u32 %s, 0;", r("par").c_str());
    wait(r("accb"), r("par"), L + "drain");
    o.label(L + "drain");
    o("tcgen05.fence::after_thread_sync;");
    o("mad.lo.u32 %s, %s, 32, %s;", r("t").c_str(), r("warp").c_str(), r("lane").c_str());   // row of the tile
    o("mul.wide.u32 %s, %s, %lld;", r("w").c_str(), r("t").c_str(), ldd * 2);
    o("add.u64 %s, %s, %s;", r("crow").c_str(), s.d.c_str(), r("w").c_str());
    o("shl.b32 %s, %s, 21;", r("lb").c_str(), r("warp").c_str());   // (warp*32) << 16: the warp's TMEM lanes
    o("add.u32 %s, %s, %s;", r("lb").c_str(), r("lb").c_str(), r("tmem").c_str());
    for (int c = 0; c < 128; c += 16) {
        std::string list;
        for (int i = 0; i < 16; i++) list += (i ? ", " : "") + P + "v" + std::to_string(i);
        o("add.u32 %s, %s, %d;", r("x").c_str(), r("lb").c_str(), c);
        o("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%s}, [%s];", list.c_str(), r("x").c_str());
        o("tcgen05.wait::ld.sync.aligned;");
        for (int i = 0; i < 8; i++) o("cvt.rn.f16x2.f32 %sh%d, %sv%d, %sv%d;", P.c_str(), i, P.c_str(), 2 * i + 1, P.c_str(), 2 * i);
        o("st.global.v4.b32 [%s+%d], {%sh0, %sh1, %sh2, %sh3};", r("crow").c_str(), c * 2, P.c_str(), P.c_str(), P.c_str(), P.c_str());
        o("st.global.v4.b32 [%s+%d], {%sh4, %sh5, %sh6, %sh7};", r("crow").c_str(), c * 2 + 16, P.c_str(), P.c_str(), P.c_str(), P.c_str());
    }
    o("setp.ne.u32 %s, %s, 0;", r("p").c_str(), r("ok").c_str());
    o("@%s bra %sstatus_done;", r("p").c_str(), L.c_str());
    o("mov.u32 %s, 1;", r("t").c_str());
    o("atom.global.exch.b32 %s, [%s], %s;", r("g").c_str(), r("status").c_str(), r("t").c_str());
    o.label(L + "status_done");
    o("tcgen05.fence::before_thread_sync;");
    o("bar.sync 0;");
    o("@!%s bra %sskip;", r("w1").c_str(), L.c_str());
    o("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %s, 128;", r("tmem").c_str());
    o.label(L + "skip");
    char pl[512];
    // tmap=<param>:<element bytes>:<row elements>:<row pitch bytes>:<box inner>:<box outer>:<swizzle bytes>
    snprintf(pl, sizeof pl, "//!basalt.plan %s block=128,1,1 smem=%u params=%u tmap=%d:2:%lld:%lld:64:128:128 tmap=%d:2:%lld:%lld:64:%d:128 status=1", s.kernel.c_str(), smem, s.nparams,
             s.a_param, lda, lda * 2, s.b_param, ldb, ldb * 2, b_nk ? 128 : 64);
    plan->push_back(pl);
    return true;
}


// The fp16 kernel whose CTAs each compute one 128x128 tile addressed as
//   a = A + bid.y*128 rows, b = B + bid.x*128 columns, d = D + (bid.y*128 rows, bid.x*128 columns)
// and do nothing else.  Such a grid is re-scheduled: one persistent CTA per SM (192 threads) walks
// pairs of horizontally adjacent logical CTAs as 128x256 tiles (a 128-wide tile when the logical
// grid is odd in x), in bands of 16 tile rows.  Warp 0 is the TMA producer (four 48 KB stages),
// warp 1 issues tcgen05.mma M128 N256 K16 into one of two 256-column TMEM accumulators, warps 2-5
// drain the other accumulator, so the epilogue of a tile overlaps the main loop of the next.  The
// runtime passes the logical grid as two trailing u32 parameters and launches min(SMs, tiles) CTAs.
bool matmul_tcgen05_persistent(const MmaSite& s, std::vector<std::string>* decls, std::vector<std::string>* lines, std::vector<std::string>* plan) {
    const Inst& in = *s.inst;
    if (in.in_dt != Scalar::F16 || in.acc_dt != Scalar::F32 || in.out_dt != Scalar::F16 || in.a_col) return false;
    if (in.m != 128 || in.n != 128 || in.k % 64 != 0 || !s.c_is_null || !in.has_ld || !s.sole_mma || !s.pure_kernel || !s.affine) return false;
    if (s.sa != Space::Global || s.sb != Space::Global || s.sd != Space::Global || s.max_threads != 128) return false;
    if (!s.extra_params || !s.module_decls || !s.maxntid) return false;
    const bool b_nk = in.b_col;
    const long long lda = in.ld[0] ? in.ld[0] : in.k, ldb = in.ld[1] ? in.ld[1] : (b_nk ? in.k : in.n), ldd = in.ld[3] ? in.ld[3] : in.n;
    if (lda % 8 || ldb % 8 || ldd % 8) return false;
    // the tiling the re-scheduling relies on
    if (s.a_c0 || s.a_cx || s.a_cy != 128 * lda * 2) return false;
    if (s.b_c0 || s.b_cy || s.b_cx != (b_nk ? 128 * ldb * 2 : 256)) return false;
    if (s.d_c0 || s.d_cx != 256 || s.d_cy != 128 * ldd * 2) return false;
    const int u = s.uid, num_kb = (int)(in.k / 64), STAGE_BYTES = 49152;
    const unsigned smem = 4 * STAGE_BYTES + 1024 + 16384;   // the two-SM twin (six 32 KB stages + 16 KB of epilogue staging) is launched with the same size
    const std::string P = "%mp" + std::to_string(u) + "_", L = "$mp" + std::to_string(u) + "_";
    auto r = [&](const char* n) { return P + n; };
    std::string b32 = "\t.reg .b32 ";
    for (const char* n : {"tid", "warp", "lane", "t", "u", "tiles", "bars", "slot", "gu", "tmem", "ok", "kb", "s", "ph", "par", "full", "empty", "adst", "bdst", "m0", "n0",
                          "x", "it", "g", "idesc", "lgx", "lgy", "tn2", "ntiles", "perband", "band", "first", "rows", "rr", "mi", "nj", "width", "tile", "gstep", "local",
                          "buf", "use", "bar2", "acc", "bytes", "ew", "c", "src", "spin"})
        b32 += P + n + ", ";
    b32 += P + "h<16>, " + P + "v<32>, " + P + "wo<8>, " + P + "ro<8>, " + P + "rb<32>;";
    decls->push_back(b32);
    std::string b64 = "\t.reg .b64 ";
    for (const char* n : {"w", "da", "db", "t0", "now", "dt", "crow", "status", "ma", "mb", "pb", "pz", "pq"}) b64 += P + n + ", ";
    b64 += P + "z;";
    decls->push_back(b64);
    std::string pr = "\t.reg .pred ";
    for (const char* n : {"p", "q", "w0", "w1", "l0", "prod", "mma", "epi", "accp", "done", "wide", "all"}) pr += P + n + ", ";
    pr += P + "bx<4>;";
    decls->push_back(pr);
    char d[256];
    snprintf(d, sizeof d, "\t.shared .align 8 .b8 __mp%d_bars[96];", u);   // full[4] @0, empty[4] @32, tfull[2] @64, tempty[2] @80
    decls->push_back(d);
    snprintf(d, sizeof d, "\t.shared .align 4 .b8 __mp%d_misc[8];", u);
    decls->push_back(d);
    s.module_decls->push_back(".extern .shared .align 1024 .b8 __basalt_dyn_smem[];");
    const std::string ta = s.kernel + "_tmap_a", tb = s.kernel + "_tmap_b", stp = s.kernel + "_status", pgx = s.kernel + "_lgrid_x", pgy = s.kernel + "_lgrid_y";
    s.extra_params->push_back(".param .align 64 .b8 " + ta + "[128]");
    s.extra_params->push_back(".param .align 64 .b8 " + tb + "[128]");
    s.extra_params->push_back(".param .u64 " + stp);
    s.extra_params->push_back(".param .u32 " + pgx);
    s.extra_params->push_back(".param .u32 " + pgy);
    *s.maxntid = 192;
    Out o{lines};
    int wait_n = 0;
    auto wait = [&](const std::string& bar, const std::string& par, const std::string& fail) {
        std::string base = L + "w" + std::to_string(wait_n++);
        o("mov.u64 %s, 0;", r("t0").c_str());
        o("mov.u32 %s, 0;", r("spin").c_str());
        o.label(base + "_loop");
        o("mbarrier.try_wait.parity.shared::cta.b64 %s, [%s], %s;", r("done").c_str(), bar.c_str(), par.c_str());
        o("@%s bra %s_done;", r("done").c_str(), base.c_str());
        o("ld.volatile.shared.u32 %s, [%s];", r("g").c_str(), r("gu").c_str());
        o("setp.ne.u32 %s, %s, 0;", r("q").c_str(), r("g").c_str());
        o("@%s bra %s_fail;", r("q").c_str(), base.c_str());
        o("add.u32 %s, %s, 1;", r("spin").c_str(), r("spin").c_str());
        o("and.b32 %s, %s, 63;", r("g").c_str(), r("spin").c_str());
        o("setp.ne.u32 %s, %s, 0;", r("q").c_str(), r("g").c_str());
        o("@%s bra %s_loop;", r("q").c_str(), base.c_str());
        o("mov.u64 %s, %%globaltimer;", r("now").c_str());
        o("setp.ne.u64 %s, %s, 0;", r("q").c_str(), r("t0").c_str());
        o("@%s bra %s_t;", r("q").c_str(), base.c_str());
        o("mov.u64 %s, %s;", r("t0").c_str(), r("now").c_str());
        o("bra %s_loop;", base.c_str());
        o.label(base + "_t");
        o("sub.u64 %s, %s, %s;", r("dt").c_str(), r("now").c_str(), r("t0").c_str());
        o("setp.lt.u64 %s, %s, 200000000;", r("q").c_str(), r("dt").c_str());
        o("@%s bra %s_loop;", r("q").c_str(), base.c_str());
        o("st.volatile.shared.u32 [%s], 1;", r("gu").c_str());
        o.label(base + "_fail");
        o("mov.u32 %s, 0;", r("ok").c_str());
        o("bra %s;", fail.c_str());
        o.label(base + "_done");
    };
    // tile -> (m0, n0, width): bands of 16 tile rows, row-fastest inside a band
    auto coords = [&]() {
        o("div.u32 %s, %s, %s;", r("band").c_str(), r("tile").c_str(), r("perband").c_str());
        o("shl.b32 %s, %s, 4;", r("first").c_str(), r("band").c_str());
        o("sub.u32 %s, %s, %s;", r("rows").c_str(), r("lgy").c_str(), r("first").c_str());
        o("min.u32 %s, %s, 16;", r("rows").c_str(), r("rows").c_str());
        o("mul.lo.u32 %s, %s, %s;", r("t").c_str(), r("band").c_str(), r("perband").c_str());
        o("sub.u32 %s, %s, %s;", r("rr").c_str(), r("tile").c_str(), r("t").c_str());
        o("rem.u32 %s, %s, %s;", r("mi").c_str(), r("rr").c_str(), r("rows").c_str());
        o("add.u32 %s, %s, %s;", r("mi").c_str(), r("mi").c_str(), r("first").c_str());
        o("div.u32 %s, %s, %s;", r("nj").c_str(), r("rr").c_str(), r("rows").c_str());
        o("shl.b32 %s, %s, 7;", r("m0").c_str(), r("mi").c_str());
        o("shl.b32 %s, %s, 8;", r("n0").c_str(), r("nj").c_str());
        o("shl.b32 %s, %s, 1;", r("t").c_str(), r("nj").c_str());
        o("add.u32 %s, %s, 1;", r("t").c_str(), r("t").c_str());
        o("setp.lt.u32 %s, %s, %s;", r("wide").c_str(), r("t").c_str(), r("lgx").c_str());   // the pair's second logical CTA exists
        o("selp.u32 %s, 256, 128, %s;", r("width").c_str(), r("wide").c_str());
    };

    o("// mma f16->f32->f16 128x128x%u over a tiled grid: persistent TMA + tcgen05, 128x256 tiles, %s B", in.k, b_nk ? "K-major" : "MN-major");
    o("mov.u32 %s, %%ntid.x;", r("t").c_str());
    o("setp.ne.u32 %s, %s, 192;", r("p").c_str(), r("t").c_str());
    o("@%s bra %sskip;", r("p").c_str(), L.c_str());
    o("ld.param.u64 %s, [%s];", r("status").c_str(), stp.c_str());
    o("ld.volatile.global.u32 %s, [%s];", r("t").c_str(), r("status").c_str());
    o("setp.ne.u32 %s, %s, 0;", r("p").c_str(), r("t").c_str());
    o("@%s bra %sskip;", r("p").c_str(), L.c_str());
    o("ld.param.u32 %s, [%s];", r("lgx").c_str(), pgx.c_str());
    o("ld.param.u32 %s, [%s];", r("lgy").c_str(), pgy.c_str());
    o("mov.b64 %s, %s;", r("ma").c_str(), ta.c_str());
    o("cvta.param.u64 %s, %s;", r("ma").c_str(), r("ma").c_str());
    o("mov.b64 %s, %s;", r("mb").c_str(), tb.c_str());
    o("cvta.param.u64 %s, %s;", r("mb").c_str(), r("mb").c_str());
    o("mov.u32 %s, %%tid.x;", r("tid").c_str());
    o("shr.u32 %s, %s, 5;", r("warp").c_str(), r("tid").c_str());
    o("and.b32 %s, %s, 31;", r("lane").c_str(), r("tid").c_str());
    o("mov.u64 %s, __basalt_dyn_smem;", r("w").c_str());
    o("cvt.u32.u64 %s, %s;", r("tiles").c_str(), r("w").c_str());
    o("add.u32 %s, %s, 1023;", r("tiles").c_str(), r("tiles").c_str());
    o("and.b32 %s, %s, 0xFFFFFC00;", r("tiles").c_str(), r("tiles").c_str());
    o("mov.u64 %s, __mp%d_bars;", r("w").c_str(), u);
    o("cvt.u32.u64 %s, %s;", r("bars").c_str(), r("w").c_str());
    o("mov.u64 %s, __mp%d_misc;", r("w").c_str(), u);
    o("cvt.u32.u64 %s, %s;", r("slot").c_str(), r("w").c_str());
    o("add.u32 %s, %s, 4;", r("gu").c_str(), r("slot").c_str());
    o("add.u32 %s, %s, 1;", r("tn2").c_str(), r("lgx").c_str());
    o("shr.u32 %s, %s, 1;", r("tn2").c_str(), r("tn2").c_str());
    o("mul.lo.u32 %s, %s, %s;", r("ntiles").c_str(), r("tn2").c_str(), r("lgy").c_str());
    o("shl.b32 %s, %s, 4;", r("perband").c_str(), r("tn2").c_str());
    o("setp.ne.u32 %s, %s, 0;", r("p").c_str(), r("tid").c_str());
    o("@%s bra %sinit_done;", r("p").c_str(), L.c_str());
    o("st.volatile.shared.u32 [%s], 0;", r("gu").c_str());
    for (int i = 0; i < 10; i++) o("mbarrier.init.shared::cta.b64 [%s+%d], 1;", r("bars").c_str(), 8 * i);
    for (int i = 10; i < 12; i++) o("mbarrier.init.shared::cta.b64 [%s+%d], 4;", r("bars").c_str(), 8 * i);   // one arrival per epilogue warp
    o("fence.mbarrier_init.release.cluster;");
    o("fence.proxy.async.shared::cta;");
    o.label(L + "init_done");
    o("setp.eq.u32 %s, %s, 1;", r("w1").c_str(), r("warp").c_str());
    o("@!%s bra %salloc_done;", r("w1").c_str(), L.c_str());
    if (s.tmem_cols) *s.tmem_cols = 512;
    o("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%s], 512;", r("slot").c_str());
    o("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    o.label(L + "alloc_done");
    o("tcgen05.fence::before_thread_sync;");
    o("bar.sync 0;");
    o("tcgen05.fence::after_thread_sync;");
    o("ld.shared.u32 %s, [%s];", r("tmem").c_str(), r("slot").c_str());
    o("mov.u32 %s, 1;", r("ok").c_str());
    o("mov.u32 %s, %%ctaid.x;", r("tile").c_str());
    o("mov.u32 %s, %%nctaid.x;", r("gstep").c_str());
    o("mov.u32 %s, 0;", r("local").c_str());
    o("mov.u32 %s, 0;", r("it").c_str());
    o("setp.eq.u32 %s, %s, 0;", r("l0").c_str(), r("lane").c_str());
    o("setp.eq.u32 %s, %s, 0;", r("w0").c_str(), r("warp").c_str());
    o("and.pred %s, %s, %s;", r("prod").c_str(), r("w0").c_str(), r("l0").c_str());
    o("and.pred %s, %s, %s;", r("mma").c_str(), r("w1").c_str(), r("l0").c_str());
    o("setp.ge.u32 %s, %s, 2;", r("epi").c_str(), r("warp").c_str());
    o("@%s bra %sp_tile;", r("prod").c_str(), L.c_str());
    o("@%s bra %sm_tile;", r("mma").c_str(), L.c_str());
    o("@%s bra %se_tile;", r("epi").c_str(), L.c_str());
    o("bra %send;", L.c_str());

    // ---- producer ----
    o.label(L + "p_tile");
    o("setp.ge.u32 %s, %s, %s;", r("p").c_str(), r("tile").c_str(), r("ntiles").c_str());
    o("@%s bra %send;", r("p").c_str(), L.c_str());
    coords();
    o("shl.b32 %s, %s, 7;", r("bytes").c_str(), r("width").c_str());   // B slab: width x 64 halves
    o("add.u32 %s, %s, 16384;", r("bytes").c_str(), r("bytes").c_str());
    o("mov.u32 %s, 0;", r("kb").c_str());
    o.label(L + "p_kb");
    o("and.b32 %s, %s, 3;", r("s").c_str(), r("it").c_str());
    o("shr.u32 %s, %s, 2;", r("ph").c_str(), r("it").c_str());
    o("and.b32 %s, %s, 1;", r("ph").c_str(), r("ph").c_str());
    o("xor.b32 %s, %s, 1;", r("par").c_str(), r("ph").c_str());
    o("mad.lo.u32 %s, %s, 8, %s;", r("full").c_str(), r("s").c_str(), r("bars").c_str());
    o("add.u32 %s, %s, 32;", r("empty").c_str(), r("full").c_str());
    wait(r("empty"), r("par"), L + "p_fail");
    o("mad.lo.u32 %s, %s, %d, %s;", r("adst").c_str(), r("s").c_str(), STAGE_BYTES, r("tiles").c_str());
    o("add.u32 %s, %s, 16384;", r("bdst").c_str(), r("adst").c_str());
    o("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%s], %s;", r("full").c_str(), r("bytes").c_str());
    o("shl.b32 %s, %s, 6;", r("x").c_str(), r("kb").c_str());
    const char* tma = "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes";
    o("%s [%s], [%s, {%s, %s}], [%s];", tma, r("adst").c_str(), r("ma").c_str(), r("x").c_str(), r("m0").c_str(), r("full").c_str());
    if (b_nk) {   // boxes of 64 k x 128 n rows
        o("%s [%s], [%s, {%s, %s}], [%s];", tma, r("bdst").c_str(), r("mb").c_str(), r("x").c_str(), r("n0").c_str(), r("full").c_str());
        o("add.u32 %s, %s, 128;", r("t").c_str(), r("n0").c_str());
        o("add.u32 %s, %s, 16384;", r("u").c_str(), r("bdst").c_str());
        o("@%s %s [%s], [%s, {%s, %s}], [%s];", r("wide").c_str(), tma, r("u").c_str(), r("mb").c_str(), r("x").c_str(), r("t").c_str(), r("full").c_str());
    } else {      // boxes of 64 n x 64 k rows
        for (int h = 0; h < 4; h++) {
            o("add.u32 %s, %s, %d;", r("t").c_str(), r("n0").c_str(), 64 * h);
            o("add.u32 %s, %s, %d;", r("u").c_str(), r("bdst").c_str(), 8192 * h);
            if (h < 2) o("%s [%s], [%s, {%s, %s}], [%s];", tma, r("u").c_str(), r("mb").c_str(), r("t").c_str(), r("x").c_str(), r("full").c_str());
            else o("@%s %s [%s], [%s, {%s, %s}], [%s];", r("wide").c_str(), tma, r("u").c_str(), r("mb").c_str(), r("t").c_str(), r("x").c_str(), r("full").c_str());
        }
    }
    o("add.u32 %s, %s, 1;", r("it").c_str(), r("it").c_str());
    o("add.u32 %s, %s, 1;", r("kb").c_str(), r("kb").c_str());
    o("setp.lt.u32 %s, %s, %d;", r("p").c_str(), r("kb").c_str(), num_kb);
    o("@%s bra %sp_kb;", r("p").c_str(), L.c_str());
    o("add.u32 %s, %s, %s;", r("tile").c_str(), r("tile").c_str(), r("gstep").c_str());
    o("bra %sp_tile;", L.c_str());
    o.label(L + "p_fail");   // let the copies already issued land (2 ms, bounded) before the CTA can exit
    o("mov.u64 %s, %%globaltimer;", r("t0").c_str());
    o.label(L + "p_spin");
    o("mov.u64 %s, %%globaltimer;", r("now").c_str());
    o("sub.u64 %s, %s, %s;", r("dt").c_str(), r("now").c_str(), r("t0").c_str());
    o("setp.lt.u64 %s, %s, 2000000;", r("q").c_str(), r("dt").c_str());
    o("@%s bra %sp_spin;", r("q").c_str(), L.c_str());
    o("bra %send;", L.c_str());

    // ---- MMA issuer ----
    const unsigned idesc128 = (1u << 4) | ((b_nk ? 0u : 1u) << 16) | (16u << 17) | (8u << 24), idesc256 = (1u << 4) | ((b_nk ? 0u : 1u) << 16) | (32u << 17) | (8u << 24);
    const unsigned long long desc_a_hi = (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
    const unsigned long long desc_b_hi = b_nk ? desc_a_hi : ((512ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61));
    o.label(L + "m_tile");
    o("setp.ge.u32 %s, %s, %s;", r("p").c_str(), r("tile").c_str(), r("ntiles").c_str());
    o("@%s bra %send;", r("p").c_str(), L.c_str());
    coords();
    o("selp.u32 %s, %u, %u, %s;", r("idesc").c_str(), idesc256, idesc128, r("wide").c_str());
    o("and.b32 %s, %s, 1;", r("buf").c_str(), r("local").c_str());
    o("shr.u32 %s, %s, 1;", r("use").c_str(), r("local").c_str());
    o("and.b32 %s, %s, 1;", r("par").c_str(), r("use").c_str());
    o("xor.b32 %s, %s, 1;", r("par").c_str(), r("par").c_str());
    o("mad.lo.u32 %s, %s, 8, %s;", r("bar2").c_str(), r("buf").c_str(), r("bars").c_str());
    o("add.u32 %s, %s, 80;", r("bar2").c_str(), r("bar2").c_str());   // tempty[buf]: the epilogue has drained this accumulator
    wait(r("bar2"), r("par"), L + "end");
    o("tcgen05.fence::after_thread_sync;");
    o("mad.lo.u32 %s, %s, 256, %s;", r("acc").c_str(), r("buf").c_str(), r("tmem").c_str());
    o("mov.u32 %s, 0;", r("kb").c_str());
    o.label(L + "m_kb");
    o("and.b32 %s, %s, 3;", r("s").c_str(), r("it").c_str());
    o("shr.u32 %s, %s, 2;", r("ph").c_str(), r("it").c_str());
    o("and.b32 %s, %s, 1;", r("ph").c_str(), r("ph").c_str());
    o("mad.lo.u32 %s, %s, 8, %s;", r("full").c_str(), r("s").c_str(), r("bars").c_str());
    o("add.u32 %s, %s, 32;", r("empty").c_str(), r("full").c_str());
    wait(r("full"), r("ph"), L + "end");
    o("tcgen05.fence::after_thread_sync;");
    o("mad.lo.u32 %s, %s, %d, %s;", r("adst").c_str(), r("s").c_str(), STAGE_BYTES, r("tiles").c_str());
    o("add.u32 %s, %s, 16384;", r("bdst").c_str(), r("adst").c_str());
    // One descriptor pair per slab, stepped by constant adds: the one issuing thread has about 500 clocks
    // per slab, and a dependent chain of shifts, masks and ors per MMA is a large part of that.
    o("shr.u32 %s, %s, 4;", r("x").c_str(), r("adst").c_str());      // stage addresses are 1 KB aligned and below 256 KB: no masking needed
    o("cvt.u64.u32 %s, %s;", r("da").c_str(), r("x").c_str());
    o("or.b64 %s, %s, 0x%llX;", r("da").c_str(), r("da").c_str(), desc_a_hi);
    o("shr.u32 %s, %s, 4;", r("x").c_str(), r("bdst").c_str());
    o("cvt.u64.u32 %s, %s;", r("db").c_str(), r("x").c_str());
    o("or.b64 %s, %s, 0x%llX;", r("db").c_str(), r("db").c_str(), desc_b_hi);
    o("setp.ne.u32 %s, %s, 0;", r("accp").c_str(), r("kb").c_str());   // the tile's first MMA overwrites the accumulator
    for (int k = 0; k < 4; k++) {
        if (k) {   // 16 k: 32 bytes along a K-major row; 16 rows of 128 bytes in an MN-major slab
            o("add.u64 %s, %s, 2;", r("da").c_str(), r("da").c_str());
            o("add.u64 %s, %s, %d;", r("db").c_str(), r("db").c_str(), b_nk ? 2 : 128);
        }
        if (k == 1) o("setp.ne.u32 %s, %s, 0;", r("accp").c_str(), r("idesc").c_str());
        o("tcgen05.mma.cta_group::1.kind::f16 [%s], %s, %s, %s, %s;", r("acc").c_str(), r("da").c_str(), r("db").c_str(), r("idesc").c_str(), r("accp").c_str());
    }
    o("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%s];", r("empty").c_str());
    o("add.u32 %s, %s, 1;", r("it").c_str(), r("it").c_str());
    o("add.u32 %s, %s, 1;", r("kb").c_str(), r("kb").c_str());
    o("setp.lt.u32 %s, %s, %d;", r("p").c_str(), r("kb").c_str(), num_kb);
    o("@%s bra %sm_kb;", r("p").c_str(), L.c_str());
    o("sub.u32 %s, %s, 16;", r("bar2").c_str(), r("bar2").c_str());   // tfull[buf]
    o("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%s];", r("bar2").c_str());
    o("add.u32 %s, %s, %s;", r("tile").c_str(), r("tile").c_str(), r("gstep").c_str());
    o("add.u32 %s, %s, 1;", r("local").c_str(), r("local").c_str());
    o("bra %sm_tile;", L.c_str());

    // ---- epilogue warps ----
    o.label(L + "e_tile");
    o("setp.ge.u32 %s, %s, %s;", r("p").c_str(), r("tile").c_str(), r("ntiles").c_str());
    o("@%s bra %send;", r("p").c_str(), L.c_str());
    coords();
    o("and.b32 %s, %s, 1;", r("buf").c_str(), r("local").c_str());
    o("shr.u32 %s, %s, 1;", r("use").c_str(), r("local").c_str());
    o("and.b32 %s, %s, 1;", r("par").c_str(), r("use").c_str());
    o("mad.lo.u32 %s, %s, 8, %s;", r("bar2").c_str(), r("buf").c_str(), r("bars").c_str());
    o("add.u32 %s, %s, 64;", r("bar2").c_str(), r("bar2").c_str());   // tfull[buf]
    wait(r("bar2"), r("par"), L + "e_after" + std::to_string(0));
    o.label(L + "e_after0");
    o("setp.ne.u32 %s, %s, 0;", r("p").c_str(), r("ok").c_str());
    o("vote.sync.all.pred %s, %s, 0xffffffff;", r("all").c_str(), r("p").c_str());   // the warp stays together: tcgen05.ld is warp-collective
    o("@!%s bra %send;", r("all").c_str(), L.c_str());
    o("tcgen05.fence::after_thread_sync;");
    // Line-sized stores, as in the two-SM form: each 32-row x 64-column piece of the warp's part of the accumulator is
    // transposed through 4 KB of shared memory (16-byte units rotated by the row) and stored as whole 128-byte lines.
    o("and.b32 %s, %s, 3;", r("ew").c_str(), r("warp").c_str());   // this warp may touch TMEM lanes 32*ew .. 32*ew+31
    o("mad.lo.u32 %s, %s, 32, %s;", r("t").c_str(), r("ew").c_str(), r("m0").c_str());       // the warp's first row
    o("mul.wide.u32 %s, %s, %lld;", r("w").c_str(), r("t").c_str(), ldd * 2);
    o("add.u64 %s, %s, %s;", r("crow").c_str(), s.d_base.c_str(), r("w").c_str());
    o("mul.wide.u32 %s, %s, 2;", r("w").c_str(), r("n0").c_str());
    o("add.u64 %s, %s, %s;", r("crow").c_str(), r("crow").c_str(), r("w").c_str());
    o("shr.u32 %s, %s, 3;", r("t").c_str(), r("lane").c_str());                               // reading back: row 4i + lane/8 ...
    o("and.b32 %s, %s, 7;", r("u").c_str(), r("lane").c_str());                               // ... 16-byte unit lane%8
    o("mul.wide.u32 %s, %s, %lld;", r("w").c_str(), r("t").c_str(), ldd * 2);
    o("add.u64 %s, %s, %s;", r("crow").c_str(), r("crow").c_str(), r("w").c_str());
    o("mul.wide.u32 %s, %s, 16;", r("w").c_str(), r("u").c_str());
    o("add.u64 %s, %s, %s;", r("crow").c_str(), r("crow").c_str(), r("w").c_str());
    o("mad.lo.u32 %s, %s, 4096, %s;", r("x").c_str(), r("ew").c_str(), r("tiles").c_str());
    o("add.u32 %s, %s, %d;", r("x").c_str(), r("x").c_str(), 4 * STAGE_BYTES);                 // this warp's staging rows, past the four stages
    for (int j = 0; j < 8; j++) {
        o("xor.b32 %s, %s, %d;", r("g").c_str(), r("u").c_str(), j);
        o("shl.b32 %s, %s, 4;", r("g").c_str(), r("g").c_str());
        o("mad.lo.u32 %swo%d, %s, 128, %s;", P.c_str(), j, r("lane").c_str(), r("g").c_str());
        o("add.u32 %swo%d, %swo%d, %s;", P.c_str(), j, P.c_str(), j, r("x").c_str());
        o("add.u32 %s, %s, %d;", r("g").c_str(), r("t").c_str(), 4 * j);
        o("and.b32 %s, %s, 7;", r("c").c_str(), r("g").c_str());
        o("xor.b32 %s, %s, %s;", r("c").c_str(), r("c").c_str(), r("u").c_str());
        o("shl.b32 %s, %s, 4;", r("c").c_str(), r("c").c_str());
        o("mad.lo.u32 %sro%d, %s, 128, %s;", P.c_str(), j, r("g").c_str(), r("c").c_str());
        o("add.u32 %sro%d, %sro%d, %s;", P.c_str(), j, P.c_str(), j, r("x").c_str());
    }
    o("mad.lo.u32 %s, %s, 256, %s;", r("src").c_str(), r("buf").c_str(), r("tmem").c_str());
    o("shl.b32 %s, %s, 21;", r("t").c_str(), r("ew").c_str());
    o("add.u32 %s, %s, %s;", r("src").c_str(), r("src").c_str(), r("t").c_str());
    o("mov.u32 %s, 0;", r("c").c_str());
    o.label(L + "e_c");
    {
        std::string list;
        for (int i = 0; i < 32; i++) list += (i ? ", " : "") + P + "v" + std::to_string(i);
        for (int half = 0; half < 2; half++) {
            o("add.u32 %s, %s, %s;", r("x").c_str(), r("src").c_str(), r("c").c_str());
            if (half) o("add.u32 %s, %s, 32;", r("x").c_str(), r("x").c_str());
            o("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%s}, [%s];", list.c_str(), r("x").c_str());
            o("tcgen05.wait::ld.sync.aligned;");
            for (int i = 0; i < 16; i++) o("cvt.rn.f16x2.f32 %sh%d, %sv%d, %sv%d;", P.c_str(), i, P.c_str(), 2 * i + 1, P.c_str(), 2 * i);
            for (int q = 0; q < 4; q++)
                o("st.shared.v4.b32 [%swo%d], {%sh%d, %sh%d, %sh%d, %sh%d};", P.c_str(), 4 * half + q, P.c_str(), 4 * q, P.c_str(), 4 * q + 1, P.c_str(), 4 * q + 2, P.c_str(), 4 * q + 3);
        }
        o("bar.warp.sync 0xffffffff;");
        for (int i = 0; i < 8; i++)
            o("ld.shared.v4.b32 {%srb%d, %srb%d, %srb%d, %srb%d}, [%sro%d];", P.c_str(), 4 * i, P.c_str(), 4 * i + 1, P.c_str(), 4 * i + 2, P.c_str(), 4 * i + 3, P.c_str(), i);
        o("bar.warp.sync 0xffffffff;");   // the next piece may overwrite the staging rows
        o("mul.wide.u32 %s, %s, 2;", r("z").c_str(), r("c").c_str());
        o("add.u64 %s, %s, %s;", r("z").c_str(), r("z").c_str(), r("crow").c_str());
        for (int i = 0; i < 8; i++)
            o("st.global.v4.b32 [%s+%lld], {%srb%d, %srb%d, %srb%d, %srb%d};", r("z").c_str(), 4ll * i * ldd * 2, P.c_str(), 4 * i, P.c_str(), 4 * i + 1, P.c_str(), 4 * i + 2, P.c_str(), 4 * i + 3);
    }
    o("add.u32 %s, %s, 64;", r("c").c_str(), r("c").c_str());
    o("setp.lt.u32 %s, %s, %s;", r("p").c_str(), r("c").c_str(), r("width").c_str());
    o("@%s bra %se_c;", r("p").c_str(), L.c_str());
    o("tcgen05.fence::before_thread_sync;");
    o("bar.warp.sync 0xffffffff;");
    o("add.u32 %s, %s, 16;", r("bar2").c_str(), r("bar2").c_str());   // tempty[buf]
    o("@%s mbarrier.arrive.shared::cta.b64 _, [%s];", r("l0").c_str(), r("bar2").c_str());
    o("add.u32 %s, %s, %s;", r("tile").c_str(), r("tile").c_str(), r("gstep").c_str());
    o("add.u32 %s, %s, 1;", r("local").c_str(), r("local").c_str());
    o("bra %se_tile;", L.c_str());

    o.label(L + "end");
    o("setp.ne.u32 %s, %s, 0;", r("p").c_str(), r("ok").c_str());
    o("@%s bra %sstatus_done;", r("p").c_str(), L.c_str());
    o("mov.u32 %s, 1;", r("t").c_str());
    o("atom.global.exch.b32 %s, [%s], %s;", r("g").c_str(), r("status").c_str(), r("t").c_str());
    o.label(L + "status_done");
    o("bar.warp.sync 0xffffffff;");
    o("tcgen05.fence::before_thread_sync;");
    o("bar.sync 0;");
    o("@!%s bra %sskip;", r("w1").c_str(), L.c_str());
    o("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %s, 512;", r("tmem").c_str());
    o.label(L + "skip");
    char pl[640];
    snprintf(pl, sizeof pl,
             // an eighth tmap field gives the matrix's row count, so that the tensor map clamps: a constant, or the
             // caller's grid extent in x or y times the tile rows (A has 128 rows per grid row; B stored [N x K] has
             // 128 rows per grid column, B stored [K x N] has K rows)
             "//!basalt.plan %s logical_block=128,1,1 block=192,1,1 smem=%u params=%u tmap=%d:2:%lld:%lld:64:128:128:y128 tmap=%d:2:%lld:%lld:64:%d:128:%s status=1 lgrid=2 pair=%s__pair pair_block=256 gather=%d",
             s.kernel.c_str(), smem, s.nparams, s.a_param, lda, lda * 2, s.b_param, ldb, ldb * 2, b_nk ? 128 : 64, b_nk ? "x128" : std::to_string(in.k).c_str(), s.kernel.c_str(), s.d_param);
    plan->push_back(pl);
    return true;
}


// The same kernel as matmul_tcgen05_persistent, lowered for PAIRS of SMs (`<name>__pair`, launched by the
// runtime instead of `<name>` when the logical grid is even in x and y, i.e. M and N are multiples of
// 256).  A cluster of two CTAs owns one 256x256 tile: CTA r loads its 128 rows of A and its 128 columns of
// B (32 KB per K slab per SM instead of 48 KB, so six stages fit), both producers signal the leader's
// "full" barrier (a cta_group::2 bulk-tensor load names the barrier by its shared::cluster address; no
// multicast), the leader's warp 1 issues tcgen05.mma.cta_group::2 M256 N256 K16 for both, its commits
// (multicast to both CTAs' barriers) release the stage and publish the accumulator, the epilogue warps
// of both CTAs drain their own 128 TMEM lanes and arrive on the leader's "accumulator empty" barrier,
// and the pair meets at a cluster barrier before tensor memory is released.  Parameters, tensor maps and
// shared-memory size are those of the one-SM form, so the runtime launches either with one argument list.
bool matmul_tcgen05_pair(const MmaSite& s, std::vector<std::string>* decls, std::vector<std::string>* lines, std::vector<std::string>* plan) {
    const Inst& in = *s.inst;
    if (in.in_dt != Scalar::F16 || in.acc_dt != Scalar::F32 || in.out_dt != Scalar::F16 || in.a_col) return false;
    if (in.m != 128 || in.n != 128 || in.k % 64 != 0 || !s.c_is_null || !in.has_ld || !s.sole_mma || !s.pure_kernel || !s.affine) return false;
    if (s.sa != Space::Global || s.sb != Space::Global || s.sd != Space::Global || s.max_threads != 128) return false;
    if (!s.extra_params || !s.module_decls || !s.maxntid || !s.cluster) return false;
    const bool b_nk = in.b_col;
    const long long lda = in.ld[0] ? in.ld[0] : in.k, ldb = in.ld[1] ? in.ld[1] : (b_nk ? in.k : in.n), ldd = in.ld[3] ? in.ld[3] : in.n;
    if (lda % 8 || ldb % 8 || ldd % 8) return false;
    if (s.a_c0 || s.a_cx || s.a_cy != 128 * lda * 2) return false;
    if (s.b_c0 || s.b_cy || s.b_cx != (b_nk ? 128 * ldb * 2 : 256)) return false;
    if (s.d_c0 || s.d_cx != 256 || s.d_cy != 128 * ldd * 2) return false;
    // Six 32 KB stages: five and seven measured the same (1440 / 1444 / 1433 TFLOP/s at 8192^3), and prefetching later
    // slabs into L2 from the producers cost 13 %, so neither depth nor L2 latency is what bounds this loop.
    const int u = s.uid, num_kb = (int)(in.k / 64), STAGES = 6, STAGE_BYTES = 32768;
    const int FULL = 0, EMPTY = 8 * STAGES, TFULL = 16 * STAGES, TEMPTY = 16 * STAGES + 16;
    const std::string P = "%mq" + std::to_string(u) + "_", L = "$mq" + std::to_string(u) + "_";
    auto r = [&](const char* n) { return P + n; };
    std::string b32 = "\t.reg .b32 ";
    for (const char* n : {"tid", "warp", "lane", "t", "u", "tiles", "bars", "slot", "gu", "tmem", "ok", "kb", "s", "ph", "par", "full", "empty", "fb", "adst", "bdst", "m0", "n0",
                          "x", "it", "g", "lgx", "lgy", "tm", "tn", "ntiles", "perband", "band", "first", "rows", "rr", "mi", "nj", "tile", "gstep", "local",
                          "buf", "use", "bar2", "acc", "ew", "c", "src", "spin", "rank", "zero", "idesc", "np", "pi", "ts", "want", "row"})
        b32 += P + n + ", ";
    b32 += P + "h<16>, " + P + "v<32>, " + P + "wo<8>, " + P + "ro<8>, " + P + "rb<32>;";
    decls->push_back(b32);
    std::string b64 = "\t.reg .b64 ";
    for (const char* n : {"w", "da", "db", "t0", "now", "dt", "crow", "status", "ma", "mb", "pb", "pz", "pq"}) b64 += P + n + ", ";
    b64 += P + "z;";
    decls->push_back(b64);
    decls->push_back("\t.reg .b16 " + P + "both;");
    std::string pr = "\t.reg .pred ";
    for (const char* n : {"p", "q", "w0", "w1", "l0", "prod", "mma", "epi", "accp", "done", "all", "lead", "pk", "relay", "mc"}) pr += P + n + ", ";
    pr += P + "unused;";
    decls->push_back(pr);
    char d[256];
    snprintf(d, sizeof d, "\t.shared .align 8 .b8 __mq%d_bars[%d];", u, TEMPTY + 16);   // full[6], empty[6], tfull[2], tempty[2]
    decls->push_back(d);
    snprintf(d, sizeof d, "\t.shared .align 4 .b8 __mq%d_misc[12];", u);   // TMEM base, give-up flag, tiles stored by the epilogue warps
    decls->push_back(d);
    const std::string dyn = ".extern .shared .align 1024 .b8 __basalt_dyn_smem[];";
    if (std::find(s.module_decls->begin(), s.module_decls->end(), dyn) == s.module_decls->end()) s.module_decls->push_back(dyn);
    const std::string ta = s.kernel + "_tmap_a", tb = s.kernel + "_tmap_b", stp = s.kernel + "_status", pgx = s.kernel + "_lgrid_x", pgy = s.kernel + "_lgrid_y";
    s.extra_params->push_back(".param .align 64 .b8 " + ta + "[128]");
    s.extra_params->push_back(".param .align 64 .b8 " + tb + "[128]");
    s.extra_params->push_back(".param .u64 " + stp);
    s.extra_params->push_back(".param .u32 " + pgx);
    s.extra_params->push_back(".param .u32 " + pgy);
    // the fused gather: base addresses of the same result matrix in up to seven peers' memory (the output
    // parameter's value on each peer, mapped into this GPU's address space) and how many of them are set
    const std::string ppeers = s.kernel + "_peers", pnpeers = s.kernel + "_npeers";
    s.extra_params->push_back(".param .align 8 .b8 " + ppeers + "[56]");
    s.extra_params->push_back(".param .u32 " + pnpeers);
    *s.maxntid = 256;   // warps 0-1 producer and MMA issuer, 2-5 epilogue, 6-7 relay the finished tiles to the peers
    *s.cluster = 2;
    Out o{lines};
    int wait_n = 0;
    // Bounded wait on a barrier of this CTA: 200 ms on %globaltimer, then the CTA-wide give-up flag.
    auto wait = [&](const std::string& bar, const std::string& par, const std::string& fail) {
        std::string base = L + "w" + std::to_string(wait_n++);
        o("mov.u64 %s, 0;", r("t0").c_str());
        o("mov.u32 %s, 0;", r("spin").c_str());
        o.label(base + "_loop");
        o("mbarrier.try_wait.parity.shared::cta.b64 %s, [%s], %s;", r("done").c_str(), bar.c_str(), par.c_str());
        o("@%s bra %s_done;", r("done").c_str(), base.c_str());
        o("ld.volatile.shared.u32 %s, [%s];", r("g").c_str(), r("gu").c_str());
        o("setp.ne.u32 %s, %s, 0;", r("q").c_str(), r("g").c_str());
        o("@%s bra %s_fail;", r("q").c_str(), base.c_str());
        o("add.u32 %s, %s, 1;", r("spin").c_str(), r("spin").c_str());
        o("and.b32 %s, %s, 63;", r("g").c_str(), r("spin").c_str());
        o("setp.ne.u32 %s, %s, 0;", r("q").c_str(), r("g").c_str());
        o("@%s bra %s_loop;", r("q").c_str(), base.c_str());
        o("mov.u64 %s, %%globaltimer;", r("now").c_str());
        o("setp.ne.u64 %s, %s, 0;", r("q").c_str(), r("t0").c_str());
        o("@%s bra %s_t;", r("q").c_str(), base.c_str());
        o("mov.u64 %s, %s;", r("t0").c_str(), r("now").c_str());
        o("bra %s_loop;", base.c_str());
        o.label(base + "_t");
        o("sub.u64 %s, %s, %s;", r("dt").c_str(), r("now").c_str(), r("t0").c_str());
        o("setp.lt.u64 %s, %s, 200000000;", r("q").c_str(), r("dt").c_str());
        o("@%s bra %s_loop;", r("q").c_str(), base.c_str());
        o("st.volatile.shared.u32 [%s], 1;", r("gu").c_str());
        o.label(base + "_fail");
        o("mov.u32 %s, 0;", r("ok").c_str());
        o("bra %s;", fail.c_str());
        o.label(base + "_done");
    };
    // tile -> (mi, nj): bands of 8 tile rows, row-fastest inside a band
    auto coords = [&]() {
        o("div.u32 %s, %s, %s;", r("band").c_str(), r("tile").c_str(), r("perband").c_str());
        o("shl.b32 %s, %s, 3;", r("first").c_str(), r("band").c_str());
        o("sub.u32 %s, %s, %s;", r("rows").c_str(), r("tm").c_str(), r("first").c_str());
        o("min.u32 %s, %s, 8;", r("rows").c_str(), r("rows").c_str());
        o("mul.lo.u32 %s, %s, %s;", r("t").c_str(), r("band").c_str(), r("perband").c_str());
        o("sub.u32 %s, %s, %s;", r("rr").c_str(), r("tile").c_str(), r("t").c_str());
        o("rem.u32 %s, %s, %s;", r("mi").c_str(), r("rr").c_str(), r("rows").c_str());
        o("add.u32 %s, %s, %s;", r("mi").c_str(), r("mi").c_str(), r("first").c_str());
        o("div.u32 %s, %s, %s;", r("nj").c_str(), r("rr").c_str(), r("rows").c_str());
        o("shl.b32 %s, %s, 8;", r("m0").c_str(), r("mi").c_str());
        o("mad.lo.u32 %s, %s, 128, %s;", r("m0").c_str(), r("rank").c_str(), r("m0").c_str());   // this CTA's 128 rows of the tile
        o("shl.b32 %s, %s, 8;", r("n0").c_str(), r("nj").c_str());
    };
    // s and ph are kept as running counters (s = slab count mod STAGES, ph = its wrap parity): the one
    // thread that issues the MMAs has about 500 clocks per slab, and a dependent chain of divisions,
    // shifts and ors for every slab and every descriptor was most of that
    auto stage = [&]() {
        o("mad.lo.u32 %s, %s, 8, %s;", r("full").c_str(), r("s").c_str(), r("bars").c_str());
        o("add.u32 %s, %s, %d;", r("empty").c_str(), r("full").c_str(), EMPTY);
        o("mad.lo.u32 %s, %s, %d, %s;", r("adst").c_str(), r("s").c_str(), STAGE_BYTES, r("tiles").c_str());
        o("add.u32 %s, %s, 16384;", r("bdst").c_str(), r("adst").c_str());
    };

    auto next_stage = [&]() {
        o("add.u32 %s, %s, 1;", r("s").c_str(), r("s").c_str());
        o("setp.eq.u32 %s, %s, %d;", r("q").c_str(), r("s").c_str(), STAGES);
        o("@%s mov.u32 %s, 0;", r("q").c_str(), r("s").c_str());
        o("@%s xor.b32 %s, %s, 1;", r("q").c_str(), r("ph").c_str(), r("ph").c_str());
    };

    o("// mma f16->f32->f16 128x128x%u over a tiled grid: TMA + tcgen05.cta_group::2, 256x256 tiles on pairs of SMs, %s B", in.k, b_nk ? "K-major" : "MN-major");
    o("mov.u32 %s, %%ntid.x;", r("t").c_str());
    o("setp.ne.u32 %s, %s, 256;", r("p").c_str(), r("t").c_str());
    o("@%s bra %sskip;", r("p").c_str(), L.c_str());
    o("ld.param.u64 %s, [%s];", r("status").c_str(), stp.c_str());
    o("ld.param.u32 %s, [%s];", r("lgx").c_str(), pgx.c_str());
    o("ld.param.u32 %s, [%s];", r("lgy").c_str(), pgy.c_str());
    o("ld.param.u32 %s, [%s];", r("np").c_str(), pnpeers.c_str());
    o("mov.b64 %s, %s;", r("ma").c_str(), ta.c_str());
    o("cvta.param.u64 %s, %s;", r("ma").c_str(), r("ma").c_str());
    o("mov.b64 %s, %s;", r("mb").c_str(), tb.c_str());
    o("cvta.param.u64 %s, %s;", r("mb").c_str(), r("mb").c_str());
    o("mov.u32 %s, %%tid.x;", r("tid").c_str());
    o("shr.u32 %s, %s, 5;", r("warp").c_str(), r("tid").c_str());
    o("and.b32 %s, %s, 31;", r("lane").c_str(), r("tid").c_str());
    o("mov.u32 %s, %%cluster_ctarank;", r("rank").c_str());
    o("setp.eq.u32 %s, %s, 0;", r("lead").c_str(), r("rank").c_str());
    o("mov.u32 %s, 0;", r("zero").c_str());
    o("mov.b16 %s, 3;", r("both").c_str());
    o("mov.u64 %s, __basalt_dyn_smem;", r("w").c_str());
    o("cvt.u32.u64 %s, %s;", r("tiles").c_str(), r("w").c_str());
    o("add.u32 %s, %s, 1023;", r("tiles").c_str(), r("tiles").c_str());
    o("and.b32 %s, %s, 0xFFFFFC00;", r("tiles").c_str(), r("tiles").c_str());
    o("mov.u64 %s, __mq%d_bars;", r("w").c_str(), u);
    o("cvt.u32.u64 %s, %s;", r("bars").c_str(), r("w").c_str());
    o("mov.u64 %s, __mq%d_misc;", r("w").c_str(), u);
    o("cvt.u32.u64 %s, %s;", r("slot").c_str(), r("w").c_str());
    o("add.u32 %s, %s, 4;", r("gu").c_str(), r("slot").c_str());
    o("add.u32 %s, %s, 8;", r("ts").c_str(), r("slot").c_str());
    o("shr.u32 %s, %s, 1;", r("tn").c_str(), r("lgx").c_str());
    o("shr.u32 %s, %s, 1;", r("tm").c_str(), r("lgy").c_str());
    o("mul.lo.u32 %s, %s, %s;", r("ntiles").c_str(), r("tn").c_str(), r("tm").c_str());
    o("shl.b32 %s, %s, 3;", r("perband").c_str(), r("tn").c_str());
    o("setp.ne.u32 %s, %s, 0;", r("p").c_str(), r("tid").c_str());
    o("@%s bra %sinit_done;", r("p").c_str(), L.c_str());
    o("st.volatile.shared.u32 [%s], 0;", r("gu").c_str());
    o("st.volatile.shared.u32 [%s], 0;", r("ts").c_str());
    for (int i = 0; i < 2 * STAGES + 2; i++) o("mbarrier.init.shared::cta.b64 [%s+%d], 1;", r("bars").c_str(), 8 * i);   // full, empty, tfull
    for (int i = 0; i < 2; i++) o("mbarrier.init.shared::cta.b64 [%s+%d], 8;", r("bars").c_str(), TEMPTY + 8 * i);      // four epilogue warps in each CTA
    o("fence.mbarrier_init.release.cluster;");
    o("fence.proxy.async.shared::cta;");
    o.label(L + "init_done");
    o("setp.eq.u32 %s, %s, 1;", r("w1").c_str(), r("warp").c_str());
    o("@!%s bra %salloc_done;", r("w1").c_str(), L.c_str());
    if (s.tmem_cols) *s.tmem_cols = 512;
    o("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%s], 512;", r("slot").c_str());   // the same warp of both CTAs allocates for the pair
    o("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
    o.label(L + "alloc_done");
    o("tcgen05.fence::before_thread_sync;");
    o("bar.sync 0;");
    o("barrier.cluster.arrive.release.aligned;");   // the peer's barriers are initialised before anything can signal them
    o("barrier.cluster.wait.acquire.aligned;");
    o("tcgen05.fence::after_thread_sync;");
    o("ld.shared.u32 %s, [%s];", r("tmem").c_str(), r("slot").c_str());
    o("mov.u32 %s, 1;", r("ok").c_str());
    o("mov.u32 %s, %%ctaid.x;", r("tile").c_str());
    o("shr.u32 %s, %s, 1;", r("tile").c_str(), r("tile").c_str());
    o("mov.u32 %s, %%nctaid.x;", r("gstep").c_str());
    o("shr.u32 %s, %s, 1;", r("gstep").c_str(), r("gstep").c_str());
    o("mov.u32 %s, 0;", r("local").c_str());
    o("mov.u32 %s, 0;", r("s").c_str());
    o("mov.u32 %s, 0;", r("ph").c_str());
    o("setp.eq.u32 %s, %s, 0;", r("l0").c_str(), r("lane").c_str());
    o("setp.eq.u32 %s, %s, 0;", r("w0").c_str(), r("warp").c_str());
    o("and.pred %s, %s, %s;", r("prod").c_str(), r("w0").c_str(), r("l0").c_str());
    o("and.pred %s, %s, %s;", r("mma").c_str(), r("w1").c_str(), r("l0").c_str());
    o("and.pred %s, %s, %s;", r("mma").c_str(), r("mma").c_str(), r("lead").c_str());
    o("setp.ge.u32 %s, %s, 2;", r("epi").c_str(), r("warp").c_str());
    o("setp.ge.u32 %s, %s, 6;", r("relay").c_str(), r("warp").c_str());
    o("setp.ne.u32 %s, %s, 0;", r("pk").c_str(), r("np").c_str());           // pk: this launch gathers
    // bit 31 of the count: the first table entry is the result's address in an NVLink multicast mapping that covers every
    // GPU of the group, and a tile leaves with one multimem.st per 16 bytes, which the switch replicates
    o("setp.ge.u32 %s, %s, 0x80000000;", r("mc").c_str(), r("np").c_str());
    o("and.b32 %s, %s, 0x7fffffff;", r("np").c_str(), r("np").c_str());
    o("@%s bra %sp_tile;", r("prod").c_str(), L.c_str());
    o("@%s bra %sm_tile;", r("mma").c_str(), L.c_str());
    o("@%s bra %sr_tile;", r("relay").c_str(), L.c_str());
    o("@%s bra %se_tile;", r("epi").c_str(), L.c_str());
    o("bra %send;", L.c_str());

    // ---- producers (one thread in each CTA) ----
    o.label(L + "p_tile");
    o("setp.ge.u32 %s, %s, %s;", r("p").c_str(), r("tile").c_str(), r("ntiles").c_str());
    o("@%s bra %send;", r("p").c_str(), L.c_str());
    coords();
    o("mad.lo.u32 %s, %s, 128, %s;", r("n0").c_str(), r("rank").c_str(), r("n0").c_str());   // this CTA's 128 columns of B
    o("mov.u32 %s, 0;", r("kb").c_str());
    o.label(L + "p_kb");
    stage();
    o("xor.b32 %s, %s, 1;", r("par").c_str(), r("ph").c_str());
    wait(r("empty"), r("par"), L + "p_fail");
    o("mapa.shared::cluster.u32 %s, %s, %s;", r("fb").c_str(), r("full").c_str(), r("zero").c_str());   // the leader's barrier collects both CTAs' bytes
    o("@%s mbarrier.arrive.expect_tx.shared::cta.b64 _, [%s], %d;", r("lead").c_str(), r("full").c_str(), 2 * STAGE_BYTES);
    o("shl.b32 %s, %s, 6;", r("x").c_str(), r("kb").c_str());
    const char* tma = "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes";
    o("%s [%s], [%s, {%s, %s}], [%s];", tma, r("adst").c_str(), r("ma").c_str(), r("x").c_str(), r("m0").c_str(), r("fb").c_str());
    if (b_nk) {   // one box of 64 k x 128 n rows
        o("%s [%s], [%s, {%s, %s}], [%s];", tma, r("bdst").c_str(), r("mb").c_str(), r("x").c_str(), r("n0").c_str(), r("fb").c_str());
    } else {      // two boxes of 64 n x 64 k rows
        for (int h = 0; h < 2; h++) {
            o("add.u32 %s, %s, %d;", r("t").c_str(), r("n0").c_str(), 64 * h);
            o("add.u32 %s, %s, %d;", r("u").c_str(), r("bdst").c_str(), 8192 * h);
            o("%s [%s], [%s, {%s, %s}], [%s];", tma, r("u").c_str(), r("mb").c_str(), r("t").c_str(), r("x").c_str(), r("fb").c_str());
        }
    }
    next_stage();
    o("add.u32 %s, %s, 1;", r("kb").c_str(), r("kb").c_str());
    o("setp.lt.u32 %s, %s, %d;", r("p").c_str(), r("kb").c_str(), num_kb);
    o("@%s bra %sp_kb;", r("p").c_str(), L.c_str());
    o("add.u32 %s, %s, %s;", r("tile").c_str(), r("tile").c_str(), r("gstep").c_str());
    o("bra %sp_tile;", L.c_str());
    o.label(L + "p_fail");   // let the copies already issued land (2 ms, bounded) before the CTA can exit
    o("mov.u64 %s, %%globaltimer;", r("t0").c_str());
    o.label(L + "p_spin");
    o("mov.u64 %s, %%globaltimer;", r("now").c_str());
    o("sub.u64 %s, %s, %s;", r("dt").c_str(), r("now").c_str(), r("t0").c_str());
    o("setp.lt.u64 %s, %s, 2000000;", r("q").c_str(), r("dt").c_str());
    o("@%s bra %sp_spin;", r("q").c_str(), L.c_str());
    o("bra %send;", L.c_str());

    // ---- MMA issuer (one thread of the leader) ----
    const unsigned idesc = (1u << 4) | ((b_nk ? 0u : 1u) << 16) | (32u << 17) | (16u << 24);   // f32 accumulate, N = 256, M = 256
    const unsigned long long desc_a_hi = (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
    const unsigned long long desc_b_hi = b_nk ? desc_a_hi : ((512ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61));
    const char* commit = "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64";
    o.label(L + "m_tile");
    o("setp.ge.u32 %s, %s, %s;", r("p").c_str(), r("tile").c_str(), r("ntiles").c_str());
    o("@%s bra %send;", r("p").c_str(), L.c_str());
    o("mov.u32 %s, %u;", r("idesc").c_str(), idesc);
    o("and.b32 %s, %s, 1;", r("buf").c_str(), r("local").c_str());
    o("shr.u32 %s, %s, 1;", r("use").c_str(), r("local").c_str());
    o("and.b32 %s, %s, 1;", r("par").c_str(), r("use").c_str());
    o("xor.b32 %s, %s, 1;", r("par").c_str(), r("par").c_str());
    o("mad.lo.u32 %s, %s, 8, %s;", r("bar2").c_str(), r("buf").c_str(), r("bars").c_str());
    o("add.u32 %s, %s, %d;", r("bar2").c_str(), r("bar2").c_str(), TEMPTY);   // both epilogues have drained this accumulator
    wait(r("bar2"), r("par"), L + "end");
    o("tcgen05.fence::after_thread_sync;");
    o("mad.lo.u32 %s, %s, 256, %s;", r("acc").c_str(), r("buf").c_str(), r("tmem").c_str());
    o("mov.u32 %s, 0;", r("kb").c_str());
    o.label(L + "m_kb");
    stage();
    o("shr.u32 %s, %s, 4;", r("x").c_str(), r("adst").c_str());      // stage addresses are 1 KB aligned and below 256 KB: no masking needed
    o("cvt.u64.u32 %s, %s;", r("da").c_str(), r("x").c_str());
    o("or.b64 %s, %s, 0x%llX;", r("da").c_str(), r("da").c_str(), desc_a_hi);
    o("shr.u32 %s, %s, 4;", r("x").c_str(), r("bdst").c_str());
    o("cvt.u64.u32 %s, %s;", r("db").c_str(), r("x").c_str());
    o("or.b64 %s, %s, 0x%llX;", r("db").c_str(), r("db").c_str(), desc_b_hi);
    o("setp.ne.u32 %s, %s, 0;", r("accp").c_str(), r("kb").c_str());   // the tile's first MMA overwrites the accumulator
    wait(r("full"), r("ph"), L + "end");   // everything above is ready when the slab lands
    o("tcgen05.fence::after_thread_sync;");
    for (int k = 0; k < 4; k++) {
        if (k) {   // 16 k: 32 bytes along a K-major row; 16 rows of 128 bytes in an MN-major slab
            o("add.u64 %s, %s, 2;", r("da").c_str(), r("da").c_str());
            o("add.u64 %s, %s, %d;", r("db").c_str(), r("db").c_str(), b_nk ? 2 : 128);
        }
        if (k == 1) o("setp.eq.u32 %s, %s, 0;", r("accp").c_str(), r("zero").c_str());
        o("tcgen05.mma.cta_group::2.kind::f16 [%s], %s, %s, %s, {%s, %s, %s, %s, %s, %s, %s, %s}, %s;", r("acc").c_str(), r("da").c_str(), r("db").c_str(), r("idesc").c_str(),
          r("zero").c_str(), r("zero").c_str(), r("zero").c_str(), r("zero").c_str(), r("zero").c_str(), r("zero").c_str(), r("zero").c_str(), r("zero").c_str(), r("accp").c_str());
    }
    o("%s [%s], %s;", commit, r("empty").c_str(), r("both").c_str());   // the stage is free in both CTAs once these MMAs have read it
    next_stage();
    o("add.u32 %s, %s, 1;", r("kb").c_str(), r("kb").c_str());
    o("setp.lt.u32 %s, %s, %d;", r("p").c_str(), r("kb").c_str(), num_kb);
    o("@%s bra %sm_kb;", r("p").c_str(), L.c_str());
    o("sub.u32 %s, %s, 16;", r("bar2").c_str(), r("bar2").c_str());   // tfull[buf], in both CTAs
    o("%s [%s], %s;", commit, r("bar2").c_str(), r("both").c_str());
    o("add.u32 %s, %s, %s;", r("tile").c_str(), r("tile").c_str(), r("gstep").c_str());
    o("add.u32 %s, %s, 1;", r("local").c_str(), r("local").c_str());
    o("bra %sm_tile;", L.c_str());

    // ---- epilogue warps (four in each CTA, each CTA drains its own 128 rows) ----
    o.label(L + "e_tile");
    o("setp.ge.u32 %s, %s, %s;", r("p").c_str(), r("tile").c_str(), r("ntiles").c_str());
    o("@%s bra %send;", r("p").c_str(), L.c_str());
    coords();
    o("and.b32 %s, %s, 1;", r("buf").c_str(), r("local").c_str());
    o("shr.u32 %s, %s, 1;", r("use").c_str(), r("local").c_str());
    o("and.b32 %s, %s, 1;", r("par").c_str(), r("use").c_str());
    o("mad.lo.u32 %s, %s, 8, %s;", r("bar2").c_str(), r("buf").c_str(), r("bars").c_str());
    o("add.u32 %s, %s, %d;", r("bar2").c_str(), r("bar2").c_str(), TFULL);
    wait(r("bar2"), r("par"), L + "e_after");
    o.label(L + "e_after");
    o("setp.ne.u32 %s, %s, 0;", r("p").c_str(), r("ok").c_str());
    o("vote.sync.all.pred %s, %s, 0xffffffff;", r("all").c_str(), r("p").c_str());   // the warp stays together: tcgen05.ld is warp-collective
    o("@!%s bra %send;", r("all").c_str(), L.c_str());
    o("tcgen05.fence::after_thread_sync;");
    // The warp's 32 rows x 256 columns leave tensor memory in pieces of 64 columns.  A lane holds one row of a piece
    // (that is how tcgen05.ld 32x32b hands it out); storing from there would write 32 separate 16-byte pieces of 32
    // rows per instruction.  Instead the piece is transposed through 4 KB of shared memory (16-byte units rotated by
    // the row, so neither side has bank conflicts) and stored as whole 128-byte lines, four per instruction.
    o("and.b32 %s, %s, 3;", r("ew").c_str(), r("warp").c_str());   // this warp may touch TMEM lanes 32*ew .. 32*ew+31
    o("mad.lo.u32 %s, %s, 32, %s;", r("t").c_str(), r("ew").c_str(), r("m0").c_str());       // the warp's first row
    o("mul.wide.u32 %s, %s, %lld;", r("w").c_str(), r("t").c_str(), ldd * 2);
    o("add.u64 %s, %s, %s;", r("crow").c_str(), s.d_base.c_str(), r("w").c_str());
    o("mul.wide.u32 %s, %s, 2;", r("w").c_str(), r("n0").c_str());
    o("add.u64 %s, %s, %s;", r("crow").c_str(), r("crow").c_str(), r("w").c_str());
    o("shr.u32 %s, %s, 3;", r("t").c_str(), r("lane").c_str());                               // reading back: row 4i + lane/8 ...
    o("and.b32 %s, %s, 7;", r("u").c_str(), r("lane").c_str());                               // ... 16-byte unit lane%8
    o("mul.wide.u32 %s, %s, %lld;", r("w").c_str(), r("t").c_str(), ldd * 2);
    o("add.u64 %s, %s, %s;", r("crow").c_str(), r("crow").c_str(), r("w").c_str());
    o("mul.wide.u32 %s, %s, 16;", r("w").c_str(), r("u").c_str());
    o("add.u64 %s, %s, %s;", r("crow").c_str(), r("crow").c_str(), r("w").c_str());
    o("mad.lo.u32 %s, %s, 4096, %s;", r("x").c_str(), r("ew").c_str(), r("tiles").c_str());
    o("add.u32 %s, %s, %d;", r("x").c_str(), r("x").c_str(), STAGES * STAGE_BYTES);            // this warp's staging rows
    for (int j = 0; j < 8; j++) {   // where unit j of this lane's row goes / where read-back i comes from
        o("xor.b32 %s, %s, %d;", r("g").c_str(), r("u").c_str(), j);
        o("shl.b32 %s, %s, 4;", r("g").c_str(), r("g").c_str());
        o("mad.lo.u32 %swo%d, %s, 128, %s;", P.c_str(), j, r("lane").c_str(), r("g").c_str());
        o("add.u32 %swo%d, %swo%d, %s;", P.c_str(), j, P.c_str(), j, r("x").c_str());
        o("add.u32 %s, %s, %d;", r("g").c_str(), r("t").c_str(), 4 * j);                       // row = 4j + lane/8
        o("and.b32 %s, %s, 7;", r("c").c_str(), r("g").c_str());
        o("xor.b32 %s, %s, %s;", r("c").c_str(), r("c").c_str(), r("u").c_str());
        o("shl.b32 %s, %s, 4;", r("c").c_str(), r("c").c_str());
        o("mad.lo.u32 %sro%d, %s, 128, %s;", P.c_str(), j, r("g").c_str(), r("c").c_str());
        o("add.u32 %sro%d, %sro%d, %s;", P.c_str(), j, P.c_str(), j, r("x").c_str());
    }
    o("mad.lo.u32 %s, %s, 256, %s;", r("src").c_str(), r("buf").c_str(), r("tmem").c_str());
    o("shl.b32 %s, %s, 21;", r("t").c_str(), r("ew").c_str());
    o("add.u32 %s, %s, %s;", r("src").c_str(), r("src").c_str(), r("t").c_str());
    o("mov.u32 %s, 0;", r("c").c_str());
    o.label(L + "e_c");
    {
        std::string list;
        for (int i = 0; i < 32; i++) list += (i ? ", " : "") + P + "v" + std::to_string(i);
        for (int half = 0; half < 2; half++) {
            o("add.u32 %s, %s, %s;", r("x").c_str(), r("src").c_str(), r("c").c_str());
            if (half) o("add.u32 %s, %s, 32;", r("x").c_str(), r("x").c_str());
            o("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%s}, [%s];", list.c_str(), r("x").c_str());
            o("tcgen05.wait::ld.sync.aligned;");
            for (int i = 0; i < 16; i++) o("cvt.rn.f16x2.f32 %sh%d, %sv%d, %sv%d;", P.c_str(), i, P.c_str(), 2 * i + 1, P.c_str(), 2 * i);
            for (int q = 0; q < 4; q++)
                o("st.shared.v4.b32 [%swo%d], {%sh%d, %sh%d, %sh%d, %sh%d};", P.c_str(), 4 * half + q, P.c_str(), 4 * q, P.c_str(), 4 * q + 1, P.c_str(), 4 * q + 2, P.c_str(), 4 * q + 3);
        }
        o("bar.warp.sync 0xffffffff;");
        for (int i = 0; i < 8; i++)
            o("ld.shared.v4.b32 {%srb%d, %srb%d, %srb%d, %srb%d}, [%sro%d];", P.c_str(), 4 * i, P.c_str(), 4 * i + 1, P.c_str(), 4 * i + 2, P.c_str(), 4 * i + 3, P.c_str(), i);
        o("bar.warp.sync 0xffffffff;");   // the next piece may overwrite the staging rows
        o("mul.wide.u32 %s, %s, 2;", r("z").c_str(), r("c").c_str());
        o("add.u64 %s, %s, %s;", r("z").c_str(), r("z").c_str(), r("crow").c_str());
        for (int i = 0; i < 8; i++)
            o("st.global.v4.b32 [%s+%lld], {%srb%d, %srb%d, %srb%d, %srb%d};", r("z").c_str(), 4ll * i * ldd * 2, P.c_str(), 4 * i, P.c_str(), 4 * i + 1, P.c_str(), 4 * i + 2, P.c_str(), 4 * i + 3);
    }
    o("add.u32 %s, %s, 64;", r("c").c_str(), r("c").c_str());
    o("setp.lt.u32 %s, %s, 256;", r("p").c_str(), r("c").c_str());
    o("@%s bra %se_c;", r("p").c_str(), L.c_str());
    o("tcgen05.fence::before_thread_sync;");
    o("bar.warp.sync 0xffffffff;");
    o("add.u32 %s, %s, %d;", r("bar2").c_str(), r("bar2").c_str(), TEMPTY - TFULL);   // tempty[buf] ...
    o("mapa.shared::cluster.u32 %s, %s, %s;", r("fb").c_str(), r("bar2").c_str(), r("zero").c_str());      // ... of the leader
    o("@%s mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%s];", r("l0").c_str(), r("fb").c_str());
    // gathering: once every lane's stores of the tile are visible device-wide, the warp counts itself for the relay warps
    // (after the accumulator has been handed back: the fence is not on the MMA warp's path)
    o("@!%s bra %se_counted;", r("pk").c_str(), L.c_str());
    o("membar.gl;");
    o("bar.warp.sync 0xffffffff;");
    o("@%s red.shared.add.u32 [%s], 1;", r("l0").c_str(), r("ts").c_str());
    o.label(L + "e_counted");
    o("add.u32 %s, %s, %s;", r("tile").c_str(), r("tile").c_str(), r("gstep").c_str());
    o("add.u32 %s, %s, 1;", r("local").c_str(), r("local").c_str());
    o("bra %se_tile;", L.c_str());

    // ---- relay warps (6 and 7; only when the launch gathers): the fused gather.  The epilogue warps store a tile to this
    // GPU's result only; these two warps read every finished tile of the CTA back (it is still in L2) and store it at the
    // same offset behind every peer's base address, over NVLink, 64 rows each.  The epilogue therefore never waits on a
    // link, and link back-pressure cannot hold an accumulator back from the MMA warp. ----
    o.label(L + "r_tile");
    o("@!%s bra %send;", r("pk").c_str(), L.c_str());
    o("setp.ge.u32 %s, %s, %s;", r("p").c_str(), r("tile").c_str(), r("ntiles").c_str());
    o("@%s bra %send;", r("p").c_str(), L.c_str());
    coords();
    // bounded wait until the four epilogue warps have counted this tile: tiles stored >= 4 * (local + 1)
    o("mad.lo.u32 %s, %s, 4, 4;", r("want").c_str(), r("local").c_str());
    o("mov.u64 %s, 0;", r("t0").c_str());
    o("mov.u32 %s, 0;", r("spin").c_str());
    o.label(L + "r_wait");
    o("ld.volatile.shared.u32 %s, [%s];", r("g").c_str(), r("ts").c_str());
    o("setp.ge.u32 %s, %s, %s;", r("done").c_str(), r("g").c_str(), r("want").c_str());
    o("@%s bra %sr_ready;", r("done").c_str(), L.c_str());
    o("ld.volatile.shared.u32 %s, [%s];", r("g").c_str(), r("gu").c_str());
    o("setp.ne.u32 %s, %s, 0;", r("q").c_str(), r("g").c_str());
    o("@%s bra %sr_fail;", r("q").c_str(), L.c_str());
    o("add.u32 %s, %s, 1;", r("spin").c_str(), r("spin").c_str());
    o("and.b32 %s, %s, 63;", r("g").c_str(), r("spin").c_str());
    o("setp.ne.u32 %s, %s, 0;", r("q").c_str(), r("g").c_str());
    o("@%s bra %sr_wait;", r("q").c_str(), L.c_str());
    o("mov.u64 %s, %%globaltimer;", r("now").c_str());
    o("setp.ne.u64 %s, %s, 0;", r("q").c_str(), r("t0").c_str());
    o("@%s bra %sr_timed;", r("q").c_str(), L.c_str());
    o("mov.u64 %s, %s;", r("t0").c_str(), r("now").c_str());
    o("bra %sr_wait;", L.c_str());
    o.label(L + "r_timed");
    o("sub.u64 %s, %s, %s;", r("dt").c_str(), r("now").c_str(), r("t0").c_str());
    o("setp.lt.u64 %s, %s, 200000000;", r("q").c_str(), r("dt").c_str());
    o("@%s bra %sr_wait;", r("q").c_str(), L.c_str());
    o("st.volatile.shared.u32 [%s], 1;", r("gu").c_str());
    o.label(L + "r_fail");
    o("mov.u32 %s, 0;", r("ok").c_str());
    o("bra %send;", L.c_str());
    o.label(L + "r_ready");
    o("membar.gl;");
    // this lane's 16 bytes of the warp's first row: D + ((m0 + 64 * (warp - 6)) * ldd + n0 + 8 * lane) * 2
    o("sub.u32 %s, %s, 6;", r("t").c_str(), r("warp").c_str());
    o("mad.lo.u32 %s, %s, 64, %s;", r("t").c_str(), r("t").c_str(), r("m0").c_str());
    o("mul.wide.u32 %s, %s, %lld;", r("w").c_str(), r("t").c_str(), ldd * 2);
    o("add.u64 %s, %s, %s;", r("z").c_str(), s.d_base.c_str(), r("w").c_str());
    o("mul.wide.u32 %s, %s, 2;", r("w").c_str(), r("n0").c_str());
    o("add.u64 %s, %s, %s;", r("z").c_str(), r("z").c_str(), r("w").c_str());
    o("mul.wide.u32 %s, %s, 16;", r("w").c_str(), r("lane").c_str());
    o("add.u64 %s, %s, %s;", r("z").c_str(), r("z").c_str(), r("w").c_str());
    o("mov.u32 %s, 0;", r("row").c_str());
    o.label(L + "r_rows");
    for (int i = 0; i < 4; i++)
        o("ld.global.cg.v4.b32 {%srb%d, %srb%d, %srb%d, %srb%d}, [%s+%lld];", P.c_str(), 4 * i, P.c_str(), 4 * i + 1, P.c_str(), 4 * i + 2, P.c_str(), 4 * i + 3, r("z").c_str(), (long long)i * ldd * 2);
    o("sub.u64 %s, %s, %s;", r("pq").c_str(), r("z").c_str(), s.d_base.c_str());   // offset of these rows in the result
    o("mov.u32 %s, 0;", r("pi").c_str());
    o("mov.b64 %s, %s;", r("pb").c_str(), ppeers.c_str());
    o.label(L + "r_peer");
    o("ld.param.u64 %s, [%s];", r("pz").c_str(), r("pb").c_str());
    o("add.u64 %s, %s, %s;", r("pz").c_str(), r("pz").c_str(), r("pq").c_str());
    o("@%s bra %sr_mcast;", r("mc").c_str(), L.c_str());
    for (int i = 0; i < 4; i++)
        o("st.global.v4.b32 [%s+%lld], {%srb%d, %srb%d, %srb%d, %srb%d};", r("pz").c_str(), (long long)i * ldd * 2, P.c_str(), 4 * i, P.c_str(), 4 * i + 1, P.c_str(), 4 * i + 2, P.c_str(), 4 * i + 3);
    o("add.u64 %s, %s, 8;", r("pb").c_str(), r("pb").c_str());
    o("add.u32 %s, %s, 1;", r("pi").c_str(), r("pi").c_str());
    o("setp.lt.u32 %s, %s, %s;", r("q").c_str(), r("pi").c_str(), r("np").c_str());
    o("@%s bra %sr_peer;", r("q").c_str(), L.c_str());
    o("bra %sr_sent;", L.c_str());
    o.label(L + "r_mcast");
    for (int i = 0; i < 4; i++)
        o("multimem.st.weak.global.v4.f32 [%s+%lld], {%srb%d, %srb%d, %srb%d, %srb%d};", r("pz").c_str(), (long long)i * ldd * 2, P.c_str(), 4 * i, P.c_str(), 4 * i + 1, P.c_str(), 4 * i + 2, P.c_str(), 4 * i + 3);
    o.label(L + "r_sent");
    o("add.u64 %s, %s, %lld;", r("z").c_str(), r("z").c_str(), 4ll * ldd * 2);
    o("add.u32 %s, %s, 4;", r("row").c_str(), r("row").c_str());
    o("setp.lt.u32 %s, %s, 64;", r("q").c_str(), r("row").c_str());
    o("@%s bra %sr_rows;", r("q").c_str(), L.c_str());
    o("add.u32 %s, %s, %s;", r("tile").c_str(), r("tile").c_str(), r("gstep").c_str());
    o("add.u32 %s, %s, 1;", r("local").c_str(), r("local").c_str());
    o("bra %sr_tile;", L.c_str());

    o.label(L + "end");
    o("setp.ne.u32 %s, %s, 0;", r("p").c_str(), r("ok").c_str());
    o("@%s bra %sstatus_done;", r("p").c_str(), L.c_str());
    o("mov.u32 %s, 1;", r("t").c_str());
    o("atom.global.exch.b32 %s, [%s], %s;", r("g").c_str(), r("status").c_str(), r("t").c_str());
    o.label(L + "status_done");
    // The relay warps' stores into peer memory are performed before the kernel can end.  Only they stored there: the
    // same fence in every thread of the CTA cost 8 % of a gathering launch at four GPUs (0.284 against 0.263 ms).
    o("setp.ne.u32 %s, %s, 0;", r("pk").c_str(), r("np").c_str());
    o("and.pred %s, %s, %s;", r("q").c_str(), r("pk").c_str(), r("relay").c_str());
    o("@%s fence.acq_rel.sys;", r("q").c_str());
    o("bar.warp.sync 0xffffffff;");
    o("tcgen05.fence::before_thread_sync;");
    o("bar.sync 0;");
    o("barrier.cluster.arrive.release.aligned;");   // the peer has stopped naming this CTA's barriers, shared and tensor memory
    o("barrier.cluster.wait.acquire.aligned;");
    o("tcgen05.fence::after_thread_sync;");
    o("@!%s bra %sskip;", r("w1").c_str(), L.c_str());
    o("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %s, 512;", r("tmem").c_str());
    o.label(L + "skip");
    (void)FULL;
    (void)plan;   // launched through the plan of the one-SM entry, whose `pair=` key names this one
    return true;
}

}  // namespace

bool emit_mma_fast(const MmaSite& site, std::vector<std::string>* decls, std::vector<std::string>* lines, std::vector<std::string>* plan) {
    if (site.pair_twin) return matmul_tcgen05_pair(site, decls, lines, plan);
    return sgemm_ffma(site, decls, lines, plan) || matmul_tcgen05_persistent(site, decls, lines, plan) || matmul_tcgen05(site, decls, lines, plan);
}

}  // namespace basalt
