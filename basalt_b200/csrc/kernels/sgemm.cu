// Hand-written fp32 SGEMM for sm_100a: C = A*B, row-major, FFMA only (no TF32 tensor cores).
//
// FP32-pipe bound: 128x128 CTA tile, K slab of 16, 256 threads each owning an 8x8 block of C as
// four 4x4 quadrants so that every shared-memory read is a conflict-free 16-byte access; the next
// K slab is loaded into four float4 registers before the current one is multiplied and stored to the
// other half of a shared-memory double buffer after it (staging it with 4-byte cp.async copies
// instead, one LSU instruction per element of the transposed A slab, measured 50.6 against 56.3
// TFLOP/s at 4096^3; that form is kept behind an A/B switch).  Per K step a
// thread issues 4 LDS.128 for 32 packed FMAs (__ffma2_rn: two IEEE fused multiply-adds per
// instruction, the same bits as two fmaf).  The transposed A slab is swizzled -- column m of row k
// sits at m ^ 8 * ((k >> 2) & 3) -- so that the four threads staging one row of A hit different banks.
// Two CTAs are resident per SM (32 KB shared each).
//
// Tail wave.  With R resident CTAs (2 per SM) and T tiles, the last T mod R tiles would run as a
// mostly empty wave (4096^2 in 128x128 tiles: 1024 tiles on 296 slots is 3.46 waves, paid as 4; a
// 1024-row shard of it is 256 tiles, 0.86 of a wave paid as one).  Those tail tiles are instead
// worked off by R stream units: their K slabs (16 columns of A each) are laid end to end, tile after
// tile, and unit u takes slabs [u * per, (u + 1) * per) with per = ceil(tail slabs / R), so every slot
// is busy for per / (K / 16) of a tile's time.  A unit's range may end one tile and begin the next: a
// segment that covers a whole tile is stored; any other segment leaves its 128x128 partial sums in
// the workspace (two slots per unit) and takes a ticket of its tile; the segment that takes the
// tile's last ticket adds all of the tile's segments in unit order -- the result does not depend on
// arrival order -- stores the tile, and sets the ticket back to zero, so the workspace needs no
// clearing between launches.  The grid is one-dimensional: CTA c below F (the full tiles) computes
// tile c over all of K; CTA F + u is stream unit u.  CTAs are dispatched in index order, so the
// units form the last wave.
#include <algorithm>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "../../../include/basalt_b200_kernels.h"
#include "common.cuh"

namespace {

template <int BYTES>
__device__ __forceinline__ void cp_async(void* smem_dst, const void* gmem_src) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    if constexpr (BYTES == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem_src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(dst), "l"(gmem_src), "n"(BYTES) : "memory");
}

constexpr int BM = 128, BN = 128, BK = 16, THREADS = 256;

// WARP_ROWS: how the 128 x 128 tile is cut into per-thread 64-output blocks.  false: an 8 x 8 block as four 4 x 4
// quadrants (rows ty*4 + {0..3} + {0, 64}, columns tx*4 + {0..3} + {0, 64}; a warp is 2 x 16 threads).  true: a 16 x 4
// block -- warp w owns rows 16w .. 16w+15 of the tile over all 128 columns, lane l columns 4l .. 4l+3 -- so that the
// four A fragments of a K step are the same address for the whole warp (pure broadcasts, one shared-memory wavefront
// each) and the one B fragment is 512 contiguous bytes (four wavefronts): eight wavefronts per K step instead of
// thirteen, and a warp's stores are whole 512-byte rows.
// One segment: K slabs [k0, k0 + nk) of tile `tile`, by the whole CTA.  A whole tile (nk == K / 16) is stored; any other
// segment goes through the workspace as described above.  Not inlined: as a function of its own it is allocated
// registers for its main loop alone (inlined at both call sites of the kernel it measured 55.0 against 57.9 TFLOP/s).
template <bool REG_STAGE, bool WARP_ROWS>
__device__ __noinline__ void sgemm_segment(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int N, int K, int tile, int k0, int nk,
                                           int full_tiles, int per, float* __restrict__ workspace, unsigned* __restrict__ tickets) {
    // As holds the A slab transposed ([k][m]) so a thread's 4 consecutive rows are one float4.
    __shared__ __align__(16) float As[2][BK][BM];
    __shared__ __align__(16) float Bs[2][BK][BN];
    __shared__ unsigned ticket_word;
    unsigned* const ticket_s = &ticket_word;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int tiles_n = N / BN, nkt = K / BK;
    // global -> register staging: A slab is 128 rows x 16 floats (4 float4 per row), B slab is
    // 16 rows x 128 floats (32 float4 per row); two float4 of each per thread.
    const int a_row = tid >> 2, a_col = (tid & 3) * 4;   // rows a_row and a_row + 64
    const int a_sw = a_row ^ ((tid & 3) << 3);           // swizzled column of the transposed slab: rows a_col .. a_col+3 all have (k >> 2) & 3 == tid & 3
    const int b_row = tid >> 5, b_col = (tid & 31) * 4;  // rows b_row and b_row + 8
    // four running pointers, advanced by one K slab per iteration; set at the start of every segment
    const float *Ag0 = nullptr, *Ag1 = nullptr, *Bg0 = nullptr, *Bg1 = nullptr;
    const size_t b_step = (size_t)BK * N;
    // global -> shared with cp.async, no staging registers: A lands transposed as eight 4-byte
    // copies per thread, B as two 16-byte copies; one commit group per K slab.
    auto copy_slab = [&](int buf) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
            cp_async<4>(&As[buf][a_col + c][a_sw], Ag0 + c);
            cp_async<4>(&As[buf][a_col + c][a_sw + 64], Ag1 + c);
        }
        cp_async<16>(&Bs[buf][b_row][b_col], Bg0);
        cp_async<16>(&Bs[buf][b_row + 8][b_col], Bg1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        Ag0 += BK; Ag1 += BK; Bg0 += b_step; Bg1 += b_step;
    };

    constexpr int RI = WARP_ROWS ? 16 : 8, PJ = WARP_ROWS ? 2 : 4;
    const int lane = tid & 31, wrp = tid >> 5;
    float2 acc2[RI][PJ];   // acc2[i][p] = (C[i][2p], C[i][2p+1]) of the thread's block
    // position of output row i / first column of the thread's block inside the tile
    auto out_row = [&](int i) { return WARP_ROWS ? wrp * 16 + i : ty * 4 + (i & 3) + (i >> 2) * 64; };
    const int out_col = WARP_ROWS ? lane * 4 : tx * 4;

    // REG_STAGE: the next slab is loaded into four float4 registers before the multiply and stored to the other
    // half of the double buffer after it (the transposed A slab as eight 4-byte stores), instead of 4-byte cp.async
    // copies, which cost an LSU instruction per element: 16-byte global loads, the latency behind the multiply.
    float4 ra0, ra1, rb0, rb1;
    auto fetch = [&]() {
        ra0 = __ldg(reinterpret_cast<const float4*>(Ag0)); ra1 = __ldg(reinterpret_cast<const float4*>(Ag1));
        rb0 = __ldg(reinterpret_cast<const float4*>(Bg0)); rb1 = __ldg(reinterpret_cast<const float4*>(Bg1));
        Ag0 += BK; Ag1 += BK; Bg0 += b_step; Bg1 += b_step;
    };
    auto stash = [&](int buf) {
        As[buf][a_col + 0][a_sw] = ra0.x; As[buf][a_col + 1][a_sw] = ra0.y; As[buf][a_col + 2][a_sw] = ra0.z; As[buf][a_col + 3][a_sw] = ra0.w;
        As[buf][a_col + 0][a_sw + 64] = ra1.x; As[buf][a_col + 1][a_sw + 64] = ra1.y; As[buf][a_col + 2][a_sw + 64] = ra1.z; As[buf][a_col + 3][a_sw + 64] = ra1.w;
        *reinterpret_cast<float4*>(&Bs[buf][b_row][b_col]) = rb0;
        *reinterpret_cast<float4*>(&Bs[buf][b_row + 8][b_col]) = rb1;
    };
    const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
    Ag0 = A + (size_t)(m0 + a_row) * K + k0 * BK + a_col;
    Ag1 = Ag0 + (size_t)64 * K;
    Bg0 = B + (size_t)(k0 * BK + b_row) * N + n0 + b_col;
    Bg1 = Bg0 + (size_t)8 * N;
#pragma unroll
    for (int i = 0; i < RI; i++)
#pragma unroll
        for (int p = 0; p < PJ; p++) acc2[i][p] = make_float2(0.0f, 0.0f);
    if (REG_STAGE) { fetch(); stash(0); }
    else { copy_slab(0); asm volatile("cp.async.wait_group 0;" ::: "memory"); }
    __syncthreads();
    for (int kb = 0; kb < nk; kb++) {
        const int buf = kb & 1;
        if (kb + 1 < nk) { if (REG_STAGE) fetch(); else copy_slab(buf ^ 1); }   // lands while this slab is multiplied
#pragma unroll
        for (int k = 0; k < BK; k++) {
            if constexpr (WARP_ROWS) {
                const int sw = ((k >> 2) & 3) << 3;
                const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][lane * 4]);
                const float2 bp0 = make_float2(b0.x, b0.y), bp1 = make_float2(b0.z, b0.w);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const float4 aq = *reinterpret_cast<const float4*>(&As[buf][k][(wrp * 16 + q * 4) ^ sw]);
                    const float a[4] = {aq.x, aq.y, aq.z, aq.w};
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        const float2 ai = make_float2(a[r], a[r]);
                        acc2[q * 4 + r][0] = __ffma2_rn(ai, bp0, acc2[q * 4 + r][0]);
                        acc2[q * 4 + r][1] = __ffma2_rn(ai, bp1, acc2[q * 4 + r][1]);
                    }
                }
                continue;
            }
            const int m = (ty * 4) ^ (((k >> 2) & 3) << 3);
            const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][m]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][m + 64]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4 + 64]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float2 b[4] = {make_float2(b0.x, b0.y), make_float2(b0.z, b0.w), make_float2(b1.x, b1.y), make_float2(b1.z, b1.w)};
            if constexpr (!WARP_ROWS) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float2 ai = make_float2(a[i], a[i]);
#pragma unroll
                    for (int p = 0; p < 4; p++) acc2[i][p] = __ffma2_rn(ai, b[p], acc2[i][p]);
                }
            }
        }
        if (REG_STAGE) { if (kb + 1 < nk) stash(buf ^ 1); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
    }
    if (nk != nkt) {
        // A segment that is not a whole tile leaves its partial sums in the workspace: slot 2u + 1 when it starts the
        // tile (then it is the last segment of unit u), slot 2u otherwise (then it is the first): [slot][128][128].
        const unsigned t = (unsigned)(tile - full_tiles), unit = blockIdx.x - (unsigned)full_tiles;
        float* mine = workspace + (size_t)(2 * unit + (k0 == 0 ? 1u : 0u)) * (BM * BN);
#pragma unroll
        for (int i = 0; i < RI; i++) {
            float* prow = mine + out_row(i) * BN + out_col;
            *reinterpret_cast<float4*>(prow) = make_float4(acc2[i][0].x, acc2[i][0].y, acc2[i][1].x, acc2[i][1].y);
            if constexpr (!WARP_ROWS) *reinterpret_cast<float4*>(prow + 64) = make_float4(acc2[i][PJ - 2].x, acc2[i][PJ - 2].y, acc2[i][PJ - 1].x, acc2[i][PJ - 1].y);
        }
        // the units that hold a segment of this tile: the first starts the tile, every later one begins inside it
        const unsigned u_first = t * (unsigned)nkt / (unsigned)per, u_last = ((t + 1) * (unsigned)nkt - 1) / (unsigned)per;
        __threadfence();
        __syncthreads();
        if (tid == 0) *ticket_s = atomicAdd(&tickets[t], 1u);
        __syncthreads();
        if (*ticket_s != u_last - u_first) return;   // not the last segment of this tile to finish
        __threadfence();
#pragma unroll
        for (int i = 0; i < RI; i++)
#pragma unroll
            for (int p = 0; p < PJ; p++) acc2[i][p] = make_float2(0.0f, 0.0f);
        for (unsigned u = u_first; u <= u_last; u++) {   // segments are added in unit order, whichever finished last
            const float* base = workspace + (size_t)(2 * u + (u == u_first ? 1u : 0u)) * (BM * BN);
#pragma unroll
            for (int i = 0; i < RI; i++) {
                const int off = out_row(i) * BN + out_col, hi_off = WARP_ROWS ? 0 : 64;
                const float4 lo = __ldcg(reinterpret_cast<const float4*>(base + off)), hi = __ldcg(reinterpret_cast<const float4*>(base + off + hi_off));
                acc2[i][0].x += lo.x; acc2[i][0].y += lo.y; acc2[i][1].x += lo.z; acc2[i][1].y += lo.w;
                if constexpr (!WARP_ROWS) { acc2[i][PJ - 2].x += hi.x; acc2[i][PJ - 2].y += hi.y; acc2[i][PJ - 1].x += hi.z; acc2[i][PJ - 1].y += hi.w; }
            }
        }
        if (tid == 0) tickets[t] = 0;   // ready for the next launch
    }
#pragma unroll
    for (int i = 0; i < RI; i++) {
        float* crow = C + (size_t)(m0 + out_row(i)) * N + n0 + out_col;
        *reinterpret_cast<float4*>(crow) = make_float4(acc2[i][0].x, acc2[i][0].y, acc2[i][1].x, acc2[i][1].y);
        if constexpr (!WARP_ROWS) *reinterpret_cast<float4*>(crow + 64) = make_float4(acc2[i][PJ - 2].x, acc2[i][PJ - 2].y, acc2[i][PJ - 1].x, acc2[i][PJ - 1].y);
    }
}

template <bool REG_STAGE, bool WARP_ROWS>
__global__ void __launch_bounds__(THREADS, 2) sgemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                                                               int M, int N, int K, int full_tiles, int per, float* __restrict__ workspace,
                                                               unsigned* __restrict__ tickets) {
    const int nkt = K / BK;
    // CTA c < full_tiles computes tile c over all of K.
    if ((int)blockIdx.x < full_tiles) {
        sgemm_segment<REG_STAGE, WARP_ROWS>(A, B, C, N, K, (int)blockIdx.x, 0, nkt, full_tiles, per, workspace, tickets);
        return;
    }
    // CTA full_tiles + u is stream unit u: it walks K slabs [u * per, (u + 1) * per) of the tail tiles' slabs laid end
    // to end, segment by segment; a segment ends with the tile it falls in.
    const unsigned total = (unsigned)((M / BM) * (N / BN) - full_tiles) * (unsigned)nkt;
    unsigned it0 = (blockIdx.x - (unsigned)full_tiles) * (unsigned)per;
    const unsigned it1 = min(it0 + (unsigned)per, total);
    while (it0 < it1) {
        const int tile = full_tiles + (int)(it0 / (unsigned)nkt), k0 = (int)(it0 % (unsigned)nkt), nk = min(nkt - k0, (int)(it1 - it0));
        sgemm_segment<REG_STAGE, WARP_ROWS>(A, B, C, N, K, tile, k0, nk, full_tiles, per, workspace, tickets);
        it0 += (unsigned)nk;
        __syncthreads();   // the slabs of this segment are no longer read
    }
}

// Workspace of the tail wave, one per device: two partial tiles per stream unit and one ticket per
// tail tile (never more than the unit count).  Allocated on first use and kept.
struct TailWorkspace {
    float* partials = nullptr;
    unsigned* tickets = nullptr;
    int slots = 0;
};
TailWorkspace* tail_workspace(int slots) {
    static TailWorkspace per_device[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    TailWorkspace& w = per_device[dev];
    if (w.slots >= slots) return &w;
    if (w.partials) { cudaFree(w.partials); cudaFree(w.tickets); w = TailWorkspace{}; }
    if (cudaMalloc(&w.partials, (size_t)slots * BM * BN * sizeof(float)) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
    if (cudaMalloc(&w.tickets, (size_t)slots * sizeof(unsigned)) != cudaSuccess || cudaMemset(w.tickets, 0, (size_t)slots * sizeof(unsigned)) != cudaSuccess) {
        (void)cudaGetLastError();
        cudaFree(w.partials);
        w = TailWorkspace{};
        return nullptr;
    }
    w.slots = slots;
    return &w;
}

// Plans the tail wave: tiles [0, *full) run whole, the rest are worked off by *units stream units of *per K slabs
// each.  The units take per / (K / 16) of a tile's time instead of one; the traffic of the partial sums (at most two
// 64 KB tiles written and read per unit, charged at 6 TB/s against a tile time of 0.17 us per K step) is set
// against that, and a gain of less than 3 % is not taken.  `max_units` bounds the unit count (0 = the slots).
void plan_tail(int tiles, int slots, int K, int max_units, int* full, int* per, int* units) {
    *full = tiles;
    *per = 0;
    *units = 0;
    const long long tail = tiles % slots, nkt = K / BK;   // the whole problem, when it is less than one wave
    if (tail == 0 || tail * nkt >= (1ll << 31)) return;
    long long u = slots;
    if (max_units > 0 && u > max_units) u = max_units;
    const long long p = (tail * nkt + u - 1) / u;
    if (p >= nkt) return;                                 // no more units than tiles: nothing to gain
    u = (tail * nkt + p - 1) / p;
    const double cost = (double)p / (double)nkt + (double)(2 * u) * 131072.0 / 6.0e6 / (0.17 * (double)K);
    if (cost > 0.97) return;
    *full = tiles - (int)tail;
    *per = (int)p;
    *units = (int)u;
}

}  // namespace

extern "C" int basalt_k_sgemm_f32(const float* A, const float* B, float* C, int M, int N, int K, void* stream) {
    return basalt_k_sgemm_f32_variant(A, B, C, M, N, K, 0, stream);
}

extern "C" int basalt_k_sgemm_f32_variant(const float* A, const float* B, float* C, int M, int N, int K, int flags, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (M % BM || N % BN || K % BK) return basalt_k::record_msg(1, "sgemm_f32", "M and N must be multiples of 128 and K of 16");
    if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) return basalt_k::record_msg(1, "sgemm_f32", "matrices must be 16-byte aligned");
    static int resident = 0;
    if (!resident) resident = basalt_k::resident_ctas(sgemm_f32_kernel<true, false>, THREADS);
    const int tiles = (M / BM) * (N / BN), slots = resident * basalt_k::sm_count();
    int full = tiles, per = 0, units = 0;
    if (!(flags & BASALT_K_SGEMM_NO_TAIL_SPLIT)) plan_tail(tiles, slots, K, 0, &full, &per, &units);
    TailWorkspace* w = nullptr;
    if (units > 0) {
        w = tail_workspace(2 * slots);   // two partial tiles per unit, one ticket per tail tile
        if (!w) { full = tiles; per = units = 0; }   // no workspace: the plain schedule is still correct
    }
    const int grid = full + units;
    if (flags & BASALT_K_SGEMM_CP_ASYNC)   // the earlier staging with 4-byte cp.async copies
        sgemm_f32_kernel<false, false><<<grid, THREADS, 0, (cudaStream_t)stream>>>(A, B, C, M, N, K, full, per, w ? w->partials : nullptr, w ? w->tickets : nullptr);
    else if (flags & BASALT_K_SGEMM_WARP_ROWS)
        sgemm_f32_kernel<true, true><<<grid, THREADS, 0, (cudaStream_t)stream>>>(A, B, C, M, N, K, full, per, w ? w->partials : nullptr, w ? w->tickets : nullptr);
    else sgemm_f32_kernel<true, false><<<grid, THREADS, 0, (cudaStream_t)stream>>>(A, B, C, M, N, K, full, per, w ? w->partials : nullptr, w ? w->tickets : nullptr);
    return basalt_k::record(cudaGetLastError(), "sgemm_f32");
}

// ---- the same SGEMM with its tail workspace in a static device array: allocates nothing ----------
namespace {
constexpr int STATIC_MAX_PARTS = 304;    // partial tiles: two per stream unit, so at most 152 units
constexpr int STATIC_MAX_TICKETS = 256;  // tail tiles (fewer than the units)
constexpr size_t STATIC_PARTIAL_BYTES = (size_t)STATIC_MAX_PARTS * BM * BN * sizeof(float);   // 19 MiB
constexpr size_t STATIC_WS_BYTES = STATIC_PARTIAL_BYTES + STATIC_MAX_TICKETS * sizeof(unsigned);
static __device__ __align__(256) unsigned char g_static_tail_ws[STATIC_WS_BYTES];

struct StaticWs {
    unsigned char* base = nullptr;   // device address of g_static_tail_ws on this device
};
}  // namespace

extern "C" int basalt_k_sgemm_f32_static_workspace(const float* A, const float* B, float* C, int M, int N, int K, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (M % BM || N % BN || K % BK) return basalt_k::record_msg(1, "sgemm_f32_static_workspace", "M and N must be multiples of 128 and K of 16");
    if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) return basalt_k::record_msg(1, "sgemm_f32_static_workspace", "matrices must be 16-byte aligned");
    static StaticWs per_device[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return basalt_k::record(e, "sgemm_f32_static_workspace (cudaGetDevice)");
    if (dev < 0 || dev >= 64) return basalt_k::record_msg(1, "sgemm_f32_static_workspace", "device ordinal out of range");
    StaticWs& w = per_device[dev];
    if (!w.base) {   // set-up, once per device, with that device current
        unsigned char* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_static_tail_ws);
        if (e != cudaSuccess) return basalt_k::record(e, "sgemm_f32_static_workspace (cudaGetSymbolAddress)");
        w.base = p;
    }
    static int resident = 0;
    if (!resident) resident = basalt_k::resident_ctas(sgemm_f32_kernel<true, false>, THREADS);
    const int tiles = (M / BM) * (N / BN), slots = resident * basalt_k::sm_count();
    int full = tiles, per = 0, units = 0;
    plan_tail(tiles, slots, K, STATIC_MAX_PARTS / 2, &full, &per, &units);   // no more units than the array has slot pairs for
    const int tail = tiles - full;
    if (units > 0 && (2 * units > STATIC_MAX_PARTS || tail > STATIC_MAX_TICKETS)) {
        char msg[200];
        snprintf(msg, sizeof msg, "the tail wave needs %d partial tiles and %d tickets; the static workspace holds %d and %d", 2 * units, tail, STATIC_MAX_PARTS, STATIC_MAX_TICKETS);
        return basalt_k::record_msg(1, "sgemm_f32_static_workspace", msg);
    }
    float* partials = reinterpret_cast<float*>(w.base);
    unsigned* tickets = reinterpret_cast<unsigned*>(w.base + STATIC_PARTIAL_BYTES);
    if (units > 0) {   // the tickets must start at zero; the kernel leaves them at zero again
        e = cudaMemsetAsync(tickets, 0, (size_t)tail * sizeof(unsigned), (cudaStream_t)stream);
        if (e != cudaSuccess) return basalt_k::record(e, "sgemm_f32_static_workspace (cudaMemsetAsync)");
    }
    const int grid = full + units;
    sgemm_f32_kernel<true, false><<<grid, THREADS, 0, (cudaStream_t)stream>>>(A, B, C, M, N, K, full, per, partials, tickets);
    return basalt_k::record(cudaGetLastError(), "sgemm_f32_static_workspace");
}
