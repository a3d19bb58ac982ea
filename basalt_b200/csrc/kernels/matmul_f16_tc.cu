// Hand-written fp16 matmul for sm_100a on the fifth-generation tensor cores.
//
//   C[M x N] (f16) = A[M x K] (f16) * B (f16), fp32 accumulation in tensor memory.
//
// One CTA of 128 threads computes one 128 x 128 tile of C (the BLOCK_M = BLOCK_N = 128,
// BLOCK_K = 64 tiling of the Triton-style source kernel):
//   * thread 0 of warp 0 is the TMA producer: per 64-deep K slab it issues tiled bulk-tensor
//     loads of the A tile (128 rows x 128 bytes) and the B tile into a ring of shared-memory
//     stages laid out with the 128-byte swizzle the tensor core's matrix descriptors expect;
//   * thread 0 of warp 1 issues the MMAs: four tcgen05.mma (M128 N128 K16) per slab read A and B
//     straight from shared memory through 64-bit matrix descriptors and accumulate into 128
//     columns of TMEM; tcgen05.commit arrives on the stage's "empty" barrier when the MMAs that
//     read it have finished, and on the "accumulator ready" barrier after the last slab;
//   * all four warps then drain the accumulator: warp w owns TMEM lanes 32w..32w+31 (rows of the
//     tile), reads 16 columns at a time with tcgen05.ld, converts to f16 and stores 32-byte runs.
// Two CTAs fit on an SM (3 stages x 32 KB each, 128 TMEM columns each), so one CTA's epilogue
// overlaps the other's main loop.
//
// Every wait on an mbarrier is bounded; when a wait gives up the kernel records a code in
// `status`, carries on without the data (the result is then wrong, and the host reports it), and
// still releases its tensor memory before it returns; CTAs that start after that return at once.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../../include/basalt_b200_kernels.h"
#include "common.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 64, UMMA_K = 16, THREADS = 128;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr uint32_t TMEM_COLS = 128;
constexpr uint64_t WAIT_LIMIT_NS = 200ull * 1000 * 1000;   // a wait gives up after 200 ms

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait for the phase with the given parity. Gives up after WAIT_LIMIT_NS, or at once when
// another wait of this CTA has already given up (`*gave_up`, in shared memory); returns false then.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* gave_up) {
    uint64_t t0 = 0;
    for (uint32_t i = 0;; i++) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
        if (*gave_up) return false;
        if ((i & 63) == 63) {
            const uint64_t now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_LIMIT_NS) { *gave_up = 1; return false; }
        }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst), "l"(map),
                 "r"(bar), "r"(x), "r"(y)
                 : "memory");
}
// 64-bit shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.
// Addresses and offsets are encoded in 16-byte units.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <int STAGES, bool B_IS_NK>
__global__ void __launch_bounds__(THREADS) matmul_f16_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                                __half* __restrict__ C, int N, int K, int32_t* status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile uint32_t gave_up;
    // The swizzle pattern is a function of the absolute shared address: stages start on 1 KB.
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int num_kb = K / BK;

    if (status && *reinterpret_cast<volatile int32_t*>(status) != 0) return;   // an earlier CTA gave up: do not pile on
    if (threadIdx.x == 0) {
        gave_up = 0;
        for (int s = 0; s < STAGES; s++) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(&acc_bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {   // one warp allocates the accumulator's TMEM columns for the CTA
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_acc = tmem_slot;
    bool ok = true;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        for (int kb = 0; kb < num_kb; kb++) {
            const int s = kb % STAGES;
            const uint32_t parity = ((kb / STAGES) & 1) ^ 1;   // a fresh barrier passes a wait on parity 1
            ok &= mbar_wait(smem_u32(&empty_bar[s]), parity, &gave_up);
            if (!ok) break;   // issue nothing more; the copies already in flight land long before the CTA exits
            const uint32_t fb = smem_u32(&full_bar[s]), a_dst = tiles + s * STAGE_BYTES, b_dst = a_dst + A_BYTES;
            mbar_expect_tx(fb, STAGE_BYTES);
            tma_load_2d(a_dst, &map_a, fb, kb * BK, m0);               // box: 64 k (128 B) x 128 rows
            if (B_IS_NK) tma_load_2d(b_dst, &map_b, fb, kb * BK, n0);  // box: 64 k (128 B) x 128 n
            else {                                                     // box: 64 n (128 B) x 64 k, twice
                tma_load_2d(b_dst, &map_b, fb, n0, kb * BK);
                tma_load_2d(b_dst + B_BYTES / 2, &map_b, fb, n0 + 64, kb * BK);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        // Instruction descriptor: D = f32 (bits 4-5 = 1), A = B = f16 (0), A K-major, B K-major or
        // MN-major (bit 16), N/8 in bits 17-22, M/16 in bits 24-28.
        const uint32_t idesc = (1u << 4) | ((B_IS_NK ? 0u : 1u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
        for (int kb = 0; kb < num_kb; kb++) {
            const int s = kb % STAGES;
            ok &= mbar_wait(smem_u32(&full_bar[s]), (kb / STAGES) & 1, &gave_up);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_src = tiles + s * STAGE_BYTES, b_src = a_src + A_BYTES;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; k++) {
                // K-major tile: rows of 128 B, 8-row groups 1024 B apart; a K step of 16 halves is
                // 32 B along the row.  MN-major B: 64-wide n halves 8192 B apart (leading offset),
                // 8-row k groups 1024 B apart; a K step of 16 rows is 2048 B.
                const uint64_t da = smem_desc(a_src + k * UMMA_K * 2, 16, 1024);
                const uint64_t db = B_IS_NK ? smem_desc(b_src + k * UMMA_K * 2, 16, 1024) : smem_desc(b_src + k * UMMA_K * 128, B_BYTES / 2, 1024);
                umma_f16(tmem_acc, da, db, idesc, (kb | k) != 0);
            }
            umma_commit(smem_u32(&empty_bar[s]));   // stage reusable once these MMAs have read it
        }
        umma_commit(smem_u32(&acc_bar));            // accumulator complete
    }
    __syncwarp();

    // ---- epilogue: TMEM -> registers -> f16 -> global ----
    ok &= mbar_wait(smem_u32(&acc_bar), 0, &gave_up);   // on give-up the drain still runs (warp-uniformly) on whatever TMEM holds
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __half* crow = C + (size_t)(m0 + warp * 32 + lane) * N + n0;
    const uint32_t lane_base = tmem_acc + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
    for (int c = 0; c < BN; c += 16) {
        uint32_t r[16];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
              "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(lane_base + (uint32_t)c));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        uint32_t h[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            __half2 v = __floats2half2_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
            h[i] = *reinterpret_cast<uint32_t*>(&v);
        }
        *reinterpret_cast<uint4*>(crow + c) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(crow + c + 8) = make_uint4(h[4], h[5], h[6], h[7]);
    }
    if (!ok && status) atomicExch(status, 1);

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(TMEM_COLS) : "memory");
}

// ---- persistent, warp-specialised kernel: 128 x 256 tiles ---------------------------------------
//
// One CTA per SM (192 threads) walks a list of 128 x 256 output tiles:
//   warp 0 (one lane)  TMA producer, four 48 KB stages (A 128x64, B 64x256 per stage);
//   warp 1 (one lane)  tcgen05.mma M128 N256 K16 into one of two 256-column TMEM accumulators;
//   warps 2-5          epilogue: drain the other accumulator (tcgen05.ld), convert, store.
// The epilogue of tile i therefore overlaps the main loop of tile i+1, and a 256-wide tile reads
// 12 KB of shared memory per 128x256x16 MMA instead of 16 KB for two 128-wide ones.  Tiles are
// visited in bands of 16 tile rows so that the tiles in flight share A and B panels in L2.
namespace v2 {
constexpr int BN2 = 256, STAGES = 4, THREADS2 = 192, B_BYTES2 = BN2 * BK * 2, STAGE_BYTES2 = A_BYTES + B_BYTES2;
constexpr int GROUP_M = 16;
constexpr uint32_t TMEM_COLS2 = 512;

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int* m_idx, int* n_idx) {
    const int per_band = GROUP_M * tiles_n, band = t / per_band, first = band * GROUP_M;
    const int rows = min(GROUP_M, tiles_m - first), r = t - band * per_band;
    *m_idx = first + r % rows;
    *n_idx = r / rows;
}

template <bool B_IS_NK>
__global__ void __launch_bounds__(THREADS2, 1) matmul_f16_tc_persistent(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                                        __half* __restrict__ C, int M, int N, int K, int32_t* status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], tfull_bar[2], tempty_bar[2];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile uint32_t gave_up;
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = M / BM, tiles_n = N / BN2, num_tiles = tiles_m * tiles_n, num_kb = K / BK;

    if (status && *reinterpret_cast<volatile int32_t*>(status) != 0) return;
    if (threadIdx.x == 0) {
        gave_up = 0;
        for (int s = 0; s < STAGES; s++) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(smem_u32(&tfull_bar[b]), 1);
            mbar_init(smem_u32(&tempty_bar[b]), 4);   // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS2) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;   // running k-slab count across tiles: stage = it % STAGES, phase = (it / STAGES) & 1
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                int mi, ni;
                tile_coords(t, tiles_m, tiles_n, &mi, &ni);
                const int m0 = mi * BM, n0 = ni * BN2;
                for (int kb = 0; kb < num_kb; kb++, it++) {
                    const uint32_t s = it % STAGES, parity = ((it / STAGES) & 1) ^ 1;
                    ok &= mbar_wait(smem_u32(&empty_bar[s]), parity, &gave_up);
                    if (!ok) break;
                    const uint32_t fb = smem_u32(&full_bar[s]), a_dst = tiles + s * STAGE_BYTES2, b_dst = a_dst + A_BYTES;
                    mbar_expect_tx(fb, STAGE_BYTES2);
                    tma_load_2d(a_dst, &map_a, fb, kb * BK, m0);
                    if (B_IS_NK) tma_load_2d(b_dst, &map_b, fb, kb * BK, n0);   // box 64 k x 256 n
                    else {
#pragma unroll
                        for (int h = 0; h < 4; h++) tma_load_2d(b_dst + h * 8192, &map_b, fb, n0 + 64 * h, kb * BK);   // box 64 n x 64 k
                    }
                }
            }
            if (!ok) {   // let the copies already issued land before the CTA can exit
                const uint64_t t0 = global_ns();
                while (global_ns() - t0 < 2000000ull) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | ((B_IS_NK ? 0u : 1u) << 16) | ((uint32_t)(BN2 >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            uint32_t it = 0, local = 0;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, local++) {
                const uint32_t buf = local & 1, use = local >> 1;
                ok &= mbar_wait(smem_u32(&tempty_bar[buf]), (use & 1) ^ 1, &gave_up);   // epilogue has drained this accumulator
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + buf * BN2;
                for (int kb = 0; kb < num_kb; kb++, it++) {
                    const uint32_t s = it % STAGES;
                    ok &= mbar_wait(smem_u32(&full_bar[s]), (it / STAGES) & 1, &gave_up);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_src = tiles + s * STAGE_BYTES2, b_src = a_src + A_BYTES;
                    const uint64_t da = smem_desc(a_src, 16, 1024);   // one descriptor pair per slab, stepped by constant adds
                    const uint64_t db = B_IS_NK ? smem_desc(b_src, 16, 1024) : smem_desc(b_src, 8192, 1024);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++)
                        umma_f16(acc, da + (uint64_t)(2 * k), db + (uint64_t)((B_IS_NK ? 2 : 128) * k), idesc, (kb | k) != 0);
                    umma_commit(smem_u32(&empty_bar[s]));
                }
                umma_commit(smem_u32(&tfull_bar[buf]));
            }
        }
    } else {
        const int ew = warp & 3;   // this warp may touch TMEM lanes 32*ew .. 32*ew+31
        uint32_t local = 0;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, local++) {
            int mi, ni;
            tile_coords(t, tiles_m, tiles_n, &mi, &ni);
            const uint32_t buf = local & 1, use = local >> 1;
            ok &= mbar_wait(smem_u32(&tfull_bar[buf]), use & 1, &gave_up);
            ok = __all_sync(0xffffffffu, ok);   // the warp stays together: tcgen05.ld below is warp-collective
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            __half* crow = C + (size_t)(mi * BM + ew * 32 + lane) * N + (size_t)ni * BN2;
            const uint32_t src = tmem_base + buf * BN2 + ((uint32_t)(ew * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN2; c += 32) {
                uint32_t r[32];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
                      "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
                      "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
                      "=r"(r[31])
                    : "r"(src + (uint32_t)c));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                uint32_t h[16];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    __half2 v = __floats2half2_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                    h[i] = *reinterpret_cast<uint32_t*>(&v);
                }
#pragma unroll
                for (int q = 0; q < 4; q++) *reinterpret_cast<uint4*>(crow + c + 8 * q) = make_uint4(h[4 * q], h[4 * q + 1], h[4 * q + 2], h[4 * q + 3]);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&tempty_bar[buf])) : "memory");
        }
    }
    if (!ok && status) atomicExch(status, 1);
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS2) : "memory");
}
}  // namespace v2


// ---- v3: a pair of CTAs (a cluster of two SMs) per 256 x 256 tile, tcgen05.mma.cta_group::2 ----
//
// CTA r of the pair owns rows 128r..128r+127 of the tile: it loads that half of A and columns
// 128r..128r+127 of B (so each SM stages 32 KB per K slab instead of 48 KB for the same math),
// and its tensor memory receives its 128 rows of the accumulator.  The even CTA (the leader)
// issues every MMA; the instruction reads both CTAs' shared memory at the same offsets.
//   * both producers signal the LEADER's "full" barrier (the bulk-tensor load names it through its
//     shared::cluster address, no multicast); the leader's producer posts the expected byte count
//     of both halves;
//   * the MMA warp's commit arrives on the "empty" barrier of both CTAs (commit with a CTA mask),
//     and, after a tile's last slab, on both CTAs' "accumulator full" barriers;
//   * the epilogue warps of both CTAs arrive on the leader's "accumulator empty" barrier.
// Every wait is bounded as in the other kernels; the pair meets at a cluster barrier before tensor
// memory is released, so neither CTA leaves while the other may still name its barriers or memory.
namespace v3 {
constexpr int TM = 256, TN = 256, HALF_N = 128;   // a stage is 16 KB of A + 16 KB of B per CTA
// How the epilogue leaves the SM.
//   DIRECT  16-byte pieces straight from the registers tcgen05.ld filled (a lane holds one row);
//   LINES   each 32-row x 64-column piece is transposed through shared memory and stored by the warp as
//           whole 128-byte lines (and, in the fused gather, again into every peer's buffer);
//   BULK    the piece is written to shared memory in the 128-byte-swizzled layout and one lane hands it
//           to the copy engine of the SM as bulk-tensor stores (cp.async.bulk.tensor, shared -> global),
//           one per destination: the warp goes straight back to tensor memory while the stores drain.
//   RELAY   as LINES for this GPU's buffer; the copies for the peers are made by two further warps of the CTA that read each
//           finished tile back (from L2) and store it behind every peer: the epilogue warps never wait on NVLink, so
//           link back-pressure cannot hold an accumulator back from the MMA warp.
enum Epilogue { DIRECT = 0, LINES = 1, BULK = 2, RELAY = 3 };
constexpr int PIECE_BYTES = 32 * 128;   // 32 rows x 64 columns of f16
// ring depth of the K-slab stages and staging pieces per epilogue warp: everything fits 227 KB
__host__ __device__ constexpr int stages_of(int epi, bool deep, int tn = 256) { return tn == 128 ? 8 : epi == BULK && deep ? 5 : 6; }   // 24 KB stages when the tile is 128 wide
__host__ __device__ constexpr int pieces_of(int epi, bool deep) { return epi == DIRECT ? 0 : (epi == LINES || epi == RELAY) ? 1 : deep ? 4 : 2; }
__host__ __device__ constexpr int threads_of(int epi) { return epi == RELAY ? 256 : 192; }   // RELAY: warps 6 and 7 carry the tiles to the peers
constexpr int GROUP_M = 8;
constexpr uint32_t TMEM_COLS3 = 512;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same variable in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t cta_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// bulk-tensor load into this CTA's shared memory whose completion bytes go to a barrier that may
// live in the peer CTA (`bar_cluster` is a shared::cluster address)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(map), "r"(bar_cluster), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// arrives (once the MMAs issued so far have finished) on the barrier at this offset in both CTAs
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"((uint16_t)3)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int* m_idx, int* n_idx) {
    const int per_band = GROUP_M * tiles_n, band = t / per_band, first = band * GROUP_M;
    const int rows = min(GROUP_M, tiles_m - first), r = t - band * per_band;
    *m_idx = first + r % rows;
    *n_idx = r / rows;
}

// The same rows of the result in the other ranks' buffers (peer-mapped device memory), for the fused
// gather: the epilogue stores every 16-byte piece of a tile to this GPU's buffer and to each of these.
struct PeerRows {
    __half* c[BASALT_K_MAX_PEERS - 1];
    int n;
};
// BULK: tensor maps of the result rows, this GPU's first, then the same rows in each peer's buffer
// (box: 64 columns x 32 rows, 128-byte swizzle)
struct StoreMaps {
    CUtensorMap c[BASALT_K_MAX_PEERS];
    int n;
};

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}

// Over NVLink the difference between LINES and DIRECT is a line-sized against a 16-byte write per request,
// which is why the fused gather needs at least LINES; BULK also takes the copies off the warps.
// TILE_N = 256: the 256 x 256 tile.  TILE_N = 128: a 256 x 128 tile (each CTA stages 128 rows of A and 64 columns of B
// per K slab, 24 KB; MMA M256 N128 K16): half the work per tile, so a row shard of few tiles (the 8-GPU split) starts
// handing finished tiles to its epilogue -- and, in the fused gather, to NVLink -- after half the time.
template <bool B_IS_NK, int EPI, bool DEEP, int TILE_N>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(threads_of(EPI), 1)
    matmul_f16_tc_pair(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, __half* __restrict__ C, int M, int N, int K,
                       int32_t* status, const PeerRows peers, const __grid_constant__ StoreMaps out) {
    constexpr int TN = TILE_N, HALF_N = TILE_N / 2, STAGE_BYTES3 = A_BYTES + HALF_N * BK * 2;   // shadow the 256-wide constants of the namespace
    constexpr int STAGES = stages_of(EPI, DEEP, TILE_N), PIECES = pieces_of(EPI, DEEP);
    constexpr bool STAGED = EPI == LINES || EPI == RELAY;
    const bool PUSH = EPI != RELAY && peers.n > 0;      // RELAY: the epilogue warps store locally only
    __shared__ volatile uint32_t tiles_stored;          // RELAY: epilogue warps that have finished storing a tile (four per tile)
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], tfull_bar[2], tempty_bar[2];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile uint32_t gave_up;
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int tiles_m = M / TM, tiles_n = N / TN, num_tiles = tiles_m * tiles_n, num_kb = K / BK;

    if (threadIdx.x == 0) {
        gave_up = 0;
        tiles_stored = 0;
        for (int s = 0; s < STAGES; s++) {
            mbar_init(smem_u32(&full_bar[s]), 1);    // the leader's producer; bytes arrive from both CTAs
            mbar_init(smem_u32(&empty_bar[s]), 1);   // one commit from the leader's MMA warp
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(smem_u32(&tfull_bar[b]), 1);
            mbar_init(smem_u32(&tempty_bar[b]), 8);  // four epilogue warps in each CTA (used in the leader only)
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {   // the same warp of both CTAs allocates for the pair
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS3) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();   // the peer's barriers are initialised before anything can signal them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t s = 0, ph = 0;   // stage and its wrap parity, as running counters
            for (int t = pair; t < num_tiles && ok; t += pairs) {
                int mi, ni;
                tile_coords(t, tiles_m, tiles_n, &mi, &ni);
                const int m0 = mi * TM + (int)rank * BM, n0 = ni * TN + (int)rank * HALF_N;
                for (int kb = 0; kb < num_kb; kb++) {
                    ok &= mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, &gave_up);
                    if (!ok) break;
                    const uint32_t fb_local = smem_u32(&full_bar[s]), fb = map_to_cta(fb_local, 0);
                    const uint32_t a_dst = tiles + s * STAGE_BYTES3, b_dst = a_dst + A_BYTES;
                    if (leader) mbar_expect_tx(fb_local, 2 * STAGE_BYTES3);
                    tma_load_2d_pair(a_dst, &map_a, fb, kb * BK, m0);
                    if (B_IS_NK) tma_load_2d_pair(b_dst, &map_b, fb, kb * BK, n0);   // box 64 k x 128 n
                    else {
#pragma unroll
                        for (int h = 0; h < HALF_N / 64; h++) tma_load_2d_pair(b_dst + h * 8192, &map_b, fb, n0 + 64 * h, kb * BK);   // box 64 n x 64 k
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
            if (!ok) {   // let the copies already issued land before the CTA can exit
                const uint64_t t0 = global_ns();
                while (global_ns() - t0 < 2000000ull) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            const uint32_t idesc = (1u << 4) | ((B_IS_NK ? 0u : 1u) << 16) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);
            // This one thread has about 500 clocks per K slab: the stage index is a running counter and the
            // descriptors are built once per slab and stepped by constant adds (a 16-k step is 32 bytes along a
            // K-major row, 16 rows of 128 bytes in an MN-major slab; descriptors count 16-byte units).
            uint32_t s = 0, ph = 0, local = 0;
            for (int t = pair; t < num_tiles && ok; t += pairs, local++) {
                const uint32_t buf = local & 1, use = local >> 1;
                ok &= mbar_wait(smem_u32(&tempty_bar[buf]), (use & 1) ^ 1, &gave_up);   // both epilogues have drained this accumulator
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + buf * TN;
                for (int kb = 0; kb < num_kb; kb++) {
                    ok &= mbar_wait(smem_u32(&full_bar[s]), ph, &gave_up);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_src = tiles + s * STAGE_BYTES3, b_src = a_src + A_BYTES;
                    const uint64_t da = smem_desc(a_src, 16, 1024);
                    const uint64_t db = B_IS_NK ? smem_desc(b_src, 16, 1024) : smem_desc(b_src, 8192, 1024);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++)
                        umma_f16_pair(acc, da + (uint64_t)(2 * k), db + (uint64_t)((B_IS_NK ? 2 : 128) * k), idesc, (kb | k) != 0);
                    umma_commit_pair(smem_u32(&empty_bar[s]));
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                umma_commit_pair(smem_u32(&tfull_bar[buf]));
            }
        }
    } else if (warp >= 6) {
        // ---- RELAY: warps 6 and 7 carry every finished tile of this CTA (128 rows x TN columns) to the peers ----
        if constexpr (EPI == RELAY) {
            const int half = warp - 6;   // rows 64 half .. 64 half + 63 of the CTA's 128
            uint32_t local = 0;
            for (int t = pair; t < num_tiles && ok && peers.n > 0; t += pairs, local++) {
                int mi, ni;
                tile_coords(t, tiles_m, tiles_n, &mi, &ni);
                // bounded wait for the four epilogue warps to have stored this tile (their stores are fenced before they count)
                uint64_t t0 = 0;
                for (uint32_t i = 0; tiles_stored < 4 * (local + 1); i++) {
                    if (gave_up) { ok = false; break; }
                    if ((i & 63) == 63) {
                        const uint64_t now = global_ns();
                        if (t0 == 0) t0 = now;
                        else if (now - t0 > WAIT_LIMIT_NS) { gave_up = 1; ok = false; break; }
                    }
                }
                if (!ok) break;
                __threadfence();
                const size_t first = (size_t)(mi * TM + (int)rank * BM + half * 64) * N + (size_t)ni * TN + 8 * lane;   // this lane's 16 bytes of the first row
#pragma unroll 1
                for (int r = 0; r < 64; r += 4) {
                    uint4 v[4][TN / 256 ? TN / 256 : 1];
#pragma unroll
                    for (int i = 0; i < 4; i++)
#pragma unroll
                        for (int c = 0; c < TN / 256; c++) v[i][c] = __ldcg(reinterpret_cast<const uint4*>(C + first + (size_t)(r + i) * N + 256 * c));
                    for (int p = 0; p < peers.n; p++) {
#pragma unroll
                        for (int i = 0; i < 4; i++)
#pragma unroll
                            for (int c = 0; c < TN / 256; c++) *reinterpret_cast<uint4*>(peers.c[p] + first + (size_t)(r + i) * N + 256 * c) = v[i][c];
                    }
                }
            }
            if (peers.n > 0) __threadfence_system();
        }
    } else {
        const int ew = warp & 3;
        uint32_t local = 0, piece = 0;
        (void)piece;
        for (int t = pair; t < num_tiles && ok; t += pairs, local++) {
            int mi, ni;
            tile_coords(t, tiles_m, tiles_n, &mi, &ni);
            const uint32_t buf = local & 1, use = local >> 1;
            ok &= mbar_wait(smem_u32(&tfull_bar[buf]), use & 1, &gave_up);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const size_t tile_off = (size_t)(mi * TM + (int)rank * BM + ew * 32 + lane) * N + (size_t)ni * TN;
            __half* crow = C + tile_off;
            const uint32_t src = tmem_base + buf * TN + ((uint32_t)(ew * 32) << 16);
            if constexpr (EPI == BULK) {
                const uint32_t ring = tiles + STAGES * STAGE_BYTES3 + ew * (PIECES * PIECE_BYTES);   // 1 KB aligned: the swizzle is a function of the address
                const int y = mi * TM + (int)rank * BM + ew * 32;
#pragma unroll 1
                for (int c = 0; c < TN; c += 64, piece++) {
                    const uint32_t stg = ring + (piece % PIECES) * PIECE_BYTES;
                    // the stores that last read this piece of the ring have finished reading it
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(PIECES - 1) : "memory");
                    __syncwarp();
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        uint32_t r[32];
                        asm volatile(
                            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                              "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
                              "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
                              "=r"(r[30]), "=r"(r[31])
                            : "r"(src + (uint32_t)(c + 32 * half)));
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int q = 0; q < 4; q++) {   // 16-byte unit 4*half + q of row `lane`, where the 128-byte swizzle puts it
                            uint32_t h[4];
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                __half2 v = __floats2half2_rn(__uint_as_float(r[8 * q + 2 * i]), __uint_as_float(r[8 * q + 2 * i + 1]));
                                h[i] = *reinterpret_cast<uint32_t*>(&v);
                            }
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg + lane * 128 + (((4 * half + q) ^ (lane & 7)) << 4)), "r"(h[0]), "r"(h[1]),
                                         "r"(h[2]), "r"(h[3])
                                         : "memory");
                        }
                    }
                    if (c + 64 == TN) {   // the accumulator is drained: the MMA warp may overwrite it while the stores go out
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the copy engine reads what the warp wrote
                    __syncwarp();
                    if (lane == 0) {
                        if (c + 64 == TN) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[buf]), 0));
                        for (int d = 0; d < out.n; d++) tma_store_2d(&out.c[d], stg, ni * TN + c, y);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
                continue;
            }
            if (STAGED) {
                uint8_t* stg = smem_raw + (tiles - smem_u32(smem_raw)) + STAGES * STAGE_BYTES3 + ew * (32 * 128);
                const size_t warp_off = (size_t)(mi * TM + (int)rank * BM + ew * 32) * N + (size_t)ni * TN;   // the warp's first row
                const int rrow = lane >> 3, piece = lane & 7;   // reading back: eight lanes cover one 128-byte row
#pragma unroll 1
                for (int c = 0; c < TN; c += 64) {
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        uint32_t r[32];
                        asm volatile(
                            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                              "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
                              "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
                              "=r"(r[30]), "=r"(r[31])
                            : "r"(src + (uint32_t)(c + 32 * half)));
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int q = 0; q < 4; q++) {   // 16-byte piece 4*half + q of this lane's row, at a column rotated by the row: no bank conflicts
                            uint32_t h[4];
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                __half2 v = __floats2half2_rn(__uint_as_float(r[8 * q + 2 * i]), __uint_as_float(r[8 * q + 2 * i + 1]));
                                h[i] = *reinterpret_cast<uint32_t*>(&v);
                            }
                            *reinterpret_cast<uint4*>(stg + lane * 128 + (((4 * half + q) ^ (lane & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
                        }
                    }
                    __syncwarp();
                    uint4 v[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int row = 4 * i + rrow;
                        v[i] = *reinterpret_cast<const uint4*>(stg + row * 128 + ((piece ^ (row & 7)) << 4));
                    }
                    __syncwarp();   // the next piece may overwrite the staging rows
                    __half* dst = C + warp_off + c + 8 * piece;
#pragma unroll
                    for (int i = 0; i < 8; i++) *reinterpret_cast<uint4*>(dst + (size_t)(4 * i + rrow) * N) = v[i];
                    if (PUSH) {   // the same lines into every peer's buffer, over NVLink
                        for (int p = 0; p < peers.n; p++) {
                            __half* pdst = peers.c[p] + warp_off + c + 8 * piece;
#pragma unroll
                            for (int i = 0; i < 8; i++) *reinterpret_cast<uint4*>(pdst + (size_t)(4 * i + rrow) * N) = v[i];
                        }
                    }
                }
            } else {
#pragma unroll 1
            for (int c = 0; c < TN; c += 32) {
                uint32_t r[32];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
                      "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
                      "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
                      "=r"(r[31])
                    : "r"(src + (uint32_t)c));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                uint32_t h[16];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    __half2 v = __floats2half2_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                    h[i] = *reinterpret_cast<uint32_t*>(&v);
                }
#pragma unroll
                for (int q = 0; q < 4; q++) *reinterpret_cast<uint4*>(crow + c + 8 * q) = make_uint4(h[4 * q], h[4 * q + 1], h[4 * q + 2], h[4 * q + 3]);
                if (PUSH) {   // the same 64 bytes of this row into every peer's buffer, over NVLink
                    for (int p = 0; p < peers.n; p++) {
                        __half* prow = peers.c[p] + tile_off + c;
#pragma unroll
                        for (int q = 0; q < 4; q++) *reinterpret_cast<uint4*>(prow + 8 * q) = make_uint4(h[4 * q], h[4 * q + 1], h[4 * q + 2], h[4 * q + 3]);
                    }
                }
            }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[buf]), 0));
            if (EPI == RELAY && peers.n > 0) {   // after the accumulator is handed back: the fence is not on the MMA warp's path
                __threadfence();                  // this lane's stores of the tile are visible device-wide before the warp counts itself
                __syncwarp();
                if (lane == 0) atomicAdd(const_cast<uint32_t*>(&tiles_stored), 1u);
            }
        }
        if (EPI == BULK && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // every bulk store of this warp is complete
        if (PUSH) __threadfence_system();   // this thread's peer stores are performed before the kernel can end
    }
    if (!ok && status) atomicExch(status, 1);
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();   // the peer has stopped naming this CTA's barriers, shared and tensor memory
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS3) : "memory");
}
}  // namespace v3

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)p;
    }
    return fn;
}

// Row-major f16 matrix [rows x cols] -> tensor map with a (box_cols x box_rows) box, 128B swizzle.
int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols, uint32_t box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return basalt_k::record_msg(1, "matmul_f16", "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return basalt_k::record_msg((int)r, "matmul_f16", "cuTensorMapEncodeTiled failed");
    return 0;
}

template <int STAGES, bool B_IS_NK>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, __half* C, int M, int N, int K, int32_t* status, cudaStream_t s) {
    constexpr int smem = STAGES * STAGE_BYTES + 1024;
    auto kern = matmul_f16_tc_kernel<STAGES, B_IS_NK>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return basalt_k::record(e, "matmul_f16 (shared memory size)");
        configured = true;
    }
    dim3 grid(N / BN, M / BM);
    kern<<<grid, THREADS, smem, s>>>(ma, mb, C, N, K, status);
    return basalt_k::record(cudaGetLastError(), "matmul_f16");
}

template <bool B_IS_NK>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, __half* C, int M, int N, int K, int32_t* status, cudaStream_t s) {
    constexpr int smem = v2::STAGES * v2::STAGE_BYTES2 + 1024;
    auto kern = v2::matmul_f16_tc_persistent<B_IS_NK>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return basalt_k::record(e, "matmul_f16 (shared memory size)");
        configured = true;
    }
    const int tiles = (M / BM) * (N / v2::BN2), sms = basalt_k::sm_count();
    kern<<<tiles < sms ? tiles : sms, v2::THREADS2, smem, s>>>(ma, mb, C, M, N, K, status);
    return basalt_k::record(cudaGetLastError(), "matmul_f16");
}


template <bool B_IS_NK, int EPI, bool DEEP, int TILE_N = 256>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, __half* C, int M, int N, int K, int32_t* status, cudaStream_t s, const v3::PeerRows& peers,
                const v3::StoreMaps& out) {
    constexpr int smem = v3::stages_of(EPI, DEEP, TILE_N) * (A_BYTES + TILE_N / 2 * BK * 2) + 1024 + 4 * v3::pieces_of(EPI, DEEP) * v3::PIECE_BYTES;
    auto kern = v3::matmul_f16_tc_pair<B_IS_NK, EPI, DEEP, TILE_N>;
    static int max_pairs = 0;
    if (!max_pairs) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return basalt_k::record(e, "matmul_f16 (shared memory size)");
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * basalt_k::sm_count());
        cfg.blockDim = dim3(v3::threads_of(EPI));
        cfg.dynamicSmemBytes = smem;
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);   // the kernel's own __cluster_dims__ (2,1,1) applies
        if (e != cudaSuccess || n < 1) { (void)cudaGetLastError(); n = basalt_k::sm_count() / 2; }
        max_pairs = n;
    }
    const int tiles = (M / v3::TM) * (N / TILE_N);
    const int pairs = tiles < max_pairs ? tiles : max_pairs;
    kern<<<2 * pairs, v3::threads_of(EPI), smem, s>>>(ma, mb, C, M, N, K, status, peers, out);
    return basalt_k::record(cudaGetLastError(), "matmul_f16");
}

// Row-major f16 result rows -> tensor map for the BULK epilogue's stores (box 64 columns x 32 rows).
int make_store_maps(v3::StoreMaps* out, void* C, void* const* peer_c, int n_peers, int M, int N) {
    out->n = 1 + n_peers;
    int rc = make_map(&out->c[0], C, (uint64_t)M, (uint64_t)N, 64, 32);
    for (int i = 0; i < n_peers && !rc; i++) rc = make_map(&out->c[1 + i], peer_c[i], (uint64_t)M, (uint64_t)N, 64, 32);
    return rc;
}

template <bool B_IS_NK>
int launch_pair_variant(int variant, const CUtensorMap& ma, const CUtensorMap& mb, void* C, int M, int N, int K, int32_t* status, cudaStream_t s,
                        void* const* peer_c, int n_peers) {
    v3::PeerRows peers = {};
    peers.n = n_peers;
    for (int i = 0; i < n_peers; i++) peers.c[i] = (__half*)peer_c[i];
    if (variant == BASALT_K_MATMUL_PAIR_DIRECT) return launch_pair<B_IS_NK, v3::DIRECT, false>(ma, mb, (__half*)C, M, N, K, status, s, peers, v3::StoreMaps{});
    if (variant == BASALT_K_MATMUL_PAIR_LINES) return launch_pair<B_IS_NK, v3::LINES, false>(ma, mb, (__half*)C, M, N, K, status, s, peers, v3::StoreMaps{});
    if (variant == BASALT_K_MATMUL_PAIR_RELAY) return launch_pair<B_IS_NK, v3::RELAY, false>(ma, mb, (__half*)C, M, N, K, status, s, peers, v3::StoreMaps{});
    if (variant == BASALT_K_MATMUL_PAIR_LINES_NARROW) return launch_pair<B_IS_NK, v3::LINES, false, 128>(ma, mb, (__half*)C, M, N, K, status, s, peers, v3::StoreMaps{});
    v3::StoreMaps out = {};
    int rc = make_store_maps(&out, C, peer_c, n_peers, M, N);
    if (rc) return rc;
    peers.n = 0;   // the bulk stores carry the peers' copies
    if (variant == BASALT_K_MATMUL_PAIR_BULK) return launch_pair<B_IS_NK, v3::BULK, false>(ma, mb, (__half*)C, M, N, K, status, s, peers, out);
    return launch_pair<B_IS_NK, v3::BULK, true>(ma, mb, (__half*)C, M, N, K, status, s, peers, out);
}

int matmul_f16_any(const void* A, const void* B, void* C, int M, int N, int K, int b_is_nk, int variant, void* const* peer_c, int n_peers, int32_t* status,
                   void* stream, const char* who) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (M % BM || N % BN || K % BK) return basalt_k::record_msg(1, who, "M and N must be multiples of 128 and K of 64");
    if (n_peers < 0 || n_peers > BASALT_K_MAX_PEERS - 1 || (n_peers && !peer_c)) return basalt_k::record_msg(1, who, "bad peer list");
    uintptr_t all = (uintptr_t)A | (uintptr_t)B | (uintptr_t)C;
    for (int i = 0; i < n_peers; i++) all |= (uintptr_t)peer_c[i];
    if (all & 15) return basalt_k::record_msg(1, who, "matrices must be 16-byte aligned");
    const bool pair_shape = M % v3::TM == 0 && N % v3::TN == 0;
    if (variant == BASALT_K_MATMUL_AUTO) {
        if (n_peers) variant = BASALT_K_MATMUL_PAIR_RELAY;
        else if (pair_shape) variant = BASALT_K_MATMUL_PAIR_LINES;
        else variant = N % v2::BN2 == 0 ? BASALT_K_MATMUL_ONE_SM_256 : BASALT_K_MATMUL_ONE_CTA_128;
    }
    if (variant < BASALT_K_MATMUL_ONE_CTA_128 || variant > BASALT_K_MATMUL_PAIR_RELAY) return basalt_k::record_msg(1, who, "unknown variant");
    const bool is_pair = variant >= BASALT_K_MATMUL_PAIR_DIRECT;
    if (is_pair && !pair_shape) return basalt_k::record_msg(1, who, "the CTA-pair kernels need M and N to be multiples of 256");
    if (!is_pair && n_peers) return basalt_k::record_msg(1, who, "only the CTA-pair kernels store to peers");
    if (variant == BASALT_K_MATMUL_ONE_SM_256 && N % v2::BN2) return basalt_k::record_msg(1, who, "the 128x256 kernel needs N to be a multiple of 256");
    CUtensorMap ma, mb;
    int rc = make_map(&ma, A, (uint64_t)M, (uint64_t)K, BK, BM);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (is_pair) {   // 256 x 256 tiles on pairs of SMs
        rc = b_is_nk ? make_map(&mb, B, (uint64_t)N, (uint64_t)K, BK, variant == BASALT_K_MATMUL_PAIR_LINES_NARROW ? 64 : v3::HALF_N)
                     : make_map(&mb, B, (uint64_t)K, (uint64_t)N, 64, BK);
        if (rc) return rc;
        return b_is_nk ? launch_pair_variant<true>(variant, ma, mb, C, M, N, K, status, s, peer_c, n_peers)
                       : launch_pair_variant<false>(variant, ma, mb, C, M, N, K, status, s, peer_c, n_peers);
    }
    if (variant == BASALT_K_MATMUL_ONE_SM_256) {   // 128 x 256 tiles, persistent
        rc = b_is_nk ? make_map(&mb, B, (uint64_t)N, (uint64_t)K, BK, v2::BN2) : make_map(&mb, B, (uint64_t)K, (uint64_t)N, 64, BK);
        if (rc) return rc;
        return b_is_nk ? launch_persistent<true>(ma, mb, (__half*)C, M, N, K, status, s) : launch_persistent<false>(ma, mb, (__half*)C, M, N, K, status, s);
    }
    rc = b_is_nk ? make_map(&mb, B, (uint64_t)N, (uint64_t)K, BK, BN) : make_map(&mb, B, (uint64_t)K, (uint64_t)N, 64, BK);
    if (rc) return rc;
    return b_is_nk ? launch<3, true>(ma, mb, (__half*)C, M, N, K, status, s) : launch<3, false>(ma, mb, (__half*)C, M, N, K, status, s);
}

}  // namespace

extern "C" int basalt_k_matmul_f16(const void* A, const void* B, void* C, int M, int N, int K, int b_is_nk, int32_t* status, void* stream) {
    return matmul_f16_any(A, B, C, M, N, K, b_is_nk, BASALT_K_MATMUL_AUTO, nullptr, 0, status, stream, "matmul_f16");
}

// C = A * B for this rank's rows, every tile stored to this GPU's result buffer and to the same rows of
// each peer's buffer from the epilogue of the tcgen05 kernel: compute and gather in one kernel.
extern "C" int basalt_k_matmul_f16_allgather(const void* A, const void* B, void* C, int M, int N, int K, int b_is_nk, void* const* peer_c, int n_peers,
                                             int32_t* status, void* stream) {
    if (M % v3::TM || N % v3::TN) return basalt_k::record_msg(1, "matmul_f16_allgather", "M and N must be multiples of 256 and K of 64");
    return matmul_f16_any(A, B, C, M, N, K, b_is_nk, BASALT_K_MATMUL_AUTO, peer_c, n_peers, status, stream, "matmul_f16_allgather");
}

extern "C" int basalt_k_matmul_f16_variant(const void* A, const void* B, void* C, int M, int N, int K, int b_is_nk, int variant, void* const* peer_c,
                                           int n_peers, int32_t* status, void* stream) {
    return matmul_f16_any(A, B, C, M, N, K, b_is_nk, variant, peer_c, n_peers, status, stream, "matmul_f16_variant");
}
