/* Hand-written sm_100a CUDA kernels for the five benchmark workloads: the comparators that every
 * emitted kernel is measured against.  The reference ships no CUDA kernels at all (its .cu files
 * are compiler inputs, tests/kernels/ in the reference project); each entry below names the
 * reference example whose kernel signature and result it reproduces at benchmark scale.
 *
 * All pointers are device pointers; `stream` is a cudaStream_t / CUstream (NULL = default
 * stream).  Launches are asynchronous.  Return value: 0, or a cudaError_t / CUresult code
 * (basalt_k_last_error() gives the text).
 */
#ifndef BASALT_B200_KERNELS_H
#define BASALT_B200_KERNELS_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

const char *basalt_k_last_error(void);

/* c[i] = a[i] + b[i], wrapping int32, for i < n: the vector_add kernel of
 * examples/cpu_launch_vadd.c (there f32, N = 1024) at int32. */
int basalt_k_vadd_i32(const int32_t *a, const int32_t *b, int32_t *c, int64_t n, void *stream);

/* atomicMax(out, max_i x[i]) signed: out must hold the running maximum on entry (INT32_MIN for
 * a fresh reduction).  Named after examples/cpu_launch_max_i32.c, which in the reference is a
 * two-argument scalar max; the reduction is this benchmark's workload. */
int basalt_k_max_i32(const int32_t *x, int64_t n, int32_t *out, void *stream);

/* out[i] = step_0(in[i]) with step_j(x) = step_{j+1}(x*x + 2654435761*j mod 2^32), 32 levels:
 * tests/kernels/device_helper_chain.cu (there 3 levels) at depth 32. */
int basalt_k_helper_chain_u32(const uint32_t *in, uint32_t *out, int64_t n, void *stream);

/* The three streaming kernels above with the grid capped at `waves` resident waves of CTAs instead of
 * the defaults (64, 16 and 8), for A/B timing of the launch geometry: on this part several waves of
 * short CTAs stream faster than one wave of long ones.  Same results.  No counterpart in the reference. */
int basalt_k_vadd_i32_waves(const int32_t *a, const int32_t *b, int32_t *c, int64_t n, int waves, void *stream);
int basalt_k_max_i32_waves(const int32_t *x, int64_t n, int32_t *out, int waves, void *stream);
int basalt_k_helper_chain_u32_waves(const uint32_t *in, uint32_t *out, int64_t n, int waves, void *stream);

/* Measures the INT32 pipe: one wave of CTAs, each thread running `iters` x 32 independent
 * multiply-adds (mod 2^32). *imads receives the number of multiply-adds executed; `out` (at least
 * out_elems uint32) receives one word per thread so the work cannot be optimised away. The
 * roofline denominator for the helper-chain workload; no counterpart in the reference. */
int basalt_k_imad_peak(uint32_t *out, int64_t out_elems, int iters, int64_t *imads, void *stream);

/* C[MxN] = A[MxK] * B[KxN], row-major fp32, FFMA only (no TF32): the workload of
 * examples/cpu_launch_tiled_sgemm.c (there 32^3 with a C addend). M, N multiples of 128, K of 16.
 * A problem whose last wave of tiles is sparse (or which is smaller than one wave) has those tiles
 * worked off by stream units -- one per resident CTA, each an equal run of the tail tiles' K slabs,
 * summed per tile in a fixed order -- through a workspace that is allocated on first use and shared by all calls on a device: such calls must not overlap in
 * time on one device (issue them on one stream, or order the streams with events); calls on one
 * stream never overlap. */
int basalt_k_sgemm_f32(const float *A, const float *B, float *C, int M, int N, int K, void *stream);

/* basalt_k_sgemm_f32 with parts of its schedule switched off, for A/B timing: NO_TAIL_SPLIT runs every
 * tile whole (no stream units for a sparse last wave or for a problem smaller than one wave); CP_ASYNC
 * stages the A slab with 4-byte cp.async copies instead of through registers.  flags = 0 is
 * basalt_k_sgemm_f32.  No counterpart in the reference. */
enum { BASALT_K_SGEMM_NO_TAIL_SPLIT = 1, BASALT_K_SGEMM_CP_ASYNC = 2, BASALT_K_SGEMM_WARP_ROWS = 4 };
int basalt_k_sgemm_f32_variant(const float *A, const float *B, float *C, int M, int N, int K, int flags, void *stream);

/* basalt_k_sgemm_f32 with the workspace of its tail wave in a static device array instead
 * of device memory allocated on first use: this entry point allocates nothing (no cudaMalloc,
 * cudaFree or allocating library call).  Same arguments and results.  The array holds 304 partial
 * 128x128 f32 tiles (19 MiB: two per stream unit of the tail wave, so at most 152 units where
 * basalt_k_sgemm_f32 uses one per resident CTA) and 256 tickets; when the two entry points cut a
 * tail wave differently, its sums are added in another order.  The first
 * call on each device looks the array's address up (cudaGetSymbolAddress) with that device current;
 * make that first call before any stream capture.  All calls on a device share the one array:
 * calls that overlap in time (different streams) race; calls on one stream do not.  Every call
 * zeroes the tickets it will use on `stream` before the kernel, and the kernel leaves them at zero.
 * No counterpart in the reference. */
int basalt_k_sgemm_f32_static_workspace(const float *A, const float *B, float *C, int M, int N, int K,
                                        void *stream);

/* C[MxN] (fp16) = A[MxK] (fp16) * B (fp16) with fp32 accumulation on tcgen05 tensor cores, TMA
 * loads, TMEM accumulator: the workload of examples/cpu_launch_triton_matmul.c (there f32 4x5x3).
 * b_is_nk = 0: B is [K x N] row-major; 1: B is stored transposed, [N x K] row-major.
 * M, N multiples of 128, K of 64.  `status` (device int32, may be NULL) receives a non-zero code
 * if a bounded wait inside the kernel expired. */
int basalt_k_matmul_f16(const void *A, const void *B, void *C, int M, int N, int K, int b_is_nk,
                        int32_t *status, void *stream);

/* The exchange step of the sharded max_i32 (one process per GPU): allreduce(max) of one int32 over
 * inboxes in peer-mapped device memory, in place of ncclAllReduce(count 1, ncclInt32, ncclMax).
 * inboxes[r] is the device address, valid on this GPU, of rank r's inbox: 2 x BASALT_K_MAX_PEERS
 * uint64 words, zeroed before the first call (inboxes[rank] is this rank's own).  `epoch` counts
 * the calls from 1 and must be the same on every rank; all ranks must make the same calls in the
 * same order.  *partial is this rank's value, *result receives the maximum over all ranks; both
 * are device pointers and the call is ordered on `stream`.  A peer that has not answered after
 * timeout_ns sets bit r of *status (device uint32) and is left out of the result; its word, should it
 * arrive later, matches no later epoch either (a word is accepted only when it carries exactly the
 * epoch being waited for), so after a non-zero status the group's inboxes must be zeroed and the
 * epochs restarted on every rank (basalt_rt_peer_group_destroy / _create).  With `reset`
 * non-zero, *partial is set to reset_value once it has been read, ready for the next accumulation
 * (the reduction kernel folds into it with atomicMax).  No counterpart in the reference, which has
 * no multi-GPU path. */
#define BASALT_K_MAX_PEERS 8
int basalt_k_peer_allreduce_max_i32(const uint64_t *inboxes, int nranks, int rank, uint32_t epoch,
                                    int32_t *partial, int32_t *result, uint32_t *status,
                                    uint64_t timeout_ns, int reset, int32_t reset_value, void *stream);

/* The sharded max_i32 step as ONE kernel: the reduction of this rank's shard x[0..n) (as
 * basalt_k_max_i32) and, in the CTA that finishes last, the exchange of basalt_k_peer_allreduce_max_i32.
 * *partial must hold INT32_MIN and *ticket 0 before the first call; the kernel leaves them so.
 * *result receives the maximum over all ranks' shards.  x must be 16-byte aligned.  The other
 * arguments are those of basalt_k_peer_allreduce_max_i32.  No counterpart in the reference. */
int basalt_k_max_i32_allreduce(const int32_t *x, int64_t n, int32_t *partial, const uint64_t *inboxes, int nranks,
                               int rank, uint32_t epoch, int32_t *result, uint32_t *status, uint32_t *ticket,
                               uint64_t timeout_ns, void *stream);

/* The row-sharded fp16 matmul with its gather fused in: C = A * B for this rank's M rows as
 * basalt_k_matmul_f16 (CTA pairs, tcgen05.mma.cta_group::2), and every tile is stored both to C and
 * to the same position behind each of the n_peers pointers in peer_c (host array; each entry the
 * address, in this process, of the same rows of another rank's result buffer, mapped with
 * basalt_rt_ipc_open): the epilogue warps store to C, two further warps of each CTA read the finished
 * tile back from L2 and store it to the peers over NVLink while the next tiles are computed.  Each
 * storing thread ends with a system-scope fence, so a
 * stream-ordered basalt_k_peer_allreduce_max_i32 after this kernel is the barrier after which every
 * rank holds the whole result.  The peers are served in the order given: pass rank + 1, rank + 2, ...
 * (mod the group size) so that at no moment two ranks store into the same receiver.  M, N multiples of
 * 256, K of 64, n_peers <= BASALT_K_MAX_PEERS - 1.
 * No counterpart in the reference, which has no multi-GPU path. */
int basalt_k_matmul_f16_allgather(const void *A, const void *B, void *C, int M, int N, int K, int b_is_nk,
                                  void *const *peer_c, int n_peers, int32_t *status, void *stream);

/* The same product through one named kernel form, for tests and A/B timing (basalt_k_matmul_f16 and
 * basalt_k_matmul_f16_allgather choose for themselves: the CTA-pair kernel with line-sized stores
 * when M and N are multiples of 256 and nothing is gathered, the relay form for the gather).
 * ONE_CTA_128: one 128x128 tile per CTA of 128 threads.  ONE_SM_256: persistent, 128x256 tiles, one
 * SM each.  PAIR_*: 256x256 tiles on clusters of two SMs (tcgen05.mma.cta_group::2), differing in
 * how the epilogue leaves the SM: DIRECT = 16-byte pieces straight from the registers; LINES = each
 * 32-row x 64-column piece transposed through shared memory and stored as whole 128-byte lines;
 * BULK = the piece handed to the SM's copy engine as one bulk-tensor store per destination
 * (cp.async.bulk.tensor shared -> global; six K-slab stages and two staging pieces per warp);
 * BULK_DEEP = the same with five stages and four staging pieces per warp.  peer_c / n_peers as in
 * basalt_k_matmul_f16_allgather (PAIR_* only; NULL / 0 for a local product).  No counterpart in the
 * reference. */
enum {
    BASALT_K_MATMUL_AUTO = 0,
    BASALT_K_MATMUL_ONE_CTA_128 = 1,
    BASALT_K_MATMUL_ONE_SM_256 = 2,
    BASALT_K_MATMUL_PAIR_DIRECT = 3,
    BASALT_K_MATMUL_PAIR_LINES = 4,
    BASALT_K_MATMUL_PAIR_BULK = 5,
    BASALT_K_MATMUL_PAIR_BULK_DEEP = 6,
    BASALT_K_MATMUL_PAIR_LINES_NARROW = 7,  /* PAIR_LINES on 256x128 tiles (MMA M256 N128 K16, eight 24 KB stages) */
    BASALT_K_MATMUL_PAIR_RELAY = 8          /* PAIR_LINES for this GPU's buffer; two further warps per CTA read each finished tile back
                                               from L2 and store it behind every peer, so the epilogue never waits on NVLink */
};
int basalt_k_matmul_f16_variant(const void *A, const void *B, void *C, int M, int N, int K, int b_is_nk, int variant,
                                void *const *peer_c, int n_peers, int32_t *status, void *stream);

/* Seeded synthetic inputs of the benchmark workloads, generated on the device: element i of the
 * output is draw `start + i` of the SplitMix64 counter stream of `seed`, mapped as the host
 * generator (basalt_b200/workloads.py) and the CPU oracle map it -- the three produce identical
 * bytes.  U32: all 32-bit patterns (the max_i32 and helper-chain inputs).  I32_PM30: int32 uniform
 * in [-2^30, 2^30) (vadd_i32).  F32_PM1: f32 uniform in [-1, 1) (SGEMM).  F16_NORMAL01: binary16
 * N(0,1) * 0.1 as a twelve-term Irwin-Hall sum (fp16 matmul; three draws per element).  No
 * counterpart in the reference, whose inputs are the closed-form arrays of examples/cpu_launch_*.c. */
enum { BASALT_K_FILL_U32 = 0, BASALT_K_FILL_I32_PM30 = 1, BASALT_K_FILL_F32_PM1 = 2, BASALT_K_FILL_F16_NORMAL01 = 3 };
int basalt_k_fill(int kind, uint64_t seed, uint64_t start, int64_t n, void *out, void *stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* BASALT_B200_KERNELS_H */
