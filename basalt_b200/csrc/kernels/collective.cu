// One-shot allreduce(max) of one int32 over peer-mapped memory (NVLink/NVSwitch), for the sharded
// max_i32 reduction: the exchange step that follows each rank's partial maximum.
//
// Every rank owns an inbox of 2 x 8 64-bit words, mapped into every other rank's address space.
// A call with epoch e writes (e << 32 | partial) into word [e & 1][my rank] of every peer's inbox
// with a system-scope release store, then reads word [e & 1][r] of its own inbox for every peer r
// with system-scope acquire loads until its upper half equals e.  Two parities are enough: a rank
// can write epoch e + 2 only after it has finished epoch e + 1, which needed every peer's e + 1 word,
// which a peer sends only after its epoch-e call has returned.  Epochs start at 1 (the inbox starts
// zeroed).  One warp does all of it; the latency is two NVLink hops instead of a library collective.
//
// Every wait is bounded by the global timer; a lane that gives up sets its bit in *status and the
// result is the maximum over the ranks that did answer.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../../include/basalt_b200_kernels.h"
#include "common.cuh"

namespace {

struct PeerTable {
    unsigned long long* inbox[BASALT_K_MAX_PEERS];
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// The exchange itself, run by one full warp: lane r talks to rank r.  Returns the maximum over the
// ranks that answered (every lane gets it).
__device__ __forceinline__ int exchange_max(const PeerTable& peers, int nranks, int rank, unsigned epoch, int mine, unsigned* status,
                                            unsigned long long timeout_ns) {
    const int lane = threadIdx.x & 31;
    const unsigned parity = epoch & 1u;
    int v = INT32_MIN;
    if (lane < nranks) {
        v = mine;
        if (lane != rank) {
            const unsigned long long word = ((unsigned long long)epoch << 32) | (unsigned)mine;
            unsigned long long* dst = peers.inbox[lane] + parity * BASALT_K_MAX_PEERS + rank;
            asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(word) : "memory");
            const unsigned long long* src = peers.inbox[rank] + parity * BASALT_K_MAX_PEERS + lane;
            const unsigned long long t0 = global_ns();
            unsigned long long got = 0;
            bool ok = false;
            for (;;) {
                asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(got) : "l"(src) : "memory");
                if ((unsigned)(got >> 32) == epoch) { ok = true; break; }
                if (global_ns() - t0 > timeout_ns) break;
            }
            if (ok) v = (int)(unsigned)got;
            else { v = INT32_MIN; atomicOr(status, 1u << lane); }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__global__ void __launch_bounds__(32, 1) peer_allreduce_max_i32_kernel(PeerTable peers, int nranks, int rank, unsigned epoch, int* partial,
                                                                       int* __restrict__ result, unsigned* status, unsigned long long timeout_ns, int reset, int reset_value) {
    // Launched with programmatic stream serialisation: this grid may be set up while the kernel before it
    // on the stream (the reduction that produces *partial) is still draining, which hides its launch latency;
    // nothing of that kernel's output is read before this wait, which returns once it has completed and its
    // writes are visible.
    // The kernel after this one on the stream (the next step's reduction, launched the same way) may be set up while
    // this warp waits for its peers; it touches memory only after this grid has completed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int v = exchange_max(peers, nranks, rank, epoch, *reinterpret_cast<volatile int*>(partial), status, timeout_ns);
    if (threadIdx.x == 0) {
        *result = v;
        if (reset) *partial = reset_value;   // every lane has read it: ready for the next accumulation
    }
}

// ---- the reduction and its exchange in one kernel -------------------------------------------------
// The max_i32 reduction of this rank's shard (four 16-byte loads in flight per thread, one atomicMax
// per CTA into *partial) followed, in the CTA that finishes last (a ticket counter), by the exchange
// above: the last CTA's first warp reads the rank's maximum, trades it with the peers, writes the
// result and puts *partial and the ticket back to their starting values.  One launch per step
// instead of reset + reduction + exchange.
constexpr int kFusedThreads = 256;

__device__ __forceinline__ int max4(int4 v) { return max(max(v.x, v.y), max(v.z, v.w)); }

__global__ void __launch_bounds__(kFusedThreads, 8) max_i32_allreduce_kernel(const int4* __restrict__ x4, int64_t n4, const int32_t* __restrict__ xs, int64_t n,
                                                                             int* partial, PeerTable peers, int nranks, int rank, unsigned epoch,
                                                                             int* __restrict__ result, unsigned* status, unsigned* ticket,
                                                                             unsigned long long timeout_ns) {
    __shared__ int warp_best[kFusedThreads / 32];
    __shared__ unsigned last_s;
    const int64_t T = (int64_t)gridDim.x * blockDim.x, g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int m = INT32_MIN;
    int64_t j = g;
#pragma unroll 1
    for (; j + 3 * T < n4; j += 4 * T) {
        int4 v0 = x4[j], v1 = x4[j + T], v2 = x4[j + 2 * T], v3 = x4[j + 3 * T];
        m = max(m, max(max(max4(v0), max4(v1)), max(max4(v2), max4(v3))));
    }
    for (; j < n4; j += T) m = max(m, max4(x4[j]));
    for (int64_t i = n4 * 4 + g; i < n; i += T) m = max(m, xs[i]);
    m = __reduce_max_sync(0xffffffffu, m);
    if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        int b = warp_best[0];
#pragma unroll
        for (int w = 1; w < kFusedThreads / 32; w++) b = max(b, warp_best[w]);
        atomicMax(partial, b);
        __threadfence();
        last_s = atomicAdd(ticket, 1u) == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (!last_s || threadIdx.x >= 32) return;
    __threadfence();   // every CTA's atomicMax precedes its ticket; this CTA took the last ticket
    const int mine = *reinterpret_cast<volatile int*>(partial);
    const int v = exchange_max(peers, nranks, rank, epoch, mine, status, timeout_ns);
    if (threadIdx.x == 0) {
        *result = v;
        *reinterpret_cast<volatile int*>(partial) = INT32_MIN;
        *reinterpret_cast<volatile unsigned*>(ticket) = 0;
    }
}

}  // namespace

extern "C" int basalt_k_peer_allreduce_max_i32(const uint64_t* inboxes, int nranks, int rank, uint32_t epoch, int32_t* partial, int32_t* result,
                                               uint32_t* status, uint64_t timeout_ns, int reset, int32_t reset_value, void* stream) {
    if (!inboxes || !partial || !result || !status) return basalt_k::record_msg(1, "peer_allreduce_max_i32", "null argument");
    if (nranks < 1 || nranks > BASALT_K_MAX_PEERS || rank < 0 || rank >= nranks) return basalt_k::record_msg(1, "peer_allreduce_max_i32", "rank or world size out of range");
    if (epoch == 0) return basalt_k::record_msg(1, "peer_allreduce_max_i32", "epochs start at 1");
    PeerTable t{};
    for (int r = 0; r < nranks; r++) {
        if (!inboxes[r] || (inboxes[r] & 7)) return basalt_k::record_msg(1, "peer_allreduce_max_i32", "an inbox pointer is null or misaligned");
        t.inbox[r] = (unsigned long long*)(uintptr_t)inboxes[r];
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    unsigned long long timeout = timeout_ns;
    cudaError_t e = cudaLaunchKernelEx(&cfg, peer_allreduce_max_i32_kernel, t, nranks, rank, (unsigned)epoch, (int*)partial, (int*)result, (unsigned*)status, timeout, reset,
                                       (int)reset_value);
    return basalt_k::record(e != cudaSuccess ? e : cudaGetLastError(), "peer_allreduce_max_i32");
}

extern "C" int basalt_k_max_i32_allreduce(const int32_t* x, int64_t n, int32_t* partial, const uint64_t* inboxes, int nranks, int rank, uint32_t epoch,
                                          int32_t* result, uint32_t* status, uint32_t* ticket, uint64_t timeout_ns, void* stream) {
    if (!x || !partial || !inboxes || !result || !status || !ticket) return basalt_k::record_msg(1, "max_i32_allreduce", "null argument");
    if (n < 0 || nranks < 1 || nranks > BASALT_K_MAX_PEERS || rank < 0 || rank >= nranks) return basalt_k::record_msg(1, "max_i32_allreduce", "size, rank or world size out of range");
    if (epoch == 0) return basalt_k::record_msg(1, "max_i32_allreduce", "epochs start at 1");
    if ((uintptr_t)x & 15) return basalt_k::record_msg(1, "max_i32_allreduce", "the shard must be 16-byte aligned");
    PeerTable t{};
    for (int r = 0; r < nranks; r++) {
        if (!inboxes[r] || (inboxes[r] & 7)) return basalt_k::record_msg(1, "max_i32_allreduce", "an inbox pointer is null or misaligned");
        t.inbox[r] = (unsigned long long*)(uintptr_t)inboxes[r];
    }
    static int resident = 0;
    if (!resident) resident = basalt_k::resident_ctas(max_i32_allreduce_kernel, kFusedThreads);
    const int64_t n4 = n / 4, want = ((n4 + 3) / 4 + 4 + kFusedThreads - 1) / kFusedThreads;
    int64_t grid = (int64_t)resident * basalt_k::sm_count();   // one wave: every CTA ends with a fence and a ticket, and 16 waves of them measured slower (0.184 against 0.169 ms)
    if (want < grid) grid = want;
    if (grid < 1) grid = 1;
    max_i32_allreduce_kernel<<<(int)grid, kFusedThreads, 0, (cudaStream_t)stream>>>((const int4*)x, n4, x, n, partial, t, nranks, rank, epoch, result, status, ticket, timeout_ns);
    return basalt_k::record(cudaGetLastError(), "max_i32_allreduce");
}
