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

__global__ void __launch_bounds__(32, 1) peer_allreduce_max_i32_kernel(PeerTable peers, int nranks, int rank, unsigned epoch, int* partial,
                                                                       int* __restrict__ result, unsigned* status, unsigned long long timeout_ns, int reset, int reset_value) {
    const int lane = threadIdx.x;
    const unsigned parity = epoch & 1u;
    int v = INT32_MIN;
    if (lane < nranks) {
        const int mine = *partial;
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
    if (lane == 0) {
        *result = v;
        if (reset) *partial = reset_value;   // every lane has read it: ready for the next accumulation
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
    peer_allreduce_max_i32_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(t, nranks, rank, epoch, partial, result, status, timeout_ns, reset, reset_value);
    return basalt_k::record(cudaGetLastError(), "peer_allreduce_max_i32");
}
