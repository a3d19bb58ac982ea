// Hand-written sm_100a kernels for the three streaming / integer workloads.
//
// All three are HBM-bound (or balanced against the INT32 pipe): one 16-byte access per thread per
// array per step, several steps in flight per thread, grids sized as a multiple of the SM count so
// every SM holds the same number of resident CTAs.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../../include/basalt_b200_kernels.h"
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

// c = a + b over n4 int4 vectors, grid-stride, two vectors per array in flight per thread.
__global__ void __launch_bounds__(kThreads, 6) vadd_i32_kernel(const int4* __restrict__ a, const int4* __restrict__ b, int4* __restrict__ c,
                                                            int64_t n4, const int32_t* as, const int32_t* bs, int32_t* cs, int64_t n) {
    const int64_t T = (int64_t)gridDim.x * blockDim.x, g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t j = g;
#pragma unroll 1
    for (; j + T < n4; j += 2 * T) {
        int4 a0 = a[j], b0 = b[j], a1 = a[j + T], b1 = b[j + T];
        c[j] = make_int4(a0.x + b0.x, a0.y + b0.y, a0.z + b0.z, a0.w + b0.w);
        c[j + T] = make_int4(a1.x + b1.x, a1.y + b1.y, a1.z + b1.z, a1.w + b1.w);
    }
    if (j < n4) {
        int4 a0 = a[j], b0 = b[j];
        c[j] = make_int4(a0.x + b0.x, a0.y + b0.y, a0.z + b0.z, a0.w + b0.w);
    }
    const int64_t tail = n4 * 4 + g;   // fewer than four elements remain
    if (tail < n) cs[tail] = as[tail] + bs[tail];
}
// Fallback for pointers that are not 16-byte aligned.
__global__ void __launch_bounds__(kThreads) vadd_i32_scalar_kernel(const int32_t* a, const int32_t* b, int32_t* c, int64_t n) {
    const int64_t T = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += T) c[i] = a[i] + b[i];
}

__device__ __forceinline__ int max4(int4 v) { return max(max(v.x, v.y), max(v.z, v.w)); }

// Block max of the calling threads' values: redux.sync inside each warp, one shared-memory hop
// across the warps, result valid in thread 0.
__device__ __forceinline__ int block_max(int v) {
    __shared__ int warp_max[kThreads / 32];
    v = __reduce_max_sync(0xffffffffu, v);
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        int w = threadIdx.x < kThreads / 32 ? warp_max[threadIdx.x] : INT32_MIN;
        v = __reduce_max_sync(0xffffffffu, w);
    }
    return v;
}

// Signed max of x[0..n): four 16-byte loads in flight per thread, one red.global.max per CTA.
__global__ void __launch_bounds__(kThreads, 8) max_i32_kernel(const int4* __restrict__ x4, int64_t n4, const int32_t* __restrict__ xs, int64_t n, int32_t* out) {
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
    m = block_max(m);
    if (threadIdx.x == 0) atomicMax(out, m);
}
__global__ void __launch_bounds__(kThreads) max_i32_scalar_kernel(const int32_t* x, int64_t n, int32_t* out) {
    const int64_t T = (int64_t)gridDim.x * blockDim.x;
    int m = INT32_MIN;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += T) m = max(m, x[i]);
    m = block_max(m);
    if (threadIdx.x == 0) atomicMax(out, m);
}

// The 32-level helper chain, one level per call; the compiler inlines the chain into 32 IMADs.
template <int J>
__device__ __forceinline__ uint32_t chain_step(uint32_t x) {
    const uint32_t y = x * x + 2654435761u * (uint32_t)J;
    if constexpr (J == 31) return y;
    else return chain_step<J + 1>(y);
}
__global__ void __launch_bounds__(kThreads, 8) helper_chain_kernel(const uint4* __restrict__ in4, uint4* __restrict__ out4, int64_t n4,
                                                                const uint32_t* ins, uint32_t* outs, int64_t n) {
    const int64_t T = (int64_t)gridDim.x * blockDim.x, g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t j = g;
#pragma unroll 1
    for (; j + T < n4; j += 2 * T) {
        uint4 v0 = in4[j], v1 = in4[j + T];
        out4[j] = make_uint4(chain_step<0>(v0.x), chain_step<0>(v0.y), chain_step<0>(v0.z), chain_step<0>(v0.w));
        out4[j + T] = make_uint4(chain_step<0>(v1.x), chain_step<0>(v1.y), chain_step<0>(v1.z), chain_step<0>(v1.w));
    }
    if (j < n4) {
        uint4 v = in4[j];
        out4[j] = make_uint4(chain_step<0>(v.x), chain_step<0>(v.y), chain_step<0>(v.z), chain_step<0>(v.w));
    }
    const int64_t tail = n4 * 4 + g;
    if (tail < n) outs[tail] = chain_step<0>(ins[tail]);
}
__global__ void __launch_bounds__(kThreads) helper_chain_scalar_kernel(const uint32_t* in, uint32_t* out, int64_t n) {
    const int64_t T = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += T) out[i] = chain_step<0>(in[i]);
}

// INT32 pipe peak: eight independent multiply-add chains per thread, nothing else in the loop.
__global__ void __launch_bounds__(kThreads) imad_peak_kernel(uint32_t* out, int iters) {
    uint32_t x[8];
    const uint32_t m = 2654435761u + threadIdx.x, a = blockIdx.x * 977u + 12345u;
#pragma unroll
    for (int k = 0; k < 8; k++) x[k] = threadIdx.x * 31u + k;
    for (int i = 0; i < iters; i++) {
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int k = 0; k < 8; k++) x[k] = x[k] * m + a;
    }
    uint32_t s = 0;
#pragma unroll
    for (int k = 0; k < 8; k++) s ^= x[k];
    out[(size_t)blockIdx.x * blockDim.x + threadIdx.x] = s;
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

// CTAs: enough to cover `work` thread-steps, at most one full wave of resident CTAs (SM count x
// the kernel's occupancy) times `waves`.  One wave of long-running CTAs is not the fastest way to stream on this part:
// with several waves of shorter CTAs the hardware scheduler evens out what the SMs and memory channels get (vadd_i32 at
// 2^28: 6.16 TB/s on one wave, 7.09 on up to 64; max_i32: 6.99 on one, 7.27 on 16, 5.05 on 64, where the CTAs' atomics pile up).
template <class K>
int grid_for(K kernel, int64_t work, int waves = 1) {
    const int64_t cap = (int64_t)basalt_k::sm_count() * basalt_k::resident_ctas(kernel, kThreads) * waves;
    int64_t need = (work + kThreads - 1) / kThreads;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

}  // namespace

extern "C" {

int basalt_k_vadd_i32(const int32_t* a, const int32_t* b, int32_t* c, int64_t n, void* stream) { return basalt_k_vadd_i32_waves(a, b, c, n, 64, stream); }
int basalt_k_max_i32(const int32_t* x, int64_t n, int32_t* out, void* stream) { return basalt_k_max_i32_waves(x, n, out, 16, stream); }
int basalt_k_helper_chain_u32(const uint32_t* in, uint32_t* out, int64_t n, void* stream) { return basalt_k_helper_chain_u32_waves(in, out, n, 8, stream); }

int basalt_k_vadd_i32_waves(const int32_t* a, const int32_t* b, int32_t* c, int64_t n, int waves, void* stream) {
    if (n <= 0) return 0;
    if (waves < 1) waves = 1;
    cudaStream_t s = (cudaStream_t)stream;
    if (aligned16(a) && aligned16(b) && aligned16(c)) {
        const int64_t n4 = n / 4;
        vadd_i32_kernel<<<grid_for(vadd_i32_kernel, (n4 + 1) / 2 + 4, waves), kThreads, 0, s>>>((const int4*)a, (const int4*)b, (int4*)c, n4, a, b, c, n);
    } else vadd_i32_scalar_kernel<<<grid_for(vadd_i32_scalar_kernel, n), kThreads, 0, s>>>(a, b, c, n);
    return basalt_k::record(cudaGetLastError(), "vadd_i32");
}

int basalt_k_max_i32_waves(const int32_t* x, int64_t n, int32_t* out, int waves, void* stream) {
    if (n <= 0) return 0;
    if (waves < 1) waves = 1;
    cudaStream_t s = (cudaStream_t)stream;
    if (aligned16(x)) {
        const int64_t n4 = n / 4;
        max_i32_kernel<<<grid_for(max_i32_kernel, (n4 + 3) / 4 + 4, waves), kThreads, 0, s>>>((const int4*)x, n4, x, n, out);
    } else max_i32_scalar_kernel<<<grid_for(max_i32_scalar_kernel, n), kThreads, 0, s>>>(x, n, out);
    return basalt_k::record(cudaGetLastError(), "max_i32");
}

int basalt_k_helper_chain_u32_waves(const uint32_t* in, uint32_t* out, int64_t n, int waves, void* stream) {
    if (n <= 0) return 0;
    if (waves < 1) waves = 1;
    cudaStream_t s = (cudaStream_t)stream;
    if (aligned16(in) && aligned16(out)) {
        const int64_t n4 = n / 4;
        helper_chain_kernel<<<grid_for(helper_chain_kernel, (n4 + 1) / 2 + 4, waves), kThreads, 0, s>>>((const uint4*)in, (uint4*)out, n4, in, out, n);
    } else helper_chain_scalar_kernel<<<grid_for(helper_chain_scalar_kernel, n), kThreads, 0, s>>>(in, out, n);
    return basalt_k::record(cudaGetLastError(), "helper_chain_u32");
}

int basalt_k_imad_peak(uint32_t* out, int64_t out_elems, int iters, int64_t* imads, void* stream) {
    int grid = basalt_k::sm_count() * basalt_k::resident_ctas(imad_peak_kernel, kThreads);
    if ((int64_t)grid * kThreads > out_elems) grid = (int)(out_elems / kThreads);
    if (grid < 1 || iters < 1) return basalt_k::record_msg(1, "imad_peak", "output buffer too small");
    imad_peak_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(out, iters);
    if (imads) *imads = (int64_t)grid * kThreads * iters * 32;
    return basalt_k::record(cudaGetLastError(), "imad_peak");
}

}  // extern "C"
