// Seeded synthetic inputs generated on the device: the same counter-based generator as
// basalt_b200/workloads.py (SplitMix64 at seed + (i + 1) * golden), so that a benchmark input of
// 2^28 elements is made in a fraction of a millisecond instead of tens of seconds of host time and
// is, bit for bit, the array the host generator and the CPU oracle's generator produce for the same
// seed (the GPU tests compare them).  The reference has no generator: its inputs are the small
// closed-form arrays of its example drivers (examples/cpu_launch_*.c).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../../include/basalt_b200_kernels.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ uint64_t splitmix64(uint64_t seed, uint64_t i) {   // draw number i of the stream
    uint64_t z = seed + (i + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

template <int KIND>
__global__ void __launch_bounds__(256) fill_kernel(uint64_t seed, uint64_t start, int64_t n, void* out) {
    const int64_t T = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += T) {
        const uint64_t g = start + (uint64_t)i;
        if (KIND == BASALT_K_FILL_U32) {            // uniform over all 32-bit patterns
            ((uint32_t*)out)[i] = (uint32_t)(splitmix64(seed, g) >> 32);
        } else if (KIND == BASALT_K_FILL_I32_PM30) {   // int32 uniform in [-2^30, 2^30)
            ((int32_t*)out)[i] = (int32_t)((int64_t)(splitmix64(seed, g) >> 33) - (1ll << 30));
        } else if (KIND == BASALT_K_FILL_F32_PM1) {    // 24 random bits * 2^-23 - 1: exact in f32
            ((float*)out)[i] = __fsub_rn(__fmul_rn((float)(uint32_t)(splitmix64(seed, g) >> 40), 1.0f / 8388608.0f), 1.0f);
        } else {                                    // f16 ~ N(0,1) * 0.1: twelve 16-bit uniforms summed, centred, scaled
            uint64_t tot = 0;
#pragma unroll
            for (int d = 0; d < 3; d++) {
                const uint64_t z = splitmix64(seed, 3 * g + d);
                tot += (z & 0xFFFF) + ((z >> 16) & 0xFFFF) + ((z >> 32) & 0xFFFF) + (z >> 48);
            }
            const double zn = __dmul_rn((double)((int64_t)tot - 393210), 1.0 / 65536.0);
            ((__half*)out)[i] = __double2half(__dmul_rn(zn, 0.1));
        }
    }
}

template <int KIND>
int launch(uint64_t seed, uint64_t start, int64_t n, void* out, cudaStream_t s) {
    int64_t blocks = (n + 255) / 256;
    const int64_t cap = (int64_t)basalt_k::sm_count() * 32;
    if (blocks > cap) blocks = cap;
    fill_kernel<KIND><<<(int)blocks, 256, 0, s>>>(seed, start, n, out);
    return basalt_k::record(cudaGetLastError(), "fill");
}

}  // namespace

extern "C" int basalt_k_fill(int kind, uint64_t seed, uint64_t start, int64_t n, void* out, void* stream) {
    if (n <= 0) return 0;
    if (!out) return basalt_k::record_msg(1, "fill", "null output");
    cudaStream_t s = (cudaStream_t)stream;
    switch (kind) {
        case BASALT_K_FILL_U32: return launch<BASALT_K_FILL_U32>(seed, start, n, out, s);
        case BASALT_K_FILL_I32_PM30: return launch<BASALT_K_FILL_I32_PM30>(seed, start, n, out, s);
        case BASALT_K_FILL_F32_PM1: return launch<BASALT_K_FILL_F32_PM1>(seed, start, n, out, s);
        case BASALT_K_FILL_F16_NORMAL01: return launch<BASALT_K_FILL_F16_NORMAL01>(seed, start, n, out, s);
    }
    return basalt_k::record_msg(1, "fill", "unknown kind");
}
