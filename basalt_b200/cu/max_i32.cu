// Signed maximum of x[0..n), folded into *out (which the caller initialises, normally to INT_MIN).
//
// Each thread walks the array with a grid stride and keeps a running maximum; a warp combines its
// 32 partial results with an xor butterfly, lane 0 of every warp parks the warp's value in shared
// memory, the first warp combines those, and thread 0 issues the block's single atomicMax.
__global__ void __launch_bounds__(256, 8) max_i32(const int *x, int *out, int n) {
    __shared__ int warp_best[32];
    int tid = threadIdx.x;
    int stride = gridDim.x * blockDim.x;
    int lowest = -2147483647 - 1;
    int best = lowest;
    for (int i = blockIdx.x * blockDim.x + tid; i < n; i += stride) {
        best = max(x[i], best);
    }
    best = max(__shfl_xor_sync(0xffffffffu, best, 16), best);
    best = max(__shfl_xor_sync(0xffffffffu, best, 8), best);
    best = max(__shfl_xor_sync(0xffffffffu, best, 4), best);
    best = max(__shfl_xor_sync(0xffffffffu, best, 2), best);
    best = max(__shfl_xor_sync(0xffffffffu, best, 1), best);
    int lane = tid & 31;
    int warp = tid >> 5;
    if (lane == 0) {
        warp_best[warp] = best;
    }
    __syncthreads();
    if (tid < 32) {
        int warps = (blockDim.x + 31) >> 5;
        int v = tid < warps ? warp_best[tid] : lowest;
        v = max(__shfl_xor_sync(0xffffffffu, v, 16), v);
        v = max(__shfl_xor_sync(0xffffffffu, v, 8), v);
        v = max(__shfl_xor_sync(0xffffffffu, v, 4), v);
        v = max(__shfl_xor_sync(0xffffffffu, v, 2), v);
        v = max(__shfl_xor_sync(0xffffffffu, v, 1), v);
        if (tid == 0) {
            atomicMax(out, v);
        }
    }
}
