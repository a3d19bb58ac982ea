// The naive form of the reduction: one atomicMax per element.
__global__ void max_i32_atomic(const int *x, int *out, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        atomicMax(out, x[i]);
    }
}
