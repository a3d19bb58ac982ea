// c[i] = a[i] + b[i] on 32-bit integers (wrapping), one element per thread of a 1-D launch.
__global__ void vadd_i32(const int *a, const int *b, int *c, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        c[i] = a[i] + b[i];
    }
}
