// out[i] = in[i] * in[i] through one device function.
__device__ int squared(int v) { return v * v; }

__global__ void square_vector(const int *in, int *out, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        out[i] = squared(in[i]);
    }
}
