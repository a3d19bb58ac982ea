// A three-link chain of device functions under one kernel: out[i] = -2 * in[i] + 1.
// Every link is a real call in the BIR; the backend inlines them.
__device__ int plus_one(int v) { return v + 1; }

__device__ int twice_plus_one(int v) { return plus_one(v * 2); }

__device__ int flip_then_scale(int v) { return twice_plus_one(-v); }

__global__ void chain_vector(const int *in, int *out, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        out[i] = flip_then_scale(in[i]);
    }
}
