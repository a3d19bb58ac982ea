// Exercises loops, early exit, short-circuit operators, the conditional operator, unsigned
// arithmetic and a shared-memory exchange: out[i] depends on in[i] and on the neighbouring lane.
__device__ unsigned mix(unsigned v, unsigned k) {
    v ^= v >> 15;
    v *= 0x85ebca6bu;
    return v + k;
}

__global__ void control_flow(const int *in, int *out, int n) {
    __shared__ int stage[256];
    int tid = threadIdx.x;
    int i = blockIdx.x * blockDim.x + tid;
    int v = i < n ? in[i] : 0;
    stage[tid] = v;
    __syncthreads();
    int neighbour = stage[(tid + 1) % 256];
    if (i >= n) return;
    int acc = 0;
    for (int k = 0; k < 8; k++) {
        if (k == 5 && v < 0) break;
        if ((k & 1) != 0 || v == 7) continue;
        acc += (int)mix((unsigned)(v + k), 3u);
    }
    int steps = 0;
    while (steps < 3 && acc > -1000) {
        acc -= 400;
        steps++;
    }
    do {
        acc += neighbour / 4 + neighbour % 4;
    } while (--steps > 0);
    out[i] = !(acc & 1) ? acc : -acc;
}
