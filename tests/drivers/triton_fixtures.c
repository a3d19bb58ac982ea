/* Host driver for the two Triton example kernels with the reference's CPU-launch signatures
 * (examples/cpu_launch_triton_vadd.c, cpu_launch_triton_matmul.c): scalars are int64, nthreads
 * comes last, lanes past n must stay poisoned. */
#include <stdint.h>
#include <stdio.h>

extern void vector_add(const float *a_ptr, const float *b_ptr, float *c_ptr, int64_t n, int64_t BLOCK_SIZE, int64_t nthreads);
extern void matmul_kernel(const float *a_ptr, const float *b_ptr, const float *c_ptr, float *out_ptr, int64_t K, int64_t nthreads);

int main(void) {
    enum { N = 1000, BLOCK = 1024, CW = 32768 };
    static float a[N], b[N], c[CW];
    for (int i = 0; i < N; i++) { a[i] = (float)i; b[i] = (float)(2 * i); }
    for (int i = 0; i < CW; i++) c[i] = -1.0f;
    vector_add(a, b, c, N, BLOCK, 1);
    for (int i = 0; i < BLOCK; i++) {
        float want = i < N ? a[i] + b[i] : -1.0f;
        if (c[i] != want) { fprintf(stderr, "FAIL: vector_add at %d\n", i); return 1; }
    }
    enum { M = 4, NN = 3, K = 5 };
    float ma[M * K], mb[K * NN], mc[M * NN], out[M * NN];
    for (int i = 0; i < M; i++) for (int k = 0; k < K; k++) ma[i * K + k] = (float)((3 * i + k) % 7 + 1);
    for (int k = 0; k < K; k++) for (int j = 0; j < NN; j++) mb[k * NN + j] = (float)((k + 5 * j) % 7 + 1);
    for (int i = 0; i < M; i++) for (int j = 0; j < NN; j++) { mc[i * NN + j] = (float)((i + j) % 4); out[i * NN + j] = -1.0f; }
    matmul_kernel(ma, mb, mc, out, K, 1);
    for (int i = 0; i < M; i++)
        for (int j = 0; j < NN; j++) {
            float sum = mc[i * NN + j];
            for (int k = 0; k < K; k++) sum += ma[i * K + k] * mb[k * NN + j];
            if (out[i * NN + j] != sum) { fprintf(stderr, "FAIL: matmul_kernel at (%d,%d)\n", i, j); return 1; }
        }
    printf("PASS: masked vector_add, matmul_kernel\n");
    return 0;
}
