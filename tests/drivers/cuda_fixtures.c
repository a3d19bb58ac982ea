/* Host driver for the CUDA-C example kernels, written against the reference's CPU-launch
 * signatures (kernel parameters, then int64_t nthreads) and checking the known answers the
 * reference's examples check (examples/cpu_launch_{vadd,device_helper_chain,device_helper_square,
 * stress,mma2x2,tiled_sgemm}.c).  Links against whatever provides the kernel symbols. */
#include <stdint.h>
#include <stdio.h>

extern void vector_add(const float *a, const float *b, float *c, int n, int64_t nthreads);
extern void chain_vector(const int *in, int *out, int n, int64_t nthreads);
extern void square_vector(const int *in, int *out, int n, int64_t nthreads);
extern void stress(const float *a, float *out, int n, int64_t nthreads);
extern void mma2x2(const float *a, const float *b, const float *c, float *d, int64_t nthreads);
extern void tiled_sgemm_f32(const float *a, const float *b, const float *c, float *d, int64_t nthreads);

#define N 1024
static int fail(const char *what, int i) { fprintf(stderr, "FAIL: %s at %d\n", what, i); return 1; }

int main(void) {
    static float a[N], b[N], c[N];
    static int in[N], out[N];
    for (int i = 0; i < N; i++) { a[i] = (float)i; b[i] = (float)(2 * i); c[i] = -1.0f; }
    vector_add(a, b, c, N, (int64_t)N);
    for (int i = 0; i < N; i++) if (c[i] != a[i] + b[i]) return fail("vector_add", i);

    for (int i = 0; i < N; i++) { in[i] = i - N / 2; out[i] = 0x7fffffff; }
    chain_vector(in, out, N, (int64_t)N);
    for (int i = 0; i < N; i++) if (out[i] != -2 * in[i] + 1) return fail("chain_vector", i);
    for (int i = 0; i < N; i++) out[i] = 0x7fffffff;
    square_vector(in, out, N, (int64_t)N);
    for (int i = 0; i < N; i++) if (out[i] != in[i] * in[i]) return fail("square_vector", i);

    float s[20], sout[1] = {-1.0f};
    for (int i = 0; i < 20; i++) s[i] = (float)(i + 1) * 0.5f - 3.0f;
    stress(s, sout, 1, (int64_t)1);
    if (sout[0] != 191.0f) return fail("stress", 0);

    float ma[4] = {1, 2, 3, 4}, mb[4] = {5, 6, 7, 8}, mc[4] = {0.5f, 0.5f, 0.5f, 0.5f}, md[4] = {-1, -1, -1, -1};
    const float want[4] = {19.5f, 22.5f, 43.5f, 50.5f};
    mma2x2(ma, mb, mc, md, 1);
    for (int i = 0; i < 4; i++) if (md[i] != want[i]) return fail("mma2x2", i);

    static float ga[1024], gb[1024], gc[1024], gd[1024 + 768];
    for (int i = 0; i < 32; i++)
        for (int j = 0; j < 32; j++) {
            ga[i * 32 + j] = (float)((3 * i + j) % 7 + 1);
            gb[i * 32 + j] = (float)((i + 5 * j) % 7 + 1);
            gc[i * 32 + j] = (float)((i + j) % 4);
        }
    for (int i = 0; i < 1024 + 768; i++) gd[i] = -1.0f;
    tiled_sgemm_f32(ga, gb, gc, gd, 1);
    for (int i = 0; i < 32; i++)
        for (int j = 0; j < 32; j++) {
            float sum = gc[i * 32 + j];
            for (int k = 0; k < 32; k++) sum += ga[i * 32 + k] * gb[k * 32 + j];
            if (gd[i * 32 + j] != sum) return fail("tiled_sgemm_f32", i * 32 + j);
        }
    printf("PASS: vector_add, chain_vector, square_vector, stress, mma2x2, tiled_sgemm_f32\n");
    return 0;
}
