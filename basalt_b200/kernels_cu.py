"""CUDA-C sources of the kernels, for the front end (`basalt_b200.compile_cuda`).

The static sources live in `basalt_b200/cu/*.cu`; the parametrised ones (the helper chain's depth,
the matrix shapes of the two matmul kernels) are generated here.  Each has a hand-authored BIR twin
in `kernels_bir`, and the tests check that both routes give the same results.
"""
from __future__ import annotations

import os

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cu")

STATIC = ("vadd_i32", "vector_add_f32", "max_i32", "max_i32_atomic", "chain_vector", "square_vector", "constant_math",
          "control_flow", "switch_cases")


def path(name: str) -> str:
    return os.path.join(_DIR, name + ".cu")


def load(name: str) -> str:
    with open(path(name)) as f:
        return f.read()


def helper_chain(depth: int = 32) -> str:
    """x -> x*x + k_j (mod 2^32) applied `depth` times, link j calling link j+1, with
    k_j = (2654435761 * j) mod 2^32.  The same chain as kernels_bir.helper_chain."""
    parts = ["// A chain of %d device functions; link j squares, adds its constant and calls link j+1.\n" % depth]
    for j in reversed(range(depth)):
        k = (2654435761 * j) & 0xFFFFFFFF
        nxt = f"link{j + 1}(y)" if j + 1 < depth else "y"
        parts.append(f"__device__ unsigned link{j}(unsigned x) {{\n    unsigned y = x * x + {k}u;\n    return {nxt};\n}}\n")
    parts.append("""
__global__ void helper_chain(const unsigned *in, unsigned *out, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        out[i] = link0(in[i]);
    }
}
""")
    return "\n".join(parts)


def stress(temps: int = 18, span: int = 20) -> str:
    """`temps` products a[p]*a[q]+a[r] (indices walking a `span`-element window) all live at once,
    then summed left to right: the register-pressure kernel (kernels_bir.stress has the same
    index walk)."""
    lines, names = [], []
    for t in range(temps):
        p, q, r = (3 * t) % span, (3 * t + 1) % span, (3 * t + 2) % span
        lines.append(f"        float t{t} = a[{p}] * a[{q}] + a[{r}];")
        names.append(f"t{t}")
    body = "\n".join(lines)
    return f"""// {temps} temporaries, each a product plus an addend, all live before the first is consumed.
__global__ void stress(const float *a, float *out, int n) {{
    int i = threadIdx.x;
    if (i < n) {{
{body}
        float sum = {' + '.join(names)};
        out[i] = sum;
    }}
}}
"""


def sgemm_cta128(M: int, N: int, K: int) -> str:
    """C[MxN] = A[MxK] * B[KxN] in f32: block (x, y) owns the 128x128 tile at row 128y, column
    128x and issues one tile product over the whole K extent.  Grid (N/128, M/128), 256 threads."""
    assert M % 128 == 0 and N % 128 == 0 and K % 16 == 0
    return f"""#define ROWS {M}
#define COLS {N}
#define DEPTH {K}
__global__ void __launch_bounds__(256, 2) sgemm_f32(const float *a, const float *b, float *c) {{
    const float *a_tile = a + (size_t)blockIdx.y * (128 * DEPTH);
    const float *b_tile = b + (size_t)blockIdx.x * 128;
    float *c_tile = c + (size_t)blockIdx.y * (128 * COLS) + (size_t)blockIdx.x * 128;
    __basalt_mma_f32(128, 128, DEPTH, a_tile, b_tile, 0, c_tile, DEPTH, COLS, COLS, COLS);
}}
"""


def matmul_f16(M: int, N: int, K: int, b_is_nk: bool = False) -> str:
    """C[MxN] (f16) = A[MxK] * B with f32 accumulation, 128x128 tile per block; B is [KxN], or
    [NxK] with b_is_nk.  Grid (N/128, M/128), 128 threads."""
    assert M % 128 == 0 and N % 128 == 0 and K % 64 == 0
    if b_is_nk:
        intr, b_tile, ldb = "__basalt_mma_f16_nt", "b + (size_t)blockIdx.x * (128 * DEPTH)", "DEPTH"
    else:
        intr, b_tile, ldb = "__basalt_mma_f16", "b + (size_t)blockIdx.x * 128", "COLS"
    return f"""#define ROWS {M}
#define COLS {N}
#define DEPTH {K}
__global__ void __launch_bounds__(128, 2) matmul_kernel(const __half *a, const __half *b, __half *c) {{
    const __half *a_tile = a + (size_t)blockIdx.y * (128 * DEPTH);
    const __half *b_tile = {b_tile};
    __half *c_tile = c + (size_t)blockIdx.y * (128 * COLS) + (size_t)blockIdx.x * 128;
    {intr}(128, 128, DEPTH, a_tile, b_tile, 0, c_tile, DEPTH, {ldb}, COLS, COLS);
}}
"""
