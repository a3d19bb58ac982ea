# out = a @ b + c on one small tile: a is [M, K], b is [K, N], c and out are [M, N], all row-major
# float32.  One program covers the whole result with a single tl.dot.
import triton
import triton.language as tl


@triton.jit
def matmul_kernel(a_ptr, b_ptr, c_ptr, out_ptr, K: tl.constexpr, M: tl.constexpr = 4, N: tl.constexpr = 3):
    rows = tl.arange(0, M)
    cols = tl.arange(0, N)
    depth = tl.arange(0, K)
    a = tl.load(a_ptr + rows[:, None] * K + depth[None, :])
    b = tl.load(b_ptr + depth[:, None] * N + cols[None, :])
    c = tl.load(c_ptr + rows[:, None] * N + cols[None, :])
    acc = tl.dot(a, b, tl.zeros((M, N), dtype=tl.float32))
    tl.store(out_ptr + rows[:, None] * N + cols[None, :], acc + c)
