# out[i] = 2.5 * x[i] + y[i], written with helper functions: a @triton.jit function that another one
# calls is inlined at the call, so only `saxpy_kernel` becomes an entry.
import triton
import triton.language as tl


@triton.jit
def offsets(pid, BLOCK: tl.constexpr):
    return pid * BLOCK + tl.arange(0, BLOCK)


@triton.jit
def load_masked(ptr, offs, n, other=0.0):
    mask = offs < n
    return tl.load(ptr + offs, mask=mask, other=other)


@triton.jit
def axpy(x, y, alpha):
    t = x * alpha
    return t + y


@triton.jit
def store_masked(ptr, offs, value, n):
    tl.store(ptr + offs, value, mask=offs < n)


@triton.jit
def saxpy_kernel(x_ptr, y_ptr, out_ptr, n, BLOCK: tl.constexpr):
    pid = tl.program_id(0)
    offs = offsets(pid, BLOCK)
    x = load_masked(x_ptr, offs, n)
    y = load_masked(ptr=y_ptr, offs=offs, n=n)
    store_masked(out_ptr, offs, axpy(x, y, 2.5), n)
