# c[i] = a[i] + b[i] on 32-bit integers (wrapping), masked at n.
import triton
import triton.language as tl


@triton.jit
def vadd_i32(a_ptr, b_ptr, c_ptr, n, BLOCK: tl.constexpr):
    pid = tl.program_id(0)
    offs = pid * BLOCK + tl.arange(0, BLOCK)
    mask = offs < n
    tl.store(c_ptr + offs, tl.load(a_ptr + offs, mask=mask) + tl.load(b_ptr + offs, mask=mask), mask=mask)
