# Signed maximum of x[0..n) folded into *out (which the caller initialises, normally to INT_MIN):
# each program reduces BLOCK elements and issues one atomic per warp.
import triton
import triton.language as tl


@triton.jit
def max_i32(x_ptr, out_ptr, n, BLOCK: tl.constexpr):
    pid = tl.program_id(0)
    offs = pid * BLOCK + tl.arange(0, BLOCK)
    x = tl.load(x_ptr + offs, mask=offs < n, other=-2147483648)
    tl.atomic_max(out_ptr, tl.max(x, axis=0))
