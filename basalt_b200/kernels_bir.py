"""BIR sources of the benchmark kernels and of the reference's known-answer fixtures.

The reference's front ends (CUDA-C and Triton to BIR) are Rust and cannot run here, so each
kernel is hand-written BIR in the shape `basalt-sema` plus `basalt_passes::optimize` would hand
to the PTX backend (one element per thread behind an `i < n` guard, `ptr + sext(i)*4`
addressing, slots already promoted to SSA).  Fixed kernels live as `bir/<name>.birs` (symbolic
names) with the assembled `bir/<name>.bir` beside them; kernels specialised on a shape, the way
Triton specialises on constexprs, are generated here.
"""
from __future__ import annotations

import os

from .birasm import assemble

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "bir")

STATIC = ("vadd_i32", "vector_add_f32", "max_i32", "max_i32_atomic", "chain_vector", "square_vector", "mma2x2",
          "tiled_sgemm_f32", "tri_matmul", "tri_vadd", "sgemm_tile16", "max_i32_strided", "slot_form_sum")


def load(name: str) -> str:
    """Assembled BIR text of a fixed kernel."""
    with open(os.path.join(_DIR, name + ".bir")) as f:
        return f.read()


_ELEMENTWISE_KERNEL = """
  func @{name}(ptr.global, ptr.global, i32) -> void {{
  entry:
    %bid = bid.x i32
    %bdim = bdim.x i32
    %base = mul i32 %bid, %bdim
    %tid = tid.x i32
    %i = add i32 %base, %tid
    %inb = icmp slt i32 %i, %arg2
    condbr %inb, body, exit
  body:
    %i64 = sext i64 i32 %i
    %four = const.i i64 4
    %off = mul i64 %i64, %four
    %pin = add ptr.global %arg0, %off
    %x = load {ty} ptr.global %pin, align 4
{compute}
    %pout = add ptr.global %arg1, %off
    store {ty} ptr.global %pout, %y, align 4
    br exit
  exit:
    ret
  }}
"""


def helper_chain(depth: int = 32) -> str:
    """out[i] = step_0(in[i]); step_j(x) = step_{j+1}(x*x + k_j), k_j = 2654435761*j mod 2^32, the
    last level returning: `depth` nested `__device__` helpers, the device_helper_chain.cu pattern
    of the reference (tests/kernels/device_helper_chain.cu:9-26) at depth 32."""
    parts = ["module {\n  shared_mem_bytes 0\n  target_dtypes i32\n"]
    for j in range(depth):
        k = (2654435761 * j) & 0xFFFFFFFF
        k_signed = k - (1 << 32) if k >= (1 << 31) else k
        body = f"    %sq = mul i32 %arg0, %arg0\n    %k = const.i i32 {k_signed}\n    %y = add i32 %sq, %k\n"
        if j + 1 < depth:
            body += f"    %r = call i32 @step{j + 1} [%y]\n    ret %r\n"
        else:
            body += "    ret %y\n"
        parts.append(f"\n  host func @step{j}(i32) -> i32 {{\n  entry:\n{body}  }}\n")
    parts.append(_ELEMENTWISE_KERNEL.format(name="helper_chain", ty="i32", compute="    %y = call i32 @step0 [%x]"))
    parts.append("}\n")
    return assemble("".join(parts))


def stress() -> str:
    """The register-pressure fixture of the reference (tests/kernels/stress.cu): eighteen
    temporaries a[p]*a[q] + a[r] over a rotating index, all live at once, summed left to right."""
    ld, comp = [], []
    for e in range(20):
        ld.append(f"    %o{e} = const.i i64 {4 * e}\n    %p{e} = add ptr.global %arg0, %o{e}\n    %a{e} = load f32 ptr.global %p{e}, align 4\n")
    for j in range(18):
        p, q, r = (3 * j) % 20, (3 * j + 1) % 20, (3 * j + 2) % 20
        comp.append(f"    %m{j} = fmul f32 %a{p}, %a{q}\n    %t{j} = fadd f32 %m{j}, %a{r}\n")
    acc = "%t0"
    for j in range(1, 18):
        comp.append(f"    %s{j} = fadd f32 {acc}, %t{j}\n")
        acc = f"%s{j}"
    text = f"""module {{
  shared_mem_bytes 0
  target_dtypes f32

  func @stress(ptr.global, ptr.global, i32) -> void {{
  entry:
    %i = tid.x i32
    %inb = icmp slt i32 %i, %arg2
    condbr %inb, body, exit
  body:
{''.join(ld)}{''.join(comp)}    %i64 = sext i64 i32 %i
    %four = const.i i64 4
    %off = mul i64 %i64, %four
    %pout = add ptr.global %arg1, %off
    store f32 ptr.global %pout, {acc}, align 4
    br exit
  exit:
    ret
  }}
}}
"""
    return assemble(text)


def sgemm_cta128(M: int, N: int, K: int) -> str:
    """C[MxN] = A[MxK] * B[KxN] in f32, row-major: CTA (bid.x, bid.y) computes the 128x128 tile at
    row bid.y*128, column bid.x*128 with one CTA-wide `mma` over the whole K extent on strided
    tiles of the full matrices (leading dimensions K, N, N).  Operand c is the null pointer: no
    addend.  Launch with grid (N/128, M/128) and 256 threads."""
    assert M % 128 == 0 and N % 128 == 0 and K % 16 == 0
    text = f"""module {{
  launch_bounds max_threads=256 min_blocks=2
  shared_mem_bytes 0
  target_dtypes f32

  func @sgemm_f32(ptr.global, ptr.global, ptr.global) -> void {{
  entry:
    %bx = bid.x i64
    %by = bid.y i64
    %arow = const.i i64 {128 * K * 4}
    %aoff = mul i64 %by, %arow
    %a = add ptr.global %arg0, %aoff
    %bcol = const.i i64 {128 * 4}
    %boff = mul i64 %bx, %bcol
    %b = add ptr.global %arg1, %boff
    %crow = const.i i64 {128 * N * 4}
    %coff0 = mul i64 %by, %crow
    %coff = add i64 %coff0, %boff
    %d = add ptr.global %arg2, %coff
    %null = const.i ptr.global 0
    mma f32 f32 row row m 128 n 128 k {K} ld {K} {N} {N} {N} %a, %b, %null, %d
    ret
  }}
}}
"""
    return assemble(text)


def matmul_f16(M: int, N: int, K: int, b_is_nk: bool = False, per_cta: bool = False) -> str:
    """C[MxN] (f16) = A[MxK] (f16) * B (f16), f32 accumulation: the tile-level form of a Triton
    matmul with BLOCK_M = BLOCK_N = 128 (the K loop over BLOCK_K = 64 slabs is inside the `mma`).
    B is [K x N] row-major, or with b_is_nk stored transposed as [N x K].  Launch with grid
    (N/128, M/128) and 128 threads.  per_cta adds a trailing barrier, which keeps the emitter from
    re-scheduling the grid as a persistent kernel (each CTA then runs its own TMA + tcgen05 pipeline)."""
    assert M % 128 == 0 and N % 128 == 0 and K % 64 == 0
    if b_is_nk:
        lb, ldb, bstep = "col", K, 128 * K * 2
    else:
        lb, ldb, bstep = "row", N, 128 * 2
    text = f"""module {{
  launch_bounds max_threads=128 min_blocks=2
  shared_mem_bytes 0
  target_dtypes f16 f32

  func @matmul_kernel(ptr.global, ptr.global, ptr.global) -> void {{
  entry:
    %bx = bid.x i64
    %by = bid.y i64
    %arow = const.i i64 {128 * K * 2}
    %aoff = mul i64 %by, %arow
    %a = add ptr.global %arg0, %aoff
    %bstep = const.i i64 {bstep}
    %boff = mul i64 %bx, %bstep
    %b = add ptr.global %arg1, %boff
    %crow = const.i i64 {128 * N * 2}
    %coff0 = mul i64 %by, %crow
    %ccol = const.i i64 {128 * 2}
    %coff1 = mul i64 %bx, %ccol
    %coff = add i64 %coff0, %coff1
    %d = add ptr.global %arg2, %coff
    %null = const.i ptr.global 0
    mma f16 f32 row {lb} m 128 n 128 k {K} ld {K} {ldb} {N} {N} out f16 %a, %b, %null, %d
{"    barrier" if per_cta else ""}
    ret
  }}
}}
"""
    return assemble(text)


def assemble_static() -> None:
    """Regenerates bir/<name>.bir from bir/<name>.birs."""
    for name in STATIC:
        with open(os.path.join(_DIR, name + ".birs")) as f:
            out = assemble(f.read())
        with open(os.path.join(_DIR, name + ".bir"), "w") as f:
            f.write(out)


if __name__ == "__main__":
    assemble_static()
