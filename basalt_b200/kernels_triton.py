"""Triton sources of the kernels, for the Triton front end (`basalt_b200.compile_triton`).

The sources live in `basalt_b200/triton/*.py` and are ordinary `@triton.jit` functions; nothing here
imports Triton.  The helpers return BIR text for the shapes the tests and the benchmark use.
"""
from __future__ import annotations

import os

from . import backend

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "triton")


def path(name: str) -> str:
    return os.path.join(_DIR, name + ".py")


def load(name: str) -> str:
    with open(path(name)) as f:
        return f.read()


def vector_add() -> str:
    """Masked c = a + b; BLOCK_SIZE stays a run-time i64 parameter (the lane-loop bound)."""
    return backend.compile_triton(load("vector_add"))


def saxpy_helpers() -> str:
    """out = 2.5 x + y written with four helper @triton.jit functions, all inlined into `saxpy_kernel`."""
    return backend.compile_triton(load("saxpy_helpers"))


def small_matmul(K: int = 5) -> str:
    """out = a @ b + c on one M x N tile (M = 4, N = 3 by default in the source), f32."""
    return backend.compile_triton(load("small_matmul"), constexprs={"K": K})


def matmul_f16(M: int, N: int, K: int, **blocks) -> str:
    """The tiled f16 matmul; grid (N / BLOCK_N, M / BLOCK_M), compiled for 4 warps."""
    return backend.compile_triton(load("matmul_f16"), constexprs=dict(M=M, N=N, K=K, **blocks),
                                  pointee={"a_ptr": "f16", "b_ptr": "f16", "c_ptr": "f16"}, num_warps=4, min_blocks=2)


def sgemm(M: int, N: int, K: int, **blocks) -> str:
    """The tiled f32 matmul; grid (N / BLOCK_N, M / BLOCK_M), compiled for 8 warps."""
    return backend.compile_triton(load("sgemm"), constexprs=dict(M=M, N=N, K=K, **blocks), num_warps=8, min_blocks=2)


def vadd_i32() -> str:
    """Masked c = a + b on int32 (wrapping); BLOCK is the run-time lane count of a program."""
    return backend.compile_triton(load("vadd_i32"), pointee={"a_ptr": "i32", "b_ptr": "i32", "c_ptr": "i32"})


def max_i32() -> str:
    """Signed maximum folded into *out: tl.max over a program's BLOCK elements, one atomic per warp."""
    return backend.compile_triton(load("max_i32"), pointee={"x_ptr": "i32", "out_ptr": "i32"})
