"""The Triton front end: `@triton.jit` sources compile to BIR the backend accepts; elementwise
tile code computes the reference's known answers in the CPU oracle's execution model (one thread
per program, crates/basalt-x86/src/oracle.rs:7-28) and the same values when a CTA's threads share
the lanes; tl.dot kernels become one `mma` with the operand layout of their hand-authored BIR twins
and take the same device lowering; what is outside the subset is refused with the reference's
codes (crates/basalt-diag/src/ecode.rs:148-181)."""
import os
import shutil
import subprocess

import numpy as np
import pytest

import basalt_b200 as b
from basalt_b200 import kernels_bir as kb
from basalt_b200 import kernels_triton as kt
from oracle.bir_interp import run_kernel
from _util import sgemm_fixture

# A checkout of the reference project, when the environment names one (BASALT_REFERENCE_TREE=<its root>).
REFERENCE_KERNELS = os.path.join(os.environ.get("BASALT_REFERENCE_TREE", ""), "tests", "kernels")


def checked(ptx, bir):
    assert ptx.supports(bir).supported, ptx.supports(bir)
    assert b.roundtrip(bir) == bir
    return bir


def ptxas(text, tmp_path):
    exe = shutil.which("ptxas") or "/usr/local/cuda/bin/ptxas"
    src = tmp_path / "k.ptx"
    src.write_text(text)
    subprocess.run([exe, "-arch=sm_100a", str(src), "-o", os.devnull], check=True)


def test_masked_vector_add_known_answer(ptx, tmp_path):
    # examples/cpu_launch_triton_vadd.c:31-58: a[i] = i, b[i] = 2i, N = 1000, BLOCK = 1024, c poisoned
    # with -1; lanes at or past N must neither load (a and b are only N long) nor store.
    bir = checked(ptx, kt.vector_add())
    assert "func @vector_add(ptr.global, ptr.global, ptr.global, i64, i64) -> void" in bir      # pointers, then i64 scalars
    # four lanes per loop iteration, two masked loads and one masked store each; masks are branches, never selects
    assert bir.count("load f32 ptr.global") == 8 and bir.count("store f32 ptr.global") == 4 and "select" not in bir and bir.count("condbr") >= 13
    n, block = 1000, 1024
    a = np.arange(n, dtype=np.float32)
    for text in (bir, ptx.optimized_bir(bir), kb.load("tri_vadd")):
        for threads in (1, 256, 7):        # one thread per program (the reference's launch), or the lanes shared by a CTA
            c = np.full(block, -1.0, np.float32)
            run_kernel(text, "vector_add", [a, 2 * a, c, n, block], threads)
            assert np.array_equal(c[:n], 3 * a) and np.all(c[n:] == -1.0), threads
    for level in (0, 2):
        ptxas(ptx.emit(bir, b.EmitOpts(opt_level=level)).text, tmp_path)


def test_small_matmul_known_answer(ptx, tmp_path):
    # examples/cpu_launch_triton_matmul.c:39-89: D = A@B + C at M=4, K=5, N=3 on small integers, exact.
    bir = checked(ptx, kt.small_matmul(5))
    assert "func @matmul_kernel(ptr.global, ptr.global, ptr.global, ptr.global, i64) -> void" in bir   # M, N have defaults: dropped; K stays
    assert "mma f32 f32 row row m 4 n 3 k 5 ld 5 3 3 3" in bir and "load" not in bir                      # tl.dot is the tile op
    A, B, C = sgemm_fixture(4, 3, 5)
    want = A @ B + C
    for text in (bir, kb.load("tri_matmul")):
        out = np.zeros((4, 3), np.float32)
        run_kernel(text, "matmul_kernel", [A, B, C, out, 5], 1)
        assert np.array_equal(out, want)
    ptxas(ptx.emit(bir).text, tmp_path)


def test_tiled_matmuls_become_one_mma_with_the_twins_lowering(ptx, tmp_path):
    plan = lambda t: [l for l in t.splitlines() if l.startswith("//!basalt.plan")]
    for M, N, K in [(256, 512, 1024), (128, 128, 64)]:
        bir = checked(ptx, kt.matmul_f16(M, N, K))
        assert f"mma f16 f32 row row m 128 n 128 k {K} ld {K} {N} {N} {N} out f16" in bir and bir.count("mma ") == 1    # the K loop is inside the op
        assert "launch_bounds max_threads=128 min_blocks=2" in bir
        mine, twin = ptx.emit(bir).text, ptx.emit(kb.matmul_f16(M, N, K)).text
        assert "tcgen05.mma" in mine and "cp.async.bulk.tensor" in mine
        # same plan apart from the parameter count: the Triton ABI keeps M, N, K as i64 parameters
        strip = lambda ls: [l.replace("params=6", "params=3") for l in ls]
        assert strip(plan(mine)) == plan(twin)
        ptxas(mine, tmp_path)
        bir = checked(ptx, kt.sgemm(M, N, K))
        assert f"mma f32 f32 row row m 128 n 128 k {K} ld {K} {N} {N} {N}" in bir and bir.count("mma ") == 1
        mine = ptx.emit(bir).text
        assert "fma.rn.f32" in mine and "tcgen05" not in mine
        ptxas(mine, tmp_path)


def test_tiled_matmul_values_on_one_small_program(ptx):
    # One program (the oracle's launch has bid = 0) with small tiles: 16 x 16 x 32 in slabs of 8.
    M = N = 16
    K = 32
    rng = np.random.default_rng(3)
    A = rng.integers(-3, 4, (M, K)).astype(np.float32)
    B = rng.integers(-3, 4, (K, N)).astype(np.float32)
    bir = checked(ptx, kt.sgemm(M, N, K, BLOCK_M=16, BLOCK_N=16, BLOCK_K=8))
    assert f"mma f32 f32 row row m 16 n 16 k {K} ld {K} {N} {N} {N}" in bir
    out = np.zeros((M, N), np.float32)
    run_kernel(bir, "sgemm_f32", [A, B, out, M, N, K], 1)
    assert np.array_equal(out, A @ B)
    bir = checked(ptx, kt.matmul_f16(M, N, K, BLOCK_M=16, BLOCK_N=16, BLOCK_K=8))
    out = np.zeros((M, N), np.float16)
    run_kernel(bir, "matmul_kernel", [A.astype(np.float16), B.astype(np.float16), out, M, N, K], 1)
    assert np.array_equal(out, (A @ B).astype(np.float16))


def test_int32_sources_wrap_and_reduce(ptx, orc, tmp_path):
    import ctypes
    from _util import vp
    from basalt_b200 import workloads as w
    bir = checked(ptx, kt.vadd_i32())
    assert "add i32" in bir and "load i32 ptr.global" in bir and "store i32 ptr.global" in bir       # 32-bit data stays 32 bits wide
    n = 1000
    a = w.i32_pm30(1, n) * 2; bb = w.i32_pm30(2, n) * 2                                             # sums overflow and must wrap
    want = np.zeros(n, np.int32)
    orc.orc_vadd_i32(vp(a), vp(bb), vp(want), ctypes.c_int32(n), ctypes.c_int64(n))
    for threads in (1, 64):
        c = np.full(1024, 0x7fffffff, np.int32)
        run_kernel(bir, "vadd_i32", [a, bb, c, n, 1024], threads)
        assert np.array_equal(c[:n], want) and np.all(c[n:] == 0x7fffffff)
    # the reduction: per-thread fold in a lane loop, a warp step, the warps combined through shared memory, one atomic per
    # program (values are checked on the device: the CPU oracle's launch has no warps)
    bir = checked(ptx, kt.max_i32())
    assert bir.count("warp.reduce.max i32") == 2 and bir.count("atomic.max i32 ptr.global") == 1 and "shuffle" not in bir
    assert "shared_obj 0 bytes 128 align 16" in bir and bir.count("barrier") == 1
    # the program's lanes are consecutive int32 words: four 16-byte loads per loop iteration, a one-word loop for the rest
    assert bir.count("load v4i32 ptr.global") == 4 and bir.count("load i32 ptr.global") == 1
    assert "phi i32" in bir and "const.i i32 -2147483648" in bir
    text = ptx.emit(bir).text
    assert "redux.sync.max.s32" in text
    ptxas(text, tmp_path)
    # float32 sums use an xor butterfly of shuffles
    src = "@triton.jit\ndef total(x_ptr, out_ptr, n, BLOCK: tl.constexpr):\n    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)\n" \
          "    tl.atomic_add(out_ptr, tl.sum(tl.load(x_ptr + offs, mask=offs < n, other=0.0), axis=0))\n"
    bir = checked(ptx, b.compile_triton(src))
    assert bir.count("shuffle.xor f32") == 10 and bir.count("atomic.add f32 ptr.global") == 1
    ptxas(ptx.emit(bir).text, tmp_path)
    # elementwise atomics run under the oracle: a histogram-like scatter with a mask
    src = "@triton.jit\ndef scatter(idx_ptr, out_ptr, n, BLOCK: tl.constexpr = 16):\n    offs = tl.arange(0, BLOCK)\n    m = offs < n\n" \
          "    i = tl.load(idx_ptr + offs, mask=m, other=0)\n    tl.atomic_add(out_ptr + i, offs + 1, mask=m)\n"
    bir = checked(ptx, b.compile_triton(src, pointee={"idx_ptr": "i64", "out_ptr": "i64"}))
    idx = np.array([0, 2, 2, 1, 0, 3, 3, 3, 9, 9, 9, 9, 9, 9, 9, 9], np.int64)
    out = np.zeros(10, np.int64)
    run_kernel(bir, "scatter", [idx, out, 8], 4)
    assert out.tolist() == [1 + 5, 4, 2 + 3, 6 + 7 + 8, 0, 0, 0, 0, 0, 0]


ELEMENTWISE = '''
import triton
import triton.language as tl

@triton.jit
def scale_clip(x_ptr, y_ptr, n, lo, BLOCK: tl.constexpr = 64):
    """y = where(x > lo, 2 * x + 1, lo) on int64 data, two-dimensional tile of 4 x 16 lanes."""
    pid = tl.program_id(0)
    rows = tl.arange(0, 4)
    cols = tl.arange(0, BLOCK // 4)
    offs = pid * BLOCK + rows[:, None] * (BLOCK // 4) + cols[None, :]
    mask = offs < n
    x = tl.load(x_ptr + offs, mask=mask, other=0)
    y = tl.where(x > lo, x * 2 + 1, lo)
    tl.store(y_ptr + offs, tl.maximum(y, -5), mask=mask)
'''


def test_rank2_elementwise_tile_code(ptx):
    bir = checked(ptx, b.compile_triton(ELEMENTWISE, pointee={"x_ptr": "i64", "y_ptr": "i64"}))
    assert "func @scale_clip(ptr.global, ptr.global, i64, i64) -> void" in bir
    n = 50
    x = np.random.default_rng(5).integers(-20, 20, 64).astype(np.int64)
    for threads in (1, 32):
        y = np.full(64, 777, np.int64)
        run_kernel(bir, "scale_clip", [x, y, n, -3], threads)
        want = np.maximum(np.where(x > -3, 2 * x + 1, -3), -5)
        assert np.array_equal(y[:n], want[:n]) and np.all(y[n:] == 777)


@pytest.mark.parametrize("code, source, kw", [
    ("E201", "@triton.jit\ndef k(x_ptr):\n    tl.store(x_ptr, 1 + )\n", {}),
    ("E201", "import triton\n", {}),
    ("E202", "@triton.jit\ndef k(x_ptr):\n    '''never closed\n", {}),
    ("E200", "@triton.jit\ndef k(x_ptr):\n    tl.store(x_ptr, 1 $ 2)\n", {}),
    ("E301", "@triton.jit\ndef k(x_ptr):\n    tl.store(x_ptr, missing)\n", {}),
    ("E301", "@triton.jit\ndef k(x_ptr):\n    tl.store(x_ptr, tl.frobnicate(1))\n", {}),
    ("E300", "@triton.jit\ndef k(x_ptr, y_ptr):\n    tl.store(x_ptr + y_ptr, 1.0)\n", {"pointee": {"y_ptr": "f32"}}),
    ("E300", "@triton.jit\ndef k(x_ptr):\n    tl.store(x_ptr, tl.load(x_ptr, mask=1))\n", {}),
    ("E304", "@triton.jit\ndef k(x_ptr, n):\n    while n:\n        pass\n", {}),
    ("E304", "@triton.jit\ndef k(x_ptr):\n    tl.store(x_ptr, tl.exp(tl.load(x_ptr)))\n", {}),
    ("E304", "@triton.jit\ndef k(x_ptr, n):\n    if n > 0:\n        tl.store(x_ptr, 1.0)\n", {}),
    ("E305", "@triton.jit\ndef k(x_ptr):\n    a = tl.arange(0, 4)\n    b = tl.arange(0, 8)\n    tl.store(x_ptr + a, tl.load(x_ptr + b))\n", {}),
    ("E305", "@triton.jit\ndef k(x_ptr):\n    a = tl.arange(0, 4)\n    tl.store(x_ptr + a, tl.load(x_ptr + a[:, None]))\n", {}),
    ("E306", "@triton.jit\ndef k(x_ptr, n):\n    a = tl.arange(0, n + 1)\n    tl.store(x_ptr + a, 1.0)\n", {}),
    ("E306", kt.load("small_matmul"), {}),                                  # K left unbound: tl.dot needs constant extents
    ("E307", "@triton.jit\ndef k(x_ptr):\n    a = tl.arange(0, 4)\n    tl.store(x_ptr, tl.sum(tl.load(x_ptr + a)))\n", {}),
    ("E307", "@triton.jit\ndef k(x_ptr):\n    a = tl.arange(0, 4)\n    tl.atomic_max(x_ptr, tl.sum(tl.load(x_ptr + a)))\n", {}),
    ("E307", "@triton.jit\ndef k(x_ptr):\n    a = tl.arange(0, 4)\n    tl.atomic_xchg(x_ptr + a, 1.0)\n", {}),
    ("E307", "@triton.jit\ndef k(x_ptr):\n    a = tl.arange(0, 8)\n    tl.store(x_ptr + a[1:], 1.0)\n", {}),
    ("E307", kt.load("small_matmul").replace("acc + c)", "acc + c, mask=rows[:, None] < 3)"), {"constexprs": {"K": 5}}),
    ("E307", kt.load("small_matmul").replace("tl.load(a_ptr + rows[:, None] * K + depth[None, :])", "tl.load(a_ptr + rows[:, None] * K + depth[None, :]) * 2.0"),
     {"constexprs": {"K": 5}}),
])
def test_refusals_carry_the_reference_codes(code, source, kw):
    with pytest.raises(b.Diag) as e:
        b.compile_triton(source, **kw)
    assert e.value.code == code, (e.value.code, e.value.arg)


def test_bindings_are_checked():
    with pytest.raises(b.Diag) as e:
        b.compile_triton(kt.load("vector_add"), pointee={"a_ptr": "f8"})
    assert e.value.code == "E102"


def test_cli_accepts_triton_sources(tmp_path):
    import basalt_b200.build as build
    out = subprocess.run([build.CLI, "--emit-bir", kt.path("small_matmul"), "--bind", "K=5"], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout == kt.small_matmul(5)
    out = subprocess.run([build.CLI, "--nvidia-ptx", kt.path("vector_add")], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout == b.Ptx().emit(kt.vector_add()).text
    out = subprocess.run([build.CLI, "--nvidia-ptx", kt.path("small_matmul")], capture_output=True, text=True)
    assert out.returncode == 1 and out.stderr.startswith("E306: ")


@pytest.mark.skipif(not os.environ.get("BASALT_REFERENCE_TREE") or not os.path.isdir(REFERENCE_KERNELS), reason="BASALT_REFERENCE_TREE does not name a checkout of the reference")
def test_the_reference_tree_triton_kernels(ptx):
    """The reference's own Triton sources (tests/kernels/tri_*.py), read where they lie, with the
    inputs and answers of examples/cpu_launch_triton_{vadd,matmul}.c."""
    def src(name):
        with open(os.path.join(REFERENCE_KERNELS, name)) as f:
            return f.read()
    bir = checked(ptx, b.compile_triton(src("tri_vadd.py")))
    a = np.arange(1000, dtype=np.float32)
    c = np.full(1024, -1.0, np.float32)
    run_kernel(bir, "vector_add", [a, 2 * a, c, 1000, 1024], 1)
    assert np.array_equal(c[:1000], 3 * a) and np.all(c[1000:] == -1.0)
    bir = checked(ptx, b.compile_triton(src("tri_matmul.py"), constexprs={"K": 5}))
    A, B, C = sgemm_fixture(4, 3, 5)
    out = np.zeros((4, 3), np.float32)
    run_kernel(bir, "matmul_kernel", [A, B, C, out, 5], 1)
    assert np.array_equal(out, A @ B + C)


# ---- calls between @triton.jit functions ----
SAXPY_INLINE = '''
import triton
import triton.language as tl

@triton.jit
def saxpy_kernel(x_ptr, y_ptr, out_ptr, n, BLOCK: tl.constexpr):
    pid = tl.program_id(0)
    offs = pid * BLOCK + tl.arange(0, BLOCK)
    x = tl.load(x_ptr + offs, mask=offs < n, other=0.0)
    y = tl.load(y_ptr + offs, mask=offs < n, other=0.0)
    t = x * 2.5
    tl.store(out_ptr + offs, t + y, mask=offs < n)
'''


def test_helper_functions_are_inlined(ptx):
    # four helpers (positional, keyword and defaulted arguments, a helper that only stores): one entry, and the
    # same BIR as the kernel written in one piece; pointer-ness of x_ptr / y_ptr / out_ptr flows through the calls
    bir = kt.saxpy_helpers()
    assert bir.count("func @") == 1 and "func @saxpy_kernel(ptr.global, ptr.global, ptr.global, i64, i64)" in bir
    assert bir == b.compile_triton(SAXPY_INLINE)
    n = 100
    x = np.arange(n, dtype=np.float32); y = np.ones(n, np.float32)
    for text in (bir, ptx.optimized_bir(bir)):
        out = np.full(128 + 4, -1.0, np.float32)
        run_kernel(text, "saxpy_kernel", [x, y, out, n, 128], 1)
        assert np.array_equal(out[:n], 2.5 * x + y) and np.all(out[n:] == -1.0)


@pytest.mark.parametrize("code, body", [
    ("E304", "@triton.jit\ndef f(x):\n    return f(x)\n@triton.jit\ndef k(p, n):\n    tl.store(p + tl.arange(0, 4), f(tl.load(p + tl.arange(0, 4))))\n"),
    ("E300", "@triton.jit\ndef f(x, y):\n    return x + y\n@triton.jit\ndef k(p):\n    tl.store(p + tl.arange(0, 4), f(tl.load(p + tl.arange(0, 4))))\n"),
    ("E300", "@triton.jit\ndef f(x):\n    return x\n@triton.jit\ndef k(p):\n    tl.store(p + tl.arange(0, 4), f(tl.load(p + tl.arange(0, 4)), z=1))\n"),
    ("E300", "@triton.jit\ndef f(x):\n    return x\n@triton.jit\ndef k(p):\n    tl.store(p + tl.arange(0, 4), f(1, 2))\n"),
    ("E307", "@triton.jit\ndef f(x):\n    return (x, x)\n@triton.jit\ndef k(p):\n    a = f(tl.load(p + tl.arange(0, 4)))\n"),
    ("E304", "@triton.jit\ndef f(x):\n    return g(x)\n@triton.jit\ndef g(x):\n    return f(x)\n"),
])
def test_helper_call_refusals(code, body):
    with pytest.raises(b.Diag) as e:
        b.compile_triton("import triton\nimport triton.language as tl\n" + body)
    assert e.value.code == code, e.value
