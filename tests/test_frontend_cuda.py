"""The CUDA-C front end: sources compile to slot-form BIR that the backend accepts, the BIR
computes what the source says (checked in the CPU oracle's execution model, before and after the
backend's passes, against the C oracle and against the hand-authored BIR twins), and what is
outside the subset is refused with the reference's front-end codes
(crates/basalt-diag/src/ecode.rs:148-181)."""
import ctypes
import os
import shutil
import subprocess

import numpy as np
import pytest

import basalt_b200 as b
from basalt_b200 import kernels_bir as kb
from basalt_b200 import kernels_cu as kc
from oracle.bir_interp import run_kernel
from _util import vp

# A checkout of the reference project, when the environment names one (BASALT_REFERENCE_TREE=<its root>).
REFERENCE_KERNELS = os.path.join(os.environ.get("BASALT_REFERENCE_TREE", ""), "tests", "kernels")


def _both(ptx, source):
    """(slot-form BIR, optimised BIR) of a CUDA-C source."""
    bir = b.compile_cuda(source)
    assert ptx.supports(bir).supported, ptx.supports(bir)
    assert b.roundtrip(bir) == bir          # the front end prints canonical BIR
    return bir, ptx.optimized_bir(bir)


def _ptxas(text, tmp_path):
    exe = shutil.which("ptxas") or "/usr/local/cuda/bin/ptxas"
    src = tmp_path / "k.ptx"
    src.write_text(text)
    subprocess.run([exe, "-arch=sm_100a", str(src), "-o", os.devnull], check=True)


@pytest.mark.parametrize("name", kc.STATIC)
def test_static_sources_compile_emit_and_assemble(ptx, name, tmp_path):
    bir, opt = _both(ptx, kc.load(name))
    assert "ptr.param" in bir and "ptr.param" not in opt        # slots in, SSA out
    for level in (0, 2):
        _ptxas(ptx.emit(bir, b.EmitOpts(opt_level=level)).text, tmp_path)


def test_slot_form_matches_the_reference_conventions(ptx):
    # crates/basalt-sema/src/lower.rs:882-898, 992-1063: parameter i is spilled to `ptr.param` cell
    # i*65536 in the entry block; locals take the following cells in `ptr.local`; an index is
    # widened with sext and scaled by the element size before the pointer add.
    bir = b.compile_cuda(kc.load("vector_add_f32"))
    assert "func @vector_add(ptr.global, ptr.global, ptr.global, i32) -> void" in bir
    for i in range(4):
        assert f"const.i ptr.param {i * 65536}\n" in bir
    assert "store i32 ptr.param" in bir and "const.i ptr.local 262144" in bir
    assert "sext i64 i32" in bir and "const.i i64 4" in bir and "fadd f32" in bir
    assert "launch_bounds" not in bir and "shared_mem_bytes 0" in bir
    helper = b.compile_cuda(kc.load("chain_vector"))
    assert helper.count("host func @") == 3 and "call i32 @plus_one" in helper      # __device__ -> `host func`


LAUNCHES = [(1000, 1024), (1003, 1024), (7, 8), (0, 4), (100, 40), (33, 33)]


@pytest.mark.parametrize("name, kernel, twin", [("vadd_i32", "vadd_i32", "vadd_i32"), ("vector_add_f32", "vector_add", "vector_add_f32"),
                                                ("chain_vector", "chain_vector", "chain_vector"), ("square_vector", "square_vector", "square_vector")])
def test_elementwise_sources_match_their_bir_twins(ptx, name, kernel, twin):
    bir, opt = _both(ptx, kc.load(name))
    assert "load v4" in opt and "call" not in opt and f"@{kernel}__coarse" in opt     # the vectoriser recognises front-end output
    reference = kb.load(twin)
    rng = np.random.default_rng(23)
    nin = 2 if "add" in name else 1
    for n, threads in LAUNCHES:
        size = max(n, 1) + 8
        if name == "vector_add_f32":
            ins = [rng.uniform(-1e3, 1e3, size).astype(np.float32) for _ in range(nin)]
            poison = np.full(size, -1.0, np.float32)
        else:
            ins = [rng.integers(-2**30, 2**30, size, dtype=np.int64).astype(np.int32) for _ in range(nin)]
            poison = np.full(size, 0x7fffffff, np.int32)
        outs = []
        for text in (reference, bir, opt):
            o = poison.copy()
            run_kernel(text, kernel, ins + [o, n], threads)
            outs.append(o)
        assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32)), (n, threads)
        assert np.array_equal(outs[0].view(np.uint32), outs[2].view(np.uint32)), (n, threads)


def test_reference_fixture_values(ptx, orc):
    # The known answers of the reference's example drivers, through sources written for this repo:
    # chain_vector -2x+1 (examples/cpu_launch_device_helper_chain.c:18-35), square_vector x*x
    # (cpu_launch_device_helper_square.c:19-36), stress 191.0 (cpu_launch_stress.c:14-47), and the
    # folded constant 20 (cpu_launch_mymathhomework.c:15-24).
    x = (np.arange(1024) - 512).astype(np.int32)
    for name, want in (("chain_vector", -2 * x + 1), ("square_vector", x * x)):
        for text in _both(ptx, kc.load(name)):
            out = np.full(1024, 0x7fffffff, np.int32)
            run_kernel(text, name, [x, out, 1024], 1024)
            assert np.array_equal(out, want)
    a = ((np.arange(20) + 1) * 0.5 - 3.0).astype(np.float32)
    for text in _both(ptx, kc.stress()):
        out = np.zeros(4, np.float32)
        run_kernel(text, "stress", [a, out, 4], 4)
        assert np.all(out == np.float32(191.0))
    want = np.zeros(4, np.float32)
    orc.orc_stress(vp(a), vp(want), ctypes.c_int32(4), ctypes.c_int64(4))
    assert np.all(want == np.float32(191.0))
    bir, opt = _both(ptx, kc.load("constant_math"))
    assert "const.i i32 20" in opt and "mul" not in opt and opt.count("const.i i32") == 1      # folded, dead temporary gone
    for text in (bir, opt):
        out = np.zeros(1, np.int32)
        run_kernel(text, "constant_math", [out], 1)
        assert out[0] == 20


def test_helper_chain_source_matches_the_oracle(ptx, orc):
    bir, opt = _both(ptx, kc.helper_chain())
    assert bir.count("host func @link") == 32 and "call" not in opt and "load v4i32" in opt
    x = np.random.default_rng(5).integers(0, 2**32, 300, dtype=np.uint64).astype(np.uint32)
    want = np.zeros(300, np.uint32)
    orc.orc_helper_chain_u32(vp(x), vp(want), ctypes.c_int32(297), ctypes.c_int64(320))
    for text in (bir, opt):
        got = np.zeros(300, np.uint32)
        run_kernel(text, "helper_chain", [x, got, 297], 320)
        assert np.array_equal(got, want)


def test_atomic_max_source_matches_the_oracle(ptx, orc):
    bir, opt = _both(ptx, kc.load("max_i32_atomic"))
    x = np.random.default_rng(3).integers(-2**31, 2**31, 777, dtype=np.int64).astype(np.int32)
    want = np.array([-2**31], np.int32)
    orc.orc_max_i32(vp(x), vp(want), ctypes.c_int32(777), ctypes.c_int64(800))
    for text in (bir, opt):
        got = np.array([-2**31], np.int32)
        run_kernel(text, "max_i32_atomic", [x, got, 777], 800)
        assert got[0] == want[0] == x.max()


def test_block_max_source_takes_the_reduction_lowering(ptx):
    # The oracle's execution model has no shuffles (crates/basalt-x86/src/oracle.rs:94-97), so this
    # kernel's values are checked on the device; here: the loop is vectorised and both butterflies
    # are fused, exactly as for the hand-authored BIR.
    bir, opt = _both(ptx, kc.load("max_i32"))
    assert "launch_bounds max_threads=256 min_blocks=8" in bir and "shared_obj" in bir and "bytes 128" in bir
    assert bir.count("shuffle.xor i32") == 10 and bir.count("select i32") >= 11
    twin = ptx.optimized_bir(kb.load("max_i32"))
    for text in (opt, twin):
        assert text.count("warp.reduce.max i32") == 2 and "shuffle" not in text
        assert text.count("load v4i32") == 5 and "atomic.max i32 ptr.global" in text and "barrier" in text


def control_flow_expected(x, n, block=256, sequential=False):
    """A restatement of basalt_b200/cu/control_flow.cu in Python integers.  `sequential` gives the
    values under the CPU oracle's launch (threads run one after another and the barrier does
    nothing, crates/basalt-x86/src/oracle.rs:7-28): a thread then sees its neighbour's staged value
    only if the neighbour ran earlier, and zero-filled storage otherwise."""
    out = {}
    m32 = 0xFFFFFFFF

    def s32(v):
        v &= m32
        return v - (1 << 32) if v >> 31 else v

    def cdiv(a, d):     # C division truncates toward zero
        q = abs(a) // abs(d)
        return q if (a >= 0) == (d > 0) else -q

    for i in range(((n + block - 1) // block) * block):
        if i >= n:
            continue
        v = int(x[i])
        j = (i // block) * block + ((i % block) + 1) % block
        nb = int(x[j]) if j < n else 0
        if sequential and not (j % block) < (i % block):
            nb = 0
        acc = 0
        for k in range(8):
            if k == 5 and v < 0:
                break
            if (k & 1) != 0 or v == 7:
                continue
            u = (v + k) & m32
            u ^= u >> 15
            u = (u * 0x85EBCA6B) & m32
            acc = s32(acc + s32(u + 3))
        steps = 0
        while steps < 3 and acc > -1000:
            acc = s32(acc - 400)
            steps += 1
        while True:
            acc = s32(acc + cdiv(nb, 4) + (nb - 4 * cdiv(nb, 4)))
            steps -= 1
            if not steps > 0:
                break
        out[i] = acc if not (acc & 1) else s32(-acc)
    return out


def test_control_flow_source(ptx):
    # One block of 256 threads under the oracle's flat launch (tid.x = t); the device test checks
    # the same source with real barriers.
    bir, opt = _both(ptx, kc.load("control_flow"))
    assert "shared_obj" in bir and "bytes 1024" in bir and "phi i1" in bir     # && and || are real control flow
    rng = np.random.default_rng(41)
    n = 200
    x = rng.integers(-50, 50, 256, dtype=np.int64).astype(np.int32)
    x[3] = 7
    want = control_flow_expected(x, n, sequential=True)
    for text in (bir, opt):
        out = np.full(256, 0x7fffffff, np.int32)
        run_kernel(text, "control_flow", [x, out, n], 256)
        for i in range(256):
            assert out[i] == (want[i] if i < n else 0x7fffffff), i


@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 384, 128)])
def test_matmul_sources_lower_to_the_same_tile_op_as_their_twins(ptx, shape, tmp_path):
    M, N, K = shape
    for source, twin, needle in ((kc.sgemm_cta128(M, N, K), kb.sgemm_cta128(M, N, K), f"mma f32 f32 row row m 128 n 128 k {K} ld {K} {N} {N} {N}"),
                                 (kc.matmul_f16(M, N, K), kb.matmul_f16(M, N, K), f"mma f16 f32 row row m 128 n 128 k {K} ld {K} {N} {N} {N} out f16"),
                                 (kc.matmul_f16(M, N, K, True), kb.matmul_f16(M, N, K, True), f"mma f16 f32 row col m 128 n 128 k {K} ld {K} {K} {N} {N} out f16")):
        bir = b.compile_cuda(source)
        assert needle in bir and needle in twin
        mine, theirs = ptx.emit(bir).text, ptx.emit(twin).text
        # same fast path, same plan (tensor maps, geometry), so the same machine code shape
        plan = lambda t: [l for l in t.splitlines() if l.startswith("//!basalt.plan")]
        assert plan(mine) == plan(theirs) and plan(mine)
        assert ("tcgen05.mma" in mine) == ("tcgen05.mma" in theirs) and ("fma.rn.f32" in mine) == ("fma.rn.f32" in theirs)
        _ptxas(mine, tmp_path)


@pytest.mark.parametrize("code, source", [
    ("E200", "__global__ void k(int *o) { o[0] = 1 @ 2; }"),
    ("E201", "__global__ void k(int *o) { o[0] = ; }"),
    ("E201", "__global__ void k(int *o) { if o[0] { } }"),
    ("E202", "__global__ void k(int *o) { /* never closed "),
    ("E300", "__global__ void k(int *o, float *p) { o = p; }"),
    ("E300", "__global__ void k(int *o) { o[0] = 1.5f % 2; }"),
    ("E300", "__device__ int f(int a) { return a; } __global__ void k(int *o) { o[0] = f(1, 2); }"),
    ("E301", "__global__ void k(int *o) { o[0] = missing; }"),
    ("E301", "__global__ void k(int *o) { o[0] = undeclared_fn(3); }"),
    ("E302", "__global__ void k(int *o) { int a = 1; int a = 2; o[0] = a; }"),
    ("E302", "__global__ void k(int *o) { } __global__ void k(int *o) { }"),
    ("E303", "__global__ int k(int *o) { return 0; }"),
    ("E303", "__global__ __device__ void k(int *o) { }"),
    ("E303", "__global__ void a(int *o) { } __global__ void k(int *o) { a(o); }"),
    ("E304", "__global__ void k(int *o) { goto done; }"),
    ("E302", "__global__ void k(int *o) { switch (o[0]) { case 1: case 1: o[0] = 2; } }"),
    ("E302", "__global__ void k(int *o) { switch (o[0]) { default: o[0] = 1; default: o[0] = 2; } }"),
    ("E300", "__global__ void k(float *o) { switch (o[0]) { case 1: o[0] = 2; } }"),
    ("E201", "__global__ void k(int *o) { switch (o[0]) { case 1: continue; } }"),
    ("E201", "__global__ void k(int *o) { case 1: o[0] = 2; }"),
    ("E304", "struct S { int a; }; __global__ void k(int *o) { }"),
    ("E304", "__global__ void k(unsigned long *o, unsigned long d) { o[0] = o[1] / d; }"),
    ("E304", "__global__ void k(float *o) { o[0] = sqrtf(o[1]); }"),
    ("E304", "__global__ void k(int *o) { o[0] = __shfl_xor_sync(0xff, o[1], 1); }"),
    ("E304", "int table[4]; __global__ void k(int *o) { }"),
    ("E308", "__global__ void k(const int *o) { o[0] = 1; }"),
    ("E308", "__global__ void k(int *o) { const int a = 1; a = 2; o[0] = a; }"),
    ("E308", "__global__ void k(const int *o) { atomicMax(o, 3); }"),
])
def test_refusals_carry_the_reference_codes(code, source):
    with pytest.raises(b.Diag) as e:
        b.compile_cuda(source)
    assert e.value.code == code, (e.value.code, e.value.arg)


def test_cli_accepts_cuda_sources(tmp_path):
    import basalt_b200.build as build
    exe = build.CLI
    out = subprocess.run([exe, "--emit-bir", kc.path("vadd_i32")], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout == b.compile_cuda(kc.load("vadd_i32"))
    out = subprocess.run([exe, "--nvidia-ptx", kc.path("vadd_i32")], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout == b.Ptx().emit(b.compile_cuda(kc.load("vadd_i32"))).text
    bad = tmp_path / "bad.cu"
    bad.write_text("__global__ void k(int *o) { o[0] = nope; }\n")
    out = subprocess.run([exe, "--nvidia-ptx", str(bad)], capture_output=True, text=True)
    assert out.returncode == 1 and out.stderr.startswith("E301: ")


@pytest.mark.skipif(not os.environ.get("BASALT_REFERENCE_TREE") or not os.path.isdir(REFERENCE_KERNELS), reason="BASALT_REFERENCE_TREE does not name a checkout of the reference")
def test_the_reference_tree_kernels_compile_and_give_their_known_answers(ptx):
    """The reference's own device sources (tests/kernels/*.cu), read where they lie, through this
    front end, with the inputs and answers of the matching examples/cpu_launch_*.c drivers."""
    def src(name):
        with open(os.path.join(REFERENCE_KERNELS, name)) as f:
            return f.read()
    a = np.arange(1024, dtype=np.float32)
    for text in _both(ptx, src("vector_add.cu")):
        c = np.full(1024, -1.0, np.float32)
        run_kernel(text, "vector_add", [a, 2 * a, c, 1024], 1024)
        assert np.array_equal(c, 3 * a)
    x = (np.arange(1024) - 512).astype(np.int32)
    for file, kernel, want in (("device_helper_chain.cu", "chain_vector", -2 * x + 1), ("device_helper_square.cu", "square_vector", x * x)):
        for text in _both(ptx, src(file)):
            out = np.full(1024, 0x7fffffff, np.int32)
            run_kernel(text, kernel, [x, out, 1024], 1024)
            assert np.array_equal(out, want)
    s = ((np.arange(20) + 1) * 0.5 - 3.0).astype(np.float32)
    for text in _both(ptx, src("stress.cu")):
        out = np.zeros(2, np.float32)
        run_kernel(text, "stress", [s, out, 2], 2)
        assert np.all(out == np.float32(191.0))
    for text in _both(ptx, src("mymathhomework.cu")):
        out = np.zeros(1, np.int32)
        run_kernel(text, "mymathhomework", [out], 1)
        assert out[0] == 20
    with pytest.raises(b.Diag):
        b.compile_cuda(src("deliberate_errors.cu"))


def test_loop_invariants_move_to_the_preheader(ptx):
    # crates/basalt-passes/src/licm.rs: a pure computation on values that do not change in the loop is
    # done once, before it; a division is left in place (it could trap where the loop would have skipped it).
    src = """
__global__ void weighted(const int *x, int *out, int n, int a, int b) {
    int acc = 0;
    for (int i = 0; i < n; i++) {
        int scale = a * b + 7;
        int risky = (x[i] != 0) ? a / b : 0;
        acc += x[i] * scale + risky;
    }
    out[0] = acc;
}
"""
    bir = b.compile_cuda(src)
    opt = ptx.optimized_bir(bir)
    blocks = opt.split("\n  bb")
    entry = blocks[1]
    assert "mul i32 %arg3, %arg4" in entry and "const.i i32 7" in entry            # hoisted into the block before the loop
    assert "div i32" in opt and "div i32" not in entry                              # the division stays guarded inside the loop
    x = np.array([3, 0, -2, 5, 0, 1], np.int32)
    for n in (0, 1, 6):
        o0, o1 = np.zeros(1, np.int32), np.zeros(1, np.int32)
        run_kernel(bir, "weighted", [x, o0, n, 6, 4], 1)
        run_kernel(opt, "weighted", [x, o1, n, 6, 4], 1)
        want = sum(int(v) * (6 * 4 + 7) + (1 if v else 0) for v in x[:n])
        assert o0[0] == o1[0] == want, n
    # b = 0 with an all-zero input: the division must not run at all
    z = np.zeros(4, np.int32)
    o = np.zeros(1, np.int32)
    run_kernel(opt, "weighted", [z, o, 4, 6, 0], 1)
    assert o[0] == 0


def switch_cases_expected(x):
    """basalt_b200/cu/switch_cases.cu restated in Python integers (C division and remainder truncate toward zero)."""
    out = []
    for v in map(int, x):
        r = int(np.fmod(v, 6))
        if r == 0: acc = 100
        elif r == 1: acc = 17              # 10, then falls through into `acc += 7`
        elif r == 2: acc = 7
        elif r == 4: acc = 0
        elif r == 5: acc = int(v / 6) - 1
        else: acc = -3                     # default, then falls through into `acc *= 3`
        for k in range(4):
            if k == 1: continue
            acc += 1000 if k == 2 else k
            acc += 1
        out.append(acc)
    return np.array(out, np.int32)


def test_switch_source(ptx):
    # labels open blocks the code above falls into, `break` leaves the switch, `continue` the enclosing loop's body
    bir, opt = _both(ptx, kc.load("switch_cases"))
    assert "switch %" in bir and "default bb" in bir
    n = 200
    x = (np.arange(n) * 37 % 101 - 50).astype(np.int32)
    for text in (bir, opt):
        out = np.zeros(n, np.int32)
        run_kernel(text, "switch_cases", [x, out, n], n)
        assert np.array_equal(out, switch_cases_expected(x))


def test_function_like_macros():
    # arguments are expanded as they are read, a macro may use earlier ones, `NAME (` with a space is still a call,
    # an empty parameter list takes an empty argument list
    src = """
#define N 16
#define IDX(i, j) ((i) * N + (j))
#define SQ(x) ((x) * (x))
#define CLAMP(v, lo, hi) ((v) < (lo) ? (lo) : ((v) > (hi) ? (hi) : (v)))
#define TWICE(e) (SQ(e) + SQ(e))
#define ZERO() 0
__global__ void k(const int *in, int *out, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int r = i / N, c = i % N;
    int v = in[IDX(r, c)];
    out[IDX(r, c)] = CLAMP(TWICE(v + 1), ZERO(), 500) + SQ(c) - IDX (1, 2);
}
"""
    bir = b.compile_cuda(src)
    n = 256
    x = (np.arange(n) % 23 - 11).astype(np.int32); out = np.zeros(n, np.int32)
    run_kernel(bir, "k", [x, out, n], n)
    c = np.arange(n) % 16
    assert np.array_equal(out, np.clip(2 * (x + 1) ** 2, 0, 500) + c * c - 18)
    for bad, code in (("#define F(a, b) ((a)+(b))\n__global__ void k(int*o){ o[0]=F(1); }", "E300"),
                      ("#define F(a,...) (a)\n__global__ void k(int*o){ o[0]=F(1); }", "E304"),
                      ("#define F(a) ((a)\n__global__ void k(int*o){ o[0]=F(1; }", "E202")):
        with pytest.raises(b.Diag) as e:
            b.compile_cuda(bad)
        assert e.value.code == code, e.value


def test_unsigned_division_goes_through_64_bits():
    # BIR division is signed: a 32-bit unsigned divide is done on the zero-extended operands in 64 bits,
    # a power-of-two constant divisor stays a shift or a mask, a 64-bit unsigned divide is refused
    src = """
__global__ void k(const unsigned *a, const unsigned *d, unsigned *q, unsigned *r, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    q[i] = a[i] / d[i] + a[i] / 7u;
    r[i] = a[i] % d[i] + a[i] % 10u + (a[i] / 8u) + (a[i] % 16u);
}
"""
    bir = b.compile_cuda(src)
    assert bir.count(" div i64 ") == 2 and bir.count(" rem i64 ") == 2 and " lshr i32 " in bir
    n = 512
    rng = np.random.default_rng(1)
    a = rng.integers(0, 2**32, n, dtype=np.uint64).astype(np.uint32); d = rng.integers(1, 2**32, n, dtype=np.uint64).astype(np.uint32)
    a[:4] = [0, 2**32 - 1, 2**31, 2**31 - 1]; d[:4] = [2**32 - 1, 1, 3, 2**31]
    q = np.zeros(n, np.uint32); r = np.zeros(n, np.uint32)
    run_kernel(bir, "k", [a, d, q, r, n], n)
    assert np.array_equal(q, (a // d + a // 7).astype(np.uint32)) and np.array_equal(r, (a % d + a % 10 + a // 8 + a % 16).astype(np.uint32))
    with pytest.raises(b.Diag) as e:
        b.compile_cuda("__global__ void k(unsigned long *o) { o[0] = o[1] / 3ul; }")
    assert e.value.code == "E304"


def test_conditional_groups():
    # #ifdef / #ifndef / #if / #elif / #else / #endif / #undef: untaken groups are skipped as text (they need not lex)
    src = """
#ifndef SCALE
#define SCALE 3
#endif
#define FAST 1
#ifdef NEVER
this is not C at all @@@
#elif 0
#define OFFSET 99
#else
#define OFFSET 10
#endif
#if FAST
#define STEP(x) ((x) * SCALE)
#else
#define STEP(x) (x)
#endif
#if !defined(OFFSET)
#error no offset
#endif
#undef FAST
#ifdef FAST
#define OFFSET2 1000
#else
#define OFFSET2 0
#endif
__global__ void k(const int *in, int *out, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = STEP(in[i]) + OFFSET + OFFSET2;
}
"""
    bir = b.compile_cuda(src)
    n = 64
    x = np.arange(n, dtype=np.int32); out = np.zeros(n, np.int32)
    run_kernel(bir, "k", [x, out, n], n)
    assert np.array_equal(out, x * 3 + 10)
    for bad, code in (("#ifdef A\n__global__ void k(int*o){}\n", "E202"), ("#endif\n__global__ void k(int*o){}", "E201"),
                      ("#if 1+1\n#endif\n__global__ void k(int*o){}", "E304"), ("#if defined(A) && 0\n#endif\n__global__ void k(int*o){}", "E304"),
                      ("#ifndef A\n#error A is required\n#endif\n__global__ void k(int*o){}", "E304")):
        with pytest.raises(b.Diag) as e:
            b.compile_cuda(bad)
        assert e.value.code == code, e.value
