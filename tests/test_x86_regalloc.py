"""The restatement of the reference's register-allocating x86-64 CPU back end (oracle/x86_regalloc.cpp,
test infrastructure; the timed CPU baseline of the benchmark): pinned to the known answers of the
reference's own tests of that back end (crates/basalt-x86/tests/link_and_run_regalloc.rs, pressure.rs),
to its refusal surface (crates/basalt-x86/src/regalloc.rs:132-207, 1516-1745), and compared with the two
independent CPU oracles (C loops and the BIR interpreter) on the workloads and on generated kernels."""
import ctypes

import numpy as np
import pytest

from _util import vp
from basalt_b200 import EmitOpts, kernels_bir as kb, kernels_cu as kc, workloads as w
from oracle import x86_regalloc as x86
from oracle.bir_interp import run_kernel

i32, i64 = ctypes.c_int32, ctypes.c_int64


def module(body: str, target="i32") -> str:
    return f"module {{\n  shared_mem_bytes 0\n  target_dtypes {target}\n\n{body}}}\n"


ADD_I32 = module("""  func @add_i32(i32, i32) -> i32 {
  bb0:
    %0 = add i32 %arg0, %arg1
    ret %0
  }
""")

SPILL_HEAVY_SUM = module("""  func @spill_heavy_sum(i32, i32, i32, i32, i32) -> i32 {
  bb0:
    %0 = add i32 %arg0, %arg1
    %1 = add i32 %0, %arg2
    %2 = add i32 %1, %arg3
    %3 = add i32 %2, %arg4
    ret %3
  }
""")

MAX_VIA_PHI = module("""  func @max_i32(i32, i32) -> i32 {
  bb0:
    %0 = icmp sgt i32 %arg0, %arg1
    condbr %0, bb1, bb2
  bb1:
    br bb3
  bb2:
    br bb3
  bb3:
    %1 = phi i32 [bb1 -> %arg0, bb2 -> %arg1]
    ret %1
  }
""")


@pytest.fixture(scope="module", autouse=True)
def _built(orc):
    return orc


def test_add_i32_known_answers():
    # examples/cpu_launch_add_i32.c:27-31: the sum does not depend on how many threads recompute it
    k = x86.compile(ADD_I32)
    assert (k.params, k.ret, k.int_spills) == (["i32", "i32"], "i32", 0)
    for a, b, nthreads, want in ((3, 4, 1, 7), (3, 4, 1000, 7), (-5, 10, 1, 5), (-1, -1, 1, -2)):
        assert k(a, b, nthreads) == want


def test_spill_heavy_sum_known_answers():
    # link_and_run_regalloc.rs:187-236: five parameters live at once against four registers, so at
    # least two values spill; examples/cpu_launch_spill_heavy_sum.c:14: the plain sum
    k = x86.compile(SPILL_HEAVY_SUM)
    assert k.int_spills >= 2
    for args in ((1, 2, 3, 4, 5), (-7, 100, 0, 2**31 - 1, -2**31), (10, -20, 30, -40, 50)):
        want = int(np.sum(np.array(args, np.int64)).astype(np.int32))
        for nthreads in (1, 17):
            assert k(*args, nthreads) == want


def test_max_via_phi_known_answers():
    # link_and_run_regalloc.rs:266-321, examples/cpu_launch_max_i32.c:12: a phi resolved in the predecessors
    k = x86.compile(MAX_VIA_PHI)
    for a, b in ((1, 2), (2, 1), (-3, -3), (-2**31, 2**31 - 1), (7, -7)):
        assert k(a, b, 1) == max(a, b)
        assert k(a, b, 5) == max(a, b)


def test_vector_add_known_answer():
    # link_and_run_regalloc.rs:90-130 with examples/cpu_launch_vadd.c:18-37: a[i]=i, b[i]=2i, c=-1, N=1024
    n = 1024
    a = np.arange(n, dtype=np.float32); b = (2 * np.arange(n)).astype(np.float32)
    c = np.full(n, -1.0, np.float32)
    k = x86.compile(kb.load("vector_add_f32"))
    k(a, b, c, n, n)
    assert np.array_equal(c, a + b)


def test_stress_is_191_and_spills(orc):
    # pressure.rs:196-274: stress gives the oracle's answer (191.0, tests/diff/golden/stress.txt) through
    # the register allocator; eighteen live temporaries against five xmm registers must spill
    a = ((np.arange(20) + 1) * 0.5 - 3.0).astype(np.float32)
    out = np.array([-1.0], np.float32)
    k = x86.compile(kb.stress())
    k(a, out, 1, 1)
    assert out[0] == np.float32(191.0)
    assert k.float_spills > 0


def test_stress_from_cuda_c_source_in_slot_form():
    # the front end's slot-form output is what the reference's emit receives: construct_ssa runs first
    # (regalloc.rs:110-116)
    from basalt_b200 import compile_cuda
    a = ((np.arange(20) + 1) * 0.5 - 3.0).astype(np.float32)
    out = np.array([-1.0], np.float32)
    k = x86.compile(compile_cuda(kc.stress()))
    k(a, out, 1, 1)
    assert out[0] == np.float32(191.0)


@pytest.mark.parametrize("text,code", [
    (module("""  func @k(i32) -> i32 {
  bb0:
    %0 = const.i i32 1
    %1 = shuffle.xor i32 %arg0, %0
    ret %1
  }
"""), "E090"),
    (module("""  func @k(i32) -> i32 {
  bb0:
    %0 = icmp ne i32 %arg0, %arg0
    %1 = ballot i32 %0
    ret %1
  }
"""), "E090"),
    (module("""  func @k(f16) -> void {
  bb0:
    ret
  }
""", "f16"), "E091"),
    (module("""  func @k(ptr.global) -> void {
  bb0:
    %0 = load f16 ptr.global %arg0, align 2
    ret
  }
""", "f16"), "E091"),
    (module("""  func @k(ptr.global) -> void {
  bb0:
    %0 = load v4i32 ptr.global %arg0, align 16
    ret
  }
"""), "E091"),
    (module("""  host func @k(i32) -> i32 {
  bb0:
    ret %arg0
  }
"""), "E093"),
    (module("""  func @a() -> void {
  bb0:
    ret
  }

  func @b() -> void {
  bb0:
    ret
  }
"""), "E093"),
    # six integer parameters leave no integer register for the trailing nthreads (regalloc.rs:1719-1736)
    (module("""  func @k(i32, i32, i32, i32, i32, i32) -> void {
  bb0:
    ret
  }
"""), "E093"),
])
def test_refusals(text, code):
    with pytest.raises(x86.Refused) as e:
        x86.compile(text)
    assert e.value.code == code


def test_refuses_calls_and_mma():
    for name in ("chain_vector", "mma2x2"):
        with pytest.raises(x86.Refused) as e:
            x86.compile(kb.load(name))
        assert e.value.code in ("E090", "E093")      # a helper makes the module multi-function first


def test_emit_is_deterministic():
    # regalloc.rs:1821-1838
    for text in (SPILL_HEAVY_SUM, MAX_VIA_PHI, kb.stress(), kb.load("vadd_i32")):
        assert x86.compile(text).code == x86.compile(text).code


def test_vadd_i32_matches_c_oracle(orc):
    n = 10007
    a = w.u32(w.SEEDS["vadd_i32"], 2 * n).view(np.int32)
    x, y = a[:n].copy(), a[n:].copy()
    want = np.zeros(n, np.int32); got = np.full(n + 5, 77, np.int32)
    orc.orc_vadd_i32(vp(x), vp(y), vp(want), i32(n), i64(n))
    x86.compile(kb.load("vadd_i32"))(x, y, got, n, n)
    assert np.array_equal(got[:n], want) and np.all(got[n:] == 77)
    # an under-sized launch touches only its own threads' elements
    got2 = np.full(n, 77, np.int32)
    x86.compile(kb.load("vadd_i32"))(x, y, got2, n, 1000)
    assert np.array_equal(got2[:1000], want[:1000]) and np.all(got2[1000:] == 77)


def test_max_i32_atomic_matches_c_oracle(orc):
    # the CPU-runnable form of the reduction (warp shuffles are refused): one atomic max per element
    k = x86.compile(kb.load("max_i32_atomic"))
    for n in (1, 31, 4096, 100003):
        x = w.u32(w.SEEDS["max_i32"], n).view(np.int32)
        want = np.array([-2**31], np.int32); got = np.array([-2**31], np.int32)
        orc.orc_max_i32(vp(x), vp(want), i32(n), i64(n))
        k(x, got, n, n)
        assert got[0] == want[0] == x.max()


def test_helper_chain_after_inlining_matches_c_oracle(orc, ptx):
    # calls are refused, so the chain reaches this back end inlined (the library's inliner at level 0)
    n = 5000
    x = w.u32(w.SEEDS["helper_chain"], n)
    inlined = ptx.optimized_bir(kb.helper_chain(), EmitOpts(opt_level=0))
    want = np.zeros(n, np.uint32); got = np.zeros(n, np.uint32)
    orc.orc_helper_chain_u32(vp(x), vp(want), i32(n), i64(n))
    x86.compile(inlined)(x, got, n, n)
    assert np.array_equal(got, want)


def test_cuda_c_sources_match_interpreter(ptx):
    # kernels with loops, nested branches, shared cells and helper calls, compiled from CUDA-C source and
    # inlined (this back end refuses `call`): the JIT against the BIR interpreter under the same launch model
    from basalt_b200 import compile_cuda
    n, nthreads = 200, 256      # one block of 256 threads, as control_flow's shared array expects
    x = (np.arange(nthreads) * 37 % 101 - 50).astype(np.int32)
    for name in ("control_flow", "constant_math", "square_vector", "chain_vector", "vadd_i32", "max_i32_atomic"):
        bir = ptx.optimized_bir(compile_cuda(kc.load(name)), EmitOpts(opt_level=0))
        k = x86.compile(bir)
        ins = [x.copy() if p.startswith("ptr") else n for p in k.params]
        ins2 = [a.copy() if isinstance(a, np.ndarray) else a for a in ins]
        k(*ins, nthreads)
        run_kernel(bir, k.name, ins2, nthreads)
        for a, b in zip(ins, ins2):
            if isinstance(a, np.ndarray):
                assert np.array_equal(a, b), name


import _opkernels as ops


@pytest.mark.parametrize("ty", ops.INT_TYPES)
def test_integer_binops_match_interpreter(ty):
    n = 300
    for op in ops.INT_BINOPS:
        a, bb = ops.int_inputs(ty, op, n)
        got = np.zeros(n, ops.NP[ty]); want = np.zeros(n, ops.NP[ty])
        text = ops.binop_kernel(ty, op)
        x86.compile(text)(a, bb, got, n)
        run_kernel(text, "k", [a, bb, want], n)
        assert np.array_equal(got, want), (ty, op)


@pytest.mark.parametrize("ty", ops.INT_TYPES + ("f32", "f64"))
def test_compares_and_select_match_interpreter(ty):
    n = 200
    a, bb = ops.float_inputs(ty, n) if ty.startswith("f") else ops.int_inputs(ty, "add", n)
    if not ty.startswith("f"):
        bb[8:12] = a[8:12]
    for pred in (ops.FCMP_PREDS if ty.startswith("f") else ops.ICMP_PREDS):
        got = np.zeros(n, np.int32); want = np.zeros(n, np.int32)
        text = ops.compare_kernel(ty, pred)
        x86.compile(text)(a, bb, got, n)
        run_kernel(text, "k", [a, bb, want], n)
        assert np.array_equal(got, want), (ty, pred)
    got = np.zeros(n, ops.NP[ty]); want = np.zeros(n, ops.NP[ty])
    text = ops.select_kernel(ty)
    x86.compile(text)(a, bb, got, n)
    run_kernel(text, "k", [a, bb, want], n)
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), ty


@pytest.mark.parametrize("ty", ("f32", "f64"))
def test_float_binops_match_interpreter(ty):
    n = 200
    a, bb = ops.float_inputs(ty, n)
    for op in ops.FLOAT_BINOPS:
        got = np.zeros(n, ops.NP[ty]); want = np.zeros(n, ops.NP[ty])
        text = ops.binop_kernel(ty, op)
        x86.compile(text)(a, bb, got, n)
        run_kernel(text, "k", [a, bb, want], n)
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (ty, op)


@pytest.mark.parametrize("op,src,dst", ops.CASTS)
def test_casts_match_interpreter(op, src, dst):
    n = 128
    a = ops.cast_inputs(op, src, dst, n)
    text = ops.cast_kernel(op, src, dst)
    got = np.zeros(n, ops.NP[dst]); want = np.zeros(n, ops.NP[dst])
    x86.compile(text)(a, got, n)
    run_kernel(text, "k", [a, want], n)
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (op, src, dst)


def test_loop_with_two_swapping_phis():
    # two phis of one block that read each other: the staging slots keep the copies parallel (regalloc.rs:47-58)
    text = module("""  func @k(ptr.global, i32) -> void {
  bb0:
    %0 = const.i i32 0
    %1 = const.i i32 1
    br bb1
  bb1:
    %2 = phi i32 [bb0 -> %0, bb2 -> %3]
    %3 = phi i32 [bb0 -> %1, bb2 -> %2]
    %4 = phi i32 [bb0 -> %0, bb2 -> %7]
    %5 = icmp slt i32 %4, %arg1
    condbr %5, bb2, bb3
  bb2:
    %6 = const.i i32 1
    %7 = add i32 %4, %6
    br bb1
  bb3:
    %8 = const.i i32 10
    %9 = mul i32 %2, %8
    %10 = add i32 %9, %3
    store i32 ptr.global %arg0, %10, align 4
    ret
  }
""")
    k = x86.compile(text)
    for trips, want in ((0, 1), (1, 10), (2, 1), (5, 10)):
        out = np.zeros(1, np.int32); ref = np.zeros(1, np.int32)
        k(out, trips, 1)
        run_kernel(text, "k", [ref, trips], 1)
        assert out[0] == ref[0] == want


def test_select_switch_atomics_and_cas():
    text = module("""  func @k(ptr.global, ptr.global) -> void {
  bb0:
    %0 = tid.x i32
    %1 = const.i i32 3
    %2 = rem i32 %0, %1
    switch %2, default bb3 [0 -> bb1, 1 -> bb2]
  bb1:
    %3 = atomic.add i32 ptr.global %arg0, %0
    br bb4
  bb2:
    %4 = const.i i64 4
    %5 = add ptr.global %arg0, %4
    %6 = atomic.min i32 ptr.global %5, %0
    br bb4
  bb3:
    %7 = const.i i64 8
    %8 = add ptr.global %arg0, %7
    %9 = const.i i32 0
    %10 = atomic.cas i32 ptr.global %8, %9, %0
    br bb4
  bb4:
    %11 = const.i i32 7
    %12 = icmp sgt i32 %0, %11
    %13 = const.i i32 100
    %14 = select i32 %12, %13, %0
    %15 = sext i64 i32 %0
    %16 = const.i i64 4
    %17 = mul i64 %15, %16
    %18 = add ptr.global %arg1, %17
    store i32 ptr.global %18, %14, align 4
    ret
  }
""")
    n = 20
    cells = np.array([0, 1000, 0], np.int32); out = np.zeros(n, np.int32)
    cells2 = cells.copy(); out2 = out.copy()
    x86.compile(text)(cells, out, n)
    run_kernel(text, "k", [cells2, out2], n)
    assert np.array_equal(cells, cells2) and np.array_equal(out, out2)
    assert list(cells) == [sum(range(0, n, 3)), 1, 2]


def test_shared_array_cell_has_its_declared_size():
    # a shared array sized by `shared_obj` lives in the frame and persists across the threads of one launch
    text = """module {
  shared_mem_bytes 0
  target_dtypes i32
  shared_obj 65536 bytes 256 align 16

  func @k(ptr.global) -> void {
  bb0:
    %0 = tid.x i64
    %1 = const.i i64 4
    %2 = mul i64 %0, %1
    %3 = const.i ptr.shared 65536
    %4 = add ptr.shared %3, %2
    %5 = trunc i32 i64 %0
    store i32 ptr.shared %4, %5, align 4
    %7 = const.i i64 63
    %8 = icmp eq i64 %0, %7
    condbr %8, bb1, bb2
  bb1:
    %9 = const.i i64 40
    %10 = add ptr.shared %3, %9
    %11 = load i32 ptr.shared %10, align 4
    store i32 ptr.global %arg0, %11, align 4
    br bb2
  bb2:
    ret
  }
}
"""
    out = np.zeros(1, np.int32)
    x86.compile(text)(out, 64)
    assert out[0] == 10
