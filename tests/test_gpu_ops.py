"""Per-op parity of the PTX lowering (arithmetic, shifts, division, compares, select, casts at every
width) against the CPU oracle: each op runs as a one-instruction kernel on the device through the
reference's CPU launch ABI and through the BIR interpreter on the same seeded inputs, and the bytes
must match.  Both optimisation levels: level 0 lowers one to one, level 2 vectorises these kernels.
Inputs stay inside the domain where the source languages define the result (shift counts below the
width, no division by zero, float -> integer in range): outside it PTX and x86 differ by design."""
import numpy as np
import pytest

import _opkernels as ops
from _gpu import emitted
from oracle.bir_interp import run_kernel

pytestmark = pytest.mark.gpu
LEVELS = [0, 2]
N = 1024          # four blocks of 256 threads


def both(gpu, text, arrays, level):
    dev = [a.copy() for a in arrays]
    cpu = [a.copy() for a in arrays]
    gpu.cpu_launch(emitted(gpu, text, "k", level), dev, N)
    run_kernel(text, "k", cpu, N)
    return dev[-1], cpu[-1]


@pytest.mark.parametrize("level", LEVELS)
@pytest.mark.parametrize("ty", ops.INT_TYPES)
def test_integer_binops(gpu, ty, level):
    for op in ops.INT_BINOPS:
        a, b = ops.int_inputs(ty, op, N)
        got, want = both(gpu, ops.binop_kernel(ty, op), [a, b, np.zeros(N, ops.NP[ty])], level)
        bad = np.flatnonzero(got != want)
        assert len(bad) == 0, (ty, op, level, int(a[bad[0]]), int(b[bad[0]]), int(got[bad[0]]), int(want[bad[0]]))


@pytest.mark.parametrize("level", LEVELS)
@pytest.mark.parametrize("ty", ("f32", "f64"))
def test_float_binops(gpu, ty, level):
    a, b = ops.float_inputs(ty, N)
    for op in ops.FLOAT_BINOPS:
        got, want = both(gpu, ops.binop_kernel(ty, op), [a, b, np.zeros(N, ops.NP[ty])], level)
        # a NaN result may carry a different payload on the two ISAs; everything else is bit for bit
        same = (got.view(np.uint8).reshape(N, -1) == want.view(np.uint8).reshape(N, -1)).all(axis=1) | (np.isnan(got) & np.isnan(want))
        assert same.all(), (ty, op, level, np.flatnonzero(~same)[:4])


@pytest.mark.parametrize("level", LEVELS)
@pytest.mark.parametrize("ty", ops.INT_TYPES + ("f32", "f64"))
def test_compares_and_select(gpu, ty, level):
    a, b = ops.float_inputs(ty, N) if ty.startswith("f") else ops.int_inputs(ty, "add", N)
    if not ty.startswith("f"):
        b[8:12] = a[8:12]
    for pred in (ops.FCMP_PREDS if ty.startswith("f") else ops.ICMP_PREDS):
        got, want = both(gpu, ops.compare_kernel(ty, pred), [a, b, np.zeros(N, np.int32)], level)
        assert np.array_equal(got, want), (ty, pred, level, np.flatnonzero(got != want)[:4])
    got, want = both(gpu, ops.select_kernel(ty), [a, b, np.zeros(N, ops.NP[ty])], level)
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (ty, "select", level)


@pytest.mark.parametrize("level", LEVELS)
@pytest.mark.parametrize("op,src,dst", ops.CASTS)
def test_casts(gpu, op, src, dst, level):
    a = ops.cast_inputs(op, src, dst, N)
    got, want = both(gpu, ops.cast_kernel(op, src, dst), [a, np.zeros(N, ops.NP[dst])], level)
    bad = np.flatnonzero((got.view(np.uint8).reshape(N, -1) != want.view(np.uint8).reshape(N, -1)).any(axis=1))
    assert len(bad) == 0, (op, src, dst, level, a[bad[0]], got[bad[0]], want[bad[0]])


# ---- warp collectives: the CPU back ends refuse them, so the expectation is CUDA's definition in numpy ----
def _collective_kernel(ty: str, line: str) -> str:
    sz = ops.size(ty)
    return ops.module(f"""  func @k(ptr.global, ptr.global) -> void {{
  bb0:
{ops._INDEX}    %5 = const.i i64 {sz}
    %6 = mul i64 %4, %5
    %7 = add ptr.global %arg0, %6
    %8 = load {ty} ptr.global %7, align {sz}
{line}
    %11 = add ptr.global %arg1, %6
    store {ty} ptr.global %11, %10, align {sz}
    ret
  }}
""")


@pytest.mark.parametrize("level", LEVELS)
@pytest.mark.parametrize("ty", ("i32", "f32", "i64", "f64"))
def test_shuffles(gpu, ty, level):
    rng = np.random.default_rng(3)
    a = rng.integers(-1000, 1000, N).astype(ops.NP[ty])
    warps = a.reshape(-1, 32)
    lane = np.arange(32)
    for mode, d in (("xor", 1), ("xor", 16), ("xor", 21), ("up", 1), ("up", 5), ("down", 3), ("down", 31), ("idx", 0), ("idx", 17), ("idx", 40)):
        text = _collective_kernel(ty, f"    %9 = const.i i32 {d}\n    %10 = shuffle.{mode} {ty} %8, %9")
        got = np.zeros(N, ops.NP[ty])
        dev = [a.copy(), got]
        gpu.cpu_launch(emitted(gpu, text, "k", level), dev, N)
        src = {"xor": lane ^ d, "up": np.where(lane >= d, lane - d, lane), "down": np.where(lane + d <= 31, lane + d, lane), "idx": np.full(32, d & 31)}[mode]
        assert np.array_equal(dev[1].reshape(-1, 32), warps[:, src]), (ty, mode, d, level)


@pytest.mark.parametrize("level", LEVELS)
def test_ballot_and_votes(gpu, level):
    rng = np.random.default_rng(5)
    a = rng.integers(-3, 4, N).astype(np.int32)
    a[32:64] = 5          # a warp where every lane votes yes
    a[64:96] = -5         # and one where none does
    pred = (a > 0).reshape(-1, 32)
    want = {"ballot": (pred * (1 << np.arange(32, dtype=np.uint64))).sum(axis=1).astype(np.uint32).view(np.int32),
            "vote.any": pred.any(axis=1).astype(np.int32), "vote.all": pred.all(axis=1).astype(np.int32)}
    for op in ("ballot", "vote.any", "vote.all"):
        text = ops.module(f"""  func @k(ptr.global, ptr.global) -> void {{
  bb0:
{ops._INDEX}    %5 = const.i i64 4
    %6 = mul i64 %4, %5
    %7 = add ptr.global %arg0, %6
    %8 = load i32 ptr.global %7, align 4
    %9 = const.i i32 0
    %10 = icmp sgt i32 %8, %9
    %11 = {op} i32 %10
    %12 = add ptr.global %arg1, %6
    store i32 ptr.global %12, %11, align 4
    ret
  }}
""")
        dev = [a.copy(), np.zeros(N, np.int32)]
        gpu.cpu_launch(emitted(gpu, text, "k", level), dev, N)
        assert np.array_equal(dev[1].reshape(-1, 32), np.repeat(want[op][:, None], 32, axis=1)), (op, level)


# ---- atomics: order-independent ops on one cell against the sequential oracle; exch / cas on private cells ----
@pytest.mark.parametrize("level", LEVELS)
@pytest.mark.parametrize("ty", ("i32", "i64"))
def test_integer_atomics_on_one_cell(gpu, ty, level):
    rng = np.random.default_rng(9)
    sz = ops.size(ty)
    a = rng.integers(-2**20, 2**20, N).astype(ops.NP[ty])
    for op, start in (("add", 5), ("sub", 5), ("min", 2**30), ("max", -2**30), ("and", -1), ("or", 0), ("xor", 0)):
        text = ops.module(f"""  func @k(ptr.global, ptr.global) -> void {{
  bb0:
{ops._INDEX}    %5 = const.i i64 {sz}
    %6 = mul i64 %4, %5
    %7 = add ptr.global %arg0, %6
    %8 = load {ty} ptr.global %7, align {sz}
    %9 = atomic.{op} {ty} ptr.global %arg1, %8
    ret
  }}
""")
        got, want = both(gpu, text, [a, np.array([start], ops.NP[ty])], level)
        assert got[0] == want[0], (ty, op, level, int(got[0]), int(want[0]))


@pytest.mark.parametrize("level", LEVELS)
def test_float_atomic_add_exch_and_cas(gpu, level):
    a = (np.arange(N) % 7).astype(np.float32)          # small integers: the sum is exact in any order
    text = ops.module(f"""  func @k(ptr.global, ptr.global) -> void {{
  bb0:
{ops._INDEX}    %5 = const.i i64 4
    %6 = mul i64 %4, %5
    %7 = add ptr.global %arg0, %6
    %8 = load f32 ptr.global %7, align 4
    %9 = atomic.add f32 ptr.global %arg1, %8
    ret
  }}
""", "f32")
    got, want = both(gpu, text, [a, np.array([1.0], np.float32)], level)
    assert got[0] == want[0] == 1.0 + a.sum()
    # exch and cas on the thread's own cell: old values come back, new ones land
    cells = np.arange(N, dtype=np.int32)
    text = ops.module(f"""  func @k(ptr.global, ptr.global, ptr.global) -> void {{
  bb0:
{ops._INDEX}    %5 = const.i i64 4
    %6 = mul i64 %4, %5
    %7 = add ptr.global %arg0, %6
    %8 = trunc i32 i64 %4
    %9 = const.i i32 100
    %10 = add i32 %8, %9
    %11 = atomic.exch i32 ptr.global %7, %10
    %12 = atomic.cas i32 ptr.global %7, %10, %11
    %13 = const.i i32 1
    %14 = add i32 %8, %13
    %15 = atomic.cas i32 ptr.global %7, %14, %9
    %16 = add i32 %12, %15
    %17 = add ptr.global %arg1, %6
    store i32 ptr.global %17, %16, align 4
    ret
  }}
""")
    dev = [cells.copy(), np.zeros(N, np.int32), np.zeros(1, np.int32)]
    cpu = [cells.copy(), np.zeros(N, np.int32), np.zeros(1, np.int32)]
    gpu.cpu_launch(emitted(gpu, text, "k", level), dev, N)
    run_kernel(text, "k", cpu, N)
    # exch stores i+100 and returns i; the first cas sees i+100 and restores i; the second expects i+1, sees i, fails
    assert np.array_equal(dev[0], cells) and np.array_equal(dev[1], cells + 100 + cells)
    assert np.array_equal(dev[0], cpu[0]) and np.array_equal(dev[1], cpu[1])


# ---- control flow: phis that read each other, a switch, a data-dependent loop ----
SWAPPING_PHIS = ops.module("""  func @k(ptr.global, ptr.global) -> void {
  bb0:
    %0 = bid.x i64
    %1 = bdim.x i64
    %2 = mul i64 %0, %1
    %3 = tid.x i64
    %4 = add i64 %2, %3
    %5 = const.i i64 4
    %6 = mul i64 %4, %5
    %7 = add ptr.global %arg0, %6
    %8 = load i32 ptr.global %7, align 4
    %9 = const.i i32 0
    %10 = const.i i32 1
    br bb1
  bb1:
    %11 = phi i32 [bb0 -> %9, bb2 -> %12]
    %12 = phi i32 [bb0 -> %10, bb2 -> %11]
    %13 = phi i32 [bb0 -> %9, bb2 -> %16]
    %14 = icmp slt i32 %13, %8
    condbr %14, bb2, bb3
  bb2:
    %15 = const.i i32 1
    %16 = add i32 %13, %15
    br bb1
  bb3:
    %17 = const.i i32 10
    %18 = mul i32 %11, %17
    %19 = add i32 %18, %12
    %20 = add ptr.global %arg1, %6
    store i32 ptr.global %20, %19, align 4
    ret
  }
""")

SWITCH_AND_LOOP = ops.module("""  func @k(ptr.global, ptr.global) -> void {
  bb0:
    %0 = bid.x i64
    %1 = bdim.x i64
    %2 = mul i64 %0, %1
    %3 = tid.x i64
    %4 = add i64 %2, %3
    %5 = const.i i64 4
    %6 = mul i64 %4, %5
    %7 = add ptr.global %arg0, %6
    %8 = load i32 ptr.global %7, align 4
    %9 = const.i i32 5
    %10 = rem i32 %8, %9
    switch %10, default bb4 [0 -> bb1, 1 -> bb2, 3 -> bb3]
  bb1:
    %11 = const.i i32 1000
    br bb5
  bb2:
    %12 = const.i i32 3
    %13 = mul i32 %8, %12
    br bb5
  bb3:
    %14 = const.i i32 0
    %15 = sub i32 %14, %8
    br bb5
  bb4:
    %16 = const.i i32 7
    %17 = xor i32 %8, %16
    br bb5
  bb5:
    %18 = phi i32 [bb1 -> %11, bb2 -> %13, bb3 -> %15, bb4 -> %17]
    %19 = const.i i32 0
    br bb6
  bb6:
    %20 = phi i32 [bb5 -> %18, bb7 -> %25]
    %21 = phi i32 [bb5 -> %19, bb7 -> %27]
    %22 = const.i i32 100
    %23 = icmp sgt i32 %20, %22
    condbr %23, bb7, bb8
  bb7:
    %24 = const.i i32 2
    %25 = div i32 %20, %24
    %26 = const.i i32 1
    %27 = add i32 %21, %26
    br bb6
  bb8:
    %28 = const.i i32 4096
    %29 = mul i32 %21, %28
    %30 = add i32 %29, %20
    %31 = add ptr.global %arg1, %6
    store i32 ptr.global %31, %30, align 4
    ret
  }
""")


@pytest.mark.parametrize("level", LEVELS)
def test_control_flow(gpu, level):
    rng = np.random.default_rng(21)
    trips = rng.integers(0, 9, N).astype(np.int32)
    got, want = both(gpu, SWAPPING_PHIS, [trips, np.zeros(N, np.int32)], level)
    assert np.array_equal(got, want) and np.array_equal(got, np.where(trips % 2 == 0, 1, 10))
    vals = rng.integers(0, 5000, N).astype(np.int32)
    got, want = both(gpu, SWITCH_AND_LOOP, [vals, np.zeros(N, np.int32)], level)
    assert np.array_equal(got, want)
