"""parse(print(m)) == m, the BIR round-trip invariant (crates/basalt-bir/tests/roundtrip.rs), and
the parser's numbering rules (crates/basalt-bir/src/parse.rs:423-499)."""
import pytest

import basalt_b200 as b
from basalt_b200 import kernels_bir as kb

HAND_WRITTEN = """module {
  launch_bounds max_threads=128 min_blocks=1
  shared_mem_bytes 0
  target_dtypes i32

  func @select_max(i32, i32) -> i32 {
  bb0:
    %0 = icmp sgt i32 %arg0, %arg1
    condbr %0, bb1, bb2
  bb1:
    br bb3
  bb2:
    %1 = const.i i32 1
    %2 = add i32 %arg1, %1
    br bb3
  bb3:
    %3 = phi i32 [bb1 -> %arg0, bb2 -> %2]
    ret %3
  }
}
"""

EVERY_FORM = """module {
  shared_mem_bytes 16
  target_dtypes i32 f32 f16

  host func @host(ptr.global, i64) -> void {
  bb0:
    %0 = cuda.malloc ptr.global %arg1
    %1 = const.i i32 1
    cuda.memcpy %0, %arg0, %arg1, %1
    %3 = const.i i32 4
    %4 = const.i i64 0
    %5 = const.i ptr.global 0
    kernel.launch @k grid %3, %1, %1 block %3, %1, %1 shared %4 stream %5 [%0, %arg1]
    cuda.device_sync
    cuda.free %0
    ret
  }

  func @k(ptr.global, i64) -> void {
  bb0:
    %0 = tid.x i32
    %1 = const.f f32 0.5
    %2 = const.f f64 -1
    %3 = const.f f32 inf
    %4 = load v4f32 ptr.global %arg0, align 16, volatile
    %5 = fadd v4f32 %4, %4
    store v4f32 ptr.global %arg0, %5, align 16
    %7 = shuffle.down i32 %0, %0
    %8 = ballot i32 %0
    %9 = vote.any i32 %0
    %10 = vote.all i32 %0
    %11 = atomic.add i32 ptr.global %arg0, %0
    %12 = atomic.cas i32 ptr.shared %arg0, %0, %0
    barrier
    %14 = fcmp uno f32 %1, %1
    %15 = select i32 %14, %0, %0
    %16 = fptosi i32 f32 %1
    %17 = call i32 @h [%0]
    mma f32 f32 row col m 16 n 16 k 16 %arg0, %arg0, %arg0, %arg0
    switch %0, default bb1 [0 -> bb1, -3 -> bb2]
  bb1:
    br bb2
  bb2:
    ret %15
  }

  host func @h(i32) -> i32 {
  bb0:
    ret %arg0
  }
}
"""


@pytest.mark.parametrize("name", list(kb.STATIC))
def test_static_kernels_round_trip(name):
    src = kb.load(name)
    assert b.roundtrip(src) == src


def test_generated_kernels_round_trip():
    for src in (kb.helper_chain(), kb.stress(), kb.sgemm_cta128(256, 128, 32), kb.matmul_f16(128, 256, 64), kb.matmul_f16(128, 128, 64, True)):
        assert b.roundtrip(src) == src


def test_reference_style_modules_round_trip():
    assert b.roundtrip(HAND_WRITTEN) == HAND_WRITTEN
    assert b.roundtrip(EVERY_FORM) == EVERY_FORM


def test_optimised_modules_round_trip(ptx):
    for src in (kb.load("vadd_i32"), kb.load("max_i32"), kb.helper_chain()):
        opt = ptx.optimized_bir(src)
        assert b.roundtrip(opt) == opt


@pytest.mark.parametrize("bad, why", [
    (HAND_WRITTEN.replace("%1 = const.i", "%2 = const.i"), "out of order"),
    (HAND_WRITTEN.replace("bb2:", "bb5:"), "out of order"),
    (HAND_WRITTEN.replace("%3 = phi", "phi"), "produces a result"),
    (HAND_WRITTEN.replace("icmp sgt", "icmp weird"), "predicate"),
    (HAND_WRITTEN.replace("add i32 %arg1, %1", "add i32 %arg1, %9"), "undefined"),
    (HAND_WRITTEN.replace("br bb3\n  bb2", "br bb7\n  bb2"), "missing block"),
    ("module { shared_mem_bytes 0 target_dtypes", "expected"),
    ("", "expected"),
])
def test_malformed_bir_is_e400(bad, why):
    with pytest.raises(b.Diag) as e:
        b.roundtrip(bad)
    assert e.value.code == "E400"
    assert why in e.value.arg
    assert b.Ptx().supports(bad) == b.Support(False, "E400")
