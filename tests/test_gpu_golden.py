"""The differential lane: every integer workload, from each of its three source forms (BIR text,
CUDA-C, Triton where one exists) at both optimisation levels, must give on the device exactly the
bytes whose SHA-256 tests/golden/golden.json holds for the CPU oracle on the same seeded input --
at a small ragged size and at the benchmark configuration's full size.  The reference's harness does
the same between its back ends (tests/diff/run_diff.sh: oracle output against a stored golden, every
other back end against the oracle)."""
import ctypes
import hashlib
import json
import os

import numpy as np
import pytest

import basalt_b200 as b
from basalt_b200 import kernels, kernels_bir as kb, kernels_cu as kc, kernels_triton as kt, workloads as w
from _gpu import dev, emitted, grid_for
from _util import vp

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "golden.json")) as f:
    GOLDEN = json.load(f)["cases"]


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).view(np.uint8)).hexdigest()


def sources(name):
    """(label, BIR text, kernel name) for every source form of a workload."""
    if name == "vadd_i32":
        return [("bir", kb.load("vadd_i32"), "vadd_i32"), ("cuda", b.compile_cuda(kc.load("vadd_i32")), "vadd_i32")]
    if name == "helper_chain":
        return [("bir", kb.helper_chain(), "helper_chain"), ("cuda", b.compile_cuda(kc.helper_chain()), "helper_chain")]
    if name == "max_i32":
        return [("bir", kb.load("max_i32"), "max_i32"), ("cuda", b.compile_cuda(kc.load("max_i32")), "max_i32")]
    if name == "vector_add_f32":
        return [("bir", kb.load("vector_add_f32"), "vector_add"), ("cuda", b.compile_cuda(kc.load("vector_add_f32")), "vector_add")]
    raise KeyError(name)


@pytest.mark.parametrize("label", ["small", "full"])
@pytest.mark.parametrize("level", [0, 2])
def test_vadd_i32(gpu, label, level):
    g = GOLDEN["vadd_i32"][label]
    n = g["n"]
    a = w.i32_pm30(w.SEEDS["vadd_i32"], n); bb = w.i32_pm30(w.SEEDS["vadd_i32"] + 1, n)
    da, db = dev(gpu, a), dev(gpu, bb)
    for form, bir, kernel in sources("vadd_i32"):
        dc = dev(gpu, np.full(n, 0x7fffffff, np.int32))
        emitted(gpu, bir, kernel, level).launch(grid_for(n), 256, 0, [da, db, dc, b.i32(n)])
        assert sha(dc.to_numpy(np.int32)) == g["sha256"], (form, level)
    dc = dev(gpu, np.full(n, 0x7fffffff, np.int32))
    emitted(gpu, kt.vadd_i32(), "vadd_i32", level).launch((n + 1023) // 1024, 256, 0, [da, db, dc, b.i64(n), b.i64(1024)])      # programs of 1024 lanes
    assert sha(dc.to_numpy(np.int32)) == g["sha256"], ("triton", level)
    dc = dev(gpu, np.full(n, 0x7fffffff, np.int32))
    kernels.vadd_i32(da, db, dc, n)
    gpu.synchronize()
    assert sha(dc.to_numpy(np.int32)) == g["sha256"], "hand-written"


@pytest.mark.parametrize("label", ["small", "full"])
@pytest.mark.parametrize("level", [0, 2])
def test_helper_chain(gpu, orc, label, level):
    g = GOLDEN["helper_chain"][label]
    n = g["n"]
    x = np.empty(n, np.uint32)
    orc.orc_fill_u32(ctypes.c_uint64(w.SEEDS["helper_chain"]), ctypes.c_int64(n), vp(x))     # the generator only: the oracle's kernels are not run here
    dx = dev(gpu, x)
    for form, bir, kernel in sources("helper_chain"):
        dy = dev(gpu, np.zeros(n, np.uint32))
        emitted(gpu, bir, kernel, level).launch(grid_for(n), 256, 0, [dx, dy, b.i32(n)])
        assert sha(dy.to_numpy(np.uint32)) == g["sha256"], (form, level)
        dy.free()
    dy = dev(gpu, np.zeros(n, np.uint32))
    kernels.helper_chain_u32(dx, dy, n)
    gpu.synchronize()
    assert sha(dy.to_numpy(np.uint32)) == g["sha256"], "hand-written"
    dy.free(); dx.free()


@pytest.mark.parametrize("label", ["small", "full"])
@pytest.mark.parametrize("level", [0, 2])
def test_max_i32(gpu, orc, label, level):
    g = GOLDEN["max_i32"][label]
    n = g["n"]
    x = np.empty(n, np.uint32)
    orc.orc_fill_u32(ctypes.c_uint64(w.SEEDS["max_i32"]), ctypes.c_int64(n), vp(x))
    dx = dev(gpu, x)
    for form, bir, kernel in sources("max_i32"):
        fn = emitted(gpu, bir, kernel, level)
        out = dev(gpu, np.array([-2**31], np.int32))
        fn.launch(fn.streaming_grid(256, n), 256, 0, [dx, out, b.i32(n)])
        assert int(out.to_numpy(np.int32)[0]) == g["value"], (form, level)
    out = dev(gpu, np.array([-2**31], np.int32))
    emitted(gpu, kt.max_i32(), "max_i32", level).launch((n + 8191) // 8192, 256, 0, [dx, out, b.i64(n), b.i64(8192)])      # tl.max over 8192 lanes per program
    assert int(out.to_numpy(np.int32)[0]) == g["value"], ("triton", level)
    out = dev(gpu, np.array([-2**31], np.int32))
    kernels.max_i32(dx, n, out)
    gpu.synchronize()
    assert int(out.to_numpy(np.int32)[0]) == g["value"], "hand-written"
    dx.free()


@pytest.mark.parametrize("level", [0, 2])
def test_vector_add_f32_including_the_triton_source(gpu, level):
    g = GOLDEN["vector_add_f32"]["small"]
    n = g["n"]
    a = w.f32_pm1(31, n); bb = w.f32_pm1(32, n)
    da, db = dev(gpu, a), dev(gpu, bb)
    for form, bir, kernel in sources("vector_add_f32"):
        dc = dev(gpu, np.zeros(n, np.float32))
        emitted(gpu, bir, kernel, level).launch(grid_for(n), 256, 0, [da, db, dc, b.i32(n)])
        assert sha(dc.to_numpy(np.float32)) == g["sha256"], (form, level)
    dc = dev(gpu, np.zeros(n, np.float32))
    emitted(gpu, kt.vector_add(), "vector_add", level).launch((n + 255) // 256, 128, 0, [da, db, dc, b.i64(n), b.i64(256)])
    assert sha(dc.to_numpy(np.float32)) == g["sha256"], ("triton", level)
