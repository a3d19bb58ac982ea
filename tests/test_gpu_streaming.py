"""Parity of the three integer workloads (vadd_i32, max_i32, helper chain): emitted PTX at both
optimisation levels and the hand-written kernels against the CPU oracle on the same seeded
inputs.  Bit-exact.  Sizes include empty-adjacent, ragged and unaligned cases and the benchmark's
full sizes."""
import ctypes

import numpy as np
import pytest

import basalt_b200 as b
from basalt_b200 import kernels, kernels_bir as kb, workloads as w
from _gpu import dev, emitted, grid_for
from _util import vp

pytestmark = pytest.mark.gpu
SIZES = [1, 3, 31, 32, 33, 255, 256, 257, 1023, 1025, 4099, 1 << 20]
POISON = 0x7fffffff


def oracle_vadd(orc, a, bb):
    c = np.full(len(a), POISON, np.int32)
    orc.orc_vadd_i32(vp(a), vp(bb), vp(c), ctypes.c_int32(len(a)), ctypes.c_int64(len(a)))
    return c


@pytest.mark.parametrize("level", [0, 2])
def test_vadd_emitted(gpu, orc, level):
    fn = emitted(gpu, kb.load("vadd_i32"), "vadd_i32", level)
    for n in SIZES:
        a = w.i32_pm30(w.SEEDS["vadd_i32"], n); bb = w.i32_pm30(w.SEEDS["vadd_i32"] + 1, n)
        da, db, dc = dev(gpu, a), dev(gpu, bb), dev(gpu, np.full(n + 8, POISON, np.int32))
        fn.launch(grid_for(n), 256, 0, [da, db, dc, b.i32(n)])
        got = dc.to_numpy(np.int32)
        assert np.array_equal(got[:n], oracle_vadd(orc, a, bb)), n
        assert np.all(got[n:] == POISON), n


def test_vadd_emitted_unaligned_and_undersized_launch(gpu, orc):
    fn = emitted(gpu, kb.load("vadd_i32"), "vadd_i32", 2)
    n = 5000
    a = w.i32_pm30(1, n + 1); bb = w.i32_pm30(2, n + 1)
    da, db, dc = dev(gpu, a), dev(gpu, bb), dev(gpu, np.full(n + 9, POISON, np.int32))
    # pointers 4 bytes past a 16-byte boundary take the scalar path
    fn.launch(grid_for(n), 256, 0, [b.ptr(da.device_ptr() + 4), b.ptr(db.device_ptr() + 4), b.ptr(dc.device_ptr() + 4), b.i32(n)])
    got = dc.to_numpy(np.int32)
    assert got[0] == POISON and np.array_equal(got[1:n + 1], oracle_vadd(orc, a[1:], bb[1:])) and np.all(got[n + 1:] == POISON)
    # a launch with fewer threads than elements processes only the first gridDim*blockDim elements
    dc2 = dev(gpu, np.full(n, POISON, np.int32))
    fn.launch(4, 256, 0, [da, db, dc2, b.i32(n)])
    got = dc2.to_numpy(np.int32)
    assert np.array_equal(got[:1024], oracle_vadd(orc, a[:1024], bb[:1024])) and np.all(got[1024:] == POISON)


def test_vadd_handwritten(gpu, orc):
    for n in SIZES:
        a = w.i32_pm30(3, n); bb = w.i32_pm30(4, n)
        da, db, dc = dev(gpu, a), dev(gpu, bb), dev(gpu, np.full(n + 8, POISON, np.int32))
        kernels.vadd_i32(da, db, dc, n)
        gpu.synchronize()
        got = dc.to_numpy(np.int32)
        assert np.array_equal(got[:n], oracle_vadd(orc, a, bb)) and np.all(got[n:] == POISON), n
    n = 4099
    a = w.i32_pm30(5, n + 1); bb = w.i32_pm30(6, n + 1)
    da, db, dc = dev(gpu, a), dev(gpu, bb), dev(gpu, np.full(n + 1, POISON, np.int32))
    kernels.vadd_i32(da.device_ptr() + 4, db.device_ptr() + 4, dc.device_ptr() + 4, n)
    gpu.synchronize()
    assert np.array_equal(dc.to_numpy(np.int32)[1:], oracle_vadd(orc, a[1:], bb[1:]))


def oracle_max(orc, x):
    out = np.array([-2**31], np.int32)
    orc.orc_max_i32(vp(x), vp(out), ctypes.c_int32(len(x)), ctypes.c_int64(len(x)))
    return int(out[0])


def gpu_max(gpu, how, dx, n, level=2):
    out = dev(gpu, np.array([-2**31], np.int32))
    if how == "hand":
        kernels.max_i32(dx, n, out)
        gpu.synchronize()
    elif how == "atomic":
        emitted(gpu, kb.load("max_i32_atomic"), "max_i32_atomic", level).launch(grid_for(n), 256, 0, [dx, out, b.i32(n)])
    else:
        fn = emitted(gpu, kb.load("max_i32"), "max_i32", level)
        fn.launch(fn.streaming_grid(256, n), 256, 0, [dx, out, b.i32(n)])
    return int(out.to_numpy(np.int32)[0])


@pytest.mark.parametrize("how, level", [("emitted", 0), ("emitted", 2), ("hand", 2), ("atomic", 2)])
def test_max_i32_small_and_ragged(gpu, orc, how, level):
    for n in [1, 5, 31, 33, 255, 257, 1023, 4099, 100003, 1 << 20]:
        x = w.u32(w.SEEDS["max_i32"], n).view(np.int32)
        assert gpu_max(gpu, how, dev(gpu, x), n, level) == oracle_max(orc, x), (how, n)
    # all-negative input: the identity INT32_MIN must not leak
    x = -np.abs(w.i32_pm30(9, 5000)) - 5
    assert gpu_max(gpu, how, dev(gpu, x), 5000, level) == oracle_max(orc, x)


@pytest.mark.parametrize("how", ["emitted", "hand"])
def test_max_i32_full_size_with_planted_maxima(gpu, orc, how):
    n = 1 << 28
    x = np.empty(n, np.uint32)
    orc.orc_fill_u32(ctypes.c_uint64(w.SEEDS["max_i32"]), ctypes.c_int64(n), vp(x))
    x = x.view(np.int32)
    dx = dev(gpu, x)
    assert gpu_max(gpu, how, dx, n) == oracle_max(orc, x)
    np.minimum(x, 2**31 - 2, out=x)
    for plant in (0, n - 1, n // 8, n // 8 - 1, 123456789):   # ends, a shard boundary, an arbitrary index
        x[plant] = 2**31 - 1
        dx.copy_from_host(x)
        assert gpu_max(gpu, how, dx, n) == 2**31 - 1, plant
        x[plant] = 2**31 - 2
    dx.free()


def oracle_chain(orc, x):
    out = np.zeros(len(x), np.uint32)
    orc.orc_helper_chain_u32(vp(x), vp(out), ctypes.c_int32(len(x)), ctypes.c_int64(len(x)))
    return out


@pytest.mark.parametrize("how, level", [("emitted", 0), ("emitted", 2), ("hand", 2)])
def test_helper_chain(gpu, orc, how, level):
    for n in [1, 31, 33, 257, 4099, 1 << 20]:
        x = w.u32(w.SEEDS["helper_chain"], n)
        dx, dout = dev(gpu, x), dev(gpu, np.full(n + 4, 0xDEADBEEF, np.uint32))
        if how == "hand":
            kernels.helper_chain_u32(dx, dout, n)
            gpu.synchronize()
        else:
            emitted(gpu, kb.helper_chain(), "helper_chain", level).launch(grid_for(n), 256, 0, [dx, dout, b.i32(n)])
        got = dout.to_numpy(np.uint32)
        assert np.array_equal(got[:n], oracle_chain(orc, x)) and np.all(got[n:] == 0xDEADBEEF), (how, n)


def test_helper_chain_full_size(gpu, orc):
    n = 1 << 26
    x = np.empty(n, np.uint32)
    orc.orc_fill_u32(ctypes.c_uint64(w.SEEDS["helper_chain"]), ctypes.c_int64(n), vp(x))
    want = oracle_chain(orc, x)
    dx, dout = dev(gpu, x), gpu.alloc(4 * n)
    emitted(gpu, kb.helper_chain(), "helper_chain", 2).launch(grid_for(n), 256, 0, [dx, dout, b.i32(n)])
    assert np.array_equal(dout.to_numpy(np.uint32), want)
    kernels.helper_chain_u32(dx, dout, n)
    gpu.synchronize()
    assert np.array_equal(dout.to_numpy(np.uint32), want)


@pytest.mark.parametrize("kind, host, dtype", [("u32", w.u32, np.uint32), ("i32_pm30", w.i32_pm30, np.int32), ("f32_pm1", w.f32_pm1, np.float32),
                                               ("f16_normal01", w.f16_normal01, np.float16)])
def test_device_generator_matches_the_host_generator(gpu, kind, host, dtype):
    # bench.py makes its inputs on the device; they must be the bytes the host generator (and, by
    # tests/test_golden.py, the oracle's generator) produces for the same seed, at any offset.
    from basalt_b200 import kernels
    n = (1 << 18) + 13
    want = host(w.SEEDS["vadd_i32"] + 5, n)
    buf = gpu.alloc(n * want.itemsize)
    kernels.fill(kind, w.SEEDS["vadd_i32"] + 5, n, buf)
    gpu.synchronize()
    got = buf.to_numpy(dtype, n)
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8))
    kernels.fill(kind, w.SEEDS["vadd_i32"] + 5, 1000, buf, start=777)
    gpu.synchronize()
    assert np.array_equal(buf.to_numpy(dtype, 1000).view(np.uint8), want[777:1777].view(np.uint8))
