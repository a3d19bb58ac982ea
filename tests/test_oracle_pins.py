"""Pins the CPU oracle (C restatement and BIR interpreter) to the reference's own known-answer
fixtures, the only results the reference states for this path."""
import ctypes

import numpy as np
import pytest

from _util import orc_matmul_f16_rows, orc_sgemm_rows, sgemm_fixture, vp
from basalt_b200 import kernels_bir as kb
from basalt_b200 import workloads as w
from oracle.bir_interp import OracleRefusal, run_kernel

i32, i64 = ctypes.c_int32, ctypes.c_int64


def test_vector_add_f32_fixture(orc):
    # examples/cpu_launch_vadd.c:18-37: a[i]=i, b[i]=2i, c=-1, N=1024, exact a+b
    n = 1024
    a = np.arange(n, dtype=np.float32); b = (2 * np.arange(n)).astype(np.float32)
    c = np.full(n, -1.0, np.float32)
    orc.orc_vector_add_f32(vp(a), vp(b), vp(c), i32(n), i64(n))
    assert np.array_equal(c, a + b)
    c2 = np.full(n, -1.0, np.float32)
    run_kernel(kb.load("vector_add_f32"), "vector_add", [a, b, c2, n], n)
    assert np.array_equal(c2, a + b)


def test_chain_and_square_fixtures(orc):
    # examples/cpu_launch_device_helper_chain.c:18-35 and cpu_launch_device_helper_square.c:19-36
    n = 1024
    x = (np.arange(n) - n // 2).astype(np.int32)
    for name, kern, fn, want in (("chain_vector", "chain_vector", orc.orc_chain_vector, -2 * x + 1),
                                 ("square_vector", "square_vector", orc.orc_square_vector, x * x)):
        out = np.full(n, 0x7fffffff, np.int32)
        fn(vp(x), vp(out), i32(n), i64(n))
        assert np.array_equal(out, want)
        out2 = np.full(n, 0x7fffffff, np.int32)
        run_kernel(kb.load(name), kern, [x, out2, n], n)
        assert np.array_equal(out2, want)


def test_stress_fixture_is_191(orc):
    # examples/cpu_launch_stress.c:14-47, tests/diff/golden/stress.txt: the fold is exactly 191.0
    a = ((np.arange(20) + 1) * 0.5 - 3.0).astype(np.float32)
    out = np.array([-1.0], np.float32)
    orc.orc_stress(vp(a), vp(out), i32(1), i64(1))
    assert out[0] == np.float32(191.0)
    out2 = np.array([-1.0], np.float32)
    run_kernel(kb.stress(), "stress", [a, out2, 1], 1)
    assert out2[0] == np.float32(191.0)


def test_mma2x2_fixture(orc):
    # examples/cpu_launch_mma2x2.c:17-21
    a = np.array([1, 2, 3, 4], np.float32); b = np.array([5, 6, 7, 8], np.float32)
    c = np.full(4, 0.5, np.float32); want = np.array([19.5, 22.5, 43.5, 50.5], np.float32)
    d = np.full(4, -1.0, np.float32)
    orc.orc_mma_f32(vp(a), vp(b), vp(c), vp(d), 2, 2, 2, 0, 0, i64(0), i64(0), i64(0), i64(0))
    assert np.array_equal(d, want)
    d2 = np.full(4, -1.0, np.float32)
    run_kernel(kb.load("mma2x2"), "mma2x2", [a, b, c, d2], 1)
    assert np.array_equal(d2, want)


def test_tiled_sgemm_32_fixture(orc):
    # examples/cpu_launch_tiled_sgemm.c:25-66: D = A@B + C on 32^3, small integers, exact
    a, b, c = sgemm_fixture(32, 32, 32)
    want = (a.astype(np.int64) @ b.astype(np.int64) + c.astype(np.int64)).astype(np.float32)
    d = np.full(1024 + 768, -1.0, np.float32)
    run_kernel(kb.load("tiled_sgemm_f32"), "tiled_sgemm_f32", [a, b, c, d], 1)
    assert np.array_equal(d[:1024].reshape(32, 32), want)
    assert np.all(d[1024:] == -1.0)
    got = orc_sgemm_rows(orc, a, b, 0, 32) + c
    assert np.array_equal(got, want)


def test_triton_matmul_fixture(orc):
    # examples/cpu_launch_triton_matmul.c:39-89: 4x3 output, K=5
    a, b, c = sgemm_fixture(4, 3, 5)
    want = (a.astype(np.int64) @ b.astype(np.int64) + c.astype(np.int64)).astype(np.float32)
    out = np.full(65536, -1.0, np.float32)
    run_kernel(kb.load("tri_matmul"), "matmul_kernel", [a, b, c, out, 5], 1)
    assert np.array_equal(out[:12].reshape(4, 3), want)
    dot = np.empty((4, 3), np.float32)
    orc.orc_tl_dot_f32(vp(a), vp(b), None, vp(dot), 4, 3, 5)
    assert np.array_equal(dot + c, want)


def test_triton_masked_vadd_fixture(orc):
    # examples/cpu_launch_triton_vadd.c:31-58: N=1000, BLOCK=1024, lanes >= N stay poisoned
    n, block = 1000, 1024
    a = np.arange(n, dtype=np.float32); b = (2 * np.arange(n)).astype(np.float32)
    for run in ("c", "interp"):
        c = np.full(32768, -1.0, np.float32)
        if run == "c":
            orc.orc_triton_vadd_f32(vp(a), vp(b), vp(c), i64(n), i64(block), i64(1))
        else:
            run_kernel(kb.load("tri_vadd"), "vector_add", [a, b, c, n, block], 1)
        assert np.array_equal(c[:n], a + b)
        assert np.all(c[n:] == -1.0)


def test_f16_matmul_rule_on_the_32_cubed_integer_case(orc):
    # crates/basalt-llvm/tests/tiled_sgemm_wmma.rs:289-307 uses the same integer inputs in f16 with
    # f32 accumulation; every partial sum is an integer below 2048, so the result is exact.
    a, b, _ = sgemm_fixture(32, 32, 32)
    want = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float16)
    got = orc_matmul_f16_rows(orc, a.astype(np.float16), b.astype(np.float16), 32, False, 0, 32)
    assert np.array_equal(got, want)
    got_nk = orc_matmul_f16_rows(orc, a.astype(np.float16), np.ascontiguousarray(b.T).astype(np.float16), 32, True, 0, 32)
    assert np.array_equal(got_nk, want)


def test_blocked_references_match_the_scalar_loops(orc):
    rng = np.random.default_rng(7)
    A = rng.uniform(-1, 1, (48, 40)).astype(np.float32); B = rng.uniform(-1, 1, (40, 56)).astype(np.float32)
    scalar = np.empty((48, 56), np.float32)
    orc.orc_sgemm_f32_scalar(vp(A), vp(B), vp(scalar), 48, 56, 40)
    assert np.array_equal(orc_sgemm_rows(orc, A, B, 0, 48), scalar)
    Ah, Bh = A.astype(np.float16), B.astype(np.float16)
    sc16 = np.empty((48, 56), np.float16)
    orc.orc_matmul_f16_scalar(vp(Ah), vp(Bh), vp(sc16), 48, 56, 40)
    assert np.array_equal(orc_matmul_f16_rows(orc, Ah, Bh, 56, False, 0, 48).view(np.uint16), sc16.view(np.uint16))


def test_f16_conversions_match_numpy(orc):
    rng = np.random.default_rng(3)
    vals = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 1e-6, 2000), rng.normal(0, 7e4, 500),
                           [0.0, -0.0, 65504.0, 65520.0, 6e-8, 2.98e-8, 2.9802322387695312e-08, np.inf, -np.inf]])
    for v in vals:
        assert orc.orc_f64_to_f16(float(v)) == int(np.float64(v).astype(np.float16).view(np.uint16)), v
    for bits in rng.integers(0, 65536, 3000):
        h = np.uint16(bits).view(np.float16)
        if np.isnan(h):
            continue
        assert orc.orc_f16_to_f32(int(bits)) == np.float32(h)


def test_generators_agree_with_the_product_generators(orc):
    n = 70000
    for name, fn, dt in (("orc_fill_i32_pm30", w.i32_pm30, np.int32), ("orc_fill_u32", w.u32, np.uint32),
                         ("orc_fill_f32_pm1", w.f32_pm1, np.float32), ("orc_fill_f16_normal01", w.f16_normal01, np.float16)):
        a = np.empty(n, dtype=dt)
        getattr(orc, name)(ctypes.c_uint64(0xBA5A1701), i64(n), vp(a))
        assert np.array_equal(a.view(np.uint8), fn(0xBA5A1701, n).view(np.uint8)), name
    x = w.i32_pm30(1, 50000)
    assert x.min() >= -2**30 and x.max() < 2**30
    f = w.f32_pm1(2, 50000)
    assert f.min() >= -1.0 and f.max() < 1.0
    h = w.f16_normal01(3, 200000).astype(np.float64)
    assert abs(h.mean()) < 2e-3 and abs(h.std() - 0.1) < 2e-3


def test_max_and_helper_chain_restatements(orc):
    x = w.u32(5, 10007).view(np.int32)
    out = np.array([-2**31], np.int32)
    orc.orc_max_i32(vp(x), vp(out), i32(len(x)), i64(len(x)))
    assert out[0] == x.max()
    u = w.u32(6, 999)
    got = np.zeros(999, np.uint32)
    orc.orc_helper_chain_u32(vp(u), vp(got), i32(999), i64(999))
    v = u.astype(np.uint64)
    for j in range(32):
        v = (v * v + ((2654435761 * j) & 0xFFFFFFFF)) & 0xFFFFFFFF
    assert np.array_equal(got, v.astype(np.uint32))


def test_oracle_model_refuses_shuffles():
    # crates/basalt-x86/src/oracle.rs:651-655: warp collectives are E090 under the CPU model
    x = np.zeros(32, np.int32); out = np.zeros(1, np.int32)
    with pytest.raises(OracleRefusal) as e:
        run_kernel(kb.load("max_i32"), "max_i32", [x, out, 32], 32)
    assert e.value.code == "E090"
