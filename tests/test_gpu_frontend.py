"""CUDA-C sources through the whole path on the device: front end -> BIR -> sm_100a PTX -> JIT ->
launch, against the CPU oracle on the same seeded inputs.  Integer kernels bit-exact; SGEMM within
1e-4 and the fp16 matmul within 2e-3 relative Frobenius error (the benchmark's tolerances)."""
import ctypes

import numpy as np
import pytest

import basalt_b200 as b
from basalt_b200 import kernels_cu as kc, workloads as w
from _gpu import dev, emitted, grid_for
from _util import orc_matmul_f16_rows, orc_sgemm_rows, rel_fro, sgemm_fixture, vp
from test_frontend_cuda import control_flow_expected

pytestmark = pytest.mark.gpu
POISON = 0x7fffffff


def from_cuda(gpu, source, kernel, level=2):
    return emitted(gpu, b.compile_cuda(source), kernel, level)


@pytest.mark.parametrize("level", [0, 2])
def test_vadd_source(gpu, orc, level):
    fn = from_cuda(gpu, kc.load("vadd_i32"), "vadd_i32", level)
    for n in [1, 33, 257, 4099, (1 << 20) + 3]:
        a = w.i32_pm30(w.SEEDS["vadd_i32"], n); bb = w.i32_pm30(w.SEEDS["vadd_i32"] + 1, n)
        want = np.full(n, POISON, np.int32)
        orc.orc_vadd_i32(vp(a), vp(bb), vp(want), ctypes.c_int32(n), ctypes.c_int64(n))
        da, db, dc = dev(gpu, a), dev(gpu, bb), dev(gpu, np.full(n + 8, POISON, np.int32))
        fn.launch(grid_for(n), 256, 0, [da, db, dc, b.i32(n)])
        got = dc.to_numpy(np.int32)
        assert np.array_equal(got[:n], want) and np.all(got[n:] == POISON), n


@pytest.mark.parametrize("level", [0, 2])
def test_block_max_source(gpu, orc, level):
    fn = from_cuda(gpu, kc.load("max_i32"), "max_i32", level)
    for n in [1, 5, 31, 33, 255, 257, 1023, 4099, 100003, 1 << 22]:
        x = w.u32(w.SEEDS["max_i32"], n).view(np.int32)
        want = np.array([-2**31], np.int32)
        orc.orc_max_i32(vp(x), vp(want), ctypes.c_int32(n), ctypes.c_int64(n))
        out = dev(gpu, np.array([-2**31], np.int32))
        fn.launch(fn.streaming_grid(256, n), 256, 0, [dev(gpu, x), out, b.i32(n)])
        assert int(out.to_numpy(np.int32)[0]) == int(want[0]), n
    x = -np.abs(w.i32_pm30(9, 5000)) - 5          # all negative: the identity must not leak
    out = dev(gpu, np.array([-2**31], np.int32))
    fn.launch(8, 256, 0, [dev(gpu, x), out, b.i32(5000)])
    assert int(out.to_numpy(np.int32)[0]) == int(x.max())


@pytest.mark.parametrize("level", [0, 2])
def test_helper_chain_source(gpu, orc, level):
    fn = from_cuda(gpu, kc.helper_chain(), "helper_chain", level)
    for n in [1, 257, 4099, 1 << 20]:
        x = w.u32(w.SEEDS["helper_chain"], n)
        want = np.zeros(n, np.uint32)
        orc.orc_helper_chain_u32(vp(x), vp(want), ctypes.c_int32(n), ctypes.c_int64(n))
        dout = dev(gpu, np.full(n + 4, 0xDEADBEEF, np.uint32))
        fn.launch(grid_for(n), 256, 0, [dev(gpu, x), dout, b.i32(n)])
        got = dout.to_numpy(np.uint32)
        assert np.array_equal(got[:n], want) and np.all(got[n:] == 0xDEADBEEF), n


@pytest.mark.parametrize("level", [0, 2])
def test_control_flow_source_with_real_barriers(gpu, level):
    fn = from_cuda(gpu, kc.load("control_flow"), "control_flow", level)
    n = 1000
    x = np.random.default_rng(41).integers(-50, 50, 1024, dtype=np.int64).astype(np.int32)
    x[3] = 7
    want = control_flow_expected(x, n)
    dout = dev(gpu, np.full(1024, POISON, np.int32))
    fn.launch(4, 256, 0, [dev(gpu, x), dout, b.i32(n)])
    got = dout.to_numpy(np.int32)
    for i in range(1024):
        assert got[i] == (want[i] if i < n else POISON), i


def test_stress_and_constant_sources(gpu):
    a = ((np.arange(20) + 1) * 0.5 - 3.0).astype(np.float32)
    out = dev(gpu, np.zeros(32, np.float32))
    from_cuda(gpu, kc.stress(), "stress").launch(1, 32, 0, [dev(gpu, a), out, b.i32(32)])
    assert np.all(out.to_numpy(np.float32) == np.float32(191.0))      # examples/cpu_launch_stress.c:14-47
    out = dev(gpu, np.zeros(1, np.int32))
    from_cuda(gpu, kc.load("constant_math"), "constant_math").launch(1, 1, 0, [out])
    assert out.to_numpy(np.int32)[0] == 20                            # examples/cpu_launch_mymathhomework.c:15-24


def test_sgemm_source(gpu, orc):
    A, B, _ = sgemm_fixture(128, 256, 64)
    dC = dev(gpu, np.full((128, 256), np.nan, np.float32))
    from_cuda(gpu, kc.sgemm_cta128(128, 256, 64), "sgemm_f32").launch((2, 1), 256, 0, [dev(gpu, A), dev(gpu, B), dC])
    assert np.array_equal(dC.to_numpy(np.float32).reshape(128, 256), (A.astype(np.int64) @ B.astype(np.int64)).astype(np.float32))
    M, N, K = 512, 256, 512
    A = w.f32_pm1(w.SEEDS["sgemm_f32"], M * K).reshape(M, K)
    B = w.f32_pm1(w.SEEDS["sgemm_f32"] + 1, K * N).reshape(K, N)
    dC = dev(gpu, np.full((M, N), np.nan, np.float32))
    from_cuda(gpu, kc.sgemm_cta128(M, N, K), "sgemm_f32").launch((N // 128, M // 128), 256, 0, [dev(gpu, A), dev(gpu, B), dC])
    assert rel_fro(dC.to_numpy(np.float32).reshape(M, N), orc_sgemm_rows(orc, A, B, 0, M)) <= 1e-4


@pytest.mark.parametrize("b_is_nk", [False, True])
def test_matmul_f16_source(gpu, orc, b_is_nk):
    M, N, K = 256, 512, 1024
    A = w.f16_normal01(w.SEEDS["matmul_f16"], M * K).reshape(M, K)
    B = w.f16_normal01(w.SEEDS["matmul_f16"] + 1, K * N).reshape(K, N)
    Bdev = np.ascontiguousarray(B.T) if b_is_nk else B
    fn = from_cuda(gpu, kc.matmul_f16(M, N, K, b_is_nk), "matmul_kernel")
    dC = dev(gpu, np.full((M, N), np.nan, np.float16))
    fn.launch((N // 128, M // 128), 128, 0, [dev(gpu, A), dev(gpu, Bdev), dC])
    assert fn.status() == 0, "a bounded wait inside the emitted kernel expired"
    got = dC.to_numpy(np.float16).reshape(M, N)
    assert rel_fro(got, orc_matmul_f16_rows(orc, A, Bdev, N, b_is_nk, 0, M)) <= 2e-3


@pytest.mark.parametrize("level", [0, 2])
def test_switch_source(gpu, level):
    from test_frontend_cuda import switch_cases_expected
    n = 5000
    x = (np.arange(n) * 37 % 1013 - 500).astype(np.int32)
    out = np.zeros(n, np.int32)
    gpu.cpu_launch(emitted(gpu, b.compile_cuda(kc.load("switch_cases")), "switch_cases", level), [x, out, b.i32(n)], n)
    assert np.array_equal(out, switch_cases_expected(x))
