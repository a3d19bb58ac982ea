"""Triton sources through the whole path on the device: front end -> BIR -> sm_100a PTX -> JIT ->
launch, with a program per CTA.  The masked vector add is bit-exact against its definition (no
lane at or past n is read or written); the tiled matmuls are checked against the CPU oracle with
the benchmark's tolerances (SGEMM 1e-4, f16 2e-3 relative Frobenius) and exactly on small
integers."""
import numpy as np
import pytest

import basalt_b200 as b
from basalt_b200 import kernels_triton as kt, workloads as w
from _gpu import dev, emitted
from _util import orc_matmul_f16_rows, orc_sgemm_rows, rel_fro, sgemm_fixture

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("level", [0, 2])
@pytest.mark.parametrize("block_size, threads", [(1024, 256), (1024, 1024), (256, 64), (96, 128)])
def test_masked_vector_add(gpu, level, block_size, threads):
    fn = emitted(gpu, kt.vector_add(), "vector_add", level)
    for n in [1, 1000, 4099, (1 << 18) + 5]:
        a = w.f32_pm1(11, n); bb = w.f32_pm1(12, n)
        programs = (n + block_size - 1) // block_size
        # the buffers end exactly at n: a lane past n that loaded or stored would run off the allocation's data
        da, db = dev(gpu, a), dev(gpu, bb)
        dc = dev(gpu, np.full(programs * block_size + 8, -1.0, np.float32))
        fn.launch(programs, threads, 0, [da, db, dc, b.i64(n), b.i64(block_size)])
        got = dc.to_numpy(np.float32)
        assert np.array_equal(got[:n], a + bb) and np.all(got[n:] == -1.0), (n, block_size, threads)


def test_small_matmul_fixture(gpu):
    # examples/cpu_launch_triton_matmul.c:39-89 on the device: one program, any CTA size
    A, B, C = sgemm_fixture(4, 3, 5)
    fn = emitted(gpu, kt.small_matmul(5), "matmul_kernel")
    for threads in (1, 32, 128):
        out = dev(gpu, np.full((4, 3), np.nan, np.float32))
        fn.launch(1, threads, 0, [dev(gpu, A), dev(gpu, B), dev(gpu, C), out, b.i64(5)])
        assert np.array_equal(out.to_numpy(np.float32).reshape(4, 3), A @ B + C), threads


def test_tiled_sgemm(gpu, orc):
    M, N, K = 256, 384, 128
    A, B, _ = sgemm_fixture(M, N, K)
    dC = dev(gpu, np.full((M, N), np.nan, np.float32))
    emitted(gpu, kt.sgemm(M, N, K), "sgemm_f32").launch((N // 128, M // 128), 256, 0, [dev(gpu, A), dev(gpu, B), dC, b.i64(M), b.i64(N), b.i64(K)])
    assert np.array_equal(dC.to_numpy(np.float32).reshape(M, N), (A.astype(np.int64) @ B.astype(np.int64)).astype(np.float32))
    A = w.f32_pm1(w.SEEDS["sgemm_f32"], M * K).reshape(M, K)
    B = w.f32_pm1(w.SEEDS["sgemm_f32"] + 1, K * N).reshape(K, N)
    dC = dev(gpu, np.full((M, N), np.nan, np.float32))
    emitted(gpu, kt.sgemm(M, N, K), "sgemm_f32").launch((N // 128, M // 128), 256, 0, [dev(gpu, A), dev(gpu, B), dC, b.i64(M), b.i64(N), b.i64(K)])
    assert rel_fro(dC.to_numpy(np.float32).reshape(M, N), orc_sgemm_rows(orc, A, B, 0, M)) <= 1e-4


@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 512, 1024), (384, 256, 192)])
def test_tiled_matmul_f16_on_tensor_cores(gpu, orc, shape):
    M, N, K = shape
    A = w.f16_normal01(w.SEEDS["matmul_f16"], M * K).reshape(M, K)
    B = w.f16_normal01(w.SEEDS["matmul_f16"] + 1, K * N).reshape(K, N)
    fn = emitted(gpu, kt.matmul_f16(M, N, K), "matmul_kernel")
    dC = dev(gpu, np.full((M, N), np.nan, np.float16))
    fn.launch((N // 128, M // 128), 128, 0, [dev(gpu, A), dev(gpu, B), dC, b.i64(M), b.i64(N), b.i64(K)])
    assert fn.status() == 0, "a bounded wait inside the emitted kernel expired"
    got = dC.to_numpy(np.float16).reshape(M, N)
    assert rel_fro(got, orc_matmul_f16_rows(orc, A, B, N, False, 0, M)) <= 2e-3


def test_reductions_and_atomics(gpu):
    # tl.sum over float32 through the shuffle butterfly: small integers, so the order of the additions cannot matter
    src = "@triton.jit\ndef total(x_ptr, out_ptr, n, BLOCK: tl.constexpr):\n    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)\n" \
          "    tl.atomic_add(out_ptr, tl.sum(tl.load(x_ptr + offs, mask=offs < n, other=0.0), axis=0))\n"
    fn = emitted(gpu, b.compile_triton(src), "total")
    for n, block, threads in [(1000, 1024, 256), (100003, 2048, 128), (5, 64, 32)]:
        x = np.random.default_rng(n).integers(-8, 9, n).astype(np.float32)
        out = dev(gpu, np.zeros(1, np.float32))
        fn.launch((n + block - 1) // block, threads, 0, [dev(gpu, x), out, b.i64(n), b.i64(block)])
        assert out.to_numpy(np.float32)[0] == x.sum(dtype=np.float64), (n, block, threads)
    # tl.min over int32, one atomic per warp
    src = "@triton.jit\ndef lowest(x_ptr, out_ptr, n, BLOCK: tl.constexpr):\n    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)\n" \
          "    tl.atomic_min(out_ptr, tl.min(tl.load(x_ptr + offs, mask=offs < n, other=2147483647), axis=0))\n"
    fn = emitted(gpu, b.compile_triton(src, pointee={"x_ptr": "i32", "out_ptr": "i32"}), "lowest")
    x = w.u32(5, 70001).view(np.int32)
    out = dev(gpu, np.array([2**31 - 1], np.int32))
    fn.launch((70001 + 4095) // 4096, 256, 0, [dev(gpu, x), out, b.i64(70001), b.i64(4096)])
    assert int(out.to_numpy(np.int32)[0]) == int(x.min())


@pytest.mark.parametrize("level", [0, 2])
def test_kernel_written_with_helper_functions(gpu, level):
    # four @triton.jit helpers inlined into one entry; many programs, ragged n, nothing past n touched
    fn = emitted(gpu, kt.saxpy_helpers(), "saxpy_kernel", level)
    block = 512
    for n in (1, 777, (1 << 16) + 3):
        x = w.f32_pm1(21, n); y = w.f32_pm1(22, n)
        programs = (n + block - 1) // block
        out = dev(gpu, np.full(programs * block + 8, -1.0, np.float32))
        fn.launch(programs, 128, 0, [dev(gpu, x), dev(gpu, y), out, b.i64(n), b.i64(block)])
        got = out.to_numpy(np.float32)
        assert np.array_equal(got[:n], np.float32(2.5) * x + y) and np.all(got[n:] == -1.0), (n, level)


@pytest.mark.parametrize("op, np_red, other, init", [("max", np.max, "-2147483648", -2**31), ("min", np.min, "2147483647", 2**31 - 1),
                                                     ("max", np.max, "5", -2**31), ("add", None, "0", 0)])
def test_int32_reduction_takes_vectors_and_stays_exact(gpu, op, np_red, other, init):
    # int32 reductions read the program's consecutive lanes as 16-byte vectors.  Ragged sizes (a last program that
    # is partly or wholly masked off), a base that is not 16-byte aligned (the one-word loop takes everything), a
    # block that is not a multiple of four, an `other` that changes the answer when a lane is masked off, and a
    # sum that wraps must all give the bits of the lane-by-lane definition.
    red = "sum" if op == "add" else op
    src = f"@triton.jit\ndef red(x_ptr, out_ptr, n, BLOCK: tl.constexpr):\n    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)\n" \
          f"    tl.atomic_{op}(out_ptr, tl.{red}(tl.load(x_ptr + offs, mask=offs < n, other={other}), axis=0))\n"
    bir = b.compile_triton(src, pointee={"x_ptr": "i32", "out_ptr": "i32"})
    assert "load v4i32 ptr.global" in bir
    fn = emitted(gpu, bir, "red")
    for n, block, threads, shift in [(1 << 20, 8192, 128, 0), (100003, 2048, 128, 0), (100003, 2048, 128, 1), (5, 64, 32, 0), (777, 100, 64, 0), (4096, 1024, 256, 3),
                                     (9000, 4096, 128, 0)]:
        x = w.u32(n + 17, n + 4).view(np.int32)
        if op == "max" and other == "5":
            x = np.minimum(x, -1)                    # every element is negative: a masked-off lane's 5 must win when there is one
        dx = dev(gpu, x)
        out = dev(gpu, np.array([init], np.int32))
        programs = (n + block - 1) // block
        fn.launch(programs, threads, 0, [b.ptr(dx.device_ptr() + 4 * shift), out, b.i64(n), b.i64(block)])
        data = x[shift:shift + n]
        if op == "add":
            want = int(data.astype(np.int64).sum() & 0xffffffff)
            got = int(out.to_numpy(np.int32)[0]) & 0xffffffff
        else:
            want = int(np_red(data))
            if programs * block > n:
                want = max(want, int(other)) if op == "max" else min(want, int(other))
            got = int(out.to_numpy(np.int32)[0])
        assert got == want, (n, block, threads, shift)
