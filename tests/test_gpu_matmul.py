"""Parity of the two matmul workloads against the CPU oracle.

fp32 SGEMM: relative Frobenius error <= 1e-4 (the benchmark's stated tolerance; the oracle
multiplies and adds separately in ascending k, the device kernels use FFMA and a tiled order).
fp16 matmul with fp32 accumulation: <= 2e-3 relative.  Small-integer inputs, where every partial
sum is exactly representable, must match exactly.  At the benchmark's full sizes the oracle is
evaluated on sampled rows, and the whole result is checked with Freivalds' identity
C*v == A*(B*v), a size-independent property."""
import ctypes
import os

import numpy as np
import pytest

import basalt_b200 as b
from basalt_b200 import kernels, kernels_bir as kb, workloads as w
from _gpu import dev, emitted
from _util import orc_matmul_f16_rows, orc_sgemm_rows, rel_fro, sgemm_fixture, vp

pytestmark = pytest.mark.gpu
SGEMM_TOL = 1e-4
F16_TOL = 2e-3


def freivalds(A, B, C, seed=1):
    v = np.random.default_rng(seed).standard_normal(B.shape[1])
    lhs = C.astype(np.float64) @ v
    rhs = A.astype(np.float64) @ (B.astype(np.float64) @ v)
    return float(np.linalg.norm(lhs - rhs) / np.linalg.norm(rhs))


def run_sgemm(gpu, how, A, B):
    M, K = A.shape
    N = B.shape[1]
    dA, dB, dC = dev(gpu, A), dev(gpu, B), dev(gpu, np.full((M, N), np.nan, np.float32))
    if how == "hand":
        kernels.sgemm_f32(dA, dB, dC, M, N, K)
        gpu.synchronize()
    elif how == "cta128":
        emitted(gpu, kb.sgemm_cta128(M, N, K), "sgemm_f32").launch((N // 128, M // 128), 256, 0, [dA, dB, dC])
    else:
        emitted(gpu, kb.load("sgemm_tile16"), "sgemm_tile16").launch((N // 16, M // 16), (16, 16), 0, [dA, dB, dC, b.i32(M), b.i32(N), b.i32(K)])
    return dC.to_numpy(np.float32).reshape(M, N)


@pytest.mark.parametrize("how", ["hand", "cta128", "tile16"])
def test_sgemm_exact_on_small_integers(gpu, how):
    A, B, _ = sgemm_fixture(128, 256, 64)
    got = run_sgemm(gpu, how, A, B)
    assert np.array_equal(got, (A.astype(np.int64) @ B.astype(np.int64)).astype(np.float32))


@pytest.mark.parametrize("how", ["hand", "cta128", "tile16"])
@pytest.mark.parametrize("shape", [(128, 128, 16), (256, 384, 80), (512, 256, 512)])
def test_sgemm_vs_oracle(gpu, orc, how, shape):
    M, N, K = shape
    A = w.f32_pm1(w.SEEDS["sgemm_f32"], M * K).reshape(M, K)
    B = w.f32_pm1(w.SEEDS["sgemm_f32"] + 1, K * N).reshape(K, N)
    got = run_sgemm(gpu, how, A, B)
    assert rel_fro(got, orc_sgemm_rows(orc, A, B, 0, M)) <= SGEMM_TOL


@pytest.mark.parametrize("how", ["hand", "cta128"])
def test_sgemm_full_size(gpu, orc, how):
    M = N = K = 4096
    A = w.f32_pm1(w.SEEDS["sgemm_f32"], M * K).reshape(M, K)
    B = w.f32_pm1(w.SEEDS["sgemm_f32"] + 1, K * N).reshape(K, N)
    got = run_sgemm(gpu, how, A, B)
    assert np.isfinite(got).all()
    rows = [0, 1, 127, 128, 2047, 2048, 4095] + list(np.random.default_rng(2).integers(0, M, 9))
    for r in rows:
        assert rel_fro(got[r], orc_sgemm_rows(orc, A, B, int(r), int(r) + 1)[0]) <= SGEMM_TOL, r
    assert freivalds(A, B, got) <= SGEMM_TOL


@pytest.mark.parametrize("how", ["hand", "cta128"])
@pytest.mark.parametrize("shape", [(2560, 1920, 64), (2560, 1920, 48), (4096, 4736, 32), (2432, 2048, 16)])
def test_sgemm_tail_wave(gpu, how, shape):
    # More tiles than resident CTAs with a sparse last wave: 300 tiles (tail 4, split in 4 or, for
    # K = 48, in 3 parts), 1184 tiles (no tail on 296 slots), 304 tiles with K too short to split.
    # Small integers: every partial sum is exact, so any split of K must give the same bits; run
    # twice, since a split tail leaves its tickets behind for the next launch.
    M, N, K = shape
    A, B, _ = sgemm_fixture(M, N, K)
    want = (A.astype(np.int64) @ B.astype(np.int64)).astype(np.float32)
    for _ in range(2):
        assert np.array_equal(run_sgemm(gpu, how, A, B), want)


def run_matmul_f16(gpu, how, A, B, N, b_is_nk):
    M, K = A.shape
    dA, dB = dev(gpu, A), dev(gpu, B)
    dC = dev(gpu, np.full((M, N), np.nan, np.float16))
    status = dev(gpu, np.zeros(1, np.int32))
    if how == "hand":
        kernels.matmul_f16(dA, dB, dC, M, N, K, b_is_nk, status)
        gpu.synchronize()
        assert status.to_numpy(np.int32)[0] == 0, "a bounded wait inside the kernel expired"
    else:
        # "emitted" takes the two-SM entry whenever the grid is even in x and y; "emitted_one_sm" keeps the one-SM entry
        if how == "emitted_one_sm":
            os.environ["BASALT_RT_NO_PAIR"] = "1"
        try:
            fn = emitted(gpu, kb.matmul_f16(M, N, K, b_is_nk, per_cta=(how == "emitted_per_cta")), "matmul_kernel")
        finally:
            os.environ.pop("BASALT_RT_NO_PAIR", None)
        fn.launch((N // 128, M // 128), 128, 0, [dA, dB, dC])
        assert fn.status() == 0, "a bounded wait inside the emitted kernel expired"
    return dC.to_numpy(np.float16).reshape(M, N)


@pytest.mark.parametrize("how", ["hand", "emitted", "emitted_one_sm", "emitted_per_cta"])
@pytest.mark.parametrize("b_is_nk", [True, False])
@pytest.mark.parametrize("shape", [(128, 128, 64), (128, 128, 256), (256, 384, 192), (256, 512, 192), (384, 256, 64), (2304, 512, 64), (256, 256, 1024)])
def test_matmul_f16_exact_on_small_integers(gpu, how, b_is_nk, shape):
    M, N, K = shape
    A, B, _ = sgemm_fixture(M, N, K)
    A = (A % 4).astype(np.float16); B = (B % 3).astype(np.float16)   # sums stay below 2048: exact in f16
    want = (A.astype(np.int64) @ B.astype(np.int64)).astype(np.float16)
    Bdev = np.ascontiguousarray(B.T) if b_is_nk else B
    got = run_matmul_f16(gpu, how, A, Bdev, N, b_is_nk)
    bad = np.argwhere(got != want)
    assert len(bad) == 0, f"{len(bad)} mismatches, first at {bad[:5].tolist()}: got {got[tuple(bad[0])]}, want {want[tuple(bad[0])]}"


@pytest.mark.parametrize("how", ["hand", "emitted"])
@pytest.mark.parametrize("b_is_nk", [True, False])
def test_matmul_f16_vs_oracle(gpu, orc, how, b_is_nk):
    M, N, K = 256, 512, 1024
    A = w.f16_normal01(w.SEEDS["matmul_f16"], M * K).reshape(M, K)
    B = w.f16_normal01(w.SEEDS["matmul_f16"] + 1, K * N).reshape(K, N)
    Bdev = np.ascontiguousarray(B.T) if b_is_nk else B
    got = run_matmul_f16(gpu, how, A, Bdev, N, b_is_nk)
    want = orc_matmul_f16_rows(orc, A, Bdev, N, b_is_nk, 0, M)
    assert rel_fro(got, want) <= F16_TOL


@pytest.mark.parametrize("b_is_nk", [True, False])
def test_matmul_f16_pairs_over_many_waves(gpu, b_is_nk):
    # 4864 x 4096: 19 x 16 tiles of 256 x 256 on 74 pairs of SMs (4.1 waves: both accumulators and all six
    # stages wrap several times, the last band has 3 tile rows); the two entries must agree bit for bit
    M, N, K = 4864, 4096, 192
    A = w.f16_normal01(w.SEEDS["matmul_f16"] + 7, M * K).reshape(M, K)
    B = w.f16_normal01(w.SEEDS["matmul_f16"] + 8, K * N).reshape(K, N)
    Bdev = np.ascontiguousarray(B.T) if b_is_nk else B
    pair = run_matmul_f16(gpu, "emitted", A, Bdev, N, b_is_nk)
    one = run_matmul_f16(gpu, "emitted_one_sm", A, Bdev, N, b_is_nk)
    hand = run_matmul_f16(gpu, "hand", A, Bdev, N, b_is_nk)
    assert np.isfinite(pair).all()
    assert np.array_equal(pair.view(np.uint16), one.view(np.uint16)) and np.array_equal(pair.view(np.uint16), hand.view(np.uint16))


@pytest.mark.parametrize("how", ["hand", "emitted", "emitted_one_sm"])
def test_matmul_f16_full_size(gpu, orc, how):
    M = N = K = 8192
    A = np.empty(M * K, np.float16); B = np.empty(K * N, np.float16)
    orc.orc_fill_f16_normal01(ctypes.c_uint64(w.SEEDS["matmul_f16"]), ctypes.c_int64(M * K), vp(A))
    orc.orc_fill_f16_normal01(ctypes.c_uint64(w.SEEDS["matmul_f16"] + 1), ctypes.c_int64(K * N), vp(B))
    A = A.reshape(M, K); B = B.reshape(K, N)
    got = run_matmul_f16(gpu, how, A, B, N, False)
    assert np.isfinite(got).all()
    for r in [0, 127, 128, 4095, 4096, 8191, 777, 5000]:
        want = orc_matmul_f16_rows(orc, A, B, N, False, r, r + 1)[0]
        assert rel_fro(got[r], want) <= F16_TOL, r
    # Freivalds on a row block (float64 on the host: keep it to 1024 rows)
    blk = slice(3072, 4096)
    v = np.random.default_rng(4).standard_normal(N)
    rhs = A[blk].astype(np.float64) @ (B.astype(np.float32) @ v.astype(np.float32)).astype(np.float64)
    lhs = got[blk].astype(np.float64) @ v
    assert np.linalg.norm(lhs - rhs) / np.linalg.norm(rhs) <= F16_TOL
