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
@pytest.mark.parametrize("shape", [(2560, 1920, 64), (2560, 1920, 48), (4096, 4736, 32), (2432, 2048, 16), (2048, 4096, 1024), (1024, 4096, 2048)])
def test_sgemm_tail_wave(gpu, how, shape):
    # A last wave that does not fill the 296 CTA slots is worked off by stream units over the tail tiles' K slabs:
    # 300 tiles (tail 4: 16 units of one slab for K = 64, 12 for K = 48), 1184 tiles (no tail), 304 tiles with one
    # slab per tile (nothing to stream), 512 tiles (tail 216: 295 units of 47 slabs, which cross tile boundaries at
    # 64), 256 tiles (less than one wave: 293 units of 112 of a tile's 128 slabs).
    # Small integers: every partial sum is exact, so any cut of K must give the same bits; run
    # twice, since a streamed tail leaves its tickets behind for the next launch.
    M, N, K = shape
    A, B, _ = sgemm_fixture(M, N, K)
    want = (A.astype(np.float64) @ B.astype(np.float64)).astype(np.float32)   # exact: the sums stay far below 2^53
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
        fn = emitted(gpu, kb.matmul_f16(M, N, K, b_is_nk, per_cta=(how == "emitted_per_cta")), "matmul_kernel")
        fn.tune("pair", 0 if how == "emitted_one_sm" else 1)
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


PAIR_VARIANTS = ["pair_direct", "pair_lines", "pair_bulk", "pair_bulk_deep", "pair_lines_narrow", "pair_relay"]


@pytest.mark.parametrize("b_is_nk", [True, False])
@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 768, 192), (4864, 4096, 192)])
def test_matmul_f16_kernel_forms_agree(gpu, b_is_nk, shape):
    # Every hand-written form (one CTA per tile, one SM per 128x256 tile, CTA pairs with each of the
    # four epilogues) accumulates in the same order, so the results must agree bit for bit; the large
    # shape wraps the stage ring, both accumulators and the staging pieces many times.
    M, N, K = shape
    A = w.f16_normal01(w.SEEDS["matmul_f16"] + 11, M * K).reshape(M, K)
    B = w.f16_normal01(w.SEEDS["matmul_f16"] + 12, K * N).reshape(K, N)
    dA, dB = dev(gpu, A), dev(gpu, np.ascontiguousarray(B.T) if b_is_nk else B)
    status = dev(gpu, np.zeros(1, np.int32))
    results = {}
    for variant in ["one_cta_128", "one_sm_256"] + PAIR_VARIANTS:
        dC = dev(gpu, np.full((M, N), np.nan, np.float16))
        kernels.matmul_f16_variant(dA, dB, dC, M, N, K, variant, b_is_nk=b_is_nk, status=status)
        gpu.synchronize()
        assert status.to_numpy(np.int32)[0] == 0, variant
        results[variant] = dC.to_numpy(np.float16).reshape(M, N).view(np.uint16)
        dC.free()
    assert np.isfinite(results["one_cta_128"].view(np.float16)).all()
    for variant, got in results.items():
        assert np.array_equal(got, results["one_cta_128"]), variant


@pytest.mark.parametrize("variant", ["pair_direct", "pair_lines", "pair_bulk", "pair_bulk_deep", "pair_lines_narrow", "pair_relay", "auto"])
@pytest.mark.parametrize("n_peers", [1, 7])
def test_fused_gather_into_loop_back_peers(gpu, orc, variant, n_peers):
    # The fused matmul + gather on ONE GPU: the "peers" are further buffers of this GPU, so the peer
    # stores of the epilogue are exercised without a second device.  The rank's rows must land at the
    # same offset of every buffer, the other rows of every buffer must stay untouched.
    M_all, N, K, rows, row0 = 1024, 512, 256, 256, 512
    A = w.f16_normal01(w.SEEDS["matmul_f16"] + 21, rows * K).reshape(rows, K)
    B = w.f16_normal01(w.SEEDS["matmul_f16"] + 22, K * N).reshape(K, N)
    want = orc_matmul_f16_rows(orc, A, B, N, False, 0, rows)
    dA, dB = dev(gpu, A), dev(gpu, B)
    poison = np.full((M_all, N), -7.0, np.float16)
    bufs = [dev(gpu, poison) for _ in range(1 + n_peers)]
    status = dev(gpu, np.zeros(1, np.int32))
    mine = bufs[0].device_ptr() + row0 * N * 2
    others = [b_.device_ptr() + row0 * N * 2 for b_ in bufs[1:]]
    for _ in range(2):
        kernels.matmul_f16_variant(dA, dB, mine, rows, N, K, variant, peer_ptrs=others, status=status)
    gpu.synchronize()
    assert status.to_numpy(np.int32)[0] == 0
    first = None
    for b_ in bufs:
        got = b_.to_numpy(np.float16).reshape(M_all, N)
        assert np.array_equal(got[:row0], poison[:row0]) and np.array_equal(got[row0 + rows:], poison[row0 + rows:])
        assert rel_fro(got[row0:row0 + rows], want) <= F16_TOL
        if first is None:
            first = got[row0:row0 + rows].view(np.uint16).copy()
        assert np.array_equal(got[row0:row0 + rows].view(np.uint16), first)


@pytest.mark.parametrize("n_peers", [1, 7])
def test_emitted_fused_gather_into_loop_back_peers_f16(gpu, orc, n_peers):
    # basalt_rt_launch_gather on the emitted tcgen05 kernel (two-SM entry), the "peers" being further
    # result buffers on this GPU: same bits in every buffer, nothing outside the rank's rows touched,
    # and the same bits as the plain launch.
    M_all, N, K, rows, row0 = 1024, 512, 256, 256, 512
    A = w.f16_normal01(w.SEEDS["matmul_f16"] + 21, rows * K).reshape(rows, K)
    B = w.f16_normal01(w.SEEDS["matmul_f16"] + 22, K * N).reshape(K, N)
    want = orc_matmul_f16_rows(orc, A, B, N, False, 0, rows)
    dA, dB = dev(gpu, A), dev(gpu, B)
    poison = np.full((M_all, N), -7.0, np.float16)
    bufs = [dev(gpu, poison) for _ in range(1 + n_peers)]
    fn = emitted(gpu, kb.matmul_f16(rows, N, K), "matmul_kernel")
    go = fn.bind_gather((N // 128, rows // 128), 128, 0, [dA, dB, b.ptr(bufs[0].device_ptr() + row0 * N * 2)],
                        [b_.device_ptr() + row0 * N * 2 for b_ in bufs[1:]])
    for _ in range(2):
        go()
    gpu.synchronize()
    assert fn.status() == 0
    plain = dev(gpu, np.zeros((rows, N), np.float16))
    fn.launch((N // 128, rows // 128), 128, 0, [dA, dB, plain])
    first = plain.to_numpy(np.float16).reshape(rows, N).view(np.uint16)
    for b_ in bufs:
        got = b_.to_numpy(np.float16).reshape(M_all, N)
        assert np.array_equal(got[:row0], poison[:row0]) and np.array_equal(got[row0 + rows:], poison[row0 + rows:])
        assert rel_fro(got[row0:row0 + rows], want) <= F16_TOL
        assert np.array_equal(got[row0:row0 + rows].view(np.uint16), first)


@pytest.mark.parametrize("shape,rounds", [((256, 256, 64), 0), ((2560, 1920, 64), 0), ((512, 4096, 256), 0), ((512, 4096, 2048), 0), ((512, 4096, 2048), 3)])
def test_emitted_fused_gather_into_loop_back_peers_f32(gpu, shape, rounds):
    # the FFMA matmul's gathering epilogue, whole tiles and the streamed tail wave (300 tiles: the last four are
    # summed from one-slab segments by the segment that finishes last, which then stores to every buffer); the
    # third and fourth shapes are 8-GPU shards: 128 tiles, less than half a wave, worked off by one round of stream
    # units (K = 256: seven slabs to a unit) or, with enough slabs, by two rounds -- three when tuned so
    rows, N, K = shape
    A, B, _ = sgemm_fixture(rows, N, K)
    want = (A.astype(np.float64) @ B.astype(np.float64)).astype(np.float32)   # exact: small integers
    dA, dB = dev(gpu, A), dev(gpu, B)
    row0, M_all = 128, rows + 256
    poison = np.full((M_all, N), -7.0, np.float32)
    bufs = [dev(gpu, poison) for _ in range(3)]
    fn = emitted(gpu, kb.sgemm_cta128(rows, N, K), "sgemm_f32")
    fn.tune("tail_rounds", rounds)
    go = fn.bind_gather((N // 128, rows // 128), 256, 0, [dA, dB, b.ptr(bufs[0].device_ptr() + row0 * N * 4)],
                        [b_.device_ptr() + row0 * N * 4 for b_ in bufs[1:]])
    for _ in range(2):
        go()
    gpu.synchronize()
    for b_ in bufs:
        got = b_.to_numpy(np.float32).reshape(M_all, N)
        assert np.array_equal(got[:row0], poison[:row0]) and np.array_equal(got[row0 + rows:], poison[row0 + rows:])
        assert np.array_equal(got[row0:row0 + rows], want)


def test_launch_gather_refuses_kernels_without_the_epilogue(gpu):
    fn = emitted(gpu, kb.load("vadd_i32"), "vadd_i32")
    x = dev(gpu, np.zeros(256, np.int32))
    with pytest.raises(b.CudaError) as e:
        fn.bind_gather(1, 256, 0, [x, x, x, b.i32(256)], [x.device_ptr()])()
    assert e.value.kind == 4
    odd = emitted(gpu, kb.matmul_f16(384, 256, 64), "matmul_kernel")     # three tile rows: only the one-SM entry can run it
    c = dev(gpu, np.zeros((384, 256), np.float16))
    with pytest.raises(b.CudaError) as e:
        odd.bind_gather((2, 3), 128, 0, [dev(gpu, np.zeros((384, 64), np.float16)), dev(gpu, np.zeros((64, 256), np.float16)), c], [c.device_ptr()])()
    assert e.value.kind == 4 and "even" in e.value.message
    # the multicast form refuses the same kernels, and an address that is null or not 16-byte aligned
    with pytest.raises(b.CudaError) as e:
        fn.bind_gather_multicast(1, 256, 0, [x, x, x, b.i32(256)], x.device_ptr())()
    assert e.value.kind == 4
    ok = emitted(gpu, kb.matmul_f16(256, 256, 64), "matmul_kernel")
    c2 = dev(gpu, np.zeros((256, 256), np.float16))
    prm = [dev(gpu, np.zeros((256, 64), np.float16)), dev(gpu, np.zeros((64, 256), np.float16)), c2]
    for bad in (0, c2.device_ptr() + 2):
        with pytest.raises(b.CudaError) as e:
            ok.bind_gather_multicast((2, 2), 128, 0, prm, bad)()
        assert e.value.kind == 4
