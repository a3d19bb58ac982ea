"""The SGEMM entry point that allocates nothing (its tail-wave workspace is a static device array):
through the C ABI it gives the same bits as the entry point it is a variant of, on two calls in a
row, for shapes with and without a split tail wave.  Collected last; passes alone and after the
other tests."""
import numpy as np
import pytest

from basalt_b200 import kernels, workloads as w
from _gpu import dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(2560, 1920, 64), (2560, 1920, 48), (256, 384, 80), (4096, 4736, 32)])
def test_static_workspace_sgemm_matches_the_allocating_entry_point(gpu, shape):
    M, N, K = shape      # 300 tiles: a tail of 4 split in 4 (K = 64) or 3 (K = 48) parts; 6 tiles; 1184 tiles, no tail
    A = w.f32_pm1(71, M * K).reshape(M, K)
    B = w.f32_pm1(72, K * N).reshape(K, N)
    dA, dB = dev(gpu, A), dev(gpu, B)
    want = dev(gpu, np.full((M, N), np.nan, np.float32))
    kernels.sgemm_f32(dA, dB, want, M, N, K)
    gpu.synchronize()
    want = want.to_numpy(np.float32)
    assert np.isfinite(want).all()
    for call in range(2):
        got = dev(gpu, np.full((M, N), np.nan, np.float32))
        kernels.sgemm_f32_static_workspace(dA, dB, got, M, N, K)
        gpu.synchronize()
        assert np.array_equal(got.to_numpy(np.float32).view(np.uint32), want.view(np.uint32)), (shape, call)
