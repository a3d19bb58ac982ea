"""Helpers shared by the tests: fixture inputs built from the formulas of the reference's
examples (examples/cpu_launch_*.c), and calls into the CPU oracle."""
import ctypes

import numpy as np


def vp(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def sgemm_fixture(m, n, k):
    """A=((3i+j)%7)+1, B=((i+5j)%7)+1, C=(i+j)%4 (examples/cpu_launch_tiled_sgemm.c:28-34,
    cpu_launch_triton_matmul.c:47-61): small integers, so every product and sum is exact."""
    i = np.arange(m)[:, None]
    a = ((3 * i + np.arange(k)[None, :]) % 7 + 1).astype(np.float32)
    b = ((np.arange(k)[:, None] + 5 * np.arange(n)[None, :]) % 7 + 1).astype(np.float32)
    c = ((i + np.arange(n)[None, :]) % 4).astype(np.float32)
    return a, b, c


def rel_fro(x, ref):
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.linalg.norm(x - ref) / max(np.linalg.norm(ref), 1e-30))


def orc_sgemm_rows(orc, A, B, row0, row1):
    M, K = A.shape
    N = B.shape[1]
    out = np.empty((row1 - row0, N), dtype=np.float32)
    orc.orc_sgemm_f32_rows(vp(A), vp(B), vp(out), M, N, K, row0, row1)
    return out


def orc_matmul_f16_rows(orc, A, B, N, b_is_nk, row0, row1):
    M, K = A.shape
    out = np.empty((row1 - row0, N), dtype=np.float16)
    orc.orc_matmul_f16_rows(vp(A), vp(B), vp(out), M, N, K, int(b_is_nk), row0, row1)
    return out
