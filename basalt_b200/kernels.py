"""The hand-written sm_100a kernels of include/basalt_b200_kernels.h. Every argument is a device
pointer (int) or DeviceBuffer; launches are asynchronous on `stream`."""
from __future__ import annotations

import ctypes as C

from ._lib import lib
from .runtime import DeviceBuffer


class KernelError(Exception):
    pass


def _p(x) -> C.c_void_p:
    return C.c_void_p(x.device_ptr() if isinstance(x, DeviceBuffer) else int(x))


def _check(rc: int):
    if rc:
        raise KernelError(f"{lib.basalt_k_last_error().decode()} (code {rc})")


def vadd_i32(a, b, c, n: int, stream=None):
    _check(lib.basalt_k_vadd_i32(_p(a), _p(b), _p(c), n, C.c_void_p(stream)))


def max_i32(x, n: int, out, stream=None):
    """atomicMax(out, max(x[0..n))); out must already hold the running maximum."""
    _check(lib.basalt_k_max_i32(_p(x), n, _p(out), C.c_void_p(stream)))


def helper_chain_u32(inp, out, n: int, stream=None):
    _check(lib.basalt_k_helper_chain_u32(_p(inp), _p(out), n, C.c_void_p(stream)))


def imad_peak(out, out_elems: int, iters: int, stream=None) -> int:
    """Launches the INT32-pipe microbenchmark; returns the number of multiply-adds it executes."""
    n = C.c_int64()
    _check(lib.basalt_k_imad_peak(_p(out), out_elems, iters, C.byref(n), C.c_void_p(stream)))
    return n.value


def sgemm_f32(A, B, Cm, M: int, N: int, K: int, stream=None):
    _check(lib.basalt_k_sgemm_f32(_p(A), _p(B), _p(Cm), M, N, K, C.c_void_p(stream)))


def sgemm_f32_static_workspace(A, B, Cm, M: int, N: int, K: int, stream=None):
    """sgemm_f32 with its tail-wave workspace in a static device array: the call allocates nothing."""
    _check(lib.basalt_k_sgemm_f32_static_workspace(_p(A), _p(B), _p(Cm), M, N, K, C.c_void_p(stream)))


def matmul_f16_allgather(A, B, Cm, M: int, N: int, K: int, peer_ptrs, b_is_nk: bool = False, status=None, stream=None):
    """This rank's rows of C = A * B, stored to `Cm` and, from the same epilogue, to each address in
    `peer_ptrs` (the same rows of the other ranks' result buffers, peer-mapped).  Follow it with the
    peer exchange on the same stream: that is the barrier after which every rank holds all rows."""
    arr = (C.c_void_p * max(1, len(peer_ptrs)))(*[C.c_void_p(int(p)) for p in peer_ptrs])
    _check(lib.basalt_k_matmul_f16_allgather(_p(A), _p(B), _p(Cm), M, N, K, int(b_is_nk), arr, len(peer_ptrs),
                                             _p(status) if status is not None else None, C.c_void_p(stream)))


MATMUL_VARIANTS = {"auto": 0, "one_cta_128": 1, "one_sm_256": 2, "pair_direct": 3, "pair_lines": 4, "pair_bulk": 5, "pair_bulk_deep": 6, "pair_lines_narrow": 7, "pair_relay": 8}


def matmul_f16_variant(A, B, Cm, M: int, N: int, K: int, variant: str, peer_ptrs=(), b_is_nk: bool = False, status=None, stream=None):
    """basalt_k_matmul_f16_variant: the product through one named kernel form (MATMUL_VARIANTS), with
    the result also stored behind each address of `peer_ptrs` (CTA-pair forms only)."""
    arr = (C.c_void_p * max(1, len(peer_ptrs)))(*[C.c_void_p(int(p)) for p in peer_ptrs])
    _check(lib.basalt_k_matmul_f16_variant(_p(A), _p(B), _p(Cm), M, N, K, int(b_is_nk), MATMUL_VARIANTS[variant], arr, len(peer_ptrs),
                                           _p(status) if status is not None else None, C.c_void_p(stream)))


def matmul_f16(A, B, Cm, M: int, N: int, K: int, b_is_nk: bool = False, status=None, stream=None):
    _check(lib.basalt_k_matmul_f16(_p(A), _p(B), _p(Cm), M, N, K, int(b_is_nk), _p(status) if status is not None else None,
                                   C.c_void_p(stream)))


FILL_KINDS = {"u32": 0, "i32_pm30": 1, "f32_pm1": 2, "f16_normal01": 3}


def fill(kind: str, seed: int, n: int, out, start: int = 0, stream=None):
    """Draws start .. start+n-1 of the seeded stream into device memory, as workloads.{u32, i32_pm30,
    f32_pm1, f16_normal01} produce them on the host (identical bytes)."""
    _check(lib.basalt_k_fill(FILL_KINDS[kind], seed, start, n, _p(out), C.c_void_p(stream)))


def sgemm_f32_variant(A, B, Cm, M: int, N: int, K: int, no_tail_split: bool = False, cp_async: bool = False, warp_rows: bool = False, stream=None):
    """basalt_k_sgemm_f32_variant: the hand-written SGEMM with parts of its schedule switched (A/B timing)."""
    flags = (1 if no_tail_split else 0) | (2 if cp_async else 0) | (4 if warp_rows else 0)
    _check(lib.basalt_k_sgemm_f32_variant(_p(A), _p(B), _p(Cm), M, N, K, flags, C.c_void_p(stream)))
