"""ctypes binding of libbasalt_b200.so, the C-ABI library of include/basalt_b200.h and
include/basalt_b200_kernels.h.  There is no Python fallback for anything in it: if the library has
not been built, importing this module raises."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbasalt_b200.so")


class EmitOpts(C.Structure):
    _fields_ = [("target_variant", C.c_char_p), ("opt_level", C.c_int), ("out_name_hint", C.c_char_p), ("snap", C.c_int)]


class DiagStruct(C.Structure):
    _fields_ = [("code", C.c_char * 8), ("message", C.c_char * 504)]


class RtError(C.Structure):
    _fields_ = [("kind", C.c_int), ("code", C.c_int), ("call", C.c_char * 64), ("message", C.c_char * 440)]


class _ArgValue(C.Union):
    _fields_ = [("i32", C.c_int32), ("i64", C.c_int64), ("f32", C.c_float), ("f64", C.c_double)]


class RtArg(C.Structure):
    _fields_ = [("kind", C.c_int), ("value", _ArgValue), ("host", C.c_void_p), ("bytes", C.c_size_t)]


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m basalt_b200.build` (needs nvcc). "
            "basalt_b200 has no CPU or pure-Python path.")
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    vp, cp, sz, u64, i64, i32p = C.c_void_p, C.c_char_p, C.c_size_t, C.c_uint64, C.c_int64, C.POINTER(C.c_int32)
    P = C.POINTER
    sig = {
        "basalt_b200_name": (cp, []),
        "basalt_b200_supports": (C.c_int, [cp, sz, C.c_char * 8]),
        "basalt_b200_emit": (C.c_int, [cp, sz, P(EmitOpts), P(vp), P(sz), P(DiagStruct)]),
        "basalt_b200_optimize": (C.c_int, [cp, sz, P(EmitOpts), P(vp), P(sz), P(DiagStruct)]),
        "basalt_b200_roundtrip": (C.c_int, [cp, sz, P(vp), P(sz), P(DiagStruct)]),
        "basalt_b200_compile_cuda": (C.c_int, [cp, sz, P(vp), P(sz), P(DiagStruct)]),
        "basalt_b200_compile_triton": (C.c_int, [cp, sz, cp, P(vp), P(sz), P(DiagStruct)]),
        "basalt_b200_free": (None, [vp]),
        "basalt_rt_last_error": (None, [P(RtError)]),
        "basalt_rt_driver_load": (C.c_int, [P(vp)]),
        "basalt_rt_driver_unload": (None, [vp]),
        "basalt_rt_device_count": (C.c_int, [vp, P(C.c_int)]),
        "basalt_rt_ctx_create": (C.c_int, [vp, C.c_int, P(vp)]),
        "basalt_rt_ctx_destroy": (None, [vp]),
        "basalt_rt_device_attr": (C.c_int, [vp, C.c_int, P(C.c_int)]),
        "basalt_rt_module_load": (C.c_int, [vp, cp, P(vp)]),
        "basalt_rt_module_unload": (None, [vp]),
        "basalt_rt_get_function": (C.c_int, [vp, cp, P(vp)]),
        "basalt_rt_alloc": (C.c_int, [vp, sz, P(vp)]),
        "basalt_rt_buffer_free": (None, [vp]),
        "basalt_rt_buffer_ptr": (u64, [vp]),
        "basalt_rt_buffer_size": (sz, [vp]),
        "basalt_rt_copy_from_host": (C.c_int, [vp, vp, sz, vp]),
        "basalt_rt_copy_to_host": (C.c_int, [vp, vp, sz, vp]),
        "basalt_rt_host_alloc": (C.c_int, [vp, sz, P(vp)]),
        "basalt_rt_host_free": (None, [vp, vp]),
        "basalt_rt_launch": (C.c_int, [vp, C.c_uint32 * 3, C.c_uint32 * 3, C.c_uint32, vp, P(vp)]),
        "basalt_rt_function_tune": (C.c_int, [vp, C.c_char_p, C.c_int]),
        "basalt_rt_launch_gather": (C.c_int, [vp, C.c_uint32 * 3, C.c_uint32 * 3, C.c_uint32, vp, P(vp), P(u64), C.c_int]),
        "basalt_rt_launch_gather_multicast": (C.c_int, [vp, C.c_uint32 * 3, C.c_uint32 * 3, C.c_uint32, vp, P(vp), u64]),
        "basalt_rt_planned_geometry": (C.c_int, [vp, P(vp), C.c_uint32 * 3, C.c_uint32 * 3, P(C.c_uint32)]),
        "basalt_rt_ctx_sync": (C.c_int, [vp]),
        "basalt_rt_kernel_status": (C.c_int, [vp, i32p]),
        "basalt_rt_occupancy": (C.c_int, [vp, C.c_uint32, C.c_uint32, P(C.c_int), P(C.c_int)]),
        "basalt_rt_tail_plan": (None, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, P(C.c_uint32)]),
        "basalt_rt_stream_create": (C.c_int, [vp, P(vp)]),
        "basalt_rt_stream_destroy": (C.c_int, [vp, vp]),
        "basalt_rt_stream_sync": (C.c_int, [vp, vp]),
        "basalt_rt_event_create": (C.c_int, [vp, P(vp)]),
        "basalt_rt_event_destroy": (C.c_int, [vp, vp]),
        "basalt_rt_event_record": (C.c_int, [vp, vp, vp]),
        "basalt_rt_event_sync": (C.c_int, [vp, vp]),
        "basalt_rt_event_elapsed_ms": (C.c_int, [vp, vp, vp, P(C.c_float)]),
        "basalt_rt_cpu_launch": (C.c_int, [vp, vp, P(RtArg), C.c_int, i64, C.c_uint32]),
        "basalt_rt_shard_range": (None, [u64, C.c_int, C.c_int, u64, P(u64), P(u64)]),
        "basalt_rt_comm_unique_id": (C.c_int, [C.c_char * 128]),
        "basalt_rt_comm_init": (C.c_int, [vp, C.c_char * 128, C.c_int, C.c_int, P(vp)]),
        "basalt_rt_comm_destroy": (None, [vp]),
        "basalt_rt_allreduce_max_i32": (C.c_int, [vp, u64, u64, sz, vp]),
        "basalt_rt_allgather": (C.c_int, [vp, u64, u64, sz, vp]),
        "basalt_rt_ipc_export": (C.c_int, [vp, C.c_char * 64]),
        "basalt_rt_ipc_open": (C.c_int, [vp, C.c_char_p, P(u64)]),
        "basalt_rt_ipc_close": (C.c_int, [vp, u64]),
        "basalt_rt_copy_device_async": (C.c_int, [vp, u64, u64, sz, vp]),
        "basalt_rt_stream_wait_event": (C.c_int, [vp, vp, vp]),
        "basalt_rt_peer_group_create": (C.c_int, [vp, C.c_int, C.c_int, P(vp)]),
        "basalt_rt_peer_group_handle": (C.c_int, [vp, C.c_char * 64]),
        "basalt_rt_peer_group_connect": (C.c_int, [vp, C.c_char_p, sz]),
        "basalt_rt_peer_allreduce_max_i32": (C.c_int, [vp, u64, u64, C.c_int, C.c_int32, vp]),
        "basalt_rt_peer_max_i32": (C.c_int, [vp, u64, i64, u64, vp]),
        "basalt_rt_peer_group_status": (C.c_int, [vp, P(C.c_uint32)]),
        "basalt_rt_peer_group_destroy": (C.c_int, [vp]),
        "basalt_k_last_error": (cp, []),
        "basalt_k_vadd_i32": (C.c_int, [vp, vp, vp, i64, vp]),
        "basalt_k_max_i32": (C.c_int, [vp, i64, vp, vp]),
        "basalt_k_helper_chain_u32": (C.c_int, [vp, vp, i64, vp]),
        "basalt_k_imad_peak": (C.c_int, [vp, i64, C.c_int, P(C.c_int64), vp]),
        "basalt_k_sgemm_f32": (C.c_int, [vp, vp, vp, C.c_int, C.c_int, C.c_int, vp]),
        "basalt_k_sgemm_f32_variant": (C.c_int, [vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, vp]),
        "basalt_k_vadd_i32_waves": (C.c_int, [vp, vp, vp, i64, C.c_int, vp]),
        "basalt_k_max_i32_waves": (C.c_int, [vp, i64, vp, C.c_int, vp]),
        "basalt_k_helper_chain_u32_waves": (C.c_int, [vp, vp, i64, C.c_int, vp]),
        "basalt_k_sgemm_f32_static_workspace": (C.c_int, [vp, vp, vp, C.c_int, C.c_int, C.c_int, vp]),
        "basalt_k_matmul_f16": (C.c_int, [vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp]),
        "basalt_k_matmul_f16_allgather": (C.c_int, [vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, P(vp), C.c_int, vp, vp]),
        "basalt_k_fill": (C.c_int, [C.c_int, u64, u64, i64, vp, vp]),
        "basalt_k_matmul_f16_variant": (C.c_int, [vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, P(vp), C.c_int, vp, vp]),
        "basalt_k_max_i32_allreduce": (C.c_int, [vp, i64, vp, P(u64), C.c_int, C.c_int, C.c_uint32, vp, vp, vp, u64, vp]),
        "basalt_k_peer_allreduce_max_i32": (C.c_int, [P(u64), C.c_int, C.c_int, C.c_uint32, vp, vp, vp, u64, C.c_int, C.c_int32, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    lib._basalt_signatures = sig
    return lib


lib = _load()
