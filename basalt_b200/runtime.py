"""The launch side of the drop-in: mirrors of the reference runtime's types
(crates/basalt-runtime/src/lib.rs:34-42) over the C ABI -- CudaDriver, CudaContext, DeviceBuffer,
CudaModule, CudaFunction, CudaError -- with the additions the B200 path needs (streams, events,
pinned host memory, launch plans for tensor-map kernels, NCCL communicators)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import RtArg, RtError, lib


class CudaError(Exception):
    """CudaError (crates/basalt-runtime/src/error.rs:9-22). kind: 1 DriverNotFound,
    2 SymbolNotFound, 3 DriverCallFailed, 4 host-side check, 5 NCCL."""

    def __init__(self, kind: int, call: str, code: int, message: str):
        super().__init__(f"{call} failed with code {code}: {message}" if kind in (3, 5) else message)
        self.kind, self.call, self.code, self.message = kind, call, code, message


def _check(rc: int) -> None:
    if rc:
        e = RtError()
        lib.basalt_rt_last_error(C.byref(e))
        raise CudaError(e.kind, e.call.decode(), e.code, e.message.decode(errors="replace"))


def i32(v): return C.c_int32(int(v))
def i64(v): return C.c_int64(int(v))
def f32(v): return C.c_float(float(v))
def f64(v): return C.c_double(float(v))
def ptr(v): return C.c_uint64(int(v))


class CudaDriver:
    """CudaDriver (driver.rs:94-163)."""

    def __init__(self, handle):
        self._h = handle

    @staticmethod
    def load() -> "CudaDriver":
        h = C.c_void_p()
        _check(lib.basalt_rt_driver_load(C.byref(h)))
        return CudaDriver(h)

    def device_count(self) -> int:
        n = C.c_int()
        _check(lib.basalt_rt_device_count(self._h, C.byref(n)))
        return n.value

    def create_context(self, device_index: int = 0) -> "CudaContext":
        h = C.c_void_p()
        _check(lib.basalt_rt_ctx_create(self._h, device_index, C.byref(h)))
        return CudaContext(self, h, device_index)


class CudaContext:
    """CudaContext (context.rs:30-91); holds the device's primary context."""

    def __init__(self, driver: CudaDriver, handle, device_index: int):
        self.driver, self._h, self.device_index = driver, handle, device_index

    def close(self):
        if self._h:
            lib.basalt_rt_ctx_destroy(self._h)
            self._h = None

    def device_attr(self, attr: int) -> int:
        v = C.c_int()
        _check(lib.basalt_rt_device_attr(self._h, attr, C.byref(v)))
        return v.value

    def sm_count(self) -> int:
        return self.device_attr(16)   # CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT

    def load_module(self, ptx: str) -> "CudaModule":
        h = C.c_void_p()
        _check(lib.basalt_rt_module_load(self._h, ptx.encode(), C.byref(h)))
        return CudaModule(self, h)

    def alloc(self, nbytes: int) -> "DeviceBuffer":
        h = C.c_void_p()
        _check(lib.basalt_rt_alloc(self._h, nbytes, C.byref(h)))
        return DeviceBuffer(self, h)

    def upload(self, array: np.ndarray) -> "DeviceBuffer":
        buf = self.alloc(array.nbytes)
        buf.copy_from_host(array)
        return buf

    def synchronize(self):
        _check(lib.basalt_rt_ctx_sync(self._h))

    def host_alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        _check(lib.basalt_rt_host_alloc(self._h, nbytes, C.byref(p)))
        return p.value

    def host_free(self, p: int):
        lib.basalt_rt_host_free(self._h, C.c_void_p(p))

    def pinned_array(self, shape, dtype) -> np.ndarray:
        """A numpy array over page-locked memory (freed when the context closes, never before)."""
        dtype = np.dtype(dtype)
        n = int(np.prod(shape)) * dtype.itemsize
        p = self.host_alloc(max(n, 1))
        buf = (C.c_char * max(n, 1)).from_address(p)
        return np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)

    def create_stream(self) -> int:
        s = C.c_void_p()
        _check(lib.basalt_rt_stream_create(self._h, C.byref(s)))
        return s.value

    def destroy_stream(self, s: int):
        _check(lib.basalt_rt_stream_destroy(self._h, C.c_void_p(s)))

    def stream_sync(self, s):
        _check(lib.basalt_rt_stream_sync(self._h, C.c_void_p(s)))

    def create_event(self) -> int:
        e = C.c_void_p()
        _check(lib.basalt_rt_event_create(self._h, C.byref(e)))
        return e.value

    def destroy_event(self, e: int):
        _check(lib.basalt_rt_event_destroy(self._h, C.c_void_p(e)))

    def record(self, event: int, stream=None):
        _check(lib.basalt_rt_event_record(self._h, C.c_void_p(event), C.c_void_p(stream)))

    def event_sync(self, event: int):
        _check(lib.basalt_rt_event_sync(self._h, C.c_void_p(event)))

    def stream_wait_event(self, stream, event: int):
        """Work issued to `stream` after this call starts only when `event` (recorded on another stream) has happened."""
        _check(lib.basalt_rt_stream_wait_event(self._h, C.c_void_p(stream), C.c_void_p(event)))

    def copy_device_async(self, dst_ptr: int, src_ptr: int, nbytes: int, stream=None):
        """Device-to-device copy by the copy engines; either address may be a peer mapping (ipc_open)."""
        _check(lib.basalt_rt_copy_device_async(self._h, dst_ptr, src_ptr, nbytes, C.c_void_p(stream)))

    def ipc_open(self, handle: bytes) -> int:
        """Maps another process's exported buffer (DeviceBuffer.ipc_handle); returns its address on this device."""
        if len(handle) != 64:
            raise ValueError("a CUDA IPC handle is 64 bytes")
        out = C.c_uint64(0)
        _check(lib.basalt_rt_ipc_open(self._h, handle, C.byref(out)))
        return int(out.value)

    def ipc_close(self, ptr: int):
        _check(lib.basalt_rt_ipc_close(self._h, ptr))

    def elapsed_ms(self, start: int, end: int) -> float:
        ms = C.c_float()
        _check(lib.basalt_rt_event_elapsed_ms(self._h, C.c_void_p(start), C.c_void_p(end), C.byref(ms)))
        return ms.value

    def cpu_launch(self, fn: "CudaFunction", args: list, nthreads: int, block: int = 256):
        """Runs a kernel through the reference's CPU launch ABI (kernel parameters then nthreads,
        crates/basalt-x86/src/oracle.rs:75-83) on the device: numpy arrays are copied in, the kernel
        runs ceil(nthreads/block) blocks, and writable arrays are copied back in place.
        args: numpy arrays (all treated as read-write) or i32()/i64()/f32()/f64() scalars."""
        arr = (RtArg * len(args))()
        keep = []
        for k, a in enumerate(args):
            if isinstance(a, np.ndarray):
                if not a.flags["C_CONTIGUOUS"]:
                    raise ValueError("array arguments must be contiguous")
                arr[k].kind = 6 if a.flags["WRITEABLE"] else 4
                arr[k].host = a.ctypes.data
                arr[k].bytes = a.nbytes
                keep.append(a)
            elif isinstance(a, C.c_int32):
                arr[k].kind = 0; arr[k].value.i32 = a.value
            elif isinstance(a, C.c_int64):
                arr[k].kind = 1; arr[k].value.i64 = a.value
            elif isinstance(a, C.c_float):
                arr[k].kind = 2; arr[k].value.f32 = a.value
            elif isinstance(a, C.c_double):
                arr[k].kind = 3; arr[k].value.f64 = a.value
            else:
                raise TypeError(f"argument {k}: pass a numpy array or i32()/i64()/f32()/f64()")
        _check(lib.basalt_rt_cpu_launch(self._h, fn._h, arr, len(args), nthreads, block))


class DeviceBuffer:
    """DeviceBuffer (context.rs:95-168): bounds-checked copies, freed explicitly or on collection."""

    def __init__(self, ctx: CudaContext, handle):
        self.ctx, self._h = ctx, handle

    def device_ptr(self) -> int:
        return lib.basalt_rt_buffer_ptr(self._h)

    def __len__(self) -> int:
        return lib.basalt_rt_buffer_size(self._h)

    def copy_from_host(self, array: np.ndarray, stream=None):
        a = np.ascontiguousarray(array)
        _check(lib.basalt_rt_copy_from_host(self._h, a.ctypes.data, a.nbytes, C.c_void_p(stream)))

    def copy_to_host(self, array: np.ndarray, stream=None):
        if not array.flags["C_CONTIGUOUS"] or not array.flags["WRITEABLE"]:
            raise ValueError("destination must be a writable contiguous array")
        _check(lib.basalt_rt_copy_to_host(self._h, array.ctypes.data, array.nbytes, C.c_void_p(stream)))

    def to_numpy(self, dtype, count: int | None = None) -> np.ndarray:
        dtype = np.dtype(dtype)
        out = np.empty(len(self) // dtype.itemsize if count is None else count, dtype=dtype)
        self.copy_to_host(out)
        return out

    def ipc_handle(self) -> bytes:
        """The 64-byte CUDA IPC handle of this allocation, for CudaContext.ipc_open in another process."""
        buf = (C.c_char * 64)()
        _check(lib.basalt_rt_ipc_export(self._h, buf))
        return bytes(buf.raw)

    def free(self):
        if self._h:
            lib.basalt_rt_buffer_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class CudaModule:
    """CudaModule (module.rs:11-60)."""

    def __init__(self, ctx: CudaContext, handle):
        self.ctx, self._h = ctx, handle

    def get_function(self, name: str) -> "CudaFunction":
        h = C.c_void_p()
        _check(lib.basalt_rt_get_function(self._h, name.encode(), C.byref(h)))
        return CudaFunction(self, h)

    def unload(self):
        if self._h:
            lib.basalt_rt_module_unload(self._h)
            self._h = None


class CudaFunction:
    """CudaFunction (module.rs:62-123)."""

    def __init__(self, module: CudaModule, handle):
        self.module, self._h = module, handle

    def planned_geometry(self):
        """(grid, block, shared bytes) the emitter fixed for this kernel, zeros when it left the
        choice to the caller."""
        g, b, s = (C.c_uint32 * 3)(), (C.c_uint32 * 3)(), C.c_uint32()
        _check(lib.basalt_rt_planned_geometry(self._h, None, g, b, C.byref(s)))
        return tuple(g), tuple(b), s.value

    def one_wave(self, block_threads: int, shared_mem_bytes: int = 0) -> int:
        """Number of CTAs that are resident at once on the whole device for this kernel: the grid
        for a grid-stride (persistent) launch."""
        per_sm, sms = C.c_int(), C.c_int()
        _check(lib.basalt_rt_occupancy(self._h, block_threads, shared_mem_bytes, C.byref(per_sm), C.byref(sms)))
        return max(1, per_sm.value) * sms.value

    def streaming_grid(self, block_threads: int, elements: int, per_thread: int = 64, max_waves: int = 16) -> int:
        """Grid for a grid-stride kernel that streams `elements` items: enough CTAs that a thread handles about
        `per_thread` of them, at most `max_waves` resident waves (each CTA of a reduction ends with an atomic), at
        least one CTA.  Several waves of short CTAs stream faster than one wave of long ones (max_i32 at 2^28:
        7.27 against 6.98 TB/s)."""
        want = (elements + block_threads * per_thread - 1) // (block_threads * per_thread)
        return max(1, min(want, max_waves * self.one_wave(block_threads)))

    def bind(self, grid, block, shared_mem_bytes: int, params: list, stream=None):
        """Pre-marshals a launch; the returned callable issues it with a single foreign call
        (asynchronous; `go(stream=...)` overrides the stream given here). Use for launch-latency-sensitive loops."""
        vals = [C.c_uint64(p.device_ptr()) if isinstance(p, DeviceBuffer) else p for p in params]
        arr = (C.c_void_p * max(len(vals), 1))(*[C.cast(C.pointer(v), C.c_void_p) for v in vals])
        g = (C.c_uint32 * 3)(*_dim3(grid))
        b = (C.c_uint32 * 3)(*_dim3(block))
        s = C.c_void_p(stream)
        h, fn = self._h, lib.basalt_rt_launch

        def go(stream=None, _keep=(vals, arr, g, b)):
            if fn(h, g, b, shared_mem_bytes, s if stream is None else C.c_void_p(stream), arr):
                _check(1)
        return go

    def tune(self, key: str, value: int) -> "CudaFunction":
        """basalt_rt_function_tune: "pair" / "tail_split" (0 switches the policy off), "coarse_waves" (w > 0)."""
        _check(lib.basalt_rt_function_tune(self._h, key.encode(), int(value)))
        return self

    def bind_gather(self, grid, block, shared_mem_bytes: int, params: list, peer_out: list[int], stream=None):
        """`bind` for basalt_rt_launch_gather: the kernel's epilogue also stores every tile of its result,
        at the same offset, behind each address of `peer_out` (the output parameter's value on the other
        ranks, mapped into this device's address space)."""
        vals = [C.c_uint64(p.device_ptr()) if isinstance(p, DeviceBuffer) else p for p in params]
        arr = (C.c_void_p * max(len(vals), 1))(*[C.cast(C.pointer(v), C.c_void_p) for v in vals])
        g = (C.c_uint32 * 3)(*_dim3(grid))
        b = (C.c_uint32 * 3)(*_dim3(block))
        peers = (C.c_uint64 * max(len(peer_out), 1))(*[int(p) for p in peer_out])
        s = C.c_void_p(stream)
        h, fn, n = self._h, lib.basalt_rt_launch_gather, len(peer_out)

        def go(stream=None, _keep=(vals, arr, g, b, peers)):
            if fn(h, g, b, shared_mem_bytes, s if stream is None else C.c_void_p(stream), arr, peers, n):
                _check(1)
        return go

    def bind_gather_multicast(self, grid, block, shared_mem_bytes: int, params: list, multicast_out: int, stream=None):
        """`bind` for basalt_rt_launch_gather_multicast: every finished tile also leaves once, with multimem.st,
        for `multicast_out` (the output parameter's value inside an NVLink multicast mapping of the same result
        buffer on every rank), and the switch replicates it."""
        vals = [C.c_uint64(p.device_ptr()) if isinstance(p, DeviceBuffer) else p for p in params]
        arr = (C.c_void_p * max(len(vals), 1))(*[C.cast(C.pointer(v), C.c_void_p) for v in vals])
        g = (C.c_uint32 * 3)(*_dim3(grid))
        b = (C.c_uint32 * 3)(*_dim3(block))
        s = C.c_void_p(stream)
        h, fn, mc = self._h, lib.basalt_rt_launch_gather_multicast, C.c_uint64(int(multicast_out))

        def go(stream=None, _keep=(vals, arr, g, b)):
            if fn(h, g, b, shared_mem_bytes, s if stream is None else C.c_void_p(stream), arr, mc):
                _check(1)
        return go

    def status(self) -> int:
        """The kernel's device status word (synchronous read): non-zero when a bounded wait inside
        the kernel gave up and the last output is not valid. Always 0 for kernels without waits."""
        v = C.c_int32()
        _check(lib.basalt_rt_kernel_status(self._h, C.byref(v)))
        return v.value

    def launch(self, grid, block, shared_mem_bytes: int, params: list, stream=None, sync: bool | None = None):
        """cuLaunchKernel. With stream=None and sync unset this behaves like the reference: launch
        on the NULL stream, then cuCtxSynchronize (module.rs:101-122). Pass a stream, or sync=False,
        for an asynchronous launch. params: DeviceBuffer, ptr()/i32()/i64()/f32()/f64() values."""
        vals = []
        for p in params:
            if isinstance(p, DeviceBuffer):
                vals.append(C.c_uint64(p.device_ptr()))
            elif isinstance(p, (C.c_int32, C.c_int64, C.c_uint64, C.c_float, C.c_double, C.c_uint32)):
                vals.append(p)
            else:
                raise TypeError("kernel parameters must be DeviceBuffer or ptr()/i32()/i64()/f32()/f64() values")
        arr = (C.c_void_p * max(len(vals), 1))(*[C.cast(C.pointer(v), C.c_void_p) for v in vals])
        g = (C.c_uint32 * 3)(*_dim3(grid))
        b = (C.c_uint32 * 3)(*_dim3(block))
        _check(lib.basalt_rt_launch(self._h, g, b, shared_mem_bytes, C.c_void_p(stream), arr if vals else None))
        if sync if sync is not None else stream is None:
            self.module.ctx.synchronize()


def _dim3(d):
    if isinstance(d, int):
        return (d, 1, 1)
    d = tuple(d)
    return d + (1,) * (3 - len(d))


def shard_range(total: int, nranks: int, rank: int, align: int = 1) -> tuple[int, int]:
    """Contiguous range of `total` units owned by `rank`, boundaries on multiples of `align`."""
    b, e = C.c_uint64(), C.c_uint64()
    lib.basalt_rt_shard_range(total, nranks, rank, align, C.byref(b), C.byref(e))
    return b.value, e.value


class Communicator:
    """One NCCL rank per process over NVLink; the reference has no multi-GPU path at all."""

    def __init__(self, ctx: CudaContext, handle, nranks: int, rank: int):
        self.ctx, self._h, self.nranks, self.rank = ctx, handle, nranks, rank

    @staticmethod
    def unique_id() -> bytes:
        buf = (C.c_char * 128)()
        _check(lib.basalt_rt_comm_unique_id(buf))
        return bytes(buf.raw)

    @staticmethod
    def create(ctx: CudaContext, uid: bytes, nranks: int, rank: int) -> "Communicator":
        h = C.c_void_p()
        buf = (C.c_char * 128)(*uid)
        _check(lib.basalt_rt_comm_init(ctx._h, buf, nranks, rank, C.byref(h)))
        return Communicator(ctx, h, nranks, rank)

    def allreduce_max_i32(self, send_ptr: int, recv_ptr: int, count: int, stream=None):
        _check(lib.basalt_rt_allreduce_max_i32(self._h, send_ptr, recv_ptr, count, C.c_void_p(stream)))

    def allgather(self, send_ptr: int, recv_ptr: int, bytes_per_rank: int, stream=None):
        _check(lib.basalt_rt_allgather(self._h, send_ptr, recv_ptr, bytes_per_rank, C.c_void_p(stream)))

    def destroy(self):
        if self._h:
            lib.basalt_rt_comm_destroy(self._h)
            self._h = None


class PeerGroup:
    """The sharded max_i32's exchange step over peer-mapped memory instead of a library collective
    (basalt_rt_peer_group_*): each rank's inbox is exported as a CUDA IPC handle, every rank maps
    every other rank's inbox, and `allreduce_max_i32` is one small kernel of release stores to the
    peers and acquire loads of its own inbox."""

    def __init__(self, ctx: CudaContext, handle, nranks: int, rank: int):
        self.ctx, self._h, self.nranks, self.rank = ctx, handle, nranks, rank

    @staticmethod
    def create(ctx: CudaContext, nranks: int, rank: int) -> "PeerGroup":
        h = C.c_void_p()
        _check(lib.basalt_rt_peer_group_create(ctx._h, nranks, rank, C.byref(h)))
        return PeerGroup(ctx, h, nranks, rank)

    def handle(self) -> bytes:
        buf = (C.c_char * 64)()
        _check(lib.basalt_rt_peer_group_handle(self._h, buf))
        return bytes(buf.raw)

    def connect(self, handles: list[bytes]):
        """`handles[r]` is rank r's `handle()`; the entry of this rank is ignored."""
        if len(handles) != self.nranks or any(len(x) != 64 for x in handles):
            raise ValueError("expected one 64-byte handle per rank")
        blob = b"".join(handles)
        _check(lib.basalt_rt_peer_group_connect(self._h, blob, len(blob)))

    def allreduce_max_i32(self, partial_ptr: int, result_ptr: int, stream=None, reset_to: int | None = None):
        """`reset_to`: value stored into the partial word once it has been read (None leaves it)."""
        _check(lib.basalt_rt_peer_allreduce_max_i32(self._h, partial_ptr, result_ptr, 0 if reset_to is None else 1,
                                                    0 if reset_to is None else reset_to, C.c_void_p(stream)))

    def max_i32(self, shard_ptr: int, n: int, result_ptr: int, stream=None):
        """The whole sharded step in one launch: the reduction of this rank's shard and the exchange
        (basalt_rt_peer_max_i32); the running maximum and the ticket live in the group."""
        _check(lib.basalt_rt_peer_max_i32(self._h, shard_ptr, n, result_ptr, C.c_void_p(stream)))

    def status(self) -> int:
        """Synchronises the context; non-zero bits name ranks that did not answer within the bound."""
        out = C.c_uint32(0)
        _check(lib.basalt_rt_peer_group_status(self._h, C.byref(out)))
        return int(out.value)

    def destroy(self):
        if self._h:
            lib.basalt_rt_peer_group_destroy(self._h)
            self._h = None
