"""Host-side logic of the 1/2/4/8-GPU configurations: one process per GPU, each owning a
contiguous range of the work (its own slice of every buffer), and a collective only where the
workload has a real exchange step -- the 4-byte allreduce(max) of the reduction's partial maxima
and the allgather of the row-sharded matmul output.  The reference has no multi-GPU path
(crates/basalt-runtime/src/ffi.rs:38-42; every test uses device ordinal 0).

`torch.distributed` is used for the process rendezvous only (rank, world size, broadcasting the
NCCL id, barriers, max-over-ranks of a timing); on GPUs the data-path collectives run through this
library's own NCCL communicator (include/basalt_b200.h, basalt_rt_allreduce_max_i32 /
basalt_rt_allgather).  With the gloo backend on CPUs the same code paths run with host tensors,
which is how the N>1 host logic is tested without GPUs."""
from __future__ import annotations

import os
from dataclasses import dataclass

import numpy as np

from .runtime import Communicator, CudaContext, PeerGroup, shard_range


def bind_to_gpu_cpus(device_index: int) -> list[int]:
    """Restricts this process to the CPUs NVML reports as local to the GPU (its NUMA node), so that
    pinned host buffers allocated afterwards sit on the memory closest to the GPU's PCIe root.  Only
    reads NVML (nvmlDeviceGetCpuAffinity) and changes this process's own CPU affinity mask; returns
    the CPUs chosen, or an empty list when NVML or the affinity call is unavailable."""
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        finally:
            pynvml.nvmlShutdown()
        cpus = [64 * w + bit for w, word in enumerate(words) for bit in range(64) if (int(word) >> bit) & 1]
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if allowed:
            os.sched_setaffinity(0, allowed)
        return allowed
    except Exception:   # noqa: BLE001 - an optimisation only
        return []


@dataclass
class RankGroup:
    rank: int = 0
    world: int = 1
    dist: object = None   # torch.distributed, when world > 1

    @staticmethod
    def from_env(backend: str | None = None) -> "RankGroup":
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world <= 1:
            return RankGroup()
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group(backend=backend or "gloo")
        return RankGroup(dist.get_rank(), dist.get_world_size(), dist)

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()

    def broadcast_bytes(self, payload: bytes | None, src: int = 0) -> bytes:
        if self.dist is None:
            return payload
        box = [payload]
        self.dist.broadcast_object_list(box, src=src)
        return box[0]

    def max_float(self, v: float) -> float:
        """Max over ranks of a host scalar (the timing rule: a step takes as long as its slowest rank)."""
        if self.dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64)
        if self.dist.get_backend() == "nccl":
            t = t.cuda()
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def max_i32_host(self, v: int) -> int:
        """allreduce(max) of a host int32: the CPU stand-in for the device collective."""
        if self.dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.int32)
        if self.dist.get_backend() == "nccl":
            t = t.cuda()
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return int(t.item())

    def nccl(self, ctx: CudaContext) -> Communicator | None:
        """This library's NCCL communicator over the ranks of the group (None for one rank)."""
        if self.world <= 1:
            return None
        uid = Communicator.unique_id() if self.rank == 0 else None
        uid = self.broadcast_bytes(uid, 0)
        return Communicator.create(ctx, uid, self.world, self.rank)

    def all_gather_bytes(self, payload: bytes) -> list[bytes]:
        if self.dist is None:
            return [payload]
        box = [None] * self.world
        self.dist.all_gather_object(box, payload)
        return box

    def peers(self, ctx: CudaContext) -> PeerGroup | None:
        """The peer-memory exchange group over the ranks of the group (None for one rank): every
        rank exports its inbox, the handles travel through torch.distributed, every rank maps the
        others.  Needs one process per GPU on GPUs that can map each other's memory."""
        if self.world <= 1:
            return None
        g = PeerGroup.create(ctx, self.world, self.rank)
        g.connect(self.all_gather_bytes(g.handle()))
        self.barrier()
        return g

    def map_peers(self, ctx: CudaContext, buf) -> list[int]:
        """Device addresses, valid on this rank's GPU, of every rank's copy of `buf` (a DeviceBuffer every
        rank allocated with the same size); entry `rank` is this rank's own.  Close the others with
        ctx.ipc_close before the owners free their buffers."""
        if self.world <= 1:
            return [buf.device_ptr()]
        handles = self.all_gather_bytes(buf.ipc_handle())
        return [buf.device_ptr() if r == self.rank else ctx.ipc_open(handles[r]) for r in range(self.world)]

    def peer_order(self) -> list[int]:
        """The other ranks, starting with the next one: rank + 1, rank + 2, ... (mod world).  A rank that sends
        something to every peer in this order makes every step of the exchange a permutation -- at each moment
        no two ranks send to the same receiver -- instead of all ranks starting on rank 0's ingress ports."""
        return [(self.rank + k) % self.world for k in range(1, self.world)]

    def shard(self, total: int, align: int = 1) -> tuple[int, int]:
        return shard_range(total, self.world, self.rank, align)


def reduce_max_sharded(group: RankGroup, local_slice: np.ndarray, reduce_local) -> int:
    """Sharded max: `reduce_local(slice) -> int` is the per-rank reduction (the GPU kernel on the
    device path; any callable in tests); the partial maxima are then combined with allreduce(max).
    An empty shard contributes INT32_MIN, the identity."""
    partial = int(reduce_local(local_slice)) if len(local_slice) else -2**31
    return group.max_i32_host(partial)


class MulticastResult:
    """One result buffer of `nbytes` per rank behind an NVLink multicast mapping (NVLS), for
    basalt_rt_launch_gather_multicast: `local_ptr` is this rank's buffer, `multicast_ptr` the address through which
    one multimem.st lands at the same offset in every rank's buffer, `peer_ptrs[r]` rank r's buffer mapped here.
    The allocation, the handle exchange between the processes and the multicast object are
    torch.distributed._symmetric_memory's (cuMemCreate / cuMulticastCreate / cuMulticastBindMem): plumbing.

    `open` returns None with the reason in `MulticastResult.why_not` when the box or this torch build has no
    multicast support.  Every rank must call `close` (collectively) before it exits: a rank that leaves while its
    memory is bound to a multicast object other ranks still use faults their NVLink."""
    why_not = ""

    def __init__(self, tensor, handle, group: "RankGroup"):
        self.tensor, self._handle, self._group = tensor, handle, group
        off = int(getattr(handle, "offset", 0) or 0)
        self.local_ptr = int(tensor.data_ptr())
        self.multicast_ptr = int(handle.multicast_ptr) + off
        self.peer_ptrs = [int(p) + off for p in handle.buffer_ptrs]

    @staticmethod
    def open(group: "RankGroup", nbytes: int, device_index: int) -> "MulticastResult | None":
        import torch
        import torch.distributed as dist
        try:
            import torch.distributed._symmetric_memory as symm
            t = symm.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", device_index))
            h = symm.rendezvous(t, dist.group.WORLD)
            ok = int(h.multicast_ptr) != 0
            reason = "" if ok else "the symmetric-memory handle carries no multicast address"
        except Exception as e:   # no multicast support, or a torch build without symmetric memory
            t = h = None
            ok, reason = False, f"{type(e).__name__}: {e}"[:200]
        # every rank takes the same branch: one that failed alone must not leave the others bound
        if group.max_i32_host(0 if ok else 1) != 0:
            MulticastResult.why_not = reason or "another rank has no multicast support"
            del h, t
            return None
        return MulticastResult(t, h, group)

    def close(self):
        import torch
        torch.cuda.synchronize()
        self._group.barrier()
        self._handle = None
        self.tensor = None
        self._group.barrier()


class PushGather:
    """The gather of a row-sharded result, overlapped with the compute that produces it.

    Every rank owns rows [row0, row0 + rows) of a result every rank wants whole.  The shard is
    computed in `bands` row bands, band k by `launch_band(k, stream)` on one of two compute streams;
    as soon as band k is done, the copy engines push its rows into every peer's result buffer (one
    cuMemcpyDtoDAsync per peer; up to four ranks each peer on its own copy stream) while band k + 1 computes.  `finish` orders the
    caller's stream after the last push and runs the peer exchange as a barrier: when it returns in
    stream order, every peer's pushes into this rank's buffer have landed (a peer's exchange word is
    sent in stream order after that peer's copies).  An allgather does compute, then communication;
    this does both at once and needs no SM for the transfer."""

    def __init__(self, ctx: CudaContext, group: RankGroup, peers, result_ptrs: list[int], row_bytes: int, row0: int, rows: int, bands: int):
        if rows % bands:
            raise ValueError("the bands must divide the shard's rows")
        self.ctx, self.group, self.peers, self.ptrs = ctx, group, peers, result_ptrs
        self.row_bytes, self.row0, self.rows, self.bands = row_bytes, row0, rows, bands
        self.compute = [ctx.create_stream(), ctx.create_stream()]
        # One copy stream per peer up to four ranks: the pushes to different peers then run on different copy engines at
        # once (0.37-0.40 ms against 0.38 for NCCL at 4 ranks).  Beyond that a single copy stream: at 8 ranks seven
        # streams per rank measured 0.476 ms against 0.368 for one (56 concurrent copies thrash the engines).
        self.copies = [ctx.create_stream() for _ in range(max(1, group.world - 1) if group.world <= 4 else 1)]
        self.band_done = [ctx.create_event() for _ in range(bands)]
        self.pushed = [ctx.create_event() for _ in self.copies]
        self.start, self.copied = ctx.create_event(), ctx.create_event()
        self.flag = ctx.upload(np.zeros(2, np.int32))

    def run(self, launch_band, stream=None):
        ctx, me, world = self.ctx, self.group.rank, self.group.world
        ctx.record(self.start, stream)                          # the inputs are ready in the caller's stream order
        band_rows = self.rows // self.bands
        for k in range(self.bands):
            cs = self.compute[k & 1]
            if k < 2:
                ctx.stream_wait_event(cs, self.start)
            launch_band(k, cs)
            ctx.record(self.band_done[k], cs)
            off = (self.row0 + k * band_rows) * self.row_bytes
            for step in range(1, world):                         # stream `step - 1` serves the rank `step` places after this one
                r = (me + step) % world
                cs_copy = self.copies[min(step - 1, len(self.copies) - 1)]
                ctx.stream_wait_event(cs_copy, self.band_done[k])
                ctx.copy_device_async(self.ptrs[r] + off, self.ptrs[me] + off, band_rows * self.row_bytes, cs_copy)
        last = self.copies[0]
        if world == 1:
            ctx.stream_wait_event(last, self.band_done[self.bands - 1])
        for i in range(1, len(self.copies)):                     # gather the copy streams on the first one
            ctx.record(self.pushed[i], self.copies[i])
            ctx.stream_wait_event(last, self.pushed[i])
        if self.peers is not None:                               # barrier: every peer's pushes precede its word
            self.peers.allreduce_max_i32(self.flag.device_ptr(), self.flag.device_ptr() + 4, last)
        ctx.record(self.copied, last)
        ctx.stream_wait_event(stream, self.copied)              # the next run's `start` is recorded after this: no band starts early

    def close(self):
        for s in self.compute + self.copies:
            self.ctx.destroy_stream(s)
        for e in self.band_done + self.pushed + [self.start, self.copied]:
            self.ctx.destroy_event(e)
        self.flag.free()
