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

    def shard(self, total: int, align: int = 1) -> tuple[int, int]:
        return shard_range(total, self.world, self.rank, align)


def reduce_max_sharded(group: RankGroup, local_slice: np.ndarray, reduce_local) -> int:
    """Sharded max: `reduce_local(slice) -> int` is the per-rank reduction (the GPU kernel on the
    device path; any callable in tests); the partial maxima are then combined with allreduce(max).
    An empty shard contributes INT32_MIN, the identity."""
    partial = int(reduce_local(local_slice)) if len(local_slice) else -2**31
    return group.max_i32_host(partial)
