"""One rank of the multi-GPU parity run (launched by test_gpu_multi.py under torch.distributed.run).

Each rank owns a contiguous shard of the work on its own GPU and runs the emitted kernels through
the C-ABI runtime; the only exchanges are the ones the workloads need: allreduce(max) of one int32
for the reduction (over this library's NCCL communicator and, beside it, over peer-mapped memory),
allgather of the row-sharded C for the two matmuls.  Results are compared with the CPU oracle on every rank."""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import basalt_b200 as b  # noqa: E402
from basalt_b200 import kernels, kernels_bir as kb, sharding, workloads as w  # noqa: E402
from _util import orc_matmul_f16_rows, orc_sgemm_rows, rel_fro, vp  # noqa: E402


def main():
    import torch
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    group = sharding.RankGroup.from_env("gloo")     # host rendezvous only; data moves over our NCCL communicator
    ctx = b.CudaDriver.load().create_context(local)
    comm = group.nccl(ctx)
    peers = group.peers(ctx)
    orc = ctypes.CDLL(os.path.join(ROOT, "oracle", "liborc.so"))
    ptx = b.Ptx()

    # ---- max_i32: contiguous shards, planted maxima on both sides of every shard boundary ----
    n = (1 << 22) + 37
    x = w.u32(w.SEEDS["max_i32"], n).view(np.int32).copy()
    np.minimum(x, 2**31 - 2, out=x)
    fn = ctx.load_module(ptx.emit(kb.load("max_i32")).text).get_function("max_i32")
    lo, hi = group.shard(n, 4)
    plants = [None, 0, n - 1] + [p for r in range(1, group.world) for p in (group_bound(n, group.world, r) - 1, group_bound(n, group.world, r))]
    for plant in plants:
        y = x.copy()
        if plant is not None:
            y[plant] = 2**31 - 1
        want = np.array([-2**31], np.int32)
        orc.orc_max_i32(vp(y), vp(want), ctypes.c_int32(n), ctypes.c_int64(n))
        dshard = ctx.upload(y[lo:hi])
        partial = ctx.upload(np.array([-2**31], np.int32)); result = ctx.alloc(4)
        if hi > lo:
            fn.launch(fn.streaming_grid(256, hi - lo), 256, 0, [dshard, partial, b.i32(hi - lo)])
        comm.allreduce_max_i32(partial.device_ptr(), result.device_ptr(), 1)
        ctx.synchronize()
        got = int(result.to_numpy(np.int32)[0])
        assert got == int(want[0]), (plant, got, int(want[0]))
        # the same exchange over peer-mapped memory instead of NCCL
        result2 = ctx.upload(np.array([12345], np.int32))
        peers.allreduce_max_i32(partial.device_ptr(), result2.device_ptr())
        assert peers.status() == 0
        assert int(result2.to_numpy(np.int32)[0]) == int(want[0]), (plant, "peer exchange")
        # reduction and exchange in one kernel (hand-written), twice in a row: it must leave its own state ready
        for again in range(2):
            result3 = ctx.upload(np.array([54321], np.int32))
            peers.max_i32(dshard.device_ptr(), hi - lo, result3.device_ptr())
            assert peers.status() == 0
            assert int(result3.to_numpy(np.int32)[0]) == int(want[0]), (plant, "fused", again)

    # ---- peer exchange: many back-to-back epochs with values that change every call ----
    calls = 300
    table = lambda r: (np.arange(calls, dtype=np.int64) * 2654435761 * (r + 1) % (1 << 32)).astype(np.uint32).view(np.int32)
    mine = ctx.upload(table(group.rank))
    outs = ctx.upload(np.zeros(calls, np.int32))
    for i in range(calls):
        peers.allreduce_max_i32(mine.device_ptr() + 4 * i, outs.device_ptr() + 4 * i)
    assert peers.status() == 0
    want_all = np.max(np.stack([table(r) for r in range(group.world)]), axis=0)
    assert np.array_equal(outs.to_numpy(np.int32), want_all)

    # ---- SGEMM: rows of A and C sharded, B replicated, allgather of C ----
    M, N, K = 128 * 2 * group.world, 256, 128
    A = w.f32_pm1(w.SEEDS["sgemm_f32"], M * K).reshape(M, K); B = w.f32_pm1(w.SEEDS["sgemm_f32"] + 1, K * N).reshape(K, N)
    r0, r1 = group.shard(M, 128)
    Ml = r1 - r0
    dA, dB, dCl, dC = ctx.upload(A[r0:r1]), ctx.upload(B), ctx.alloc(Ml * N * 4), ctx.alloc(M * N * 4)
    fn = ctx.load_module(ptx.emit(kb.sgemm_cta128(Ml, N, K)).text).get_function("sgemm_f32")
    fn.launch((N // 128, Ml // 128), 256, 0, [dA, dB, dCl])
    comm.allgather(dCl.device_ptr(), dC.device_ptr(), Ml * N * 4)
    ctx.synchronize()
    got = dC.to_numpy(np.float32).reshape(M, N)
    assert rel_fro(got, orc_sgemm_rows(orc, A, B, 0, M)) <= 1e-4

    # ---- fp16 matmul: the same sharding, tensor-core kernel ----
    M, N, K = 128 * group.world, 256, 256
    A = w.f16_normal01(w.SEEDS["matmul_f16"], M * K).reshape(M, K); B = w.f16_normal01(w.SEEDS["matmul_f16"] + 1, K * N).reshape(K, N)
    r0, r1 = group.shard(M, 128)
    Ml = r1 - r0
    dA, dB, dCl, dC = ctx.upload(A[r0:r1]), ctx.upload(B), ctx.alloc(Ml * N * 2), ctx.alloc(M * N * 2)
    fn = ctx.load_module(ptx.emit(kb.matmul_f16(Ml, N, K)).text).get_function("matmul_kernel")
    fn.launch((N // 128, Ml // 128), 128, 0, [dA, dB, dCl])
    assert fn.status() == 0
    comm.allgather(dCl.device_ptr(), dC.device_ptr(), Ml * N * 2)
    ctx.synchronize()
    got = dC.to_numpy(np.float16).reshape(M, N)
    assert rel_fro(got, orc_matmul_f16_rows(orc, A, B, N, False, 0, M)) <= 2e-3

    # ---- the same fp16 matmul with the gather pushed by the copy engines, band by band ----
    M, N, K = 256 * group.world, 256, 256
    A = w.f16_normal01(w.SEEDS["matmul_f16"] + 7, M * K).reshape(M, K); B = w.f16_normal01(w.SEEDS["matmul_f16"] + 8, K * N).reshape(K, N)
    want = orc_matmul_f16_rows(orc, A, B, N, False, 0, M)
    r0, r1 = group.shard(M, 128)
    Ml = r1 - r0
    dA, dB, dC = ctx.upload(A[r0:r1]), ctx.upload(B), ctx.upload(np.zeros((M, N), np.float16))
    ptrs = group.map_peers(ctx, dC)
    for bands in (1, 2):
        rows_b = Ml // bands
        fb = ctx.load_module(ptx.emit(kb.matmul_f16(rows_b, N, K)).text).get_function("matmul_kernel")
        pg = sharding.PushGather(ctx, group, peers, ptrs, N * 2, r0, Ml, bands)
        for _ in range(3):      # back-to-back runs reuse the streams and events
            pg.run(lambda k, s: fb.launch((N // 128, rows_b // 128), 128, 0,
                                          [b.ptr(dA.device_ptr() + k * rows_b * K * 2), dB, b.ptr(dC.device_ptr() + (r0 + k * rows_b) * N * 2)], stream=s), None)
        ctx.synchronize()
        assert fb.status() == 0 and peers.status() == 0
        got = dC.to_numpy(np.float16).reshape(M, N)
        assert rel_fro(got, want) <= 2e-3, ("pushed gather", bands)
        group.barrier()
        dC.copy_from_host(np.zeros((M, N), np.float16))
        ctx.synchronize()
        group.barrier()
        pg.close()
    for r, p in enumerate(ptrs):
        if r != group.rank:
            ctx.ipc_close(p)

    # ---- the same, gather fused into the tensor-core kernel: its epilogue stores every tile to every rank ----
    M, N, K = 512 * group.world, 512, 192
    A = w.f16_normal01(w.SEEDS["matmul_f16"] + 11, M * K).reshape(M, K); B = w.f16_normal01(w.SEEDS["matmul_f16"] + 12, K * N).reshape(K, N)
    want = orc_matmul_f16_rows(orc, A, B, N, False, 0, M)
    r0, r1 = group.shard(M, 256)
    Ml = r1 - r0
    dA, dB, dC = ctx.upload(A[r0:r1]), ctx.upload(B), ctx.upload(np.full((M, N), np.nan, np.float16))
    st, flag = ctx.upload(np.zeros(1, np.int32)), ctx.upload(np.zeros(2, np.int32))
    ptrs = group.map_peers(ctx, dC)
    group.barrier()      # every rank's buffer holds its NaN fill before anyone stores into it
    others = [ptrs[r] + r0 * N * 2 for r in group.peer_order()]
    for _ in range(3):
        kernels.matmul_f16_allgather(dA, dB, dC.device_ptr() + r0 * N * 2, Ml, N, K, others, status=st)
        peers.allreduce_max_i32(flag.device_ptr(), flag.device_ptr() + 4, None)      # the barrier: all ranks' stores have landed
        ctx.synchronize()
        assert st.to_numpy(np.int32)[0] == 0 and peers.status() == 0
        got = dC.to_numpy(np.float16).reshape(M, N)
        assert np.isfinite(got).all(), "rows of some rank never arrived"
        assert rel_fro(got, want) <= 2e-3, "fused gather"
        group.barrier()
    for r, p in enumerate(ptrs):
        if r != group.rank:
            ctx.ipc_close(p)

    # ---- the emitted kernels with their gathering epilogue (basalt_rt_launch_gather): fp16 on tcgen05, then fp32 FFMA ----
    for what in ("f16", "f32"):
        if what == "f16":
            M, N, K, esz = 512 * group.world, 512, 192, 2
            A = w.f16_normal01(w.SEEDS["matmul_f16"] + 31, M * K).reshape(M, K); B = w.f16_normal01(w.SEEDS["matmul_f16"] + 32, K * N).reshape(K, N)
            want, tol, dt = orc_matmul_f16_rows(orc, A, B, N, False, 0, M), 2e-3, np.float16
        else:
            M, N, K, esz = 256 * group.world, 384, 96, 4
            A = w.f32_pm1(w.SEEDS["sgemm_f32"] + 31, M * K).reshape(M, K); B = w.f32_pm1(w.SEEDS["sgemm_f32"] + 32, K * N).reshape(K, N)
            want, tol, dt = orc_sgemm_rows(orc, A, B, 0, M), 1e-4, np.float32
        r0, r1 = group.shard(M, 256)
        Ml = r1 - r0
        dA, dB, dC = ctx.upload(A[r0:r1]), ctx.upload(B), ctx.upload(np.full((M, N), np.nan, dt))
        flag = ctx.upload(np.zeros(2, np.int32))
        ptrs = group.map_peers(ctx, dC)
        group.barrier()
        if what == "f16":
            fn = ctx.load_module(ptx.emit(kb.matmul_f16(Ml, N, K)).text).get_function("matmul_kernel")
            block = 128
        else:
            fn = ctx.load_module(ptx.emit(kb.sgemm_cta128(Ml, N, K)).text).get_function("sgemm_f32")
            block = 256
        go = fn.bind_gather((N // 128, Ml // 128), block, 0, [dA, dB, b.ptr(dC.device_ptr() + r0 * N * esz)],
                            [ptrs[r] + r0 * N * esz for r in group.peer_order()])
        for _ in range(3):
            go()
            peers.allreduce_max_i32(flag.device_ptr(), flag.device_ptr() + 4, None)      # the barrier: all ranks' stores have landed
            ctx.synchronize()
            assert fn.status() == 0 and peers.status() == 0
            got = dC.to_numpy(dt).reshape(M, N)
            assert np.isfinite(got).all(), ("rows of some rank never arrived", what)
            assert rel_fro(got, want) <= tol, ("emitted fused gather", what)
            group.barrier()
        for r, p in enumerate(ptrs):
            if r != group.rank:
                ctx.ipc_close(p)

    # ---- the same epilogues through an NVLink multicast mapping (basalt_rt_launch_gather_multicast): one multimem.st
    # per 16 bytes, replicated by the switch.  Nothing is asserted while the result is bound to the multicast object:
    # outcomes are collected, the mapping is closed by all ranks together, then checked. ----
    import torch
    outcomes = []
    for what in ("f16", "f32"):
        if what == "f16":
            M, N, K, esz = 512 * group.world, 512, 192, 2
            A = w.f16_normal01(w.SEEDS["matmul_f16"] + 41, M * K).reshape(M, K); B = w.f16_normal01(w.SEEDS["matmul_f16"] + 42, K * N).reshape(K, N)
            want, tol, dt = orc_matmul_f16_rows(orc, A, B, N, False, 0, M), 2e-3, np.float16
        else:
            M, N, K, esz = 256 * group.world, 384, 96, 4
            A = w.f32_pm1(w.SEEDS["sgemm_f32"] + 41, M * K).reshape(M, K); B = w.f32_pm1(w.SEEDS["sgemm_f32"] + 42, K * N).reshape(K, N)
            want, tol, dt = orc_sgemm_rows(orc, A, B, 0, M), 1e-4, np.float32
        r0, r1 = group.shard(M, 256)
        Ml = r1 - r0
        mcr = sharding.MulticastResult.open(group, M * N * esz, torch.cuda.current_device())
        if mcr is None:
            print(f"rank {group.rank}: no multicast mapping ({sharding.MulticastResult.why_not}); multimem gather not run", flush=True)
            break
        try:
            mcr.tensor.view(torch.float16 if what == "f16" else torch.float32).fill_(float("nan"))
            torch.cuda.synchronize()
            group.barrier()
            dA, dB = ctx.upload(A[r0:r1]), ctx.upload(B)
            flag = ctx.upload(np.zeros(2, np.int32))
            if what == "f16":
                fn = ctx.load_module(ptx.emit(kb.matmul_f16(Ml, N, K)).text).get_function("matmul_kernel"); block = 128
            else:
                fn = ctx.load_module(ptx.emit(kb.sgemm_cta128(Ml, N, K)).text).get_function("sgemm_f32"); block = 256
            go = fn.bind_gather_multicast((N // 128, Ml // 128), block, 0, [dA, dB, b.ptr(mcr.local_ptr + r0 * N * esz)], mcr.multicast_ptr + r0 * N * esz)
            for _ in range(2):
                go()
                peers.allreduce_max_i32(flag.device_ptr(), flag.device_ptr() + 4, None)      # the barrier: all ranks' tiles have landed
                ctx.synchronize()
                got = mcr.tensor.view(torch.float16 if what == "f16" else torch.float32).reshape(M, N).cpu().numpy()
                outcomes.append((what, fn.status() == 0 and peers.status() == 0, bool(np.isfinite(got).all()), float(rel_fro(got, want)) if np.isfinite(got).all() else float("inf"), tol))
                group.barrier()
        except Exception as e:      # reported after the mapping is closed
            outcomes.append((what, False, False, float("inf"), repr(e)))
        finally:
            mcr.close()
    for what, status_ok, finite, err, tol in outcomes:
        assert status_ok and finite and err <= tol, ("multimem gather", what, status_ok, finite, err, tol)
    if outcomes:
        print(f"rank {group.rank}: multimem gather checked {len(outcomes)} times", flush=True)

    group.barrier()
    peers.destroy()
    comm.destroy()
    group.barrier()
    print(f"rank {group.rank}/{group.world} ok", flush=True)


def group_bound(n, world, r):
    return b.shard_range(n, world, r, 4)[0]


if __name__ == "__main__":
    main()
