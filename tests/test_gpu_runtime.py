"""The launch runtime on a real device: the behaviours the reference's own runtime tests pin
(crates/basalt-runtime/tests/cuda_driver.rs) plus streams, events and error reporting. Failures
are provoked on the host only (bad PTX text, a missing symbol, an oversized copy)."""
import numpy as np
import pytest

import basalt_b200 as b
from basalt_b200 import kernels_bir as kb
from _gpu import emitted

pytestmark = pytest.mark.gpu


def test_device_and_round_trip(gpu):
    assert gpu.driver.device_count() >= 1
    assert gpu.sm_count() > 0
    x = np.arange(100003, dtype=np.int32)
    buf = gpu.upload(x)
    assert len(buf) == x.nbytes and buf.device_ptr() % 256 == 0
    assert np.array_equal(buf.to_numpy(np.int32), x)


def test_copies_are_bounds_checked(gpu):
    buf = gpu.alloc(64)
    with pytest.raises(b.CudaError) as e:
        buf.copy_from_host(np.zeros(17, np.int32))
    assert e.value.kind == 4 and "exceeds the device buffer" in e.value.message
    with pytest.raises(b.CudaError) as e:
        buf.copy_to_host(np.zeros(17, np.int32))
    assert e.value.kind == 4


@pytest.mark.parametrize("nbytes", [(3 << 20) + 76, 8 << 20, (37 << 20) + 12344, (64 << 20) + 4])
def test_large_pageable_buffers_take_the_staged_copy_path(gpu, nbytes):
    # Pageable host memory of 2 MiB or more is moved in 1 or 4 MiB chunks by several host threads through pinned buffers
    # (chunk counts that are and are not multiples of the lane count, a ragged last chunk); the bytes must survive
    # both directions, through the buffer API and through the CPU launch ABI.
    rng = np.random.default_rng(nbytes)
    x = rng.integers(0, 256, nbytes, dtype=np.uint8)
    buf = gpu.alloc(nbytes)
    buf.copy_from_host(x)
    back = np.zeros(nbytes, np.uint8)
    buf.copy_to_host(back)
    assert np.array_equal(back, x)
    n = nbytes // 4
    a = x[:4 * n].view(np.int32) >> 2
    bb = np.roll(a, 7)
    c = np.full(n, -1, np.int32)
    gpu.cpu_launch(gpu.load_module(b.Ptx().emit(kb.load("vadd_i32")).text).get_function("vadd_i32"), [a, bb, c, b.i32(n)], n)
    assert np.array_equal(c, a + bb)


def test_jit_failure_is_reported_not_fatal(gpu):
    with pytest.raises(b.CudaError) as e:
        gpu.load_module(".version 8.7\n.target sm_100a\n.address_size 64\n.visible .entry broken() { this is not ptx; }\n")
    assert e.value.kind == 3 and e.value.call == "cuModuleLoadData" and e.value.code != 0
    # the context is still usable
    assert np.array_equal(gpu.upload(np.arange(8, dtype=np.int32)).to_numpy(np.int32), np.arange(8))


def test_missing_function_is_reported(gpu):
    mod = gpu.load_module(b.Ptx().emit(kb.load("vadd_i32")).text)
    with pytest.raises(b.CudaError) as e:
        mod.get_function("no_such_kernel")
    assert e.value.kind == 3 and e.value.call == "cuModuleGetFunction"


def test_async_launch_streams_events_and_pinned_memory(gpu):
    n = 1 << 20
    fn = emitted(gpu, kb.load("vadd_i32"), "vadd_i32")
    a = gpu.pinned_array((n,), np.int32); bb = gpu.pinned_array((n,), np.int32); c = gpu.pinned_array((n,), np.int32)
    a[:] = np.arange(n); bb[:] = 7; c[:] = 0
    da, db, dc = gpu.alloc(a.nbytes), gpu.alloc(a.nbytes), gpu.alloc(a.nbytes)
    s = gpu.create_stream(); e0 = gpu.create_event(); e1 = gpu.create_event()
    gpu.record(e0, s)
    da.copy_from_host(a, s); db.copy_from_host(bb, s)
    fn.launch(n // 256, 256, 0, [da, db, dc, b.i32(n)], stream=s)
    dc.copy_to_host(c, s)
    gpu.record(e1, s)
    gpu.stream_sync(s)
    assert gpu.elapsed_ms(e0, e1) > 0
    assert np.array_equal(c, a + 7)
    gpu.destroy_event(e0); gpu.destroy_event(e1); gpu.destroy_stream(s)


def test_peer_exchange_wait_runs_out_and_reports_it(gpu):
    # The give-up path of the peer exchange, provoked without a second device and without a fault:
    # a group of two whose second inbox is a zeroed buffer of THIS GPU that nothing ever writes.  The
    # kernel stores its word into that inbox, polls its own inbox for rank 1's word for 1 ms, gives up,
    # sets bit 1 of the status word and returns the maximum over the ranks that answered (itself).
    import ctypes as C
    from basalt_b200._lib import lib
    words = 2 * 8
    mine, silent = gpu.upload(np.zeros(words, np.uint64)), gpu.upload(np.zeros(words, np.uint64))
    inboxes = (C.c_uint64 * 2)(mine.device_ptr(), silent.device_ptr())
    partial, result = gpu.upload(np.array([1234567], np.int32)), gpu.upload(np.array([-1], np.int32))
    status = gpu.upload(np.zeros(1, np.uint32))
    for epoch in (1, 2):          # a second call gives up the same way: the context stays usable
        rc = lib.basalt_k_peer_allreduce_max_i32(inboxes, 2, 0, epoch, C.c_void_p(partial.device_ptr()), C.c_void_p(result.device_ptr()),
                                                 C.c_void_p(status.device_ptr()), 1_000_000, 0, 0, None)
        assert rc == 0
        gpu.synchronize()
        assert status.to_numpy(np.uint32)[0] == 0b10
        assert result.to_numpy(np.int32)[0] == 1234567
        # this rank's word did reach the silent inbox (parity row, column = sender's rank)
        assert silent.to_numpy(np.uint64)[(epoch & 1) * 8 + 0] == (epoch << 32 | 1234567)
    assert np.array_equal(gpu.upload(np.arange(8, dtype=np.int32)).to_numpy(np.int32), np.arange(8))


def test_launch_policies_are_switched_per_handle_not_by_environment(gpu, monkeypatch):
    # basalt_rt_function_tune: the A/B switches are arguments; an unknown key is refused, and the
    # environment variables earlier builds read change nothing
    monkeypatch.setenv("BASALT_RT_COARSE_WAVES", "1")
    fn = emitted(gpu, kb.load("vadd_i32"), "vadd_i32")
    n = 100003
    a, c = np.arange(n, dtype=np.int32), gpu.upload(np.zeros(n, np.int32))
    da = gpu.upload(a)
    for waves in (0, 1, 3):
        fn.tune("coarse_waves", waves)
        c.copy_from_host(np.zeros(n, np.int32))
        fn.launch((n + 255) // 256, 256, 0, [da, da, c, b.i32(n)])
        assert np.array_equal(c.to_numpy(np.int32), 2 * a), waves
    with pytest.raises(b.CudaError) as e:
        fn.tune("no_such_policy", 1)
    assert e.value.kind == 4


@pytest.mark.parametrize("pdl", [1, 0])
def test_dependent_coarse_launches_keep_stream_order(gpu, pdl):
    # Coarse launches go out with programmatic stream serialisation: the next launch's CTAs are set up while the one
    # before drains, and griddepcontrol.wait holds them off memory until it has completed.  Twenty launches that each
    # read what the one before wrote (x + x -> y, y + y -> x, ...), issued back to back on one stream: 2^20 everywhere.
    fn = gpu.load_module(b.Ptx().emit(kb.load("vadd_i32")).text).get_function("vadd_i32")
    fn.tune("pdl", pdl)
    n = (1 << 20) + 13
    x, y = gpu.upload(np.ones(n, np.int32)), gpu.upload(np.zeros(n, np.int32))
    s = gpu.create_stream()
    for i in range(20):
        src, dst = (x, y) if i % 2 == 0 else (y, x)
        fn.launch((n + 255) // 256, 256, 0, [src, src, dst, b.i32(n)], stream=s)
    gpu.stream_sync(s)
    gpu.destroy_stream(s)
    assert np.array_equal(x.to_numpy(np.int32), np.full(n, 1 << 20, np.int32))
    assert np.array_equal(y.to_numpy(np.int32), np.full(n, 1 << 19, np.int32))
