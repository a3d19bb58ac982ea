"""The emitter's BIR-to-BIR passes preserve results under the CPU oracle's execution model: the
optimised module (inlined calls, 16-byte vector accesses, scalar tails) is run through the oracle
interpreter beside the original on the same inputs, including ragged and under-sized launches."""
import numpy as np
import pytest

import basalt_b200 as b
from basalt_b200 import kernels_bir as kb
from oracle.bir_interp import run_kernel

LAUNCHES = [(1000, 1024), (1003, 1024), (7, 8), (0, 4), (100, 40), (37, 64), (64, 16), (5, 1), (33, 33)]


@pytest.mark.parametrize("name, kernel, nin", [("vadd_i32", "vadd_i32", 2), ("vector_add_f32", "vector_add", 2),
                                               ("chain_vector", "chain_vector", 1), ("square_vector", "square_vector", 1)])
def test_elementwise_vectoriser(ptx, name, kernel, nin):
    src = kb.load(name)
    opt = ptx.optimized_bir(src)
    assert "load v4" in opt and "vec.build" in opt and "call" not in opt
    rng = np.random.default_rng(11)
    for n, threads in LAUNCHES:
        size = max(n, 1) + 8
        if name == "vector_add_f32":
            ins = [rng.uniform(-1e3, 1e3, size).astype(np.float32) for _ in range(nin)]
            poison = np.full(size, -1.0, np.float32)
        else:
            ins = [rng.integers(-2**30, 2**30, size, dtype=np.int64).astype(np.int32) for _ in range(nin)]
            poison = np.full(size, 0x7fffffff, np.int32)
        o0, o1 = poison.copy(), poison.copy()
        run_kernel(src, kernel, ins + [o0, n], threads)
        run_kernel(opt, kernel, ins + [o1, n], threads)
        assert np.array_equal(o0.view(np.uint32), o1.view(np.uint32)), (n, threads)
        assert np.array_equal(o0[min(n, threads):], poison[min(n, threads):])   # nothing past min(n, threads) is touched


def test_helper_chain_inlining_and_vectorising(ptx, orc):
    import ctypes
    from _util import vp
    src = kb.helper_chain()
    opt = ptx.optimized_bir(src)
    assert "call" not in opt and opt.count("func @") == 2 and "@helper_chain__coarse" in opt and "load v4i32" in opt
    x = np.random.default_rng(5).integers(0, 2**32, 300, dtype=np.uint64).astype(np.uint32)
    want = np.zeros(300, np.uint32)
    orc.orc_helper_chain_u32(vp(x), vp(want), ctypes.c_int32(297), ctypes.c_int64(320))
    for text in (src, opt):
        got = np.zeros(300, np.uint32)
        run_kernel(text, "helper_chain", [x, got, 297], 320)
        assert np.array_equal(got, want)


def test_coarse_variant_processes_the_same_elements_with_fewer_threads(ptx):
    # `<name>__coarse` takes the caller's thread count as a last i64 parameter and may be launched
    # with fewer, longer-running threads; results must equal the original under the caller's launch.
    src = kb.load("vadd_i32")
    opt = ptx.optimized_bir(src)
    rng = np.random.default_rng(17)
    for n, physical, logical in [(1000, 64, 1024), (1003, 32, 2000), (100, 8, 40), (37, 4, 64), (4099, 128, 4099), (9, 1, 9), (0, 2, 8)]:
        a = rng.integers(-2**30, 2**30, max(n, 1) + 8, dtype=np.int64).astype(np.int32)
        bb = a[::-1].copy()
        c0 = np.full(max(n, 1) + 8, 0x7fffffff, np.int32); c1 = c0.copy()
        run_kernel(src, "vadd_i32", [a, bb, c0, n], logical)
        run_kernel(opt, "vadd_i32__coarse", [a, bb, c1, n, logical], physical)
        assert np.array_equal(c0, c1), (n, physical, logical)


def test_reduction_loop_vectoriser(ptx):
    src = kb.load("max_i32_strided")
    opt = ptx.optimized_bir(src)
    assert "load v4i32" in opt
    rng = np.random.default_rng(13)
    for n, threads in [(1000, 64), (1003, 32), (5, 8), (0, 4), (64, 64), (999, 1), (17, 3), (4096, 128)]:
        x = rng.integers(-2**31, 2**31, max(n, 1), dtype=np.int64).astype(np.int32)
        for plant in (None, 0, n - 1, n // 2):
            if plant is not None and n:
                x[:] = np.minimum(x, 2**31 - 2)
                x[plant] = 2**31 - 1
            o0 = np.array([-2**31], np.int32); o1 = o0.copy()
            run_kernel(src, "max_i32_strided", [x, o0, n], threads)
            run_kernel(opt, "max_i32_strided", [x, o1, n], threads)
            assert o0[0] == o1[0] == (x[:n].max() if n else -2**31), (n, threads, plant)


def test_butterfly_becomes_one_warp_reduce_per_stage(ptx):
    opt = ptx.optimized_bir(kb.load("max_i32"))
    assert opt.count("warp.reduce.max i32") == 2 and "shuffle" not in opt
    assert "atomic.max i32 ptr.global" in opt and "barrier" in opt and "load v4i32" in opt


def test_opt_level_zero_keeps_the_module_shape(ptx):
    opt0 = ptx.optimized_bir(kb.load("max_i32"), b.EmitOpts(opt_level=0))
    assert opt0.count("shuffle.xor") == 10 and "v4" not in opt0


def _header(text, kernel):
    line = next(l for l in text.splitlines() if l.startswith(f"// kernel {kernel}:"))
    return line, int(line.split("est_regs=")[1].split()[0]), int(line.split("budget=")[1].split()[0])


def test_register_estimate_bounds_the_unroll(ptx):
    # budget = 65536 / (threads per CTA x CTAs per SM): 256 x 4 (the defaults) for a kernel without launch
    # bounds, 256 x 8 for max_i32, whose module asks for eight CTAs per SM
    line, est, budget = _header(ptx.emit(kb.load("vadd_i32")).text, "vadd_i32")
    assert budget == 64 and est <= budget and "unroll=2" in line
    line, est, budget = _header(ptx.emit(kb.load("max_i32")).text, "max_i32")
    assert budget == 32 and est <= budget + budget // 4 and "unroll=4" in line
    # a smaller budget, or a cap on the unroll, through the options: no environment variable is read
    line, est, budget = _header(ptx.emit(kb.load("max_i32"), b.EmitOpts(target_variant="sm_100a,regs=24")).text, "max_i32")
    assert "unroll=2" in line or "unroll=1" in line
    line, _, _ = _header(ptx.emit(kb.load("helper_chain" if False else "vadd_i32"), b.EmitOpts(target_variant="sm_100a,max_unroll=1")).text, "vadd_i32")
    assert "unroll=1" in line
    with pytest.raises(b.Diag):
        ptx.emit(kb.load("vadd_i32"), b.EmitOpts(target_variant="sm_100a,bogus=1"))


def test_emit_ignores_the_environment(ptx, monkeypatch):
    # Backend::emit is a pure function of (module, options): byte-identical output whatever the process
    # environment holds (crates/basalt-backend/src/backend.rs:152-156)
    before = ptx.emit(kb.load("vadd_i32")).text
    for name in ("BASALT_MAX_UNROLL", "BASALT_RT_NO_PAIR", "BASALT_K_STREAM_WAVES"):
        monkeypatch.setenv(name, "1")
    assert ptx.emit(kb.load("vadd_i32")).text == before


def test_register_estimate_against_ptxas(ptx, tmp_path):
    # The register-budget pass's figure for each of the five benchmark kernels brackets what ptxas uses:
    # ptxas <= estimate <= 1.5 x ptxas.
    import re
    import shutil
    import subprocess
    exe = shutil.which("ptxas") or "/usr/local/cuda/bin/ptxas"
    srcs = {"vadd_i32": kb.load("vadd_i32"), "max_i32": kb.load("max_i32"), "helper_chain": kb.helper_chain(),
            "sgemm_f32": kb.sgemm_cta128(4096, 4096, 4096), "matmul_f16": kb.matmul_f16(8192, 8192, 8192)}
    seen = 0
    for name, src in srcs.items():
        text = ptx.emit(src).text
        p = tmp_path / f"{name}.ptx"
        p.write_text(text)
        r = subprocess.run([exe, "-arch=sm_100a", "-v", str(p), "-o", "/dev/null"], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        used = {k: int(v) for k, v in re.findall(r"Compiling entry function '(\S+)' for 'sm_100a'\n[^\n]*\n[^\n]*\n[^\n]*Used (\d+) registers", r.stderr)}
        assert "spill" not in r.stderr or "0 bytes spill stores" in r.stderr
        for kernel, regs in used.items():
            _, est, budget = _header(text, kernel)
            assert regs <= est <= 1.5 * regs, (kernel, regs, est)
            seen += 1
    assert seen >= 8      # five kernels, the coarse twins of the two elementwise ones, the two-SM twin of the matmul


def test_construct_ssa_promotes_front_end_slots(ptx):
    # crates/basalt-passes/src/ssa.rs:4-10: local and param slots used only as load/store addresses
    # become SSA values and phis; results under the oracle model are unchanged.
    src = kb.load("slot_form_sum")
    for level in (0, 2):
        opt = ptx.optimized_bir(src, b.EmitOpts(opt_level=level))
        assert "ptr.local" not in opt and "ptr.param" not in opt and opt.count("phi i32") == 3
        for n, threads in [(10, 16), (0, 4), (-3, 4), (5, 3), (33, 64)]:
            o0 = np.full(70, -7, np.int32); o1 = o0.copy()
            run_kernel(src, "slot_form_sum", [o0, n], threads)
            run_kernel(opt, "slot_form_sum", [o1, n], threads)
            assert np.array_equal(o0, o1), (level, n, threads)
    text = ptx.emit(src).text
    assert ".local" not in text


def test_shared_slots_and_address_taken_slots_stay_in_memory(ptx):
    from basalt_b200.birasm import assemble
    src = assemble("""module {
  shared_mem_bytes 0
  target_dtypes i32

  func @k(ptr.global, i32) -> void {
  entry:
    %s = const.i ptr.shared 0
    store i32 ptr.shared %s, %arg1, align 4
    barrier
    %v = load i32 ptr.shared %s, align 4
    %l = const.i ptr.local 65536
    %eight = const.i i64 0
    %l2 = add ptr.local %l, %eight
    store i32 ptr.local %l2, %v, align 4
    %w = load i32 ptr.local %l, align 4
    store i32 ptr.global %arg0, %w, align 4
    ret
  }
}
""")
    opt = ptx.optimized_bir(src, b.EmitOpts(opt_level=0))
    assert "ptr.shared" in opt and "ptr.local" in opt   # CTA-visible memory and an indexed local are not SSA values


IN_PLACE_SOURCE = """
__global__ void in_place(int* a, int* c, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { a[i] = a[i] + a[i]; c[i] = a[i]; }
}
__global__ void two_names(const int* a, int* b, int* c, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { b[i] = 2 * a[i]; c[i] = a[i]; }
}
"""


def test_a_load_after_a_store_is_not_hoisted_above_it(ptx):
    # The vectorised body issues all loads first; a body that reads back what it has just stored
    # (the same element, or the same buffer under a second parameter) must keep program order.
    src = b.compile_cuda(IN_PLACE_SOURCE)
    opt = ptx.optimized_bir(src)
    for n, threads in [(4, 4), (1000, 1024), (37, 64), (100, 40)]:
        a0 = np.arange(1, max(n, 1) + 9, dtype=np.int32); a1 = a0.copy()
        c0 = np.full_like(a0, -1); c1 = c0.copy()
        run_kernel(src, "in_place", [a0, c0, n], threads)
        run_kernel(opt, "in_place", [a1, c1, n], threads)
        assert np.array_equal(a0, a1) and np.array_equal(c0, c1), (n, threads)
        m = min(n, threads)
        assert np.array_equal(c0[:m], 2 * np.arange(1, m + 1))
        # one buffer passed as input and as output
        x0 = np.arange(1, max(n, 1) + 9, dtype=np.int32); x1 = x0.copy()
        d0 = np.full_like(x0, -1); d1 = d0.copy()
        run_kernel(src, "two_names", [x0, x0, d0, n], threads)
        run_kernel(opt, "two_names", [x1, x1, d1, n], threads)
        assert np.array_equal(x0, x1) and np.array_equal(d0, d1), (n, threads)
        assert np.array_equal(d0[:m], 2 * np.arange(1, m + 1))
