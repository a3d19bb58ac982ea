"""The reference's known-answer fixtures (examples/cpu_launch_*.c) run on the device through the
reference's own CPU launch ABI -- host pointers in, results in host memory -- with the emitted
kernels at both optimisation levels.  Expected values come from the fixture formulas; the CPU
oracle is checked against the same values in test_oracle_pins.py."""
import numpy as np
import pytest

import basalt_b200 as b
from basalt_b200 import kernels_bir as kb
from _gpu import emitted
from _util import sgemm_fixture

pytestmark = pytest.mark.gpu
LEVELS = [0, 2]


@pytest.mark.parametrize("level", LEVELS)
def test_vector_add_f32(gpu, level):
    n = 1024
    a = np.arange(n, dtype=np.float32); bb = (2 * np.arange(n)).astype(np.float32); c = np.full(n, -1.0, np.float32)
    gpu.cpu_launch(emitted(gpu, kb.load("vector_add_f32"), "vector_add", level), [a, bb, c, b.i32(n)], n)
    assert np.array_equal(c, a + bb)


@pytest.mark.parametrize("level", LEVELS)
def test_chain_and_square(gpu, level):
    n = 1024
    x = (np.arange(n) - n // 2).astype(np.int32)
    for name, kern, want in (("chain_vector", "chain_vector", -2 * x + 1), ("square_vector", "square_vector", x * x)):
        out = np.full(n, 0x7fffffff, np.int32)
        gpu.cpu_launch(emitted(gpu, kb.load(name), kern, level), [x, out, b.i32(n)], n)
        assert np.array_equal(out, want), name


@pytest.mark.parametrize("level", LEVELS)
def test_stress_is_191(gpu, level):
    a = ((np.arange(20) + 1) * 0.5 - 3.0).astype(np.float32)
    out = np.array([-1.0], np.float32)
    gpu.cpu_launch(emitted(gpu, kb.stress(), "stress", level), [a, out, b.i32(1)], 1)
    assert out[0] == np.float32(191.0)   # bit-exact: the emitter never contracts mul+add


@pytest.mark.parametrize("threads", [1, 32, 96])
def test_mma2x2(gpu, threads):
    a = np.array([1, 2, 3, 4], np.float32); bb = np.array([5, 6, 7, 8], np.float32); c = np.full(4, 0.5, np.float32)
    d = np.full(4, -1.0, np.float32)
    gpu.cpu_launch(emitted(gpu, kb.load("mma2x2"), "mma2x2"), [a, bb, c, d], threads, block=128)
    assert np.array_equal(d, np.array([19.5, 22.5, 43.5, 50.5], np.float32))


@pytest.mark.parametrize("threads", [1, 64, 256])
def test_tiled_sgemm_32(gpu, threads):
    a, bb, c = sgemm_fixture(32, 32, 32)
    want = (a.astype(np.int64) @ bb.astype(np.int64) + c.astype(np.int64)).astype(np.float32)
    d = np.full(1024 + 768, -1.0, np.float32)
    gpu.cpu_launch(emitted(gpu, kb.load("tiled_sgemm_f32"), "tiled_sgemm_f32"), [a, bb, c, d], threads, block=256)
    assert np.array_equal(d[:1024].reshape(32, 32), want)
    assert np.all(d[1024:] == -1.0)


@pytest.mark.parametrize("level", LEVELS)
def test_triton_matmul(gpu, level):
    a, bb, c = sgemm_fixture(4, 3, 5)
    want = (a.astype(np.int64) @ bb.astype(np.int64) + c.astype(np.int64)).astype(np.float32)
    out = np.full(65536, -1.0, np.float32)
    gpu.cpu_launch(emitted(gpu, kb.load("tri_matmul"), "matmul_kernel", level), [a, bb, c, out, b.i64(5)], 1)
    assert np.array_equal(out[:12].reshape(4, 3), want)
    assert np.all(out[12:] == -1.0)


@pytest.mark.parametrize("level", LEVELS)
def test_triton_masked_vadd_leaves_poison(gpu, level):
    n, block = 1000, 1024
    a = np.arange(n, dtype=np.float32); bb = (2 * np.arange(n)).astype(np.float32); c = np.full(32768, -1.0, np.float32)
    gpu.cpu_launch(emitted(gpu, kb.load("tri_vadd"), "vector_add", level), [a, bb, c, b.i64(n), b.i64(block)], 1)
    assert np.array_equal(c[:n], a + bb)
    assert np.all(c[n:] == -1.0)


@pytest.mark.parametrize("flavour", ["cuda", "triton"])
def test_c_drivers_link_against_the_shim_libraries(gpu, tmp_path, flavour):
    """A C host program written against the reference's CPU-launch signatures (tests/drivers/*.c,
    the checks of examples/cpu_launch_*.c) links against libbasalt_cpu_launch_<flavour>.so in place
    of the x86 object file and passes on the GPU."""
    import os
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler on this box")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pkg = os.path.join(root, "basalt_b200")
    exe = tmp_path / f"{flavour}_fixtures"
    subprocess.run(["gcc", "-O1", "-o", str(exe), os.path.join(root, "tests", "drivers", f"{flavour}_fixtures.c"), f"-L{pkg}",
                    f"-lbasalt_cpu_launch_{flavour}", f"-Wl,-rpath,{pkg}"], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.startswith("PASS"), r.stdout + r.stderr


@pytest.mark.parametrize("level", LEVELS)
def test_slot_form_kernel_runs_after_ssa_construction(gpu, level):
    n = 1000
    out = np.full(n + 8, -7, np.int32)
    gpu.cpu_launch(emitted(gpu, kb.load("slot_form_sum"), "slot_form_sum", level), [out, b.i32(n)], 1024)
    assert np.array_equal(out[:n], np.arange(n) + n * (n - 1) // 2) and np.all(out[n:] == -7)
