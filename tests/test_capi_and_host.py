"""The C-ABI library loads without a GPU and exports every symbol the headers declare; host-side
runtime logic (sharding, error reporting) behaves; the N>1 path runs as two gloo ranks on CPU."""
import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest

import basalt_b200 as b
from basalt_b200._lib import LIB_PATH, lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for h in ("basalt_b200.h", "basalt_b200_kernels.h"):
        text = open(os.path.join(ROOT, "include", h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(basalt_(?:b200|rt|k)_\w+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert len(names) >= 45
    raw = ctypes.CDLL(LIB_PATH)
    for n in names:
        assert hasattr(raw, n), n
    assert set(names) == set(lib._basalt_signatures), "ctypes table and headers disagree"


def test_library_has_no_link_time_gpu_dependency():
    out = subprocess.run(["ldd", LIB_PATH], capture_output=True, text=True).stdout
    assert "libcuda" not in out and "libnccl" not in out and "libcudart" not in out


def test_driver_load_reports_a_missing_driver():
    try:
        ctypes.CDLL("libcuda.so.1")
        pytest.skip("a CUDA driver is installed here")
    except OSError:
        pass
    with pytest.raises(b.CudaError) as e:
        b.CudaDriver.load()
    assert e.value.kind == 1 and "CUDA driver library not found" in str(e.value)


@pytest.mark.parametrize("total, world, align", [(2**28, 8, 4), (1000, 3, 4), (7, 8, 1), (0, 2, 4), (4096, 4, 128), (130, 2, 128)])
def test_shard_ranges_partition_the_work(total, world, align):
    covered = 0
    prev_end = 0
    for r in range(world):
        lo, hi = b.shard_range(total, world, r, align)
        assert lo == prev_end and lo <= hi <= total
        assert lo % align == 0 or lo == total
        covered += hi - lo
        prev_end = hi
    assert covered == total and prev_end == total
    sizes = [b.shard_range(total, world, r, align)[1] - b.shard_range(total, world, r, align)[0] for r in range(world)]
    assert max(sizes) - min(sizes) <= align


def test_two_rank_sharded_max_on_gloo(tmp_path):
    script = tmp_path / "ranks.py"
    script.write_text(f"""
import sys
sys.path.insert(0, {ROOT!r})
import numpy as np
from basalt_b200 import sharding, workloads
g = sharding.RankGroup.from_env("gloo")
assert g.world == 2
n = 100003
x = workloads.u32(0xBA5A1702, n).view(np.int32).copy()
x[50001] = 2**31 - 1 if False else x[50001]
lo, hi = g.shard(n, 4)
for plant in (0, n - 1, 50000, 50004):      # first, last, and both sides of the shard boundary
    y = np.minimum(x, 2**31 - 2); y[plant] = 2**31 - 1
    got = sharding.reduce_max_sharded(g, y[lo:hi], lambda s: s.max())
    assert got == 2**31 - 1, (plant, got)
got = sharding.reduce_max_sharded(g, x[lo:hi], lambda s: s.max())
assert got == x.max()
assert sharding.reduce_max_sharded(g, x[0:0], lambda s: s.max()) == -2**31
t = g.max_float(1.0 + g.rank)
assert t == 2.0
blob = g.broadcast_bytes(b"id-from-rank-0" if g.rank == 0 else None)
assert blob == b"id-from-rank-0"
g.barrier()
print("rank", g.rank, "ok", lo, hi)
""")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29617", str(script)], capture_output=True, text=True, env=env, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("ok") == 2


def test_cli_follows_the_reference_conventions(tmp_path):
    # crates/basalt-cli/tests/nvidia_ptx_flag.rs:22-85: PTX on stdout or at -o, non-zero exit with the E-code on stderr
    from basalt_b200 import kernels_bir as kb
    cli = os.path.join(ROOT, "basalt_b200", "basalt-b200")
    src = tmp_path / "k.bir"
    src.write_text(kb.load("vadd_i32"))
    r = subprocess.run([cli, "--nvidia-ptx", str(src)], capture_output=True, text=True)
    assert r.returncode == 0 and ".target sm_100a" in r.stdout and ".visible .entry vadd_i32(" in r.stdout
    assert r.stdout == b.Ptx().emit(kb.load("vadd_i32")).text
    out = tmp_path / "k.ptx"
    r = subprocess.run([cli, "--nvidia-ptx", str(src), "-o", str(out), "-O0"], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout == "" and "v4" not in out.read_text()
    bad = tmp_path / "bad.bir"
    bad.write_text("module {")
    r = subprocess.run([cli, "--nvidia-ptx", str(bad)], capture_output=True, text=True)
    assert r.returncode == 1 and r.stderr.startswith("E400: ")
    r = subprocess.run([cli, "--nvidia-ptx", str(src), "--frobnicate"], capture_output=True, text=True)
    assert r.returncode == 1 and r.stderr.startswith("E100: ")
    r = subprocess.run([cli, "--ir", str(src)], capture_output=True, text=True)
    assert r.returncode == 0 and "load v4i32" in r.stdout


def test_multicast_result_reports_why_it_is_unavailable():
    # no CUDA device here: the helper must say so and return None on every rank instead of raising
    from basalt_b200.sharding import MulticastResult, RankGroup
    assert MulticastResult.open(RankGroup(), 4096, 0) is None
    assert MulticastResult.why_not


def test_peer_order_makes_every_step_of_an_exchange_a_permutation():
    from basalt_b200.sharding import RankGroup
    for world in (2, 4, 8):
        orders = [RankGroup(rank=r, world=world).peer_order() for r in range(world)]
        for r, o in enumerate(orders):
            assert sorted(o) == [x for x in range(world) if x != r]
        for step in range(world - 1):       # at each step no two ranks address the same receiver
            assert sorted(o[step] for o in orders) == list(range(world))
