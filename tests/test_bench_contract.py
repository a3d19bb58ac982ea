"""The reference arm of bench.py runs without a GPU (it times the CPU launch path): its one JSON line
must carry the keys the benchmark contract names, on the same metric and workload as the device arm."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, r.stdout[-2000:]
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"].startswith("max_i32") and d["unit"] == "GB/s"
    for key in ("value", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["vs_baseline"] is None and d["higher_is_better"] is True and "workload" in d["config"]
    cpu = d["cpu_baseline"]
    assert cpu["kind"] == "port" and cpu["cores"] == 1 and cpu["value"] == d["value"] and "x86-regalloc" in cpu["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert 0.05 < d["value"] < 50      # a single core streaming int32: well inside this bracket
    # the device arm prints the same `config` object and honours the same warm-up floor
    sys.path.insert(0, ROOT)
    import bench
    assert d["config"] == bench.headline_config(1 << 28, 1) and d["warmup"] == 3
