"""Writes tests/golden/golden.json: for every workload, the SHA-256 of the CPU oracle's output on the
seeded synthetic input, at a small size and at the benchmark configuration's full size, plus the
reference's own known answers.  The oracle is oracle/basalt_oracle.c (built by oracle/build.py);
inputs are basalt_b200.workloads.  Run from the repository root:

    python tests/golden/make_golden.py

The file pins three things at once: the input generators (a changed generator changes every
hash), the oracle (tests/test_golden.py recomputes the small cases on the CPU), and the device path
(tests/test_gpu_golden.py compares what the GPU computes from sources in all three input forms --
BIR, CUDA-C, Triton -- with the same hashes, at both optimisation levels).
"""
import ctypes
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from basalt_b200 import workloads as w  # noqa: E402
from oracle import build as oracle_build  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.json")
SMALL, FULL = "small", "full"


def vp(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).view(np.uint8)).hexdigest()


def cases():
    """(name, size label, n) of every hashed case."""
    return [("vadd_i32", SMALL, 4099), ("vadd_i32", FULL, 1 << 20),
            ("helper_chain", SMALL, 4099), ("helper_chain", FULL, 1 << 26),
            ("max_i32", SMALL, 100003), ("max_i32", FULL, 1 << 28),
            ("vector_add_f32", SMALL, 1000),
            ("sgemm_f32_rows", SMALL, 128), ("matmul_f16_rows", SMALL, 128)]


def compute(orc, name: str, n: int) -> dict:
    i32, i64 = ctypes.c_int32, ctypes.c_int64
    if name == "vadd_i32":
        a = w.i32_pm30(w.SEEDS[name], n); b = w.i32_pm30(w.SEEDS[name] + 1, n)
        c = np.empty(n, np.int32)
        orc.orc_vadd_i32(vp(a), vp(b), vp(c), i32(n), i64(n))
        return {"n": n, "sha256": sha(c), "first": c[:4].tolist()}
    if name == "helper_chain":
        x = np.empty(n, np.uint32)
        orc.orc_fill_u32(ctypes.c_uint64(w.SEEDS[name]), i64(n), vp(x))
        y = np.empty(n, np.uint32)
        orc.orc_helper_chain_u32(vp(x), vp(y), i32(n), i64(n))
        return {"n": n, "sha256": sha(y), "first": y[:4].tolist()}
    if name == "max_i32":
        x = np.empty(n, np.uint32)
        orc.orc_fill_u32(ctypes.c_uint64(w.SEEDS[name]), i64(n), vp(x))
        out = np.array([-2**31], np.int32)
        orc.orc_max_i32(vp(x), vp(out), i32(n), i64(n))
        return {"n": n, "value": int(out[0])}
    if name == "vector_add_f32":
        a = w.f32_pm1(31, n); b = w.f32_pm1(32, n)
        c = np.empty(n, np.float32)
        orc.orc_vector_add_f32(vp(a), vp(b), vp(c), i32(n), i64(n))
        return {"n": n, "sha256": sha(c)}
    if name == "sgemm_f32_rows":       # the oracle's unfused ascending-k rows of a 128 x 128 x 64 product: tolerance cases hash the ORACLE only
        A = w.f32_pm1(w.SEEDS["sgemm_f32"], n * 64).reshape(n, 64); B = w.f32_pm1(w.SEEDS["sgemm_f32"] + 1, 64 * n).reshape(64, n)
        C = np.empty((n, n), np.float32)
        orc.orc_sgemm_f32_rows(vp(A), vp(B), vp(C), n, n, 64, 0, n)
        return {"n": n, "k": 64, "sha256": sha(C)}
    if name == "matmul_f16_rows":
        A = w.f16_normal01(w.SEEDS["matmul_f16"], n * 64).reshape(n, 64); B = w.f16_normal01(w.SEEDS["matmul_f16"] + 1, 64 * n).reshape(64, n)
        C = np.empty((n, n), np.float16)
        orc.orc_matmul_f16_rows(vp(A), vp(B), vp(C), n, n, 64, 0, 0, n)
        return {"n": n, "k": 64, "sha256": sha(C)}
    raise KeyError(name)


# Known answers the reference itself holds for this path (file:line inside the reference project).
KNOWN = {
    "stress_fold": {"value": 191.0, "source": "examples/cpu_launch_stress.c:14-47; tests/diff/golden/stress.txt"},
    "mymathhomework": {"value": 20, "source": "examples/cpu_launch_mymathhomework.c:15-24; tests/diff/golden/mymathhomework.txt"},
    "mma2x2": {"value": [19.5, 22.5, 43.5, 50.5], "source": "examples/cpu_launch_mma2x2.c:17-21"},
    "vector_add": {"rule": "c[i] = 3 i for a[i] = i, b[i] = 2 i, N = 1024", "source": "examples/cpu_launch_vadd.c:18-37; tests/diff/golden/vector_add.txt"},
    "chain_vector": {"rule": "out[i] = -2 in[i] + 1 for in[i] = i - 512, N = 1024", "source": "examples/cpu_launch_device_helper_chain.c:18-35"},
    "tri_vadd": {"rule": "c[i] = 3 i for i < 1000, c[i] = -1 (poison) for 1000 <= i < 1024", "source": "examples/cpu_launch_triton_vadd.c:31-58; tests/diff/golden/tri_vadd.txt"},
    "tri_matmul": {"rule": "D = A@B + C, M=4 K=5 N=3, A=((3i+j)%7)+1, B=((i+5j)%7)+1, C=(i+j)%4", "source": "examples/cpu_launch_triton_matmul.c:39-89; tests/diff/golden/tri_matmul.txt"},
}


def main():
    orc = ctypes.CDLL(oracle_build.build())
    doc = {"generator": "tests/golden/make_golden.py", "seeds": {k: hex(v) for k, v in w.SEEDS.items()}, "known_answers": KNOWN, "cases": {}}
    for name, label, n in cases():
        doc["cases"].setdefault(name, {})[label] = compute(orc, name, n)
        print(name, label, doc["cases"][name][label], flush=True)
    with open(OUT, "w") as f:
        json.dump(doc, f, indent=1, sort_keys=True)
        f.write("\n")


if __name__ == "__main__":
    main()
