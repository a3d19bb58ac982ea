"""tests/golden/golden.json against the CPU oracle: the small cases and the full-size vadd are
recomputed here (seconds), so a drift of the input generators or of the oracle shows up without a
GPU.  The generating script is tests/golden/make_golden.py."""
import ctypes
import importlib.util
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_generator():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def golden():
    with open(os.path.join(HERE, "golden", "golden.json")) as f:
        return json.load(f)


def test_golden_file_matches_the_oracle(orc):
    gen, doc = load_generator(), golden()
    assert {name for name, _, _ in gen.cases()} == set(doc["cases"])
    for name, label, n in gen.cases():
        if label == gen.FULL and name != "vadd_i32":
            continue      # 2^26 chain outputs and the 2^28 maximum are recomputed by the generator only
        assert gen.compute(orc, name, n) == doc["cases"][name][label], (name, label)
    assert doc["seeds"] == {k: hex(v) for k, v in __import__("basalt_b200").workloads.SEEDS.items()}


def test_known_answers_are_the_references(orc):
    known = golden()["known_answers"]
    a = ((np.arange(20) + 1) * 0.5 - 3.0).astype(np.float32)
    out = np.zeros(1, np.float32)
    orc.orc_stress(a.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p), ctypes.c_int32(1), ctypes.c_int64(1))
    assert float(out[0]) == known["stress_fold"]["value"] == 191.0
    A = np.array([1, 2, 3, 4], np.float32); B = np.array([5, 6, 7, 8], np.float32); Cm = np.full(4, 0.5, np.float32); D = np.zeros(4, np.float32)
    p = lambda x: x.ctypes.data_as(ctypes.c_void_p)
    orc.orc_mma_f32(p(A), p(B), p(Cm), p(D), 2, 2, 2, 0, 0, ctypes.c_int64(0), ctypes.c_int64(0), ctypes.c_int64(0), ctypes.c_int64(0))
    assert D.tolist() == known["mma2x2"]["value"]
    assert known["mymathhomework"]["value"] == 2 + 3 + 15      # (2 + 3) * 4
