"""Seeded synthetic inputs for the five benchmark workloads.

The reference measures nothing at scale (its largest test is N = 1024 / 32^3), so the inputs are
synthetic with the shapes and value distributions the benchmark configuration names.  One
counter-based generator, SplitMix64 at `seed + (i+1)*golden`, feeds every workload; the CPU oracle
has its own C implementation of the same functions and the tests assert both produce the same
bytes."""
from __future__ import annotations

import numpy as np

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
SEEDS = {"vadd_i32": 0xBA5A1701, "max_i32": 0xBA5A1702, "helper_chain": 0xBA5A1703, "sgemm_f32": 0xBA5A1704,
         "matmul_f16": 0xBA5A1705}


def splitmix64(seed: int, start: int, count: int) -> np.ndarray:
    """Draws start..start+count-1 of the stream, as uint64."""
    with np.errstate(over="ignore"):
        i = np.arange(start + 1, start + count + 1, dtype=np.uint64)
        z = np.uint64(seed) + i * _GOLDEN
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _chunks(n: int, step: int = 1 << 24):
    for s in range(0, n, step):
        yield s, min(step, n - s)


def _draw32(seed: int, n: int, out: np.ndarray):
    for s, c in _chunks(n):
        out[s:s + c] = (splitmix64(seed, s, c) >> np.uint64(32)).astype(np.uint32)
    return out


def u32(seed: int, n: int, out: np.ndarray | None = None) -> np.ndarray:
    """uint32 uniform over the full range (viewed as int32: the max_i32 input)."""
    return _draw32(seed, n, out if out is not None else np.empty(n, dtype=np.uint32))


def i32_pm30(seed: int, n: int, out: np.ndarray | None = None) -> np.ndarray:
    """int32 uniform in [-2^30, 2^30): the vadd_i32 inputs."""
    out = out if out is not None else np.empty(n, dtype=np.int32)
    for s, c in _chunks(n):
        d = (splitmix64(seed, s, c) >> np.uint64(33)).astype(np.int64) - (1 << 30)
        out[s:s + c] = d.astype(np.int32)
    return out


def f32_pm1(seed: int, n: int) -> np.ndarray:
    """float32 uniform in [-1, 1): 24 random bits times 2^-23, minus 1 (all exact)."""
    out = np.empty(n, dtype=np.float32)
    for s, c in _chunks(n):
        d = (splitmix64(seed, s, c) >> np.uint64(40)).astype(np.float32)
        out[s:s + c] = d * np.float32(1.0 / 8388608.0) - np.float32(1.0)
    return out


def f16_normal01(seed: int, n: int) -> np.ndarray:
    """binary16 ~ N(0,1)*0.1: a 12-term Irwin-Hall sum of 16-bit uniforms (three 64-bit draws per
    value), centred and scaled to unit variance, times 0.1, rounded once to f16.  No transcendental
    function is involved, so every platform produces the same bits."""
    out = np.empty(n, dtype=np.float16)
    m = np.uint64(0xFFFF)
    for s, c in _chunks(n, 1 << 22):
        z = splitmix64(seed, 3 * s, 3 * c).reshape(c, 3)
        tot = ((z & m) + ((z >> np.uint64(16)) & m) + ((z >> np.uint64(32)) & m) + (z >> np.uint64(48))).sum(axis=1)
        zn = (tot.astype(np.int64) - 393210).astype(np.float64) * (1.0 / 65536.0)
        out[s:s + c] = (zn * 0.1).astype(np.float16)
    return out
