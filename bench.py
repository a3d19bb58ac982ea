#!/usr/bin/env python
"""Benchmark of the Basalt sm_100a device path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-others]
    python bench.py --profile {max_i32,vadd_i32,helper_chain,sgemm_f32,matmul_f16} [--size S]     (small cases for ncu)

Headline workload (N=1 and per rank at N>1): the max_i32 reduction over 2^28 int32 (1 GiB), the
benchmark configuration the metric is quoted on.  A step is one pass over the rank's batch: one
launch of the emitted sm_100a kernel through the C-ABI runtime, plus, at N>1, the 4-byte
allreduce(max) of the partial maxima: one small kernel of stores to and loads from peer-mapped
memory (basalt_rt_peer_allreduce_max_i32; --nccl-exchange uses ncclAllReduce instead).  Scaling is
weak: every rank owns a 2^28-element contiguous shard of an N*2^28-element array.

One JSON line is printed by rank 0.  Beside the headline keys it carries `configs`: one entry for each
of the five benchmark configurations (vadd_i32, max_i32, helper_chain, sgemm_f32, matmul_f16), each with
its own `roofline`, `cpu_baseline`, `e2e` and `parity`, the hand-written comparator kernel, and, at
N > 1, the sharded forms with the result of every variant checked on every rank.  Inputs are the
seeded synthetic arrays of basalt_b200/workloads.py, generated on the device by the same counter-based
generator (identical bytes).  `--impl reference` times the reference's CPU launch path (the restatement
of its register-allocating x86-64 back end under oracle/, one thread) on the headline workload instead.
"""
from __future__ import annotations

import argparse
import ctypes
import hashlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_MAX = 1 << 28          # elements per rank: 1 GiB of int32, far larger than the 126 MB L2
METRIC = "max_i32 reduction throughput (HBM GB/s)"
L2_BYTES = 126e6
FP32_LANES_PER_SM = 128  # FFMA per clock per SM
F16_TOL, SGEMM_TOL = 2e-3, 1e-4


def headline_config(n: int, world: int) -> dict:
    """The `config` object of the JSON line; the device arm and the reference arm print the same one."""
    return {"workload": f"max_i32: signed max over {n} int32 per GPU, uniform over the full int32 range (SplitMix64 counter stream, seed 0xBA5A1702 + rank), one pass per step",
            "elements_per_gpu": n, "l2": f"input ({4 * n >> 20} MiB per GPU) is larger than the 126 MB L2; no flush needed",
            "parallelism": f"contiguous shards x{world}"}


def measured_peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "tf_burst": float(p.get("bf16_tflops", 1590.0)), "tf_sustained": float(p.get("bf16_tflops_sustained", 1400.0)),
                "sm_max_mhz": float(p.get("sm_max_mhz", 1965.0)), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "tf_burst": 1590.0, "tf_sustained": 1400.0, "sm_max_mhz": 1965.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock, power and throttle reasons with nvidia-smi every 200 ms."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [r for t, r in self.rows if t0 - 0.1 <= t <= t1 + 0.3 and len(r) >= 7] or [r for _, r in self.rows if len(r) >= 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for k, n in enumerate(names) if any(r[3 + k] == "Active" for r in rows)]
        num = lambda s: float(s) if s.replace(".", "", 1).isdigit() else float("nan")
        return {"sm_mhz": statistics.median(num(r[0]) for r in rows), "sm_max_mhz": num(rows[0][1]),
                "power_w_max": max(num(r[2]) for r in rows), "power_w_median": statistics.median(num(r[2]) for r in rows), "reasons": reasons, "samples": len(rows)}


# ------------------------------------------------------------------------------------------------
# The CPU legs: the only places this file touches oracle/ (as the timed baseline, and as the checker
# of sampled matmul rows).
# ------------------------------------------------------------------------------------------------
_ORC = None


def load_oracle():
    global _ORC
    if _ORC is None:
        from oracle import build as oracle_build
        lib = ctypes.CDLL(oracle_build.build())
        for name in ("orc_time_max_i32", "orc_time_vadd_i32", "orc_time_helper_chain", "orc_time_sgemm_scalar", "orc_time_matmul_f16_scalar"):
            getattr(lib, name).restype = ctypes.c_double
        _ORC = lib
    return _ORC


def vp(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def time_oracle_max(x: np.ndarray, reps: int):
    """Seconds for one pass of the oracle's max_i32 over x (best of reps), and its result."""
    lib = load_oracle()
    res = ctypes.c_int32()
    t = lib.orc_time_max_i32(vp(x), ctypes.c_int32(len(x)), reps, ctypes.byref(res))
    return t, res.value


def regalloc_jit(bir_name: str):
    """The kernel compiled from its BIR text by the restatement of the reference's register-allocating
    x86-64 back end (oracle/x86_regalloc.cpp): called as the reference's CPU launch calls its object
    code, kernel(params..., nthreads), one thread (crates/basalt-x86/src/regalloc.rs:452-481)."""
    from basalt_b200 import kernels_bir as kb
    from oracle import build as oracle_build
    oracle_build.build()
    from oracle import x86_regalloc
    return x86_regalloc.compile(kb.load(bir_name))


def time_regalloc_max(x: np.ndarray, reps: int):
    """Seconds for one pass of max_i32 over x (best of reps) through the x86-regalloc restatement: the
    CPU-runnable form of the kernel (one atomic max per element; that back end refuses warp shuffles).
    Returns (seconds, result, code bytes)."""
    k = regalloc_jit("max_i32_atomic")
    out = np.array([-2**31], np.int32)
    best = float("inf")
    for _ in range(reps):
        out[0] = -2**31
        t0 = time.perf_counter()
        k(x, out, len(x), len(x))
        best = min(best, time.perf_counter() - t0)
    return best, int(out[0]), len(k.code)


def cpu_max(x: np.ndarray, reps: int):
    """The CPU baseline of the headline workload: (seconds, result, description, C-loop GB/s)."""
    t_c, r_c = time_oracle_max(x, reps)
    c_gbs = 4.0 * len(x) / t_c / 1e9
    try:
        t, r, nbytes = time_regalloc_max(x, reps)
    except OSError as e:      # no executable memory to be had: the C loop stands in
        return t_c, r_c, f"the oracle's C loop (x86 JIT unavailable: {e})", c_gbs
    if r != r_c:
        raise RuntimeError(f"the two CPU oracles disagree: {r} vs {r_c}")
    return t, r, f"restated x86-regalloc back end, {nbytes} bytes of emitted code, one atomic max per element, nthreads = n, one thread", c_gbs


def cpu_vadd(a: np.ndarray, b_: np.ndarray, want_sha: str | None):
    """vadd_i32 at its configured size through the x86-regalloc restatement, one thread; best of 20 passes."""
    n = len(a)
    c = np.empty(n, np.int32)
    try:
        k = regalloc_jit("vadd_i32")
        how = f"restated x86-regalloc back end ({len(k.code)} bytes of emitted code), kernel(a, b, c, n, nthreads = n), one thread"
        run = lambda: k(a, b_, c, n, n)
    except OSError as e:
        lib = load_oracle()
        how = f"the oracle's C loop (x86 JIT unavailable: {e})"
        run = lambda: lib.orc_vadd_i32(vp(a), vp(b_), vp(c), ctypes.c_int32(n), ctypes.c_int64(n))
    best = float("inf")
    for _ in range(20):
        t0 = time.perf_counter()
        run()
        best = min(best, time.perf_counter() - t0)
    ok = want_sha is None or hashlib.sha256(c.view(np.uint8)).hexdigest() == want_sha
    return {"value": 12.0 * n / best / 1e9, "unit": "GB/s", "cores": 1, "kind": "port", "ok": ok,
            "sample": f"best of 20 passes over the configured {n} elements; {how}"}


def cpu_chain(x: np.ndarray):
    """The helper chain through the oracle's C restatement (32 real, non-inlined calls per element): the
    register-allocating back end refuses `call` (crates/basalt-x86/src/regalloc.rs:197-201), so the
    reference itself can run this workload on its stack-everything oracle back end only."""
    lib = load_oracle()
    n = len(x)
    y = np.empty(n, np.uint32)
    t = lib.orc_time_helper_chain(vp(x), vp(y), ctypes.c_int32(n), 2)
    return {"value": 64.0 * n / t / 1e9, "unit": "G int-op/s", "gbs": 8.0 * n / t / 1e9, "cores": 1, "kind": "port",
            "sample": f"best of 2 passes over the first {n} of the 2^26 elements; the oracle's C loop with 32 non-inlined helper calls per element, one thread "
                      "(the reference's register-allocating back end refuses calls; only its oracle back end runs this kernel)"}, y


def cpu_matmul(kind: str, full: int):
    """The faithful one-thread scalar loop at 512^3 and 1024^3 and the cubic extrapolation to the full size."""
    lib = load_oracle()
    from basalt_b200 import workloads as w
    out = {}
    for m in (512, 1024):
        if kind == "sgemm":
            A = w.f32_pm1(w.SEEDS["sgemm_f32"], m * m); B = w.f32_pm1(w.SEEDS["sgemm_f32"] + 1, m * m); C = np.empty(m * m, np.float32)
            t = lib.orc_time_sgemm_scalar(vp(A), vp(B), vp(C), m, m, m)
        else:
            A = w.f16_normal01(w.SEEDS["matmul_f16"], m * m); B = w.f16_normal01(w.SEEDS["matmul_f16"] + 1, m * m); C = np.empty(m * m, np.float16)
            t = lib.orc_time_matmul_f16_scalar(vp(A.view(np.uint16)), vp(B.view(np.uint16)), vp(C.view(np.uint16)), m, m, m)
        out[m] = t
    gflops_1024 = 2.0 * 1024**3 / out[1024] / 1e9
    extrap_s = out[1024] * (full / 1024.0) ** 3
    return {"value": gflops_1024 / 1e3, "unit": "TFLOP/s", "cores": 1, "kind": "port", "seconds_512": out[512], "seconds_1024": out[1024],
            "extrapolated_seconds_full_size": extrap_s,
            "sample": f"the oracle's one-thread scalar loop (unfused multiply and add, ascending k) timed at 512^3 and 1024^3; value = the 1024^3 rate; "
                      f"{full}^3 would take about {extrap_s:.0f} s by cubic extrapolation (labelled, not measured)"}


def reference_arm(args):
    """The reference's CPU launch path for this workload: one native thread looping over the
    elements (crates/basalt-x86/src/regalloc.rs:413-500), restated in oracle/x86_regalloc.cpp."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from basalt_b200 import workloads as w
    n = N_MAX
    x = w.u32(w.SEEDS["max_i32"], n).view(np.int32)
    how, c_gbs = "", None
    for _ in range(args.warmup):
        cpu_max(x, 1)
    steps = max(1, min(args.steps, 20))      # each step is one full pass (a fraction of a second): bounded
    times = []
    for _ in range(steps):
        t, _r, how, c_gbs = cpu_max(x, 1)
        times.append(t)
    ms = 1e3 * sum(times) / len(times)
    value = 4.0 * n / (ms * 1e-3) / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "i32", "data": "synthetic",
            "config": headline_config(n, max(1, args.gpus)),
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": 1, "kind": "port", "c_loop_gbs": c_gbs,
                             "sample": f"{steps} full passes over 2^28 int32 on rank 0's host core (the other ranks do no work); {how}; the reference's CPU launch path is single-threaded by construction"},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit_line(line)


# ------------------------------------------------------------------------------------------------
# Device side
# ------------------------------------------------------------------------------------------------
class Env:
    """What every configuration's section needs: runtime context, rank group, stream, peaks."""

    def __init__(self, torch, ctx, group, comm, peers, stream, peaks, args):
        import basalt_b200 as b
        from basalt_b200 import kernels, kernels_bir as kb, kernels_cu as kc, kernels_triton as kt, workloads as w
        self.torch, self.ctx, self.group, self.comm, self.peers, self.stream, self.peaks, self.args = torch, ctx, group, comm, peers, stream, peaks, args
        self.b, self.kernels, self.kb, self.kc, self.kt, self.w = b, kernels, kb, kc, kt, w
        self.rank, self.world = group.rank, group.world
        self.launches = 0
        with open(os.path.join(ROOT, "tests", "golden", "golden.json")) as f:
            self.golden = json.load(f)["cases"]

    def dp(self, t):
        return self.b.ptr(t.data_ptr())

    def emitted(self, src: str, name: str):
        return self.ctx.load_module(self.b.Ptx().emit(src).text).get_function(name)

    def fill(self, kind: str, seed: int, n: int, dtype, start: int = 0):
        """A device tensor holding draws start..start+n-1 of the seeded stream (workloads.py's bytes)."""
        t = self.torch.empty(n, dtype=dtype, device="cuda")
        self.kernels.fill(kind, seed, n, t.data_ptr(), start=start, stream=self.stream)
        return t

    def timed(self, fn, reps: int, warm: int = 3) -> float:
        """ms per call: CUDA events on the launching stream around `reps` back-to-back calls; at N > 1 a
        barrier on both sides and the maximum over ranks."""
        torch = self.torch
        for _ in range(warm):
            fn()
        self.group.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        self.group.barrier()
        self.launches += reps
        return self.group.max_float(e0.elapsed_time(e1)) / reps

    def graphed(self, launch, reps: int) -> float:
        """ms per launch with `reps` launches captured into one CUDA graph (removes host launch latency)."""
        torch = self.torch
        side = torch.cuda.Stream()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            launch(side.cuda_stream, 0)
            side.synchronize()
            with torch.cuda.graph(g, stream=side):
                for i in range(reps):
                    launch(side.cuda_stream, i)
        return self.timed(g.replay, 10) / reps

    def host_copy(self, t, pinned: bool = True) -> np.ndarray:
        """The tensor's bytes in host memory (page-locked through the runtime, or ordinary pageable)."""
        np_dtype = {self.torch.int32: np.int32, self.torch.float32: np.float32, self.torch.float16: np.float16, self.torch.uint8: np.uint8}[t.dtype]
        if pinned:
            h = self.ctx.pinned_array(tuple(t.shape), np_dtype)
            h[...] = t.cpu().numpy()
            return h
        return t.cpu().numpy().copy()

    def all_true(self, ok: bool) -> bool:
        """`ok` on every rank."""
        return self.group.max_i32_host(0 if ok else 1) == 0


def sha_of(t) -> str:
    return hashlib.sha256(t.cpu().numpy().view(np.uint8)).hexdigest()


def rel_fro(a, b_) -> float:
    a = np.asarray(a, np.float64); b_ = np.asarray(b_, np.float64)
    return float(np.linalg.norm(a - b_) / max(np.linalg.norm(b_), 1e-300))


def e2e_entry(value, unit, h2d, d2h, ms, api, extra=None):
    out = {"value": value, "unit": unit, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "ms_per_step": ms, "api": api}
    if extra:
        out.update(extra)
    return out


def host_timed(fn, steps: int) -> float:
    fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    return (time.perf_counter() - t0) * 1e3 / steps


def best_and_sustained(env: Env, fn, flops: float, seconds: float = 2.0, flop_per_clock_per_sm: float = 8192.0) -> dict:
    """The two regimes a matmul peak is quoted in: best of 10 single launches (burst), and back-to-back
    launches for `seconds` with the SM clock and the board power sampled beside them (a 1 kW part settles
    well below its maximum clock under a dense matmul).  `pipe_util` is the throughput as a fraction of
    what the pipes can issue at the sampled clock: 8192 dense f16 flop per clock per SM on the tensor
    pipes, 256 (128 FFMA) on the FP32 pipes.  `joules_per_launch` = median sampled power x seconds / launches."""
    torch = env.torch
    for _ in range(3):
        fn()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(10)]
    for e0, e1 in ev:
        e0.record(); fn(); e1.record()
    torch.cuda.synchronize()
    best = min(e0.elapsed_time(e1) for e0, e1 in ev)
    sampler = ClockSampler(torch.cuda.current_device())
    time.sleep(0.3)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.time()
    e0.record()
    n = 0
    while time.time() - t_begin < seconds:
        for _ in range(20):
            fn()
        n += 20
        torch.cuda.current_stream().synchronize()
    e1.record()
    e1.synchronize()
    t_end = time.time()
    clk = sampler.stop(t_begin + 0.4, t_end)
    ms_total = e0.elapsed_time(e1)
    tf_sus = flops * n / ms_total / 1e9
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    util = tf_sus * 1e12 / (flop_per_clock_per_sm * sms * clk["sm_mhz"] * 1e6) if clk.get("sm_mhz") else None
    joules = clk["power_w_median"] * ms_total * 1e-3 / n if clk.get("power_w_median") else None
    env.launches += n + 13
    return {"tflops_best_of_10": flops / best / 1e9, "tflops_sustained": tf_sus, "sustained_sm_mhz": clk.get("sm_mhz"),
            "sustained_power_w_max": clk.get("power_w_max"), "sustained_power_w_median": clk.get("power_w_median"), "joules_per_launch": joules,
            "ms_x_mhz": (ms_total / n) * clk["sm_mhz"] if clk.get("sm_mhz") else None,
            "sustained_reasons": clk.get("reasons"), "pipe_util_at_sampled_clock": util}


def traffic_from_profile(name: str, units: float):
    """DRAM bytes per launch from the ncu capture kept under profiles/: `profiles/traffic.json` holds, per kernel,
    the bytes dram__bytes_read.sum + dram__bytes_write.sum reported per algorithmic unit (element or flop) on the
    captured case and a constant part; traffic grows in proportion to the units, so it is scaled to this launch."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            t = json.load(f)[name]
        return t["bytes_per_unit"] * units + t.get("constant_bytes", 0.0), t["source"]
    except Exception:
        return None, None


# ---- config 1: vadd_i32 ---------------------------------------------------------------------------
def cfg_vadd(env: Env) -> dict:
    torch, b, kernels, kb, w = env.torch, env.b, env.kernels, env.kb, env.w
    peak = env.peaks["hbm_gbs"]
    out = {"workload": "vadd_i32: c[i] = a[i] + b[i] (wrapping int32), N = 2^20, a and b uniform in [-2^30, 2^30) from the seeded generator; block 256, grid N/256 (the runtime coarsens the launch)",
           "unit": "GB/s", "algorithmic_bytes_per_element": 12}
    fn = env.emitted(kb.load("vadd_i32"), "vadd_i32")
    n = 1 << 20
    if env.world == 1:
        # the configured size against HBM: rotate over 16 buffer triples (201 MB in all, larger than the 126 MB L2),
        # so that every launch reads and writes memory the cache no longer holds
        triples = 16
        A = [env.fill("i32_pm30", w.SEEDS["vadd_i32"], n, torch.int32) for _ in range(triples)]
        Bs = [env.fill("i32_pm30", w.SEEDS["vadd_i32"] + 1, n, torch.int32) for _ in range(triples)]
        Cs = [torch.full((n,), 0x7fffffff, dtype=torch.int32, device="cuda") for _ in range(triples)]
        binds = [fn.bind(n // 256, 256, 0, [env.dp(A[i]), env.dp(Bs[i]), env.dp(Cs[i]), b.i32(n)], stream=env.stream) for i in range(triples)]
        it = [0]

        def cold():
            binds[it[0] % triples]()
            it[0] += 1
        ms_cold = env.timed(cold, 20 * triples)
        ms_cold_graph = env.graphed(lambda s_, i: binds[i % triples](stream=s_), 4 * triples)
        hand_it = [0]

        def cold_hand():
            i = hand_it[0] % triples
            kernels.vadd_i32(A[i].data_ptr(), Bs[i].data_ptr(), Cs[i].data_ptr(), n, env.stream)
            hand_it[0] += 1
        ms_cold_hand_graph = env.graphed(lambda s_, i: kernels.vadd_i32(A[i % triples].data_ptr(), Bs[i % triples].data_ptr(), Cs[i % triples].data_ptr(), n, s_), 4 * triples)
        ms_warm = env.timed(binds[0], 200)                          # the same triple every time: L2-resident
        ms_warm_graph = env.graphed(lambda s_, i: binds[0](stream=s_), 64)
        ok = sha_of(Cs[triples - 1]) == env.golden["vadd_i32"]["full"]["sha256"]
        out.update({"value": 12.0 * n / ms_cold_graph / 1e6,
                    "how": "N = 2^20 as configured, 16 rotating buffer triples (201 MB > L2), launches captured in one CUDA graph; one launch is about 2 us of HBM time, so "
                           "back-to-back launches from the host are launch-latency bound (cold_back_to_back_gbs)",
                    "cold_back_to_back_gbs": 12.0 * n / ms_cold / 1e6, "handwritten_gbs": 12.0 * n / ms_cold_hand_graph / 1e6,
                    "emitted_over_handwritten": ms_cold_hand_graph / ms_cold_graph,
                    "l2_resident_back_to_back_gbs": 12.0 * n / ms_warm / 1e6, "l2_resident_graph_gbs": 12.0 * n / ms_warm_graph / 1e6,
                    "roofline": {"bound": "hbm", "achieved": 12.0 * n / ms_cold_graph / 1e6, "peak": peak, "unit": "GB/s", "frac": 12.0 * n / ms_cold_graph / 1e6 / peak,
                                 "peak_source": env.peaks["source"], "kernel": "vadd_i32__coarse (emitted)", "kernel_ms": ms_cold_graph, "algorithmic_bytes_per_launch": 12 * n,
                                 "traffic": None, "note": "one launch moves 12.6 MB in about 2 us: the launch ramp, not the stream, is what keeps it below the 2^28 figure"}})
        # end to end at the configured size: host buffers through the reference's CPU launch ABI
        ha, hb = env.host_copy(A[0]), env.host_copy(Bs[0])
        ha.flags.writeable = False; hb.flags.writeable = False
        hc = env.ctx.pinned_array((n,), np.int32)
        ms_e2e = host_timed(lambda: env.ctx.cpu_launch(fn, [ha, hb, hc, b.i32(n)], nthreads=n, block=256), 20)
        ok = ok and hashlib.sha256(hc.view(np.uint8)).hexdigest() == env.golden["vadd_i32"]["full"]["sha256"]
        pa, pb, pc = np.array(ha), np.array(hb), np.empty(n, np.int32)
        pa.flags.writeable = False; pb.flags.writeable = False
        ms_page = host_timed(lambda: env.ctx.cpu_launch(fn, [pa, pb, pc, b.i32(n)], nthreads=n, block=256), 20)
        out["e2e"] = e2e_entry(12.0 * n / ms_e2e / 1e6, "GB/s", 12 * n, 4 * n, ms_e2e, "basalt_rt_cpu_launch (a, b, c as host pointers, n, then nthreads); pinned host buffers",
                               {"pageable_value": 12.0 * n / ms_page / 1e6, "pageable_ms_per_step": ms_page,
                                "note": "the output buffer is uploaded too (the kernel may leave part of it untouched), so 12 MB go up and 4 MB come back per step"})
        if not env.args.no_e2e:
            out["cpu_baseline"] = cpu_vadd(np.array(ha), np.array(hb), env.golden["vadd_i32"]["full"]["sha256"])
            ok = ok and out["cpu_baseline"].pop("ok")
        out["parity"] = ok
        out["parity_how"] = "SHA-256 of the device result (device-resident and end-to-end) and of the CPU baseline's result against tests/golden/golden.json (the oracle's bytes)"
        del A, Bs, Cs
    # the same kernel against HBM at 2^28 elements in all (3 GiB of traffic), contiguous shards at N > 1, no collective
    total = 1 << 28
    lo, hi = env.group.shard(total, 4)
    nl = hi - lo
    a = env.fill("i32_pm30", w.SEEDS["vadd_i32"], nl, torch.int32, start=lo); bb = env.fill("i32_pm30", w.SEEDS["vadd_i32"] + 1, nl, torch.int32, start=lo)
    c = torch.empty_like(a)
    go = fn.bind((nl + 255) // 256, 256, 0, [env.dp(a), env.dp(bb), env.dp(c), b.i32(nl)], stream=env.stream)
    ms_e = env.timed(go, 30)
    ok_big = bool(torch.equal(c, a + bb))
    ms_h = env.timed(lambda: kernels.vadd_i32(a.data_ptr(), bb.data_ptr(), c.data_ptr(), nl, env.stream), 30)
    big = {"elements_total": total, "elements_per_gpu": nl, "emitted_gbs": 12.0 * total / ms_e / 1e6, "handwritten_gbs": 12.0 * total / ms_h / 1e6,
           "ms": ms_e, "frac_of_hbm_peak_per_gpu": 12.0 * nl / ms_e / 1e6 / peak, "parity": env.all_true(ok_big),
           "parity_how": "device result equals the wrapping sum of the two inputs, element for element",
           "scaling": "strong (2^28 elements split into contiguous shards, no collective)" if env.world > 1 else None}
    traffic, tsrc = traffic_from_profile("vadd_i32", nl)
    big["roofline"] = {"bound": "hbm", "achieved": 12.0 * nl / ms_e / 1e6, "peak": peak, "unit": "GB/s", "frac": 12.0 * nl / ms_e / 1e6 / peak, "kernel_ms": ms_e,
                       "algorithmic_bytes_per_launch": 12 * nl, "traffic": traffic, "traffic_source": tsrc, "peak_source": env.peaks["source"]}
    out["n2^28_hbm"] = big
    if env.world > 1:
        out.update({"value": big["emitted_gbs"], "parity": big["parity"], "parity_how": big["parity_how"], "roofline": big["roofline"],
                    "how": "2^28 elements in all, contiguous shards, no collective (the configured 2^20 is measured in the N = 1 run)"})
    if env.world == 1:
        try:   # the same workload from its CUDA-C and Triton sources (2^26 elements per operand)
            n2 = 1 << 26
            fc = env.emitted(b.compile_cuda(env.kc.load("vadd_i32")), "vadd_i32")
            ms_c = env.timed(fc.bind((n2 + 255) // 256, 256, 0, [env.dp(a), env.dp(bb), env.dp(c), b.i32(n2)], stream=env.stream), 20)
            ok_c = bool(torch.equal(c[:n2], (a + bb)[:n2]))
            c.zero_()
            ft = env.emitted(env.kt.vadd_i32(), "vadd_i32")
            block = 4096
            ms_t = env.timed(ft.bind((n2 + block - 1) // block, 256, 0, [env.dp(a), env.dp(bb), env.dp(c), b.i64(n2), b.i64(block)], stream=env.stream), 20)
            out["n2^26_other_sources"] = {"from_cuda_c_gbs": 12.0 * n2 / ms_c / 1e6, "from_triton_gbs": 12.0 * n2 / ms_t / 1e6,
                                          "parity": ok_c and bool(torch.equal(c[:n2], (a + bb)[:n2]))}
        except Exception as e:   # noqa: BLE001 - reported, not hidden
            out["other_sources_error"] = str(e)[:200]
    return out


# ---- config 3: helper chain -----------------------------------------------------------------------
def cfg_chain(env: Env) -> dict:
    torch, b, kernels, kb, w = env.torch, env.b, env.kernels, env.kb, env.w
    total = 1 << 26
    lo, hi = env.group.shard(total, 4)
    n = hi - lo
    out = {"workload": "helper chain: 32 chained __device__ helper calls x = x*x + 2654435761*j (mod 2^32) per element, N = 2^26 uint32 uniform from the seeded generator, block 256"
                       + ("" if env.world == 1 else f", contiguous shards x{env.world}, no collective"),
           "unit": "G int-op/s", "int_ops_per_element": 64, "algorithmic_bytes_per_element": 8}
    x = env.fill("u32", w.SEEDS["helper_chain"], n, torch.int32, start=lo); y = torch.empty_like(x)
    fn = env.emitted(kb.helper_chain(), "helper_chain")
    go = fn.bind((n + 255) // 256, 256, 0, [env.dp(x), env.dp(y), b.i32(n)], stream=env.stream)
    ms_e = env.timed(go, 30)
    y_emitted_sha = sha_of(y) if env.world == 1 else None
    ms_h = env.timed(lambda: kernels.helper_chain_u32(x.data_ptr(), y.data_ptr(), n, env.stream), 30)
    scratch = torch.empty(1 << 22, dtype=torch.int32, device="cuda")
    imads = [0]

    def peak_fn():
        imads[0] = kernels.imad_peak(scratch.data_ptr(), scratch.numel(), 2000, env.stream)
    ms_p = env.timed(peak_fn, 5)
    int_peak = 2.0 * imads[0] / ms_p / 1e6                     # G int-op/s of one GPU, measured by a pure multiply-add kernel
    gops = 64.0 * total / ms_e / 1e6
    out.update({"value": gops, "handwritten_gops": 64.0 * total / ms_h / 1e6, "emitted_over_handwritten": ms_h / ms_e, "emitted_gbs": 8.0 * total / ms_e / 1e6,
                "scaling": "strong (2^26 elements split)" if env.world > 1 else None,
                "roofline": {"bound": "int32 pipe", "achieved": 64.0 * n / ms_e / 1e6, "peak": int_peak, "unit": "G int-op/s", "frac": 64.0 * n / ms_e / 1e6 / int_peak,
                             "peak_source": "measured live: basalt_k_imad_peak, one wave of independent multiply-adds", "kernel": "helper_chain__coarse (emitted)", "kernel_ms": ms_e,
                             "algorithmic_ops_per_launch": 64 * n, "hbm_frac": 8.0 * n / ms_e / 1e6 / env.peaks["hbm_gbs"], "traffic": traffic_from_profile("helper_chain", n)[0],
                             "traffic_source": traffic_from_profile("helper_chain", n)[1]}})
    if env.world == 1:
        ok = y_emitted_sha == env.golden["helper_chain"]["full"]["sha256"] and sha_of(y) == env.golden["helper_chain"]["full"]["sha256"]
        hx = env.host_copy(x).view(np.uint32)
        hx.flags.writeable = False
        hy = env.ctx.pinned_array((n,), np.uint32)
        ms_e2e = host_timed(lambda: env.ctx.cpu_launch(fn, [hx, hy, b.i32(n)], nthreads=n, block=256), 3)
        ok = ok and hashlib.sha256(hy.view(np.uint8)).hexdigest() == env.golden["helper_chain"]["full"]["sha256"]
        px, py = np.array(hx), np.empty(n, np.uint32)
        px.flags.writeable = False
        ms_page = host_timed(lambda: env.ctx.cpu_launch(fn, [px, py, b.i32(n)], nthreads=n, block=256), 2)
        out["e2e"] = e2e_entry(64.0 * n / ms_e2e / 1e6, "G int-op/s", 8 * n, 4 * n, ms_e2e, "basalt_rt_cpu_launch (in, out as host pointers, n, then nthreads); pinned host buffers",
                               {"pageable_value": 64.0 * n / ms_page / 1e6, "pageable_ms_per_step": ms_page})
        if not env.args.no_e2e:
            sample = 1 << 22
            out["cpu_baseline"], y_cpu = cpu_chain(np.array(hx[:sample]))
            ok = ok and np.array_equal(y_cpu, np.array(hy[:sample]))
        out["parity"] = ok
        out["parity_how"] = "SHA-256 of the emitted and hand-written kernels' results and of the end-to-end result against tests/golden/golden.json; the CPU sample against the same elements of the device result"
    else:
        # every rank checks its shard against the hand-written kernel's result on the same shard
        y2 = torch.empty_like(y)
        go()
        kernels.helper_chain_u32(x.data_ptr(), y2.data_ptr(), n, env.stream)
        torch.cuda.synchronize()
        out["parity"] = env.all_true(bool(torch.equal(y, y2)))
        out["parity_how"] = "emitted and hand-written kernels agree on every rank's shard (golden hashes are checked in the N = 1 run)"
    return out


# ---- configs 4 and 5: the matmuls -----------------------------------------------------------------
class MatmulCheck:
    """Checks a gathered result on this rank: Freivalds' identity C v = A (B v) over all rows, on the device in
    float64, and sampled rows (two from every rank's shard) against the CPU oracle."""

    def __init__(self, env: Env, kind: str, M: int, N: int, K: int, A_full, B_):
        torch = env.torch
        self.env, self.kind, self.M, self.N, self.K = env, kind, M, N, K
        self.tol = SGEMM_TOL if kind == "sgemm" else F16_TOL
        g = torch.Generator(device="cuda"); g.manual_seed(4)
        self.v = torch.randn(N, device="cuda", dtype=torch.float64, generator=g)
        bv = torch.mv(B_.double(), self.v) if B_.numel() <= (1 << 26) else torch.cat([torch.mv(B_[i:i + 1024].double(), self.v) for i in range(0, K, 1024)])
        self.rhs = torch.cat([torch.mv(A_full[i:i + 1024].double(), bv) for i in range(0, M, 1024)])
        rows_per = M // env.world
        self.rows = sorted({r * rows_per + off for r in range(env.world) for off in (0, rows_per - 1)} | {M // 2 + 1})
        hB = B_.cpu().numpy()
        lib = load_oracle()
        self.want = {}
        for r in self.rows:
            a_row = np.ascontiguousarray(A_full[r:r + 1].cpu().numpy())
            if kind == "sgemm":
                o = np.empty((1, N), np.float32)
                lib.orc_sgemm_f32_rows(vp(a_row), vp(hB), vp(o), 1, N, K, 0, 1)
            else:
                o = np.empty((1, N), np.float16)
                lib.orc_matmul_f16_rows(vp(a_row), vp(hB), vp(o), 1, N, K, 0, 0, 1)
            self.want[r] = o[0]

    def __call__(self, C_full) -> dict:
        torch = self.env.torch
        lhs = torch.cat([torch.mv(C_full[i:i + 1024].double(), self.v) for i in range(0, self.M, 1024)])
        frei = float(((lhs - self.rhs).norm() / self.rhs.norm()).item())
        worst = 0.0
        for r in self.rows:
            worst = max(worst, rel_fro(C_full[r].cpu().numpy(), self.want[r]))
        finite = bool(torch.isfinite(C_full).all().item())
        ok = finite and frei <= self.tol and worst <= self.tol
        return {"parity": self.env.all_true(ok), "freivalds_rel": frei, "sampled_rows_rel_max": worst, "rows_checked": len(self.rows)}


def matmul_inputs(env: Env, kind: str, M: int, N: int, K: int):
    torch, w = env.torch, env.w
    if kind == "sgemm":
        A = env.fill("f32_pm1", w.SEEDS["sgemm_f32"], M * K, torch.float32).view(M, K); B_ = env.fill("f32_pm1", w.SEEDS["sgemm_f32"] + 1, K * N, torch.float32).view(K, N)
    else:
        A = env.fill("f16_normal01", w.SEEDS["matmul_f16"], M * K, torch.float16).view(M, K); B_ = env.fill("f16_normal01", w.SEEDS["matmul_f16"] + 1, K * N, torch.float16).view(K, N)
    return A, B_


def matmul_e2e(env: Env, fn, grid, block, A, B_, C, flops: float, check: MatmulCheck) -> dict:
    """End to end through the runtime's own calls with HOST buffers: DeviceBuffer::copy_from_host of A and B,
    CudaFunction::launch, DeviceBuffer::copy_to_host of C (the reference's GPU path, crates/basalt-runtime/tests/
    ptx_gpu_proof.rs:138-200), pinned and pageable."""
    b, ctx = env.b, env.ctx
    res = {}
    nbytes = A.numel() * A.element_size()
    dA, dB, dC = ctx.alloc(nbytes), ctx.alloc(B_.numel() * B_.element_size()), ctx.alloc(C.numel() * C.element_size())
    ok = True
    for label, pinned in (("pinned", True), ("pageable", False)):
        hA, hB = env.host_copy(A, pinned), env.host_copy(B_, pinned)
        hC = ctx.pinned_array(tuple(C.shape), hA.dtype) if pinned else np.empty(tuple(C.shape), hA.dtype)

        def step():
            dA.copy_from_host(hA); dB.copy_from_host(hB)
            fn.launch(grid, block, 0, [dA, dB, dC])          # synchronous, like the reference's launch
            dC.copy_to_host(hC)
        ms = host_timed(step, 3)
        res[label] = ms
        got = env.torch.from_numpy(np.array(hC)).cuda()
        ok = ok and check(got)["parity"]
    dA.free(); dB.free(); dC.free()
    out = e2e_entry(flops / res["pinned"] / 1e9, "TFLOP/s", 2 * nbytes, C.numel() * C.element_size(), res["pinned"],
                    "DeviceBuffer::copy_from_host (A, B), CudaFunction::launch, DeviceBuffer::copy_to_host (C); pinned host buffers",
                    {"pageable_value": flops / res["pageable"] / 1e9, "pageable_ms_per_step": res["pageable"], "parity": ok})
    return out


def sharded_gather_variants(env: Env, kind: str, M: int, N: int, K: int, A_full, B_, check: MatmulCheck, compute_1gpu_ms) -> dict:
    """The row-sharded matmul whose result every rank wants whole (strong scaling): each rank computes M/world rows;
    the variants differ in how the rows reach the other ranks.  Every variant's gathered result is checked on
    every rank (Freivalds + sampled oracle rows) and carries its own `parity`."""
    torch, b, kb, ctx, group = env.torch, env.b, env.kb, env.ctx, env.group
    esz = 4 if kind == "sgemm" else 2
    dt = torch.float32 if kind == "sgemm" else torch.float16
    world, rank = env.world, env.rank
    r0, r1 = group.shard(M, 256)
    Ml = r1 - r0
    fl = 2.0 * M * N * K
    out = {"rows_per_gpu": Ml, "scaling": f"strong ({M}x{N}x{K} split by rows, B replicated, the whole result on every GPU)",
           "gather_bytes_in_per_gpu": (M - Ml) * N * esz}
    # measured link floor for this gather on this box: every rank's copy engines push its shard to every peer at once
    Al = A_full[r0:r1]
    Cbuf = ctx.alloc(M * N * esz)
    ptrs = group.map_peers(ctx, Cbuf)
    bg = group.peers(ctx)
    flag = torch.zeros(2, dtype=torch.int32, device="cuda")
    Cfull = torch.empty(M, N, dtype=dt, device="cuda")

    def barrier_kernel():
        bg.allreduce_max_i32(flag.data_ptr(), flag.data_ptr() + 4, env.stream)

    def snapshot(ptr=None):
        torch.cuda.synchronize(); group.barrier()
        ctx.copy_device_async(Cfull.data_ptr(), ptr or Cbuf.device_ptr(), M * N * esz, env.stream)
        torch.cuda.synchronize()
        return Cfull

    def clear(ptr=None):
        torch.cuda.synchronize(); group.barrier()
        Cfull.fill_(float("nan"))
        ctx.copy_device_async(ptr or Cbuf.device_ptr(), Cfull.data_ptr(), M * N * esz, env.stream)
        torch.cuda.synchronize(); group.barrier()

    mine = Cbuf.device_ptr() + r0 * N * esz
    others = [ptrs[r] + r0 * N * esz for r in group.peer_order()]      # rank + 1 first: every step of the gather is a permutation
    if kind == "sgemm":
        fn = env.emitted(kb.sgemm_cta128(Ml, N, K), "sgemm_f32"); block = 256
    else:
        fn = env.emitted(kb.matmul_f16(Ml, N, K), "matmul_kernel"); block = 128
    grid = (N // 128, Ml // 128)
    prm = [env.dp(Al), env.dp(B_), b.ptr(mine)]
    go = fn.bind(grid, block, 0, prm, stream=env.stream)
    go_gather = fn.bind_gather(grid, block, 0, prm, others, stream=env.stream)
    variants = {}

    def run_variant(name, step, reps=10, ptr=None):
        clear(ptr)
        ms = env.timed(step, reps)
        res = {"ms": ms, "tflops_total": fl / ms / 1e9}
        res.update(check(snapshot(ptr)))
        if compute_1gpu_ms:
            res["fraction_of_linear"] = compute_1gpu_ms / world / ms
        variants[name] = res

    ms_compute = env.timed(go, 10)
    out["compute_only_ms"] = ms_compute
    out["compute_only_fraction_of_linear"] = compute_1gpu_ms / world / ms_compute if compute_1gpu_ms else None

    # copy-engine floor: the shard pushed to every peer by cuMemcpyDtoDAsync, nothing else running
    push_streams = [ctx.create_stream() for _ in others]
    push_start, push_done = ctx.create_event(), [ctx.create_event() for _ in others]

    def push_only():      # every peer's copy on its own stream (its own copy engine and links), gathered back on the timing stream
        ctx.record(push_start, env.stream)
        for p_, s_, e_ in zip(others, push_streams, push_done):
            ctx.stream_wait_event(s_, push_start)
            ctx.copy_device_async(p_, mine, Ml * N * esz, s_)
            ctx.record(e_, s_)
            ctx.stream_wait_event(env.stream, e_)
        barrier_kernel()
    ms_push = env.timed(push_only, 10)
    torch.cuda.synchronize()
    for s_ in push_streams:
        ctx.destroy_stream(s_)
    for e_ in push_done + [push_start]:
        ctx.destroy_event(e_)
    out["copy_engine_push_only_ms"] = ms_push
    out["copy_engine_push_GBs_out_per_gpu"] = (world - 1) * Ml * N * esz / ms_push / 1e6

    def nccl_step():
        go()
        env.comm.allgather(mine, Cbuf.device_ptr(), Ml * N * esz, env.stream)
    run_variant("emitted_then_ncclAllGather", nccl_step)

    def fused_emitted():
        go_gather()
        barrier_kernel()
    run_variant("emitted_fused_gather", fused_emitted)
    out["emitted_fused_gather_nvlink_GBs_out_per_gpu"] = (world - 1) * Ml * N * esz / variants["emitted_fused_gather"]["ms"] / 1e6

    if kind == "sgemm":
        # rounds of stream units under the gathering launch (two by default): more rounds hide more of the gather
        # behind compute and cost more partial sums
        for rounds in (1, 3):
            fn.tune("tail_rounds", rounds)
            run_variant(f"emitted_fused_gather_rounds{rounds}", fused_emitted, reps=5)
        fn.tune("tail_rounds", 0)

    # the same kernel sending every tile once through an NVLink multicast mapping of the result (NVLS): the switch
    # replicates it, so Ml * N * esz bytes leave each GPU instead of (world - 1) times that
    from basalt_b200 import sharding as _sh
    mcr = None if env.args.no_multimem else _sh.MulticastResult.open(group, M * N * esz, torch.cuda.current_device())
    if env.args.no_multimem:
        out["emitted_fused_gather_multimem"] = {"unavailable": "switched off (--no-multimem)"}
    elif mcr is None:
        out["emitted_fused_gather_multimem"] = {"unavailable": _sh.MulticastResult.why_not}
    else:
        try:
            mine_mc = mcr.local_ptr + r0 * N * esz
            go_mc = fn.bind_gather_multicast(grid, block, 0, [env.dp(Al), env.dp(B_), b.ptr(mine_mc)], mcr.multicast_ptr + r0 * N * esz, stream=env.stream)

            def fused_multimem():
                go_mc()
                barrier_kernel()
            run_variant("emitted_fused_gather_multimem", fused_multimem, ptr=mcr.local_ptr)
            variants["emitted_fused_gather_multimem"]["nvlink_GBs_in_per_gpu"] = (world - 1) * Ml * N * esz / variants["emitted_fused_gather_multimem"]["ms"] / 1e6
        finally:
            mcr.close()          # collectively, whatever happened: no rank leaves while its memory is bound

    if kind == "matmul":
        st2 = torch.zeros(1, dtype=torch.int32, device="cuda")

        def fused_hand():
            env.kernels.matmul_f16_allgather(Al.data_ptr(), B_.data_ptr(), mine, Ml, N, K, others, status=st2.data_ptr(), stream=env.stream)
            barrier_kernel()
        run_variant("handwritten_fused_gather", fused_hand)
        out["status"] = fn.status() or int(st2.item())
        # copy engines push finished row bands while the next band computes (basalt_b200.sharding.PushGather)
        from basalt_b200 import sharding
        best = None
        for bands in (1, 2, 4):
            if (Ml // 128) % bands or (Ml // bands) % 256:
                continue
            rows_b = Ml // bands
            fb = env.emitted(kb.matmul_f16(rows_b, N, K), "matmul_kernel")
            pg = sharding.PushGather(ctx, group, bg, ptrs, N * esz, r0, Ml, bands)
            launches = [fb.bind((N // 128, rows_b // 128), 128, 0, [b.ptr(Al.data_ptr() + k * rows_b * K * esz), env.dp(B_), b.ptr(mine + k * rows_b * N * esz)]) for k in range(bands)]
            run_variant(f"emitted_pushed_gather_bands{bands}", lambda launches=launches, pg=pg: pg.run(lambda k, s: launches[k](stream=s), env.stream))
            torch.cuda.synchronize()
            pg.close()
            ms = variants[f"emitted_pushed_gather_bands{bands}"]["ms"]
            best = ms if best is None or ms < best else best
        if world == 2 and M == 8192:
            # The 8-GPU traffic between two GPUs: a 1024-row shard (what a rank owns at N = 8) whose every tile is stored
            # seven times into the peer's buffer, so that each GPU sends and receives the 112 MiB it would at N = 8.
            # Timing only (the seven copies land in row blocks that do not belong to either rank's real shard).
            rows8 = M // 8
            f8 = env.emitted(kb.matmul_f16(rows8, N, K), "matmul_kernel")
            prm8 = [env.dp(A_full[rank * rows8:(rank + 1) * rows8]), env.dp(B_), b.ptr(Cbuf.device_ptr() + rank * rows8 * N * esz)]
            blocks8 = [ptrs[1 - rank] + ((rank * 7 + i) % 8) * rows8 * N * esz for i in range(7)]
            go8 = f8.bind((N // 128, rows8 // 128), 128, 0, prm8, stream=env.stream)
            go8_gather = f8.bind_gather((N // 128, rows8 // 128), 128, 0, prm8, blocks8, stream=env.stream)

            def fused8():
                go8_gather()
                barrier_kernel()

            def push8():
                for p_ in blocks8:
                    ctx.copy_device_async(p_, prm8[2].value, rows8 * N * esz, env.stream)
                barrier_kernel()
            out["eight_gpu_volume_between_two_gpus"] = {"rows": rows8, "copies_to_the_peer": 7, "bytes_out_per_gpu": 7 * rows8 * N * esz,
                                                        "compute_only_ms": env.timed(go8, 10), "emitted_fused_gather_ms": env.timed(fused8, 10),
                                                        "copy_engine_push_only_ms": env.timed(push8, 10)}
            e8 = out["eight_gpu_volume_between_two_gpus"]
            e8["copy_engine_GBs_per_direction"] = e8["bytes_out_per_gpu"] / e8["copy_engine_push_only_ms"] / 1e6
            e8["fused_GBs_per_direction_after_first_wave"] = e8["bytes_out_per_gpu"] / max(1e-9, e8["emitted_fused_gather_ms"] - e8["compute_only_ms"] / 2) / 1e6
    else:
        out["status"] = 0
    out["variants"] = variants
    out["parity"] = all(v["parity"] for v in variants.values())
    link = env.peaks.get("nvlink_gbs", 770.0)
    out["link_floor_ms_at_770GBs"] = (M - Ml) * N * esz / link / 1e6
    bad = bg.status()
    if bad:
        out["exchange_timeouts"] = bad
    group.barrier()
    for r, p_ in enumerate(ptrs):
        if r != rank:
            ctx.ipc_close(p_)
    group.barrier()
    bg.destroy()
    Cbuf.free()
    return out


def cfg_sgemm(env: Env) -> dict:
    torch, b, kernels, kb = env.torch, env.b, env.kernels, env.kb
    M = N = K = 4096
    fl = 2.0 * M * N * K
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    fp32_peak = sms * FP32_LANES_PER_SM * 2 * env.peaks["sm_max_mhz"] * 1e6 / 1e12
    out = {"workload": "SGEMM fp32: C = A B, M = N = K = 4096, row-major, A and B uniform in [-1, 1) from the seeded generator; FFMA only (no TF32); tolerance 1e-4 relative Frobenius",
           "unit": "TFLOP/s", "flop_per_launch": fl}
    A, B_ = matmul_inputs(env, "sgemm", M, N, K)
    check = MatmulCheck(env, "sgemm", M, N, K, A, B_)
    C = torch.full((M, N), float("nan"), device="cuda")
    fn = env.emitted(kb.sgemm_cta128(M, N, K), "sgemm_f32")
    go = fn.bind((N // 128, M // 128), 256, 0, [env.dp(A), env.dp(B_), env.dp(C)], stream=env.stream)
    ms_e = env.timed(go, 5)
    par = check(C)
    C.fill_(float("nan"))
    ms_h = env.timed(lambda: kernels.sgemm_f32(A.data_ptr(), B_.data_ptr(), C.data_ptr(), M, N, K, env.stream), 5)
    par_h = check(C)
    out.update({"value_1gpu": fl / ms_e / 1e9, "handwritten_tflops": fl / ms_h / 1e9, "emitted_over_handwritten": ms_h / ms_e, "parity_1gpu": par, "handwritten_parity": par_h,
                "roofline": {"bound": "fp32 fma pipe", "achieved": fl / ms_e / 1e9, "peak": fp32_peak, "unit": "TFLOP/s", "frac": fl / ms_e / 1e9 / fp32_peak,
                             "peak_source": f"nominal: {sms} SMs x 128 FFMA x 2 flop x {env.peaks['sm_max_mhz']:.0f} MHz (MEASURED_PEAKS.json holds no fp32 figure)",
                             "kernel": "sgemm_f32 (emitted)", "kernel_ms": ms_e, "flop_per_launch": fl, "traffic": traffic_from_profile("sgemm_f32", 3.0 * M * N * 4)[0],
                             "traffic_source": traffic_from_profile("sgemm_f32", 3.0 * M * N * 4)[1]}})
    out["value"] = out["value_1gpu"]
    out["parity"] = par["parity"] and par_h["parity"]
    if env.world == 1:
        try:   # comparator only: the vendor library's fp32 (no TF32) GEMM on the same operands
            was = torch.backends.cuda.matmul.allow_tf32
            torch.backends.cuda.matmul.allow_tf32 = False
            out["cublas_fp32_same_operands_tflops"] = fl / env.timed(lambda: torch.matmul(A, B_, out=C), 5) / 1e9
            torch.backends.cuda.matmul.allow_tf32 = was
        except Exception as e:   # noqa: BLE001
            out["cublas_error"] = str(e)[:200]
        out["emitted_regimes"] = best_and_sustained(env, go, fl, seconds=1.5, flop_per_clock_per_sm=256.0)
        out["e2e"] = matmul_e2e(env, fn, (N // 128, M // 128), 256, A, B_, C, fl, check)
        out["parity"] = out["parity"] and out["e2e"]["parity"]
        if not env.args.no_e2e:
            out["cpu_baseline"] = cpu_matmul("sgemm", M)
    else:
        out["sharded"] = sharded_gather_variants(env, "sgemm", M, N, K, A, B_, check, ms_e)
        best = min(v["ms"] for v in out["sharded"]["variants"].values())
        out["value"] = fl / best / 1e9
        out["parity"] = out["parity"] and out["sharded"]["parity"]
    return out


def cfg_matmul(env: Env) -> dict:
    torch, b, kernels, kb = env.torch, env.b, env.kernels, env.kb
    M = N = K = 8192
    fl = 2.0 * M * N * K
    peak = env.peaks["tf_burst"]
    out = {"workload": "Triton-style fp16 matmul: C = A B, M = N = K = 8192, fp16 inputs N(0,1)*0.1 from the seeded generator, fp32 accumulate, fp16 output; BLOCK 128x128x64 lowered to TMA + tcgen05.mma; tolerance 2e-3 relative",
           "unit": "TFLOP/s", "flop_per_launch": fl}
    A, B_ = matmul_inputs(env, "matmul", M, N, K)
    check = MatmulCheck(env, "matmul", M, N, K, A, B_)
    C = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float16)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    fn = env.emitted(kb.matmul_f16(M, N, K), "matmul_kernel")
    go = fn.bind((N // 128, M // 128), 128, 0, [env.dp(A), env.dp(B_), env.dp(C)], stream=env.stream)
    hand = lambda: kernels.matmul_f16(A.data_ptr(), B_.data_ptr(), C.data_ptr(), M, N, K, False, st.data_ptr(), env.stream)
    if env.world == 1:
        # The kernels are timed INTERLEAVED (four rounds of five launches each, medians reported): under the 1 kW cap
        # whichever kernel runs right after a cooler phase gains about 2 %, so back-to-back blocks per kernel would
        # favour the first one.  The sustained regimes (2 s each) follow afterwards.
        cands = {"emitted": go, "handwritten": hand,
                 "handwritten_one_sm_256": lambda: kernels.matmul_f16_variant(A.data_ptr(), B_.data_ptr(), C.data_ptr(), M, N, K, "one_sm_256", status=st.data_ptr(), stream=env.stream),
                 # comparators only, never on the product path: the vendor library on the SAME operands (the power a dense
                 # matmul draws, and so the clock it settles at, depends on the data) and on the same values in bf16
                 "cublas_f16_same_operands": lambda: torch.matmul(A, B_, out=C)}
        Ab, Bb, Cb = A.bfloat16(), B_.bfloat16(), torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        cands["cublas_bf16_same_values"] = lambda: torch.matmul(Ab, Bb, out=Cb)
        rounds = {k: [] for k in cands}
        for _ in range(4):
            for k, f_ in cands.items():
                rounds[k].append(fl / env.timed(f_, 5) / 1e9)
        med = {k: statistics.median(v) for k, v in rounds.items()}
        ms_e = fl / med["emitted"] / 1e9
        go(); torch.cuda.synchronize()
        par = check(C)
        C.fill_(float("nan")); hand(); torch.cuda.synchronize()
        par_h = check(C)
        out.update({"value": med["emitted"], "handwritten_tflops": med["handwritten"], "handwritten_one_sm_256_tflops": med["handwritten_one_sm_256"],
                    "cublas_f16_same_operands_tflops": med["cublas_f16_same_operands"], "cublas_bf16_same_values_tflops": med["cublas_bf16_same_values"],
                    "how": "medians of 4 interleaved rounds of 5 launches", "status": int(st.item()) or fn.status(),
                    "emitted_over_handwritten": med["emitted"] / med["handwritten"], "emitted_over_cublas_f16_same_operands": med["emitted"] / med["cublas_f16_same_operands"],
                    "emitted_frac_of_nominal_2250": med["emitted"] / 2250.0, "parity_1gpu": par, "handwritten_parity": par_h,
                    "roofline": {"bound": "tensor", "achieved": med["emitted"], "peak": peak, "unit": "TFLOP/s", "frac": med["emitted"] / peak,
                                 "peak_source": env.peaks["source"] + ": cuBLAS bf16 burst (best of 10) of MEASURED_PEAKS.json; the kernel is timed alone in short bursts",
                                 "kernel": "matmul_kernel__pair (emitted)", "kernel_ms": ms_e, "flop_per_launch": fl, "traffic": traffic_from_profile("matmul_f16", 3.0 * M * N * 2)[0],
                                 "traffic_source": traffic_from_profile("matmul_f16", 3.0 * M * N * 2)[1]}})
        out["emitted_regimes"] = best_and_sustained(env, go, fl)
        out["handwritten_regimes"] = best_and_sustained(env, hand, fl)
        out["cublas_f16_same_operands_regimes"] = best_and_sustained(env, cands["cublas_f16_same_operands"], fl)
        s_e, s_c = out["emitted_regimes"], out["cublas_f16_same_operands_regimes"]
        out["sustained_emitted_over_cublas_f16"] = s_e["tflops_sustained"] / s_c["tflops_sustained"]
        if s_e.get("ms_x_mhz") and s_c.get("ms_x_mhz"):
            out["sustained_emitted_over_cublas_f16_clock_matched"] = s_c["ms_x_mhz"] / s_e["ms_x_mhz"]
        out["peaks"] = {"bf16_tflops_burst_best_of_10": peak, "bf16_tflops_sustained": env.peaks["tf_sustained"]}
        out["parity"] = par["parity"] and par_h["parity"]
        del Ab, Bb, Cb
        out["e2e"] = matmul_e2e(env, fn, (N // 128, M // 128), 128, A, B_, C, fl, check)
        out["parity"] = out["parity"] and out["e2e"]["parity"]
        if not env.args.no_e2e:
            out["cpu_baseline"] = cpu_matmul("matmul", M)
    else:
        ms_e = env.timed(go, 10)      # the whole product on every GPU, for the fraction-of-linear column
        par = check(C)
        out.update({"value_1gpu": fl / ms_e / 1e9, "parity_1gpu": par})
        out["sharded"] = sharded_gather_variants(env, "matmul", M, N, K, A, B_, check, ms_e)
        best = min(v["ms"] for v in out["sharded"]["variants"].values())
        out["value"] = fl / best / 1e9
        out["parity"] = par["parity"] and out["sharded"]["parity"]
    return out


def profile_one(args):
    """A few launches of one workload's two kernels on a small case, for ncu captures."""
    import torch

    import basalt_b200 as b
    from basalt_b200 import kernels, kernels_bir as kb
    torch.cuda.set_device(0)
    ctx = b.CudaDriver.load().create_context(0)
    stream = torch.cuda.current_stream().cuda_stream
    dp = lambda t: b.ptr(t.data_ptr())
    reps = max(1, min(args.steps, 5))
    name = args.profile
    if name in ("vadd_i32", "helper_chain", "max_i32"):
        n = args.size or (1 << 26)
        x = torch.randint(-2**30, 2**30, (n,), dtype=torch.int32, device="cuda"); y = torch.randint(-2**30, 2**30, (n,), dtype=torch.int32, device="cuda")
        z = torch.empty_like(x)
        if name == "vadd_i32":
            fn = ctx.load_module(b.Ptx().emit(kb.load("vadd_i32")).text).get_function("vadd_i32")
            em = lambda: fn.launch((n + 255) // 256, 256, 0, [dp(x), dp(y), dp(z), b.i32(n)], stream=stream)
            hw = lambda: kernels.vadd_i32(x.data_ptr(), y.data_ptr(), z.data_ptr(), n, stream)
        elif name == "max_i32":
            fn = ctx.load_module(b.Ptx().emit(kb.load("max_i32")).text).get_function("max_i32")
            em = lambda: fn.launch(fn.streaming_grid(256, n), 256, 0, [dp(x), dp(z), b.i32(n)], stream=stream)
            hw = lambda: kernels.max_i32(x.data_ptr(), n, z.data_ptr(), stream)
        else:
            fn = ctx.load_module(b.Ptx().emit(kb.helper_chain()).text).get_function("helper_chain")
            em = lambda: fn.launch((n + 255) // 256, 256, 0, [dp(x), dp(z), b.i32(n)], stream=stream)
            hw = lambda: kernels.helper_chain_u32(x.data_ptr(), z.data_ptr(), n, stream)
        size = {"elements": n}
    elif name == "sgemm_f32":
        m = args.size or 2048
        A = torch.rand(m, m, device="cuda") * 2 - 1; B = torch.rand(m, m, device="cuda") * 2 - 1; C = torch.empty(m, m, device="cuda")
        fn = ctx.load_module(b.Ptx().emit(kb.sgemm_cta128(m, m, m)).text).get_function("sgemm_f32")
        em = lambda: fn.launch((m // 128, m // 128), 256, 0, [dp(A), dp(B), dp(C)], stream=stream)
        hw = lambda: kernels.sgemm_f32(A.data_ptr(), B.data_ptr(), C.data_ptr(), m, m, m, stream)
        size = {"M=N=K": m}
    else:
        m = args.size or 4096
        A = (torch.randn(m, m, device="cuda") * 0.1).half(); B = (torch.randn(m, m, device="cuda") * 0.1).half(); C = torch.empty(m, m, device="cuda", dtype=torch.float16)
        st = torch.zeros(1, dtype=torch.int32, device="cuda")
        fn = ctx.load_module(b.Ptx().emit(kb.matmul_f16(m, m, m)).text).get_function("matmul_kernel")
        em = lambda: fn.launch((m // 128, m // 128), 128, 0, [dp(A), dp(B), dp(C)], stream=stream)
        hw = lambda: kernels.matmul_f16(A.data_ptr(), B.data_ptr(), C.data_ptr(), m, m, m, False, st.data_ptr(), stream)
        size = {"M=N=K": m}
    if name == "matmul_f16_forms":
        # every form of the hand-written kernel and the emitted entry, CUDA events, medians of 4 interleaved rounds of 5 launches
        forms = {v: (lambda v=v: kernels.matmul_f16_variant(A.data_ptr(), B.data_ptr(), C.data_ptr(), m, m, m, v, status=st.data_ptr(), stream=stream))
                 for v in ("one_sm_256", "pair_direct", "pair_lines", "pair_bulk", "pair_bulk_deep", "pair_lines_narrow")}
        forms["emitted"] = em
        forms["cublas_f16_same_operands"] = lambda: torch.matmul(A, B, out=C)
        rounds = {k: [] for k in forms}
        for _ in range(4):
            for k, f in forms.items():
                for _ in range(2):
                    f()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(5):
                    f()
                e1.record(); e1.synchronize()
                rounds[k].append(2.0 * m**3 * 5 / e0.elapsed_time(e1) / 1e9)
        emit_line({"profiling": name, "size": size, "tflops_median_of_4_rounds_of_5": {k: statistics.median(v) for k, v in rounds.items()}, "status": int(st.item())})
        return
    for f in (em, hw):
        for _ in range(reps):
            f()
    torch.cuda.synchronize()
    emit_line({"profiling": name, "size": size, "launches_each": reps})


_REAL_STDOUT = None


def emit_line(obj) -> None:
    """Prints the one JSON line on the process's real stdout."""
    text = json.dumps(obj) + "\n"
    sys.stdout.flush()
    if _REAL_STDOUT is None:
        sys.stdout.write(text)
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, text.encode())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="basalt_b200", choices=["basalt_b200", "reference"])
    ap.add_argument("--no-others", action="store_true", help="headline only: skip the `configs` sections of the other four configurations")
    ap.add_argument("--no-multimem", action="store_true", help="skip the gather variant that goes through an NVLink multicast mapping (torch symmetric memory)")
    ap.add_argument("--only", default=None, help="comma-separated subset of vadd_i32,helper_chain,sgemm_f32,matmul_f16 for the `configs` sections")
    ap.add_argument("--elements", type=int, default=N_MAX, help="int32 elements per GPU (profiling runs use a smaller case)")
    ap.add_argument("--nccl-exchange", action="store_true", help="at N > 1 use ncclAllReduce for the 4-byte exchange instead of the peer-memory kernel")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer and CPU-baseline legs (profiling runs)")
    ap.add_argument("--profile", default=None, choices=["max_i32", "vadd_i32", "helper_chain", "sgemm_f32", "matmul_f16", "matmul_f16_forms"],
                    help="run only this workload's emitted and hand-written kernels a few times on a small case (for ncu) and exit; "
                         "matmul_f16_forms times every form of the fp16 matmul kernels with CUDA events instead")
    ap.add_argument("--size", type=int, default=0, help="problem size for --profile (elements, or the matrix dimension)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    # Libraries (NCCL's version banner, build tools) write to file descriptor 1; the contract is one
    # JSON line on stdout, so everything else goes to stderr until that line is printed.
    sys.stdout.flush()
    global _REAL_STDOUT
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    if int(os.environ.get("LOCAL_RANK", "0")) == 0:
        from basalt_b200 import build as native_build
        native_build.build()          # no-op when libbasalt_b200.so is up to date; needs nvcc otherwise
    if args.impl == "reference":
        return reference_arm(args)
    if args.profile:
        return profile_one(args)

    import torch

    import basalt_b200 as b
    from basalt_b200 import kernels, kernels_bir as kb, sharding, workloads as w

    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    local_cpus = sharding.bind_to_gpu_cpus(local_rank)      # host buffers of the end-to-end leg land on the GPU's NUMA node
    torch.cuda.set_device(local_rank)
    group = sharding.RankGroup.from_env("nccl")
    rank, world = group.rank, group.world
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE is {world}", file=sys.stderr)
    ctx = b.CudaDriver.load().create_context(local_rank)
    comm = group.nccl(ctx)
    peers, exchange_kind = None, "none"
    if world > 1:
        exchange_kind = "ncclAllReduce(max) of 1 int32"
        if not args.nccl_exchange:
            try:
                peers = group.peers(ctx)
                exchange_kind = "allreduce(max) of 1 int32 over peer-mapped memory (release stores / acquire loads across NVLink)"
            except b.CudaError as e:
                print(f"peer-memory exchange unavailable ({e}); using NCCL", file=sys.stderr)
    stream = torch.cuda.current_stream().cuda_stream
    peaks = measured_peaks()
    peak_hbm = peaks["hbm_gbs"]
    env = Env(torch, ctx, group, comm, peers, stream, peaks, args)

    # ---- inputs: this rank's contiguous shard, generated on the device by the seeded generator and
    # copied to pinned host memory for the end-to-end and CPU legs ----
    n = args.elements
    x = env.fill("u32", w.SEEDS["max_i32"] + rank, n, torch.int32)
    torch.cuda.synchronize()
    expect_local = int(x.max().item())
    partial = torch.empty(1, dtype=torch.int32, device="cuda")
    result = torch.empty(1, dtype=torch.int32, device="cuda")
    lowest = torch.full((1,), -2**31, dtype=torch.int32, device="cuda")

    fn = ctx.load_module(b.Ptx().emit(kb.load("max_i32")).text).get_function("max_i32")
    blocks = fn.streaming_grid(256, n)   # about 64 elements per thread, at most 16 resident waves: measured faster than one wave
    launch_emitted = fn.bind(blocks, 256, 0, [b.ptr(x.data_ptr()), b.ptr(partial.data_ptr()), b.i32(n)], stream=stream)

    # The exchange step at N > 1: allreduce(max) of the 4-byte partials.  Over peer-mapped memory
    # (one small kernel of release stores and acquire loads across NVLink) when the GPUs can map
    # each other, else ncclAllReduce; both on the launching stream, so a step ends when its result
    # is in `result`.  (Issuing the collective on a second stream to overlap it with the next
    # step's kernel was measured and is slower: the collective's CTA competes with the
    # reduction's CTAs for the SMs.)
    def reset():
        if peers is None:
            partial.copy_(lowest)                              # a 4-byte device copy resets the running maximum

    def exchange():
        if peers is not None:                                  # also resets `partial` for the next step
            peers.allreduce_max_i32(partial.data_ptr(), result.data_ptr(), stream, reset_to=-2**31)
        elif comm is not None:
            comm.allreduce_max_i32(partial.data_ptr(), result.data_ptr(), 1, stream)

    partial.copy_(lowest)

    def step_emitted():
        reset()
        launch_emitted()                                       # basalt_rt_launch: the emitted sm_100a kernel
        exchange()

    def step_hand():
        reset()
        kernels.max_i32(x.data_ptr(), n, partial.data_ptr(), stream)
        exchange()

    def step_fused():                                          # hand-written: reduction and exchange in one launch
        peers.max_i32(x.data_ptr(), n, result.data_ptr(), stream)

    def last_result():
        return int((result if world > 1 else partial).item())

    def timed_loop(step_fn, steps):
        group.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step_fn()
        e1.record()
        torch.cuda.synchronize()
        group.barrier()
        return group.max_float(e0.elapsed_time(e1))

    sampler = ClockSampler(local_rank) if rank == 0 else None
    for _ in range(args.warmup):
        step_emitted()
    torch.cuda.synchronize()
    t_begin = time.time()
    total_ms = timed_loop(step_emitted, args.steps)
    got = last_result()
    # Kernel-only time of the dominant kernel, measured live: its average duration over a run of back-to-back launches
    # (as in the timed region, where the set-up of each launch overlaps the kernel before it: programmatic dependent
    # launch), and the duration of a launch that stands alone between two events.
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(min(args.steps, 200))]
    for e0, e1 in ev:
        partial.copy_(lowest)
        e0.record(); launch_emitted(); e1.record()
    torch.cuda.synchronize()
    kernel_ms_single = statistics.mean(e0.elapsed_time(e1) for e0, e1 in ev)
    partial.copy_(lowest)
    run0, run1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    run0.record()
    for _ in range(len(ev)):
        launch_emitted()
    run1.record()
    torch.cuda.synchronize()
    kernel_ms = run0.elapsed_time(run1) / len(ev)
    partial.copy_(lowest)
    for _ in range(args.warmup):
        step_hand()
    hand_ms = timed_loop(step_hand, args.steps) / args.steps
    fused = None
    if peers is not None:
        for _ in range(args.warmup):
            step_fused()
        fused_ms = timed_loop(step_fused, args.steps) / args.steps
        fused = {"ms_per_step": fused_ms, "gbs_all_ranks": 4.0 * n * world / fused_ms / 1e6, "ok": last_result() == group.max_i32_host(expect_local),
                 "what": "hand-written kernel: the shard's reduction and, in its last CTA, the peer-memory exchange; one launch per step"}
    t_end = time.time()
    clocks = sampler.stop(t_begin, t_end) if sampler else None

    # ---- BASELINE's strong-scaling reading of this configuration: 2^28 elements in all, split over the ranks ----
    strong = None
    if world > 1 and n == N_MAX:
        ns = n // world
        blocks_s = fn.streaming_grid(256, ns)
        launch_s = fn.bind(blocks_s, 256, 0, [b.ptr(x.data_ptr()), b.ptr(partial.data_ptr()), b.i32(ns)], stream=stream)

        def step_strong():
            reset(); launch_s(); exchange()

        def kernel_only():
            launch_s()
        for _ in range(args.warmup):
            step_strong()
        s_ms = timed_loop(step_strong, args.steps) / args.steps
        got_s = last_result()
        partial.copy_(lowest)
        k_ms = timed_loop(kernel_only, args.steps) / args.steps
        partial.copy_(lowest)
        want_s = group.max_i32_host(int(x[:ns].max().item()))
        strong = {"elements_total": ns * world, "elements_per_gpu": ns, "ms_per_step": s_ms, "gbs_all_ranks": 4.0 * ns * world / s_ms / 1e6,
                  "kernel_only_ms": k_ms, "exchange_share_of_step": max(0.0, 1.0 - k_ms / s_ms), "parity": got_s == want_s,
                  "note": "each rank reduces the first 2^28/N elements of its own seeded shard (the inputs differ between ranks; the sizes and the exchange are those of a 2^28-element array split N ways); "
                          "the step is the reduction kernel plus the 4-byte exchange, so the exchange's share grows as the shards shrink"}

    # ---- end to end: host buffers through the reference's CPU launch ABI on the device ----
    out_host = np.empty(1, np.int32)
    e2e_steps = max(3, min(args.steps, 10))
    got_e2e, e2e_ms, e2e_page_ms, host_x = got, float("nan"), None, None
    if not args.no_e2e:
        host_x = env.host_copy(x)                              # page-locked, through basalt_rt_host_alloc
        host_in = host_x.view()
        host_in.flags.writeable = False                        # an input of the launch: copied to the device, never back

        def step_e2e(src=host_in):
            out_host[0] = -2**31
            ctx.cpu_launch(fn, [src, out_host, b.i32(n)], nthreads=blocks * 256, block=256)   # H2D 1 GiB, launch, D2H 4 B
            return group.max_i32_host(int(out_host[0])) if world > 1 else int(out_host[0])
        step_e2e()
        group.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            got_e2e = step_e2e()
        e2e_ms = group.max_float((time.perf_counter() - t0) * 1e3) / e2e_steps
        if world == 1:     # the same call from ordinary pageable memory, which is what a caller of the reference's ABI passes
            page = np.array(host_x)
            page.flags.writeable = False
            step_e2e(page)
            t0 = time.perf_counter()
            for _ in range(3):
                got_page = step_e2e(page)
            e2e_page_ms = (time.perf_counter() - t0) * 1e3 / 3
            got_e2e = got_e2e if got_page == got_e2e else None
            del page

    expect = group.max_i32_host(expect_local)
    parity = bool(got == expect and got_e2e == expect)
    if world == 1 and n == N_MAX:
        parity = parity and got == env.golden["max_i32"]["full"]["value"]

    cpu = None
    if rank == 0 and not args.no_e2e:
        t_cpu, r_cpu, how, c_gbs = cpu_max(np.array(host_x), 3)
        parity = parity and (world > 1 or r_cpu == expect)
        cpu = {"value": 4.0 * n / t_cpu / 1e9, "unit": "GB/s", "cores": 1, "kind": "port", "c_loop_gbs": c_gbs,
               "sample": f"3 full passes over this rank's int32 shard (best); {how}"}
    del host_x

    # ---- the five configurations ----
    configs = {}
    headline_launches = args.warmup * (2 + (1 if peers else 0)) + 2 * args.steps + 2 * len(ev)
    if not args.no_others:
        wanted = args.only.split(",") if args.only else ["vadd_i32", "helper_chain", "sgemm_f32", "matmul_f16"]
        # the headline reduction from its other two source forms (the headline itself is emitted from BIR text)
        mx = {"workload": headline_config(n, world)["workload"], "unit": "GB/s", "value": 4.0 * n * world / (total_ms / args.steps) / 1e6, "see": "the top-level keys of this line"}
        if world == 1:
            try:
                from basalt_b200 import kernels_cu as kc, kernels_triton as kt
                acc = torch.full((1,), -2**31, dtype=torch.int32, device="cuda")
                f_c = env.emitted(b.compile_cuda(kc.load("max_i32")), "max_i32")
                ms_c = env.timed(f_c.bind(f_c.streaming_grid(256, n), 256, 0, [env.dp(x), env.dp(acc), b.i32(n)], stream=stream), 20)
                ok_c = int(acc.item()) == expect
                acc.fill_(-2**31)
                f_t = env.emitted(kt.max_i32(), "max_i32")
                block = 8192                       # lanes per program
                ms_t = env.timed(f_t.bind((n + block - 1) // block, 128, 0, [env.dp(x), env.dp(acc), b.i64(n), b.i64(block)], stream=stream), 20)
                mx["other_sources"] = {"from_cuda_c_gbs": 4.0 * n / ms_c / 1e6, "from_triton_gbs": 4.0 * n / ms_t / 1e6, "handwritten_gbs": 4.0 * n / hand_ms / 1e6,
                                       "from_triton_over_handwritten": hand_ms / ms_t, "parity": ok_c and int(acc.item()) == expect}
            except Exception as e:   # noqa: BLE001 - reported, not hidden
                mx["other_sources_error"] = str(e)[:200]
        if strong is not None:
            mx["strong_scaling"] = strong
        configs["max_i32"] = mx
        del x
        for name, fn_cfg in (("vadd_i32", cfg_vadd), ("helper_chain", cfg_chain), ("sgemm_f32", cfg_sgemm), ("matmul_f16", cfg_matmul)):
            if name not in wanted:
                continue
            if name in ("sgemm_f32", "matmul_f16") and world > 1 and (4096 if name == "sgemm_f32" else 8192) % (256 * world):
                continue
            try:
                configs[name] = fn_cfg(env)
            except Exception as e:   # noqa: BLE001 - reported, not hidden
                import traceback
                configs[name] = {"error": str(e)[:300], "where": traceback.format_exc()[-400:]}
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
    ms_per_step = total_ms / args.steps
    total_bytes = 4.0 * n * world
    if rank == 0:
        achieved = 4.0 * n / (kernel_ms * 1e-3) / 1e9
        traffic, traffic_source = traffic_from_profile("max_i32", n)
        cfg = headline_config(n, world)
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak_hbm, "unit": "GB/s", "frac": achieved / peak_hbm, "peak_source": peaks["source"],
                    "traffic": traffic, "traffic_source": traffic_source, "kernel": "max_i32 (emitted)", "kernel_ms": kernel_ms, "kernel_ms_single_launch": kernel_ms_single,
                    "kernel_ms_how": "average over a run of back-to-back launches, CUDA events around the run; single_launch: one launch between two events",
                    "algorithmic_bytes_per_launch": 4 * n}
        e2e = {"value": total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": 4 * n + 4, "d2h_bytes_per_step": 4,
               "ms_per_step": e2e_ms, "steps": e2e_steps, "api": "basalt_rt_cpu_launch (kernel parameters as host pointers, then nthreads)",
               "host_memory": "pinned (basalt_rt_host_alloc): the favourable case; a caller of the reference's ABI passes pageable memory, see pageable_value",
               "pageable_value": (total_bytes / (e2e_page_ms * 1e-3) / 1e9) if e2e_page_ms else None, "pageable_ms_per_step": e2e_page_ms,
               "bound": "PCIe host-to-device copy of the 1 GiB shard" + ("" if world == 1 else f"; the {world} ranks' host buffers sit on one NUMA node and share its memory and PCIe root bandwidth")}
        line = {
            "metric": METRIC, "value": total_bytes / (ms_per_step * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "i32", "data": "synthetic", "config": cfg,
            "launch": {"kernel": "emitted sm_100a max_i32 through basalt_rt_launch" + ((", then " + exchange_kind + " per step") if world > 1 else ""),
                       "grid": blocks, "block": 256, "host_cpus_bound_to_gpu_numa_node": len(local_cpus)},
            "parity": parity, "roofline": roofline,
            "handwritten": {"value": total_bytes / (hand_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": hand_ms},
            "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": args.steps * (2 if peers is not None else 1),
            "gpu_launches_whole_run": headline_launches + env.launches,
            "clocks": clocks,
        }
        if configs:
            configs["max_i32"].update({"roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "parity": parity, "handwritten_gbs": total_bytes / (hand_ms * 1e-3) / 1e9})
            line["configs"] = configs
            line["parity_all_configs"] = bool(parity and all(c.get("parity", False) for c in configs.values()))
        if fused is not None:
            line["handwritten_fused_reduce_exchange"] = fused
        emit_line(line)
    if peers is not None:
        bad = peers.status()
        if bad:
            print(f"rank {rank}: peer exchange gave up waiting for ranks with bits {bad:#x}", file=sys.stderr)
        group.barrier()
        peers.destroy()
    if comm is not None:
        comm.destroy()
    if group.dist is not None:
        group.barrier()
        group.dist.destroy_process_group()


if __name__ == "__main__":
    main()
