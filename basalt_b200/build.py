"""Builds libbasalt_b200.so in-tree: the C++ backend and runtime (g++) plus the hand-written
sm_100a kernels (nvcc, -gencode arch=compute_100a,code=sm_100a), linked with the static CUDA
runtime.  The driver API and NCCL are resolved with dlopen at run time, so the library loads on a
machine without a GPU.

    python -m basalt_b200.build [--force]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libbasalt_b200.so")
CLI = os.path.join(HERE, "basalt-b200")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")

CXX_SOURCES = ["bir.cpp", "passes.cpp", "emit.cpp", "emit_mma.cpp", "regbudget.cpp", "frontend_c.cpp", "frontend_triton.cpp", "capi.cpp", "runtime.cpp"]
CU_SOURCES = ["kernels/common.cu", "kernels/streaming.cu", "kernels/sgemm.cu", "kernels/matmul_f16_tc.cu", "kernels/collective.cu", "kernels/workload_fill.cu"]
HEADERS = ["bir.hpp", "passes.hpp", "emit.hpp", "frontend_c.hpp", "frontend_triton.hpp", "kernels/common.cuh", "../../include/basalt_b200.h",
           "../../include/basalt_b200_kernels.h"]
CXXFLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-Wextra", "-fvisibility=hidden", f"-I{CUDA_HOME}/include"]
NVCCFLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler",
             "-fPIC,-fvisibility=hidden"]


def _nvcc() -> str:
    path = shutil.which("nvcc") or os.path.join(CUDA_HOME, "bin", "nvcc")
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return path


def _stale(out: str, deps: list[str]) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


SHIM_KERNELS = ("vector_add_f32", "chain_vector", "square_vector", "mma2x2", "tiled_sgemm_f32", "tri_vadd", "tri_matmul")


def _build_shims(force: bool, run) -> None:
    """libbasalt_cpu_launch_{cuda,triton}.so: the reference's example kernels under their own symbols."""
    src = os.path.join(CSRC, "shims", "cpu_launch_shims.cpp")
    inc = os.path.join(OBJ, "shim_bir.inc")
    bir_dir = os.path.join(HERE, "bir")
    deps = [os.path.join(bir_dir, k + ".bir") for k in SHIM_KERNELS] + [os.path.join(HERE, "kernels_bir.py"), os.path.abspath(__file__)]
    if force or _stale(inc, deps):
        sys.path.insert(0, os.path.dirname(HERE))
        from basalt_b200 import kernels_bir   # pure Python; the package resolves native names lazily
        texts = {k: kernels_bir.load(k) for k in SHIM_KERNELS}
        texts["stress"] = kernels_bir.stress()
        with open(inc, "w") as f:
            for k, t in texts.items():
                f.write(f'static const char kBir_{k}[] = R"BIR({t})BIR";\n')
    for flavour, flag in (("cuda", []), ("triton", ["-DBASALT_SHIMS_TRITON"])):
        out = os.path.join(HERE, f"libbasalt_cpu_launch_{flavour}.so")
        if force or _stale(out, [src, inc, LIB]):
            run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", *flag, f"-I{OBJ}", "-o", out, src, f"-L{HERE}", "-lbasalt_b200",
                 "-Wl,-rpath,$ORIGIN", "-lpthread"])


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdrs = [os.path.join(CSRC, h) for h in HEADERS] + [os.path.abspath(__file__)]
    jobs, objs = [], []
    for src in CXX_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src.replace("/", "_") + ".o")
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            jobs.append(["g++", *CXXFLAGS, "-c", s, "-o", o])
    nvcc = _nvcc()
    for src in CU_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src.replace("/", "_") + ".o")
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            jobs.append([nvcc, *NVCCFLAGS, "-c", s, "-o", o])

    def run(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(run, jobs))
    if force or jobs or _stale(LIB, objs):
        run([nvcc, "-shared", "-o", LIB, *objs, "-cudart", "static", "-Xlinker", "--no-undefined", "-ldl", "-lpthread", "-lrt"])
    _build_shims(force, run)
    cli_src = os.path.join(CSRC, "cli.cpp")
    if force or _stale(CLI, [cli_src, LIB]):
        run(["g++", "-std=c++17", "-O2", "-o", CLI, cli_src, f"-L{HERE}", "-lbasalt_b200", "-Wl,-rpath,$ORIGIN"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
