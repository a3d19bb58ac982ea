"""Builds the CPU oracle (test infrastructure) into oracle/liborc.so.

    python oracle/build.py

-ffp-contract=off keeps every multiply and add separate, as the reference's x86 oracle emits them
(mulss then addss, crates/basalt-x86/src/oracle.rs:1530-1543).  -fno-tree-vectorize keeps the
timed per-thread loops scalar, like the reference's emitted code; the two `_rows` helpers that
only serve as full-size parity references opt back in with OpenMP and are vectorised per lane,
which does not change any rounding.

The reference itself is Rust and there is no cargo/rustc in this environment, so no oracle/_ref
build exists.  Two restatements stand in for it: basalt_oracle.c (launch model and arithmetic of the
workloads as C loops) and x86_regalloc.cpp (the reference's register-allocating x86-64 back end as a
JIT, oracle/libx86regalloc.so; it is linked with the BIR parser and construct_ssa of the library under
test, which are the input format and first pass of the reference's own emit).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "basalt_oracle.c")
OUT = os.path.join(HERE, "liborc.so")
JIT_SRC = os.path.join(HERE, "x86_regalloc.cpp")
JIT_OUT = os.path.join(HERE, "libx86regalloc.so")
CSRC = os.path.join(os.path.dirname(HERE), "basalt_b200", "csrc")
JIT_DEPS = [os.path.join(CSRC, n) for n in ("bir.cpp", "passes.cpp", "bir.hpp", "passes.hpp")]


def _fresh(out: str, deps: list) -> bool:
    return os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in deps)


def build(force: bool = False) -> str:
    if force or not _fresh(OUT, [SRC]):
        subprocess.check_call(["gcc", "-O2", "-march=x86-64-v2", "-ffp-contract=off", "-fno-tree-vectorize", "-fopenmp", "-fPIC",
                               "-shared", "-fvisibility=hidden", "-Wall", "-Wextra", "-o", OUT, SRC, "-lm"])
    if force or not _fresh(JIT_OUT, [JIT_SRC] + JIT_DEPS):
        subprocess.check_call(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall", "-Wextra", "-Wl,--no-undefined",
                               "-o", JIT_OUT, JIT_SRC, JIT_DEPS[0], JIT_DEPS[1]])
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
