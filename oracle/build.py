"""Builds the CPU oracle (test infrastructure) into oracle/liborc.so.

    python oracle/build.py

-ffp-contract=off keeps every multiply and add separate, as the reference's x86 oracle emits them
(mulss then addss, crates/basalt-x86/src/oracle.rs:1530-1543).  -fno-tree-vectorize keeps the
timed per-thread loops scalar, like the reference's emitted code; the two `_rows` helpers that
only serve as full-size parity references opt back in with OpenMP and are vectorised per lane,
which does not change any rounding.

The reference itself is Rust and there is no cargo/rustc in this environment, so no oracle/_ref
build exists: the restatement in basalt_oracle.c is the only CPU arm.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "basalt_oracle.c")
OUT = os.path.join(HERE, "liborc.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = ["gcc", "-O2", "-march=x86-64-v2", "-ffp-contract=off", "-fno-tree-vectorize", "-fopenmp", "-fPIC",
           "-shared", "-fvisibility=hidden", "-Wall", "-Wextra", "-o", OUT, SRC, "-lm"]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
