"""The compile side of the drop-in: `Ptx`, a mirror of the reference's `impl Backend for Ptx`
(crates/basalt-ptx/src/emit.rs:1973-1994; trait in crates/basalt-backend/src/backend.rs:144-157),
over the C ABI.  A module crosses the boundary as BIR text."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

from ._lib import DiagStruct, EmitOpts as _COpts, lib


class Diag(Exception):
    """A refusal: `code` is one of the reference's stable E-codes
    (crates/basalt-diag/src/ecode.rs:148-181), `arg` the text it would render."""

    def __init__(self, code: str, arg: str):
        super().__init__(f"{code}: {arg}")
        self.code = code
        self.arg = arg


@dataclass(frozen=True)
class Support:
    """Support::{Supported, Unsupported(ECode)} (backend.rs:17-25)."""
    supported: bool
    code: str | None = None


@dataclass(frozen=True)
class EmitOpts:
    """EmitOpts (backend.rs:123-137). opt_level 0 lowers one to one, 2 runs the B200 passes."""
    target_variant: str | None = None
    opt_level: int = 2
    out_name_hint: str | None = None
    snap: bool = False


@dataclass(frozen=True)
class Artifact:
    """Artifact{kind: Ptx, payload: Text} (backend.rs:36-73)."""
    kind: str
    text: str


def _copts(o: EmitOpts | None):
    if o is None:
        return None
    return C.byref(_COpts(o.target_variant.encode() if o.target_variant else None, o.opt_level,
                          o.out_name_hint.encode() if o.out_name_hint else None, int(o.snap)))


def _text_call(fn, bir: str, opts) -> str:
    src = bir.encode()
    out, n, d = C.c_void_p(), C.c_size_t(), DiagStruct()
    args = [src, len(src)] + ([opts] if opts is not False else []) + [C.byref(out), C.byref(n), C.byref(d)]
    rc = fn(*args)
    if rc != 0:
        raise Diag(d.code.decode(), d.message.decode())
    try:
        return C.string_at(out.value, n.value).decode()
    finally:
        lib.basalt_b200_free(out)


class Ptx:
    """The sm_100a PTX backend. Stateless, like the reference's unit struct."""

    def name(self) -> str:
        return lib.basalt_b200_name().decode()

    def supports(self, bir: str) -> Support:
        src = bir.encode()
        code = (C.c_char * 8)()
        rc = lib.basalt_b200_supports(src, len(src), code)
        if rc == 1:
            return Support(True)
        return Support(False, code.value.decode())

    def emit(self, bir: str, opts: EmitOpts | None = None) -> Artifact:
        return Artifact("ptx", _text_call(lib.basalt_b200_emit, bir, _copts(opts)))

    def optimized_bir(self, bir: str, opts: EmitOpts | None = None) -> str:
        """The module as lowered, after inlining and the vectorising passes (no reference
        counterpart; lets the passes be checked against the CPU oracle)."""
        return _text_call(lib.basalt_b200_optimize, bir, _copts(opts))


def roundtrip(bir: str) -> str:
    """parse then print (crates/basalt-bir/src/lib.rs:79-85)."""
    return _text_call(lib.basalt_b200_roundtrip, bir, False)


def compile_cuda(source: str) -> str:
    """CUDA-C subset -> slot-form BIR text: the front half of the reference CLI's CUDA-C lane
    (crates/basalt-cli/src/main.rs:286-327; crates/basalt-frontend-c, crates/basalt-sema/src/lower.rs).
    Raises Diag with the reference's front-end codes (E200-E202, E300-E304, E308)."""
    return _text_call(lib.basalt_b200_compile_cuda, source, False)


def compile_triton(source: str, constexprs: dict | None = None, pointee: dict | None = None, num_warps: int | None = None,
                   min_blocks: int | None = None) -> str:
    """`@triton.jit` source -> tile-level BIR text: the front half of the reference CLI's Triton lane
    (crates/basalt-cli/src/main.rs:329-372), with tl.dot lowered to `mma` and a program mapped to a
    CTA.  `constexprs` binds tl.constexpr parameters that have no literal default, `pointee` names
    the element type behind pointer parameters ("f16", "f32", "f64", "i64"; f32 when absent),
    `num_warps` the CTA size the kernel is compiled for."""
    items = [f"{k}={int(v)}" for k, v in (constexprs or {}).items()] + [f"{k}=*{v}" for k, v in (pointee or {}).items()]
    if num_warps is not None:
        items.append(f"num_warps={int(num_warps)}")
    if min_blocks is not None:
        items.append(f"min_blocks={int(min_blocks)}")
    return _text_call(lib.basalt_b200_compile_triton, source, " ".join(items).encode())
