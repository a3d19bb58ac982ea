"""A small assembler for hand-written BIR.

BIR's text form numbers every value by its position in the function (`%N` must be the arena
index, `bbN` the block index; crates/basalt-bir/src/parse.rs:423-499 of the reference), which makes
editing a kernel by hand tedious.  `assemble` accepts the same grammar with symbolic names --
`%acc = add i32 %acc0, %x`, `loop:`, `br loop`, `phi i32 [entry -> %g, body -> %next]` -- and
returns canonical, numbered BIR text.  `%argN` parameter references pass through unchanged.

The config-sized kernels under basalt_b200/bir/ are written this way (`*.birs` sources, assembled
`*.bir` committed beside them) because the reference's CUDA-C and Triton front ends are Rust and
cannot run here.
"""
from __future__ import annotations

import re

_LABEL = re.compile(r"^\s*([A-Za-z_][A-Za-z0-9_.]*)\s*:\s*$")
_DEF = re.compile(r"^\s*(%[A-Za-z_][A-Za-z0-9_.]*)\s*=\s*(.*)$")
_VAL = re.compile(r"%[A-Za-z_][A-Za-z0-9_.]*")
_TERMS = ("br", "condbr", "switch", "ret")


def assemble(text: str) -> str:
    out: list[str] = []
    lines = [re.sub(r"\s*;.*$", "", l) for l in text.splitlines()]
    lines = [l for k, l in enumerate(lines) if l.strip() or (k > 0 and lines[k - 1].strip())]
    i = 0
    while i < len(lines):
        ln = lines[i]
        if re.match(r"^\s*(host\s+)?func\s+@", ln):
            j = i + 1
            while not re.match(r"^\s*}\s*$", lines[j]):
                j += 1
            out.append(ln.rstrip())
            out.extend(_assemble_func(lines[i + 1:j]))
            out.append("  }")
            i = j + 1
        else:
            out.append(ln.rstrip())
            i += 1
    return "\n".join(out) + "\n"


def _assemble_func(body: list[str]) -> list[str]:
    body = [re.sub(r"\s*;.*$", "", l) for l in body]
    body = [l for l in body if l.strip()]
    labels: dict[str, int] = {}
    values: dict[str, int] = {}
    n_inst = 0
    for l in body:
        m = _LABEL.match(l)
        if m:
            if m.group(1) in labels:
                raise ValueError(f"duplicate label {m.group(1)}")
            labels[m.group(1)] = len(labels)
            continue
        word = l.split()[0]
        if word in _TERMS:
            continue
        d = _DEF.match(l)
        if d and not re.match(r"%arg\d+$", d.group(1)):
            if d.group(1) in values:
                raise ValueError(f"value {d.group(1)} defined twice")
            values[d.group(1)] = n_inst
        n_inst += 1

    def sub_vals(s: str) -> str:
        def rep(m):
            name = m.group(0)
            if re.match(r"%arg\d+$", name):
                return name
            if name not in values:
                raise ValueError(f"undefined value {name}")
            return f"%{values[name]}"
        return _VAL.sub(rep, s)

    def sub_labels(s: str) -> str:
        def rep(m):
            w = m.group(0)
            return f"bb{labels[w]}" if w in labels else w
        return re.sub(r"(?<![%@A-Za-z0-9_.])[A-Za-z_][A-Za-z0-9_.]*", rep, s)

    out = []
    for l in body:
        m = _LABEL.match(l)
        if m:
            out.append(f"  bb{labels[m.group(1)]}:")
            continue
        s = l.strip()
        word = s.split()[0]
        if word in _TERMS:
            out.append("    " + sub_vals(sub_labels(s)))
            continue
        d = _DEF.match(l)
        rhs = d.group(2) if d else s
        if rhs.split()[0] == "phi":
            head, _, tail = rhs.partition("[")
            rhs = head + "[" + sub_labels(tail)
        rhs = sub_vals(rhs)
        out.append("    " + (f"%{values[d.group(1)]} = {rhs}" if d else rhs))
    return out
