"""BIR interpreter with the semantics of Basalt's x86-64 oracle backend.

TEST INFRASTRUCTURE ONLY: the product package never imports this module. It exists so that any
BIR module -- the hand-authored kernels and the output of the emitter's own BIR-to-BIR passes --
can be executed on the CPU under the reference's CPU launch model and compared with what the
GPU produced. Pure Python, so only for small cases (thousands of threads).

Rules restated (crates/basalt-x86/src/oracle.rs in the reference project):
  * launch model (oracle.rs:7-28, 1058-1098, 1418-1437): threads of one flat block run one at a
    time to completion, `for t in range(nthreads)`; tid.x = t, bdim.x = nthreads, tid.y/z = 0,
    bid.* = 0, bdim.y/z = gdim.* = 1; `barrier` does nothing;
  * shuffle / ballot / vote are refused with E090 (oracle.rs:651-655);
  * integers wrap at their declared width, div/rem are signed (oracle.rs:1546-1610), compares use
    the predicate's signedness (oracle.rs:1629-1653);
  * floats are IEEE round-to-nearest and never fused; frem = a - trunc(a/b)*b (oracle.rs:1530-1543,
    1618-1627);
  * atomics are load-op-store returning the old value, integer min/max signed (oracle.rs:1910-2021);
  * `mma`: acc = 0; for k: acc = acc + a*b; D = C + acc (oracle.rs:2178-2337);
  * `call` is a plain by-value call (oracle.rs:2086-2115);
  * a synthetic `const.i ptr.<space> K` address names one storage cell that lives for the whole
    launch (oracle.rs "Synthesizing local/param/shared/constant addresses").
Extensions of this project that the interpreter also honours: `shared_obj <K> bytes <n> align <a>`
module lines (a sized cell instead of 8 bytes), explicit leading dimensions and an output dtype on
`mma` (`ld <lda> <ldb> <ldc> <ldd>` / `out <ty>`), the `vec.extract` / `vec.build` ops the emitter's
passes produce (`warp.reduce.*` parses but is refused like a shuffle), and the f16 type (widen to f32, operate, round
once back) which the reference's CPU backends refuse.

The text grammar is the reference's (crates/basalt-bir/src/lib.rs:21-68, print.rs:200-259); this
file has its own small parser so that it shares no code with the product's C++ parser.
"""
from __future__ import annotations

import re
import struct
from dataclasses import dataclass, field

import numpy as np


class OracleRefusal(Exception):
    """Raised with the reference's E-code when the oracle model cannot run a module."""

    def __init__(self, code: str, why: str):
        super().__init__(f"{code}: {why}")
        self.code = code


_INT_BITS = {"i1": 1, "i8": 8, "i16": 16, "i32": 32, "i64": 64}
_FLOATS = {"f16": np.float16, "f32": np.float32, "f64": np.float64}
_SIZE = {"i1": 1, "i8": 1, "i16": 2, "i32": 4, "i64": 8, "f16": 2, "f32": 4, "f64": 8}
_BIN = {"add", "sub", "mul", "div", "rem", "fadd", "fsub", "fmul", "fdiv", "frem", "and", "or", "xor",
        "shl", "lshr", "ashr"}
_CAST = {"trunc", "zext", "sext", "fptrunc", "fpext", "fptosi", "fptoui", "sitofp", "uitofp", "bitcast"}
_INDEX = {f"{a}.{d}" for a in ("tid", "bid", "bdim", "gdim") for d in "xyz"}
_ATOMIC = {"atomic." + s for s in ("add", "sub", "exch", "min", "max", "and", "or", "xor")}
_SHUFFLE = {"shuffle.idx", "shuffle.up", "shuffle.down", "shuffle.xor"}
_TOK = re.compile(r"->|[(){}\[\],:=]|[A-Za-z0-9_.@%\-+]+")


def _is_ptr(ty: str) -> bool:
    return ty.startswith("ptr.")


def _vec(ty: str):
    m = re.fullmatch(r"v(\d+)(i1|i8|i16|i32|i64|f16|f32|f64)", ty)
    return (int(m.group(1)), m.group(2)) if m else None


def _bits(ty: str) -> int:
    return 64 if _is_ptr(ty) else _INT_BITS[ty]


def _wrap(v: int, bits: int) -> int:
    return v & ((1 << bits) - 1)


def _signed(v: int, bits: int) -> int:
    v &= (1 << bits) - 1
    return v - (1 << bits) if v >> (bits - 1) else v


@dataclass
class Inst:
    op: str
    ty: str
    args: list = field(default_factory=list)   # operand value refs ("%3" / "%arg0")
    attr: dict = field(default_factory=dict)


@dataclass
class Block:
    insts: list
    term: tuple


@dataclass
class Func:
    name: str
    is_kernel: bool
    params: list
    ret: str
    blocks: list
    insts: list   # arena: index == %N


@dataclass
class Module:
    funcs: list
    shared_objs: dict   # K -> (bytes, align)
    shared_mem_bytes: int


def parse(text: str) -> Module:
    toks = _TOK.findall(text)
    pos = 0

    def peek():
        return toks[pos] if pos < len(toks) else None

    def nxt():
        nonlocal pos
        t = toks[pos]
        pos += 1
        return t

    def expect(t):
        got = nxt()
        if got != t:
            raise ValueError(f"expected {t!r}, found {got!r}")

    expect("module"); expect("{")
    if peek() == "launch_bounds":
        nxt(); expect("max_threads"); expect("="); nxt(); expect("min_blocks"); expect("="); nxt()
    expect("shared_mem_bytes"); smem = int(nxt())
    expect("target_dtypes")
    while peek() in _SIZE:
        nxt()
    shared_objs = {}
    while peek() == "shared_obj":
        nxt(); k = int(nxt()); expect("bytes"); nb = int(nxt()); expect("align"); al = int(nxt())
        shared_objs[k] = (nb, al)
    funcs = []
    while peek() in ("func", "host"):
        is_kernel = True
        if peek() == "host":
            nxt(); is_kernel = False
        expect("func")
        name = nxt()[1:]
        expect("(")
        params = []
        while peek() != ")":
            params.append(nxt())
            if peek() == ",":
                nxt()
        expect(")"); expect("->"); ret = nxt(); expect("{")
        blocks, arena = [], []
        while peek() != "}":
            label = nxt(); assert label == f"bb{len(blocks)}", label
            expect(":")
            ids = []
            while peek() not in ("br", "condbr", "switch", "ret"):
                has_res = peek().startswith("%") and toks[pos + 1] == "="
                if has_res:
                    assert int(nxt()[1:]) == len(arena)
                    expect("=")
                inst = _parse_inst(nxt, peek, expect)
                assert has_res == (inst.ty != "void"), inst
                arena.append(inst); ids.append(len(arena) - 1)
            t = nxt()
            if t == "br":
                term = ("br", int(nxt()[2:]))
            elif t == "condbr":
                c = nxt(); expect(","); a = int(nxt()[2:]); expect(","); b = int(nxt()[2:])
                term = ("condbr", c, a, b)
            elif t == "switch":
                v = nxt(); expect(","); expect("default"); d = int(nxt()[2:]); expect("[")
                cases = []
                while peek() != "]":
                    cv = int(nxt()); expect("->"); cases.append((cv, int(nxt()[2:])))
                    if peek() == ",":
                        nxt()
                expect("]")
                term = ("switch", v, d, cases)
            else:
                term = ("ret", nxt() if peek() is not None and peek().startswith("%") else None)
            blocks.append(Block(ids, term))
        expect("}")
        funcs.append(Func(name, is_kernel, params, ret, blocks, arena))
    expect("}")
    return Module(funcs, shared_objs, smem)


def _parse_inst(nxt, peek, expect) -> Inst:
    op = nxt()

    def vals(n):
        out = []
        for i in range(n):
            if i:
                expect(",")
            out.append(nxt())
        return out

    def vlist():
        expect("[")
        out = []
        while peek() != "]":
            out.append(nxt())
            if peek() == ",":
                nxt()
        expect("]")
        return out

    if op in _BIN or op in _SHUFFLE:
        ty = nxt(); return Inst(op, ty, vals(2))
    if op in _CAST:
        dst = nxt(); src = nxt(); return Inst(op, dst, [nxt()], {"src": src})
    if op in _ATOMIC:
        ty = nxt(); sp = nxt(); return Inst(op, ty, vals(2), {"space": sp})
    if op in _INDEX:
        return Inst(op, nxt())
    if op == "const.i":
        ty = nxt(); return Inst(op, ty, [], {"v": int(nxt())})
    if op == "const.f":
        ty = nxt(); return Inst(op, ty, [], {"v": float(nxt())})
    if op in ("icmp", "fcmp"):
        pred = nxt(); oty = nxt(); return Inst(op, "i1", vals(2), {"pred": pred, "oty": oty})
    if op == "select":
        ty = nxt(); return Inst(op, ty, vals(3))
    if op == "load":
        ty = nxt(); sp = nxt(); p = nxt(); expect(","); expect("align"); al = int(nxt())
        if peek() == ",":
            nxt(); expect("volatile")
        return Inst(op, ty, [p], {"space": sp, "align": al})
    if op == "store":
        sty = nxt(); sp = nxt(); p = nxt(); expect(","); v = nxt(); expect(","); expect("align"); al = int(nxt())
        if peek() == ",":
            nxt(); expect("volatile")
        return Inst(op, "void", [p, v], {"space": sp, "sty": sty, "align": al})
    if op == "phi":
        ty = nxt(); expect("[")
        inc = []
        while peek() != "]":
            bb = int(nxt()[2:]); expect("->"); inc.append((bb, nxt()))
            if peek() == ",":
                nxt()
        expect("]")
        return Inst(op, ty, [], {"inc": inc})
    if op == "barrier":
        return Inst(op, "void")
    if op in ("ballot", "vote.any", "vote.all"):
        ty = nxt(); return Inst(op, ty, [nxt()])
    if op == "atomic.cas":
        ty = nxt(); sp = nxt(); return Inst(op, ty, vals(3), {"space": sp})
    if op == "mma":
        a = {"in": nxt(), "acc": nxt(), "la": nxt(), "lb": nxt()}
        expect("m"); a["m"] = int(nxt()); expect("n"); a["n"] = int(nxt()); expect("k"); a["k"] = int(nxt())
        if peek() == "ld":
            nxt(); a["ld"] = [int(nxt()) for _ in range(4)]
        if peek() == "out":
            nxt(); a["out"] = nxt()
        return Inst(op, "void", vals(4), a)
    if op == "call":
        ty = nxt(); callee = nxt()[1:]; return Inst(op, ty, vlist(), {"callee": callee})
    if op == "vec.extract":
        ty = nxt(); v = nxt(); expect(","); return Inst(op, ty, [v], {"lane": int(nxt())})
    if op == "vec.build":
        ty = nxt(); return Inst(op, ty, vlist())
    if op.startswith("warp.reduce."):
        ty = nxt(); return Inst(op, ty, [nxt()])
    if op in ("kernel.launch", "cuda.malloc", "cuda.memcpy", "cuda.free", "cuda.device_sync"):
        raise OracleRefusal("E090", f"host op {op} inside an interpreted kernel")
    raise ValueError(f"unknown opcode {op}")


class Memory:
    """A flat byte-addressed space holding the launch's buffers and storage cells."""

    def __init__(self):
        self.segs = []   # (base, bytearray-like memoryview)
        self.next = 0x10000

    def map(self, buf) -> int:
        mv = memoryview(buf).cast("B")
        base = (self.next + 255) & ~255
        self.segs.append((base, mv))
        self.next = base + len(mv) + 256
        return base

    def _find(self, addr, n):
        for base, mv in self.segs:
            if base <= addr and addr + n <= base + len(mv):
                return mv, addr - base
        raise IndexError(f"out-of-bounds access at {addr:#x} (+{n})")

    def read(self, addr, n) -> bytes:
        mv, off = self._find(addr, n)
        return bytes(mv[off:off + n])

    def write(self, addr, data: bytes):
        mv, off = self._find(addr, len(data))
        mv[off:off + len(data)] = data


_FMT = {"i1": "<B", "i8": "<B", "i16": "<H", "i32": "<I", "i64": "<Q"}


def _load_scalar(mem: Memory, addr: int, ty: str):
    if ty in _FLOATS:
        return np.frombuffer(mem.read(addr, _SIZE[ty]), dtype=_FLOATS[ty])[0]
    if _is_ptr(ty):
        return struct.unpack("<Q", mem.read(addr, 8))[0]
    return struct.unpack(_FMT[ty], mem.read(addr, _SIZE[ty]))[0] & ((1 << _INT_BITS[ty]) - 1)


def _store_scalar(mem: Memory, addr: int, ty: str, v):
    if ty in _FLOATS:
        mem.write(addr, _FLOATS[ty](v).tobytes())
    elif _is_ptr(ty):
        mem.write(addr, struct.pack("<Q", v & (2**64 - 1)))
    else:
        mem.write(addr, struct.pack(_FMT[ty], _wrap(v, 8 * _SIZE[ty])))


def _fbin(op, ty, a, b):
    f = _FLOATS[ty]
    if ty == "f16":   # widen, operate in f32, round once
        a32, b32 = np.float32(a), np.float32(b)
        return np.float16(_fbin(op, "f32", a32, b32))
    a, b = f(a), f(b)
    with np.errstate(all="ignore"):
        if op == "fadd":
            return f(a + b)
        if op == "fsub":
            return f(a - b)
        if op == "fmul":
            return f(a * b)
        if op == "fdiv":
            return f(a / b)
        q = f(a / b)
        return f(a - f(f(np.trunc(q)) * b))


class Interp:
    def __init__(self, module: Module, mem: Memory):
        self.m = module
        self.mem = mem
        self.funcs = {f.name: f for f in module.funcs}
        self.cells = {}   # (func, space, K) -> address; lives for the whole launch

    def cell(self, fn: Func, space: str, k: int) -> int:
        key = (fn.name, space, k)
        if key not in self.cells:
            nbytes = 8
            if space == "ptr.shared" and k in self.m.shared_objs:
                nbytes = self.m.shared_objs[k][0]
            self.cells[key] = self.mem.map(bytearray(nbytes))
        return self.cells[key]

    def launch(self, name: str, args: list, nthreads: int):
        fn = self.funcs[name]
        if not fn.is_kernel:
            raise OracleRefusal("E093", "launch target is not a kernel")
        for t in range(nthreads):
            self.run(fn, args, t, nthreads, depth=0)

    def run(self, fn: Func, args: list, tid: int, nthreads: int, depth: int):
        if depth > 64:
            raise OracleRefusal("E094", "call depth")
        vals = {}

        def get(ref):
            return args[int(ref[4:])] if ref.startswith("%arg") else vals[int(ref[1:])]

        bb, prev = 0, None
        while True:
            block = fn.blocks[bb]
            # phis read their incoming values simultaneously
            phis = [i for i in block.insts if fn.insts[i].op == "phi"]
            newv = {}
            for i in phis:
                for src, ref in fn.insts[i].attr["inc"]:
                    if src == prev:
                        newv[i] = get(ref)
                        break
                else:
                    raise ValueError(f"phi %{i} has no incoming for bb{prev}")
            vals.update(newv)
            for i in block.insts:
                inst = fn.insts[i]
                if inst.op == "phi":
                    continue
                r = self.exec(fn, inst, get, tid, nthreads, depth)
                if inst.ty != "void":
                    vals[i] = r
            t = block.term
            prev = bb
            if t[0] == "br":
                bb = t[1]
            elif t[0] == "condbr":
                bb = t[2] if get(t[1]) & 1 else t[3]
            elif t[0] == "switch":
                v = get(t[1])
                bb = t[2]
                for cv, tgt in t[3]:
                    if _wrap(cv, 64) == _wrap(v, 64) or cv == v:
                        bb = tgt
                        break
            else:
                return get(t[1]) if t[1] else None

    def exec(self, fn, inst: Inst, get, tid, nthreads, depth):
        op, ty = inst.op, inst.ty
        vec = _vec(ty) if ty != "void" else None
        if op == "const.i":
            if _is_ptr(ty) and ty != "ptr.global":
                return self.cell(fn, ty, inst.attr["v"])
            return _wrap(inst.attr["v"], _bits(ty))
        if op == "const.f":
            return _FLOATS[ty](inst.attr["v"])
        if op in _BIN:
            a, b = get(inst.args[0]), get(inst.args[1])
            if vec:
                return [self._bin(op, vec[1], x, y) for x, y in zip(a, b)]
            return self._bin(op, ty, a, b)
        if op == "icmp":
            oty = inst.attr["oty"]; bits = _bits(oty); p = inst.attr["pred"]
            a, b = get(inst.args[0]), get(inst.args[1])
            if p[0] == "s" and not _is_ptr(oty):
                a, b = _signed(a, bits), _signed(b, bits)
            else:
                a, b = _wrap(a, bits), _wrap(b, bits)
            return int({"eq": a == b, "ne": a != b, "lt": a < b, "le": a <= b, "gt": a > b,
                        "ge": a >= b}[p if p in ("eq", "ne") else p[1:]])
        if op == "fcmp":
            a, b = np.float64(get(inst.args[0])), np.float64(get(inst.args[1]))
            nan = bool(np.isnan(a) or np.isnan(b)); p = inst.attr["pred"]
            if p == "ord":
                return int(not nan)
            if p == "uno":
                return int(nan)
            if nan:
                return 0
            return int({"oeq": a == b, "one": a != b, "olt": a < b, "ole": a <= b, "ogt": a > b,
                        "oge": a >= b}[p])
        if op == "select":
            c = get(inst.args[0])
            return get(inst.args[1]) if c & 1 else get(inst.args[2])
        if op in _CAST:
            v = get(inst.args[0]); src = inst.attr["src"]
            sv = _vec(src)
            if vec:
                return [self._cast(op, vec[1], sv[1], x) for x in v]
            return self._cast(op, ty, src, v)
        if op == "load":
            addr = get(inst.args[0])
            if vec:
                return [_load_scalar(self.mem, addr + l * _SIZE[vec[1]], vec[1]) for l in range(vec[0])]
            return _load_scalar(self.mem, addr, ty)
        if op == "store":
            addr, v = get(inst.args[0]), get(inst.args[1]); sty = inst.attr["sty"]; sv = _vec(sty)
            if sv:
                for l in range(sv[0]):
                    _store_scalar(self.mem, addr + l * _SIZE[sv[1]], sv[1], v[l])
            else:
                _store_scalar(self.mem, addr, sty, v)
            return None
        if op in _INDEX:
            which, dim = op.split(".")
            v = {"tid": tid if dim == "x" else 0, "bid": 0, "bdim": nthreads if dim == "x" else 1,
                 "gdim": 1}[which]
            return _wrap(v, _bits(ty))
        if op == "barrier":
            return None
        if op == "vec.extract":
            return get(inst.args[0])[inst.attr["lane"]]
        if op == "vec.build":
            return [get(a) for a in inst.args]
        if op in _SHUFFLE or op in ("ballot", "vote.any", "vote.all") or op.startswith("warp.reduce."):
            raise OracleRefusal("E090", f"{op} is warp-collective; the oracle runs one thread at a time")
        if op in _ATOMIC:
            addr, v = get(inst.args[0]), get(inst.args[1])
            old = _load_scalar(self.mem, addr, ty)
            kind = op.split(".")[1]
            if ty in _FLOATS:
                f = _FLOATS[ty]
                new = {"add": lambda: f(old + f(v)), "sub": lambda: f(old - f(v)), "exch": lambda: f(v),
                       "min": lambda: min(old, f(v)), "max": lambda: max(old, f(v))}[kind]()
            else:
                bits = _bits(ty)
                so, sv_ = _signed(old, bits), _signed(v, bits)
                new = {"add": old + v, "sub": old - v, "exch": v, "min": min(so, sv_), "max": max(so, sv_),
                       "and": old & v, "or": old | v, "xor": old ^ v}[kind]
                new = _wrap(new, bits)
            _store_scalar(self.mem, addr, ty, new)
            return old
        if op == "atomic.cas":
            addr, cmp_, new = (get(a) for a in inst.args)
            old = _load_scalar(self.mem, addr, ty)
            if _wrap(old, _bits(ty)) == _wrap(cmp_, _bits(ty)):
                _store_scalar(self.mem, addr, ty, new)
            return old
        if op == "mma":
            self._mma(inst, get)
            return None
        if op == "call":
            callee = self.funcs[inst.attr["callee"]]
            if callee.is_kernel:
                raise OracleRefusal("E093", "a kernel is launched, never called")
            return self.run(callee, [get(a) for a in inst.args], tid, nthreads, depth + 1)
        raise ValueError(op)

    def _bin(self, op, ty, a, b):
        if op in ("fadd", "fsub", "fmul", "fdiv", "frem"):
            return _fbin(op, ty, a, b)
        bits = _bits(ty)
        if op == "add":
            return _wrap(a + b, bits)
        if op == "sub":
            return _wrap(a - b, bits)
        if op == "mul":
            return _wrap(a * b, bits)
        if op in ("div", "rem"):
            sa, sb = _signed(a, bits), _signed(b, bits)
            if sb == 0:
                raise ZeroDivisionError("integer division by zero traps on x86")
            q = abs(sa) // abs(sb)
            if (sa < 0) != (sb < 0):
                q = -q
            return _wrap(q if op == "div" else sa - q * sb, bits)
        if op == "and":
            return a & b
        if op == "or":
            return a | b
        if op == "xor":
            return a ^ b
        cnt = b & (63 if bits == 64 else 31)   # x86 masks the count in cl
        if op == "shl":
            return _wrap(a << cnt, bits)
        if op == "lshr":
            return _wrap(a, bits) >> cnt
        if op == "ashr":
            return _wrap(_signed(a, bits) >> cnt, bits)
        raise ValueError(op)

    def _cast(self, op, dst, src, v):
        if op == "trunc":
            return _wrap(v, _bits(dst))
        if op == "zext":
            return _wrap(v, _bits(src))
        if op == "sext":
            return _wrap(_signed(v, _bits(src)), _bits(dst))
        if op in ("fptrunc", "fpext"):
            return _FLOATS[dst](v)
        if op in ("fptosi", "fptoui"):
            f = np.float64(v)
            if np.isnan(f) or np.isinf(f):
                return _wrap(1 << (_bits(dst) - 1), _bits(dst))   # x86 "integer indefinite"
            return _wrap(int(np.trunc(f)), _bits(dst))
        if op == "sitofp":
            return _FLOATS[dst](_signed(v, _bits(src)))
        if op == "uitofp":
            return _FLOATS[dst](_wrap(v, _bits(src)))
        if op == "bitcast":
            if dst in _FLOATS and src not in _FLOATS:
                n = _SIZE[dst]
                return np.frombuffer(int(v).to_bytes(n, "little"), dtype=_FLOATS[dst])[0]
            if src in _FLOATS and dst not in _FLOATS:
                return int.from_bytes(_FLOATS[src](v).tobytes(), "little")
            return v
        raise ValueError(op)

    def _mma(self, inst: Inst, get):
        at = inst.attr
        a, b, c, d = (get(x) for x in inst.args)
        m, n, k = at["m"], at["n"], at["k"]
        ity, aty = at["in"], at["acc"]
        oty = at.get("out", aty)
        lda, ldb, ldc, ldd = at.get("ld", [0, 0, 0, 0])
        lda = lda or (k if at["la"] == "row" else m)
        ldb = ldb or (n if at["lb"] == "row" else k)
        ldc = ldc or n
        ldd = ldd or n
        isz, asz, osz = _SIZE[ity], _SIZE[aty], _SIZE[oty]
        is_f = aty in _FLOATS
        for i in range(m):
            for j in range(n):
                acc = _FLOATS[aty](0) if is_f else 0
                for kk in range(k):
                    ao = (i * lda + kk) if at["la"] == "row" else (kk * lda + i)
                    bo = (kk * ldb + j) if at["lb"] == "row" else (j * ldb + kk)
                    av = _load_scalar(self.mem, a + ao * isz, ity)
                    bv = _load_scalar(self.mem, b + bo * isz, ity)
                    if is_f:
                        f = _FLOATS[aty]
                        acc = f(acc + f(f(av) * f(bv)))
                    else:
                        bits = _bits(aty)
                        acc = _wrap(acc + _signed(av, _bits(ity)) * _signed(bv, _bits(ity)), bits)
                cv = _load_scalar(self.mem, c + (i * ldc + j) * asz, aty) if c else (0 if not is_f else _FLOATS[aty](0))
                res = _FLOATS[aty](cv + acc) if is_f else _wrap(cv + acc, _bits(aty))
                _store_scalar(self.mem, d + (i * ldd + j) * osz, oty, res)


def run_kernel(bir_text: str, kernel: str, args: list, nthreads: int):
    """Runs `kernel` from the BIR text under the oracle's launch model.

    `args` holds one entry per kernel parameter: a numpy array (or any writable buffer) for a
    pointer parameter -- it is mapped into the launch's address space and modified in place --
    or a Python int / float for a scalar. Returns nothing; results are in the buffers.
    """
    module = parse(bir_text)
    mem = Memory()
    fn = {f.name: f for f in module.funcs}[kernel]
    vals = []
    for ty, a in zip(fn.params, args):
        if _is_ptr(ty):
            vals.append(mem.map(a) if a is not None else 0)
        elif ty in _FLOATS:
            vals.append(_FLOATS[ty](a))
        else:
            vals.append(_wrap(int(a), _bits(ty)))
    Interp(module, mem).launch(kernel, vals, nthreads)
