"""One-instruction kernels for the per-op differential tests: out[i] = op(a[i], b[i]) with i the global
thread index, for every integer width x binary op, every float compare and a table of casts, plus the
inputs that go with them.  The same text runs through the BIR interpreter, the restated x86-64 back end
and the emitted PTX."""
import numpy as np

NP = {"i8": np.int8, "i16": np.int16, "i32": np.int32, "i64": np.int64, "f32": np.float32, "f64": np.float64}
INT_TYPES = ("i8", "i16", "i32", "i64")
INT_BINOPS = ("add", "sub", "mul", "and", "or", "xor", "shl", "lshr", "ashr", "div", "rem")
FLOAT_BINOPS = ("fadd", "fsub", "fmul", "fdiv")
FCMP_PREDS = ("oeq", "one", "olt", "ole", "ogt", "oge", "ord", "uno")
ICMP_PREDS = ("eq", "ne", "slt", "sle", "sgt", "sge", "ult", "ule", "ugt", "uge")
CASTS = [("sext", "i8", "i32"), ("zext", "i8", "i32"), ("sext", "i16", "i64"), ("zext", "i16", "i64"), ("sext", "i32", "i64"),
         ("zext", "i32", "i64"), ("trunc", "i64", "i8"), ("trunc", "i32", "i16"), ("sitofp", "i32", "f32"), ("sitofp", "i64", "f64"),
         ("sitofp", "i8", "f32"), ("uitofp", "i32", "f32"), ("uitofp", "i64", "f64"), ("uitofp", "i64", "f32"), ("uitofp", "i16", "f64"),
         ("fptosi", "f32", "i32"), ("fptosi", "f64", "i64"), ("fptoui", "f32", "i32"), ("fptoui", "f64", "i64"), ("fptoui", "f32", "i64"),
         ("fpext", "f32", "f64"), ("fptrunc", "f64", "f32"), ("bitcast", "f32", "i32"), ("bitcast", "i64", "f64")]


def module(body: str, target="i32") -> str:
    return f"module {{\n  shared_mem_bytes 0\n  target_dtypes {target}\n\n{body}}}\n"


_INDEX = """    %0 = bid.x i64
    %1 = bdim.x i64
    %2 = mul i64 %0, %1
    %3 = tid.x i64
    %4 = add i64 %2, %3
"""


def size(ty: str) -> int:
    return np.dtype(NP[ty]).itemsize


def binop_kernel(ty: str, op: str) -> str:
    sz = size(ty)
    return module(f"""  func @k(ptr.global, ptr.global, ptr.global) -> void {{
  bb0:
{_INDEX}    %5 = const.i i64 {sz}
    %6 = mul i64 %4, %5
    %7 = add ptr.global %arg0, %6
    %8 = load {ty} ptr.global %7, align {sz}
    %9 = add ptr.global %arg1, %6
    %10 = load {ty} ptr.global %9, align {sz}
    %11 = {op} {ty} %8, %10
    %12 = add ptr.global %arg2, %6
    store {ty} ptr.global %12, %11, align {sz}
    ret
  }}
""")


def compare_kernel(ty: str, pred: str) -> str:
    """out[i] (i32) = zext(a[i] <pred> b[i]); icmp for integer types, fcmp for float types."""
    sz = size(ty)
    op = "fcmp" if ty.startswith("f") else "icmp"
    return module(f"""  func @k(ptr.global, ptr.global, ptr.global) -> void {{
  bb0:
{_INDEX}    %5 = const.i i64 {sz}
    %6 = mul i64 %4, %5
    %7 = add ptr.global %arg0, %6
    %8 = load {ty} ptr.global %7, align {sz}
    %9 = add ptr.global %arg1, %6
    %10 = load {ty} ptr.global %9, align {sz}
    %11 = {op} {pred} {ty} %8, %10
    %12 = zext i32 i1 %11
    %13 = const.i i64 4
    %14 = mul i64 %4, %13
    %15 = add ptr.global %arg2, %14
    store i32 ptr.global %15, %12, align 4
    ret
  }}
""")


def select_kernel(ty: str) -> str:
    """out[i] = a[i] < b[i] ? a[i] : b[i] through `select` (signed / ordered less-than)."""
    sz = size(ty)
    cmp = f"fcmp olt {ty}" if ty.startswith("f") else f"icmp slt {ty}"
    return module(f"""  func @k(ptr.global, ptr.global, ptr.global) -> void {{
  bb0:
{_INDEX}    %5 = const.i i64 {sz}
    %6 = mul i64 %4, %5
    %7 = add ptr.global %arg0, %6
    %8 = load {ty} ptr.global %7, align {sz}
    %9 = add ptr.global %arg1, %6
    %10 = load {ty} ptr.global %9, align {sz}
    %11 = {cmp} %8, %10
    %12 = select {ty} %11, %8, %10
    %13 = add ptr.global %arg2, %6
    store {ty} ptr.global %13, %12, align {sz}
    ret
  }}
""")


def cast_kernel(op: str, src: str, dst: str) -> str:
    ssz, dsz = size(src), size(dst)
    return module(f"""  func @k(ptr.global, ptr.global) -> void {{
  bb0:
{_INDEX}    %5 = const.i i64 {ssz}
    %6 = mul i64 %4, %5
    %7 = add ptr.global %arg0, %6
    %8 = load {src} ptr.global %7, align {ssz}
    %9 = {op} {dst} {src} %8
    %10 = const.i i64 {dsz}
    %11 = mul i64 %4, %10
    %12 = add ptr.global %arg1, %11
    store {dst} ptr.global %12, %9, align {dsz}
    ret
  }}
""")


def int_inputs(ty: str, op: str, n: int, seed: int = 7):
    """Operands for an integer binary op: full range, the extremes planted, shift counts inside the type's
    width, no division by zero and no INT_MIN / -1 (x86 traps on both)."""
    rng = np.random.default_rng(seed)
    bits = size(ty) * 8
    info = np.iinfo(NP[ty])
    a = rng.integers(info.min, info.max, n, dtype=NP[ty], endpoint=True)
    b = rng.integers(info.min, info.max, n, dtype=NP[ty], endpoint=True)
    a[:4] = [info.min, info.max, -1, 0]
    if op in ("shl", "lshr", "ashr"):
        b = (b.astype(np.int64) % bits).astype(NP[ty])
    if op in ("div", "rem"):
        b[b == 0] = 3
        b[(a == info.min) & (b == -1)] = 5
    return a, b


def float_inputs(ty: str, n: int, seed: int = 11):
    rng = np.random.default_rng(seed)
    a = (rng.standard_normal(n) * 100).astype(NP[ty]); b = (rng.standard_normal(n) * 10).astype(NP[ty])
    a[:3] = [0.0, np.inf, np.nan]; b[:3] = [-0.0, 1.0, 2.0]; b[5] = np.nan
    a[8:12] = b[8:12]      # equal pairs for the equality predicates
    return a, b


def cast_inputs(op: str, src: str, dst: str, n: int, seed: int = 13):
    """In-range values only for float -> integer (out-of-range results differ between ISAs by design)."""
    rng = np.random.default_rng(seed)
    if src.startswith("f"):
        lim = 2.0**31 - 256 if dst == "i32" else 2.0**62
        a = (rng.random(n) * lim).astype(NP[src])
        if op == "fptosi":
            a[::2] *= -1
        if op == "fptoui" and dst == "i64":
            a[:8] = NP[src](2.0**63) + (np.arange(8) * 2.0**40).astype(NP[src])      # the path above 2^63
        return a
    info = np.iinfo(NP[src])
    a = rng.integers(info.min, info.max, n, dtype=NP[src], endpoint=True)
    a[:3] = [info.min, info.max, -1]
    return a
