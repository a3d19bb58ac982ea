"""The Backend contract (crates/basalt-backend/src/backend.rs:144-157): name, supports and emit
share one refusal function, refusals carry the reference's E-codes, output is deterministic.
Modelled on the reference emitter's own tests (crates/basalt-ptx/src/emit/tests.rs:43-831)."""
import shutil
import subprocess

import pytest

import basalt_b200 as b
from basalt_b200 import kernels_bir as kb
from basalt_b200.birasm import assemble


def kernel(body: str, params: str = "ptr.global, i32, i32, f32, f32", extra: str = "", name: str = "k") -> str:
    return assemble(f"module {{\n  shared_mem_bytes 0\n  target_dtypes\n{extra}\n  func @{name}({params}) -> void {{\n  entry:\n{body}\n    ret\n  }}\n}}\n")


def emit0(ptx, src):
    return ptx.emit(src, b.EmitOpts(opt_level=0)).text


def test_name_and_preamble(ptx):
    assert ptx.name() == "nvidia-ptx-sm100"
    text = emit0(ptx, kernel("", params=""))
    assert ".version 8.7\n" in text and ".target sm_100a\n" in text and ".address_size 64\n" in text
    assert ".visible .entry k()" in text


def test_bin_arithmetic_mnemonics(ptx):
    body = "\n".join(f"    %v{i} = {op} i32 %arg1, %arg2" for i, op in enumerate(("add", "sub", "mul", "div", "rem", "and", "shl", "ashr", "lshr")))
    body += "\n    %f0 = fadd f32 %arg3, %arg4\n    %f1 = fdiv f32 %arg3, %arg4\n    %f2 = frem f32 %arg3, %arg4\n    %f3 = fmul f32 %arg3, %arg4"
    text = emit0(ptx, kernel(body))
    for want in ("add.s32", "sub.s32", "mul.lo.s32", "div.s32", "rem.s32", "and.b32", "shl.b32", "shr.s32", "shr.u32",
                 "add.rn.f32", "div.rn.f32", "mul.rn.f32", "cvt.rzi.f32.f32"):
        assert want in text, want
    assert "fma" not in text   # multiply and add stay separate: the oracle never fuses


def test_i64_and_pointer_arithmetic_share_the_64_bit_class(ptx):
    text = emit0(ptx, kernel("    %o = const.i i64 8\n    %p = add ptr.global %arg0, %o\n    %v = load i32 ptr.global %p, align 4"))
    assert "add.s64" in text and "ld.global.u32" in text


def test_compares_and_casts(ptx):
    body = """    %a = icmp slt i32 %arg1, %arg2
    %b = icmp ult i32 %arg1, %arg2
    %c = fcmp olt f32 %arg3, %arg4
    %d = fcmp uno f32 %arg3, %arg4
    %e = sext i64 i32 %arg1
    %f = sitofp f32 i32 %arg1
    %g = fptosi i32 f32 %arg3
    %h = bitcast i32 f32 %arg3
    %i = trunc i8 i32 %arg1
    %j = zext i32 i8 %i
    %k = fptrunc f16 f32 %arg3
    %l = fpext f32 f16 %k"""
    text = emit0(ptx, kernel(body))
    for want in ("setp.lt.s32", "setp.lt.u32", "setp.lt.f32", "setp.nan.f32", "cvt.s64.s32", "cvt.rn.f32.s32", "cvt.rzi.s32.f32",
                 "mov.b32", "bfe.s32", "cvt.rn.f16.f32", "cvt.f32.f16"):
        assert want in text, want


def test_load_store_cover_every_address_space(ptx):
    # volatile keeps the local/param/constant cells in memory (non-volatile ones are promoted to SSA values)
    for space, word in (("global", "global"), ("shared", "shared"), ("local", "local"), ("constant", "local"), ("param", "local")):
        body = f"    %p = const.i ptr.{space} 65536\n    %v = load i32 ptr.{space} %p, align 4, volatile\n    store i32 ptr.{space} %p, %v, align 4, volatile"
        text = emit0(ptx, kernel(body))
        assert f"ld.volatile.{word}.u32" in text and f"st.volatile.{word}.u32" in text, space


def test_sized_shared_object_becomes_an_array(ptx):
    body = "    %p = const.i ptr.shared 0\n    %v = load i32 ptr.shared %p, align 4"
    assert ".shared .align 8 .b8 __shared_0[8];" in emit0(ptx, kernel(body))
    text = emit0(ptx, kernel(body, extra="  shared_obj 0 bytes 1024 align 16").replace("target_dtypes\n  shared_obj", "target_dtypes\n  shared_obj"))
    assert ".shared .align 16 .b8 __shared_0[1024];" in text


def test_index_ops_barrier_shuffles_votes(ptx):
    regs = {"tid": "%tid", "bid": "%ctaid", "bdim": "%ntid", "gdim": "%nctaid"}
    body = "\n".join(f"    %{a}{d} = {a}.{d} i32" for a in regs for d in "xyz")
    body += "\n    %w = bid.x i64\n    barrier"
    body += "".join(f"\n    %s{k} = shuffle.{k} i32 %tidx, %tidy" for k in ("idx", "up", "down", "xor"))
    body += "\n    %l = sext i64 i32 %tidx\n    %s64 = shuffle.idx i64 %l, %tidy"
    body += "\n    %bal = ballot i32 %tidx\n    %any = vote.any i32 %tidx\n    %p = icmp eq i32 %tidx, %tidy\n    %all = vote.all i1 %p"
    text = emit0(ptx, kernel(body))
    for a, r in regs.items():
        for d in "xyz":
            assert f"{r}.{d};" in text
    for want in ("cvt.u64.u32", "bar.sync 0;", "shfl.sync.idx.b32", "shfl.sync.up.b32", "shfl.sync.down.b32", "shfl.sync.bfly.b32",
                 "mov.b64", "vote.sync.ballot.b32", "vote.sync.any.pred", "vote.sync.all.pred", "0xffffffff"):
        assert want in text, want


def test_atomics(ptx):
    ops = ("add", "sub", "exch", "min", "max", "and", "or", "xor")
    body = "\n".join(f"    %o{o} = atomic.{o} i32 ptr.global %arg0, %arg1" for o in ops)
    body += "\n    %c = atomic.cas i32 ptr.global %arg0, %arg1, %arg2"
    body += "\n" + "\n".join(f"    %u{o} = add i32 %o{o}, %c" for o in ops)   # keep every result live
    body += "\n    %fm = atomic.min f32 ptr.global %arg0, %arg3\n    %fu = fadd f32 %fm, %arg3"
    text = emit0(ptx, kernel(body))
    for want in ("atom.global.add.u32", "neg.s32", "atom.global.exch.b32", "atom.global.min.s32", "atom.global.max.s32",
                 "atom.global.and.b32", "atom.global.or.b32", "atom.global.xor.b32", "atom.global.cas.b32", "min.f32", "bra $atomic_fminmax_loop"):
        assert want in text, want
    unused = emit0(ptx, kernel("    %o = atomic.max i32 ptr.global %arg0, %arg1"))
    assert "red.global.max.s32" in unused and "atom." not in unused


def test_vector_load_store(ptx):
    body = "    %v = load v4f32 ptr.global %arg0, align 16\n    %s = fadd v4f32 %v, %v\n    store v4f32 ptr.global %arg0, %s, align 16"
    text = emit0(ptx, kernel(body))
    assert "ld.global.v4.f32 {" in text and "st.global.v4.f32 [" in text and text.count("add.rn.f32") == 4
    body3 = "    %v = load v3f32 ptr.global %arg0, align 4\n    store v3f32 ptr.global %arg0, %v, align 4"
    text3 = emit0(ptx, kernel(body3))
    assert ".v3." not in text3 and "+4]" in text3 and "+8]" in text3


def test_phi_moves_sit_on_the_incoming_edge(ptx):
    text = emit0(ptx, b.roundtrip(open("/dev/null").read() or __import__("test_bir_roundtrip").HAND_WRITTEN))
    assert "\tret;\n" in text and "mov.b32" in text and "@%p" in text


def test_optimised_lowering_uses_the_blackwell_forms(ptx):
    v = ptx.emit(kb.load("vadd_i32")).text
    assert "ld.global.v4.u32" in v and "st.global.v4.u32" in v and "elementwise lanes=4" in v
    m = ptx.emit(kb.load("max_i32")).text
    assert "redux.sync.max.s32" in m and "red.global.max.s32" in m and "ld.global.v4.u32" in m and "shfl" not in m
    assert ".maxntid 256, 1, 1" in m
    h = ptx.emit(kb.helper_chain()).text
    assert "call" not in h and h.count(".entry") == 2 and "helper_chain__coarse" in h and "ld.global.v4.u32" in h
    h0 = emit0(ptx, kb.helper_chain())
    assert h0.count("mul.lo.s32") == 33 and "v4" not in h0   # 32 squarings plus the index product


def test_power_of_two_products_are_shifts_and_entries_admit_dependent_launch(ptx):
    # a multiply by a constant power of two is a shift (ptxas would keep mul.lo on the multiply-add pipe); any other
    # constant, and a product of two values, stay multiplies
    body = ("    %c16 = const.i i64 16\n    %c12 = const.i i64 12\n    %w = sext i64 i32 %arg1\n    %a = mul i64 %w, %c16\n    %b = mul i64 %c16, %w\n"
            "    %c = mul i64 %w, %c12\n    %c8 = const.i i32 8\n    %d = mul i32 %arg1, %c8\n    %e = mul i32 %arg1, %arg2\n"
            "    %s = add i64 %a, %b\n    %t = add i64 %s, %c\n    %p = add ptr.global %arg0, %t\n    %de = add i32 %d, %e\n    store i32 ptr.global %p, %de, align 4")
    text = emit0(ptx, kernel(body))
    assert text.count("shl.b64") == 2 and text.count("shl.b32") == 1 and text.count("mul.lo.s64") == 1 and text.count("mul.lo.s32") == 1
    # every entry begins with the programmatic-dependent-launch pair, and only coarse entries are planned for it
    v = ptx.emit(kb.load("vadd_i32")).text
    assert v.count("griddepcontrol.launch_dependents;") == v.count(".entry") == v.count("griddepcontrol.wait;") == 2
    plan = [l for l in v.splitlines() if l.startswith("//!basalt.plan")]
    assert plan[0] == "//!basalt.plan vadd_i32 pdl=1" and len(plan) == 2      # the later line of the same kernel is the one the runtime keeps
    assert "coarse=vadd_i32__coarse" in plan[1] and plan[1].endswith("pdl=1")
    assert "//!basalt.plan max_i32 pdl=1" in ptx.emit(kb.load("max_i32")).text
    for entry in v.split(".entry")[1:]:
        first_access = min(entry.index(op) for op in ("ld.global", "st.global") if op in entry)
        assert entry.index("griddepcontrol.wait;") < first_access


def test_emit_is_deterministic(ptx):
    for src in (kb.load("max_i32"), kb.helper_chain(), kb.load("sgemm_tile16"), kb.matmul_f16(256, 256, 128)):
        assert ptx.emit(src).text == ptx.emit(src).text


CALL = """module {{
  shared_mem_bytes 0
  target_dtypes
{funcs}
}}
"""
F_KERNEL = "\n  func @k(i32) -> void {\n  bb0:\n    %0 = call i32 @a [%arg0]\n    ret\n  }\n"
F_A_CALLS_B = "\n  host func @a(i32) -> i32 {\n  bb0:\n    %0 = call i32 @b [%arg0]\n    ret %0\n  }\n"
F_B_CALLS_A = "\n  host func @b(i32) -> i32 {\n  bb0:\n    %0 = call i32 @a [%arg0]\n    ret %0\n  }\n"
F_B_LEAF = "\n  host func @b(i32) -> i32 {\n  bb0:\n    ret %arg0\n  }\n"
F_ORPHAN = "\n  host func @orphan(i32) -> i32 {\n  bb0:\n    ret %arg0\n  }\n"
F_A_CALLS_K = "\n  host func @a(i32) -> i32 {\n  bb0:\n    call void @k [%arg0]\n    ret %arg0\n  }\n"


@pytest.mark.parametrize("src, code", [
    (CALL.format(funcs=F_KERNEL + F_A_CALLS_B + F_B_CALLS_A), "E094"),      # cycle
    (CALL.format(funcs=F_KERNEL + F_A_CALLS_B + F_B_LEAF + F_ORPHAN), "E095"),   # unreachable helper
    (CALL.format(funcs=F_KERNEL + F_A_CALLS_K), "E093"),                    # a kernel is never called
    (CALL.format(funcs=F_B_LEAF), "E093"),                                  # no kernel at all
    (kernel("    %m = cuda.malloc ptr.global %arg1", params="ptr.global, i64"), "E090"),
    (kernel("    cuda.device_sync"), "E090"),
    (kernel("    %c = icmp eq v4i32 %arg0, %arg0", params="v4i32"), "E091"),
    (kernel("    %p = icmp eq i32 %arg1, %arg2\n    %c = bitcast i8 i1 %p"), "E091"),
    (kernel("    %p = icmp eq i32 %arg1, %arg2\n    %c = add i1 %p, %p"), "E090"),
    (kernel("    %t = trunc i16 i32 %arg1\n    %c = atomic.add i16 ptr.global %arg0, %t"), "E091"),
    (kernel("    %p = icmp eq i32 %arg1, %arg2\n    %c = shuffle.idx i1 %p, %arg1"), "E091"),
    (kernel("    %c = const.i v4i32 1"), "E091"),
    (kernel("    mma i32 f32 row row m 2 n 2 k 2 %arg0, %arg0, %arg0, %arg0"), "E091"),
])
def test_refusals_carry_reference_codes(ptx, src, code):
    assert ptx.supports(src) == b.Support(False, code)
    with pytest.raises(b.Diag) as e:
        ptx.emit(src)
    assert e.value.code == code


def test_things_the_reference_refuses_and_this_backend_lowers(ptx):
    # crates/basalt-ptx/src/emit.rs:357-376, 469-475, 503-509: f16 E091, mma E090, call E090 there
    for src in (kb.load("chain_vector"), kb.load("mma2x2"), kb.matmul_f16(128, 128, 64),
                kernel("    %h = fptrunc f16 f32 %arg3\n    %s = fadd f16 %h, %h\n    store f16 ptr.global %arg0, %s, align 2")):
        assert ptx.supports(src).supported
        assert ".entry" in ptx.emit(src).text


def test_unknown_target_variant_is_refused(ptx):
    with pytest.raises(b.Diag) as e:
        ptx.emit(kb.load("vadd_i32"), b.EmitOpts(target_variant="gfx1100"))
    assert e.value.code == "E093"
    assert ptx.emit(kb.load("vadd_i32"), b.EmitOpts(target_variant="sm_100a")).kind == "ptx"


@pytest.mark.skipif(shutil.which("ptxas") is None, reason="ptxas not installed")
@pytest.mark.parametrize("level", [0, 2])
def test_every_kernel_assembles_for_sm_100a(ptx, tmp_path, level):
    srcs = {n: kb.load(n) for n in kb.STATIC}
    srcs.update(helper_chain=kb.helper_chain(), stress=kb.stress(), sgemm=kb.sgemm_cta128(256, 256, 64),
                matmul=kb.matmul_f16(256, 256, 128), matmul_nk=kb.matmul_f16(256, 256, 128, True))
    for name, src in srcs.items():
        p = tmp_path / f"{name}.ptx"
        p.write_text(ptx.emit(src, b.EmitOpts(opt_level=level)).text)
        r = subprocess.run(["ptxas", "-arch=sm_100a", str(p), "-o", "/dev/null"], capture_output=True, text=True)
        assert r.returncode == 0, f"{name}: {r.stderr}"


def test_tiled_fp16_matmul_gets_a_two_sm_twin(ptx):
    # the persistent tcgen05 form is emitted twice: `<name>` for one SM per tile and `<name>__pair` for clusters
    # of two (the plan's `pair=` key tells the runtime, which takes it on grids that are even in x and y)
    for nk in (False, True):
        text = ptx.emit(kb.matmul_f16(512, 512, 256, nk)).text
        plans = [l for l in text.splitlines() if l.startswith("//!basalt.plan")]
        assert len(plans) == 1 and " lgrid=2 " in plans[0] and " pair=matmul_kernel__pair " in plans[0] and plans[0].endswith("gather=2")   # output = parameter 2
        one, two = text.split(".visible .entry matmul_kernel__pair")
        assert ".visible .entry matmul_kernel(" in one and ".reqnctapercluster" not in one
        assert ".reqnctapercluster 2, 1, 1" in two and two.count("tcgen05.mma.cta_group::2.kind::f16") == 4
        assert "tcgen05.alloc.cta_group::2" in two and "tcgen05.dealloc.cta_group::2" in two and two.count("barrier.cluster.arrive") == 2
        # both entries take the same argument list: the runtime launches either with one set of tensor maps
        params = lambda t: [l.strip().rstrip(",").split()[-1].split("_", 2)[-1] for l in t.split(")")[0].splitlines() if ".param" in l]
        # (the twin takes two more: the peer table and count of the gathering epilogue)
        two_params = [p.replace("_pair_", "", 1) if p.startswith("_pair_") else p for p in params(two)]
        assert params(one.split(".visible .entry matmul_kernel(")[1]) == two_params[:-2] and "peers[56]" in two_params[-2] and "npeers" in two_params[-1]
        assert "fence.acq_rel.sys" in two and two.count("st.global.v4.b32") == 12      # eight line stores locally, four rows per peer in the relay warps
        assert ".maxntid 256" in two and " pair_block=256 " in plans[0] and two.count("ld.global.cg.v4.b32") == 4
        # bulk-tensor loads never multicast: a cta_group::2 load names the leader's barrier by address instead
        for line in text.splitlines():
            if "cp.async.bulk" in line:
                assert "multicast" not in line, line
        # every wait in the twin is bounded: each try_wait loop reads the clock and can leave through the give-up flag
        assert two.count("mbarrier.try_wait.parity") == two.count("setp.lt.u64") - 2    # + the 2 ms drain of the producer and the relay warps' bounded wait for a stored tile
