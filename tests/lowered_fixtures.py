"""Hand-lowered modules of the reference's test programs (test data, not a test).

Each function returns the `lowering.GpuModule`s that the reference's pipeline would hand to its renderer for the hexpr
program cited — derived by hand from the lowering rules (SSA order of the definition's operations, products flattened
into separate wires, erased type-level wires kept as `erased` variables, closures converted to an environment plus a
function symbol: catena-lang/src/codegen/mod.rs:107-146, 229-330; src/codegen/ops/ifc.rs, reducec.rs;
tests/compile/closures/reduce.rs:30-60 for the component sizes of `reducec`).  The Rust front end cannot run here,
so variable names and closure symbols are this file's own; the operations, their order and the component sizes are
the reference's.
"""
from catena_lang_b200.lowering import FnSymbol, GpuAssign, GpuFunction, GpuModule, GpuVar
from catena_lang_b200 import symbol_for


def v(name, lowered):
    return GpuVar(name, lowered)


def fn(name):
    return FnSymbol(name)


def A(op, ins=(), outs=(), in_sizes=None, out_sizes=None, call=None):
    return GpuAssign(op, list(ins), list(outs), call, list(in_sizes) if in_sizes is not None else None,
                     list(out_sizes) if out_sizes is not None else None)


def M(source_name, sources, targets, assigns, name=None):
    sym = name or symbol_for(source_name)
    return GpuModule(sym, source_name, GpuFunction(sym, list(sources), list(targets), list(assigns)))


def closure(name, sources, targets, assigns=()):
    """A generated closure body: an internal module without a source name."""
    return GpuModule(name, None, GpuFunction(name, list(sources), list(targets), list(assigns)))


# ---------------------------------------------------------------- tests/runtime.rs:37-128 (bool programs)
def bool_programs():
    b = lambda n: v(n, "bool")                                               # noqa: E731
    return [
        M("not", [b("x0")], [b("x1")], [A("bool.not", [b("x0")], [b("x1")])]),
        # {defer (name.bool.not lift)} compose run: the composed closure applied at once is one `eval` of the symbol
        M("not-via-function-value", [b("x0")], [b("x1")], [A("eval", [b("x0"), fn("bool.not")], [b("x1")])]),
        M("bool-ifc-primitives", [b("flag"), b("arg")], [b("r")], [
            A("bool.t", [], [b("t0")]), A("bool.t", [], [b("t1")]),
            A("bool.ifc", [b("t0"), fn("bool.and"), b("t1"), fn("bool.or"), b("flag"), b("arg")], [b("r")], [1, 1, 1, 1, 1, 1], [1])]),
        M("copy-via-function-value", [], [b("l"), b("r")], [
            A("bool.t", [], [b("t")]), A("eval", [b("t"), fn("bool.copy")], [b("l"), b("r")])]),
    ]


# ---------------------------------------------------------------- tests/runtime.rs:170-331 (u64 / u32 / f32 arithmetic)
def arithmetic_programs():
    out = []
    for ty, name in (("u64", "two-times-two-u64"), ("u32", "two-times-two-u32"), ("f32", "two-times-two-f32")):
        t = lambda n: v(n, ty)                                               # noqa: E731
        out.append(M(name, [], [t("x3")], [A(f"{ty}.one", [], [t("x0")]), A(f"{ty}.one", [], [t("x1")]),
                                            A(f"{ty}.add", [t("x0"), t("x1")], [t("x2")]),
                                            A(f"{ty}.mul", [t("x2"), t("x2")], [t("x3")])]))
    u = lambda n: v(n, "u64")                                                # noqa: E731
    out.append(M("sub-basic", [], [u("r")], [A("u64.one", [], [u("a")]), A("u64.one", [], [u("b")]), A("u64.add", [u("a"), u("b")], [u("two")]),
                                             A("u64.one", [], [u("c")]), A("u64.sub", [u("two"), u("c")], [u("r")])]))
    for op in ("ne", "lt", "lte", "gte"):
        out.append(M(f"u64-{op}-test", [], [v("r", "bool")], [
            A("const.u64.0x0000000000000002", [], [u("lhs")]), A("const.u64.0x0000000000000003", [], [u("rhs")]),
            A(f"u64.{op}", [u("lhs"), u("rhs")], [v("r", "bool")])]))
    f = lambda n: v(n, "f32")                                                # noqa: E731
    out.append(M("fma-basic", [], [f("r")], [A("f32.one", [], [f("a")]), A("f32.one", [], [f("b")]), A("f32.one", [], [f("c")]),
                                             A("f32.fma", [f("a"), f("b"), f("c")], [f("r")])]))
    out.append(M("fma-fused-bits", [f("a"), f("b"), f("c")], [v("bits", "u32")], [
        A("f32.fma", [f("a"), f("b"), f("c")], [f("r")]), A("f32.bitcast-u32", [f("r")], [v("bits", "u32")])]))
    # the unfused counterpart (`f32.mul` then `f32.add`), for the pair of bit patterns of tests/runtime.rs:333-343
    out.append(M("mul-add-bits", [f("a"), f("b"), f("c")], [v("bits", "u32")], [
        A("f32.mul", [f("a"), f("b")], [f("p")]), A("f32.add", [f("p"), f("c")], [f("r")]), A("f32.bitcast-u32", [f("r")], [v("bits", "u32")])]))
    return out


# ---------------------------------------------------------------- tests/runtime.rs:408-740 (bitcasts, shifts, bitwise, compares, constants)
def bit_programs():
    w = lambda n: v(n, "u32")                                                # noqa: E731
    f = lambda n: v(n, "f32")                                                # noqa: E731
    out = [
        M("bitcast-one", [], [f("r")], [A("const.u32.0x3F800000", [], [w("c")]), A("u32.bitcast-f32", [w("c")], [f("r")])]),
        M("bitcast-one-bits", [], [w("r")], [A("f32.one", [], [f("o")]), A("f32.bitcast-u32", [f("o")], [w("r")])]),
        M("shift-and-sub", [], [w("r")], [
            A("const.u32.0x00000020", [], [w("lhs")]), A("const.u32.0x00000003", [], [w("shift")]), A("const.u32.0x00000001", [], [w("one")]),
            A("u32.shr", [w("lhs"), w("shift")], [w("shr")]), A("u32.shl", [w("one"), w("shift")], [w("shl")]),
            A("u32.sub", [w("shr"), w("shl")], [w("r")])]),
        M("u32-not-test", [], [w("r")], [A("const.u32.0x00FF00FF", [], [w("x")]), A("u32.not", [w("x")], [w("r")])]),
        M("deadbeef", [], [v("r", "u64")], [A("const.u64.0xDEADBEEFDEADBEEF", [], [v("r", "u64")])]),
        M("deadbeef32", [], [w("r")], [A("const.u32.0xDEADBEEF", [], [w("r")])]),
    ]
    for op in ("and", "or", "xor"):
        out.append(M(f"u32-{op}-test", [], [w("r")], [A("const.u32.0x00FF00FF", [], [w("lhs")]), A("const.u32.0x0F0F0F0F", [], [w("rhs")]),
                                                       A(f"u32.{op}", [w("lhs"), w("rhs")], [w("r")])]))
    for op in ("eq", "ne", "lt", "gt", "lte", "gte"):
        out.append(M(f"u32-{op}-test", [], [v("r", "bool")], [A("const.u32.0x00000002", [], [w("lhs")]), A("const.u32.0x00000003", [], [w("rhs")]),
                                                               A(f"u32.{op}", [w("lhs"), w("rhs")], [v("r", "bool")])]))
        out.append(M(f"f32-{op}-test", [], [v("r", "bool")], [
            A("const.u32.0x3FC00000", [], [w("lb")]), A("u32.bitcast-f32", [w("lb")], [f("lhs")]),
            A("const.u32.0x40200000", [], [w("rb")]), A("u32.bitcast-f32", [w("rb")], [f("rhs")]),
            A(f"f32.{op}", [f("lhs"), f("rhs")], [v("r", "bool")])]))
    return out


# ---------------------------------------------------------------- tests/runtime.rs:713-740
def array_head_program():
    u = lambda n: v(n, "u64")                                                # noqa: E731
    e = lambda n: v(n, "erased")                                             # noqa: E731
    return [M("array-head-u64", [v("m", "mem")], [u("head")], [
        A("mem.cast.u64", [v("m", "mem")], [u("n"), v("buf", "ptr<u64>")]),
        # u64.assert-nz = ({[x] u64.zero} u64.gt [b ht hf. b ht] assert-then), assert-then = ({assert [h]} ax-mp)  (stdlib/data.hex:20-25, 131-135)
        A("u64.zero", [], [u("z")]), A("u64.gt", [u("n"), u("z")], [v("nz", "bool"), e("ht"), e("hf")]),
        A("assert", [v("nz", "bool")], [e("h")]), A("ax-mp", [e("h"), e("ht")], [e("proof")]),
        A("ix.zero", [e("proof")], [u("i0")]), A("ix", [u("i0"), v("buf", "ptr<u64>")], [u("head")])])]


# ---------------------------------------------------------------- tests/cases/reducec/basic.hex
def reducec_programs():
    u = lambda n: v(n, "u64")                                                # noqa: E731
    e = lambda n: v(n, "erased")                                             # noqa: E731
    p = lambda n: v(n, "ptr<u64>")                                           # noqa: E731
    add_env = M("u64.add-env", [u("acc"), u("value")], [u("r")], [A("u64.add", [u("acc"), u("value")], [u("r")])])
    sum_at = M("sum-u64-at", [p("input"), u("i")], [u("r")], [A("ix", [u("i"), p("input")], [u("r")])])
    sum_u64 = M("sum-u64", [v("m", "mem")], [u("r")], [
        A("mem.cast.u64", [v("m", "mem")], [u("len"), p("input")]),
        A("const.u64.0x0000000000000000", [], [u("zero")]), A("unit.intro", [], [e("unit")]),
        A("reducec", [u("zero"), e("unit"), fn("u64.add-env"), p("input"), fn("sum-u64-at"), u("len")], [u("r")], [1, 1, 1, 1, 1, 1], [1])])
    product_at = M("dot-u64-product-at", [p("lhs"), p("rhs"), u("i")], [u("r")], [
        A("ix", [u("i"), p("lhs")], [u("lval")]), A("ix", [u("i"), p("rhs")], [u("rval")]), A("u64.mul", [u("lval"), u("rval")], [u("r")])])
    same_len = M("mem.cast.u64.same-length", [v("a", "mem"), v("b", "mem")], [u("n"), p("lhs"), p("rhs2")], [
        A("mem.cast.u64", [v("a", "mem")], [u("n"), p("lhs")]), A("mem.cast.u64", [v("b", "mem")], [u("rn"), p("rhs")]),
        A("u64.eq", [u("n"), u("rn")], [v("eq", "bool"), e("if-eq"), e("if-ne")]),
        A("assert", [v("eq", "bool")], [e("h")]), A("ax-mp", [e("h"), e("if-eq")], [e("same")]),
        A("buf.u64.cast-same-length", [p("rhs"), e("same")], [p("rhs2")])])
    dot_u64 = M("dot-u64", [v("a", "mem"), v("b", "mem")], [u("r")], [
        A("mem.cast.u64.same-length", [v("a", "mem"), v("b", "mem")], [u("n"), p("lhs"), p("rhs")], call=same_len.name),
        A("const.u64.0x0000000000000000", [], [u("zero")]), A("unit.intro", [], [e("unit")]),
        A("reducec", [u("zero"), e("unit"), fn("u64.add-env"), p("lhs"), p("rhs"), fn("dot-u64-product-at"), u("n")], [u("r")],
          [1, 1, 1, 2, 1, 1], [1])])
    return [add_env, sum_at, sum_u64, product_at, same_len, dot_u64]


# ---------------------------------------------------------------- tests/cases/closures/conditionals.hex
def conditional_programs():
    f = lambda n: v(n, "f32")                                                # noqa: E731
    e = lambda n: v(n, "erased")                                             # noqa: E731
    keep = closure("program_closure_max_with_floor_0", [f("x")], [f("x")])            # ([.value] defer): returns its capture
    floor = closure("program_closure_max_with_floor_1", [f("x")], [f("x")])
    max_with_floor = M("max-with-floor", [f("value"), f("floor")], [f("r")], [
        A("f32.gte", [f("value"), f("floor")], [v("keep", "bool")]), A("unit.intro", [], [e("unit")]),
        A("bool.ifc", [f("value"), fn("closure.max-with-floor.0"), f("floor"), fn("closure.max-with-floor.1"), v("keep", "bool"), e("unit")],
          [f("r")], [1, 1, 1, 1, 1, 1], [1])])
    same = closure("program_closure_ordered_pair_0", [f("a"), f("b")], [f("a"), f("b")])   # ({[.lhs] [.rhs]} *.intro defer), flattened
    swap = closure("program_closure_ordered_pair_1", [f("a"), f("b")], [f("a"), f("b")])
    ordered_pair = M("ordered-pair", [f("lhs"), f("rhs")], [f("lo"), f("hi")], [
        A("f32.lte", [f("lhs"), f("rhs")], [v("ordered", "bool")]), A("unit.intro", [], [e("unit")]),
        A("bool.ifc", [f("lhs"), f("rhs"), fn("closure.ordered-pair.0"), f("rhs"), f("lhs"), fn("closure.ordered-pair.1"), v("ordered", "bool"),
                       e("unit")], [f("lo"), f("hi")], [2, 1, 2, 1, 1, 1], [2])])
    # a function symbol `closure.x.0` is called as `program_closure_x_0` (components.rs:100-105)
    return [keep, floor, max_with_floor, same, swap, ordered_pair]


# ---------------------------------------------------------------- tests/cases/closures/progression.hex, sequence_stats.hex
def progression_programs():
    u = lambda n: v(n, "u64")                                                # noqa: E731
    progression_at = M("progression-at", [u("base"), u("step"), u("i")], [u("r")], [
        A("ix.to-u64", [u("i")], [u("iu")]), A("u64.mul", [u("step"), u("iu")], [u("off")]), A("u64.add", [u("base"), u("off")], [u("r")])])
    progression_add = M("progression-add", [u("acc"), u("value")], [u("r")], [A("u64.add", [u("acc"), u("value")], [u("r")])])
    # the composed producer closure: (parameters, i) -> progression-at(parameters, i)
    producer = closure("program_closure_sum_progression_0", [u("base"), u("step"), u("i")], [u("r")], [
        A("progression-at", [u("base"), u("step"), u("i")], [u("r")], call=progression_at.name)])
    sum_progression = M("sum-progression", [u("len"), u("base"), u("step")], [u("r")], [
        A(":.ty", [u("len")], [u("reduce-len"), u("producer-len")]),
        A("const.u64.0x0000000000000000", [], [u("zero")]),
        A("reducec", [u("zero"), fn("progression-add"), u("base"), u("step"), fn("closure.sum-progression.0"), u("reduce-len")], [u("r")],
          [1, 0, 1, 2, 1, 1], [1])])
    moments_at = M("progression-moments-at", [u("base"), u("step"), u("i")], [u("value"), u("square")], [
        A("ix.to-u64", [u("i")], [u("iu")]), A("u64.mul", [u("step"), u("iu")], [u("off")]), A("u64.add", [u("base"), u("off")], [u("value")]),
        A("u64.mul", [u("value"), u("value")], [u("square")])])
    moments_add = M("progression-moments-add", [u("ls"), u("lq"), u("rs"), u("rq")], [u("s"), u("q")], [
        A("u64.add", [u("ls"), u("rs")], [u("s")]), A("u64.add", [u("lq"), u("rq")], [u("q")])])
    moments_producer = closure("program_closure_progression_moments_0", [u("base"), u("step"), u("i")], [u("value"), u("square")], [
        A("progression-moments-at", [u("base"), u("step"), u("i")], [u("value"), u("square")], call=moments_at.name)])
    moments = M("progression-moments", [u("len"), u("base"), u("step")], [u("sum"), u("squares")], [
        A(":.ty", [u("len")], [u("reduce-len"), u("producer-len")]),
        A("const.u64.0x0000000000000000", [], [u("z0")]), A("const.u64.0x0000000000000000", [], [u("z1")]),
        A("reducec", [u("z0"), u("z1"), fn("progression-moments-add"), u("base"), u("step"), fn("closure.progression-moments.0"), u("reduce-len")],
          [u("sum"), u("squares")], [2, 0, 1, 2, 1, 1], [2])])
    return [progression_at, progression_add, producer, sum_progression, moments_at, moments_add, moments_producer, moments]


def all_host_modules():
    return bool_programs() + arithmetic_programs() + bit_programs() + conditional_programs() + progression_programs()


# ---------------------------------------------------------------- examples/materializec.hex, tests/cases/materialize/basic.hex
def materialize_programs():
    u = lambda n: v(n, "u64")                                                # noqa: E731
    e = lambda n: v(n, "erased")                                             # noqa: E731
    p = lambda n: v(n, "ptr<u64>")                                           # noqa: E731
    # materialize-index-producer: ([env i.] u64.one) — unit environment, the index is not used
    one_producer = M("materialize-index-producer", [e("env"), u("i")], [u("r")], [A("u64.one", [], [u("r")])])
    indexes = M("materialize-indexes", [u("len")], [v("out", "mem")], [
        A("unit.intro", [], [e("unit")]), A(":.param", [u("len")], [e("n")]),
        A("materializec", [u("len"), e("unit"), fn("materialize-index-producer")], [p("buf")], [1, 1, 1], [1]),
        A("buf.to-mem", [u("len"), p("buf")], [v("out", "mem")])])
    # materialize-copy-u64-producer: ([input i.] {[.i input]} ix)
    copy_producer = M("materialize-copy-u64-producer", [p("input"), u("i")], [u("r")], [A("ix", [u("i"), p("input")], [u("r")])])
    copy = M("materialize-copy-u64", [v("m", "mem")], [v("out", "mem")], [
        A("mem.cast.u64", [v("m", "mem")], [u("len"), p("input")]), A(":.param", [u("len")], [e("n")]),
        A("materializec", [u("len"), p("input"), fn("materialize-copy-u64-producer")], [p("buf")], [1, 1, 1], [1]),
        A("buf.to-mem", [u("len"), p("buf")], [v("out", "mem")])])
    # cast-index: ([i.] [.i] ix.to-u64); source-level `materialize` closure-converts to materializec with a unit environment
    cast_index = M("cast-index", [u("i")], [u("r")], [A("ix.to-u64", [u("i")], [u("r")])])
    indexes_source = M("materialize-indexes-source", [u("len")], [v("out", "mem")], [
        A(":.param", [u("len")], [e("n")]),
        A("materializec", [u("len"), fn("cast-index")], [p("buf")], [1, 0, 1], [1]),
        A("buf.to-mem", [u("len"), p("buf")], [v("out", "mem")])])
    return [one_producer, indexes, copy_producer, copy, cast_index, indexes_source]


# ---------------------------------------------------------------- stdlib/math.hex:148-199, stdlib/nn.hex:2-22 (scalar programs)
def silu_programs():
    from catena_lang_b200.lowered_stdlib import silu_modules
    return silu_modules()


# ---------------------------------------------------------------- user programs in the reference's idiom (no file there): a map
# over a buffer through a stdlib activation, a producer with a conditional, a producer with a fold inside
def custom_map_programs():
    f = lambda n: v(n, "f32")                                                # noqa: E731
    u = lambda n: v(n, "u64")                                                # noqa: E731
    e = lambda n: v(n, "erased")                                             # noqa: E731
    pf = lambda n: v(n, "ptr<f32>")                                          # noqa: E731
    silu = silu_programs()
    silu_at = M("my.silu-at", [pf("x"), u("i")], [f("r")], [
        A("ix", [u("i"), pf("x")], [f("xi")]), A("nn.silu", [f("xi")], [f("r")], call=symbol_for("nn.silu"))])
    silu_map = M("my.silu-map", [v("m", "mem")], [v("out", "mem")], [
        A("mem.cast.f32", [v("m", "mem")], [u("len"), pf("x")]),
        A("materializec", [u("len"), pf("x"), fn("my.silu-at")], [pf("buf")], [1, 1, 1], [1]),
        A("buf.to-mem", [u("len"), pf("buf")], [v("out", "mem")])])
    # out[i] = x[i] >= floor ? x[i] : floor, through bool.ifc over two closures that return their capture (conditionals.hex)
    keep = closure("program_closure_my_clamp_0", [f("x")], [f("x")])
    low = closure("program_closure_my_clamp_1", [f("x")], [f("x")])
    clamp_at = M("my.clamp-at", [pf("x"), f("floor"), u("i")], [f("r")], [
        A("ix", [u("i"), pf("x")], [f("xi")]), A("f32.gte", [f("xi"), f("floor")], [v("keep", "bool")]), A("unit.intro", [], [e("unit")]),
        A("bool.ifc", [f("xi"), fn("closure.my-clamp.0"), f("floor"), fn("closure.my-clamp.1"), v("keep", "bool"), e("unit")], [f("r")],
          [1, 1, 1, 1, 1, 1], [1])])
    clamp_map = M("my.clamp-map", [v("m", "mem"), f("floor")], [v("out", "mem")], [
        A("mem.cast.f32", [v("m", "mem")], [u("len"), pf("x")]),
        A("materializec", [u("len"), pf("x"), f("floor"), fn("my.clamp-at")], [pf("buf")], [1, 2, 1], [1]),
        A("buf.to-mem", [u("len"), pf("buf")], [v("out", "mem")])])
    # out[row] = fold over k < cols of a[row * cols + k] * b[k], separately rounded, ascending k (the matmul cell rule for one vector)
    add_env = M("f32.add-env", [f("acc"), f("value")], [f("r")], [A("f32.add", [f("acc"), f("value")], [f("r")])])
    term_at = M("my.matvec-term-at", [pf("a"), pf("b"), u("cols"), u("row"), u("k")], [f("r")], [
        A("row-major-index", [u("cols"), u("row"), u("k")], [u("flat")]), A("ix", [u("flat"), pf("a")], [f("av")]),
        A("ix", [u("k"), pf("b")], [f("bv")]), A("f32.mul", [f("av"), f("bv")], [f("r")])])
    cell_at = M("my.matvec-at", [pf("a"), pf("b"), u("cols"), u("row")], [f("r")], [
        A("const.u32.0x00000000", [], [v("zb", "u32")]), A("u32.bitcast-f32", [v("zb", "u32")], [f("zero")]), A("unit.intro", [], [e("unit")]),
        A("reducec", [f("zero"), e("unit"), fn("f32.add-env"), pf("a"), pf("b"), u("cols"), u("row"), fn("my.matvec-term-at"), u("cols")], [f("r")],
          [1, 1, 1, 4, 1, 1], [1])])
    matvec = M("my.matvec", [v("ma", "mem"), v("mb", "mem"), u("rows")], [v("out", "mem")], [
        A("mem.cast.f32", [v("ma", "mem")], [u("alen"), pf("a")]), A("mem.cast.f32", [v("mb", "mem")], [u("cols"), pf("b")]),
        A("materializec", [u("rows"), pf("a"), pf("b"), u("cols"), fn("my.matvec-at")], [pf("buf")], [1, 3, 1], [1]),
        A("buf.to-mem", [u("rows"), pf("buf")], [v("out", "mem")])])
    # straight-line f32 arithmetic: three products that feed exactly one sum or difference (fused by the compiler), one that feeds two
    poly_at = M("my.poly-at", [pf("x"), f("s"), u("i")], [f("r")], [
        A("ix", [u("i"), pf("x")], [f("xi")]), A("f32.mul", [f("xi"), f("s")], [f("t1")]), A("f32.mul", [f("xi"), f("xi")], [f("sq")]),
        A("f32.add", [f("t1"), f("xi")], [f("t2")]), A("f32.mul", [f("t2"), f("t2")], [f("t3")]), A("f32.sub", [f("s"), f("t3")], [f("t4")]),
        A("f32.mul", [f("t4"), f("sq")], [f("t5")]), A("f32.sub", [f("t5"), f("sq")], [f("r")])])
    poly_map = M("my.poly-map", [v("m", "mem"), f("s")], [v("out", "mem")], [
        A("mem.cast.f32", [v("m", "mem")], [u("len"), pf("x")]),
        A("materializec", [u("len"), pf("x"), f("s"), fn("my.poly-at")], [pf("buf")], [1, 2, 1], [1]),
        A("buf.to-mem", [u("len"), pf("buf")], [v("out", "mem")])])
    return silu + [silu_at, silu_map, keep, low, clamp_at, clamp_map, add_env, term_at, cell_at, matvec, poly_at, poly_map]


# ---------------------------------------------------------------- folds over device buffers that match no fold kernel (user programs in
# the reference's idiom: tests/cases/reducec/basic.hex with other closures)
def custom_fold_programs():
    f = lambda n: v(n, "f32")                                                # noqa: E731
    u = lambda n: v(n, "u64")                                                # noqa: E731
    e = lambda n: v(n, "erased")                                             # noqa: E731
    pf = lambda n: v(n, "ptr<f32>")                                          # noqa: E731
    pu = lambda n: v(n, "ptr<u64>")                                          # noqa: E731
    base = custom_map_programs()                                             # nn.silu and friends, my.silu-at, f32.add-env
    # sum over i of silu(x[i]): `add` is the stdlib's f32.add-env (a prebuilt fold), the getter is not
    sum_silu = M("my.sum-silu", [v("m", "mem")], [f("r")], [
        A("mem.cast.f32", [v("m", "mem")], [u("len"), pf("x")]),
        A("const.u32.0x00000000", [], [v("zb", "u32")]), A("u32.bitcast-f32", [v("zb", "u32")], [f("zero")]), A("unit.intro", [], [e("unit")]),
        A("reducec", [f("zero"), e("unit"), fn("f32.add-env"), pf("x"), fn("my.silu-at"), u("len")], [f("r")], [1, 1, 1, 1, 1, 1], [1])])
    # acc = acc * 31 + x[i]: an `add` that is not associative — only the sequential loop gives the reference's value
    horner_add = M("my.horner-add", [u("k"), u("acc"), u("value")], [u("r")], [
        A("u64.mul", [u("acc"), u("k")], [u("t")]), A("u64.add", [u("t"), u("value")], [u("r")])])
    u64_at = M("sum-u64-at", [pu("input"), u("i")], [u("r")], [A("ix", [u("i"), pu("input")], [u("r")])])
    horner = M("my.horner", [v("m", "mem"), u("k")], [u("r")], [
        A("mem.cast.u64", [v("m", "mem")], [u("len"), pu("input")]), A("const.u64.0x0000000000000007", [], [u("seed")]),
        A("reducec", [u("seed"), u("k"), fn("my.horner-add"), pu("input"), fn("sum-u64-at"), u("len")], [u("r")], [1, 1, 1, 1, 1, 1], [1])])
    # (sum, sum of squares) of a u64 buffer: a two-component accumulator (tests/cases/closures/progression.hex, over a buffer)
    moments_at = M("my.moments-at", [pu("input"), u("i")], [u("value"), u("square")], [
        A("ix", [u("i"), pu("input")], [u("value")]), A("u64.mul", [u("value"), u("value")], [u("square")])])
    moments_add = M("my.moments-add", [u("ls"), u("lq"), u("rs"), u("rq")], [u("s"), u("q")], [
        A("u64.add", [u("ls"), u("rs")], [u("s")]), A("u64.add", [u("lq"), u("rq")], [u("q")])])
    moments = M("my.moments", [v("m", "mem")], [u("sum"), u("squares")], [
        A("mem.cast.u64", [v("m", "mem")], [u("len"), pu("input")]),
        A("const.u64.0x0000000000000000", [], [u("z0")]), A("const.u64.0x0000000000000000", [], [u("z1")]),
        A("reducec", [u("z0"), u("z1"), fn("my.moments-add"), pu("input"), fn("my.moments-at"), u("len")], [u("sum"), u("squares")],
          [2, 0, 1, 1, 1, 1], [2])])
    # x[i] / sum(x): a recognised fold (f32.add-env over f32-at) next to a producer no kernel matches — the module runs generically
    f32_at = M("f32-at", [pf("input"), u("i")], [f("r")], [A("ix", [u("i"), pf("input")], [f("r")])])
    scale_at = M("my.scale-at", [pf("x"), f("total"), u("i")], [f("r")], [
        A("ix", [u("i"), pf("x")], [f("xi")]), A("f32.div", [f("xi"), f("total")], [f("r")])])
    normalize = M("my.normalize", [v("m", "mem")], [v("out", "mem")], [
        A("mem.cast.f32", [v("m", "mem")], [u("len"), pf("x")]),
        A("const.u32.0x00000000", [], [v("zb", "u32")]), A("u32.bitcast-f32", [v("zb", "u32")], [f("zero")]), A("unit.intro", [], [e("unit")]),
        A("reducec", [f("zero"), e("unit"), fn("f32.add-env"), pf("x"), fn("f32-at"), u("len")], [f("total")], [1, 1, 1, 1, 1, 1], [1]),
        A("materializec", [u("len"), pf("x"), f("total"), fn("my.scale-at")], [pf("buf")], [1, 2, 1], [1]),
        A("buf.to-mem", [u("len"), pf("buf")], [v("out", "mem")])])
    return base + [sum_silu, horner_add, u64_at, horner, moments_at, moments_add, moments, f32_at, scale_at, normalize]
