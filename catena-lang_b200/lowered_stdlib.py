"""Scalar stdlib programs as LOWERED modules (`lowering.GpuModule`), written by hand from the hexpr sources with the
reference's lowering rules (SSA order of the definition's operations, one assignment per operation, a call of another
program as an assignment with a call symbol: catena-lang/src/codegen/mod.rs:107-146, 229-330).

The reference compiles the stdlib together with every user program, so a producer may call `nn.silu` and friends; a
host that hands this backend lowered modules passes the stdlib's modules along with its own.  The Rust front end that
would produce them is not part of this build, so the modules the generic map path is measured and tested with live here:
  math.exp-approx-nonneg, math.exp-approx      catena-lang/stdlib/math.hex:148-199
  nn.sigmoid, nn.silu                          catena-lang/stdlib/nn.hex:2-22
"""
from . import symbol_for
from .lowering import GpuAssign, GpuFunction, GpuModule, GpuVar


def _v(name, lowered):
    return GpuVar(name, lowered)


def _A(op, ins=(), outs=(), call=None):
    return GpuAssign(op, list(ins), list(outs), call)


def _M(source_name, sources, targets, assigns):
    sym = symbol_for(source_name)
    return GpuModule(sym, source_name, GpuFunction(sym, list(sources), list(targets), list(assigns)))


def silu_modules():
    """[math.exp-approx-nonneg, math.exp-approx, nn.sigmoid, nn.silu]"""
    f = lambda n: _v(n, "f32")                                               # noqa: E731
    w = lambda n: _v(n, "u32")                                               # noqa: E731
    A, M, v = _A, _M, _v

    def const_f32(bits, name):
        return [A(f"const.u32.0x{bits:08X}", [], [w(name + "_b")]), A("u32.bitcast-f32", [w(name + "_b")], [f(name)])]

    nonneg = M("math.exp-approx-nonneg", [f("x")], [f("result")],
               const_f32(0x3FB8AA3B, "inv_ln2") + const_f32(0x3F317200, "ln2_hi") + const_f32(0x35BFBE8E, "ln2_lo") +
               const_f32(0x3F7FF8FC, "c0") + const_f32(0x3F809C7E, "c1") + const_f32(0x3EEF1187, "c2") + const_f32(0x3E738A8B, "c3") + [
        A("f32.mul", [f("x"), f("inv_ln2")], [f("scaled")]), A("f32.round-to-u32", [f("scaled")], [w("k_u32")]),
        A("u32.to-f32", [w("k_u32")], [f("k_f32")]),
        A("f32.mul", [f("k_f32"), f("ln2_hi")], [f("k_ln2_hi")]), A("f32.mul", [f("k_f32"), f("ln2_lo")], [f("k_ln2_lo")]),
        A("f32.sub", [f("x"), f("k_ln2_hi")], [f("r1")]), A("f32.sub", [f("r1"), f("k_ln2_lo")], [f("xr")]),
        A("f32.mul", [f("xr"), f("c3")], [f("xr_c3")]), A("f32.add", [f("c2"), f("xr_c3")], [f("p2")]),
        A("f32.mul", [f("xr"), f("p2")], [f("xr_p2")]), A("f32.add", [f("c1"), f("xr_p2")], [f("p1")]),
        A("f32.mul", [f("xr"), f("p1")], [f("xr_p1")]), A("f32.add", [f("c0"), f("xr_p1")], [f("poly")]),
        A("const.u32.0x0000007F", [], [w("bias_u32")]), A("const.u32.0x00800000", [], [w("exp_step_u32")]),
        A("u32.add", [w("k_u32"), w("bias_u32")], [w("biased_exp")]), A("u32.mul", [w("biased_exp"), w("exp_step_u32")], [w("pow2_bits")]),
        A("u32.bitcast-f32", [w("pow2_bits")], [f("pow2k")]), A("f32.mul", [f("poly"), f("pow2k")], [f("result")])])
    exp = M("math.exp-approx", [f("x")], [f("result")], [
        A("const.u32.0x00000000", [], [w("zero_b")]), A("u32.to-f32", [w("zero_b")], [f("zero")])] + const_f32(0x3F800000, "one") + [
        A("f32.neg", [f("x")], [f("neg_x")]), A("f32.lt", [f("x"), f("zero")], [v("is_negative", "bool")]),
        A("f32.select", [v("is_negative", "bool"), f("neg_x"), f("x")], [f("magnitude")]),
        A("math.exp-approx-nonneg", [f("magnitude")], [f("base")], call=nonneg.name),
        A("f32.div", [f("one"), f("base")], [f("reciprocal")]),
        A("f32.select", [v("is_negative", "bool"), f("reciprocal"), f("base")], [f("result")])])
    sigmoid = M("nn.sigmoid", [f("x")], [f("result")], [
        A("f32.one", [], [f("one")]), A("f32.neg", [f("x")], [f("neg_x")]),
        A("math.exp-approx", [f("neg_x")], [f("exp_neg_x")], call=exp.name),
        A("f32.add", [f("one"), f("exp_neg_x")], [f("denominator")]), A("f32.div", [f("one"), f("denominator")], [f("result")])])
    silu = M("nn.silu", [f("x")], [f("result")], [
        A("nn.sigmoid", [f("x")], [f("gate")], call=sigmoid.name), A("f32.mul", [f("x"), f("gate")], [f("result")])])
    return [nonneg, exp, sigmoid, silu]
