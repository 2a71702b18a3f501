"""Native lowering selector: hand-written IR fixtures (shaped after catena-lang/src/codegen/mod.rs:107-146
and the lowering asserted in catena-lang/tests/compile/closures/matmul.rs:45-53 and reduce.rs:30) must map
to the prebuilt kernels; anything else must be refused, not silently run."""
import pytest

import catena_lang_b200 as cb
from catena_lang_b200 import lowering as lo


def mod(source_name, assigns):
    return lo.module_from_dict({"name": cb.symbol_for(source_name), "source_name": source_name,
                                "entry": {"name": cb.symbol_for(source_name), "sources": [], "targets": [],
                                          "assignments": assigns}})


def reducec(add, get):
    return {"op": "reducec", "inputs": [{"name": "zero", "lowered": "f32"}, {"fn": add}, {"name": "buf", "lowered": "ptr<f32>"},
                                        {"fn": get}, {"name": "len", "lowered": "u64"}], "outputs": [{"name": "acc", "lowered": "f32"}]}


def materializec(producer):
    return {"op": "materializec", "inputs": [{"name": "len", "lowered": "u64"}, {"name": "env", "lowered": "ptr<f32>"}, {"fn": producer}],
            "outputs": [{"name": "out", "lowered": "ptr<f32>"}]}


CAST = {"op": "mem.cast.f32", "inputs": [{"name": "m", "lowered": "mem"}], "outputs": [{"name": "len", "lowered": "u64"}, {"name": "buf", "lowered": "ptr<f32>"}]}
TO_MEM = {"op": "buf.to-mem", "inputs": [{"name": "len", "lowered": "u64"}, {"name": "out", "lowered": "ptr<f32>"}], "outputs": [{"name": "r", "lowered": "mem"}]}


def test_matmul_module_selects_the_f32_gemm():
    m = mod("matmul-2x2-via-mem", [CAST, CAST, {"op": "u64.eq", "inputs": [], "outputs": []}, {"op": "assert", "inputs": [], "outputs": []},
                                   materializec("closure.f32.matmul.row-major.cell-at.0"), TO_MEM])
    plan = lo.select(m)
    assert plan.kernel == "matmul_f32_kernel" and plan.symbol == "program_matmul_2x2_via_mem"


def test_stdlib_folds_and_fused_programs():
    assert lo.select(mod("sum-f32", [CAST, reducec("f32.add-env", "f32-at")])).kernel == "fold_sum"
    assert lo.select(mod("max-f32", [CAST, reducec("f32.max-env", "f32-at")])).kernel == "fold_max"
    assert lo.select(mod("tensor.argmax-f32", [CAST, reducec("tensor.argmax-env", "tensor.argmax-pair-at")])).kernel == "fold_argmax"
    sm = mod("nn.softmax", [CAST, reducec("f32.max-env", "f32-at"), reducec("f32.add-env", "nn.softmax-exp-shifted-at"),
                            materializec("nn.softmax-at"), TO_MEM])
    assert lo.select(sm).kernel == "softmax_fused" and lo.select(sm).symbol == "program_nn_softmax"
    rn = mod("nn.rmsnorm", [CAST, reducec("f32.add-env", "nn.squared-at"), {"op": "u64.to-f32", "inputs": [], "outputs": []},
                            {"op": "f32.div", "inputs": [], "outputs": []}, {"op": "math.sqrt", "inputs": [], "outputs": [], "call_symbol": "program_math_sqrt"},
                            materializec("nn.rmsnorm-at"), TO_MEM])
    assert lo.select(rn).kernel == "rmsnorm_fused"
    assert lo.select(mod("tensor.concat-f32", [CAST, CAST, materializec("tensor.concat-f32-at"), TO_MEM])).kernel == "copy_concat"


def test_scalar_module_runs_on_the_host():
    m = mod("nn.silu", [{"op": "f32.neg", "inputs": [], "outputs": []}, {"op": "math.exp-approx", "inputs": [], "outputs": [], "call_symbol": "program_math_exp_approx"},
                        {"op": "f32.add", "inputs": [], "outputs": []}, {"op": "f32.div", "inputs": [], "outputs": []}, {"op": "f32.mul", "inputs": [], "outputs": []}])
    assert lo.select(m).kernel == "host_scalar"


def test_unknown_producer_is_refused():
    with pytest.raises(lo.Unsupported):
        lo.select(mod("my-map", [CAST, materializec("my.custom-at"), TO_MEM]))
    with pytest.raises(lo.Unsupported):
        lo.select(mod("odd", [CAST, reducec("f32.add-env", "my.getter")]))


def test_stdlib_extension_registers_the_added_programs():
    """The hexpr extension file declares the programs this backend adds; the host mirror finds them by name
    (the file itself cannot be type-checked here: the checker is not part of this build)."""
    import os
    import catena_lang_b200 as cb
    path = os.path.join(os.path.dirname(cb.__file__), "stdlib_ext", "b200.hex")
    rt = cb.Runtime.new([path])
    for name in ("gemm-bf16-rc", "gemm-i8-rc", "attn-decode-bf16"):
        assert name in rt.signatures and rt.signatures[name][0] == cb.symbol_for(name)
    text = open(path).read()
    assert text.count("(") == text.count(")") and text.count("{") == text.count("}") and text.count("[") == text.count("]")
    # the operators of the Llama-style block are declared as primitive arrows (no `def program`: exec would drop the weights)
    for arrow in ("embed.bf16", "rmsnorm.rows.bf16", "rope.append.bf16", "attention.prefill.bf16", "swiglu.bf16",
                  "llama.block.prefill", "llama.block.decode"):
        assert f"(arr {arrow} :" in text


def test_integer_and_scalar_modules_of_the_reference_tests():
    """The hand-lowered test programs of the reference (tests/lowered_fixtures.py): buffer folds over u64 select the u64
    kernels, the buffer-head program the 8-byte copy, everything scalar the host evaluator; a scalar module that walks a
    buffer in any other way has no plan."""
    import lowered_fixtures as fx
    from catena_lang_b200.lowering import LIBRARY_ENTRY, module_map
    mods = fx.reducec_programs() + fx.array_head_program() + fx.all_host_modules()
    mm = module_map(mods)
    def callable_through_exec(m):       # no `buf` pointer on the boundary (runtime/signature.rs:63-72)
        return m.source_name and not any(v.lowered.startswith("ptr<") for v in m.entry.sources + m.entry.targets)
    plans = {m.source_name: lo.select(m, modules=mm) for m in mods if callable_through_exec(m)}
    assert plans["sum-u64"].kernel == "fold_sum_u64" and plans["sum-u64"].entry == "program_sum_u64"
    assert plans["dot-u64"].kernel == "fold_dot_u64" and plans["dot-u64"].entry == "program_dot_u64"
    assert plans["array-head-u64"].kernel == "array_head_u64" and LIBRARY_ENTRY["array_head_u64"] == "program_array_head_u64"
    for name in ("not", "bool-ifc-primitives", "shift-and-sub", "fma-fused-bits", "ordered-pair", "sum-progression", "progression-moments",
                 "u64.add-env"):
        assert plans[name].kernel == "host_scalar", name
    # `sum-u64-at` reads a buffer element on its own: on the host that is a dereference of device memory
    with pytest.raises(lo.Unsupported):
        lo.select(mm["sum-u64-at"], modules=mm)
    # a fold whose getter is unknown to the selector and whose environment holds a buffer has no plan either
    odd = fx.M("odd-fold", [fx.v("m", "mem")], [fx.v("r", "u64")], [
        fx.A("mem.cast.u64", [fx.v("m", "mem")], [fx.v("len", "u64"), fx.v("buf", "ptr<u64>")]),
        fx.A("const.u64.0x0000000000000000", [], [fx.v("zero", "u64")]),
        fx.A("reducec", [fx.v("zero", "u64"), fx.fn("u64.add-env"), fx.v("buf", "ptr<u64>"), fx.fn("some-other-getter"), fx.v("len", "u64")],
             [fx.v("r", "u64")], [1, 0, 1, 1, 1, 1], [1])])
    with pytest.raises(lo.Unsupported):
        lo.select(odd, modules=mm)


def test_runtime_from_modules_refuses_what_it_cannot_run():
    import catena_lang_b200 as cb
    import lowered_fixtures as fx
    odd = fx.M("materialize-something", [fx.v("n", "u64")], [fx.v("out", "mem")], [
        fx.A("materializec", [fx.v("n", "u64"), fx.fn("some.unknown-producer")], [fx.v("out", "mem")])])
    with pytest.raises(cb.InitError):
        cb.Runtime.from_modules([odd])
