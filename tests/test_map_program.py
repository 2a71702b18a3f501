"""The generic map path on the CPU: the selector's plan for `materializec` with an arbitrary producer, and the register
programs it builds — run by the CPU interpreter of tests/map_vm.py and compared with the host evaluator applied index by
index (the evaluator is pinned to the reference's vectors and to the oracle's primitive table in test_evaluator.py)."""
import numpy as np
import pytest

import catena_lang_b200 as cb
from catena_lang_b200 import lowering as lo
from catena_lang_b200.evaluator import Evaluator
from catena_lang_b200.map_program import compile_producer, OP, _OPS
import lowered_fixtures as fx
import map_vm
import oracle as orc


def modules_by_name(mods):
    return lo.module_map(mods)


def program_of(mods, entry):
    mm = modules_by_name(mods)
    [assign] = [a for a in mm[entry].entry.assignments if a.op == "materializec"]
    return lo.map_program_for(assign, mm), mm


def test_selector_takes_arbitrary_producers():
    mods = fx.materialize_programs() + fx.custom_map_programs()
    mm = modules_by_name(mods)
    for name in ("materialize-indexes", "materialize-copy-u64", "materialize-indexes-source", "my.clamp-map", "my.matvec"):
        assert lo.select(mm[name], modules=mm).kernel == "host_with_map_kernels"
    # a producer that only applies a scalar stdlib program to every element of a buffer has a prebuilt kernel
    plan = lo.select(mm["my.silu-map"], modules=mm)
    assert (plan.kernel, plan.notes) == ("map_unary", ["nn.silu"])
    # a producer that is not there, or is not scalar code, stays unsupported
    bad = fx.M("bad-map", [fx.v("n", "u64")], [fx.v("out", "mem")], [
        fx.A("materializec", [fx.v("n", "u64"), fx.fn("no.such-producer")], [fx.v("buf", "ptr<u64>")], [1, 0, 1], [1]),
        fx.A("buf.to-mem", [fx.v("n", "u64"), fx.v("buf", "ptr<u64>")], [fx.v("out", "mem")])])
    with pytest.raises(lo.Unsupported):
        lo.select(bad, modules=modules_by_name([bad]))


def test_reference_materialize_vectors():
    """catena-lang/tests/cases/materializec.rs:5-31 and materialize.rs:5-31: [1,1,1,1], a copy of [3,5,8,13], [0,1,2,3], empty."""
    mods = fx.materialize_programs()
    prog, _ = program_of(mods, "materialize-indexes")
    assert map_vm.run(prog, [], 4, []).tolist() == [1, 1, 1, 1]
    prog, _ = program_of(mods, "materialize-copy-u64")
    data = np.array([3, 5, 8, 13], np.uint64)
    assert map_vm.run(prog, [(0, data.nbytes)], 4, [data.view(np.uint8)]).tolist() == [3, 5, 8, 13]
    prog, _ = program_of(mods, "materialize-indexes-source")
    assert map_vm.run(prog, [], 4, []).tolist() == [0, 1, 2, 3]
    assert map_vm.run(prog, [], 0, []).tolist() == []
    assert len(prog.code) == 1 and prog.code[0].op == OP["HALT"]            # the index register IS the result


def test_silu_program_matches_the_oracle_bit_for_bit():
    """nn.silu from its primitives (stdlib/nn.hex:2-22, math.hex:148-199), inlined into one register program."""
    prog, mm = program_of(fx.custom_map_programs(), "my.silu-map")
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.normal(0, 3, 500).astype(np.float32), np.array([0.0, -0.0, 1e-30, -87.0, 88.0, 20.0, -20.0], np.float32)])
    got = map_vm.run(prog, [(0, x.nbytes)], x.size, [x.view(np.uint8)]).astype(np.uint32)
    want = orc.map_unary("nn.silu", x).view(np.uint32)
    assert np.array_equal(got, want)
    ev = Evaluator(list({id(m): m for m in mm.values()}.values()))
    for i in (0, 17, 499):
        assert int(got[i]) == int(np.float32(ev.call("nn.silu", [x[i]])[0]).view(np.uint32))
    assert prog.n_regs <= 64


def test_conditional_and_fold_inside_a_producer():
    mods = fx.custom_map_programs()
    prog, mm = program_of(mods, "my.clamp-map")
    x = np.array([1.5, -2.0, 0.25, 7.0, -0.0, 0.5], np.float32)
    got = map_vm.run(prog, [(0, x.nbytes), np.float32(0.5)], x.size, [x.view(np.uint8)]).astype(np.uint32).view(np.float32)
    assert np.array_equal(got, np.maximum(x, np.float32(0.5)))
    assert any(c.op == OP["JZ"] for c in prog.code)
    # a sequential fold per element: bit-exact against the oracle's matmul cell rule (ascending k, separately rounded)
    prog, mm = program_of(mods, "my.matvec")
    rng = np.random.default_rng(4)
    rows, cols = 7, 33
    a = rng.uniform(-1, 1, rows * cols).astype(np.float32)
    b = rng.uniform(-1, 1, cols).astype(np.float32)
    got = map_vm.run(prog, [(0, a.nbytes), (0, b.nbytes), cols], rows, [a.view(np.uint8), b.view(np.uint8)]).astype(np.uint32)
    want = np.asarray(orc.matmul_f32(a, b, rows, 1, cols)).reshape(-1).view(np.uint32)
    assert np.array_equal(got, want)


def test_faults_of_a_program_are_reported_not_executed():
    mods = fx.materialize_programs()
    prog, _ = program_of(mods, "materialize-copy-u64")
    data = np.array([3, 5], np.uint64)
    with pytest.raises(map_vm.Fault):
        map_vm.run(prog, [(0, data.nbytes)], 3, [data.view(np.uint8)])          # index 2 of a 2-element buffer


def test_programs_stay_within_the_kernel_limits():
    from catena_lang_b200.map_program import MAX_INSNS, MAX_REGS
    for entry in ("my.silu-map", "my.clamp-map", "my.matvec"):
        prog, _ = program_of(fx.custom_map_programs(), entry)
        assert len(prog.code) <= MAX_INSNS and prog.n_regs <= MAX_REGS
        assert prog.code[-1].op == OP["HALT"]
        n_init = len(prog.presets)
        for c in prog.code:
            if c.op not in (OP["HALT"], OP["JMP"], OP["JZ"], OP["ASSERT"]):
                assert n_init <= c.dst < prog.n_regs and c.dst != prog.index_reg


def test_generic_folds_compile_and_match_the_sequential_loop():
    """A `reducec` over buffers that matches no fold kernel: the selector's plan, and its sequential register programs
    against the loop written out in Python (the reference's left fold, catena-lang/src/codegen/ops/reducec.rs:75-131)."""
    mods = fx.custom_fold_programs()
    mm = modules_by_name(mods)
    for name in ("my.sum-silu", "my.horner", "my.moments", "my.normalize"):
        assert lo.select(mm[name], modules=mm).kernel == "host_with_map_kernels"
    fold = lambda name: [a for a in mm[name].entry.assignments if a.op == "reducec"][0]        # noqa: E731
    # acc = acc * k + x[i] from 7: not associative
    plan = lo.fold_plan_for(fold("my.horner"), mm)
    assert plan.staged is None and len(plan.sequential) == 1
    data = np.array([3, 5, 8, 13, 2 ** 63 + 5], np.uint64)
    # runtime inputs of the reducec in order: seed, k, input, len
    [got] = map_vm.run(plan.sequential[0], [7, 31, (0, data.nbytes), data.size], 1, [data.view(np.uint8)])
    want = 7
    for x in data.tolist():
        want = (want * 31 + x) % 2 ** 64
    assert int(got) == want
    # two accumulator components: one program each
    plan = lo.fold_plan_for(fold("my.moments"), mm)
    assert plan.staged is None and len(plan.sequential) == 2
    got = [int(map_vm.run(p, [0, 0, (0, data.nbytes), data.size], 1, [data.view(np.uint8)])[0]) for p in plan.sequential]
    assert got == [sum(data.tolist()) % 2 ** 64, sum(x * x for x in data.tolist()) % 2 ** 64]
    # the stdlib's f32.add-env with another getter: staged through the prebuilt sum, and sequential = the oracle's fold
    plan = lo.fold_plan_for(fold("my.sum-silu"), mm)
    assert plan.staged is not None and plan.staged[2] == "sum_f32"
    x = np.random.default_rng(8).normal(0, 2, 300).astype(np.float32)
    [got] = map_vm.run(plan.sequential[0], [np.float32(0.0), (0, x.nbytes), x.size], 1, [x.view(np.uint8)])
    assert int(got) == int(np.float32(orc.sum_f32(orc.map_unary("nn.silu", x))).view(np.uint32))
    # an empty fold returns its zero
    [got] = map_vm.run(plan.sequential[0], [np.float32(2.5), (0, 0), 0], 1, [np.zeros(0, np.uint8)])
    assert int(got) == int(np.float32(2.5).view(np.uint32))


@pytest.mark.parametrize("seed", range(12))
def test_random_producers_compile_to_what_the_evaluator_computes(seed):
    """Random well-typed producers (tests/random_programs.py): the register program run by the CPU interpreter gives, index by
    index, the bits the host evaluator computes from the lowered assignments — folding, aliasing, register reuse, the
    conditional and the loop included."""
    import random_programs as rp
    result = "u64" if seed % 2 == 0 else "f32"
    mods, name = rp.generate(seed, n_ops=40, result=result, control=seed % 3 != 0)
    mm = modules_by_name(mods)
    [launch] = [a for a in mm[name].entry.assignments if a.op == "materializec"]
    prog = lo.map_program_for(launch, mm)
    table, xs = rp.tables(seed)
    n, sd, scale = 24, 0x0123456789ABCDEF ^ seed, np.float32(1.5 + seed)
    got = map_vm.run(prog, [sd, scale, (0, table.nbytes), (0, xs.nbytes)], n, [table.view(np.uint8), xs.view(np.uint8)])
    ev = Evaluator(mods)
    for i in range(n):
        [want] = ev.call(f"{name}.at", [sd, scale, table, xs, i])
        bits = int(want) if result == "u64" else int(np.float32(want).view(np.uint32))
        assert int(got[i]) == bits, (seed, i)


def test_products_sink_into_the_sums_that_alone_read_them():
    """F32_MUL + F32_ADD / F32_SUB as one instruction when the product has no other reader: fewer instructions, the same bits
    (two roundings, not an fma)."""
    prog, mm = program_of(fx.custom_map_programs(), "my.poly-map")
    ops = [c.op for c in prog.code]
    # x*s feeds one sum, (..)^2 one difference, t4*x^2 one difference; x^2 has two readers and stays a product
    assert [_OPS[o] for o in ops] == ["LOAD_F32", "F32_MUL", "F32_MULADD", "F32_SUBMUL", "F32_MULSUB", "HALT"]
    x = np.random.default_rng(9).normal(0, 3, 200).astype(np.float32)
    got = map_vm.run(prog, [(0, x.nbytes), np.float32(1.25)], x.size, [x.view(np.uint8)]).astype(np.uint32)
    ev = Evaluator(list({id(m): m for m in mm.values()}.values()))
    for i in range(x.size):
        [want] = ev.call("my.poly-at", [x, np.float32(1.25), i])
        assert int(got[i]) == int(np.float32(want).view(np.uint32))
