"""The host evaluator of lowered scalar modules against the reference's own integer / bit / conditional vectors, through
the reference-shaped `Runtime.exec` (registered with `Runtime.from_modules`; no GPU is touched: scalar modules run on
the host, as the reference's non-materialize code does).  Every expected value below is the one the reference's test
asserts, with its file:line."""
import numpy as np
import pytest

import catena_lang_b200 as cb
from catena_lang_b200 import evaluator as ev
from catena_lang_b200.lowering import module_map, select

import lowered_fixtures as fx


@pytest.fixture(scope="module")
def rt():
    return cb.Runtime.from_modules(fx.all_host_modules())


def one(rt, name, args=()):
    [r] = rt.exec(name, list(args))
    return r


def test_every_fixture_is_planned_for_the_host():
    mods = fx.all_host_modules()
    mm = module_map(mods)
    for m in mods:
        if m.source_name:
            assert select(m, modules=mm).kernel == "host_scalar", m.source_name


def test_bool_programs(rt):
    # tests/runtime.rs:37-52, 54-75, 77-104, 106-128
    r = one(rt, "not", [False])
    assert r.kind is cb.ValueKind.Bool and r.v == 1
    for x, want in [(False, 1), (True, 0)]:
        assert one(rt, "not-via-function-value", [x]).v == want
    for flag, arg, want in [(True, False, 0), (True, True, 1), (False, False, 1), (False, True, 1)]:
        assert one(rt, "bool-ifc-primitives", [flag, arg]).v == want
    left, right = rt.exec("copy-via-function-value", [])
    assert (left.v, right.v) == (1, 1)


def test_exec_validates_name_arity_and_types(rt):
    # tests/runtime.rs:130-168
    with pytest.raises(cb.ExecError) as e:
        rt.exec("missing", [])
    assert e.value.kind == "UnknownSourceFunction"
    with pytest.raises(cb.ExecError) as e:
        rt.exec("not", [])
    assert e.value.kind == "InputArityMismatch"
    with pytest.raises(cb.ExecError) as e:
        rt.exec("not", [False], n_outputs=0)
    assert e.value.kind == "OutputArityMismatch"
    with pytest.raises(cb.ExecError) as e:
        rt.exec("not", [0])
    assert e.value.kind == "TypeMismatch"


def test_integer_and_float_arithmetic(rt):
    # tests/runtime.rs:170-188, 190-212, 214-271, 273-290, 292-311, 313-331
    r = one(rt, "two-times-two-u64")
    assert r.kind is cb.ValueKind.U64 and r.v == 4
    assert one(rt, "sub-basic").v == 1
    for name, want in [("u64-ne-test", 1), ("u64-lt-test", 1), ("u64-lte-test", 1), ("u64-gte-test", 0)]:
        assert one(rt, name).v == want
    r = one(rt, "two-times-two-u32")
    assert r.kind is cb.ValueKind.U32 and r.v == 4
    r = one(rt, "two-times-two-f32")
    assert r.kind is cb.ValueKind.F32 and r.v == 4.0
    assert one(rt, "fma-basic").v == 2.0


def test_fma_is_fused(rt):
    # tests/runtime.rs:333-363
    a = b = float(np.uint32(0x3F800001).view(np.float32))
    c = float(np.uint32(0x33800000).view(np.float32))
    assert one(rt, "fma-fused-bits", [a, b, c]).v == 0x3F800003
    assert one(rt, "mul-add-bits", [a, b, c]).v == 0x3F800002


def test_bitcasts_shifts_bitwise_and_compares(rt):
    # tests/runtime.rs:408-426, 428-446, 448-473, 475-530, 532-605, 607-680
    assert one(rt, "bitcast-one").v == 1.0
    assert one(rt, "bitcast-one-bits").v == 0x3F800000
    assert one(rt, "shift-and-sub").v == 0xFFFFFFFC
    for name, want in [("u32-and-test", 0x000F000F), ("u32-or-test", 0x0FFF0FFF), ("u32-xor-test", 0x0FF00FF0), ("u32-not-test", 0xFF00FF00)]:
        assert one(rt, name).v == want
    for name, want in [("u32-eq-test", 0), ("u32-ne-test", 1), ("u32-lt-test", 1), ("u32-gt-test", 0), ("u32-lte-test", 1), ("u32-gte-test", 0)]:
        assert one(rt, name).v == want
    for name, want in [("f32-lt-test", 1), ("f32-eq-test", 0), ("f32-ne-test", 1), ("f32-gt-test", 0), ("f32-lte-test", 1), ("f32-gte-test", 0)]:
        assert one(rt, name).v == want


def test_integer_constants(rt):
    # tests/runtime.rs:682-711
    assert one(rt, "deadbeef").v == 0xDEADBEEFDEADBEEF
    assert one(rt, "deadbeef32").v == 0xDEADBEEF


def test_conditionals_with_captured_branches(rt):
    # tests/cases/closures.rs:9-50
    for value, floor, want in [(3.5, 2.0, 3.5), (-4.0, -1.5, -1.5), (2.25, 2.25, 2.25)]:
        assert one(rt, "max-with-floor", [value, floor]).v == want
    for lhs, rhs, want in [(3.5, 2.0, (2.0, 3.5)), (-4.0, -1.5, (-4.0, -1.5)), (2.25, 2.25, (2.25, 2.25))]:
        lo, hi = rt.exec("ordered-pair", [lhs, rhs])
        assert (lo.v, hi.v) == want


def test_host_reducec_progressions(rt):
    # tests/cases/closures.rs:52-104
    for length, base, step, want in [(0, 7, 3, 0), (4, 2, 3, 26), (5, 1, 1, 15)]:
        assert one(rt, "sum-progression", [length, base, step]).v == want
    for length, base, step, want_sum, want_sq in [(0, 7, 3, 0, 0), (4, 2, 3, 26, 214), (3, 1, 1, 6, 14)]:
        s, q = rt.exec("progression-moments", [length, base, step])
        assert (s.v, q.v) == (want_sum, want_sq)
    # wraparound of the u64 accumulator is C unsigned arithmetic
    assert one(rt, "sum-progression", [3, 2 ** 63, 2 ** 62]).v == (3 * 2 ** 63 + 3 * 2 ** 62) % 2 ** 64


def test_reducec_over_host_buffers_and_the_head_program():
    """The buffer programs of tests/cases/reducec.rs:6-48 and tests/runtime.rs:713-740 evaluated on HOST arrays (the
    device versions are kernels, tested on the GPU): the evaluator's `mem.cast.u64`, `ix`, `reducec` and assertions."""
    e = ev.Evaluator(fx.reducec_programs() + fx.array_head_program())
    mem = lambda xs: np.asarray(xs, dtype=np.uint64).view(np.uint8)           # noqa: E731
    assert e.call("sum-u64", [mem([2, 3, 5, 7, 11])]) == [28]
    assert e.call("dot-u64", [mem([2, 3, 5, 7]), mem([11, 13, 17, 19])]) == [2 * 11 + 3 * 13 + 5 * 17 + 7 * 19]
    with pytest.raises(ev.AssertFailed):
        e.call("dot-u64", [mem([1, 2]), mem([1, 2, 3])])
    assert e.call("array-head-u64", [mem([0x123456789ABCDEF0, 7, 11])]) == [0x123456789ABCDEF0]
    with pytest.raises(ev.AssertFailed):
        e.call("array-head-u64", [mem([])])
    assert e.call("sum-u64", [mem([2 ** 64 - 1, 2])]) == [1]


def test_primitive_table_against_the_oracle(orc):
    """Every primitive of the table on random and edge operands: the evaluator and the CPU oracle (which evaluates the C
    expression the reference's renderer prints) must agree bit for bit."""
    rng = np.random.default_rng(0)
    edge32 = [0, 1, 2, 31, 32, 0x7FFFFFFF, 0x80000000, 0xFFFFFFFF, 0x3F800000, 0x00FF00FF]
    edge64 = [0, 1, 2, 2 ** 24, 2 ** 24 + 1, 2 ** 53 + 1, 2 ** 63, 2 ** 64 - 1, 0xDEADBEEFDEADBEEF, 2 ** 63 + 2 ** 39 + 1]
    u32s = edge32 + [int(x) for x in rng.integers(0, 2 ** 32, 200)]
    u64s = edge64 + [int(x) for x in rng.integers(0, 2 ** 64, 200, dtype=np.uint64)]
    fbits = [0x00000000, 0x80000000, 0x3F800000, 0xBF800000, 0x3F800001, 0x33800000, 0x7F800000, 0xFF800000, 0x00000001, 0x7F7FFFFF,
             0x4B000001, 0x3FC00000, 0x40200000] + [int(x) for x in rng.integers(0, 2 ** 32, 300)]
    fbits = [b for b in fbits if (b & 0x7F800000) != 0x7F800000 or (b & 0x007FFFFF) == 0]           # no NaN inputs
    def run(op, *raw):
        kinds = orc.PRIM_KINDS[op]
        args = [ev.bits_f32(x) if k == "f32" else x for k, x in zip(kinds[0], raw)]
        with np.errstate(all="ignore"):
            got = ev.PRIMITIVES[op](*args)[0]
        got_bits = ev.f32_bits(got) if kinds[1] == "f32" else int(got)
        want = orc.prim(op, *raw)
        if kinds[1] == "f32" and np.isnan(ev.bits_f32(want)):
            assert np.isnan(got), (op, raw)                   # NaN payloads are hardware properties
        else:
            assert got_bits == want, (op, [hex(x) for x in raw], hex(got_bits), hex(want))
    for op, (ins, _out) in orc.PRIM_KINDS.items():
        pools = [{"u32": u32s, "u64": u64s, "f32": fbits, "bool": [0, 1]}[k] for k in ins]
        n = 1 if not ins else 300
        for t in range(n):
            raw = [p[(t * (7 + 2 * j) + j) % len(p)] for j, p in enumerate(pools)]
            if op in ("u32.shl", "u32.shr"):
                raw[1] %= 32                                   # a shift by 32 or more is undefined in C
            if op == "f32.round-to-u32":
                x = ev.bits_f32(raw[0])
                if not (x >= 0 and x < 4294967296.0):
                    continue
            run(op, *raw)
    with pytest.raises(ev.UndefinedBehaviour):
        ev.PRIMITIVES["u32.shl"](1, 32)
    with pytest.raises(ev.UndefinedBehaviour):
        ev.PRIMITIVES["f32.round-to-u32"](np.float32(-1.0))
