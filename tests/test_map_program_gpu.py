"""The generic map on the GPU: `materializec` with producers that no prebuilt kernel matches, run through
`Runtime.from_modules(...).exec(...)` — the reference's own vectors, equality with the prebuilt bit-exact kernels and the
oracle, the CPU interpreter of tests/map_vm.py at sizes that need many CTAs, and the refusals that keep a malformed or
faulting program away from the device.  A register program runs either as its own compiled kernel (csrc/map_jit.cu, the
default) or on the library's interpreter (csrc/map_program.cu): the tests that launch programs directly run both and want
the same bits and the same statuses."""
import ctypes as C

import numpy as np
import pytest

import catena_lang_b200 as cb
from catena_lang_b200 import lowering as lo
from catena_lang_b200.map_program import OP, Insn
import lowered_fixtures as fx
import map_vm
import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    return cb.Runtime.from_modules(fx.materialize_programs() + fx.custom_map_programs())


def test_reference_materialize_vectors(rt):
    """catena-lang/tests/cases/materializec.rs:5-31, tests/cases/materialize.rs:5-31"""
    [out] = rt.exec("materialize-indexes", [4])
    assert out.v.to_u64_vec().tolist() == [1, 1, 1, 1]
    [out] = rt.exec("materialize-copy-u64", [rt.mem_u64([3, 5, 8, 13])])
    assert out.v.to_u64_vec().tolist() == [3, 5, 8, 13]
    [out] = rt.exec("materialize-indexes-source", [4])
    assert out.v.to_u64_vec().tolist() == [0, 1, 2, 3]
    [out] = rt.exec("materialize-indexes-source", [0])
    assert out.v.is_null() and out.v.to_u64_vec().tolist() == []


@pytest.mark.parametrize("n", [1, 255, 257, 100_003, 1 << 21])
def test_silu_from_its_primitives_equals_the_prebuilt_kernel(rt, n):
    """nn.silu built from its primitives, compiled and interpreted = the prebuilt map kernel = the oracle, bit for bit."""
    rng = np.random.default_rng(n)
    x = rng.normal(0, 4, n).astype(np.float32)
    x[: min(n, 6)] = np.array([0.0, -0.0, 88.0, -87.0, 1e-30, -1e-30], np.float32)[: min(n, 6)]
    # through the runtime the selector recognises `out[i] = nn.silu(x[i])` and takes the prebuilt kernel; the register
    # program of the same producer is launched directly
    [out] = rt.exec("my.silu-map", [rt.mem_f32(x)])
    selected = out.v.to_f32_vec().view(np.uint32)
    mm = lo.module_map(fx.custom_map_programs())
    [launch] = [a for a in mm["my.silu-map"].entry.assignments if a.op == "materializec"]
    m = cb.upload(x)
    prog = lo.map_program_for(launch, mm)
    for compiled in (True, False):
        raw = prog.launch(n, [(m.data, m.len)], compiled=compiled)
        got = cb.download(raw, np.float32).view(np.uint32)
        cb.free(raw)
        assert np.array_equal(got, selected)
    cb.free(m)
    m = cb.upload(x)
    o = cb.CatenaMem()
    cb.check(cb.lib().catena_b200_map_f32_s(b"nn.silu", m, C.byref(o)))
    prebuilt = cb.download(o, np.float32).view(np.uint32)
    cb.free(m)
    cb.free(o)
    assert np.array_equal(got, prebuilt)
    if n <= 100_003:
        assert np.array_equal(got, orc.map_unary("nn.silu", x).view(np.uint32))


def test_conditional_and_fold_inside_a_producer(rt):
    x = np.random.default_rng(5).normal(0, 1, 10_000).astype(np.float32)
    [out] = rt.exec("my.clamp-map", [rt.mem_f32(x), np.float32(0.25)])
    assert np.array_equal(out.v.to_f32_vec(), np.maximum(x, np.float32(0.25)))
    rows, cols = 300, 257
    rng = np.random.default_rng(6)
    a = rng.uniform(-1, 1, rows * cols).astype(np.float32)
    b = rng.uniform(-1, 1, cols).astype(np.float32)
    [out] = rt.exec("my.matvec", [rt.mem_f32(a), rt.mem_f32(b), rows])
    want = np.asarray(orc.matmul_f32(a, b, rows, 1, cols)).reshape(-1)
    assert np.array_equal(out.v.to_f32_vec().view(np.uint32), want.view(np.uint32))


def test_kernel_equals_the_cpu_interpreter_on_integer_programs():
    """u64 / u32 arithmetic with wraparound, shifts, compares and selects over the index: one program, every opcode family."""
    u, w, b = (lambda n: fx.v(n, "u64")), (lambda n: fx.v(n, "u32")), (lambda n: fx.v(n, "bool"))
    producer = fx.M("my.hash-at", [u("seed"), u("i")], [u("r")], [
        fx.A("const.u64.0x9E3779B97F4A7C15", [], [u("g")]), fx.A("u64.mul", [u("i"), u("g")], [u("h0")]),
        fx.A("u64.add", [u("h0"), u("seed")], [u("h1")]), fx.A("u64.sub", [u("h1"), u("i")], [u("h2")]),
        fx.A("const.u64.0x00000000FFFFFFFF", [], [u("mask")]), fx.A("u64.lt", [u("h2"), u("mask")], [b("small")]),
        fx.A("u64.select", [b("small"), u("h1"), u("h2")], [u("h3")]),
        fx.A("const.u32.0x0000000D", [], [w("s13")]), fx.A("const.u32.0x85EBCA6B", [], [w("m1")]),
        fx.A("const.u32.0x00000011", [], [w("s17")]),
        # the low word through u32 operations: a bitcast round trip narrows nothing, so take it by comparing and selecting
        fx.A("u64.to-f32", [u("h3")], [fx.v("hf", "f32")]), fx.A("f32.bitcast-u32", [fx.v("hf", "f32")], [w("x0")]),
        fx.A("u32.shl", [w("x0"), w("s13")], [w("x1")]), fx.A("u32.xor", [w("x0"), w("x1")], [w("x2")]),
        fx.A("u32.mul", [w("x2"), w("m1")], [w("x3")]), fx.A("u32.shr", [w("x3"), w("s17")], [w("x4")]),
        fx.A("u32.not", [w("x4")], [w("x5")]), fx.A("u32.or", [w("x5"), w("x1")], [w("x6")]), fx.A("u32.and", [w("x6"), w("x3")], [w("x7")]),
        fx.A("u32.sub", [w("x7"), w("x2")], [w("x8")]), fx.A("u32.add", [w("x8"), w("s13")], [w("x9")]),
        fx.A("u32.gte", [w("x9"), w("m1")], [b("big")]), fx.A("bool.not", [b("big")], [b("nb")]), fx.A("bool.or", [b("nb"), b("small")], [b("c")]),
        fx.A("u32.to-f32", [w("x9")], [fx.v("xf", "f32")]), fx.A("f32.bitcast-u32", [fx.v("xf", "f32")], [w("y")]),
        fx.A("u32.select", [b("c"), w("y"), w("x9")], [w("z")]),
        fx.A("u32.bitcast-f32", [w("z")], [fx.v("zf", "f32")]), fx.A("f32.bitcast-u32", [fx.v("zf", "f32")], [w("z2")]),
        fx.A("u32.eq", [w("z"), w("z2")], [b("same")]), fx.A("assert", [b("same")], [fx.v("h", "erased")]),
        fx.A("u64.add", [u("h3"), u("h0")], [u("r")])])
    entry = fx.M("my.hash", [u("n"), u("seed")], [fx.v("out", "mem")], [
        fx.A("materializec", [u("n"), u("seed"), fx.fn("my.hash-at")], [fx.v("buf", "ptr<u64>")], [1, 1, 1], [1]),
        fx.A("buf.to-mem", [u("n"), fx.v("buf", "ptr<u64>")], [fx.v("out", "mem")])])
    mods = [producer, entry]
    rt = cb.Runtime.from_modules(mods)
    n, seed = 5000, 0xFFFFFFFFFFFFFF00
    [out] = rt.exec("my.hash", [n, seed])
    mm = lo.module_map(mods)
    prog = lo.map_program_for(entry.entry.assignments[0], mm)
    assert np.array_equal(out.v.to_u64_vec(), map_vm.run(prog, [seed], n, []))


def test_faults_of_a_program_come_back_as_statuses(rt):
    """An index past its buffer (the reference would read out of bounds) and a failed assert: CATENA_E_ASSERT, nothing faults,
    and the library works afterwards."""
    mods = fx.materialize_programs()
    mm = lo.module_map(mods)
    prog = lo.map_program_for([a for a in mm["materialize-copy-u64"].entry.assignments if a.op == "materializec"][0], mm)
    data = cb.upload(np.array([3, 5], np.uint64))
    for compiled in (True, False):
        with pytest.raises(cb.CatenaError) as err:
            prog.launch(3, [(data.data, data.len)], compiled=compiled)
        assert err.value.status == cb.E_ASSERT
        out = prog.launch(2, [(data.data, data.len)], compiled=compiled)
        assert cb.download(out, np.uint64).tolist() == [3, 5]
        cb.free(out)
    cb.free(data)
    [ok] = rt.exec("materialize-indexes", [3])
    assert ok.v.to_u64_vec().tolist() == [1, 1, 1]


def test_malformed_programs_are_refused_before_the_launch():
    L = cb.lib()

    def call(code, n_init=0, n_regs=4, index_reg=0, result_reg=0, n_buffers=0, elem=8, length=4):
        arr = (Insn * len(code))(*code)
        init = (C.c_uint64 * 4)()
        bufs = (cb.CatenaMem * 1)()
        out = cb.CatenaMem()
        s = L.catena_b200_map_program_s(arr, len(code), init, n_init, n_regs, index_reg, result_reg, bufs, n_buffers, elem, length, C.byref(out))
        if s == cb.OK:
            cb.free(out)
        return s

    halt = Insn(OP["HALT"], 0, 0, 0, 0, 0, 0)
    assert call([halt]) == cb.OK
    assert call([Insn(OP["MOV"], 1, 0, 0, 0, 0, 0)]) == cb.E_BAD_ARG                       # no HALT at the end
    assert call([Insn(OP["MOV"], 9, 0, 0, 0, 0, 0), halt]) == cb.E_BAD_ARG                 # register past the file
    assert call([Insn(OP["MOV"], 1, 9, 0, 0, 0, 0), halt]) == cb.E_BAD_ARG
    assert call([Insn(OP["JMP"], 0, 0, 0, 0, 0, 7), halt]) == cb.E_BAD_ARG                 # jump target past the program
    assert call([Insn(len(OP), 1, 0, 0, 0, 0, 0), halt]) == cb.E_BAD_ARG                   # unknown opcode
    assert call([Insn(OP["LOAD_U64"], 1, 0, 0, 0, 0, 0), halt]) == cb.E_BAD_ARG            # buffer 0 of none
    assert call([Insn(OP["MOV"], 0, 1, 0, 0, 0, 0), halt]) == cb.E_BAD_ARG                 # writes the index register
    assert call([Insn(OP["MOV"], 0, 1, 0, 0, 0, 0), halt], n_init=1, index_reg=1) == cb.E_BAD_ARG   # writes a preset register
    assert call([halt], elem=2) == cb.E_BAD_ARG
    assert call([halt], n_regs=300) == cb.E_BAD_ARG
    # an endless loop ends at the budget of backward jumps and is reported; the library stays usable
    assert call([Insn(OP["JMP"], 0, 0, 0, 0, 0, 0), halt], length=1) == cb.E_ASSERT
    assert call([halt]) == cb.OK


@pytest.mark.parametrize("n_insn,n_regs", [(300, 8), (300, 70), (240, 250), (150, 140), (2000, 40)])
def test_every_kernel_geometry_agrees_with_the_cpu_interpreter(n_insn, n_regs):
    """Programs built by hand so that every launch shape is taken: programs carried in the kernel parameters and programs
    staged in shared memory (more than 192 instructions), four lanes per thread and one (more than 128 registers), 256
    threads per CTA and 128 (a register file that would not fit otherwise)."""
    from catena_lang_b200.map_program import MapProgram
    index = 3
    presets = [("const", 0x9E3779B97F4A7C15), ("const", 7), ("env", 0)]
    # well typed, as the compiler's programs are: even registers hold u64 values, odd ones bool / u32 values
    wide_ops, narrow_ops = ["U64_ADD", "U64_MUL", "U64_SUB", "MOV", "SELECT"], ["U64_LT", "U32_XOR", "U32_ADD", "U32_MUL", "MOV32", "U64_GTE"]
    rng = np.random.default_rng(n_insn * 1000 + n_regs)
    code, wide, narrow = [], [0, 1, 2, index], []
    for k in range(n_insn - 2):
        slot = 4 + k % (n_regs - 4)
        if slot % 2 == 0:
            op = wide_ops[(k // 2) % len(wide_ops)]
            if op == "SELECT" and not narrow:
                op = "U64_ADD"
            a = int(rng.choice(narrow)) if op == "SELECT" else int(rng.choice(wide))
            code.append(Insn(OP[op], slot, a, int(rng.choice(wide)), int(rng.choice(wide)), 0, 0))
            if slot not in wide:
                wide.append(slot)
        else:
            op = narrow_ops[(k // 2) % len(narrow_ops)]
            if not narrow:
                op = "U64_LT"
            src = wide if op.startswith("U64") else narrow
            code.append(Insn(OP[op], slot, int(rng.choice(src)), int(rng.choice(src)), 0, 0, 0))
            if slot not in narrow:
                narrow.append(slot)
    last = max(w for w in wide if w >= 4)
    code.append(Insn(OP["U64_ADD"], last, last, index, 0, 0, 0))            # every element differs
    code.append(Insn(OP["HALT"], 0, 0, 0, 0, 0, 0))
    prog = MapProgram("by-hand", code, presets, n_regs, index, code[-2].dst, ["u64"], 8)
    length = 3000
    want = map_vm.run(prog, [123456789], length, [])
    for compiled in (False, True):
        out = prog.launch(length, [123456789], compiled=compiled)
        got = cb.download(out, np.uint64)
        cb.free(out)
        assert np.array_equal(got, want)


def test_generic_folds_through_the_runtime():
    """`reducec` over device buffers with closures that match no fold kernel: the sequential loop on one device thread for an
    `add` that is not associative and for a two-component accumulator; two stages (generic map + prebuilt fold) for the
    stdlib's adds with another getter; and a module where a recognised fold sits next to a generic producer."""
    rt = cb.Runtime.from_modules(fx.custom_fold_programs())
    rng = np.random.default_rng(21)
    data = rng.integers(0, 2 ** 63, 5000, dtype=np.uint64)
    [got] = rt.exec("my.horner", [rt.mem_u64(data), 31])
    want = 7
    for x in data.tolist():
        want = (want * 31 + x) % 2 ** 64
    assert got.v == want
    s, q = rt.exec("my.moments", [rt.mem_u64(data)])
    assert s.v == sum(data.tolist()) % 2 ** 64 and q.v == sum(x * x for x in data.tolist()) % 2 ** 64
    # an empty buffer: the fold's zero
    s, q = rt.exec("my.moments", [rt.mem_u64([])])
    assert (s.v, q.v) == (0, 0)
    # sum of silu(x[i]): sequential below 1024 elements, staged above; both are the oracle's sequential sum up to 65536 elements
    for n in (300, 40_000):
        x = rng.normal(0, 2, n).astype(np.float32)
        [got] = rt.exec("my.sum-silu", [rt.mem_f32(x)])
        want = np.float32(orc.sum_f32(orc.map_unary("nn.silu", x)))
        assert np.float32(got.v).view(np.uint32) == want.view(np.uint32)
    # x[i] / sum(x)
    x = rng.uniform(0.5, 1.5, 3000).astype(np.float32)
    [out] = rt.exec("my.normalize", [rt.mem_f32(x)])
    total = np.float32(orc.sum_f32(x))
    assert np.array_equal(out.v.to_f32_vec().view(np.uint32), (x / total).astype(np.float32).view(np.uint32))
    # a fold longer than the loop budget of one thread is reported, not run forever
    big = cb.Runtime.from_modules(fx.custom_fold_programs())
    with pytest.raises(cb.ExecError) as err:
        big.exec("my.horner", [big.mem_u64(np.zeros((1 << 22) + 10, np.uint64)), 3])
    assert err.value.status == cb.E_ASSERT


@pytest.mark.parametrize("seed,control", [(100, True), (101, True), (102, False), (103, False), (104, True), (105, False)])
def test_random_producers_on_the_device(seed, control):
    """Random well-typed producers (tests/random_programs.py) through `Runtime.exec`: the kernel gives the bits of the CPU
    interpreter (which test_map_program.py ties to the host evaluator) — with a conditional and a loop (one element per
    thread) and without (four per thread)."""
    import random_programs as rp
    result = "u64" if seed % 2 == 0 else "f32"
    mods, name = rp.generate(seed, n_ops=60, result=result, control=control)
    rt = cb.Runtime.from_modules(mods)
    table, xs = rp.tables(seed)
    n, sd, scale = 2500, 0xFEDCBA9876543210 ^ seed, np.float32(0.75 * seed)
    [out] = rt.exec(name, [sd, scale, rt.mem_u64(table), rt.mem_f32(xs), n])
    got = out.v.to_u64_vec() if result == "u64" else out.v.to_f32_vec().view(np.uint32)
    mm = lo.module_map(mods)
    [launch] = [a for a in mm[name].entry.assignments if a.op == "materializec"]
    prog = lo.map_program_for(launch, mm)
    want = map_vm.run(prog, [sd, scale, (0, table.nbytes), (0, xs.nbytes)], n, [table.view(np.uint8), xs.view(np.uint8)])
    assert np.array_equal(got, want.astype(got.dtype))
    mt, mx = cb.upload(table), cb.upload(xs)
    for compiled in (True, False):
        raw = prog.launch(n, [sd, scale, (mt.data, mt.len), (mx.data, mx.len)], compiled=compiled)
        assert np.array_equal(cb.download(raw, got.dtype), got)
        cb.free(raw)
    cb.free(mt)
    cb.free(mx)


def test_a_map_sharded_by_index_ranges_gives_the_unsharded_bits():
    """Elements of a map are independent, so it shards over GPUs by contiguous index ranges, every rank running the same
    register program with its range's first index: the ranges of 1, 2, 4 and 8 ranks, run here one after the other on one
    GPU, concatenate to the unsharded result (an index-dependent integer producer and a buffer-reading f32 producer)."""
    from catena_lang_b200 import shard
    import random_programs as rp
    for seed, result in ((200, "u64"), (201, "f32")):
        mods, name = rp.generate(seed, n_ops=50, result=result, control=False)
        mm = lo.module_map(mods)
        [launch] = [a for a in mm[name].entry.assignments if a.op == "materializec"]
        prog = lo.map_program_for(launch, mm)
        table, xs = rp.tables(seed)
        mt, mx = cb.upload(table), cb.upload(xs)
        env = [77 + seed, np.float32(2.5), (mt.data, mt.len), (mx.data, mx.len)]
        dtype = np.uint64 if result == "u64" else np.uint32
        n = 10_007
        whole = prog.launch(n, env)
        want = cb.download(whole, dtype)
        cb.free(whole)
        for compiled in (True, False):
            for world in (2, 4, 8):
                parts = []
                for r in shard.index_ranges(n, world, align=4):
                    raw = prog.launch(r.i1 - r.i0, env, index0=r.i0, compiled=compiled)
                    parts.append(cb.download(raw, dtype))
                    cb.free(raw)
                assert np.array_equal(np.concatenate(parts), want)
        cb.free(mt)
        cb.free(mx)


def test_compiled_kernels_keep_the_bounds_of_the_interpreter():
    """What keeps a program from hanging or faulting the GPU holds in the compiled kernel too: an endless loop ends at the
    budget of backward jumps, the undefined cases (shift by 32 or more, round-to-u32 out of range, division by zero) yield 0 and
    CATENA_E_ASSERT, and the next launch works."""
    from catena_lang_b200.map_program import MapProgram
    halt = Insn(OP["HALT"], 0, 0, 0, 0, 0, 0)
    loop = MapProgram("endless", [Insn(OP["JMP"], 0, 0, 0, 0, 0, 0), halt], [], 2, 0, 1, [], 8)
    with pytest.raises(cb.CatenaError) as err:
        loop.launch(1, [], compiled=True)
    assert err.value.status == cb.E_ASSERT
    cases = {
        "shift": [Insn(OP["U32_SHL"], 2, 1, 0, 0, 0, 0), halt],              # index << 40
        "divide": [Insn(OP["U64_SUB"], 3, 1, 1, 0, 0, 0), Insn(OP["U64_DIV"], 2, 1, 3, 0, 0, 0), halt],
        "round": [Insn(OP["F32_ROUND_TO_U32"], 2, 0, 0, 0, 0, 0), halt],     # preset 0 holds -1.0f
    }
    for name, code in cases.items():
        preset = 0xBF800000 if name == "round" else 40
        prog = MapProgram(name, code, [("const", preset)], 4, 1, 2, [], 8 if name == "divide" else 4)
        for compiled in (True, False):
            with pytest.raises(cb.CatenaError) as err:
                prog.launch(5, [], compiled=compiled)
            assert err.value.status == cb.E_ASSERT, (name, compiled)
    ok = MapProgram("index", [halt], [], 1, 0, 0, [], 8)
    out = ok.launch(1000, [], compiled=True)
    assert cb.download(out, np.uint64).tolist() == list(range(1000))
    cb.free(out)


def test_one_compiled_kernel_serves_every_environment():
    """Environment scalars and buffers are kernel parameters: one compilation, any number of launches with other values."""
    mm = lo.module_map(fx.custom_map_programs())
    [launch] = [a for a in mm["my.clamp-map"].entry.assignments if a.op == "materializec"]
    prog = lo.map_program_for(launch, mm)
    handle = prog.compiled().value
    rng = np.random.default_rng(8)
    for n, floor in ((10, 0.5), (70_001, -0.25), (3, 7.0)):
        x = rng.normal(0, 1, n).astype(np.float32)
        m = cb.upload(x)
        raw = prog.launch(n, [(m.data, m.len), np.float32(floor)], compiled=True)
        assert np.array_equal(cb.download(raw, np.float32), np.maximum(x, np.float32(floor)))
        cb.free(raw)
        cb.free(m)
    assert prog.compiled().value == handle


def test_compiled_reciprocal_is_the_ieee_reciprocal_for_every_class_of_operand():
    """`1 / x` in a compiled kernel is `rcp.rn`, in the interpreter an IEEE division: the same bits for zeros, subnormals,
    infinities, negative and huge values (NaN results compared as NaNs), and numpy's quotient."""
    from catena_lang_b200.map_program import MapProgram
    rng = np.random.default_rng(77)
    bits = np.concatenate([
        rng.integers(0, 2 ** 32, 200_000, dtype=np.uint64).astype(np.uint32),                      # every class, NaNs included
        rng.uniform(0.5, 4.0, 100_000).astype(np.float32).view(np.uint32),
        np.array([0x3F000000, 0x3EFFFFFF, 0x717FFFFF, 0x71800000, 0x00000000, 0x80000000, 0x00000001, 0x007FFFFF, 0x00800000,
                  0x7F800000, 0xFF800000, 0x7F7FFFFF, 0x3F800000, 0x3F7FFFFF, 0x3F800001, 0x7E800000, 0x7F000000], np.uint32)])
    x = bits.view(np.float32)
    # registers: 0 = 1.0f (constant), 1 = index, 2 = x[i], 3 = 1 / x[i]
    code = [Insn(OP["LOAD_F32"], 2, 1, 0, 0, 0, 0), Insn(OP["F32_DIV"], 3, 0, 2, 0, 0, 0), Insn(OP["HALT"], 0, 0, 0, 0, 0, 0)]
    prog = MapProgram("reciprocal", code, [("const", 0x3F800000)], 4, 1, 3, ["buffer"], 4)
    m = cb.upload(x)
    outs = []
    for compiled in (True, False):
        raw = prog.launch(x.size, [(m.data, m.len)], compiled=compiled)
        outs.append(cb.download(raw, np.uint32))
        cb.free(raw)
    cb.free(m)
    got, want = outs[0].view(np.float32), outs[1].view(np.float32)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    assert np.array_equal(outs[0][ok], outs[1][ok])
    with np.errstate(divide="ignore", invalid="ignore", over="ignore", under="ignore"):
        host = (np.float32(1.0) / x).astype(np.float32)
    assert np.array_equal(outs[1][ok], host.view(np.uint32)[ok])          # and both are numpy's IEEE quotient


def test_a_producer_beyond_256_registers_runs_compiled():
    """A long producer with a conditional and a fold (no register reuse across branches: more than the interpreter's 256
    registers) runs as a compiled kernel and gives the bits of the CPU interpreter; the interpreter's entry point refuses it."""
    import random_programs as rp
    from catena_lang_b200.map_program import MAX_REGS
    mods, name = rp.generate(1124, n_ops=130, result="u64", control=True)
    mm = lo.module_map(mods)
    [launch] = [a for a in mm[name].entry.assignments if a.op == "materializec"]
    prog = lo.map_program_for(launch, mm)
    assert prog.n_regs > MAX_REGS
    table, xs = rp.tables(1124)
    mt, mx = cb.upload(table), cb.upload(xs)
    env = [0x0123456789ABCDEF, np.float32(1.5), (mt.data, mt.len), (mx.data, mx.len)]
    n = 2000
    raw = prog.launch(n, env, compiled=True)
    got = cb.download(raw, np.uint64)
    cb.free(raw)
    want = map_vm.run(prog, [env[0], env[1], (0, table.nbytes), (0, xs.nbytes)], n, [table.view(np.uint8), xs.view(np.uint8)])
    assert np.array_equal(got, want.astype(np.uint64))
    with pytest.raises(cb.CatenaError) as err:
        prog.launch(n, env, compiled=False)
    assert err.value.status == cb.E_BAD_ARG
    cb.free(mt)
    cb.free(mx)
    # through the runtime (compiled by default)
    rt = cb.Runtime.from_modules(mods)
    [out] = rt.exec(name, [env[0], env[1], rt.mem_u64(table), rt.mem_f32(xs), n])
    assert np.array_equal(out.v.to_u64_vec(), got)
