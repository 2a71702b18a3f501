"""Random well-typed producers over the primitive table (test data generator, seeded): straight-line scalar code over an
environment (a u64 seed, an f32 scale, a u64 table, an f32 table) and the index, with a conditional and a small fold thrown in.
Operands for which the reference's generated C is undefined never occur (shift counts are masked to 0..31, `round-to-u32` sees
values clamped to [0, 1e9], f32 values are clamped to [-1e3, 1e3] after every operation so that no NaN — whose bit pattern
differs between x86 and the GPU — can arise, divisors are made non-zero)."""
import numpy as np

import lowered_fixtures as fx

TABLE = 64          # elements of the two tables; loads use index mod TABLE


def generate(seed, n_ops=40, result="u64", control=True):
    """-> (modules, entry source name): `entry(seed: u64, scale: f32, table: mem, xs: mem, n: u64) -> mem` materialises
    out[i] = producer(seed, scale, table, xs, i) for i < n.  Without `control` the producer has no conditional and no fold
    (straight-line code: the kernel then carries four elements per thread in lockstep)."""
    rng = np.random.default_rng(seed)
    u, w, f, b = (lambda n: fx.v(n, "u64")), (lambda n: fx.v(n, "u32")), (lambda n: fx.v(n, "f32")), (lambda n: fx.v(n, "bool"))
    mk = {"u64": u, "u32": w, "f32": f, "bool": b}
    body, pools, counter = [], {"u64": ["seed", "i"], "u32": [], "f32": ["scale"], "bool": []}, [0]

    def new(ty):
        counter[0] += 1
        return f"t{counter[0]}"

    def emit(op, ins, ty, extra_outs=()):
        name = new(ty)
        body.append(fx.A(op, ins, [mk[ty](name)] + list(extra_outs)))
        return name

    def pick(ty):
        return mk[ty](str(rng.choice(pools[ty])))

    def const(ty, value):
        if ty == "u64":
            return emit(f"const.u64.0x{value:016X}", [], "u64")
        if ty == "u32":
            return emit(f"const.u32.0x{value:08X}", [], "u32")
        bits = emit(f"const.u32.0x{int(np.float32(value).view(np.uint32)):08X}", [], "u32")
        return emit("u32.bitcast-f32", [w(bits)], "f32")

    lo_c, hi_c, zero_f, one_f = const("f32", -1000.0), const("f32", 1000.0), const("f32", 0.0), const("f32", 1.0)
    table_len = const("u64", TABLE)
    pools["u32"].append(const("u32", 0x9E3779B9))
    pools["u64"].append(const("u64", 0xD1B54A32D192ED03))
    mask31 = const("u32", 31)

    def clamp(name):
        below = emit("f32.lt", [f(name), f(lo_c)], "bool")
        x1 = emit("f32.select", [b(below), f(lo_c), f(name)], "f32")
        above = emit("f32.gt", [f(x1), f(hi_c)], "bool")
        return emit("f32.select", [b(above), f(hi_c), f(x1)], "f32")

    def table_index():
        return emit("row-major-col", [u(table_len), pick("u64")], "u64")

    for _ in range(n_ops):
        kind = rng.choice(["u64", "u32", "f32", "cmp", "select", "convert", "load", "bool"])
        if kind == "u64":
            pools["u64"].append(emit(str(rng.choice(["u64.add", "u64.sub", "u64.mul"])), [pick("u64"), pick("u64")], "u64"))
        elif kind == "u32" and pools["u32"]:
            op = str(rng.choice(["u32.add", "u32.sub", "u32.mul", "u32.and", "u32.or", "u32.xor", "u32.not", "u32.shl", "u32.shr"]))
            if op == "u32.not":
                pools["u32"].append(emit(op, [pick("u32")], "u32"))
            elif op in ("u32.shl", "u32.shr"):
                count = emit("u32.and", [pick("u32"), w(mask31)], "u32")
                pools["u32"].append(emit(op, [pick("u32"), w(count)], "u32"))
            else:
                pools["u32"].append(emit(op, [pick("u32"), pick("u32")], "u32"))
        elif kind == "f32":
            op = str(rng.choice(["f32.add", "f32.sub", "f32.mul", "f32.div", "f32.neg", "f32.fma"]))
            if op == "f32.neg":
                pools["f32"].append(emit(op, [pick("f32")], "f32"))
            elif op == "f32.div":
                d = pick("f32")
                is_zero = emit("f32.eq", [d, f(zero_f)], "bool")
                safe = emit("f32.select", [b(is_zero), f(one_f), d], "f32")
                pools["f32"].append(clamp(emit(op, [pick("f32"), f(safe)], "f32")))
            elif op == "f32.fma":
                pools["f32"].append(clamp(emit(op, [pick("f32"), pick("f32"), pick("f32")], "f32")))
            else:
                pools["f32"].append(clamp(emit(op, [pick("f32"), pick("f32")], "f32")))
        elif kind == "cmp":
            ty = str(rng.choice([t for t in ("u64", "u32", "f32") if pools[t]]))
            op = str(rng.choice(["eq", "ne", "lt", "lte", "gt", "gte"]))
            extra = [fx.v(new("e"), "erased"), fx.v(new("e"), "erased")] if ty == "u64" and op in ("eq", "gt") else []
            pools["bool"].append(emit(f"{ty}.{op}", [pick(ty), pick(ty)], "bool", extra))
        elif kind == "select" and pools["bool"]:
            ty = str(rng.choice([t for t in ("u64", "u32", "f32", "bool") if pools[t]]))
            pools[ty].append(emit(f"{ty}.select", [pick("bool"), pick(ty), pick(ty)], ty))
        elif kind == "bool" and pools["bool"]:
            op = str(rng.choice(["bool.not", "bool.and", "bool.or"]))
            pools["bool"].append(emit(op, [pick("bool")] if op == "bool.not" else [pick("bool"), pick("bool")], "bool"))
        elif kind == "convert":
            which = str(rng.choice(["u64.to-f32", "u32.to-f32", "f32.round-to-u32", "f32.bitcast-u32", "u32.bitcast-f32"]))
            if which == "u64.to-f32":
                pools["f32"].append(clamp(emit(which, [pick("u64")], "f32")))
            elif which == "u32.to-f32" and pools["u32"]:
                pools["f32"].append(clamp(emit(which, [pick("u32")], "f32")))
            elif which == "f32.round-to-u32":
                x = pick("f32")
                negative = emit("f32.lt", [x, f(zero_f)], "bool")
                magnitude = emit("f32.select", [b(negative), f(zero_f), x], "f32")
                pools["u32"].append(emit(which, [f(magnitude)], "u32"))
            elif which == "f32.bitcast-u32":
                pools["u32"].append(emit(which, [pick("f32")], "u32"))
            elif pools["u32"]:
                # any bit pattern may be a NaN or an infinity: clamp, and replace what the clamp cannot order
                raw = emit("u32.bitcast-f32", [pick("u32")], "f32")
                ordered = emit("f32.eq", [f(raw), f(raw)], "bool")
                pools["f32"].append(clamp(emit("f32.select", [b(ordered), f(raw), f(one_f)], "f32")))
        elif kind == "load":
            if rng.integers(2):
                pools["u64"].append(emit("ix", [u(table_index()), fx.v("table", "ptr<u64>")], "u64"))
            else:
                pools["f32"].append(clamp(emit("ix", [u(table_index()), fx.v("xs", "ptr<f32>")], "f32")))
    keep, other = fx.closure(f"program_closure_rand{seed}_0", [u("x")], [u("x")]), fx.closure(f"program_closure_rand{seed}_1", [u("x")], [u("x")])
    add = fx.M(f"rand{seed}.add", [u("k"), u("acc"), u("value")], [u("r")], [
        fx.A("u64.mul", [u("acc"), u("k")], [u("t")]), fx.A("u64.add", [u("t"), u("value")], [u("r")])])
    get = fx.M(f"rand{seed}.get", [fx.v("table", "ptr<u64>"), u("j")], [u("r")], [fx.A("ix", [u("j"), fx.v("table", "ptr<u64>")], [u("r")])])
    folded = str(rng.choice(pools["u64"]))
    if control:
        # a conditional through bool.ifc over two closures that return their capture, and a small fold over the u64 table
        if not pools["bool"]:
            pools["bool"].append(emit("u64.lt", [pick("u64"), pick("u64")], "bool"))
        body.append(fx.A("unit.intro", [], [fx.v("unit", "erased")]))
        chosen = new("u64")
        body.append(fx.A("bool.ifc", [pick("u64"), fx.fn(f"closure.rand{seed}.0"), pick("u64"), fx.fn(f"closure.rand{seed}.1"), pick("bool"),
                                      fx.v("unit", "erased")], [u(chosen)], [1, 1, 1, 1, 1, 1], [1]))
        pools["u64"].append(chosen)
        count = const("u64", 5)
        folded = new("u64")
        body.append(fx.A("reducec", [pick("u64"), pick("u64"), fx.fn(f"rand{seed}.add"), fx.v("table", "ptr<u64>"), fx.fn(f"rand{seed}.get"), u(count)],
                         [u(folded)], [1, 1, 1, 1, 1, 1], [1]))
        pools["u64"].append(folded)
    if result == "u64":
        last = emit("u64.add", [u(folded), pick("u64")], "u64")
        out = emit("u64.add", [u(last), u("i")], "u64")
    else:
        out = clamp(emit("f32.add", [pick("f32"), pick("f32")], "f32"))
    ptr = "ptr<u64>" if result == "u64" else "ptr<f32>"
    producer = fx.M(f"rand{seed}.at", [u("seed"), f("scale"), fx.v("table", "ptr<u64>"), fx.v("xs", "ptr<f32>"), u("i")], [mk[result](out)], body)
    entry = fx.M(f"rand{seed}", [u("seed"), f("scale"), fx.v("mt", "mem"), fx.v("mx", "mem"), u("n")], [fx.v("out", "mem")], [
        fx.A("mem.cast.u64", [fx.v("mt", "mem")], [u("tlen"), fx.v("table", "ptr<u64>")]),
        fx.A("mem.cast.f32", [fx.v("mx", "mem")], [u("xlen"), fx.v("xs", "ptr<f32>")]),
        fx.A("materializec", [u("n"), u("seed"), f("scale"), fx.v("table", "ptr<u64>"), fx.v("xs", "ptr<f32>"), fx.fn(f"rand{seed}.at")],
             [fx.v("buf", ptr)], [1, 4, 1], [1]),
        fx.A("buf.to-mem", [u("n"), fx.v("buf", ptr)], [fx.v("out", "mem")])])
    return [keep, other, add, get, producer, entry], f"rand{seed}"


def tables(seed):
    rng = np.random.default_rng(seed + 10_000)
    return rng.integers(0, 2 ** 64, TABLE, dtype=np.uint64), rng.uniform(-50, 50, TABLE).astype(np.float32)
