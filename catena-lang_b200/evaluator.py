"""Host evaluator of a lowered catena module whose assignments are scalar work.

This is what runs behind the lowering selector's `host_scalar` plan: where the reference renders such a
`GpuFunction` as plain C++ statements and calls the compiled symbol on the host
(catena-lang/src/codegen/gpu.rs:235-261, 287-316), this backend has no source generator, so it evaluates the
same assignments directly, one primitive at a time, with the semantics of the C expression the renderer would
have printed for it:

  primitive table          catena-lang/src/codegen/gpu.rs:322-447 (+ the helpers at :449-718)
  integer constants        gpu.rs:672-698 (`const.u32.0x...` / `const.u64.0x...`)
  row-major index ops      catena-lang/src/codegen/ops/row_major.rs:9-68
  `bool.ifc`               catena-lang/src/codegen/ops/ifc.rs:11-41   (flag ? true_fn(true_env, arg) : false_fn(...))
  `eval`                   gpu.rs:986-991
  `reducec`                catena-lang/src/codegen/ops/reducec.rs:34-133  (acc = zero; for i < n: acc = add(env, acc, get(env, i)))
  program calls            gpu.rs:894-916 (runtime inputs by value, runtime outputs by pointer)
  function application     gpu.rs:918-968 (a primitive symbol is inlined through the same table)

Integer arithmetic is C unsigned arithmetic of the operand width (wraparound); `f32.add/sub/mul/div` are single
IEEE binary32 operations, never contracted (catena-lang/src/runtime/artifact.rs:59-80); `f32.fma` is `fmaf`;
`f32.round-to-u32` is `(uint32_t)nearbyintf(x)`, defined for 0 <= x < 2^32 only; `u32.shl/shr` by 32 or more and
`f32.round-to-u32` outside its range are undefined behaviour in the generated C and raise `UndefinedBehaviour` here.
A failed `assert` raises `AssertFailed` (the generated code traps, catena-lang/src/codegen/prelude.rs:38-55).

Values: bool / u32 / u64 are Python ints, f32 is numpy.float32, `ptr<u64>` / `ptr<f32>` are numpy arrays (host
views) or `DeviceMem`s (device buffers: cast and passed on, never dereferenced), `mem` is a numpy uint8 array or a
`DeviceMem`, erased wires are None.  `materializec` is a kernel launch: the evaluator hands it to the `materialize`
callback it was built with (runtime.py launches the generic map kernel there) and refuses it otherwise; modules whose
`materializec` matches a prebuilt kernel never come here.
"""
import ctypes
import ctypes.util

import numpy as np

from .lowering import FnSymbol, GpuVar

M32 = 0xFFFFFFFF
M64 = 0xFFFFFFFFFFFFFFFF


class AssertFailed(Exception):
    """A `catena_assert` of the program failed (the reference traps)."""


class UndefinedBehaviour(Exception):
    """The generated C of the reference would have undefined behaviour for these operands."""


class NotScalar(Exception):
    """The assignment is a kernel launch or names a function this evaluator does not have."""


_libm = None


def _fmaf(a, b, c):
    """fmaf of three binary32 values: one rounding (gpu.rs:589-604)."""
    global _libm
    if _libm is None:
        _libm = ctypes.CDLL(ctypes.util.find_library("m") or "libm.so.6")
        _libm.fmaf.restype = ctypes.c_float
        _libm.fmaf.argtypes = [ctypes.c_float] * 3
    return np.float32(_libm.fmaf(float(a), float(b), float(c)))


def u_to_f32(x):
    """(float)x for an unsigned integer: round to nearest even in ONE step (Python's int -> float -> float32 would
    round twice above 2^53)."""
    x = int(x)
    if x < (1 << 24):
        return np.float32(x)
    shift = x.bit_length() - 24
    top, rest = x >> shift, x & ((1 << shift) - 1)
    half = 1 << (shift - 1)
    if rest > half or (rest == half and (top & 1)):
        top += 1
    return np.float32(np.ldexp(np.float32(top), shift))               # exact: top has at most 25 significant bits, 24 of them or a power of two


def f32_bits(x):
    return int(np.float32(x).view(np.uint32))


def bits_f32(u):
    return np.uint32(u & M32).view(np.float32)


def _parse_const(op, prefix):
    lit = op[len(prefix):].replace("_", "")
    if not lit.startswith("0x"):
        raise ValueError(f"invalid integer constant `{op}`")
    return int(lit[2:], 16)


def _runtime(values):
    return [v for v in values if v is not None and not isinstance(v, FnSymbol)]


def _binary_u(mask, fn):
    return lambda a, b: [fn(int(a), int(b)) & mask]


def _shift(left):
    def run(a, b):
        a, b = int(a), int(b)
        if b >= 32:
            raise UndefinedBehaviour("u32 shift by 32 or more")
        return [((a << b) if left else (a >> b)) & M32]
    return run


def _round_to_u32(x):
    x = np.float32(x)
    if not (x >= 0 and x < np.float32(4294967296.0)):
        raise UndefinedBehaviour("f32.round-to-u32 outside [0, 2^32)")
    return [int(np.rint(x))]            # nearbyintf in the default rounding mode: to nearest, ties to even


def _cmp(fn):
    return lambda a, b: [1 if fn(a, b) else 0]


def _fcmp(fn):
    return lambda a, b: [1 if fn(np.float32(a), np.float32(b)) else 0]


def _farith(fn):
    def run(a, b):
        with np.errstate(all="ignore"):
            return [np.float32(fn(np.float32(a), np.float32(b)))]
    return run


def _select(flag, a, b):
    return [a if flag else b]


class DeviceMem:
    """A buffer in device memory as host code sees it: it can be cast, truncated and handed to a kernel, but not
    dereferenced (the reference's host code reads managed memory; this backend's buffers are plain device memory)."""
    __slots__ = ("ptr", "nbytes", "dtype")

    def __init__(self, ptr, nbytes, dtype=np.uint8):
        self.ptr, self.nbytes, self.dtype = int(ptr or 0), int(nbytes), np.dtype(dtype)

    @property
    def size(self):
        return self.nbytes // self.dtype.itemsize

    def view(self, dtype):
        return DeviceMem(self.ptr, self.nbytes, dtype)

    def truncated(self, length):
        return DeviceMem(self.ptr, int(length) * self.dtype.itemsize, self.dtype)


def _to_mem(length, buffer):
    if isinstance(buffer, DeviceMem):
        return [buffer.truncated(length).view(np.uint8)]
    return [np.ascontiguousarray(buffer[: int(length)]).view(np.uint8)]


# op -> function(*positional inputs) -> list of outputs (erased outputs are padded with None by the caller)
PRIMITIVES = {
    "bool.t": lambda: [1], "bool.f": lambda: [0],
    "bool.not": lambda a: [0 if a else 1],
    "bool.id": lambda a: [a], "bool.copy": lambda a: [a, a],
    "bool.and": lambda a, b: [1 if (a and b) else 0], "bool.or": lambda a, b: [1 if (a or b) else 0],
    ":.forget": lambda a: [a], "u64.name": lambda a: [a], "ix.to-u64": lambda a: [a],
    "u64.zero": lambda: [0], "u64.one": lambda: [1], "u32.one": lambda: [1], "f32.one": lambda: [np.float32(1.0)],
    "u64.add": _binary_u(M64, lambda a, b: a + b), "u64.sub": _binary_u(M64, lambda a, b: a - b),
    "u64.mul": _binary_u(M64, lambda a, b: a * b),
    "u64.ne": _cmp(lambda a, b: a != b), "u64.lt": _cmp(lambda a, b: a < b), "u64.lte": _cmp(lambda a, b: a <= b),
    "u64.gte": _cmp(lambda a, b: a >= b),
    "u64.eq": _cmp(lambda a, b: a == b), "u64.gt": _cmp(lambda a, b: a > b),     # + two erased witnesses
    "u32.add": _binary_u(M32, lambda a, b: a + b), "u32.sub": _binary_u(M32, lambda a, b: a - b),
    "u32.mul": _binary_u(M32, lambda a, b: a * b), "u32.and": _binary_u(M32, lambda a, b: a & b),
    "u32.or": _binary_u(M32, lambda a, b: a | b), "u32.xor": _binary_u(M32, lambda a, b: a ^ b),
    "u32.shl": _shift(True), "u32.shr": _shift(False), "u32.not": lambda a: [~int(a) & M32],
    "u32.eq": _cmp(lambda a, b: a == b), "u32.ne": _cmp(lambda a, b: a != b), "u32.lt": _cmp(lambda a, b: a < b),
    "u32.gt": _cmp(lambda a, b: a > b), "u32.lte": _cmp(lambda a, b: a <= b), "u32.gte": _cmp(lambda a, b: a >= b),
    "u32.to-f32": lambda a: [u_to_f32(a)], "u64.to-f32": lambda a: [u_to_f32(a)],
    "u32.bitcast-f32": lambda a: [bits_f32(int(a))], "f32.bitcast-u32": lambda a: [f32_bits(a)],
    "f32.add": _farith(lambda a, b: a + b), "f32.sub": _farith(lambda a, b: a - b),
    "f32.mul": _farith(lambda a, b: a * b), "f32.div": _farith(lambda a, b: a / b),
    "f32.neg": lambda a: [np.float32(-np.float32(a))], "f32.fma": lambda a, b, c: [_fmaf(a, b, c)],
    "f32.eq": _fcmp(lambda a, b: a == b), "f32.ne": _fcmp(lambda a, b: a != b), "f32.lt": _fcmp(lambda a, b: a < b),
    "f32.gt": _fcmp(lambda a, b: a > b), "f32.lte": _fcmp(lambda a, b: a <= b), "f32.gte": _fcmp(lambda a, b: a >= b),
    "f32.select": _select, "u32.select": _select, "u64.select": _select, "bool.select": _select,
    "f32.round-to-u32": _round_to_u32,
    "ix.zero": lambda _proof: [0],
    "ix": lambda index, buffer: [_load(buffer, index)],
    "buf.u64.cast-same-length": lambda buffer, _same: [buffer],
    "buf.f32.cast-same-length": lambda buffer, _same: [buffer],
    "mem.cast.u64": lambda mem: [mem.size // 8, mem.view(np.uint64)],
    "mem.cast.f32": lambda mem: [mem.size // 4, mem.view(np.float32)],
    "buf.to-mem": _to_mem,
}
# rendered as nothing (gpu.rs:372-373): their outputs are type-level
NO_OPS = {"unit.intro", "ax-mp", "assert-then", ":.param"}


def _load(buffer, index):
    if isinstance(buffer, DeviceMem):
        raise NotScalar("host code cannot dereference device memory")
    v = buffer[int(index)]          # an index past the end is out of contract (the type system bounds `ix n`)
    return np.float32(v) if buffer.dtype == np.float32 else int(v)


def is_primitive(op):
    return (op in PRIMITIVES or op in NO_OPS or op in (":.ty", "assert", "u64.to-ix", "row-major-index", "row-major-row",
                                                       "row-major-col") or op.startswith(("const.u64.", "const.u32.")))


class Evaluator:
    """Evaluates functions of a module map {symbol or source name -> GpuModule}."""

    def __init__(self, modules, materialize=None, reduce=None):
        """`materialize(assignment, length, environment values, function symbol) -> buffer` runs a `materializec` (a kernel
        launch); without it such an assignment is refused.  `reduce(assignment, input values) -> accumulator values` runs a
        `reducec` one of whose inputs is a device buffer (the host cannot read it); without it such a fold fails when its
        getter dereferences the buffer."""
        from .lowering import module_map
        self.by_name = module_map(modules)
        self.materialize = materialize
        self.reduce = reduce

    # ---- one function ----
    def call(self, name, args):
        """Runs module `name` (generated symbol, or source name) on its runtime inputs; returns its runtime outputs."""
        from .lowering import find_module
        module = find_module(self.by_name, name)
        if module is None:
            raise NotScalar(f"no lowered module for `{name}`")
        fn = module.entry
        sources = [s for s in fn.sources if s.lowered != "erased"]
        if len(sources) != len(args):
            raise TypeError(f"{fn.name}: expected {len(sources)} runtime inputs, got {len(args)}")
        env = {s.name: a for s, a in zip(sources, args)}
        for a in fn.assignments:
            self._assign(env, a)
        return [env[t.name] for t in fn.targets if t.lowered != "erased"]

    def _value(self, env, v):
        if isinstance(v, FnSymbol):
            return v
        if v.lowered == "erased":
            return None
        return env[v.name]

    def _bind(self, env, outputs, values):
        """Writes `values` to the runtime outputs in order; erased outputs take None."""
        runtime = [o for o in outputs if o.lowered != "erased"]
        if len(values) == len(outputs):
            runtime, values = outputs, values
        elif len(values) != len(runtime):
            raise TypeError(f"{len(values)} values for {len(runtime)} runtime outputs")
        for o, val in zip(runtime, values):
            if o.lowered != "erased":
                env[o.name] = val

    def _components(self, sizes, items, what):
        if sum(sizes) != len(items):
            raise TypeError(f"{what}: component sizes {sizes} do not cover {len(items)} values")
        out, off = [], 0
        for s in sizes:
            out.append(items[off:off + s])
            off += s
        return out

    def _assign(self, env, a):
        ins = [self._value(env, v) for v in a.inputs]
        if a.call_symbol:                                                    # gpu.rs:894-916
            self._bind(env, a.outputs, self.call(a.call_symbol, _runtime(ins)))
            return
        if self._primitive(env, a.op, ins, a.outputs, getattr(a, "input_sizes", None)):
            return
        if a.op == "bool.ifc":                                               # ops/ifc.rs:11-41
            comps = self._components(a.input_sizes, ins, "bool.ifc")
            if len(comps) != 6:
                raise TypeError("bool.ifc expects 6 input components")
            true_env, true_fn, false_env, false_fn, flag, argument = comps
            [flag_value] = _runtime(flag)
            env_, fn_ = (true_env, true_fn) if flag_value else (false_env, false_fn)
            [fn_sym] = [v for v in fn_ if isinstance(v, FnSymbol)]
            self._apply(env, fn_sym, list(env_) + list(argument), a.outputs)
        elif a.op == "eval":                                                 # gpu.rs:986-991
            *args, fn_sym = ins
            self._apply(env, fn_sym, args, a.outputs)
        elif a.op == "reducec" and self.reduce is not None and any(isinstance(x, DeviceMem) for x in ins):
            self._bind(env, a.outputs, self.reduce(a, ins))
        elif a.op == "reducec":                                              # ops/reducec.rs:34-133
            comps = self._components(a.input_sizes, ins, "reducec")
            if len(comps) != 6:
                raise TypeError("reducec expects 6 input components")
            zero, add_env, add_fn, get_env, get_fn, n = comps
            [add_sym] = [v for v in add_fn if isinstance(v, FnSymbol)]
            [get_sym] = [v for v in get_fn if isinstance(v, FnSymbol)]
            [count] = _runtime(n)
            if len(zero) != len(a.outputs) or not a.outputs:
                raise TypeError("reducec: the zero input must match the accumulator arity")
            acc = list(zero)
            slots = [GpuVar(f"reduce_value_{o.name}", o.lowered) for o in a.outputs]
            nexts = [GpuVar(f"reduce_next_{o.name}", o.lowered) for o in a.outputs]
            scratch = {}
            for i in range(int(count)):
                self._apply(scratch, get_sym, list(get_env) + [i], slots)
                values = [scratch[s.name] for s in slots]
                self._apply(scratch, add_sym, list(add_env) + acc + values, nexts)
                acc = [scratch[x.name] for x in nexts]
            self._bind(env, a.outputs, acc)
        elif a.op == "materializec" and self.materialize is not None:       # ops/materializec.rs:84-145: len, env..., producer
            from .lowering import materializec_parts
            length, env_values, fn_sym = materializec_parts(a, ins)
            self._bind(env, a.outputs, [self.materialize(a, int(length), env_values, fn_sym)])
        else:
            raise NotScalar(f"`{a.op}` is not a scalar assignment")

    def _apply(self, env, fn_sym, inputs, outputs):
        """gpu.rs:918-968: a primitive symbol goes through the primitive table with the inputs as they stand; any other
        symbol is a generated program called with the runtime inputs only."""
        if not isinstance(fn_sym, FnSymbol):
            raise TypeError("function application needs a function symbol")
        if self._primitive(env, fn_sym.name, inputs, outputs, None):
            return
        self._bind(env, outputs, self.call(fn_sym.name, _runtime(inputs)))

    def _primitive(self, env, op, ins, outputs, input_sizes):
        if op in NO_OPS:
            return True
        if op in PRIMITIVES:
            self._bind(env, outputs, PRIMITIVES[op](*ins))
            return True
        if op.startswith("const.u64."):
            self._bind(env, outputs, [_parse_const(op, "const.u64.") & M64])
            return True
        if op.startswith("const.u32."):
            self._bind(env, outputs, [_parse_const(op, "const.u32.") & M32])
            return True
        if op == ":.ty":                                                     # gpu.rs:471-497
            [x] = _runtime(ins)
            for o in outputs:
                if o.lowered != "erased":
                    env[o.name] = x
            return True
        if op == "assert":                                                   # gpu.rs:449-458
            [flag] = ins
            if not flag:
                raise AssertFailed("catena assertion failed")
            return True
        if op == "u64.to-ix":                                                # gpu.rs:866-892: components [index, bound, proof]
            comps = self._components(input_sizes, ins, "u64.to-ix") if input_sizes else [[ins[0]]]
            [index] = _runtime(comps[0])
            self._bind(env, outputs, [index])
            return True
        if op == "row-major-index":                                          # ops/row_major.rs:9-28
            cols, row, col = _runtime(ins)
            self._bind(env, outputs, [(int(row) * int(cols) + int(col)) & M64])
            return True
        if op in ("row-major-row", "row-major-col"):                         # ops/row_major.rs:30-68 (division by 0: UB in C)
            cols, flat = _runtime(ins)
            if int(cols) == 0:
                raise UndefinedBehaviour("row-major division by zero columns")
            self._bind(env, outputs, [int(flat) // int(cols) if op == "row-major-row" else int(flat) % int(cols)])
            return True
        return False
