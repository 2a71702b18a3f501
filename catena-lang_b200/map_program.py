"""Register programs for the generic map kernel: what this backend does with a `materializec` whose producer no
prebuilt kernel matches.

The reference renders such a producer as C++ inside a one-thread-per-element kernel and compiles it with nvcc when the
Runtime is built (catena-lang/src/codegen/ops/materializec.rs:36-82; function application gpu.rs:918-968).  Here the
producer's lowered assignments are translated ONCE into a small register program — the same walk the host evaluator
(evaluator.py) does, emitting an instruction where the evaluator computes a value — and the kernel library's
`catena_b200_map_program_s` interprets it for every index (csrc/map_program.cu):

  primitive                        one instruction (the table of catena-lang/src/codegen/gpu.rs:322-447)
  constants, `*.one`, `bool.t/f`   preset registers
  program call, `eval`             inlined
  `bool.ifc`                       JZ / JMP around the two inlined functions (ops/ifc.rs:11-41)
  `reducec` inside the producer    a loop: acc = zero; for i < n: acc = add(env, acc, get(env, i)) (ops/reducec.rs:34-133)
  `row-major-index/row/col`        MUL + ADD / DIV / REM on u64 (ops/row_major.rs:9-68)
  `ix` on a buffer                 bounds-checked LOAD; buffers are known when the program is built, so `mem.cast.*` and
                                   `buf.*.cast-same-length` cost nothing and a buffer's length is a preset register

The environment of the producer (scalars and buffers) is bound at launch time: `MapProgram.launch(len, env)`.

By default a launch runs the program COMPILED: the library writes PTX for it and the driver compiles that for the device
(csrc/map_jit.cu; once per program and device), which is what the reference's nvcc step amounts to for one producer.
`CATENA_B200_MAP_COMPILED=0` in the environment runs every launch on the interpreter instead; both give the same bits.
"""
import ctypes as C
import os
import threading

import numpy as np

from .evaluator import NO_OPS, PRIMITIVES, UndefinedBehaviour, _parse_const, bits_f32, f32_bits
from .lowering import FnSymbol, GpuVar, Unsupported

# opcodes: enum catena_b200_map_op of include/catena_b200.h, in order
_OPS = ["HALT", "MOV", "JMP", "JZ", "ASSERT", "SELECT", "BOOL_NOT", "BOOL_AND", "BOOL_OR",
        "U64_ADD", "U64_SUB", "U64_MUL", "U64_DIV", "U64_REM", "U64_EQ", "U64_NE", "U64_LT", "U64_LTE", "U64_GT", "U64_GTE", "U64_TO_F32",
        "U32_ADD", "U32_SUB", "U32_MUL", "U32_AND", "U32_OR", "U32_XOR", "U32_NOT", "U32_SHL", "U32_SHR",
        "U32_EQ", "U32_NE", "U32_LT", "U32_LTE", "U32_GT", "U32_GTE", "U32_TO_F32",
        "F32_ADD", "F32_SUB", "F32_MUL", "F32_DIV", "F32_NEG", "F32_FMA", "F32_EQ", "F32_NE", "F32_LT", "F32_LTE", "F32_GT", "F32_GTE",
        "F32_ROUND_TO_U32", "LOAD_U64", "LOAD_F32", "MOV32", "SELECT32", "F32_MULADD", "F32_MULSUB", "F32_SUBMUL"]
OP = {name: i for i, name in enumerate(_OPS)}

# primitive -> opcode, for the primitives that are one instruction over their runtime inputs
_DIRECT = {
    "bool.not": "BOOL_NOT", "bool.and": "BOOL_AND", "bool.or": "BOOL_OR",
    "u64.add": "U64_ADD", "u64.sub": "U64_SUB", "u64.mul": "U64_MUL", "u64.eq": "U64_EQ", "u64.ne": "U64_NE", "u64.lt": "U64_LT",
    "u64.lte": "U64_LTE", "u64.gt": "U64_GT", "u64.gte": "U64_GTE", "u64.to-f32": "U64_TO_F32",
    "u32.add": "U32_ADD", "u32.sub": "U32_SUB", "u32.mul": "U32_MUL", "u32.and": "U32_AND", "u32.or": "U32_OR", "u32.xor": "U32_XOR",
    "u32.not": "U32_NOT", "u32.shl": "U32_SHL", "u32.shr": "U32_SHR", "u32.eq": "U32_EQ", "u32.ne": "U32_NE", "u32.lt": "U32_LT",
    "u32.lte": "U32_LTE", "u32.gt": "U32_GT", "u32.gte": "U32_GTE", "u32.to-f32": "U32_TO_F32",
    "f32.add": "F32_ADD", "f32.sub": "F32_SUB", "f32.mul": "F32_MUL", "f32.div": "F32_DIV", "f32.neg": "F32_NEG", "f32.fma": "F32_FMA",
    "f32.eq": "F32_EQ", "f32.ne": "F32_NE", "f32.lt": "F32_LT", "f32.lte": "F32_LTE", "f32.gt": "F32_GT", "f32.gte": "F32_GTE",
    "f32.round-to-u32": "F32_ROUND_TO_U32",
    "f32.select": "SELECT32", "u32.select": "SELECT32", "u64.select": "SELECT", "bool.select": "SELECT32",
}
# primitives whose single runtime output is their single runtime input (bitcasts included: registers hold bit patterns)
_ALIASES = {"bool.id", ":.forget", "u64.name", "ix.to-u64", "u32.bitcast-f32", "f32.bitcast-u32", ":.ty"}
_PRESETS = {"bool.t": 1, "bool.f": 0, "u64.zero": 0, "u64.one": 1, "u32.one": 1, "f32.one": 0x3F800000}
_ELEM = {"ptr<f32>": ("LOAD_F32", 4), "ptr<u64>": ("LOAD_U64", 8)}

MAX_REGS, MAX_INSNS, MAX_BUFFERS = 256, 2048, 16       # what the interpreter takes
MAX_REGS_COMPILED = 4096                                # a compiled kernel's registers are PTX virtual registers


def _mov(lowered):
    """bool / u32 / f32 values live in the low half of a register: their moves leave the high half alone"""
    return "MOV32" if lowered in ("f32", "u32", "bool") else "MOV"


class Insn(C.Structure):
    """catena_b200_map_insn_t"""
    _fields_ = [("op", C.c_uint16), ("dst", C.c_uint16), ("a", C.c_uint16), ("b", C.c_uint16), ("c", C.c_uint16),
                ("reserved", C.c_uint16), ("target", C.c_uint32)]


class _Buffer:
    """A buffer value while the program is built: slot of the launch's buffer table (+ the element kind once cast)."""
    __slots__ = ("slot", "lowered")

    def __init__(self, slot, lowered):
        self.slot, self.lowered = slot, lowered


_COMPILE_LOCK = threading.Lock()


class MapProgram:
    """A compiled producer.  `env_kinds` lists the runtime environment values the launch must supply, in order: 'f32',
    'u32', 'u64', 'bool' (scalars) or 'buffer'."""

    def __init__(self, producer, code, presets, n_regs, index_reg, result_reg, env_kinds, elem_bytes):
        self.producer, self.code, self.presets = producer, code, presets
        self.n_regs, self.index_reg, self.result_reg = n_regs, index_reg, result_reg
        self.env_kinds, self.elem_bytes = env_kinds, elem_bytes

    def init_registers(self, env):
        """Preset register values for one launch.  `env` holds one value per entry of `env_kinds`: a number, or for a
        buffer a (device pointer, length in bytes) pair."""
        if len(env) != len(self.env_kinds):
            raise TypeError(f"{self.producer}: expected {len(self.env_kinds)} environment values, got {len(env)}")
        init, buffers = [], []
        for what in self.presets:
            if what[0] == "const":
                init.append(what[1])
            elif what[0] == "env":
                value, kind = env[what[1]], self.env_kinds[what[1]]
                init.append(f32_bits(value) if kind == "f32" else int(value) & (0xFFFFFFFF if kind == "u32" else 0xFFFFFFFFFFFFFFFF))
            else:                                   # ("buflen", environment position, element bytes)
                init.append(int(env[what[1]][1]) // what[2])
        for value, kind in zip(env, self.env_kinds):
            if kind == "buffer":
                buffers.append((int(value[0] or 0), int(value[1])))
        return init, buffers

    def _spec(self, init):
        """The arguments every compiled-map entry point starts with; the returned arrays must outlive the call."""
        code = (Insn * len(self.code))(*self.code)
        init_arr = (C.c_uint64 * max(1, len(init)))(*init)
        is_const = (C.c_uint8 * max(1, len(self.presets)))(*[1 if what[0] == "const" else 0 for what in self.presets])
        n_buffers = sum(1 for kind in self.env_kinds if kind == "buffer")
        return [code, len(self.code), init_arr, is_const, len(init), self.n_regs, self.index_reg, self.result_reg, n_buffers, self.elem_bytes]

    def ptx(self):
        """The PTX text of the compiled kernel (needs no GPU).  Environment presets are kernel parameters, so any values do."""
        from . import check, lib
        init = [what[1] if what[0] == "const" else 0 for what in self.presets]
        spec = self._spec(init)
        need = C.c_uint64(0)
        check(lib().catena_b200_map_ptx_s(*spec, None, 0, C.byref(need)))
        text = C.create_string_buffer(need.value)
        check(lib().catena_b200_map_ptx_s(*spec, text, need.value, None))
        return text.value.decode()

    def compiled(self):
        """Handle of the kernel compiled for the current device (built on first use, kept for the program's lifetime)."""
        from . import check, lib
        device = int(lib().catena_b200_current_device())
        if device < 0:                       # no call has bound a device yet: the library's lazy default, device 0
            check(lib().catena_b200_init(0))
            device = 0
        with _COMPILE_LOCK:                 # two host threads launching a new program compile it once
            if not hasattr(self, "_kernels"):
                self._kernels = {}
            if device not in self._kernels:
                init = [what[1] if what[0] == "const" else 0 for what in self.presets]
                handle = C.c_void_p()
                check(lib().catena_b200_map_compile_s(*self._spec(init), C.byref(handle)))
                self._kernels[device] = handle
            return self._kernels[device]

    def __del__(self):
        for handle in getattr(self, "_kernels", {}).values():
            try:
                from . import lib
                lib().catena_b200_map_kernel_release(handle)
            except Exception:      # interpreter shutdown: the library may be gone already
                pass

    def launch(self, length, env, index0=0, compiled=None):
        """out[j] = producer(env..., index0 + j) for j < length on the device; returns the library's CatenaMem (owned by the
        caller).  `index0` is how a map shards over GPUs: contiguous index ranges, the same program on every rank.
        `compiled`: True = the program's own kernel, False = the interpreter, None = what CATENA_B200_MAP_COMPILED says
        (default: compiled)."""
        from . import CatenaMem, check, lib
        init, buffers = self.init_registers(env)
        init_arr = (C.c_uint64 * max(1, len(init)))(*init)
        bufs = (CatenaMem * max(1, len(buffers)))(*[CatenaMem(p, n) for p, n in buffers])
        out = CatenaMem()
        if compiled is None:
            compiled = os.environ.get("CATENA_B200_MAP_COMPILED", "1") != "0"
        if compiled and int(length) > 0:
            check(lib().catena_b200_map_kernel_launch_s(self.compiled(), init_arr, len(init), bufs, len(buffers), int(index0), int(length),
                                                        C.byref(out)))
            return out
        code = (Insn * len(self.code))(*self.code)
        check(lib().catena_b200_map_program_range_s(code, len(self.code), init_arr, len(init), self.n_regs, self.index_reg, self.result_reg,
                                                    bufs, len(buffers), self.elem_bytes, int(index0), int(length), C.byref(out)))
        return out


class _Builder:
    def __init__(self, modules):
        from .lowering import module_map
        self.by_name = modules if isinstance(modules, dict) else module_map(modules)
        self.code = []
        self.presets = []             # register k < len(presets) is preset: ("const", value) | ("env", position) | ("buflen", position, bytes)
        self.preset_regs = {}
        self.next_reg = None          # first temporary; set by _compile, which walks the producer twice
        self.fixed_presets = None     # pass 2: preset -> register, as pass 1 discovered them
        self.depth = 0

    # ---- registers ----
    def preset(self, what):
        if self.fixed_presets is not None:
            return self.fixed_presets[what]
        if what not in self.preset_regs:
            self.preset_regs[what] = len(self.presets)
            self.presets.append(what)
        return self.preset_regs[what]

    def const(self, value):
        return self.preset(("const", int(value)))

    def fresh(self):
        r = self.next_reg
        self.next_reg += 1
        if self.fixed_presets is not None and self.next_reg > MAX_REGS_COMPILED:
            raise Unsupported("the producer needs more than 4096 registers")
        return r

    def const_value(self, reg):
        what = self.presets[reg] if reg < len(self.presets) else None
        return what[1] if what is not None and what[0] == "const" else None

    def fold(self, op, regs, outputs):
        """A primitive over constants is a constant: evaluated now with the host evaluator's table, unless the reference's
        generated code leaves it undefined for these operands (then it stays an instruction and is reported at run time)."""
        values = [self.const_value(x) for x in regs]
        if not values or any(v is None for v in values):
            return None
        family = op.split(".")[0]
        typed = [bits_f32(v) if family == "f32" else v for v in values]
        if op.endswith(".select"):
            typed[0] = values[0]
        try:
            [result] = PRIMITIVES[op](*typed)
        except (UndefinedBehaviour, ZeroDivisionError):
            return None
        [out] = [o for o in outputs if o.lowered != "erased"]
        return self.const(f32_bits(result) if out.lowered == "f32" else int(result))

    def emit(self, op, dst=0, a=0, b=0, c=0, target=0):
        if len(self.code) >= MAX_INSNS - 1:
            raise Unsupported("the producer needs more than 2048 instructions")
        self.code.append(Insn(OP[op], dst, a, b, c, 0, target))
        return len(self.code) - 1

    # ---- the evaluator's walk, emitting instead of computing ----
    def call(self, name, args):
        from .lowering import find_module
        module = find_module(self.by_name, name)
        if module is None:
            raise Unsupported(f"no lowered module for `{name}`")
        if self.depth > 64:
            raise Unsupported(f"`{name}`: calls nest deeper than 64 (recursion?)")
        fn = module.entry
        sources = [s for s in fn.sources if s.lowered != "erased"]
        if len(sources) != len(args):
            raise Unsupported(f"{fn.name}: expected {len(sources)} runtime inputs, got {len(args)}")
        env = {s.name: a for s, a in zip(sources, args)}
        self.depth += 1
        for a in fn.assignments:
            self.assign(env, a)
        self.depth -= 1
        return [env[t.name] for t in fn.targets if t.lowered != "erased"]

    def value(self, env, v):
        if isinstance(v, FnSymbol):
            return v
        return None if v.lowered == "erased" else env[v.name]

    @staticmethod
    def runtime(values):
        return [v for v in values if v is not None and not isinstance(v, FnSymbol)]

    def bind(self, env, outputs, values):
        runtime = [o for o in outputs if o.lowered != "erased"]
        if len(values) == len(outputs):
            runtime = outputs
        elif len(values) != len(runtime):
            raise Unsupported(f"{len(values)} values for {len(runtime)} runtime outputs")
        for o, val in zip(runtime, values):
            if o.lowered != "erased":
                env[o.name] = val

    @staticmethod
    def components(sizes, items, what):
        if sizes is None or sum(sizes) != len(items):
            raise Unsupported(f"{what}: component sizes {sizes} do not cover {len(items)} values")
        out, off = [], 0
        for s in sizes:
            out.append(items[off:off + s])
            off += s
        return out

    def assign(self, env, a):
        ins = [self.value(env, v) for v in a.inputs]
        if a.call_symbol:
            self.bind(env, a.outputs, self.call(a.call_symbol, self.runtime(ins)))
        elif self.primitive(env, a.op, ins, a.outputs, a.input_sizes):
            pass
        elif a.op == "bool.ifc":
            comps = self.components(a.input_sizes, ins, "bool.ifc")
            if len(comps) != 6:
                raise Unsupported("bool.ifc expects 6 input components")
            true_env, true_fn, false_env, false_fn, flag, argument = comps
            [flag_reg] = self.runtime(flag)
            outs = [o for o in a.outputs if o.lowered != "erased"]
            dst = [self.fresh() for _ in outs]
            jz = self.emit("JZ", a=flag_reg)
            self.branch(true_env, true_fn, argument, outs, dst)
            jmp = self.emit("JMP")
            self.code[jz].target = len(self.code)
            self.branch(false_env, false_fn, argument, outs, dst)
            self.code[jmp].target = len(self.code)
            self.bind(env, outs, dst)
        elif a.op == "eval":
            *args, fn_sym = ins
            self.apply(env, fn_sym, args, a.outputs)
        elif a.op == "reducec":
            self.reduce(env, a, ins)
        else:
            raise Unsupported(f"`{a.op}` cannot run inside a map kernel")

    def branch(self, env_values, fn_values, argument, outs, dst):
        [fn_sym] = [v for v in fn_values if isinstance(v, FnSymbol)]
        scratch = {}
        self.apply(scratch, fn_sym, list(env_values) + list(argument), outs)
        for o, d in zip(outs, dst):
            src = scratch[o.name]
            if isinstance(src, _Buffer):
                raise Unsupported("bool.ifc that chooses between buffers")
            self.emit(_mov(o.lowered), dst=d, a=src)

    def reduce(self, env, a, ins):
        comps = self.components(a.input_sizes, ins, "reducec")
        if len(comps) != 6:
            raise Unsupported("reducec expects 6 input components")
        zero, add_env, add_fn, get_env, get_fn, n = comps
        [add_sym] = [v for v in add_fn if isinstance(v, FnSymbol)]
        [get_sym] = [v for v in get_fn if isinstance(v, FnSymbol)]
        [count] = self.runtime(n)
        if len(zero) != len(a.outputs) or not a.outputs or any(isinstance(z, _Buffer) for z in zero):
            raise Unsupported("reducec: the zero input must match a scalar accumulator")
        acc = [self.fresh() for _ in zero]
        for d, z, o in zip(acc, zero, a.outputs):
            self.emit(_mov(o.lowered), dst=d, a=z)
        counter, more = self.fresh(), self.fresh()
        self.emit("MOV", dst=counter, a=self.const(0))
        top = self.emit("U64_LT", dst=more, a=counter, b=count)
        leave = self.emit("JZ", a=more)
        slots = [GpuVar(f"reduce_value_{o.name}", o.lowered) for o in a.outputs]
        nexts = [GpuVar(f"reduce_next_{o.name}", o.lowered) for o in a.outputs]
        scratch = {}
        self.apply(scratch, get_sym, list(get_env) + [counter], slots)
        self.apply(scratch, add_sym, list(add_env) + acc + [scratch[s.name] for s in slots], nexts)
        for d, x in zip(acc, nexts):
            self.emit(_mov(x.lowered), dst=d, a=scratch[x.name])
        self.emit("U64_ADD", dst=counter, a=counter, b=self.const(1))
        self.emit("JMP", target=top)
        self.code[leave].target = len(self.code)
        self.bind(env, a.outputs, acc)

    def apply(self, env, fn_sym, inputs, outputs):
        if not isinstance(fn_sym, FnSymbol):
            raise Unsupported("function application needs a function symbol")
        if self.primitive(env, fn_sym.name, inputs, outputs, None):
            return
        self.bind(env, outputs, self.call(fn_sym.name, self.runtime(inputs)))

    def primitive(self, env, op, ins, outputs, input_sizes):
        if op in NO_OPS:
            return True
        rt = self.runtime(ins)
        if op in _DIRECT:
            if any(isinstance(x, _Buffer) for x in rt):
                raise Unsupported(f"`{op}` applied to a buffer")
            folded = self.fold(op, rt, outputs)
            if folded is not None:
                self.bind(env, outputs, [folded])
                return True
            d = self.fresh()
            regs = rt + [0] * (3 - len(rt))
            self.emit(_DIRECT[op], dst=d, a=regs[0], b=regs[1], c=regs[2])
            self.bind(env, outputs, [d])
            return True
        if op in _PRESETS:
            self.bind(env, outputs, [self.const(_PRESETS[op])])
            return True
        if op.startswith("const.u64."):
            self.bind(env, outputs, [self.const(_parse_const(op, "const.u64.") & 0xFFFFFFFFFFFFFFFF)])
            return True
        if op.startswith("const.u32."):
            self.bind(env, outputs, [self.const(_parse_const(op, "const.u32.") & 0xFFFFFFFF)])
            return True
        if op in _ALIASES:
            [x] = rt
            for o in outputs:
                if o.lowered != "erased":
                    env[o.name] = x
            return True
        if op == "bool.copy":
            [x] = rt
            self.bind(env, outputs, [x, x])
            return True
        if op == "assert":
            [flag] = rt
            self.emit("ASSERT", a=flag)
            return True
        if op == "ix.zero":
            self.bind(env, outputs, [self.const(0)])
            return True
        if op == "u64.to-ix":
            comps = self.components(input_sizes, ins, "u64.to-ix") if input_sizes else [[ins[0]]]
            [index] = self.runtime(comps[0])
            self.bind(env, outputs, [index])
            return True
        if op == "row-major-index":
            cols, row, col = rt
            t, d = self.fresh(), self.fresh()
            self.emit("U64_MUL", dst=t, a=row, b=cols)
            self.emit("U64_ADD", dst=d, a=t, b=col)
            self.bind(env, outputs, [d])
            return True
        if op in ("row-major-row", "row-major-col"):
            cols, flat = rt
            d = self.fresh()
            self.emit("U64_DIV" if op == "row-major-row" else "U64_REM", dst=d, a=flat, b=cols)
            self.bind(env, outputs, [d])
            return True
        if op == "ix":
            index, buffer = rt
            if not isinstance(buffer, _Buffer) or buffer.lowered not in _ELEM:
                raise Unsupported("`ix` needs a typed buffer (u64 or f32 elements)")
            d = self.fresh()
            self.emit(_ELEM[buffer.lowered][0], dst=d, a=index, b=buffer.slot)
            self.bind(env, outputs, [d])
            return True
        if op in ("mem.cast.u64", "mem.cast.f32"):
            [mem] = rt
            if not isinstance(mem, _Buffer):
                raise Unsupported(f"`{op}` of something that is not a buffer")
            lowered = "ptr<u64>" if op.endswith("u64") else "ptr<f32>"
            length = self.preset(("buflen", mem.slot, _ELEM[lowered][1]))
            self.bind(env, outputs, [length, _Buffer(mem.slot, lowered)])
            return True
        if op in ("buf.u64.cast-same-length", "buf.f32.cast-same-length"):
            buffer = rt[0]
            self.bind(env, outputs, [buffer])
            return True
        return False


_READS_B = {OP[n] for n in _OPS if n not in ("HALT", "MOV", "MOV32", "JMP", "JZ", "ASSERT", "BOOL_NOT", "U64_TO_F32", "U32_NOT", "U32_TO_F32",
                                              "F32_NEG", "F32_ROUND_TO_U32", "LOAD_U64", "LOAD_F32")}
_READS_C = {OP["SELECT"], OP["SELECT32"], OP["F32_FMA"], OP["F32_MULADD"], OP["F32_MULSUB"], OP["F32_SUBMUL"]}
_NO_WRITE = {OP["HALT"], OP["JMP"], OP["JZ"], OP["ASSERT"]}


def _reads(c):
    out = [] if c.op in (OP["HALT"], OP["JMP"]) else [c.a]
    if c.op in _READS_B:
        out.append(c.b)
    if c.op in _READS_C:
        out.append(c.c)
    return out


def _fuse_mul_add(code, result_reg):
    """Straight-line code before register reuse (every register is written once): an F32_MUL whose only reader is an F32_ADD /
    F32_SUB sinks into it as one instruction (two roundings, as before: not an fma) — one dispatch and one round trip through
    the register file less.  A sum takes at most one product."""
    uses, reader = {}, {}
    for k, c in enumerate(code):
        for reg in _reads(c):
            uses[reg] = uses.get(reg, 0) + 1
            reader.setdefault(reg, k)
    uses[result_reg] = uses.get(result_reg, 0) + 1
    fused = {}                                    # index of the sum -> index of the product it takes
    for k, c in enumerate(code):
        if c.op != OP["F32_MUL"] or uses.get(c.dst) != 1 or c.dst == result_reg:
            continue
        j = reader[c.dst]
        n = code[j]
        if j > k and j not in fused and n.op in (OP["F32_ADD"], OP["F32_SUB"]) and (n.a == c.dst) != (n.b == c.dst):
            fused[j] = k
    gone = set(fused.values())
    out = []
    for k, c in enumerate(code):
        if k in gone:
            continue
        if k in fused:
            m = code[fused[k]]
            other = c.b if c.a == m.dst else c.a
            op = "F32_MULADD" if c.op == OP["F32_ADD"] else ("F32_MULSUB" if c.a == m.dst else "F32_SUBMUL")
            out.append(Insn(OP[op], c.dst, m.a, m.b, other, 0, 0))
        else:
            out.append(c)
    return out


def _reuse_registers(code, n_init, index_reg, result_reg):
    """Straight-line code only: every temporary is written once, so a register is free again after its last read.  Keeps
    the preset registers and the index register where they are; returns (code, number of registers, result register)."""
    reads = _reads
    last = {}
    for k, c in enumerate(code):
        for reg in reads(c):
            last[reg] = k
    last[result_reg] = len(code)
    mapping, free, top = {index_reg: index_reg}, [], index_reg + 1
    out = []
    for k, c in enumerate(code):
        used = reads(c)
        a, b, cc = (mapping.get(c.a, c.a) if c.a in used else 0), c.b, (mapping.get(c.c, c.c) if c.c in used else 0)
        if c.op in _READS_B:
            b = mapping.get(c.b, c.b)
        for reg in sorted(set(used)):
            if reg >= n_init and reg != index_reg and last.get(reg) == k and reg in mapping:
                free.append(mapping[reg])
        dst = 0
        if c.op not in _NO_WRITE:
            if free:
                dst = free.pop()
            else:
                dst, top = top, top + 1
            mapping[c.dst] = dst
        out.append(Insn(c.op, dst, a, b, cc, 0, c.target))
    return out, top, mapping.get(result_reg, result_reg)


def _compile(modules, name, env_vars, elem_lowered, body):
    """Shared driver: binds `env_vars` (GpuVars) to preset registers / buffer slots, lets `body(builder, args, index)` emit
    the code and return the result register, finishes with HALT, folds the two passes and the register reuse."""
    elem_bytes = {"u64": 8, "f32": 4, "u32": 4, "bool": 4}.get(elem_lowered)
    if elem_bytes is None:
        raise Unsupported(f"a buffer of `{elem_lowered}` elements")
    env_kinds, buffer_slot = [], {}
    for position, v in enumerate(env_vars):
        if v.lowered in ("f32", "u32", "u64", "bool"):
            env_kinds.append(v.lowered)
        elif v.lowered == "mem" or v.lowered in _ELEM:
            env_kinds.append("buffer")
            buffer_slot[position] = len(buffer_slot)
        else:
            raise Unsupported(f"environment value of type `{v.lowered}`")
    if len(buffer_slot) > MAX_BUFFERS:
        raise Unsupported("more than 16 buffers in the environment")

    def run(builder):
        args = []
        for position, v in enumerate(env_vars):
            if position in buffer_slot:
                args.append(_Buffer(buffer_slot[position], v.lowered))
            else:
                args.append(builder.preset(("env", position)))
        index = builder.fresh()
        got = body(builder, args, index)
        builder.emit("HALT")
        if isinstance(got, _Buffer):
            raise Unsupported("the producer returns a buffer")
        return index, got

    # pass 1 discovers the presets (constants appear while walking), pass 2 emits with the registers behind them
    first = _Builder(modules)
    first.next_reg = 1 << 20              # away from the preset numbers; pass 1 only discovers the presets
    run(first)
    presets = list(first.presets)
    second = _Builder(modules)
    second.fixed_presets = {what: k for k, what in enumerate(presets)}
    second.presets = presets
    second.next_reg = len(presets)
    if second.next_reg >= MAX_REGS_COMPILED:
        raise Unsupported("the producer needs more than 4096 registers")
    index, result = run(second)
    code, n_regs = second.code, max(second.next_reg, 1)
    if not any(c.op in (OP["JMP"], OP["JZ"]) for c in code):
        code = _fuse_mul_add(code, result)
        code, n_regs, result = _reuse_registers(code, len(presets), index, result)
    # ("buflen", slot, bytes) presets name buffer slots; launches index the environment: translate
    slot_position = {slot: position for position, slot in buffer_slot.items()}
    presets = [("buflen", slot_position[w[1]], w[2]) if w[0] == "buflen" else w for w in presets]
    return MapProgram(name, code, presets, n_regs, index, result, env_kinds, elem_bytes)


def compile_producer(modules, producer, env_vars, elem_lowered):
    """Register program for `out[i] = producer(env_vars..., i)`.

    `env_vars`: the runtime values of the materializec's environment component as `lowering.GpuVar`s (their `lowered`
    types decide how a launch binds them); `elem_lowered`: element type of the buffer produced ('u64', 'f32', 'u32').
    Raises `lowering.Unsupported` for a producer a map kernel cannot run (an allocation inside it, a buffer chosen at run
    time, too many registers or instructions)."""
    if elem_lowered == "bool":
        raise Unsupported("materializec of `bool` elements")

    def body(builder, args, index):
        result = GpuVar("value", elem_lowered)
        scratch = {}
        builder.apply(scratch, FnSymbol(producer), args + [index], [result])
        return scratch[result.name]

    return _compile(modules, producer, env_vars, elem_lowered, body)


def fold_inputs(assign):
    """The runtime inputs of a `reducec` assignment, in order: what a launch of its fold programs binds."""
    return [v for v in assign.inputs if isinstance(v, GpuVar) and v.lowered != "erased"]


def compile_fold(modules, assign, component):
    """Register program whose ONE element is component `component` of a `reducec`'s result: the sequential left fold
    `acc = zero; for i < n: acc = add(add_env, acc, get(get_env, i))` (catena-lang/src/codegen/ops/reducec.rs:34-133) as a loop,
    run by one thread — the reference runs the same loop on one host core.  For folds whose closures read device buffers
    and match no prebuilt fold kernel.  Launch with length 1 and the values of `fold_inputs(assign)`."""
    outs = [o for o in assign.outputs if o.lowered != "erased"]
    if not 0 <= component < len(outs):
        raise Unsupported("reducec: no such accumulator component")
    env_vars = fold_inputs(assign)

    def body(builder, args, index):
        env, k = {}, 0
        for v in assign.inputs:
            if isinstance(v, GpuVar) and v.lowered != "erased":
                env[v.name] = args[k]
                k += 1
        builder.assign(env, assign)
        return env[outs[component].name]

    return _compile(modules, f"reducec[{component}]", env_vars, outs[component].lowered, body)


def compile_getter(modules, assign):
    """Register program for out[i] = get(get_env..., i) of a `reducec` with ONE accumulator component: the first stage of a
    fold whose `add` is a prebuilt kernel's (the second stage folds the materialised values).  Launch with the values of the
    runtime variables of the getter's environment component."""
    if assign.input_sizes is None or len(assign.input_sizes) != 6:
        raise Unsupported("reducec expects 6 input components")
    outs = [o for o in assign.outputs if o.lowered != "erased"]
    if len(outs) != 1:
        raise Unsupported("a two-stage fold has one accumulator component")
    sizes, items = assign.input_sizes, list(assign.inputs)
    begin = sum(sizes[:3])
    get_env = [v for v in items[begin:begin + sizes[3]] if isinstance(v, GpuVar) and v.lowered != "erased"]
    [get_fn] = [v for v in items[begin + sizes[3]:begin + sizes[3] + sizes[4]] if isinstance(v, FnSymbol)]
    return compile_producer(modules, get_fn.name, get_env, outs[0].lowered), get_env
