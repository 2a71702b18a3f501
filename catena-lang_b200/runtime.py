"""Host-side mirror of the reference's runtime surface over the prebuilt kernel library.

Names, argument meaning and error behaviour follow catena-lang/src/runtime:
  Runtime.from_sources / Runtime.new / exec / mem_f32 / mem_u64   runtime.rs:104-236
  Value, ValueKind                                                value.rs:5-73
  Mem.to_f32_vec / to_u64_vec                                     mem.rs:43-70
  ExecError variants                                              runtime.rs:80-102
  GpuDialect {Hip, Cuda}                                          codegen/mod.rs:50-54

What differs, by design of a native lowering that SELECTS prebuilt sm_100a kernels instead of
generating and compiling C++ per Runtime (runtime.rs:123-164, artifact.rs:56-103):
  * `from_sources` does not run the catena compiler (its front end, the third-party `metacat`
    crate, is Rust and not part of this build).  It scans the sources for `(def program <name>`
    and builds the signature table (signature.rs:18-61) from the catalogue of programs the library
    ships; a program it has no kernel for stays out of the table, so `exec` reports
    UnknownSourceFunction for it.  The stdlib entry points are always present.
  * `GpuDialect.Hip` is refused with InitError (no multi-backend dispatch).
  * `Mem` owns device memory (cudaMalloc pool) and copies on `to_*_vec`, instead of dereferencing
    managed memory.  Like the Rust API, `exec` consumes its `Mem` arguments: they are freed when
    the call returns (runtime.rs:175-179, mem.rs:119-125).
"""
import ctypes as C
import enum
import re

import numpy as np


class GpuDialect(enum.Enum):
    Hip = "hip"
    Cuda = "cuda"


class ValueKind(enum.Enum):
    Bool = "Bool"
    U32 = "U32"
    U64 = "U64"
    F32 = "F32"
    Mem = "Mem"


class InitError(RuntimeError):
    pass


class ExecError(RuntimeError):
    """kind is one of UnknownSourceFunction, TypeMismatch, InputArityMismatch, OutputArityMismatch
    (runtime.rs:80-102) or Device (a status from the library; the reference would have trapped)."""

    def __init__(self, kind, message, status=None):
        super().__init__(message)
        self.kind = kind
        self.status = status


class Mem:
    """Owned device buffer: fat pointer {data, len_bytes} (mem.rs:38-41)."""

    def __init__(self, raw=None):
        from . import CatenaMem
        self.raw = raw if raw is not None else CatenaMem()

    @property
    def len_bytes(self):
        return int(self.raw.len)

    def is_null(self):
        return not self.raw.data

    def to_f32_vec(self):
        from . import download
        return download(self.raw, np.float32)

    def to_u64_vec(self):
        from . import download
        return download(self.raw, np.uint64)

    def to_array(self, dtype, out=None):
        from . import download
        return download(self.raw, dtype, out=out)

    def free(self):
        from . import CatenaMem, free
        if self.raw.data:
            free(self.raw)
            self.raw = CatenaMem()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Value:
    """Tagged runtime value accepted at program boundaries (value.rs:5-11)."""

    __slots__ = ("kind", "v")

    def __init__(self, kind, v):
        self.kind = kind
        self.v = v

    @staticmethod
    def bool(v):
        return Value(ValueKind.Bool, 1 if v else 0)

    @staticmethod
    def u32(v):
        return Value(ValueKind.U32, int(v) & 0xFFFFFFFF)

    @staticmethod
    def u64(v):
        return Value(ValueKind.U64, int(v) & 0xFFFFFFFFFFFFFFFF)

    @staticmethod
    def f32(v):
        return Value(ValueKind.F32, float(np.float32(v)))

    @staticmethod
    def mem(m):
        return Value(ValueKind.Mem, m)

    @staticmethod
    def of(x):
        """`.into()` of the Rust API: bool -> Bool, int -> U64, float -> F32, Mem -> Mem."""
        if isinstance(x, Value):
            return x
        if isinstance(x, Mem):
            return Value.mem(x)
        if isinstance(x, (bool, np.bool_)):
            return Value.bool(x)
        if isinstance(x, np.uint32):
            return Value.u32(x)
        if isinstance(x, (int, np.integer)):
            return Value.u64(x)
        if isinstance(x, (float, np.floating)):
            return Value.f32(x)
        raise TypeError(f"cannot convert {type(x).__name__} into a catena Value")

    def __repr__(self):
        return f"Value.{self.kind.value}({self.v!r})"


K = ValueKind
# Catalogue: hexpr source name -> (inputs, outputs).  Symbols follow codegen/mod.rs:379-388.
# The first block is the stdlib (always registered, stdlib.rs:47-66); the second block is programs a
# user source must define for them to be callable (the reference's test program and the
# beyond-reference tensor-core / attention programs).
_SCALAR = ([K.F32], [K.F32])
STDLIB = {name: _SCALAR for name in [
    "math.sin-approx", "math.cos-approx", "math.sin-approx-full-nonneg", "math.sin-approx-full",
    "math.log-approx", "math.exp-approx-nonneg", "math.exp-approx", "math.exp2-approx", "math.log2-approx",
    "math.sqrt", "nn.sigmoid", "nn.silu", "nn.tanh", "nn.gelu-approx"]}
STDLIB.update({
    "math.powf": ([K.F32, K.F32], [K.F32]),
    "nn.softmax": ([K.Mem], [K.Mem]),
    "nn.rmsnorm": ([K.Mem], [K.Mem]),
    "sum-f32": ([K.Mem], [K.F32]),
    "mean-f32": ([K.Mem], [K.F32]),
    "max-f32": ([K.Mem], [K.F32]),
    "tensor.broadcast-f32": ([K.F32, K.U64], [K.Mem]),
    "tensor.arange-f32": ([K.U64], [K.Mem]),
    "tensor.slice-f32": ([K.Mem, K.U64, K.U64], [K.Mem]),
    "tensor.concat-f32": ([K.Mem, K.Mem], [K.Mem]),
    "tensor.argmax-f32": ([K.Mem], [K.U64]),
})
USER_PROGRAMS = {
    "matmul-2x2-via-mem": ([K.Mem, K.Mem, K.U64, K.U64, K.U64, K.U64, K.U64, K.U64], [K.Mem]),
    "matmul-right-identity-2x2-via-mem": ([K.Mem, K.U64, K.U64], [K.Mem]),
    "matmul-left-identity-2x2-via-mem": ([K.Mem, K.U64, K.U64], [K.Mem]),
    "gemm-bf16-rc": ([K.Mem, K.Mem, K.U64, K.U64, K.U64], [K.Mem]),
    "gemm-i8-rc": ([K.Mem, K.Mem, K.U64, K.U64, K.U64], [K.Mem]),
    "attn-decode-bf16": ([K.Mem, K.Mem, K.Mem, K.U64, K.U64, K.U64, K.U64, K.U64], [K.Mem]),
}

_DEF_RE = re.compile(r"\(\s*def\s+program\s+([^\s:()]+)")

_CTYPE = {K.Bool: C.c_uint8, K.U32: C.c_uint32, K.U64: C.c_uint64, K.F32: C.c_float}


class Runtime:
    def __init__(self, signatures):
        from . import lib
        self._lib = lib()
        self.signatures = signatures
        self._map_programs = {}          # id(materializec assignment) -> map_program.MapProgram
        self._map_eval = None
        self._map_outputs = {}           # device pointer -> CatenaMem of the buffers the current exec materialised

    @classmethod
    def new(cls, paths, dialect=GpuDialect.Cuda):
        texts = []
        for p in paths:
            with open(p, "r", encoding="utf-8") as fh:
                texts.append(fh.read())
        return cls.from_sources(texts, dialect)

    @classmethod
    def from_sources(cls, sources, dialect=GpuDialect.Cuda):
        if dialect is not GpuDialect.Cuda:
            raise InitError("GpuDialect.Hip is not supported: this backend only selects prebuilt sm_100a CUDA kernels")
        from . import symbol_for
        table = {name: (symbol_for(name), ins, outs) for name, (ins, outs) in STDLIB.items()}
        for text in sources:
            for name in _DEF_RE.findall(text):
                if name in USER_PROGRAMS:
                    ins, outs = USER_PROGRAMS[name]
                    table[name] = (symbol_for(name), ins, outs)
        return cls(table)

    @classmethod
    def from_modules(cls, modules, sources=(), dialect=GpuDialect.Cuda):
        """Registers LOWERED modules (`lowering.GpuModule`, the reference's IR after `codegen::codegen`,
        codegen/mod.rs:107-146) next to what `from_sources` registers.  Every module with a source name whose runtime
        interface is made of `ValueKind`s (signature.rs:63-72) becomes callable through `exec`: the lowering selector
        picks its plan — the kernel library's entry point for the recognised kernel shapes, the host evaluator
        (evaluator.py) for scalar modules, as the reference runs non-materialize code on the host.  A module no plan
        exists for is an InitError (the reference would have generated source for it; this backend ships no generator)."""
        from . import lib
        from .evaluator import Evaluator
        from .lowering import ENTRY_SIGNATURE, Unsupported, module_map, select
        rt = cls.from_sources(sources, dialect)
        mm = module_map(modules)
        evaluator = Evaluator(modules)
        kinds = {"bool": K.Bool, "u32": K.U32, "u64": K.U64, "f32": K.F32, "mem": K.Mem}
        for m in modules:
            if not m.source_name:
                continue
            ins = [v.lowered for v in m.entry.sources if v.lowered != "erased"]
            outs = [v.lowered for v in m.entry.targets if v.lowered != "erased"]
            if any(t not in kinds for t in ins + outs):
                continue                                   # a `buf` pointer on the boundary: internal, no signature
            try:
                plan = select(m, modules=mm)
            except Unsupported as exc:
                raise InitError(f"no prebuilt kernel or host plan for program '{m.source_name}': {exc}") from exc
            if plan.kernel == "host_scalar":
                rt.signatures[m.source_name] = (plan.symbol, [kinds[t] for t in ins], [kinds[t] for t in outs],
                                                (lambda args, _name=m.name: evaluator.call(_name, args)))
                continue
            if plan.kernel == "map_unary" and ins == ["mem"] and outs == ["mem"]:
                def run_map(args, _op=plan.notes[0].encode()):
                    from . import CatenaMem, check
                    from .evaluator import DeviceMem
                    raw = CatenaMem()
                    check(rt._lib.catena_b200_map_f32_s(_op, CatenaMem(args[0].ptr or None, args[0].nbytes), C.byref(raw)))
                    if raw.data:
                        rt._map_outputs[int(raw.data)] = raw
                    return [DeviceMem(raw.data, raw.len)]
                rt.signatures[m.source_name] = (plan.symbol, [K.Mem], [K.Mem], run_map)
                continue
            if plan.kernel in ("host_with_map_kernels", "map_unary"):
                # the producers' register programs are built now, so that a producer the map kernel cannot run is an
                # InitError and `exec` only binds the environment and launches
                from .lowering import _touches_memory, fold_plan_for, map_program_for
                for a in m.entry.assignments:
                    if a.op == "materializec":
                        rt._map_programs[id(a)] = map_program_for(a, mm)
                    elif a.op == "reducec" and _touches_memory(a):
                        rt._map_programs[id(a)] = fold_plan_for(a, mm)
                rt.signatures[m.source_name] = (plan.symbol, [kinds[t] for t in ins], [kinds[t] for t in outs],
                                                (lambda args, _name=m.name: rt._map_evaluator(modules).call(_name, args)))
                continue
            entry = plan.entry
            if entry is None or ENTRY_SIGNATURE.get(entry) != (ins, outs) or not hasattr(lib(), entry):
                raise InitError(f"program '{m.source_name}' lowers to {plan.kernel}, which the library has no entry point for "
                                f"with the interface {ins} -> {outs}")
            rt.signatures[m.source_name] = (entry, [kinds[t] for t in ins], [kinds[t] for t in outs])
        return rt

    # -- memory constructors (runtime.rs:166-172; mem_bytes is additive: Mem is untyped bytes) --
    def mem_f32(self, values):
        return self.mem_bytes(np.ascontiguousarray(values, dtype=np.float32))

    def mem_u64(self, values):
        return self.mem_bytes(np.ascontiguousarray(values, dtype=np.uint64))

    def mem_bytes(self, array):
        from . import upload
        return Value.mem(Mem(upload(array)))

    def exec(self, name, args, n_outputs=None):
        """Runs a source-level `program` definition (runtime.rs:175-236) and returns the list of its
        outputs.  `n_outputs` plays the role of the Rust const generic N."""
        sig = self.signatures.get(name)
        if sig is None:
            raise ExecError("UnknownSourceFunction", f"Unknown source function '{name}'")
        symbol, ins, outs = sig[:3]
        host = sig[3] if len(sig) > 3 else None
        args = [Value.of(a) for a in args]
        if len(args) != len(ins):
            raise ExecError("InputArityMismatch", f"Function '{name}' expected {len(ins)} inputs, got {len(args)}")
        if n_outputs is not None and n_outputs != len(outs):
            raise ExecError("OutputArityMismatch", f"Function '{name}' expected {len(outs)} outputs, got {n_outputs}")
        for index, (value, expected) in enumerate(zip(args, ins)):
            if value.kind is not expected:
                raise ExecError("TypeMismatch", f"Argument {index} expected {expected.value}, got {value.kind.value}")
        if host is not None:
            return self._exec_on_host(name, host, args, outs)
        from . import CatenaMem
        cargs = []
        for value in args:
            if value.kind is K.Mem:
                cargs.append(value.v.raw)
            else:
                cargs.append(_CTYPE[value.kind](value.v))
        couts = [CatenaMem() if kind is K.Mem else _CTYPE[kind](0) for kind in outs]
        fn = getattr(self._lib, symbol)
        self._lib.catena_b200_clear_status()
        fn(*cargs, *[C.byref(o) for o in couts])
        status = self._lib.catena_b200_last_status()
        # inputs are moved into exec and dropped on return (runtime.rs:175-179)
        for value in args:
            if value.kind is K.Mem:
                value.v.free()
        if status != 0:
            from . import status_string
            raise ExecError("Device", f"program '{name}' failed: {status_string(status)}", status)
        results = []
        for kind, o in zip(outs, couts):
            if kind is K.Mem:
                results.append(Value.mem(Mem(o)))
            elif kind is K.F32:
                results.append(Value.f32(o.value))
            else:
                results.append(Value(kind, int(o.value)))
        return results

    def _map_evaluator(self, modules):
        """Host evaluator whose `materializec` launches the generic map kernel with the producer's register program."""
        if self._map_eval is None:
            from .evaluator import DeviceMem, Evaluator, _runtime, f32_bits
            from .lowering import FnSymbol

            def materialize(assign, length, env_values, fn_sym):
                program = self._map_programs[id(assign)]
                env = [(v.ptr, v.nbytes) if isinstance(v, DeviceMem) else v for v in env_values if v is not None]
                raw = program.launch(length, env)
                if raw.data:
                    self._map_outputs[int(raw.data)] = raw
                return DeviceMem(raw.data, raw.len, {8: np.uint64, 4: np.float32}[program.elem_bytes])

            def bind(values):
                return [(v.ptr, v.nbytes) if isinstance(v, DeviceMem) else v for v in values if v is not None and not isinstance(v, FnSymbol)]

            def scalar_of(raw, lowered):
                from . import download, free
                value = download(raw, np.float32 if lowered == "f32" else np.uint64 if lowered == "u64" else np.uint32)[0]
                free(raw)
                return np.float32(value) if lowered == "f32" else int(value)

            def reduce(assign, ins):
                """A `reducec` over device buffers (see lowering.FoldPlan): staged through a prebuilt fold when `add` is one
                and the fold is long enough to be worth two launches, else the sequential loop on one device thread."""
                from . import CatenaMem, check, free
                plan = self._map_programs[id(assign)]
                outs = [o for o in assign.outputs if o.lowered != "erased"]
                comps = Evaluator._components(None, assign.input_sizes, ins, "reducec")
                zero, get_env, count = comps[0], comps[3], int(_runtime(comps[5])[0])
                if plan.staged is not None and count >= 1024:
                    program, _, kind = plan.staged
                    [z] = _runtime(zero)
                    if kind != "sum_f32" or f32_bits(z) == 0:          # the prebuilt f32 sum starts from +0, like `sum-f32`
                        raw = program.launch(count, bind(get_env))
                        try:
                            if kind == "sum_u64":
                                total = C.c_uint64(0)
                                check(self._lib.program_sum_u64_s(raw, C.byref(total)))
                                return [(int(z) + total.value) & 0xFFFFFFFFFFFFFFFF]
                            value = C.c_float(0)
                            check((self._lib.program_sum_f32_s if kind == "sum_f32" else self._lib.program_max_f32_s)(raw, C.byref(value)))
                            value = np.float32(value.value)
                            if kind == "max_f32":                       # f32.max-env keeps the accumulator on ties (sum.hex:73-84)
                                return [np.float32(z) if np.float32(z) >= value else value]
                            return [value]
                        finally:
                            free(raw)
                env = bind(ins)
                return [scalar_of(p.launch(1, env), o.lowered) for p, o in zip(plan.sequential, outs)]

            self._map_eval = Evaluator(modules, materialize, reduce)
        return self._map_eval

    def _exec_on_host(self, name, host, args, outs):
        """A module evaluated on the host — scalar code, possibly around launches of the generic map kernel.  A failed
        `assert` is the Device error the kernels report as CATENA_E_ASSERT (the generated code of the reference would
        have trapped).  `Mem` arguments are consumed, as in `exec`; a `Mem` result owns the buffer it was materialised
        into (or takes over the argument it aliases)."""
        from . import CatenaMem, E_ASSERT, CatenaError, free
        from .evaluator import AssertFailed, DeviceMem
        values = []
        for a in args:
            if a.kind is K.Mem:
                values.append(DeviceMem(a.v.raw.data, a.v.raw.len))
            else:
                values.append(np.float32(a.v) if a.kind is K.F32 else int(a.v))
        self._map_outputs = {}
        taken = set()
        try:
            try:
                got = host(values)
            except AssertFailed as exc:
                raise ExecError("Device", f"program '{name}' failed: {exc}", E_ASSERT) from exc
            except CatenaError as exc:
                raise ExecError("Device", f"program '{name}' failed: {exc}", exc.status) from exc
            if len(got) != len(outs):
                raise ExecError("OutputArityMismatch", f"Function '{name}' expected {len(outs)} outputs, got {len(got)}")
            arguments = {int(a.v.raw.data): a.v for a in args if a.kind is K.Mem and a.v.raw.data}
            results = []
            for kind, v in zip(outs, got):
                if kind is not K.Mem:
                    results.append(Value.f32(v) if kind is K.F32 else Value(kind, int(v)))
                elif not v.ptr or v.nbytes == 0:
                    results.append(Value.mem(Mem()))
                elif v.ptr in taken or (v.ptr not in self._map_outputs and v.ptr not in arguments):
                    raise ExecError("Device", f"program '{name}' returned a buffer it does not own")
                else:
                    taken.add(v.ptr)
                    if v.ptr in arguments and v.ptr not in self._map_outputs:
                        arguments[v.ptr].raw = CatenaMem()          # an argument handed back: the result takes it over
                    results.append(Value.mem(Mem(CatenaMem(v.ptr, v.nbytes))))
            return results
        finally:
            for ptr, raw in self._map_outputs.items():
                if ptr not in taken:
                    free(raw)
            self._map_outputs = {}
            for a in args:
                if a.kind is K.Mem:
                    a.v.free()
