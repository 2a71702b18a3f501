"""Native-CUDA lowering: selects a prebuilt sm_100a kernel for a lowered catena module instead of
rendering C++ source for it.

Input is the reference's semantic IR after `codegen::codegen` — `GpuModule { name, source_name,
entry: GpuFunction { sources, targets, assignments: [GpuAssign { op, inputs, outputs }] } }`
(catena-lang/src/codegen/mod.rs:107-146) — serialised as plain dicts / JSON.  Where the reference
calls `render_modules` (catena-lang/src/codegen/gpu.rs:111-143) this backend calls `select`, which
recognises the shapes the stdlib lowers to:

  * one `materializec` whose producer is the matmul cell chain (`f32.matmul.row-major.cell-at`,
    catena-lang/stdlib/matrix.hex:261-327; the lowering leaves exactly one materializec,
    catena-lang/tests/compile/closures/matmul.rs:45-53)                     -> f32 GEMM kernel
  * `reducec` with `f32.add-env` / `f32.max-env` / `tensor.argmax-env` and an element getter
    (catena-lang/stdlib/sum.hex, tensor.hex:171-227)                         -> fold kernels
  * max fold + exp-shifted sum fold + `nn.softmax-at` map (nn.hex:93-122)    -> fused softmax
  * squared-sum fold + `nn.rmsnorm-at` map (nn.hex:154-182)                  -> fused rmsnorm
  * `materializec` over tensor.broadcast-at / arange-at / slice-at / concat-f32-at
    (tensor.hex)                                                             -> fill / copy kernels
  * `reducec` over u64 buffers with `u64.add-env` and an element / product getter
    (catena-lang/tests/cases/reducec/basic.hex)                              -> u64 fold kernels
  * `mem.cast.u64`, `ix.zero`, `ix` (catena-lang/tests/runtime.rs:713-726)   -> buffer-head copy
  * a module of scalar primitives, `bool.ifc`, `eval`, calls of scalar modules and `reducec` whose
    closures are scalar (catena-lang/tests/cases/closures/*.hex)             -> host execution (evaluator.py)
  * a `materializec` whose producer applies a scalar stdlib program to every element of one f32 buffer
    (`out[i] = nn.silu(x[i])` and the like)                                  -> the prebuilt unary map kernel
  * any other `materializec` whose producer is scalar code over its environment and index
    (catena-lang/examples/materializec.hex, tests/cases/materialize/basic.hex) -> the generic map kernel, which
    interprets the producer as a register program (map_program.py); the code around it runs on the host
  * any other `reducec` whose closures read device buffers                   -> the same kernel: the getter's values are
    materialised and folded by a prebuilt fold when `add` is one (`u64.add-env`, `f32.add-env`, `f32.max-env`), else the
    reference's sequential loop runs as a register program on one device thread
Anything else is reported as unsupported (an allocation inside a producer, a buffer chosen at run time).

The Rust front end that produces the IR is not part of this build, so fixtures for the tests are
written by hand from the lowering rules cited above.
"""
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class GpuVar:
    name: str
    lowered: str            # "f32", "u64", "ptr<f32>", "mem", "erased", ...


@dataclass
class FnSymbol:
    name: str               # hexpr name of the function the closure points at


@dataclass
class GpuAssign:
    op: str
    inputs: list            # GpuVar | FnSymbol
    outputs: List[GpuVar]
    call_symbol: Optional[str] = None
    # how the flattened inputs / outputs group into components (env, function, flag, ...) for the structural
    # operations `bool.ifc`, `reducec`, `u64.to-ix` (catena-lang/src/codegen/components.rs:13-60)
    input_sizes: Optional[List[int]] = None
    output_sizes: Optional[List[int]] = None


@dataclass
class GpuFunction:
    name: str
    sources: List[GpuVar]
    targets: List[GpuVar]
    assignments: List[GpuAssign]


@dataclass
class GpuModule:
    name: str
    source_name: Optional[str]
    entry: GpuFunction


@dataclass
class KernelPlan:
    kernel: str                       # name of the prebuilt kernel family
    symbol: str                       # C symbol the reference would have generated for this module
    notes: List[str] = field(default_factory=list)

    @property
    def entry(self):
        """Entry point of the kernel library that implements this plan (None: host evaluation, or a family that is
        only reachable through the program of the same name)."""
        return LIBRARY_ENTRY.get(self.kernel)


# kernel family -> (library entry point, runtime inputs, runtime outputs) for the families a user-named program can map to
LIBRARY_ENTRY = {
    "fold_sum_u64": "program_sum_u64", "fold_dot_u64": "program_dot_u64", "array_head_u64": "program_array_head_u64",
    "fold_sum": "program_sum_f32", "fold_max": "program_max_f32", "fold_argmax": "program_tensor_argmax_f32",
    "softmax_fused": "program_nn_softmax", "rmsnorm_fused": "program_nn_rmsnorm",
    "fill_broadcast": "program_tensor_broadcast_f32", "fill_arange": "program_tensor_arange_f32",
    "copy_slice": "program_tensor_slice_f32", "copy_concat": "program_tensor_concat_f32",
    "matmul_f32_kernel": "program_matmul_2x2_via_mem",
}
ENTRY_SIGNATURE = {
    "program_sum_u64": (["mem"], ["u64"]), "program_dot_u64": (["mem", "mem"], ["u64"]),
    "program_array_head_u64": (["mem"], ["u64"]),
    "program_sum_f32": (["mem"], ["f32"]), "program_max_f32": (["mem"], ["f32"]),
    "program_tensor_argmax_f32": (["mem"], ["u64"]),
    "program_nn_softmax": (["mem"], ["mem"]), "program_nn_rmsnorm": (["mem"], ["mem"]),
    "program_tensor_broadcast_f32": (["f32", "u64"], ["mem"]), "program_tensor_arange_f32": (["u64"], ["mem"]),
    "program_tensor_slice_f32": (["mem", "u64", "u64"], ["mem"]), "program_tensor_concat_f32": (["mem", "mem"], ["mem"]),
    "program_matmul_2x2_via_mem": (["mem", "mem"] + ["u64"] * 6, ["mem"]),
}


class Unsupported(Exception):
    """No prebuilt kernel matches this module."""


def module_from_dict(d):
    def var(v):
        return FnSymbol(v["fn"]) if "fn" in v else GpuVar(v["name"], v.get("lowered", "erased"))
    fn = d["entry"]
    assigns = [GpuAssign(a["op"], [var(v) for v in a.get("inputs", [])], [var(v) for v in a.get("outputs", [])],
                         a.get("call_symbol"), a.get("input_sizes"), a.get("output_sizes")) for a in fn["assignments"]]
    return GpuModule(d["name"], d.get("source_name"),
                     GpuFunction(fn["name"], [var(v) for v in fn.get("sources", [])],
                                 [var(v) for v in fn.get("targets", [])], assigns))


def _fn_symbols(assign):
    return [v.name for v in assign.inputs if isinstance(v, FnSymbol)]


_FOLDS = {("u64.add-env", "sum-u64-at"): "fold_sum_u64", ("u64.add-env", "dot-u64-product-at"): "fold_dot_u64",
          ("f32.add-env", "f32-at"): "fold_sum", ("f32.max-env", "f32-at"): "fold_max",
          ("f32.add-env", "nn.squared-at"): "fold_sumsq", ("f32.add-env", "nn.softmax-exp-shifted-at"): "fold_expsum",
          ("tensor.argmax-env", "tensor.argmax-pair-at"): "fold_argmax"}
_MAPS = {"tensor.broadcast-at": "fill_broadcast", "tensor.arange-at": "fill_arange", "tensor.slice-at": "copy_slice",
         "tensor.concat-f32-at": "copy_concat", "nn.softmax-at": "softmax_map", "nn.rmsnorm-at": "rmsnorm_map"}
# scalar primitives the renderer prints as single C expressions (catena-lang/src/codegen/gpu.rs:322-447)
_SCALAR_PREFIXES = ("f32.", "u32.", "u64.", "bool.", "const.", "ix", "unit.", ":.", "ax-mp", "assert", "mem.cast", "buf.",
                    "row-major-", "math.", "nn.sigmoid", "nn.silu", "nn.tanh", "nn.gelu")


def _touches_memory(assign):
    return any(isinstance(v, GpuVar) and (v.lowered == "mem" or v.lowered.startswith("ptr<")) for v in list(assign.inputs) + list(assign.outputs))


def _scalar_function(name, modules, seen, allow_memory=False):
    """True when the function a symbol names is a primitive or a module (of `modules`) made of scalar assignments;
    unless `allow_memory`, none of them may touch a buffer (the host cannot dereference device memory)."""
    from .evaluator import is_primitive
    if is_primitive(name):
        return True
    module = find_module(modules, name)
    if module is None or name in seen:
        return False
    seen = seen | {name}
    return all(classify(a, modules, seen) == "scalar" and (allow_memory or not _touches_memory(a)) for a in module.entry.assignments)


def materializec_parts(assign, values=None):
    """(len, environment, producer symbol) of a `materializec` — the closure-converted call shape `len, env..., producer_fn`
    (catena-lang/src/codegen/ops/materializec.rs:147-189) — taken from `values` (one per input) or from the inputs."""
    items = list(assign.inputs if values is None else values)
    if assign.input_sizes is not None:
        if len(assign.input_sizes) != 3 or sum(assign.input_sizes) != len(items) or assign.input_sizes[0] != 1:
            raise Unsupported("materializec expects the components len, env, producer")
        env = items[1:1 + assign.input_sizes[1]]
        fn = items[1 + assign.input_sizes[1]:]
    else:
        env, fn = items[1:-1], items[-1:]
    fns = [v for v in fn if isinstance(v, FnSymbol)]
    if len(fns) != 1:
        raise Unsupported("materializec needs one producer symbol")
    return items[0], env, fns[0]


def unary_map_op(module, assign, modules):
    """`out[i] = S(x[i])` over the whole of one f32 buffer, S a scalar stdlib program with a prebuilt map kernel
    (`catena_b200_map_f32_s`): returns S's hexpr name, else None.  The shape: the environment is one `ptr<f32>`, the producer
    is `ix` of that buffer at the index followed by a call of S, and the length is the buffer's own (the `mem.cast.f32` that
    made the pointer)."""
    from . import SCALAR_PROGRAMS
    from .evaluator import NO_OPS
    try:
        length, env, fn = materializec_parts(assign)
    except Unsupported:
        return None
    env = [v for v in env if isinstance(v, GpuVar) and v.lowered != "erased"]
    producer = find_module(modules, fn.name)
    if producer is None or len(env) != 1 or env[0].lowered != "ptr<f32>" or not isinstance(length, GpuVar):
        return None
    if not any(a.op == "mem.cast.f32" and [o.name for o in a.outputs] == [length.name, env[0].name] for a in module.entry.assignments):
        return None
    sources = [v for v in producer.entry.sources if v.lowered != "erased"]
    targets = [v for v in producer.entry.targets if v.lowered != "erased"]
    body = [a for a in producer.entry.assignments if a.op not in NO_OPS]
    if [v.lowered for v in sources] != ["ptr<f32>", "u64"] or len(targets) != 1 or len(body) != 2:
        return None
    load, call = body
    if load.op != "ix" or [v.name for v in load.inputs if isinstance(v, GpuVar)] != [sources[1].name, sources[0].name]:
        return None
    callee = find_module(modules, call.call_symbol) if call.call_symbol else None
    name = callee.source_name if callee is not None else call.op
    args = [v.name for v in call.inputs if isinstance(v, GpuVar) and v.lowered != "erased"]
    if name not in SCALAR_PROGRAMS or args != [load.outputs[0].name] or [o.name for o in call.outputs if o.lowered != "erased"] != [targets[0].name]:
        return None
    return name


def map_program_for(assign, modules):
    """The register program of a `materializec` whose producer has no prebuilt kernel (map_program.py); raises Unsupported."""
    from .map_program import compile_producer
    if len(assign.outputs) != 1 or not assign.outputs[0].lowered.startswith("ptr<"):
        raise Unsupported("materializec produces one buffer")
    _, env, fn = materializec_parts(assign)
    env_vars = [v for v in env if isinstance(v, GpuVar) and v.lowered != "erased"]
    return compile_producer(modules or {}, fn.name, env_vars, assign.outputs[0].lowered[4:-1])


# `add` closures whose fold a prebuilt kernel computes: (accumulator type, fold kind).  With one of them a generic fold runs in
# two stages — the getter's values materialised by the generic map kernel, then the prebuilt fold over them.
_STAGED_ADDS = {"u64.add-env": ("u64", "sum_u64"), "f32.add-env": ("f32", "sum_f32"), "f32.max-env": ("f32", "max_f32")}


@dataclass
class FoldPlan:
    """How a `reducec` over device buffers that matches no fold kernel runs (map_program.py).  `sequential`: one register
    program per accumulator component, the reference's own loop run by one device thread (bit-exact for every `add`).
    `staged`: (getter program, its environment variables, fold kind) when `add` is a prebuilt fold's."""
    sequential: list
    staged: Optional[tuple] = None


def fold_plan_for(assign, modules):
    from .map_program import compile_fold, compile_getter
    outs = [o for o in assign.outputs if o.lowered != "erased"]
    if assign.op != "reducec" or not outs:
        raise Unsupported("not a reducec")
    plan = FoldPlan([compile_fold(modules or {}, assign, k) for k in range(len(outs))])
    if len(outs) == 1:
        for add, (lowered, kind) in _STAGED_ADDS.items():
            if add in _fn_symbols(assign) and outs[0].lowered == lowered:
                try:
                    program, env_vars = compile_getter(modules or {}, assign)
                    plan.staged = (program, env_vars, kind)
                except Unsupported:
                    pass
    return plan


def classify(assign, modules=None, _seen=frozenset()):
    """One assignment -> kernel family, 'scalar' or None.  `modules` maps source names (and generated symbols) to the
    lowered modules of the program, so that calls and closure symbols can be looked through."""
    if assign.op == "reducec":
        fns = _fn_symbols(assign)
        for (add, get), kernel in _FOLDS.items():
            if add in fns and get in fns:
                return kernel
        # a fold whose closures are scalar functions over scalar environments runs on the host, as in the reference
        if fns and not _touches_memory(assign) and all(_scalar_function(f, modules, _seen) for f in fns):
            return "scalar"
        if modules is not None:
            try:
                fold_plan_for(assign, modules)
                return "fold_generic"
            except Unsupported:
                return None
        return None
    if assign.op in ("materializec", "gpu.materialize"):
        fns = _fn_symbols(assign)
        if any("f32.matmul.row-major.cell-at" in f or f.startswith("closure.f32.matmul") for f in fns):
            return "gemm_f32"
        for f in fns:
            if f in _MAPS:
                return _MAPS[f]
        if assign.op == "materializec" and modules is not None:
            try:
                map_program_for(assign, modules)
                return "map_generic"
            except Unsupported:
                return None
        return None
    if assign.op in ("bool.ifc", "eval"):
        fns = _fn_symbols(assign)
        return "scalar" if fns and all(_scalar_function(f, modules, _seen) for f in fns) else None
    if assign.call_symbol:
        # a callee may cast and pass buffers on (e.g. `mem.cast.u64.same-length`): whether the caller as a whole can run
        # on the host is decided in `select`
        return "scalar" if modules is None or _scalar_function(assign.call_symbol, modules, _seen, allow_memory=True) else None
    if assign.op.startswith(_SCALAR_PREFIXES):
        return "scalar"
    return None


def module_map(modules):
    """{generated symbol, source name, `program.<source name>` -> module} for a list of lowered modules."""
    out = {}
    for m in modules:
        out[m.name] = m
        if m.source_name:
            out[m.source_name] = m
            out["program." + m.source_name] = m
    return out


def find_module(modules, name):
    """The module a call symbol, a source name or a function symbol's target names.  A function symbol `f` is called as
    `program.f` with every non-alphanumeric character replaced (catena-lang/src/codegen/components.rs:100-105)."""
    if not modules:
        return None
    m = modules.get(name)
    if m is None:
        from . import symbol_for
        m = modules.get(symbol_for(name))
    return m


def select(module, symbol_for=None, modules=None):
    """GpuModule -> KernelPlan (or raises Unsupported)."""
    if symbol_for is None:
        from . import symbol_for as _sf
        symbol_for = _sf
    kinds = []
    for a in module.entry.assignments:
        k = classify(a, modules)
        if k is None:
            raise Unsupported(f"{module.name}: no prebuilt kernel for `{a.op}` with {_fn_symbols(a)}")
        if k != "scalar":
            kinds.append(k)
    symbol = symbol_for(module.source_name) if module.source_name else module.name
    ops = [a.op for a in module.entry.assignments]
    if kinds == ["map_generic"] and modules is not None:
        # one custom producer that only applies a scalar stdlib program to every element of a buffer: the prebuilt map kernel
        [launch] = [a for a in module.entry.assignments if a.op == "materializec"]
        rest = [a.op for a in module.entry.assignments if a is not launch]
        from .evaluator import NO_OPS
        op = unary_map_op(module, launch, modules)
        if op is not None and sorted(o for o in rest if o not in NO_OPS) == ["buf.to-mem", "mem.cast.f32"]:
            return KernelPlan("map_unary", symbol, [op])
    generic = ("map_generic", "fold_generic")
    if any(k in generic for k in kinds) and not all(k in generic for k in kinds) and modules is not None:
        # a module is one of the recognised shapes, or everything in it runs generically: the recognised maps and folds it
        # also holds must compile to register programs too (their producers' modules have to be there)
        for a in module.entry.assignments:
            if a.op == "materializec":
                map_program_for(a, modules)
            elif a.op == "reducec" and _touches_memory(a):
                fold_plan_for(a, modules)
        kinds = [k if k in generic else "map_generic" for k in kinds]
    if kinds and all(k in generic for k in kinds):
        # host code around generic map / fold kernels: the host part may cast and pass buffers on, not read them
        for a in module.entry.assignments:
            if a.op not in ("materializec", "reducec") and _touches_memory(a) and not a.op.startswith(("mem.cast.", "buf.")) and not a.call_symbol:
                raise Unsupported(f"{module.name}: host code reads a device buffer (`{a.op}`)")
        return KernelPlan("host_with_map_kernels", symbol, ["producers and folds interpreted by the generic map kernel; the code around them runs on the host"])
    if not kinds:
        if any(_touches_memory(a) for a in module.entry.assignments):
            # scalar code that reads a buffer: the host cannot dereference device memory, so only the shape with a
            # kernel-side counterpart is taken — the first element of a u64 buffer
            if "mem.cast.u64" in ops and "ix.zero" in ops and ops.count("ix") == 1 and not any(o.startswith("mem.cast.f32") for o in ops):
                return KernelPlan("array_head_u64", symbol, ["8-byte device-to-host copy after the non-empty assertion"])
            raise Unsupported(f"{module.name}: scalar code over a buffer other than the head of a u64 buffer")
        return KernelPlan("host_scalar", symbol, ["runs on the host, like the reference's non-materialize code"])
    if kinds == ["gemm_f32"]:
        return KernelPlan("matmul_f32_kernel", symbol, ["bit-exact ascending-k fold, smem-tiled"])
    if kinds == ["fold_max", "fold_expsum", "softmax_map"]:
        return KernelPlan("softmax_fused", symbol, ["two host folds + one map kernel in the reference; one launch here up to 65536 elements"])
    if kinds == ["fold_sumsq", "rmsnorm_map"]:
        return KernelPlan("rmsnorm_fused", symbol, ["host fold + map kernel in the reference"])
    if len(kinds) == 1:
        return KernelPlan(kinds[0], symbol)
    raise Unsupported(f"{module.name}: unrecognised combination {kinds}")
