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
  * a module of scalar primitives only                                       -> host execution
Anything else is reported as unsupported (the reference would render a generic one-thread-per-element
kernel for it; this backend ships no source generator).

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
    symbol: str                       # C symbol of the entry point that runs it
    notes: List[str] = field(default_factory=list)


class Unsupported(Exception):
    """No prebuilt kernel matches this module."""


def module_from_dict(d):
    def var(v):
        return FnSymbol(v["fn"]) if "fn" in v else GpuVar(v["name"], v.get("lowered", "erased"))
    fn = d["entry"]
    assigns = [GpuAssign(a["op"], [var(v) for v in a.get("inputs", [])], [var(v) for v in a.get("outputs", [])],
                         a.get("call_symbol")) for a in fn["assignments"]]
    return GpuModule(d["name"], d.get("source_name"),
                     GpuFunction(fn["name"], [var(v) for v in fn.get("sources", [])],
                                 [var(v) for v in fn.get("targets", [])], assigns))


def _fn_symbols(assign):
    return [v.name for v in assign.inputs if isinstance(v, FnSymbol)]


_FOLDS = {("f32.add-env", "f32-at"): "fold_sum", ("f32.max-env", "f32-at"): "fold_max",
          ("f32.add-env", "nn.squared-at"): "fold_sumsq", ("f32.add-env", "nn.softmax-exp-shifted-at"): "fold_expsum",
          ("tensor.argmax-env", "tensor.argmax-pair-at"): "fold_argmax"}
_MAPS = {"tensor.broadcast-at": "fill_broadcast", "tensor.arange-at": "fill_arange", "tensor.slice-at": "copy_slice",
         "tensor.concat-f32-at": "copy_concat", "nn.softmax-at": "softmax_map", "nn.rmsnorm-at": "rmsnorm_map"}
# scalar primitives the renderer prints as single C expressions (catena-lang/src/codegen/gpu.rs:322-447)
_SCALAR_PREFIXES = ("f32.", "u32.", "u64.", "bool.", "const.", "ix", "unit.", ":.", "ax-mp", "assert", "mem.cast", "buf.",
                    "row-major-", "math.", "nn.sigmoid", "nn.silu", "nn.tanh", "nn.gelu")


def classify(assign):
    """One assignment -> kernel family, 'scalar' or None."""
    if assign.op == "reducec":
        fns = _fn_symbols(assign)
        for (add, get), kernel in _FOLDS.items():
            if add in fns and get in fns:
                return kernel
        return None
    if assign.op in ("materializec", "gpu.materialize"):
        fns = _fn_symbols(assign)
        if any("f32.matmul.row-major.cell-at" in f or f.startswith("closure.f32.matmul") for f in fns):
            return "gemm_f32"
        for f in fns:
            if f in _MAPS:
                return _MAPS[f]
        return None
    if assign.op.startswith(_SCALAR_PREFIXES) or assign.call_symbol:
        return "scalar"
    return None


def select(module, symbol_for=None):
    """GpuModule -> KernelPlan (or raises Unsupported)."""
    if symbol_for is None:
        from . import symbol_for as _sf
        symbol_for = _sf
    kinds = []
    for a in module.entry.assignments:
        k = classify(a)
        if k is None:
            raise Unsupported(f"{module.name}: no prebuilt kernel for `{a.op}` with {_fn_symbols(a)}")
        if k != "scalar":
            kinds.append(k)
    symbol = symbol_for(module.source_name) if module.source_name else module.name
    if not kinds:
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
