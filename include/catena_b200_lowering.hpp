// Native-CUDA lowering (header-only, C++17): selects a prebuilt sm_100a kernel for a lowered catena module instead of
// rendering C++ source for it.
//
// Input is the reference's semantic IR after `codegen::codegen` — GpuModule { name, source_name, entry: GpuFunction {
// sources, targets, assignments: [GpuAssign { op, inputs, outputs }] } } (catena-lang/src/codegen/mod.rs:107-146).
// Where the reference calls `render_modules` (catena-lang/src/codegen/gpu.rs:111-143) this backend calls `select`, which
// recognises the shapes the stdlib lowers to:
//   * one `materializec` whose producer is the matmul cell chain (`f32.matmul.row-major.cell-at`,
//     catena-lang/stdlib/matrix.hex:261-327; the lowering leaves exactly one materializec,
//     catena-lang/tests/compile/closures/matmul.rs:45-53)                     -> f32 GEMM kernel
//   * `reducec` with `f32.add-env` / `f32.max-env` / `tensor.argmax-env` and an element getter
//     (catena-lang/stdlib/sum.hex, tensor.hex:171-227)                         -> fold kernels
//   * max fold + exp-shifted sum fold + `nn.softmax-at` map (nn.hex:93-122)    -> fused softmax
//   * squared-sum fold + `nn.rmsnorm-at` map (nn.hex:154-182)                  -> fused rmsnorm
//   * `materializec` over tensor.broadcast-at / arange-at / slice-at / concat-f32-at (tensor.hex) -> fill / copy kernels
//   * `reducec` over u64 buffers with `u64.add-env` and an element / product getter
//     (catena-lang/tests/cases/reducec/basic.hex)                              -> u64 fold kernels
//   * `mem.cast.u64`, `ix.zero`, `ix` (catena-lang/tests/runtime.rs:713-726)   -> buffer-head copy
//   * a module of scalar primitives, `bool.ifc`, `eval`, `reducec` over scalar closures and calls
//     (catena-lang/tests/cases/closures/*.hex)                                 -> host execution (catena_b200_eval.hpp)
//   * any other `materializec` (catena-lang/examples/materializec.hex, tests/cases/materialize/basic.hex)
//                                                                              -> the generic map kernel, which interprets the
//     producer as a register program (catena_b200_map_program.hpp); the code around it runs on the host
// Anything else is reported as unsupported.  The Rust front end that produces the IR is not part of this build, so the
// fixtures of the tests are written by hand from the lowering rules cited above.
#ifndef CATENA_B200_LOWERING_HPP
#define CATENA_B200_LOWERING_HPP

#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace catena_b200 {
namespace lowering {

// An input or output of an assignment: a lowered variable, or the symbol of the function a closure points at.
struct Operand {
    std::string name;
    std::string lowered;      // "f32", "u64", "ptr<f32>", "mem", "erased", ...; empty for a function symbol
    bool is_fn = false;
    static Operand var(std::string n, std::string l) { return Operand{std::move(n), std::move(l), false}; }
    static Operand fn(std::string n) { return Operand{std::move(n), std::string(), true}; }
};
struct GpuAssign {
    std::string op;
    std::vector<Operand> inputs, outputs;
    std::string call_symbol;  // non-empty for a call of another program
    // how the flattened inputs / outputs group into components (environment, function, flag, ...) for `bool.ifc`, `reducec`
    // and `u64.to-ix` (catena-lang/src/codegen/components.rs:13-60); empty for everything else
    std::vector<size_t> input_sizes, output_sizes;
};
struct GpuFunction {
    std::string name;
    std::vector<Operand> sources, targets;
    std::vector<GpuAssign> assignments;
};
struct GpuModule {
    std::string name, source_name;
    GpuFunction entry;
};
struct KernelPlan {
    std::string kernel;       // name of the prebuilt kernel family
    std::string symbol;       // C symbol of the entry point that runs it
    std::string note;
};
struct Unsupported : std::runtime_error {
    using std::runtime_error::runtime_error;
};

// C symbol of a source name (catena-lang/src/codegen/mod.rs:379-388)
inline std::string symbol_for(const std::string& name) {
    std::string out;
    for (char ch : name) out += ((ch >= '0' && ch <= '9') || (ch >= 'a' && ch <= 'z') || (ch >= 'A' && ch <= 'Z')) ? ch : '_';
    if (!out.empty() && out[0] >= '0' && out[0] <= '9') out = "_" + out;
    return "program_" + out;
}

namespace detail {
inline bool has_fn(const GpuAssign& a, const std::string& name) {
    for (const Operand& o : a.inputs)
        if (o.is_fn && o.name == name) return true;
    return false;
}
inline bool starts_with(const std::string& s, const char* prefix) { return s.rfind(prefix, 0) == 0; }
}  // namespace detail

// One assignment -> kernel family, "scalar", or "" when nothing matches.
inline std::string classify(const GpuAssign& a) {
    using detail::has_fn;
    if (a.op == "reducec") {
        static const char* folds[][3] = {{"u64.add-env", "sum-u64-at", "fold_sum_u64"},
                                         {"u64.add-env", "dot-u64-product-at", "fold_dot_u64"},
                                         {"f32.add-env", "f32-at", "fold_sum"},
                                         {"f32.max-env", "f32-at", "fold_max"},
                                         {"f32.add-env", "nn.squared-at", "fold_sumsq"},
                                         {"f32.add-env", "nn.softmax-exp-shifted-at", "fold_expsum"},
                                         {"tensor.argmax-env", "tensor.argmax-pair-at", "fold_argmax"}};
        for (auto& f : folds)
            if (has_fn(a, f[0]) && has_fn(a, f[1])) return f[2];
        // a fold whose environments hold no buffer runs on the host (its closures are checked when it is evaluated); any other
        // fold over buffers goes to the generic map kernel (catena_b200_map_program.hpp: staged through a prebuilt fold when
        // `add` is one, else the sequential loop as a register program; the caller of select() builds the programs)
        for (const Operand& o : a.inputs)
            if (!o.is_fn && (o.lowered == "mem" || detail::starts_with(o.lowered, "ptr<"))) return "fold_generic";
        return "scalar";
    }
    if (a.op == "bool.ifc" || a.op == "eval") return "scalar";
    if (a.op == "materializec" || a.op == "gpu.materialize") {
        for (const Operand& o : a.inputs)
            if (o.is_fn && (o.name.find("f32.matmul.row-major.cell-at") != std::string::npos || detail::starts_with(o.name, "closure.f32.matmul")))
                return "gemm_f32";
        static const char* maps[][2] = {{"tensor.broadcast-at", "fill_broadcast"}, {"tensor.arange-at", "fill_arange"},
                                        {"tensor.slice-at", "copy_slice"},         {"tensor.concat-f32-at", "copy_concat"},
                                        {"nn.softmax-at", "softmax_map"},          {"nn.rmsnorm-at", "rmsnorm_map"}};
        for (const Operand& o : a.inputs)
            if (o.is_fn)
                for (auto& m : maps)
                    if (o.name == m[0]) return m[1];
        // any other producer: the generic map kernel interprets it as a register program, if it compiles to one
        // (catena_b200_map_program.hpp; the caller of select() builds the program and reports a producer that does not)
        return a.op == "materializec" ? "map_generic" : "";
    }
    // scalar primitives the renderer prints as single C expressions (catena-lang/src/codegen/gpu.rs:322-447)
    static const char* scalar_prefixes[] = {"f32.", "u32.", "u64.", "bool.", "const.", "ix", "unit.", ":.", "ax-mp", "assert", "mem.cast",
                                            "buf.", "row-major-", "math.", "nn.sigmoid", "nn.silu", "nn.tanh", "nn.gelu"};
    for (const char* p : scalar_prefixes)
        if (detail::starts_with(a.op, p)) return "scalar";
    return a.call_symbol.empty() ? "" : "scalar";
}

// GpuModule -> KernelPlan, or throws Unsupported.
inline KernelPlan select(const GpuModule& module) {
    std::vector<std::string> kinds;
    for (const GpuAssign& a : module.entry.assignments) {
        const std::string k = classify(a);
        if (k.empty()) throw Unsupported(module.name + ": no prebuilt kernel for `" + a.op + "`");
        if (k != "scalar") kinds.push_back(k);
    }
    const std::string symbol = module.source_name.empty() ? module.name : symbol_for(module.source_name);
    auto is = [&](std::initializer_list<const char*> want) {
        if (kinds.size() != want.size()) return false;
        size_t i = 0;
        for (const char* w : want)
            if (kinds[i++] != w) return false;
        return true;
    };
    // a module is one of the recognised shapes, or — as soon as it holds a generic producer or fold — everything in it runs
    // generically (the recognised maps and folds it also holds are compiled to register programs by the caller)
    bool any_generic = false;
    for (const std::string& k : kinds) any_generic = any_generic || k == "map_generic" || k == "fold_generic";
    if (any_generic) {
        // host code around generic map / fold kernels: it may cast buffers and pass them on, not read them
        for (const GpuAssign& a : module.entry.assignments) {
            if (a.op == "materializec" || a.op == "reducec" || !a.call_symbol.empty() || detail::starts_with(a.op, "mem.cast.") || detail::starts_with(a.op, "buf.")) continue;
            for (const Operand& o : a.inputs)
                if (!o.is_fn && (o.lowered == "mem" || detail::starts_with(o.lowered, "ptr<")))
                    throw Unsupported(module.name + ": host code reads a device buffer (`" + a.op + "`)");
        }
        for (const GpuAssign& a : module.entry.assignments)
            if (a.op == "gpu.materialize") throw Unsupported(module.name + ": gpu.materialize with an unknown kernel");
        return {"host_with_map_kernels", symbol, "producers and folds interpreted by the generic map kernel; the code around them runs on the host"};
    }
    if (kinds.empty()) {
        bool memory = false, cast_u64 = false, ix_zero = false;
        size_t ix_count = 0;
        for (const GpuAssign& a : module.entry.assignments) {
            for (const Operand& o : a.inputs) memory = memory || (!o.is_fn && (o.lowered == "mem" || detail::starts_with(o.lowered, "ptr<")));
            cast_u64 = cast_u64 || a.op == "mem.cast.u64";
            ix_zero = ix_zero || a.op == "ix.zero";
            ix_count += a.op == "ix";
        }
        if (memory) {
            // scalar code that reads a buffer: the host cannot dereference device memory; only the head of a u64 buffer
            // has a kernel-side counterpart
            if (cast_u64 && ix_zero && ix_count == 1) return {"array_head_u64", symbol, "8-byte device-to-host copy after the non-empty assertion"};
            throw Unsupported(module.name + ": scalar code over a buffer other than the head of a u64 buffer");
        }
        return {"host_scalar", symbol, "runs on the host, like the reference's non-materialize code"};
    }
    if (is({"gemm_f32"})) return {"matmul_f32_kernel", symbol, "bit-exact ascending-k fold, smem-tiled"};
    if (is({"fold_max", "fold_expsum", "softmax_map"}))
        return {"softmax_fused", symbol, "two host folds + one map kernel in the reference; one launch here up to 65536 elements"};
    if (is({"fold_sumsq", "rmsnorm_map"})) return {"rmsnorm_fused", symbol, "host fold + map kernel in the reference"};
    if (kinds.size() == 1) return {kinds[0], symbol, ""};
    std::string all;
    for (const std::string& k : kinds) all += (all.empty() ? "" : ", ") + k;
    throw Unsupported(module.name + ": unrecognised combination " + all);
}

// `out[i] = S(x[i])` over the whole of one f32 buffer, S a scalar stdlib program with a prebuilt map kernel
// (catena_b200_map_f32_s): S's hexpr name, else "".  The shape: the environment of the materializec is one ptr<f32>, the
// producer is `ix` of that buffer at the index followed by a call of S, and the length is the buffer's own (the mem.cast.f32
// that made the pointer).
inline std::string unary_map_op(const GpuModule& module, const GpuAssign& a, const std::vector<GpuModule>& modules) {
    static const char* scalar_programs[] = {"math.sin-approx", "math.cos-approx", "math.sin-approx-full-nonneg", "math.sin-approx-full",
                                            "math.log-approx", "math.exp-approx-nonneg", "math.exp-approx", "math.exp2-approx",
                                            "math.log2-approx", "math.sqrt", "nn.sigmoid", "nn.silu", "nn.tanh", "nn.gelu-approx"};
    auto find = [&](const std::string& name) -> const GpuModule* {
        for (const GpuModule& m : modules)
            if (m.name == name || (!m.source_name.empty() && (m.source_name == name || symbol_for(m.source_name) == name))) return &m;
        for (const GpuModule& m : modules)
            if (m.name == symbol_for(name)) return &m;
        return nullptr;
    };
    auto runtime = [](const std::vector<Operand>& v) {
        std::vector<Operand> out;
        for (const Operand& o : v)
            if (!o.is_fn && o.lowered != "erased") out.push_back(o);
        return out;
    };
    if (a.op != "materializec" || a.inputs.size() < 3 || a.inputs[0].is_fn) return "";
    size_t env_end = a.inputs.size() - 1;
    if (!a.input_sizes.empty()) {
        if (a.input_sizes.size() != 3 || a.input_sizes[0] != 1) return "";
        env_end = 1 + a.input_sizes[1];
    }
    const std::vector<Operand> env = runtime(std::vector<Operand>(a.inputs.begin() + 1, a.inputs.begin() + env_end));
    const Operand* fn = nullptr;
    for (size_t k = env_end; k < a.inputs.size(); ++k)
        if (a.inputs[k].is_fn) fn = &a.inputs[k];
    if (!fn || env.size() != 1 || env[0].lowered != "ptr<f32>") return "";
    bool own_length = false;
    for (const GpuAssign& c : module.entry.assignments)
        own_length = own_length || (c.op == "mem.cast.f32" && c.outputs.size() == 2 && c.outputs[0].name == a.inputs[0].name && c.outputs[1].name == env[0].name);
    const GpuModule* producer = find(fn->name);
    if (!own_length || !producer) return "";
    const std::vector<Operand> sources = runtime(producer->entry.sources), targets = runtime(producer->entry.targets);
    std::vector<const GpuAssign*> body;
    for (const GpuAssign& c : producer->entry.assignments)
        if (c.op != "unit.intro" && c.op != "ax-mp" && c.op != "assert-then" && c.op != ":.param") body.push_back(&c);
    if (sources.size() != 2 || sources[0].lowered != "ptr<f32>" || sources[1].lowered != "u64" || targets.size() != 1 || body.size() != 2) return "";
    const GpuAssign &load = *body[0], &call = *body[1];
    const std::vector<Operand> load_in = runtime(load.inputs), call_in = runtime(call.inputs), call_out = runtime(call.outputs);
    if (load.op != "ix" || load_in.size() != 2 || load_in[0].name != sources[1].name || load_in[1].name != sources[0].name || load.outputs.empty()) return "";
    const GpuModule* callee = call.call_symbol.empty() ? nullptr : find(call.call_symbol);
    const std::string name = callee ? callee->source_name : call.op;
    bool known = false;
    for (const char* p : scalar_programs) known = known || name == p;
    if (!known || call_in.size() != 1 || call_in[0].name != load.outputs[0].name || call_out.size() != 1 || call_out[0].name != targets[0].name) return "";
    return name;
}

// select() with the program's other modules at hand: a lone custom producer that only applies a scalar stdlib program to every
// element of a buffer takes the prebuilt map kernel (plan "map_unary", the program's name in `note`).
inline KernelPlan select(const GpuModule& module, const std::vector<GpuModule>& modules) {
    KernelPlan plan = select(module);
    if (plan.kernel != "host_with_map_kernels") return plan;
    const GpuAssign* launch = nullptr;
    size_t launches = 0, casts = 0, to_mem = 0, other = 0;
    for (const GpuAssign& a : module.entry.assignments) {
        if (a.op == "materializec") { launch = &a; ++launches; }
        else if (a.op == "mem.cast.f32") ++casts;
        else if (a.op == "buf.to-mem") ++to_mem;
        else if (a.op != "unit.intro" && a.op != "ax-mp" && a.op != "assert-then" && a.op != ":.param") ++other;
    }
    if (launches == 1 && casts == 1 && to_mem == 1 && other == 0) {
        const std::string op = unary_map_op(module, *launch, modules);
        if (!op.empty()) return {"map_unary", plan.symbol, op};
    }
    return plan;
}

}  // namespace lowering
}  // namespace catena_b200

#endif  // CATENA_B200_LOWERING_HPP
