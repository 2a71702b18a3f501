// The C++ kernel selector (include/catena_b200_lowering.hpp) on hand-written IR fixtures shaped after
// catena-lang/src/codegen/mod.rs:107-146 and the lowering asserted in catena-lang/tests/compile/closures/matmul.rs:45-53
// and reduce.rs:30.  The same cases as tests/test_lowering.py.  Prints "ok <n> checks" or the failed check.
#include <cstdio>
#include <string>
#include <vector>

#include "catena_b200_lowering.hpp"

using namespace catena_b200::lowering;

static int g_checks = 0;
#define CHECK(cond)                                                       \
    do {                                                                  \
        ++g_checks;                                                       \
        if (!(cond)) {                                                    \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            return 1;                                                     \
        }                                                                 \
    } while (0)

static GpuModule mod(const std::string& source_name, std::vector<GpuAssign> assigns) {
    GpuModule m;
    m.name = symbol_for(source_name);
    m.source_name = source_name;
    m.entry.name = m.name;
    m.entry.assignments = std::move(assigns);
    return m;
}
static GpuAssign prim(const std::string& op, const std::string& call = "") { return GpuAssign{op, {}, {}, call}; }
static GpuAssign reducec(const std::string& add, const std::string& get) {
    return GpuAssign{"reducec",
                     {Operand::var("zero", "f32"), Operand::fn(add), Operand::var("buf", "ptr<f32>"), Operand::fn(get), Operand::var("len", "u64")},
                     {Operand::var("acc", "f32")},
                     ""};
}
static GpuAssign materializec(const std::string& producer) {
    return GpuAssign{"materializec", {Operand::var("len", "u64"), Operand::var("env", "ptr<f32>"), Operand::fn(producer)}, {Operand::var("out", "ptr<f32>")}, ""};
}
static bool refused(const GpuModule& m) {
    try {
        select(m);
    } catch (const Unsupported&) {
        return true;
    }
    return false;
}

int main() {
    const GpuAssign cast = prim("mem.cast.f32"), to_mem = prim("buf.to-mem");
    {
        KernelPlan p = select(mod("matmul-2x2-via-mem", {cast, cast, prim("u64.eq"), prim("assert"), materializec("closure.f32.matmul.row-major.cell-at.0"), to_mem}));
        CHECK(p.kernel == "matmul_f32_kernel" && p.symbol == "program_matmul_2x2_via_mem");
    }
    CHECK(select(mod("sum-f32", {cast, reducec("f32.add-env", "f32-at")})).kernel == "fold_sum");
    CHECK(select(mod("max-f32", {cast, reducec("f32.max-env", "f32-at")})).kernel == "fold_max");
    CHECK(select(mod("tensor.argmax-f32", {cast, reducec("tensor.argmax-env", "tensor.argmax-pair-at")})).kernel == "fold_argmax");
    {
        KernelPlan p = select(mod("nn.softmax", {cast, reducec("f32.max-env", "f32-at"), reducec("f32.add-env", "nn.softmax-exp-shifted-at"),
                                                 materializec("nn.softmax-at"), to_mem}));
        CHECK(p.kernel == "softmax_fused" && p.symbol == "program_nn_softmax");
    }
    CHECK(select(mod("nn.rmsnorm", {cast, reducec("f32.add-env", "nn.squared-at"), prim("u64.to-f32"), prim("f32.div"),
                                    prim("math.sqrt", "program_math_sqrt"), materializec("nn.rmsnorm-at"), to_mem})).kernel == "rmsnorm_fused");
    CHECK(select(mod("tensor.concat-f32", {cast, cast, materializec("tensor.concat-f32-at"), to_mem})).kernel == "copy_concat");
    CHECK(select(mod("nn.silu", {prim("f32.neg"), prim("math.exp-approx", "program_math_exp_approx"), prim("f32.add"), prim("f32.div"), prim("f32.mul")})).kernel ==
          "host_scalar");
    // a producer without a prebuilt kernel goes to the generic map kernel (whether it compiles to a register program is decided
    // when the modules are registered); a `gpu.materialize` with an unknown kernel stays refused
    CHECK(select(mod("my-map", {cast, materializec("my.custom-at"), to_mem})).kernel == "host_with_map_kernels");
    {
        GpuAssign g = materializec("my.custom-at");
        g.op = "gpu.materialize";
        CHECK(refused(mod("my-launch", {cast, g, to_mem})));
    }
    // the same for a fold over a buffer whose closures match no fold kernel
    CHECK(select(mod("odd", {cast, reducec("f32.add-env", "my.getter")})).kernel == "host_with_map_kernels");
    CHECK(refused(mod("two-maps", {cast, materializec("tensor.arange-at"), materializec("tensor.slice-at"), to_mem})));
    {
        // out[i] = nn.silu(x[i]) written as a user's producer: with the modules at hand the selector takes the prebuilt map kernel
        GpuModule at = mod("my.silu-at", {GpuAssign{"ix", {Operand::var("i", "u64"), Operand::var("x", "ptr<f32>")}, {Operand::var("xi", "f32")}, ""},
                                          GpuAssign{"nn.silu", {Operand::var("xi", "f32")}, {Operand::var("r", "f32")}, "program_nn_silu"}});
        at.entry.sources = {Operand::var("x", "ptr<f32>"), Operand::var("i", "u64")};
        at.entry.targets = {Operand::var("r", "f32")};
        GpuModule silu = mod("nn.silu", {prim("f32.mul")});
        GpuModule entry = mod("my.silu-map", {GpuAssign{"mem.cast.f32", {Operand::var("m", "mem")}, {Operand::var("len", "u64"), Operand::var("x", "ptr<f32>")}, ""},
                                              GpuAssign{"materializec", {Operand::var("len", "u64"), Operand::var("x", "ptr<f32>"), Operand::fn("my.silu-at")},
                                                        {Operand::var("buf", "ptr<f32>")}, "", {1, 1, 1}, {1}},
                                              GpuAssign{"buf.to-mem", {Operand::var("len", "u64"), Operand::var("buf", "ptr<f32>")}, {Operand::var("out", "mem")}, ""}});
        const std::vector<GpuModule> all = {at, silu, entry};
        KernelPlan p = select(entry, all);
        CHECK(p.kernel == "map_unary" && p.note == "nn.silu");
        // with another length than the buffer's own it stays on the generic path
        entry.entry.assignments[1].inputs[0] = Operand::var("other", "u64");
        CHECK(select(entry, all).kernel == "host_with_map_kernels");
    }
    std::printf("ok %d checks\n", g_checks);
    return 0;
}
