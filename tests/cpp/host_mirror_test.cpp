// Exercises the C++ host mirror (include/catena_b200.hpp) the way catena-lang/tests/runtime.rs and
// catena-lang/tests/cases/{matrix,reducec}.rs exercise the Rust runtime.
//   host_mirror_test cpu   pre-call checks only (no device needed): registration, arity and type errors, Hip refusal
//   host_mirror_test gpu   the reference's known-answer vectors on the GPU
// Prints "ok <n> checks" and exits 0, or the failed check and exits 1.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "catena_b200.hpp"

using namespace catena_b200;

static int g_checks = 0;
#define CHECK(cond)                                                         \
    do {                                                                    \
        ++g_checks;                                                         \
        if (!(cond)) {                                                      \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);   \
            return 1;                                                       \
        }                                                                   \
    } while (0)

template <class F>
static bool throws_kind(ExecError::Kind kind, F f) {
    try {
        f();
    } catch (const ExecError& e) {
        return e.kind == kind;
    }
    return false;
}

// Hand-lowered modules (catena-lang/src/codegen/mod.rs:107-146) of reference test programs, for Runtime::register_modules.
namespace lw = catena_b200::lowering;
static lw::Operand var(const std::string& n, const std::string& l) { return lw::Operand::var(n, l); }
static lw::GpuModule module(const std::string& source_name, std::vector<lw::Operand> sources, std::vector<lw::Operand> targets,
                            std::vector<lw::GpuAssign> assigns) {
    lw::GpuModule m;
    m.name = lw::symbol_for(source_name);
    m.source_name = source_name;
    m.entry.name = m.name;
    m.entry.sources = std::move(sources);
    m.entry.targets = std::move(targets);
    m.entry.assignments = std::move(assigns);
    return m;
}
static std::vector<lw::GpuModule> lowered_modules() {
    std::vector<lw::GpuModule> mods;
    // tests/runtime.rs:448-473
    mods.push_back(module("shift-and-sub", {}, {var("r", "u32")},
                          {{"const.u32.0x00000020", {}, {var("lhs", "u32")}, ""}, {"const.u32.0x00000003", {}, {var("shift", "u32")}, ""},
                           {"const.u32.0x00000001", {}, {var("one", "u32")}, ""}, {"u32.shr", {var("lhs", "u32"), var("shift", "u32")}, {var("shr", "u32")}, ""},
                           {"u32.shl", {var("one", "u32"), var("shift", "u32")}, {var("shl", "u32")}, ""},
                           {"u32.sub", {var("shr", "u32"), var("shl", "u32")}, {var("r", "u32")}, ""}}));
    // tests/cases/reducec/basic.hex:27-58 and tests/runtime.rs:713-726
    mods.push_back(module("sum-u64", {var("m", "mem")}, {var("r", "u64")},
                          {{"mem.cast.u64", {var("m", "mem")}, {var("len", "u64"), var("input", "ptr<u64>")}, ""},
                           {"const.u64.0x0000000000000000", {}, {var("zero", "u64")}, ""}, {"unit.intro", {}, {var("unit", "erased")}, ""},
                           {"reducec", {var("zero", "u64"), var("unit", "erased"), lw::Operand::fn("u64.add-env"), var("input", "ptr<u64>"),
                                        lw::Operand::fn("sum-u64-at"), var("len", "u64")}, {var("r", "u64")}, "", {1, 1, 1, 1, 1, 1}, {1}}}));
    mods.push_back(module("array-head-u64", {var("m", "mem")}, {var("head", "u64")},
                          {{"mem.cast.u64", {var("m", "mem")}, {var("n", "u64"), var("buf", "ptr<u64>")}, ""}, {"u64.zero", {}, {var("z", "u64")}, ""},
                           {"u64.gt", {var("n", "u64"), var("z", "u64")}, {var("nz", "bool"), var("ht", "erased"), var("hf", "erased")}, ""},
                           {"assert", {var("nz", "bool")}, {var("h", "erased")}, ""}, {"ax-mp", {var("h", "erased"), var("ht", "erased")}, {var("proof", "erased")}, ""},
                           {"ix.zero", {var("proof", "erased")}, {var("i0", "u64")}, ""}, {"ix", {var("i0", "u64"), var("buf", "ptr<u64>")}, {var("head", "u64")}, ""}}));
    // catena-lang/examples/materializec.hex: a `materializec` whose producer has no prebuilt kernel (generic map kernel)
    mods.push_back(module("materialize-copy-u64-producer", {var("input", "ptr<u64>"), var("i", "u64")}, {var("r", "u64")},
                          {{"ix", {var("i", "u64"), var("input", "ptr<u64>")}, {var("r", "u64")}, ""}}));
    mods.push_back(module("materialize-copy-u64", {var("m", "mem")}, {var("out", "mem")},
                          {{"mem.cast.u64", {var("m", "mem")}, {var("len", "u64"), var("input", "ptr<u64>")}, ""},
                           {":.param", {var("len", "u64")}, {var("n", "erased")}, ""},
                           {"materializec", {var("len", "u64"), var("input", "ptr<u64>"), lw::Operand::fn("materialize-copy-u64-producer")},
                            {var("buf", "ptr<u64>")}, "", {1, 1, 1}, {1}},
                           {"buf.to-mem", {var("len", "u64"), var("buf", "ptr<u64>")}, {var("out", "mem")}, ""}}));
    // a fold over a buffer whose `add` is not associative (acc = acc * k + x[i] from 7): the generic map kernel runs the loop
    mods.push_back(module("my.horner-add", {var("k", "u64"), var("acc", "u64"), var("value", "u64")}, {var("r", "u64")},
                          {{"u64.mul", {var("acc", "u64"), var("k", "u64")}, {var("t", "u64")}, ""},
                           {"u64.add", {var("t", "u64"), var("value", "u64")}, {var("r", "u64")}, ""}}));
    mods.push_back(module("sum-u64-at", {var("input", "ptr<u64>"), var("i", "u64")}, {var("r", "u64")},
                          {{"ix", {var("i", "u64"), var("input", "ptr<u64>")}, {var("r", "u64")}, ""}}));
    mods.push_back(module("my.horner", {var("m", "mem"), var("k", "u64")}, {var("r", "u64")},
                          {{"mem.cast.u64", {var("m", "mem")}, {var("len", "u64"), var("input", "ptr<u64>")}, ""},
                           {"const.u64.0x0000000000000007", {}, {var("seed", "u64")}, ""},
                           {"reducec", {var("seed", "u64"), var("k", "u64"), lw::Operand::fn("my.horner-add"), var("input", "ptr<u64>"),
                                        lw::Operand::fn("sum-u64-at"), var("len", "u64")}, {var("r", "u64")}, "", {1, 1, 1, 1, 1, 1}, {1}}}));
    // tests/cases/materialize/basic.hex: out[i] = i
    mods.push_back(module("cast-index", {var("i", "u64")}, {var("r", "u64")}, {{"ix.to-u64", {var("i", "u64")}, {var("r", "u64")}, ""}}));
    mods.push_back(module("materialize-indexes-source", {var("len", "u64")}, {var("out", "mem")},
                          {{":.param", {var("len", "u64")}, {var("n", "erased")}, ""},
                           {"materializec", {var("len", "u64"), lw::Operand::fn("cast-index")}, {var("buf", "ptr<u64>")}, "", {1, 0, 1}, {1}},
                           {"buf.to-mem", {var("len", "u64"), var("buf", "ptr<u64>")}, {var("out", "mem")}, ""}}));
    return mods;
}

static const char* kMatmulSource = "(def program matmul-2x2-via-mem : x -> y = ())";

static int run_cpu() {
    Runtime rt = Runtime::from_sources({kMatmulSource});
    CHECK(rt.has("nn.softmax") && rt.has("sum-f32") && rt.has("math.exp-approx"));      // the stdlib is always there
    CHECK(rt.has("matmul-2x2-via-mem") && !rt.has("gemm-bf16-rc"));                      // only what the sources define
    CHECK(rt.signature("matmul-2x2-via-mem").symbol == "program_matmul_2x2_via_mem");   // codegen/mod.rs:379-388
    CHECK(symbol_for("tensor.argmax-f32") == "program_tensor_argmax_f32" && symbol_for("2x") == "program__2x");
    // tests/runtime.rs:128-168: errors raised before the call
    CHECK(throws_kind(ExecError::Kind::UnknownSourceFunction, [&] { rt.exec("no-such-program", {}); }));
    CHECK(throws_kind(ExecError::Kind::InputArityMismatch, [&] {
        std::vector<Value> a;
        a.push_back(Value::f32(1.0f));
        a.push_back(Value::f32(2.0f));
        rt.exec("nn.silu", std::move(a));
    }));
    CHECK(throws_kind(ExecError::Kind::TypeMismatch, [&] {
        std::vector<Value> a;
        a.push_back(Value::u64(1));
        rt.exec("nn.silu", std::move(a));
    }));
    CHECK(throws_kind(ExecError::Kind::OutputArityMismatch, [&] {
        std::vector<Value> a;
        a.push_back(Value::f32(1.0f));
        rt.exec("nn.silu", std::move(a), 2);
    }));
    bool hip_refused = false;
    try {
        Runtime::from_sources({}, GpuDialect::Hip);
    } catch (const InitError&) {
        hip_refused = true;
    }
    CHECK(hip_refused);
    // lowered modules: a scalar module runs on the host through the evaluator (no device needed)
    rt.register_modules(lowered_modules());
    CHECK(rt.has("shift-and-sub") && rt.has("sum-u64") && rt.has("array-head-u64"));
    CHECK(rt.has("materialize-copy-u64") && rt.has("materialize-indexes-source") && !rt.has("materialize-copy-u64-producer"));
    {
        // a producer that is not among the modules cannot be compiled: refused when the modules are registered
        bool refused = false;
        try {
            Runtime other = Runtime::from_sources({});
            other.register_modules({module("bad-map", {var("n", "u64")}, {var("out", "mem")},
                                           {{"materializec", {var("n", "u64"), lw::Operand::fn("no.such-producer")}, {var("buf", "ptr<u64>")}, "", {1, 0, 1}, {1}},
                                            {"buf.to-mem", {var("n", "u64"), var("buf", "ptr<u64>")}, {var("out", "mem")}, ""}})});
        } catch (const InitError&) {
            refused = true;
        }
        CHECK(refused);
    }
    {
        std::vector<Value> out = rt.exec("shift-and-sub", {}, 1);
        CHECK(out.size() == 1 && out[0].kind() == ValueKind::U32 && out[0].as_u32() == 0xFFFFFFFCu);     // tests/runtime.rs:471
    }
    Value v = Value::u32(7);
    CHECK(v.kind() == ValueKind::U32 && v.as_u32() == 7);
    Mem empty;
    CHECK(empty.is_null() && empty.len_bytes() == 0 && empty.to_f32_vec().empty());
    return 0;
}

static int run_gpu() {
    if (catena_b200_init(0) != CATENA_OK) {
        std::printf("FAILED: no device\n");
        return 1;
    }
    Runtime rt = Runtime::from_sources({kMatmulSource, "(def program gemm-bf16-rc : x -> y = ())"});
    // tests/cases/matrix.rs:6-46: [[1,2,3],[4,5,6]] . [[7,8],[9,10],[11,12]] = [58,64,139,154]
    {
        std::vector<Value> a;
        a.push_back(Value::mem(rt.mem_f32({1, 2, 3, 4, 5, 6})));
        a.push_back(Value::mem(rt.mem_f32({7, 8, 9, 10, 11, 12})));
        for (uint64_t x : {2ull, 2ull, 3ull, 6ull, 6ull, 4ull}) a.push_back(Value::u64(x));
        std::vector<Value> out = rt.exec("matmul-2x2-via-mem", std::move(a), 1);
        std::vector<float> c = out[0].as_mem().to_f32_vec();
        CHECK(c.size() == 4 && c[0] == 58.0f && c[1] == 64.0f && c[2] == 139.0f && c[3] == 154.0f);
    }
    // a length that does not match n*k is the program's runtime assert (tests/cases/matrix/matmul.hex:18-27): a status here
    CHECK(throws_kind(ExecError::Kind::Device, [&] {
        std::vector<Value> a;
        a.push_back(Value::mem(rt.mem_f32({1, 2, 3, 4, 5})));
        a.push_back(Value::mem(rt.mem_f32({7, 8, 9, 10, 11, 12})));
        for (uint64_t x : {2ull, 2ull, 3ull, 6ull, 6ull, 4ull}) a.push_back(Value::u64(x));
        rt.exec("matmul-2x2-via-mem", std::move(a));
    }));
    // tests/cases/reducec.rs:50-90
    auto fold = [&](const char* name) {
        std::vector<Value> a;
        a.push_back(Value::mem(rt.mem_f32({1.5f, -0.5f, 2.0f, 4.0f})));
        return rt.exec(name, std::move(a))[0].as_f32();
    };
    CHECK(fold("sum-f32") == 7.0f && fold("mean-f32") == 1.75f && fold("max-f32") == 4.0f);
    // tests/runtime.rs:1046-1197: argmax keeps the first index on ties; concat with an empty side
    {
        std::vector<Value> a;
        a.push_back(Value::mem(rt.mem_f32({1.0f, 5.0f, 5.0f, 2.0f})));
        CHECK(rt.exec("tensor.argmax-f32", std::move(a))[0].as_u64() == 1);
        std::vector<Value> b;
        b.push_back(Value::mem(rt.mem_f32({})));
        b.push_back(Value::mem(rt.mem_f32({3.0f, 4.0f})));
        std::vector<float> c = rt.exec("tensor.concat-f32", std::move(b))[0].as_mem().to_f32_vec();
        CHECK(c.size() == 2 && c[0] == 3.0f && c[1] == 4.0f);
    }
    // tests/runtime.rs:971-1009: softmax [1,2,4] within 6e-3 of libm, sums to 1
    {
        std::vector<Value> a;
        a.push_back(Value::mem(rt.mem_f32({1.0f, 2.0f, 4.0f})));
        std::vector<float> y = rt.exec("nn.softmax", std::move(a))[0].as_mem().to_f32_vec();
        const double e[3] = {std::exp(-3.0), std::exp(-2.0), 1.0}, d = e[0] + e[1] + e[2];
        CHECK(y.size() == 3 && std::fabs(y[0] - e[0] / d) < 6e-3 && std::fabs(y[1] - e[1] / d) < 6e-3 && std::fabs(y[2] - e[2] / d) < 6e-3);
        CHECK(std::fabs(y[0] + y[1] + y[2] - 1.0f) < 1e-5);
    }
    // the polynomial is part of the semantics: math.exp-approx(0) is 0x3F7FF8FC, not 1 (stdlib/math.hex:148-199)
    {
        std::vector<Value> a;
        a.push_back(Value::f32(0.0f));
        float r = rt.exec("math.exp-approx", std::move(a))[0].as_f32();
        uint32_t bits;
        std::memcpy(&bits, &r, 4);
        CHECK(bits == 0x3F7FF8FCu);
    }
    // lowered modules that select the u64 kernels: tests/cases/reducec.rs:6-20 and tests/runtime.rs:713-740
    rt.register_modules(lowered_modules());
    {
        std::vector<Value> a;
        a.push_back(Value::mem(rt.mem_u64({2, 3, 5, 7, 11})));
        CHECK(rt.exec("sum-u64", std::move(a))[0].as_u64() == 28);
        std::vector<Value> b;
        b.push_back(Value::mem(rt.mem_u64({0x123456789abcdef0ull, 7, 11})));
        CHECK(rt.exec("array-head-u64", std::move(b))[0].as_u64() == 0x123456789abcdef0ull);
        CHECK(throws_kind(ExecError::Kind::Device, [&] {
            std::vector<Value> c;
            c.push_back(Value::mem(rt.mem_u64({})));
            rt.exec("array-head-u64", std::move(c));
        }));
    }
    // the generic map kernel behind Runtime::exec: catena-lang/tests/cases/materializec.rs:18-31, tests/cases/materialize.rs:5-31
    {
        std::vector<Value> a;
        a.push_back(Value::mem(rt.mem_u64({3, 5, 8, 13})));
        std::vector<Value> out = rt.exec("materialize-copy-u64", std::move(a), 1);
        CHECK(out[0].as_mem().to_u64_vec() == (std::vector<uint64_t>{3, 5, 8, 13}));
        std::vector<Value> n;
        n.push_back(Value::u64(4));
        CHECK(rt.exec("materialize-indexes-source", std::move(n))[0].as_mem().to_u64_vec() == (std::vector<uint64_t>{0, 1, 2, 3}));
        std::vector<Value> z;
        z.push_back(Value::u64(0));
        std::vector<Value> empty = rt.exec("materialize-indexes-source", std::move(z));
        CHECK(empty[0].as_mem().is_null() && empty[0].as_mem().to_u64_vec().empty());
    }
    {
        std::vector<Value> a;
        a.push_back(Value::mem(rt.mem_u64({3, 5, 8, 13})));
        a.push_back(Value::u64(31));
        uint64_t want = 7;
        for (uint64_t x : {3ull, 5ull, 8ull, 13ull}) want = want * 31 + x;
        CHECK(rt.exec("my.horner", std::move(a))[0].as_u64() == want);
    }
    // bf16 GEMM through Runtime::exec: 256 x 256 x 64 of ones and twos -> every element 128 (exact in bf16)
    {
        const uint64_t m = 256, n = 256, k = 64;
        std::vector<uint16_t> a(m * k, 0x3F80), b(n * k, 0x4000);   // 1.0, 2.0
        std::vector<Value> args;
        args.push_back(Value::mem(rt.mem_bytes(a.data(), a.size() * 2)));
        args.push_back(Value::mem(rt.mem_bytes(b.data(), b.size() * 2)));
        for (uint64_t x : {m, n, k}) args.push_back(Value::u64(x));
        std::vector<uint16_t> c = rt.exec("gemm-bf16-rc", std::move(args))[0].as_mem().to_vec<uint16_t>();
        bool all = c.size() == m * n;
        for (uint16_t x : c) all = all && x == 0x4300;               // 128.0
        CHECK(all);
    }
    return 0;
}

int main(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "cpu";
    int rc = mode == "gpu" ? run_gpu() : run_cpu();
    if (rc == 0) std::printf("ok %d checks\n", g_checks);
    return rc;
}
