// The C++ host evaluator (include/catena_b200_eval.hpp) on hand-lowered modules of the reference's test programs: the
// same vectors as tests/test_evaluator.py, with the reference's file:line beside each group.  Prints "ok <n> checks".
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "catena_b200_eval.hpp"

using namespace catena_b200::lowering;
using catena_b200::eval::AssertFailed;
using catena_b200::eval::Evaluator;
using catena_b200::eval::UndefinedBehaviour;
using catena_b200::eval::Val;

static int g_checks = 0;
#define CHECK(cond)                                                       \
    do {                                                                  \
        ++g_checks;                                                       \
        if (!(cond)) {                                                    \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            return 1;                                                     \
        }                                                                 \
    } while (0)

static Operand v(const std::string& n, const std::string& l) { return Operand::var(n, l); }
static Operand f(const std::string& n) { return Operand::fn(n); }
static GpuAssign A(const std::string& op, std::vector<Operand> ins, std::vector<Operand> outs, std::vector<size_t> in_sizes = {},
                   std::vector<size_t> out_sizes = {}, const std::string& call = "") {
    return GpuAssign{op, std::move(ins), std::move(outs), call, std::move(in_sizes), std::move(out_sizes)};
}
static GpuModule M(const std::string& source_name, std::vector<Operand> sources, std::vector<Operand> targets, std::vector<GpuAssign> assigns,
                   bool internal = false) {
    GpuModule m;
    m.name = internal ? source_name : symbol_for(source_name);
    m.source_name = internal ? "" : source_name;
    m.entry.name = m.name;
    m.entry.sources = std::move(sources);
    m.entry.targets = std::move(targets);
    m.entry.assignments = std::move(assigns);
    return m;
}
static float bits_f32(uint32_t u) { float x; std::memcpy(&x, &u, 4); return x; }

int main() {
    const char *B = "bool", *U = "u64", *W = "u32", *F = "f32", *E = "erased", *P = "ptr<u64>";
    std::vector<GpuModule> mods;
    // tests/runtime.rs:37-128
    mods.push_back(M("not", {v("x0", B)}, {v("x1", B)}, {A("bool.not", {v("x0", B)}, {v("x1", B)})}));
    mods.push_back(M("not-via-function-value", {v("x0", B)}, {v("x1", B)}, {A("eval", {v("x0", B), f("bool.not")}, {v("x1", B)})}));
    mods.push_back(M("bool-ifc-primitives", {v("flag", B), v("arg", B)}, {v("r", B)},
                     {A("bool.t", {}, {v("t0", B)}), A("bool.t", {}, {v("t1", B)}),
                      A("bool.ifc", {v("t0", B), f("bool.and"), v("t1", B), f("bool.or"), v("flag", B), v("arg", B)}, {v("r", B)},
                        {1, 1, 1, 1, 1, 1}, {1})}));
    mods.push_back(M("copy-via-function-value", {}, {v("l", B), v("r", B)},
                     {A("bool.t", {}, {v("t", B)}), A("eval", {v("t", B), f("bool.copy")}, {v("l", B), v("r", B)})}));
    // tests/runtime.rs:170-212, 448-473, 333-363, 682-711
    mods.push_back(M("two-times-two", {}, {v("x3", U)},
                     {A("u64.one", {}, {v("x0", U)}), A("u64.one", {}, {v("x1", U)}), A("u64.add", {v("x0", U), v("x1", U)}, {v("x2", U)}),
                      A("u64.mul", {v("x2", U), v("x2", U)}, {v("x3", U)})}));
    mods.push_back(M("shift-and-sub", {}, {v("r", W)},
                     {A("const.u32.0x00000020", {}, {v("lhs", W)}), A("const.u32.0x00000003", {}, {v("shift", W)}),
                      A("const.u32.0x00000001", {}, {v("one", W)}), A("u32.shr", {v("lhs", W), v("shift", W)}, {v("shr", W)}),
                      A("u32.shl", {v("one", W), v("shift", W)}, {v("shl", W)}), A("u32.sub", {v("shr", W), v("shl", W)}, {v("r", W)})}));
    mods.push_back(M("fma-fused-bits", {v("a", F), v("b", F), v("c", F)}, {v("bits", W)},
                     {A("f32.fma", {v("a", F), v("b", F), v("c", F)}, {v("r", F)}), A("f32.bitcast-u32", {v("r", F)}, {v("bits", W)})}));
    mods.push_back(M("mul-add-bits", {v("a", F), v("b", F), v("c", F)}, {v("bits", W)},
                     {A("f32.mul", {v("a", F), v("b", F)}, {v("p", F)}), A("f32.add", {v("p", F), v("c", F)}, {v("r", F)}),
                      A("f32.bitcast-u32", {v("r", F)}, {v("bits", W)})}));
    mods.push_back(M("deadbeef", {}, {v("r", U)}, {A("const.u64.0xDEADBEEFDEADBEEF", {}, {v("r", U)})}));
    mods.push_back(M("f32-lt-test", {}, {v("r", B)},
                     {A("const.u32.0x3FC00000", {}, {v("lb", W)}), A("u32.bitcast-f32", {v("lb", W)}, {v("lhs", F)}),
                      A("const.u32.0x40200000", {}, {v("rb", W)}), A("u32.bitcast-f32", {v("rb", W)}, {v("rhs", F)}),
                      A("f32.lt", {v("lhs", F), v("rhs", F)}, {v("r", B)})}));
    // tests/cases/closures/conditionals.hex (tests/cases/closures.rs:9-50)
    mods.push_back(M("program_closure_ordered_pair_0", {v("a", F), v("b", F)}, {v("a", F), v("b", F)}, {}, true));
    mods.push_back(M("program_closure_ordered_pair_1", {v("a", F), v("b", F)}, {v("a", F), v("b", F)}, {}, true));
    mods.push_back(M("ordered-pair", {v("lhs", F), v("rhs", F)}, {v("lo", F), v("hi", F)},
                     {A("f32.lte", {v("lhs", F), v("rhs", F)}, {v("ordered", B)}), A("unit.intro", {}, {v("unit", E)}),
                      A("bool.ifc", {v("lhs", F), v("rhs", F), f("closure.ordered-pair.0"), v("rhs", F), v("lhs", F), f("closure.ordered-pair.1"),
                                     v("ordered", B), v("unit", E)},
                        {v("lo", F), v("hi", F)}, {2, 1, 2, 1, 1, 1}, {2})}));
    // tests/cases/closures/progression.hex + sequence_stats.hex (tests/cases/closures.rs:52-104)
    mods.push_back(M("progression-moments-at", {v("base", U), v("step", U), v("i", U)}, {v("value", U), v("square", U)},
                     {A("ix.to-u64", {v("i", U)}, {v("iu", U)}), A("u64.mul", {v("step", U), v("iu", U)}, {v("off", U)}),
                      A("u64.add", {v("base", U), v("off", U)}, {v("value", U)}), A("u64.mul", {v("value", U), v("value", U)}, {v("square", U)})}));
    mods.push_back(M("progression-moments-add", {v("ls", U), v("lq", U), v("rs", U), v("rq", U)}, {v("s", U), v("q", U)},
                     {A("u64.add", {v("ls", U), v("rs", U)}, {v("s", U)}), A("u64.add", {v("lq", U), v("rq", U)}, {v("q", U)})}));
    mods.push_back(M("program_closure_progression_moments_0", {v("base", U), v("step", U), v("i", U)}, {v("value", U), v("square", U)},
                     {A("progression-moments-at", {v("base", U), v("step", U), v("i", U)}, {v("value", U), v("square", U)}, {}, {},
                        symbol_for("progression-moments-at"))},
                     true));
    mods.push_back(M("progression-moments", {v("len", U), v("base", U), v("step", U)}, {v("sum", U), v("squares", U)},
                     {A(":.ty", {v("len", U)}, {v("reduce-len", U), v("producer-len", U)}),
                      A("const.u64.0x0000000000000000", {}, {v("z0", U)}), A("const.u64.0x0000000000000000", {}, {v("z1", U)}),
                      A("reducec", {v("z0", U), v("z1", U), f("progression-moments-add"), v("base", U), v("step", U),
                                    f("closure.progression-moments.0"), v("reduce-len", U)},
                        {v("sum", U), v("squares", U)}, {2, 0, 1, 2, 1, 1}, {2})}));
    // tests/cases/reducec/basic.hex (tests/cases/reducec.rs:6-48) and tests/runtime.rs:713-740, on host buffers
    mods.push_back(M("u64.add-env", {v("acc", U), v("value", U)}, {v("r", U)}, {A("u64.add", {v("acc", U), v("value", U)}, {v("r", U)})}));
    mods.push_back(M("sum-u64-at", {v("input", P), v("i", U)}, {v("r", U)}, {A("ix", {v("i", U), v("input", P)}, {v("r", U)})}));
    mods.push_back(M("sum-u64", {v("m", "mem")}, {v("r", U)},
                     {A("mem.cast.u64", {v("m", "mem")}, {v("len", U), v("input", P)}), A("const.u64.0x0000000000000000", {}, {v("zero", U)}),
                      A("unit.intro", {}, {v("unit", E)}),
                      A("reducec", {v("zero", U), v("unit", E), f("u64.add-env"), v("input", P), f("sum-u64-at"), v("len", U)}, {v("r", U)},
                        {1, 1, 1, 1, 1, 1}, {1})}));
    mods.push_back(M("array-head-u64", {v("m", "mem")}, {v("head", U)},
                     {A("mem.cast.u64", {v("m", "mem")}, {v("n", U), v("buf", P)}), A("u64.zero", {}, {v("z", U)}),
                      A("u64.gt", {v("n", U), v("z", U)}, {v("nz", B), v("ht", E), v("hf", E)}), A("assert", {v("nz", B)}, {v("h", E)}),
                      A("ax-mp", {v("h", E), v("ht", E)}, {v("proof", E)}), A("ix.zero", {v("proof", E)}, {v("i0", U)}),
                      A("ix", {v("i0", U), v("buf", P)}, {v("head", U)})}));

    Evaluator ev(mods);
    auto S = [](uint64_t b) { return Val::scalar(b); };
    CHECK(ev.call("not", {S(0)})[0].bits == 1);
    CHECK(ev.call("not-via-function-value", {S(0)})[0].bits == 1 && ev.call("not-via-function-value", {S(1)})[0].bits == 0);
    const int ifc[4][3] = {{1, 0, 0}, {1, 1, 1}, {0, 0, 1}, {0, 1, 1}};
    for (auto& c : ifc) CHECK(ev.call("bool-ifc-primitives", {S(c[0]), S(c[1])})[0].bits == (uint64_t)c[2]);
    {
        auto lr = ev.call("copy-via-function-value", {});
        CHECK(lr.size() == 2 && lr[0].bits == 1 && lr[1].bits == 1);
    }
    CHECK(ev.call("two-times-two", {})[0].bits == 4);
    CHECK(ev.call("shift-and-sub", {})[0].bits == 0xFFFFFFFCull);
    {
        const Val a = Val::f32(bits_f32(0x3F800001)), c = Val::f32(bits_f32(0x33800000));
        CHECK(ev.call("fma-fused-bits", {a, a, c})[0].bits == 0x3F800003);
        CHECK(ev.call("mul-add-bits", {a, a, c})[0].bits == 0x3F800002);
    }
    CHECK(ev.call("deadbeef", {})[0].bits == 0xDEADBEEFDEADBEEFull);
    CHECK(ev.call("f32-lt-test", {})[0].bits == 1);
    const float pairs[3][4] = {{3.5f, 2.0f, 2.0f, 3.5f}, {-4.0f, -1.5f, -4.0f, -1.5f}, {2.25f, 2.25f, 2.25f, 2.25f}};
    for (auto& p : pairs) {
        auto r = ev.call("ordered-pair", {Val::f32(p[0]), Val::f32(p[1])});
        CHECK(r.size() == 2 && r[0].as_f32() == p[2] && r[1].as_f32() == p[3]);
    }
    const uint64_t moments[3][5] = {{0, 7, 3, 0, 0}, {4, 2, 3, 26, 214}, {3, 1, 1, 6, 14}};
    for (auto& m : moments) {
        auto r = ev.call("progression-moments", {S(m[0]), S(m[1]), S(m[2])});
        CHECK(r.size() == 2 && r[0].bits == m[3] && r[1].bits == m[4]);
    }
    {
        std::vector<uint64_t> xs = {2, 3, 5, 7, 11};
        CHECK(ev.call("sum-u64", {Val::mem(xs.data(), xs.size() * 8)})[0].bits == 28);
        std::vector<uint64_t> hs = {0x123456789abcdef0ull, 7, 11};
        CHECK(ev.call("array-head-u64", {Val::mem(hs.data(), hs.size() * 8)})[0].bits == hs[0]);
        bool trapped = false;
        try { ev.call("array-head-u64", {Val::mem(nullptr, 0)}); } catch (const AssertFailed&) { trapped = true; }
        CHECK(trapped);
    }
    {
        std::vector<GpuModule> bad = {M("shl-32", {}, {v("r", W)}, {A("u32.one", {}, {v("o", W)}), A("const.u32.0x00000020", {}, {v("s", W)}),
                                                                    A("u32.shl", {v("o", W), v("s", W)}, {v("r", W)})})};
        bool ub = false;
        try { Evaluator(bad).call("shl-32", {}); } catch (const UndefinedBehaviour&) { ub = true; }
        CHECK(ub);
    }
    // the selector sends every one of these modules to the host, except the buffer programs
    for (const GpuModule& m : mods) {
        if (m.source_name.empty() || m.source_name == "sum-u64-at") continue;
        const KernelPlan plan = select(m);
        if (m.source_name == "sum-u64") CHECK(plan.kernel == "fold_sum_u64");
        else if (m.source_name == "array-head-u64") CHECK(plan.kernel == "array_head_u64");
        else CHECK(plan.kernel == "host_scalar");
    }
    std::printf("ok %d checks\n", g_checks);
    return 0;
}
