// The C++ map-program compiler (include/catena_b200_map_program.hpp) on hand-lowered producers: the reference's
// `materializec` programs (catena-lang/examples/materializec.hex, tests/cases/materialize/basic.hex) and three user-style
// producers (a conditional, a fold inside the producer, constants to fold).
//   list   prints every compiled program as text; tests/test_cpp_host.py compares it with the Python compiler's output for
//          the same fixtures (tests/lowered_fixtures.py), instruction by instruction
//   ptx    writes the PTX text of every program's compiled kernel into a directory (no GPU needed); tests/test_cpp_host.py
//          compares it with the Python side's text and assembles it
//   gpu    launches the programs — as their compiled kernels, then on the interpreter — and checks the reference's vectors
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "catena_b200_map_program.hpp"

using namespace catena_b200;
using lowering::GpuAssign;
using lowering::GpuModule;
using lowering::Operand;

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
static Operand u(const std::string& n) { return v(n, "u64"); }
static Operand f(const std::string& n) { return v(n, "f32"); }
static Operand e(const std::string& n) { return v(n, "erased"); }
static Operand pu(const std::string& n) { return v(n, "ptr<u64>"); }
static Operand pf(const std::string& n) { return v(n, "ptr<f32>"); }
static Operand fn(const std::string& n) { return Operand::fn(n); }
static GpuAssign A(const std::string& op, std::vector<Operand> ins, std::vector<Operand> outs, std::vector<size_t> in_sizes = {},
                   std::vector<size_t> out_sizes = {}, const std::string& call = "") {
    return GpuAssign{op, std::move(ins), std::move(outs), call, std::move(in_sizes), std::move(out_sizes)};
}
static GpuModule M(const std::string& source_name, std::vector<Operand> sources, std::vector<Operand> targets, std::vector<GpuAssign> assigns,
                   const std::string& symbol = "") {
    GpuModule m;
    m.name = symbol.empty() ? lowering::symbol_for(source_name) : symbol;
    m.source_name = symbol.empty() ? source_name : "";
    m.entry.name = m.name;
    m.entry.sources = std::move(sources);
    m.entry.targets = std::move(targets);
    m.entry.assignments = std::move(assigns);
    return m;
}

// the same modules as tests/lowered_fixtures.py: materialize_programs() and the clamp / matvec part of custom_map_programs()
static std::vector<GpuModule> fixtures() {
    std::vector<GpuModule> m;
    m.push_back(M("materialize-index-producer", {e("env"), u("i")}, {u("r")}, {A("u64.one", {}, {u("r")})}));
    m.push_back(M("materialize-indexes", {u("len")}, {v("out", "mem")},
                  {A("unit.intro", {}, {e("unit")}), A(":.param", {u("len")}, {e("n")}),
                   A("materializec", {u("len"), e("unit"), fn("materialize-index-producer")}, {pu("buf")}, {1, 1, 1}, {1}),
                   A("buf.to-mem", {u("len"), pu("buf")}, {v("out", "mem")})}));
    m.push_back(M("materialize-copy-u64-producer", {pu("input"), u("i")}, {u("r")}, {A("ix", {u("i"), pu("input")}, {u("r")})}));
    m.push_back(M("materialize-copy-u64", {v("m", "mem")}, {v("out", "mem")},
                  {A("mem.cast.u64", {v("m", "mem")}, {u("len"), pu("input")}), A(":.param", {u("len")}, {e("n")}),
                   A("materializec", {u("len"), pu("input"), fn("materialize-copy-u64-producer")}, {pu("buf")}, {1, 1, 1}, {1}),
                   A("buf.to-mem", {u("len"), pu("buf")}, {v("out", "mem")})}));
    m.push_back(M("cast-index", {u("i")}, {u("r")}, {A("ix.to-u64", {u("i")}, {u("r")})}));
    m.push_back(M("materialize-indexes-source", {u("len")}, {v("out", "mem")},
                  {A(":.param", {u("len")}, {e("n")}), A("materializec", {u("len"), fn("cast-index")}, {pu("buf")}, {1, 0, 1}, {1}),
                   A("buf.to-mem", {u("len"), pu("buf")}, {v("out", "mem")})}));
    // out[i] = x[i] >= floor ? x[i] : floor through bool.ifc over two closures that return their capture
    m.push_back(M("", {f("x")}, {f("x")}, {}, "program_closure_my_clamp_0"));
    m.push_back(M("", {f("x")}, {f("x")}, {}, "program_closure_my_clamp_1"));
    m.push_back(M("my.clamp-at", {pf("x"), f("floor"), u("i")}, {f("r")},
                  {A("ix", {u("i"), pf("x")}, {f("xi")}), A("f32.gte", {f("xi"), f("floor")}, {v("keep", "bool")}), A("unit.intro", {}, {e("unit")}),
                   A("bool.ifc", {f("xi"), fn("closure.my-clamp.0"), f("floor"), fn("closure.my-clamp.1"), v("keep", "bool"), e("unit")}, {f("r")},
                     {1, 1, 1, 1, 1, 1}, {1})}));
    m.push_back(M("my.clamp-map", {v("m", "mem"), f("floor")}, {v("out", "mem")},
                  {A("mem.cast.f32", {v("m", "mem")}, {u("len"), pf("x")}),
                   A("materializec", {u("len"), pf("x"), f("floor"), fn("my.clamp-at")}, {pf("buf")}, {1, 2, 1}, {1}),
                   A("buf.to-mem", {u("len"), pf("buf")}, {v("out", "mem")})}));
    // out[row] = fold over k < cols of a[row * cols + k] * b[k], separately rounded, ascending k
    m.push_back(M("f32.add-env", {f("acc"), f("value")}, {f("r")}, {A("f32.add", {f("acc"), f("value")}, {f("r")})}));
    m.push_back(M("my.matvec-term-at", {pf("a"), pf("b"), u("cols"), u("row"), u("k")}, {f("r")},
                  {A("row-major-index", {u("cols"), u("row"), u("k")}, {u("flat")}), A("ix", {u("flat"), pf("a")}, {f("av")}),
                   A("ix", {u("k"), pf("b")}, {f("bv")}), A("f32.mul", {f("av"), f("bv")}, {f("r")})}));
    m.push_back(M("my.matvec-at", {pf("a"), pf("b"), u("cols"), u("row")}, {f("r")},
                  {A("const.u32.0x00000000", {}, {v("zb", "u32")}), A("u32.bitcast-f32", {v("zb", "u32")}, {f("zero")}), A("unit.intro", {}, {e("unit")}),
                   A("reducec", {f("zero"), e("unit"), fn("f32.add-env"), pf("a"), pf("b"), u("cols"), u("row"), fn("my.matvec-term-at"), u("cols")},
                     {f("r")}, {1, 1, 1, 4, 1, 1}, {1})}));
    m.push_back(M("my.matvec", {v("ma", "mem"), v("mb", "mem"), u("rows")}, {v("out", "mem")},
                  {A("mem.cast.f32", {v("ma", "mem")}, {u("alen"), pf("a")}), A("mem.cast.f32", {v("mb", "mem")}, {u("cols"), pf("b")}),
                   A("materializec", {u("rows"), pf("a"), pf("b"), u("cols"), fn("my.matvec-at")}, {pf("buf")}, {1, 3, 1}, {1}),
                   A("buf.to-mem", {u("rows"), pf("buf")}, {v("out", "mem")})}));
    // straight-line f32 arithmetic: three products that feed exactly one sum or difference (fused by the compiler), one that feeds two
    m.push_back(M("my.poly-at", {pf("x"), f("s"), u("i")}, {f("r")},
                  {A("ix", {u("i"), pf("x")}, {f("xi")}), A("f32.mul", {f("xi"), f("s")}, {f("t1")}), A("f32.mul", {f("xi"), f("xi")}, {f("sq")}),
                   A("f32.add", {f("t1"), f("xi")}, {f("t2")}), A("f32.mul", {f("t2"), f("t2")}, {f("t3")}), A("f32.sub", {f("s"), f("t3")}, {f("t4")}),
                   A("f32.mul", {f("t4"), f("sq")}, {f("t5")}), A("f32.sub", {f("t5"), f("sq")}, {f("r")})}));
    m.push_back(M("my.poly-map", {v("m", "mem"), f("s")}, {v("out", "mem")},
                  {A("mem.cast.f32", {v("m", "mem")}, {u("len"), pf("x")}),
                   A("materializec", {u("len"), pf("x"), f("s"), fn("my.poly-at")}, {pf("buf")}, {1, 2, 1}, {1}),
                   A("buf.to-mem", {u("len"), pf("buf")}, {v("out", "mem")})}));
    // acc = acc * k + x[i] from 7: a fold over a buffer whose `add` is not associative (tests/lowered_fixtures.py: custom_fold_programs)
    m.push_back(M("my.horner-add", {u("k"), u("acc"), u("value")}, {u("r")},
                  {A("u64.mul", {u("acc"), u("k")}, {u("t")}), A("u64.add", {u("t"), u("value")}, {u("r")})}));
    m.push_back(M("sum-u64-at", {pu("input"), u("i")}, {u("r")}, {A("ix", {u("i"), pu("input")}, {u("r")})}));
    m.push_back(M("my.horner", {v("m", "mem"), u("k")}, {u("r")},
                  {A("mem.cast.u64", {v("m", "mem")}, {u("len"), pu("input")}), A("const.u64.0x0000000000000007", {}, {u("seed")}),
                   A("reducec", {u("seed"), u("k"), fn("my.horner-add"), pu("input"), fn("sum-u64-at"), u("len")}, {u("r")}, {1, 1, 1, 1, 1, 1}, {1})}));
    return m;
}

static const GpuAssign& reducec_of(const std::vector<GpuModule>& mods, const std::string& source_name) {
    for (const GpuModule& m : mods)
        if (m.source_name == source_name)
            for (const GpuAssign& a : m.entry.assignments)
                if (a.op == "reducec") return a;
    throw std::runtime_error("no such fixture");
}

static const GpuAssign& materializec_of(const std::vector<GpuModule>& mods, const std::string& source_name) {
    for (const GpuModule& m : mods)
        if (m.source_name == source_name)
            for (const GpuAssign& a : m.entry.assignments)
                if (a.op == "materializec") return a;
    throw std::runtime_error("no such fixture");
}

static void list(const std::string& name, const map_program::Program& p) {
    std::printf("program %s regs=%u index=%u result=%u elem=%u\n", name.c_str(), p.n_regs, p.index_reg, p.result_reg, p.elem_bytes);
    for (const auto& q : p.presets)
        std::printf("  preset %s %llu %u\n", q.kind == map_program::Preset::Const ? "const" : q.kind == map_program::Preset::Env ? "env" : "buflen",
                    (unsigned long long)q.value, q.elem);
    for (const auto& c : p.code) std::printf("  insn %u %u %u %u %u %u\n", c.op, c.dst, c.a, c.b, c.c, c.target);
}

int main(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "list";
    const std::vector<GpuModule> mods = fixtures();
    const char* names[] = {"materialize-indexes", "materialize-copy-u64", "materialize-indexes-source", "my.clamp-map", "my.matvec", "my.poly-map"};
    if (mode == "ptx") {
        // the text of every program's compiled kernel (no GPU needed): one file per program in the directory argv[2]
        const std::string dir = argc > 2 ? argv[2] : ".";
        int k = 0;
        auto write = [&](const map_program::Program& p) -> int {
            std::string text;
            CHECK(p.ptx(&text) == CATENA_OK && text.find(".target sm_100a") != std::string::npos);
            std::FILE* f = std::fopen((dir + "/program_" + std::to_string(k++) + ".ptx").c_str(), "w");
            CHECK(f != nullptr);
            std::fputs(text.c_str(), f);
            std::fclose(f);
            return 0;
        };
        for (const char* n : names) CHECK(write(map_program::for_assignment(mods, materializec_of(mods, n))) == 0);
        CHECK(write(map_program::compile_fold(mods, reducec_of(mods, "my.horner"), 0)) == 0);
        std::printf("ok %d checks\n", g_checks);
        return 0;
    }
    if (mode == "list") {
        for (const char* n : names) list(n, map_program::for_assignment(mods, materializec_of(mods, n)));
        list("my.horner", map_program::compile_fold(mods, reducec_of(mods, "my.horner"), 0));
        return 0;
    }
    // ---- gpu: the reference's vectors (catena-lang/tests/cases/materializec.rs:5-31, materialize.rs:5-31) and the two user producers
    CHECK(catena_b200_init(0) == CATENA_OK);
    auto upload = [](const void* p, uint64_t n) { catena_mem_t m{nullptr, 0}; catena_b200_mem_upload(p, n, &m); return m; };
    // every case twice: on the program's compiled kernel (the default) and on the interpreter
    for (const char* compiled : {"1", "0"}) {
    setenv("CATENA_B200_MAP_COMPILED", compiled, 1);
    {
        const auto p = map_program::for_assignment(mods, materializec_of(mods, "materialize-indexes"));
        catena_mem_t out{nullptr, 0};
        CHECK(p.launch(4, {}, &out) == CATENA_OK && out.len == 32);
        uint64_t got[4];
        CHECK(catena_b200_mem_download(out, got, 32) == CATENA_OK);
        CHECK(got[0] == 1 && got[1] == 1 && got[2] == 1 && got[3] == 1);
        catena_b200_mem_free(out);
    }
    {
        const auto p = map_program::for_assignment(mods, materializec_of(mods, "materialize-copy-u64"));
        const uint64_t data[4] = {3, 5, 8, 13};
        catena_mem_t in = upload(data, 32), out{nullptr, 0};
        CHECK(p.launch(4, {map_program::EnvValue::mem(in)}, &out) == CATENA_OK);
        uint64_t got[4];
        CHECK(catena_b200_mem_download(out, got, 32) == CATENA_OK);
        CHECK(std::memcmp(got, data, 32) == 0);
        catena_b200_mem_free(out);
        CHECK(p.launch(5, {map_program::EnvValue::mem(in)}, &out) == CATENA_E_ASSERT && out.data == nullptr);   // index 4 of 4 elements
        catena_b200_mem_free(in);
    }
    {
        const auto p = map_program::for_assignment(mods, materializec_of(mods, "materialize-indexes-source"));
        catena_mem_t out{nullptr, 0};
        CHECK(p.launch(4, {}, &out) == CATENA_OK);
        uint64_t got[4];
        CHECK(catena_b200_mem_download(out, got, 32) == CATENA_OK);
        CHECK(got[0] == 0 && got[1] == 1 && got[2] == 2 && got[3] == 3);
        catena_b200_mem_free(out);
        CHECK(p.launch(0, {}, &out) == CATENA_OK && out.data == nullptr && out.len == 0);
    }
    {
        const auto p = map_program::for_assignment(mods, materializec_of(mods, "my.clamp-map"));
        std::vector<float> x(1000);
        for (size_t i = 0; i < x.size(); ++i) x[i] = std::sin((float)i) * 2.0f;
        catena_mem_t in = upload(x.data(), x.size() * 4), out{nullptr, 0};
        CHECK(p.launch(x.size(), {map_program::EnvValue::mem(in), map_program::EnvValue::f32(0.25f)}, &out) == CATENA_OK);
        std::vector<float> got(x.size());
        CHECK(catena_b200_mem_download(out, got.data(), got.size() * 4) == CATENA_OK);
        for (size_t i = 0; i < x.size(); ++i) CHECK(got[i] == (x[i] >= 0.25f ? x[i] : 0.25f));
        catena_b200_mem_free(out);
        catena_b200_mem_free(in);
    }
    {
        const auto p = map_program::for_assignment(mods, materializec_of(mods, "my.matvec"));
        const uint64_t rows = 37, cols = 65;
        std::vector<float> a(rows * cols), b(cols);
        for (size_t i = 0; i < a.size(); ++i) a[i] = std::cos((float)i * 0.37f);
        for (size_t i = 0; i < b.size(); ++i) b[i] = std::sin((float)i * 1.3f);
        catena_mem_t ma = upload(a.data(), a.size() * 4), mb = upload(b.data(), b.size() * 4), out{nullptr, 0};
        CHECK(p.launch(rows, {map_program::EnvValue::mem(ma), map_program::EnvValue::mem(mb), map_program::EnvValue::scalar(cols)}, &out) == CATENA_OK);
        std::vector<float> got(rows);
        CHECK(catena_b200_mem_download(out, got.data(), rows * 4) == CATENA_OK);
        for (uint64_t r = 0; r < rows; ++r) {
            volatile float acc = 0.0f;          // separately rounded products and sums, ascending k (built with -ffp-contract=off)
            for (uint64_t k = 0; k < cols; ++k) {
                volatile float t = a[r * cols + k] * b[k];
                acc = acc + t;
            }
            float want = acc;
            CHECK(std::memcmp(&want, &got[r], 4) == 0);
        }
        catena_b200_mem_free(out);
        catena_b200_mem_free(ma);
        catena_b200_mem_free(mb);
    }
    {
        const auto p = map_program::for_assignment(mods, materializec_of(mods, "my.poly-map"));
        bool fused = false;
        for (const auto& c : p.code) fused = fused || c.op == CATENA_MAP_F32_MULADD || c.op == CATENA_MAP_F32_SUBMUL || c.op == CATENA_MAP_F32_MULSUB;
        CHECK(fused);
        std::vector<float> x(777);
        for (size_t i = 0; i < x.size(); ++i) x[i] = std::sin((float)i * 0.7f) * 3.0f;
        const float sc = 1.25f;
        catena_mem_t in = upload(x.data(), x.size() * 4), out{nullptr, 0};
        CHECK(p.launch(x.size(), {map_program::EnvValue::mem(in), map_program::EnvValue::f32(sc)}, &out) == CATENA_OK);
        std::vector<float> got(x.size());
        CHECK(catena_b200_mem_download(out, got.data(), got.size() * 4) == CATENA_OK);
        for (size_t i = 0; i < x.size(); ++i) {          // every operation rounded on its own (built with -ffp-contract=off)
            volatile float t1 = x[i] * sc, sq = x[i] * x[i];
            volatile float t2 = t1 + x[i];
            volatile float t3 = t2 * t2;
            volatile float t4 = sc - t3;
            volatile float t5 = t4 * sq;
            const float want = t5 - sq;
            CHECK(std::memcmp(&want, &got[i], 4) == 0);
        }
        catena_b200_mem_free(out);
        catena_b200_mem_free(in);
    }
    {
        // the sequential fold as a register program on one device thread
        const auto p = map_program::compile_fold(mods, reducec_of(mods, "my.horner"), 0);
        const uint64_t data[5] = {3, 5, 8, 13, 0x8000000000000005ull};
        catena_mem_t in = upload(data, 40), out{nullptr, 0};
        // runtime inputs of the reducec in order: seed, k, input, len
        CHECK(p.launch(1, {map_program::EnvValue::scalar(7), map_program::EnvValue::scalar(31), map_program::EnvValue::mem(in),
                           map_program::EnvValue::scalar(5)}, &out) == CATENA_OK);
        uint64_t got = 0, want = 7;
        CHECK(catena_b200_mem_download(out, &got, 8) == CATENA_OK);
        for (uint64_t x : data) want = want * 31 + x;
        CHECK(got == want);
        catena_b200_mem_free(out);
        catena_b200_mem_free(in);
    }
    }
    std::printf("ok %d checks\n", g_checks);
    return 0;
}
