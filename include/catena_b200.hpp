// C++ host-side mirror of catena-lang's runtime surface over libcatena_b200.so (header-only, C++17).
//
// Names, argument meaning and error behaviour follow the reference's Rust API:
//   Runtime::from_sources / Runtime::from_paths (`new`) / exec / mem_f32 / mem_u64   catena-lang/src/runtime/runtime.rs:104-236
//   Value, ValueKind                                                                 catena-lang/src/runtime/value.rs:5-73
//   Mem::to_f32_vec / to_u64_vec                                                     catena-lang/src/runtime/mem.rs:43-70
//   ExecError variants                                                               catena-lang/src/runtime/runtime.rs:80-102
//   GpuDialect {Hip, Cuda}                                                           catena-lang/src/codegen/mod.rs:50-54
//
// What differs, by design of a backend that SELECTS prebuilt sm_100a kernels instead of generating and compiling
// C++ per Runtime (runtime.rs:123-164, artifact.rs:56-103):
//   * from_sources does not run the catena compiler (its front end is Rust and not part of this build): it scans the
//     sources for `(def program <name>` and registers the programs the library ships a kernel for.  A program without
//     a kernel stays out of the table, so exec reports UnknownSourceFunction for it.  The stdlib is always present.
//   * register_modules takes LOWERED modules (the reference's IR after codegen, catena-lang/src/codegen/mod.rs:107-146):
//     the lowering selector (catena_b200_lowering.hpp) picks a plan for each — an entry point of the kernel library for the
//     recognised kernel shapes, the host evaluator (catena_b200_eval.hpp) for scalar modules, which the reference also
//     runs on the host, and for a `materializec` with any other scalar producer the generic map kernel, which interprets
//     the producer as a register program (catena_b200_map_program.hpp).
//   * GpuDialect::Hip is refused with InitError.
//   * Mem owns DEVICE memory and copies on to_*_vec.  Like the Rust API, exec consumes its Mem arguments: they are
//     freed when the call returns (runtime.rs:175-179, mem.rs:119-125).
//   * a failed device-side assertion or launch is ExecError::Device carrying the library status (the generated code
//     of the reference would have trapped).
// There is no CPU path: without a B200 every call that touches data fails with the library's status.
#ifndef CATENA_B200_HPP
#define CATENA_B200_HPP

#include <cstdint>
#include <cstring>
#include <fstream>
#include <functional>
#include <map>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "catena_b200.h"
#include "catena_b200_eval.hpp"
#include "catena_b200_map_program.hpp"

namespace catena_b200 {

enum class GpuDialect { Hip, Cuda };
enum class ValueKind { Bool, U32, U64, F32, Mem };

inline const char* kind_name(ValueKind k) {
    switch (k) {
        case ValueKind::Bool: return "Bool";
        case ValueKind::U32: return "U32";
        case ValueKind::U64: return "U64";
        case ValueKind::F32: return "F32";
        default: return "Mem";
    }
}

struct InitError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

struct ExecError : std::runtime_error {
    enum class Kind { UnknownSourceFunction, InputArityMismatch, OutputArityMismatch, TypeMismatch, Device };
    Kind kind;
    catena_status_t status;
    ExecError(Kind k, const std::string& what, catena_status_t s = CATENA_OK) : std::runtime_error(what), kind(k), status(s) {}
};

// Owned device buffer: fat pointer {data, len_bytes} (mem.rs:38-41).  Move-only; freed on destruction.
class Mem {
public:
    Mem() : raw_{nullptr, 0} {}
    explicit Mem(catena_mem_t raw) : raw_(raw) {}
    Mem(const Mem&) = delete;
    Mem& operator=(const Mem&) = delete;
    Mem(Mem&& o) noexcept : raw_(o.raw_) { o.raw_ = {nullptr, 0}; }
    Mem& operator=(Mem&& o) noexcept {
        if (this != &o) {
            release();
            raw_ = o.raw_;
            o.raw_ = {nullptr, 0};
        }
        return *this;
    }
    ~Mem() { release(); }

    uint64_t len_bytes() const { return raw_.len; }
    bool is_null() const { return raw_.data == nullptr; }
    catena_mem_t raw() const { return raw_; }
    // gives the buffer up without freeing it (its owner is now whoever holds raw())
    void forget() { raw_ = {nullptr, 0}; }

    template <class T>
    std::vector<T> to_vec() const {
        std::vector<T> out(raw_.len / sizeof(T));
        if (!out.empty()) {
            catena_status_t s = catena_b200_mem_download(raw_, out.data(), out.size() * sizeof(T));
            if (s != CATENA_OK) throw ExecError(ExecError::Kind::Device, std::string("mem download: ") + catena_b200_status_string(s), s);
        }
        return out;
    }
    std::vector<float> to_f32_vec() const { return to_vec<float>(); }        // mem.rs:43-56
    std::vector<uint64_t> to_u64_vec() const { return to_vec<uint64_t>(); }  // mem.rs:58-70

    static Mem from_bytes(const void* host, uint64_t bytes) {                // mem.rs:72-106
        catena_mem_t raw{nullptr, 0};
        catena_status_t s = catena_b200_mem_upload(host, bytes, &raw);
        if (s != CATENA_OK) throw ExecError(ExecError::Kind::Device, std::string("mem upload: ") + catena_b200_status_string(s), s);
        return Mem(raw);
    }

private:
    void release() {
        if (raw_.data) catena_b200_mem_free(raw_);
        raw_ = {nullptr, 0};
    }
    catena_mem_t raw_;
};

// Tagged scalar or Mem (value.rs:5-21).
class Value {
public:
    static Value boolean(bool v) { Value x(ValueKind::Bool); x.u_ = v ? 1 : 0; return x; }
    static Value u32(uint32_t v) { Value x(ValueKind::U32); x.u_ = v; return x; }
    static Value u64(uint64_t v) { Value x(ValueKind::U64); x.u_ = v; return x; }
    static Value f32(float v) { Value x(ValueKind::F32); x.f_ = v; return x; }
    static Value mem(Mem&& m) { Value x(ValueKind::Mem); x.m_ = std::move(m); return x; }

    ValueKind kind() const { return kind_; }
    bool as_bool() const { expect(ValueKind::Bool); return u_ != 0; }
    uint32_t as_u32() const { expect(ValueKind::U32); return (uint32_t)u_; }
    uint64_t as_u64() const { expect(ValueKind::U64); return u_; }
    float as_f32() const { expect(ValueKind::F32); return f_; }
    const Mem& as_mem() const { expect(ValueKind::Mem); return m_; }
    Mem& as_mem() { expect(ValueKind::Mem); return m_; }
    Mem take_mem() { expect(ValueKind::Mem); return std::move(m_); }

private:
    explicit Value(ValueKind k) : kind_(k), u_(0), f_(0.0f) {}
    void expect(ValueKind k) const {
        if (kind_ != k) throw std::logic_error(std::string("Value holds ") + kind_name(kind_) + ", not " + kind_name(k));
    }
    ValueKind kind_;
    uint64_t u_;
    float f_;
    Mem m_;
};

// C symbol of a source name (codegen/mod.rs:379-388): `program_` + name, every non-alphanumeric character replaced by `_`.
inline std::string symbol_for(const std::string& name) {
    std::string out;
    for (char ch : name) out += ((ch >= '0' && ch <= '9') || (ch >= 'a' && ch <= 'z') || (ch >= 'A' && ch <= 'Z')) ? ch : '_';
    if (!out.empty() && out[0] >= '0' && out[0] <= '9') out = "_" + out;
    return "program_" + out;
}

class Runtime {
public:
    struct Signature {
        std::string symbol;
        std::vector<ValueKind> inputs, outputs;
        // runs the program on already validated arguments; appends the outputs; returns the library status
        std::function<catena_status_t(std::vector<Value>&, std::vector<Value>&)> call;
    };

    static Runtime from_sources(const std::vector<std::string>& sources, GpuDialect dialect = GpuDialect::Cuda) {
        if (dialect != GpuDialect::Cuda)
            throw InitError("GpuDialect::Hip is not supported: this backend only selects prebuilt sm_100a CUDA kernels");
        Runtime rt;
        for (auto& kv : stdlib()) rt.table_[kv.first] = kv.second;
        const auto& user = user_programs();
        for (const std::string& text : sources) {
            size_t pos = 0;
            while ((pos = text.find("(def", pos)) != std::string::npos) {
                size_t p = pos + 4;
                auto skip_ws = [&]() { while (p < text.size() && (text[p] == ' ' || text[p] == '\t' || text[p] == '\n' || text[p] == '\r')) ++p; };
                skip_ws();
                if (text.compare(p, 7, "program") == 0) {
                    p += 7;
                    skip_ws();
                    size_t e = p;
                    while (e < text.size() && !strchr(" \t\r\n:()", text[e])) ++e;
                    auto it = user.find(text.substr(p, e - p));
                    if (it != user.end()) rt.table_[it->first] = it->second;
                }
                pos += 4;
            }
        }
        return rt;
    }
    // Runtime::new of the reference: the sources are files
    static Runtime from_paths(const std::vector<std::string>& paths, GpuDialect dialect = GpuDialect::Cuda) {
        std::vector<std::string> texts;
        for (const std::string& path : paths) {
            std::ifstream in(path);
            if (!in) throw InitError("cannot read " + path);
            std::stringstream ss;
            ss << in.rdbuf();
            texts.push_back(ss.str());
        }
        return from_sources(texts, dialect);
    }

    // Registers lowered modules: every module with a source name whose runtime interface is made of ValueKinds
    // (catena-lang/src/runtime/signature.rs:63-72) becomes callable through exec.  A module no plan exists for is an
    // InitError (the reference would have generated source for it; this backend ships no generator).
    void register_modules(std::vector<lowering::GpuModule> modules) {
        auto shared = std::make_shared<std::vector<lowering::GpuModule>>(std::move(modules));
        auto evaluator = std::make_shared<eval::Evaluator>(*shared);
        auto kind_of = [](const std::string& l, K* k) {
            if (l == "bool") *k = K::Bool; else if (l == "u32") *k = K::U32; else if (l == "u64") *k = K::U64;
            else if (l == "f32") *k = K::F32; else if (l == "mem") *k = K::Mem; else return false;
            return true;
        };
        for (const lowering::GpuModule& m : *shared) {
            if (m.source_name.empty()) continue;
            std::vector<K> ins, outs;
            bool callable = true;
            for (const auto& s : m.entry.sources) { K k; if (s.lowered == "erased") continue; if (!kind_of(s.lowered, &k)) callable = false; else ins.push_back(k); }
            for (const auto& t : m.entry.targets) { K k; if (t.lowered == "erased") continue; if (!kind_of(t.lowered, &k)) callable = false; else outs.push_back(k); }
            if (!callable) continue;                                   // a `buf` pointer on the boundary: internal
            lowering::KernelPlan plan;
            try {
                plan = lowering::select(m, *shared);
            } catch (const lowering::Unsupported& e) {
                throw InitError("no prebuilt kernel or host plan for program '" + m.source_name + "': " + e.what());
            }
            if (plan.kernel == "host_scalar") {
                const std::string name = m.name;
                std::vector<K> out_kinds = outs;
                table_[m.source_name] = Signature{plan.symbol, ins, outs, [shared, evaluator, name, out_kinds](std::vector<Value>& a, std::vector<Value>& o) {
                    std::vector<eval::Val> args;
                    for (Value& v : a) {
                        switch (v.kind()) {
                            case K::Bool: args.push_back(eval::Val::scalar(v.as_bool())); break;
                            case K::U32: args.push_back(eval::Val::scalar(v.as_u32())); break;
                            case K::U64: args.push_back(eval::Val::scalar(v.as_u64())); break;
                            case K::F32: args.push_back(eval::Val::f32(v.as_f32())); break;
                            default: return (catena_status_t)CATENA_E_BAD_ARG;       // device memory cannot be read on the host
                        }
                    }
                    std::vector<eval::Val> got;
                    try {
                        got = evaluator->call(name, args);
                    } catch (const eval::AssertFailed&) {
                        return (catena_status_t)CATENA_E_ASSERT;
                    }
                    if (got.size() != out_kinds.size()) return (catena_status_t)CATENA_E_BAD_ARG;
                    for (size_t i = 0; i < got.size(); ++i) {
                        switch (out_kinds[i]) {
                            case K::Bool: o.push_back(Value::boolean(got[i].bits != 0)); break;
                            case K::U32: o.push_back(Value::u32((uint32_t)got[i].bits)); break;
                            case K::U64: o.push_back(Value::u64(got[i].bits)); break;
                            default: o.push_back(Value::f32(got[i].as_f32())); break;
                        }
                    }
                    return (catena_status_t)CATENA_OK;
                }};
                continue;
            }
            if (plan.kernel == "map_unary" && ins == std::vector<K>{K::Mem} && outs == std::vector<K>{K::Mem}) {
                const std::string op = plan.note;
                table_[m.source_name] = Signature{plan.symbol, ins, outs, [op](std::vector<Value>& a, std::vector<Value>& o) {
                    catena_mem_t out{nullptr, 0};
                    const catena_status_t s = catena_b200_map_f32_s(op.c_str(), a[0].as_mem().raw(), &out);
                    if (s == CATENA_OK) o.push_back(Value::mem(Mem(out)));
                    return s;
                }};
                continue;
            }
            if (plan.kernel == "host_with_map_kernels" || plan.kernel == "map_unary") {
                // the producers' register programs are built now: one the map kernel cannot run is an InitError
                auto programs = std::make_shared<std::map<const lowering::GpuAssign*, map_program::Program>>();
                auto folds = std::make_shared<std::map<const lowering::GpuAssign*, map_program::FoldPlan>>();
                try {
                    for (const lowering::GpuAssign& a : m.entry.assignments) {
                        if (a.op == "materializec") (*programs)[&a] = map_program::for_assignment(*shared, a);
                        if (a.op == "reducec" && lowering::classify(a) != "scalar") (*folds)[&a] = map_program::fold_plan_for(*shared, a);
                    }
                } catch (const lowering::Unsupported& e) {
                    throw InitError("program '" + m.source_name + "': " + e.what());
                }
                const std::string name = m.name;
                std::vector<K> out_kinds = outs;
                table_[m.source_name] = Signature{plan.symbol, ins, outs, [shared, programs, folds, name, out_kinds](std::vector<Value>& a, std::vector<Value>& o) {
                    // buffers materialised during this call; what the results do not take over is freed at the end
                    std::map<void*, catena_mem_t> made;
                    catena_status_t failed = CATENA_OK;
                    eval::Evaluator ev(*shared);
                    ev.materialize = [&](const lowering::GpuAssign& assign, uint64_t len, const std::vector<eval::Val>& env, const std::string&) {
                        const map_program::Program& prog = programs->at(&assign);
                        std::vector<map_program::EnvValue> bound;
                        for (const eval::Val& v : env)
                            bound.push_back(v.kind == eval::Val::Scalar ? map_program::EnvValue::scalar(v.bits)
                                                                        : map_program::EnvValue::mem(catena_mem_t{v.ptr, v.bytes}));
                        catena_mem_t out{nullptr, 0};
                        const catena_status_t s = prog.launch(len, bound, &out);
                        if (s != CATENA_OK) { failed = s; throw eval::AssertFailed("map program failed"); }
                        if (out.data) made[out.data] = out;
                        eval::Val p = eval::Val::pointer(out.data, prog.elem_bytes);
                        p.device = true;
                        p.bytes = out.len;
                        return p;
                    };
                    auto bind_env = [](const std::vector<eval::Val>& values) {
                        std::vector<map_program::EnvValue> bound;
                        for (const eval::Val& v : values) {
                            if (v.kind == eval::Val::Scalar) bound.push_back(map_program::EnvValue::scalar(v.bits));
                            else if (v.kind == eval::Val::Ptr || v.kind == eval::Val::Mem) bound.push_back(map_program::EnvValue::mem(catena_mem_t{v.ptr, v.bytes}));
                        }
                        return bound;
                    };
                    // a `reducec` over device buffers: staged through a prebuilt fold when `add` is one and the fold is long
                    // enough to be worth two launches, else the sequential loop on one device thread
                    ev.reduce = [&](const lowering::GpuAssign& assign, const std::vector<eval::Val>& ins) {
                        const map_program::FoldPlan& plan = folds->at(&assign);
                        auto fail_with = [&](catena_status_t s) { failed = s; throw eval::AssertFailed("fold program failed"); };
                        const uint64_t count = ins.back().bits;                       // the last component is the length
                        std::vector<eval::Val> result;
                        if (plan.staged && count >= 1024 && (plan.kind != "sum_f32" || (uint32_t)ins[0].bits == 0)) {
                            std::vector<eval::Val> get_env(ins.begin() + plan.get_env_begin, ins.begin() + plan.get_env_begin + plan.get_env_size);
                            catena_mem_t values{nullptr, 0};
                            catena_status_t s = plan.getter.launch(count, bind_env(get_env), &values);
                            if (s != CATENA_OK) fail_with(s);
                            if (plan.kind == "sum_u64") {
                                uint64_t total = 0;
                                s = program_sum_u64_s(values, &total);
                                result.push_back(eval::Val::scalar(ins[0].bits + total));
                            } else {
                                float value = 0.0f;
                                s = plan.kind == "sum_f32" ? program_sum_f32_s(values, &value) : program_max_f32_s(values, &value);
                                const float zero = ins[0].as_f32();                   // f32.max-env keeps the accumulator on ties
                                result.push_back(eval::Val::f32(plan.kind == "max_f32" && zero >= value ? zero : value));
                            }
                            catena_b200_mem_free(values);
                            if (s != CATENA_OK) fail_with(s);
                            return result;
                        }
                        const std::vector<map_program::EnvValue> env = bind_env(ins);
                        for (const map_program::Program& p : plan.sequential) {
                            catena_mem_t one{nullptr, 0};
                            catena_status_t s = p.launch(1, env, &one);
                            if (s != CATENA_OK) fail_with(s);
                            uint64_t bits = 0;
                            s = catena_b200_mem_download(one, &bits, p.elem_bytes);
                            catena_b200_mem_free(one);
                            if (s != CATENA_OK) fail_with(s);
                            result.push_back(eval::Val::scalar(bits));
                        }
                        return result;
                    };
                    std::vector<eval::Val> args;
                    std::map<void*, Value*> arguments;
                    for (Value& v : a) {
                        switch (v.kind()) {
                            case K::Bool: args.push_back(eval::Val::scalar(v.as_bool())); break;
                            case K::U32: args.push_back(eval::Val::scalar(v.as_u32())); break;
                            case K::U64: args.push_back(eval::Val::scalar(v.as_u64())); break;
                            case K::F32: args.push_back(eval::Val::f32(v.as_f32())); break;
                            default:
                                args.push_back(eval::Val::device_mem(v.as_mem().raw().data, v.as_mem().raw().len));
                                if (v.as_mem().raw().data) arguments[v.as_mem().raw().data] = &v;
                        }
                    }
                    auto release = [&]() { for (auto& kv : made) catena_b200_mem_free(kv.second); made.clear(); };
                    std::vector<eval::Val> got;
                    try {
                        got = ev.call(name, args);
                    } catch (const eval::AssertFailed&) {
                        release();
                        return failed != CATENA_OK ? failed : (catena_status_t)CATENA_E_ASSERT;
                    } catch (const std::exception&) {
                        release();
                        return (catena_status_t)CATENA_E_BAD_ARG;
                    }
                    catena_status_t s = got.size() == out_kinds.size() ? CATENA_OK : CATENA_E_BAD_ARG;
                    for (size_t i = 0; s == CATENA_OK && i < got.size(); ++i) {
                        switch (out_kinds[i]) {
                            case K::Bool: o.push_back(Value::boolean(got[i].bits != 0)); break;
                            case K::U32: o.push_back(Value::u32((uint32_t)got[i].bits)); break;
                            case K::U64: o.push_back(Value::u64(got[i].bits)); break;
                            case K::F32: o.push_back(Value::f32(got[i].as_f32())); break;
                            default: {
                                if (got[i].kind != eval::Val::Mem) { s = CATENA_E_BAD_ARG; break; }
                                if (!got[i].ptr || got[i].bytes == 0) { o.push_back(Value::mem(Mem())); break; }
                                auto mine = made.find(got[i].ptr);
                                auto theirs = arguments.find(got[i].ptr);
                                if (mine != made.end()) {
                                    made.erase(mine);
                                } else if (theirs != arguments.end()) {
                                    theirs->second->as_mem().forget();       // an argument handed back: the result takes it over
                                    arguments.erase(theirs);
                                } else {
                                    s = CATENA_E_BAD_ARG;                    // a buffer the program does not own
                                    break;
                                }
                                o.push_back(Value::mem(Mem(catena_mem_t{got[i].ptr, got[i].bytes})));
                            }
                        }
                    }
                    release();
                    if (s != CATENA_OK) o.clear();
                    return s;
                }};
                continue;
            }
            // kernel shapes a user-named program can lower to: the library's entry point of that family
            typedef catena_status_t (*MemToU64)(catena_mem_t, uint64_t*);
            MemToU64 unary = plan.kernel == "fold_sum_u64" ? program_sum_u64_s : plan.kernel == "array_head_u64" ? program_array_head_u64_s : nullptr;
            if (unary && ins == std::vector<K>{K::Mem} && outs == std::vector<K>{K::U64}) {
                table_[m.source_name] = Signature{plan.symbol, ins, outs, [unary](std::vector<Value>& a, std::vector<Value>& o) {
                    uint64_t r = 0;
                    catena_status_t s = unary(a[0].as_mem().raw(), &r);
                    if (s == CATENA_OK) o.push_back(Value::u64(r));
                    return s;
                }};
            } else if (plan.kernel == "fold_dot_u64" && ins == std::vector<K>{K::Mem, K::Mem} && outs == std::vector<K>{K::U64}) {
                table_[m.source_name] = Signature{plan.symbol, ins, outs, [](std::vector<Value>& a, std::vector<Value>& o) {
                    uint64_t r = 0;
                    catena_status_t s = program_dot_u64_s(a[0].as_mem().raw(), a[1].as_mem().raw(), &r);
                    if (s == CATENA_OK) o.push_back(Value::u64(r));
                    return s;
                }};
            } else if (stdlib().count(m.source_name) || user_programs().count(m.source_name)) {
                table_[m.source_name] = stdlib().count(m.source_name) ? stdlib().at(m.source_name) : user_programs().at(m.source_name);
            } else {
                throw InitError("program '" + m.source_name + "' lowers to " + plan.kernel + ", which is only reachable under its stdlib name");
            }
        }
    }

    // memory constructors (runtime.rs:166-172; mem_bytes is additive: Mem is untyped bytes)
    Mem mem_f32(const std::vector<float>& v) const { return Mem::from_bytes(v.data(), v.size() * sizeof(float)); }
    Mem mem_u64(const std::vector<uint64_t>& v) const { return Mem::from_bytes(v.data(), v.size() * sizeof(uint64_t)); }
    Mem mem_bytes(const void* host, uint64_t bytes) const { return Mem::from_bytes(host, bytes); }

    bool has(const std::string& name) const { return table_.count(name) != 0; }
    const Signature& signature(const std::string& name) const { return table_.at(name); }

    // Runs a source-level `program` definition (runtime.rs:175-236).  `n_outputs` plays the role of the Rust const
    // generic N (pass -1 not to check it).  The Mem arguments are consumed.
    std::vector<Value> exec(const std::string& name, std::vector<Value> args, int n_outputs = -1) const {
        auto it = table_.find(name);
        if (it == table_.end()) throw ExecError(ExecError::Kind::UnknownSourceFunction, "Unknown source function '" + name + "'");
        const Signature& sig = it->second;
        if (args.size() != sig.inputs.size())
            throw ExecError(ExecError::Kind::InputArityMismatch, "Function '" + name + "' expected " + std::to_string(sig.inputs.size()) +
                                                                     " inputs, got " + std::to_string(args.size()));
        if (n_outputs >= 0 && (size_t)n_outputs != sig.outputs.size())
            throw ExecError(ExecError::Kind::OutputArityMismatch, "Function '" + name + "' expected " + std::to_string(sig.outputs.size()) +
                                                                      " outputs, got " + std::to_string(n_outputs));
        for (size_t i = 0; i < args.size(); ++i)
            if (args[i].kind() != sig.inputs[i])
                throw ExecError(ExecError::Kind::TypeMismatch, "Argument " + std::to_string(i) + " expected " + kind_name(sig.inputs[i]) +
                                                                   ", got " + kind_name(args[i].kind()));
        std::vector<Value> outs;
        catena_status_t s = sig.call(args, outs);
        args.clear();                       // inputs are moved into exec and dropped on return
        if (s != CATENA_OK)
            throw ExecError(ExecError::Kind::Device, "program '" + name + "' failed: " + catena_b200_status_string(s), s);
        return outs;
    }

private:
    using K = ValueKind;
    using Table = std::map<std::string, Signature>;
    Table table_;

    static Signature make(const std::string& name, std::vector<K> ins, std::vector<K> outs,
                          std::function<catena_status_t(std::vector<Value>&, std::vector<Value>&)> call) {
        return Signature{symbol_for(name), std::move(ins), std::move(outs), std::move(call)};
    }
    // scalar f32 -> f32 programs have no status twin: they run on the host inside the library and cannot fail
    static Signature scalar(const std::string& name, void (*fn)(float, float*)) {
        return make(name, {K::F32}, {K::F32}, [fn](std::vector<Value>& a, std::vector<Value>& o) {
            float r = 0.0f;
            fn(a[0].as_f32(), &r);
            o.push_back(Value::f32(r));
            return CATENA_OK;
        });
    }
    static Signature mem_to_mem(const std::string& name, catena_status_t (*fn)(catena_mem_t, catena_mem_t*)) {
        return make(name, {K::Mem}, {K::Mem}, [fn](std::vector<Value>& a, std::vector<Value>& o) {
            catena_mem_t r{nullptr, 0};
            catena_status_t s = fn(a[0].as_mem().raw(), &r);
            if (s == CATENA_OK) o.push_back(Value::mem(Mem(r)));
            return s;
        });
    }
    static Signature mem_to_f32(const std::string& name, catena_status_t (*fn)(catena_mem_t, float*)) {
        return make(name, {K::Mem}, {K::F32}, [fn](std::vector<Value>& a, std::vector<Value>& o) {
            float r = 0.0f;
            catena_status_t s = fn(a[0].as_mem().raw(), &r);
            if (s == CATENA_OK) o.push_back(Value::f32(r));
            return s;
        });
    }

    static const Table& stdlib() {
        static const Table t = [] {
            Table m;
            m["math.sin-approx"] = scalar("math.sin-approx", program_math_sin_approx);
            m["math.cos-approx"] = scalar("math.cos-approx", program_math_cos_approx);
            m["math.sin-approx-full-nonneg"] = scalar("math.sin-approx-full-nonneg", program_math_sin_approx_full_nonneg);
            m["math.sin-approx-full"] = scalar("math.sin-approx-full", program_math_sin_approx_full);
            m["math.log-approx"] = scalar("math.log-approx", program_math_log_approx);
            m["math.exp-approx-nonneg"] = scalar("math.exp-approx-nonneg", program_math_exp_approx_nonneg);
            m["math.exp-approx"] = scalar("math.exp-approx", program_math_exp_approx);
            m["math.exp2-approx"] = scalar("math.exp2-approx", program_math_exp2_approx);
            m["math.log2-approx"] = scalar("math.log2-approx", program_math_log2_approx);
            m["math.sqrt"] = scalar("math.sqrt", program_math_sqrt);
            m["nn.sigmoid"] = scalar("nn.sigmoid", program_nn_sigmoid);
            m["nn.silu"] = scalar("nn.silu", program_nn_silu);
            m["nn.tanh"] = scalar("nn.tanh", program_nn_tanh);
            m["nn.gelu-approx"] = scalar("nn.gelu-approx", program_nn_gelu_approx);
            m["math.powf"] = make("math.powf", {K::F32, K::F32}, {K::F32}, [](std::vector<Value>& a, std::vector<Value>& o) {
                float r = 0.0f;
                program_math_powf(a[0].as_f32(), a[1].as_f32(), &r);
                o.push_back(Value::f32(r));
                return CATENA_OK;
            });
            m["nn.softmax"] = mem_to_mem("nn.softmax", program_nn_softmax_s);
            m["nn.rmsnorm"] = mem_to_mem("nn.rmsnorm", program_nn_rmsnorm_s);
            m["sum-f32"] = mem_to_f32("sum-f32", program_sum_f32_s);
            m["mean-f32"] = mem_to_f32("mean-f32", program_mean_f32_s);
            m["max-f32"] = mem_to_f32("max-f32", program_max_f32_s);
            m["tensor.broadcast-f32"] = make("tensor.broadcast-f32", {K::F32, K::U64}, {K::Mem}, [](std::vector<Value>& a, std::vector<Value>& o) {
                catena_mem_t r{nullptr, 0};
                catena_status_t s = program_tensor_broadcast_f32_s(a[0].as_f32(), a[1].as_u64(), &r);
                if (s == CATENA_OK) o.push_back(Value::mem(Mem(r)));
                return s;
            });
            m["tensor.arange-f32"] = make("tensor.arange-f32", {K::U64}, {K::Mem}, [](std::vector<Value>& a, std::vector<Value>& o) {
                catena_mem_t r{nullptr, 0};
                catena_status_t s = program_tensor_arange_f32_s(a[0].as_u64(), &r);
                if (s == CATENA_OK) o.push_back(Value::mem(Mem(r)));
                return s;
            });
            m["tensor.slice-f32"] = make("tensor.slice-f32", {K::Mem, K::U64, K::U64}, {K::Mem}, [](std::vector<Value>& a, std::vector<Value>& o) {
                catena_mem_t r{nullptr, 0};
                catena_status_t s = program_tensor_slice_f32_s(a[0].as_mem().raw(), a[1].as_u64(), a[2].as_u64(), &r);
                if (s == CATENA_OK) o.push_back(Value::mem(Mem(r)));
                return s;
            });
            m["tensor.concat-f32"] = make("tensor.concat-f32", {K::Mem, K::Mem}, {K::Mem}, [](std::vector<Value>& a, std::vector<Value>& o) {
                catena_mem_t r{nullptr, 0};
                catena_status_t s = program_tensor_concat_f32_s(a[0].as_mem().raw(), a[1].as_mem().raw(), &r);
                if (s == CATENA_OK) o.push_back(Value::mem(Mem(r)));
                return s;
            });
            m["tensor.argmax-f32"] = make("tensor.argmax-f32", {K::Mem}, {K::U64}, [](std::vector<Value>& a, std::vector<Value>& o) {
                uint64_t r = 0;
                catena_status_t s = program_tensor_argmax_f32_s(a[0].as_mem().raw(), &r);
                if (s == CATENA_OK) o.push_back(Value::u64(r));
                return s;
            });
            return m;
        }();
        return t;
    }

    // programs a source file has to define to be callable (the reference's tests define them in .hex files)
    static const Table& user_programs() {
        static const Table t = [] {
            Table m;
            m["matmul-2x2-via-mem"] = make("matmul-2x2-via-mem", {K::Mem, K::Mem, K::U64, K::U64, K::U64, K::U64, K::U64, K::U64}, {K::Mem},
                                           [](std::vector<Value>& a, std::vector<Value>& o) {
                                               catena_mem_t r{nullptr, 0};
                                               catena_status_t s = program_matmul_2x2_via_mem_s(a[0].as_mem().raw(), a[1].as_mem().raw(), a[2].as_u64(),
                                                                                                a[3].as_u64(), a[4].as_u64(), a[5].as_u64(),
                                                                                                a[6].as_u64(), a[7].as_u64(), &r);
                                               if (s == CATENA_OK) o.push_back(Value::mem(Mem(r)));
                                               return s;
                                           });
            auto gemm = [](catena_status_t (*fn)(catena_mem_t, catena_mem_t, uint64_t, uint64_t, uint64_t, catena_mem_t*)) {
                return [fn](std::vector<Value>& a, std::vector<Value>& o) {
                    catena_mem_t r{nullptr, 0};
                    catena_status_t s = fn(a[0].as_mem().raw(), a[1].as_mem().raw(), a[2].as_u64(), a[3].as_u64(), a[4].as_u64(), &r);
                    if (s == CATENA_OK) o.push_back(Value::mem(Mem(r)));
                    return s;
                };
            };
            m["gemm-bf16-rc"] = make("gemm-bf16-rc", {K::Mem, K::Mem, K::U64, K::U64, K::U64}, {K::Mem}, gemm(program_gemm_bf16_rc_s));
            m["gemm-i8-rc"] = make("gemm-i8-rc", {K::Mem, K::Mem, K::U64, K::U64, K::U64}, {K::Mem}, gemm(program_gemm_i8_rc_s));
            m["attn-decode-bf16"] = make("attn-decode-bf16", {K::Mem, K::Mem, K::Mem, K::U64, K::U64, K::U64, K::U64, K::U64}, {K::Mem},
                                         [](std::vector<Value>& a, std::vector<Value>& o) {
                                             catena_mem_t r{nullptr, 0};
                                             catena_status_t s = program_attn_decode_bf16_s(a[0].as_mem().raw(), a[1].as_mem().raw(),
                                                                                            a[2].as_mem().raw(), a[3].as_u64(), a[4].as_u64(),
                                                                                            a[5].as_u64(), a[6].as_u64(), a[7].as_u64(), &r);
                                             if (s == CATENA_OK) o.push_back(Value::mem(Mem(r)));
                                             return s;
                                         });
            return m;
        }();
        return t;
    }
};

}  // namespace catena_b200

#endif  // CATENA_B200_HPP
