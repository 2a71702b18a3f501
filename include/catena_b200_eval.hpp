// Host evaluator of lowered catena modules whose assignments are scalar work (header-only, C++17).
//
// This runs behind the lowering selector's `host_scalar` plan.  The reference renders such a GpuFunction as plain C++
// statements and calls the compiled symbol on the host (catena-lang/src/codegen/gpu.rs:235-261, 287-316); this backend
// has no source generator, so it evaluates the same assignments directly with the semantics of the C expression the
// renderer would have printed:
//   primitive table        catena-lang/src/codegen/gpu.rs:322-447 (helpers :449-892)
//   integer constants      gpu.rs:672-698
//   row-major index ops    catena-lang/src/codegen/ops/row_major.rs:9-68
//   bool.ifc               catena-lang/src/codegen/ops/ifc.rs:11-41
//   eval                   gpu.rs:986-991
//   reducec                catena-lang/src/codegen/ops/reducec.rs:34-133  (acc = zero; for i < n: acc = add(env, acc, get(env, i)))
//   program calls          gpu.rs:894-916; function application gpu.rs:918-968 (a primitive symbol is inlined)
// Integer arithmetic is C unsigned arithmetic of the operand width; f32 add / sub / mul / div are single IEEE operations
// (compile the including file with -ffp-contract=off, the reference's own build rule, catena-lang/src/runtime/artifact.rs:59-80);
// f32.fma is fmaf; f32.round-to-u32 is (uint32_t)nearbyintf(x).  A failed `assert` throws AssertFailed (the generated code
// traps, catena-lang/src/codegen/prelude.rs:38-55); operands for which the generated C is undefined (u32 shifts by 32 or
// more, round-to-u32 outside [0, 2^32), row-major division by zero) throw UndefinedBehaviour.
// Buffers are HOST pointers — what a caller with host-addressable memory passes in — or DEVICE buffers (Val::device_mem),
// which host code may cast and pass on but not read.  `materializec` is a kernel launch: it goes to the `materialize`
// callback (catena_b200.hpp launches the generic map kernel there) and is refused without one (NotScalar).
#ifndef CATENA_B200_EVAL_HPP
#define CATENA_B200_EVAL_HPP

#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "catena_b200_lowering.hpp"

namespace catena_b200 {
namespace eval {

struct AssertFailed : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct UndefinedBehaviour : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct NotScalar : std::runtime_error {
    using std::runtime_error::runtime_error;
};

// One wire.  Scalars live in `bits` (bool 0 / 1, u32, u64, the bit pattern of an f32); a buffer is `ptr` (+ `bytes` for a mem).
struct Val {
    enum Kind { Erased, Scalar, Ptr, Mem, Fn } kind = Erased;
    uint64_t bits = 0;
    void* ptr = nullptr;
    uint64_t bytes = 0;   // Mem: length in bytes
    uint32_t elem = 8;    // Ptr: bytes per element (8 for ptr<u64>, 4 for ptr<f32>)
    bool device = false;  // Ptr / Mem: device memory — host code may cast it and pass it on, never read it
    std::string fn;       // Fn: target of the function symbol
    static Val scalar(uint64_t b) { Val v; v.kind = Scalar; v.bits = b; return v; }
    static Val f32(float f) { uint32_t u; std::memcpy(&u, &f, 4); return scalar(u); }
    static Val mem(void* p, uint64_t n) { Val v; v.kind = Mem; v.ptr = p; v.bytes = n; return v; }
    static Val pointer(void* p, uint32_t elem_bytes) { Val v; v.kind = Ptr; v.ptr = p; v.elem = elem_bytes; return v; }
    static Val device_mem(void* p, uint64_t n) { Val v = mem(p, n); v.device = true; return v; }
    float as_f32() const { uint32_t u = (uint32_t)bits; float f; std::memcpy(&f, &u, 4); return f; }
};

using lowering::GpuAssign;
using lowering::GpuModule;
using lowering::Operand;

class Evaluator {
public:
    // Runs a `materializec` (a kernel launch): (assignment, length, values of the environment component, producer symbol) ->
    // the buffer produced (a Ptr value).  Without it such an assignment is refused (NotScalar).
    std::function<Val(const GpuAssign&, uint64_t, const std::vector<Val>&, const std::string&)> materialize;
    // Runs a `reducec` one of whose inputs is a device buffer (the host cannot read it): (assignment, input values) -> the
    // accumulator's values.  Without it such a fold is refused when its getter dereferences the buffer.
    std::function<std::vector<Val>(const GpuAssign&, const std::vector<Val>&)> reduce;

    explicit Evaluator(const std::vector<GpuModule>& modules) {
        for (const GpuModule& m : modules) {
            by_name_[m.name] = &m;
            if (!m.source_name.empty()) {
                by_name_[m.source_name] = &m;
                by_name_[lowering::symbol_for(m.source_name)] = &m;
            }
        }
    }

    // Runs module `name` (generated symbol, source name, or a function symbol's target) on its runtime inputs.
    std::vector<Val> call(const std::string& name, const std::vector<Val>& args) const {
        const GpuModule* m = find(name);
        if (!m) throw NotScalar("no lowered module for `" + name + "`");
        Env env;
        size_t k = 0;
        for (const Operand& s : m->entry.sources) {
            if (s.lowered == "erased") continue;
            if (k >= args.size()) throw std::invalid_argument(m->entry.name + ": too few runtime inputs");
            env[s.name] = args[k++];
        }
        if (k != args.size()) throw std::invalid_argument(m->entry.name + ": too many runtime inputs");
        for (const GpuAssign& a : m->entry.assignments) assign(env, a);
        std::vector<Val> out;
        for (const Operand& t : m->entry.targets)
            if (t.lowered != "erased") out.push_back(env.at(t.name));
        return out;
    }

    // Value (bit pattern) of a scalar primitive with one runtime output over constant operands (bit patterns); false when
    // `op` is not such a primitive or the reference's generated code leaves it undefined for these operands.  Used by the
    // map-program compiler to fold constants.
    bool fold(const std::string& op, const std::vector<uint64_t>& operands, uint64_t* out) const {
        std::vector<Val> in;
        for (uint64_t b : operands) in.push_back(Val::scalar(b));
        Env env;
        const std::vector<Operand> outputs = {Operand::var("folded", "u64")};
        try {
            if (!primitive(env, op, in, outputs, {})) return false;
        } catch (const std::exception&) {
            return false;
        }
        auto it = env.find("folded");
        if (it == env.end() || it->second.kind != Val::Scalar) return false;
        *out = it->second.bits;
        return true;
    }
    // The module a generated symbol, a source name or a function symbol's target names; nullptr when there is none.
    const GpuModule* module(const std::string& name) const { return find(name); }

private:
    using Env = std::map<std::string, Val>;
    std::map<std::string, const GpuModule*> by_name_;

    const GpuModule* find(const std::string& name) const {
        auto it = by_name_.find(name);
        if (it == by_name_.end()) it = by_name_.find(lowering::symbol_for(name));
        return it == by_name_.end() ? nullptr : it->second;
    }
    static Val value(const Env& env, const Operand& o) {
        if (o.is_fn) { Val v; v.kind = Val::Fn; v.fn = o.name; return v; }
        if (o.lowered == "erased") return Val();
        return env.at(o.name);
    }
    static std::vector<Val> runtime(const std::vector<Val>& vs) {
        std::vector<Val> out;
        for (const Val& v : vs)
            if (v.kind != Val::Erased && v.kind != Val::Fn) out.push_back(v);
        return out;
    }
    // values -> the runtime outputs in order (or all outputs positionally when the counts match)
    static void bind(Env& env, const std::vector<Operand>& outputs, const std::vector<Val>& values) {
        std::vector<const Operand*> slots;
        if (values.size() == outputs.size()) {
            for (const Operand& o : outputs) slots.push_back(&o);
        } else {
            for (const Operand& o : outputs)
                if (o.lowered != "erased") slots.push_back(&o);
            if (slots.size() != values.size()) throw std::invalid_argument("value count does not match the runtime outputs");
        }
        for (size_t i = 0; i < slots.size(); ++i)
            if (slots[i]->lowered != "erased") env[slots[i]->name] = values[i];
    }
    static std::vector<std::vector<Val>> components(const std::vector<size_t>& sizes, const std::vector<Val>& items, const char* what) {
        size_t total = 0;
        for (size_t s : sizes) total += s;
        if (total != items.size()) throw std::invalid_argument(std::string(what) + ": component sizes do not cover the inputs");
        std::vector<std::vector<Val>> out;
        size_t off = 0;
        for (size_t s : sizes) {
            out.emplace_back(items.begin() + off, items.begin() + off + s);
            off += s;
        }
        return out;
    }
    static bool touches_device(const std::vector<Val>& vs) {
        for (const Val& v : vs)
            if ((v.kind == Val::Ptr || v.kind == Val::Mem) && v.device) return true;
        return false;
    }
    static const Val& single_fn(const std::vector<Val>& comp) {
        const Val* f = nullptr;
        for (const Val& v : comp)
            if (v.kind == Val::Fn) { if (f) throw std::invalid_argument("more than one function symbol in a component"); f = &v; }
        if (!f) throw std::invalid_argument("no function symbol in a component");
        return *f;
    }
    static uint64_t single_scalar(const std::vector<Val>& comp) {
        std::vector<Val> r = runtime(comp);
        if (r.size() != 1) throw std::invalid_argument("expected one runtime value in a component");
        return r[0].bits;
    }

    void assign(Env& env, const GpuAssign& a) const {
        std::vector<Val> ins;
        for (const Operand& o : a.inputs) ins.push_back(value(env, o));
        if (!a.call_symbol.empty()) {                                       // gpu.rs:894-916
            bind(env, a.outputs, call(a.call_symbol, runtime(ins)));
            return;
        }
        if (primitive(env, a.op, ins, a.outputs, a.input_sizes)) return;
        if (a.op == "bool.ifc") {                                           // ops/ifc.rs:11-41
            auto c = components(a.input_sizes, ins, "bool.ifc");
            if (c.size() != 6) throw std::invalid_argument("bool.ifc expects 6 input components");
            const bool flag = single_scalar(c[4]) != 0;
            std::vector<Val> inputs = flag ? c[0] : c[2];
            inputs.insert(inputs.end(), c[5].begin(), c[5].end());
            apply(env, single_fn(flag ? c[1] : c[3]), inputs, a.outputs);
        } else if (a.op == "eval") {                                        // gpu.rs:986-991
            if (ins.empty() || ins.back().kind != Val::Fn) throw std::invalid_argument("eval: the last input must be a function symbol");
            std::vector<Val> args(ins.begin(), ins.end() - 1);
            apply(env, ins.back(), args, a.outputs);
        } else if (a.op == "reducec" && reduce && touches_device(ins)) {
            bind(env, a.outputs, reduce(a, ins));
        } else if (a.op == "reducec") {                                     // ops/reducec.rs:34-133
            auto c = components(a.input_sizes, ins, "reducec");
            if (c.size() != 6) throw std::invalid_argument("reducec expects 6 input components");
            if (c[0].size() != a.outputs.size() || a.outputs.empty()) throw std::invalid_argument("reducec: zero does not match the accumulator arity");
            const Val& add_fn = single_fn(c[2]);
            const Val& get_fn = single_fn(c[4]);
            const uint64_t n = single_scalar(c[5]);
            std::vector<Val> acc = c[0];
            std::vector<Operand> slots, nexts;
            for (const Operand& o : a.outputs) {
                slots.push_back(Operand::var("reduce_value_" + o.name, o.lowered));
                nexts.push_back(Operand::var("reduce_next_" + o.name, o.lowered));
            }
            Env scratch;
            for (uint64_t i = 0; i < n; ++i) {
                std::vector<Val> gi = c[3];
                gi.push_back(Val::scalar(i));
                apply(scratch, get_fn, gi, slots);
                std::vector<Val> ai = c[1];
                ai.insert(ai.end(), acc.begin(), acc.end());
                for (const Operand& s : slots) ai.push_back(scratch.at(s.name));
                apply(scratch, add_fn, ai, nexts);
                for (size_t k = 0; k < nexts.size(); ++k) acc[k] = scratch.at(nexts[k].name);
            }
            bind(env, a.outputs, acc);
        } else if (a.op == "materializec" && materialize) {                 // ops/materializec.rs:84-145: len, env..., producer
            if (a.inputs.size() < 2) throw std::invalid_argument("materializec: expected len, env..., producer");
            size_t env_end = a.inputs.size() - 1;
            if (!a.input_sizes.empty()) {
                if (a.input_sizes.size() != 3 || a.input_sizes[0] != 1) throw std::invalid_argument("materializec expects the components len, env, producer");
                env_end = 1 + a.input_sizes[1];
            }
            std::vector<Val> env_values(ins.begin() + 1, ins.begin() + env_end);
            std::vector<Val> rest(ins.begin() + env_end, ins.end());
            bind(env, a.outputs, {materialize(a, ins[0].bits, runtime(env_values), single_fn(rest).fn)});
        } else {
            throw NotScalar("`" + a.op + "` is not a scalar assignment");
        }
    }

    // gpu.rs:918-968
    void apply(Env& env, const Val& fn, const std::vector<Val>& inputs, const std::vector<Operand>& outputs) const {
        if (fn.kind != Val::Fn) throw std::invalid_argument("function application needs a function symbol");
        if (primitive(env, fn.fn, inputs, outputs, {})) return;
        bind(env, outputs, call(fn.fn, runtime(inputs)));
    }

    static uint64_t parse_const(const std::string& op, size_t prefix) {
        std::string lit;
        for (size_t i = prefix; i < op.size(); ++i)
            if (op[i] != '_') lit += op[i];
        if (lit.size() < 3 || lit[0] != '0' || lit[1] != 'x') throw std::invalid_argument("invalid integer constant `" + op + "`");
        return std::stoull(lit.substr(2), nullptr, 16);
    }

    bool primitive(Env& env, const std::string& op, const std::vector<Val>& in, const std::vector<Operand>& outputs,
                   const std::vector<size_t>& input_sizes) const {
        auto need = [&](size_t n) { if (in.size() != n) throw std::invalid_argument("`" + op + "`: expected " + std::to_string(n) + " inputs"); };
        auto out1 = [&](uint64_t bits) { bind(env, outputs, {Val::scalar(bits)}); return true; };
        auto outf = [&](float f) { bind(env, outputs, {Val::f32(f)}); return true; };
        auto A = [&](size_t i) { return in[i].bits; };
        auto A32 = [&](size_t i) { return (uint32_t)in[i].bits; };
        auto AF = [&](size_t i) { return in[i].as_f32(); };
        if (op == "unit.intro" || op == "ax-mp" || op == "assert-then" || op == ":.param") return true;   // gpu.rs:372-373
        if (op == "bool.t") return out1(1);
        if (op == "bool.f") return out1(0);
        if (op == "bool.not") { need(1); return out1(!A(0)); }
        if (op == "bool.id" || op == ":.forget" || op == "u64.name" || op == "ix.to-u64") { need(1); bind(env, outputs, {in[0]}); return true; }
        if (op == "bool.copy") { need(1); bind(env, outputs, {in[0], in[0]}); return true; }
        if (op == "bool.and") { need(2); return out1(A(0) && A(1)); }
        if (op == "bool.or") { need(2); return out1(A(0) || A(1)); }
        if (op == ":.ty") {                                                  // gpu.rs:471-497
            std::vector<Val> r = runtime(in);
            if (r.size() != 1) throw std::invalid_argument(":.ty: expected one runtime input");
            for (const Operand& o : outputs)
                if (o.lowered != "erased") env[o.name] = r[0];
            return true;
        }
        if (op == "assert") { need(1); if (!A(0)) throw AssertFailed("catena assertion failed"); return true; }
        if (op == "u64.zero") return out1(0);
        if (op == "u64.one" || op == "u32.one") return out1(1);
        if (op == "f32.one") return outf(1.0f);
        if (op == "u64.add") { need(2); return out1(A(0) + A(1)); }
        if (op == "u64.sub") { need(2); return out1(A(0) - A(1)); }
        if (op == "u64.mul") { need(2); return out1(A(0) * A(1)); }
        if (op == "u64.ne") { need(2); return out1(A(0) != A(1)); }
        if (op == "u64.lt") { need(2); return out1(A(0) < A(1)); }
        if (op == "u64.lte") { need(2); return out1(A(0) <= A(1)); }
        if (op == "u64.gte") { need(2); return out1(A(0) >= A(1)); }
        if (op == "u64.eq") { need(2); return out1(A(0) == A(1)); }          // + two erased witnesses
        if (op == "u64.gt") { need(2); return out1(A(0) > A(1)); }
        if (op == "u32.add") { need(2); return out1((uint32_t)(A32(0) + A32(1))); }
        if (op == "u32.sub") { need(2); return out1((uint32_t)(A32(0) - A32(1))); }
        if (op == "u32.mul") { need(2); return out1((uint32_t)(A32(0) * A32(1))); }
        if (op == "u32.and") { need(2); return out1(A32(0) & A32(1)); }
        if (op == "u32.or") { need(2); return out1(A32(0) | A32(1)); }
        if (op == "u32.xor") { need(2); return out1(A32(0) ^ A32(1)); }
        if (op == "u32.shl" || op == "u32.shr") {
            need(2);
            if (A32(1) >= 32) throw UndefinedBehaviour("u32 shift by 32 or more");
            return out1(op == "u32.shl" ? (uint32_t)(A32(0) << A32(1)) : (uint32_t)(A32(0) >> A32(1)));
        }
        if (op == "u32.not") { need(1); return out1((uint32_t)~A32(0)); }
        if (op == "u32.eq") { need(2); return out1(A32(0) == A32(1)); }
        if (op == "u32.ne") { need(2); return out1(A32(0) != A32(1)); }
        if (op == "u32.lt") { need(2); return out1(A32(0) < A32(1)); }
        if (op == "u32.gt") { need(2); return out1(A32(0) > A32(1)); }
        if (op == "u32.lte") { need(2); return out1(A32(0) <= A32(1)); }
        if (op == "u32.gte") { need(2); return out1(A32(0) >= A32(1)); }
        if (op == "u32.to-f32") { need(1); return outf((float)A32(0)); }
        if (op == "u64.to-f32") { need(1); return outf((float)A(0)); }
        if (op == "u32.bitcast-f32") { need(1); return out1(A32(0)); }       // the wire keeps the bit pattern
        if (op == "f32.bitcast-u32") { need(1); return out1(A32(0)); }
        if (op == "f32.add") { need(2); return outf(AF(0) + AF(1)); }
        if (op == "f32.sub") { need(2); return outf(AF(0) - AF(1)); }
        if (op == "f32.mul") { need(2); return outf(AF(0) * AF(1)); }
        if (op == "f32.div") { need(2); return outf(AF(0) / AF(1)); }
        if (op == "f32.neg") { need(1); return outf(-AF(0)); }
        if (op == "f32.fma") { need(3); return outf(fmaf(AF(0), AF(1), AF(2))); }
        if (op == "f32.eq") { need(2); return out1(AF(0) == AF(1)); }
        if (op == "f32.ne") { need(2); return out1(AF(0) != AF(1)); }
        if (op == "f32.lt") { need(2); return out1(AF(0) < AF(1)); }
        if (op == "f32.gt") { need(2); return out1(AF(0) > AF(1)); }
        if (op == "f32.lte") { need(2); return out1(AF(0) <= AF(1)); }
        if (op == "f32.gte") { need(2); return out1(AF(0) >= AF(1)); }
        if (op == "f32.select" || op == "u32.select" || op == "u64.select" || op == "bool.select") {
            need(3);
            bind(env, outputs, {A(0) ? in[1] : in[2]});
            return true;
        }
        if (op == "f32.round-to-u32") {
            need(1);
            const float x = AF(0);
            if (!(x >= 0.0f && x < 4294967296.0f)) throw UndefinedBehaviour("f32.round-to-u32 outside [0, 2^32)");
            return out1((uint32_t)nearbyintf(x));
        }
        if (op == "ix.zero") { need(1); return out1(0); }
        if (op == "ix") {                                                    // gpu.rs:850-864: buffer[index]
            need(2);
            if (in[1].kind != Val::Ptr) throw std::invalid_argument("ix: expected (index, buffer)");
            if (in[1].device) throw NotScalar("host code cannot dereference device memory");
            if (in[1].elem == 4) return out1(reinterpret_cast<const uint32_t*>(in[1].ptr)[A(0)]);
            return out1(reinterpret_cast<const uint64_t*>(in[1].ptr)[A(0)]);
        }
        if (op == "mem.cast.u64" || op == "mem.cast.f32") {                  // gpu.rs:752-782
            need(1);
            if (in[0].kind != Val::Mem) throw std::invalid_argument(op + ": expected a mem");
            const uint32_t elem = op == "mem.cast.u64" ? 8 : 4;
            Val p = Val::pointer(in[0].ptr, elem);
            p.device = in[0].device;
            p.bytes = in[0].bytes;
            bind(env, outputs, {Val::scalar(in[0].bytes / elem), p});
            return true;
        }
        if (op == "buf.u64.cast-same-length" || op == "buf.f32.cast-same-length") { need(2); bind(env, outputs, {in[0]}); return true; }
        if (op == "buf.to-mem") {                                            // gpu.rs:808-836
            need(2);
            if (in[1].kind != Val::Ptr) throw std::invalid_argument("buf.to-mem: expected (len, buffer)");
            Val m = Val::mem(in[1].ptr, A(0) * in[1].elem);
            m.device = in[1].device;
            bind(env, outputs, {m});
            return true;
        }
        if (op == "u64.to-ix") {                                             // gpu.rs:866-892: components [index, bound, proof]
            if (input_sizes.empty()) { bind(env, outputs, {runtime(in).at(0)}); return true; }
            auto c = components(input_sizes, in, "u64.to-ix");
            bind(env, outputs, {Val::scalar(single_scalar(c.at(0)))});
            return true;
        }
        if (op == "row-major-index" || op == "row-major-row" || op == "row-major-col") {   // ops/row_major.rs:9-68
            std::vector<Val> r = runtime(in);
            if (op == "row-major-index") {
                if (r.size() != 3) throw std::invalid_argument("row-major-index: expected (cols, row, col)");
                return out1(r[1].bits * r[0].bits + r[2].bits);
            }
            if (r.size() != 2) throw std::invalid_argument(op + ": expected (cols, flat)");
            if (r[0].bits == 0) throw UndefinedBehaviour("row-major division by zero columns");
            return out1(op == "row-major-row" ? r[1].bits / r[0].bits : r[1].bits % r[0].bits);
        }
        if (op.rfind("const.u64.", 0) == 0) return out1(parse_const(op, 10));
        if (op.rfind("const.u32.", 0) == 0) return out1((uint32_t)parse_const(op, 10));
        return false;
    }
};

}  // namespace eval
}  // namespace catena_b200

#endif  // CATENA_B200_EVAL_HPP
