// Register programs for the generic map kernel (header-only, C++17): what this backend does with a `materializec` whose
// producer no prebuilt kernel matches.
//
// The reference renders such a producer as C++ inside a one-thread-per-element kernel and compiles it with nvcc when the
// Runtime is built (catena-lang/src/codegen/ops/materializec.rs:36-82; function application gpu.rs:918-968).  Here the
// producer's lowered assignments are translated once into a register program — the walk of the host evaluator
// (catena_b200_eval.hpp), emitting an instruction where the evaluator computes a value — and `catena_b200_map_program_s`
// (catena_b200.h) interprets it for every index:
//   primitive                       one instruction (the table of catena-lang/src/codegen/gpu.rs:322-447); over constants: folded
//   constants, `*.one`, `bool.t/f`  preset registers
//   program call, `eval`            inlined
//   `bool.ifc`                      JZ / JMP around the two inlined functions (ops/ifc.rs:11-41)
//   `reducec` inside the producer   a loop: acc = zero; for i < n: acc = add(env, acc, get(env, i)) (ops/reducec.rs:34-133)
//   `row-major-index/row/col`       MUL + ADD / DIV / REM on u64 (ops/row_major.rs:9-68)
//   `ix` on a buffer                bounds-checked LOAD; buffers are known when the program is built, so `mem.cast.*` and
//                                   `buf.*.cast-same-length` cost nothing and a buffer's length is a preset register
// The environment of the producer (scalars and buffers) is bound at launch time: Program::launch(len, env, &out).
#ifndef CATENA_B200_MAP_PROGRAM_HPP
#define CATENA_B200_MAP_PROGRAM_HPP

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <tuple>
#include <vector>

#include "catena_b200.h"
#include "catena_b200_eval.hpp"
#include "catena_b200_lowering.hpp"

namespace catena_b200 {
namespace map_program {

using lowering::GpuAssign;
using lowering::GpuModule;
using lowering::Operand;
using lowering::Unsupported;

// One value of a producer's environment at launch time.
struct EnvValue {
    uint64_t bits = 0;          // scalar: bool 0 / 1, u32, u64, or the bit pattern of an f32
    catena_mem_t buffer = {nullptr, 0};
    static EnvValue scalar(uint64_t b) { EnvValue e; e.bits = b; return e; }
    static EnvValue f32(float f) { uint32_t u; std::memcpy(&u, &f, 4); return scalar(u); }
    static EnvValue mem(catena_mem_t m) { EnvValue e; e.buffer = m; return e; }
};

struct Preset {
    enum Kind { Const, Env, BufLen } kind = Const;
    uint64_t value = 0;         // Const: the value; Env / BufLen: position in the environment
    uint32_t elem = 0;          // BufLen: bytes per element
    bool operator<(const Preset& o) const { return std::tie(kind, value, elem) < std::tie(o.kind, o.value, o.elem); }
};

// The kernels compiled for one program, one per device; shared by the copies of the Program and released with the last one.
struct CompiledKernels {
    std::mutex lock;
    std::map<int, catena_b200_map_kernel_t*> by_device;
    CompiledKernels() = default;
    CompiledKernels(const CompiledKernels&) = delete;
    CompiledKernels& operator=(const CompiledKernels&) = delete;
    ~CompiledKernels() {
        for (auto& kv : by_device) catena_b200_map_kernel_release(kv.second);
    }
};

// How a launch runs: the program's own compiled kernel (PTX written by the library, compiled by the driver once per device) or
// the library's interpreter.  Both give the same bits.  Default: compiled, unless CATENA_B200_MAP_COMPILED=0 is in the environment.
enum class Mode { Default, Compiled, Interpreted };

struct Program {
    std::string producer;
    std::vector<catena_b200_map_insn_t> code;
    std::vector<Preset> presets;           // register k < presets.size() is preset
    uint32_t n_regs = 1, index_reg = 0, result_reg = 0, elem_bytes = 8;
    std::vector<bool> env_is_buffer;       // one entry per runtime environment value
    // the kernels compiled from `code`, shared by copies of the program; give an edited copy a fresh one
    std::shared_ptr<CompiledKernels> kernels = std::make_shared<CompiledKernels>();

    uint32_t buffer_count() const {
        uint32_t n = 0;
        for (bool b : env_is_buffer) n += b ? 1u : 0u;
        return n;
    }

    // The kernel compiled for the calling thread's device (built on first use).
    catena_status_t compiled(catena_b200_map_kernel_t** kernel) const {
        const int device = catena_b200_current_device() < 0 ? 0 : catena_b200_current_device();
        if (!kernels) return CATENA_E_BAD_ARG;
        std::lock_guard<std::mutex> hold(kernels->lock);
        auto it = kernels->by_device.find(device);
        if (it == kernels->by_device.end()) {
            std::vector<uint64_t> init;
            std::vector<uint8_t> is_const;
            for (const Preset& p : presets) {
                init.push_back(p.kind == Preset::Const ? p.value : 0);
                is_const.push_back(p.kind == Preset::Const ? 1 : 0);
            }
            catena_b200_map_kernel_t* k = nullptr;
            const catena_status_t s = catena_b200_map_compile_s(code.data(), (uint32_t)code.size(), init.data(), is_const.data(), (uint32_t)init.size(),
                                                                n_regs, index_reg, result_reg, buffer_count(), elem_bytes, &k);
            if (s != CATENA_OK) return s;
            it = kernels->by_device.emplace(device, k).first;
        }
        *kernel = it->second;
        return CATENA_OK;
    }

    // The PTX text of the compiled kernel (needs no GPU).
    catena_status_t ptx(std::string* text) const {
        std::vector<uint64_t> init;
        std::vector<uint8_t> is_const;
        for (const Preset& p : presets) {
            init.push_back(p.kind == Preset::Const ? p.value : 0);
            is_const.push_back(p.kind == Preset::Const ? 1 : 0);
        }
        uint64_t need = 0;
        catena_status_t s = catena_b200_map_ptx_s(code.data(), (uint32_t)code.size(), init.data(), is_const.data(), (uint32_t)init.size(), n_regs,
                                                  index_reg, result_reg, buffer_count(), elem_bytes, nullptr, 0, &need);
        if (s != CATENA_OK) return s;
        std::vector<char> buf(need);
        s = catena_b200_map_ptx_s(code.data(), (uint32_t)code.size(), init.data(), is_const.data(), (uint32_t)init.size(), n_regs, index_reg,
                                  result_reg, buffer_count(), elem_bytes, buf.data(), need, nullptr);
        if (s == CATENA_OK) text->assign(buf.data());
        return s;
    }

    // out[j] = producer(env..., index0 + j) for j < len on the device; *out is owned by the caller (catena_b200_mem_free).
    // `index0` is how a map shards over GPUs: contiguous index ranges, the same program on every rank.
    catena_status_t launch(uint64_t len, const std::vector<EnvValue>& env, catena_mem_t* out, uint64_t index0 = 0, Mode mode = Mode::Default) const {
        if (env.size() != env_is_buffer.size()) return CATENA_E_BAD_ARG;
        std::vector<uint64_t> init;
        std::vector<catena_mem_t> buffers;
        for (const Preset& p : presets) {
            if (p.kind == Preset::Const) init.push_back(p.value);
            else if (p.kind == Preset::Env) init.push_back(env[p.value].bits);
            else init.push_back(env[p.value].buffer.len / p.elem);
        }
        for (size_t k = 0; k < env.size(); ++k)
            if (env_is_buffer[k]) buffers.push_back(env[k].buffer);
        if (mode == Mode::Default) {
            const char* e = getenv("CATENA_B200_MAP_COMPILED");
            mode = e && e[0] == '0' && e[1] == 0 ? Mode::Interpreted : Mode::Compiled;
        }
        if (mode == Mode::Compiled && len > 0) {
            catena_b200_map_kernel_t* k = nullptr;
            const catena_status_t s = compiled(&k);
            if (s != CATENA_OK) return s;
            return catena_b200_map_kernel_launch_s(k, init.data(), (uint32_t)init.size(), buffers.data(), (uint32_t)buffers.size(), index0, len, out);
        }
        return catena_b200_map_program_range_s(code.data(), (uint32_t)code.size(), init.data(), (uint32_t)init.size(), n_regs, index_reg,
                                               result_reg, buffers.data(), (uint32_t)buffers.size(), elem_bytes, index0, len, out);
    }
};

namespace detail {

// kMaxRegs: what the interpreter takes; a compiled kernel's registers are PTX virtual registers, up to kMaxRegsCompiled
constexpr uint32_t kMaxRegs = 256, kMaxRegsCompiled = 4096, kMaxInsns = 2048, kMaxBuffers = 16;

// a value while the program is built: a register, or a buffer of the launch's table (typed once cast)
struct Sym {
    enum Kind { Erased, Reg, Buffer, Fn } kind = Erased;
    uint32_t reg = 0;           // Reg: register; Buffer: slot
    std::string lowered;        // Buffer: "mem", "ptr<u64>", "ptr<f32>"
    std::string fn;
    static Sym r(uint32_t x) { Sym s; s.kind = Reg; s.reg = x; return s; }
    static Sym buf(uint32_t slot, std::string l) { Sym s; s.kind = Buffer; s.reg = slot; s.lowered = std::move(l); return s; }
};
using Env = std::map<std::string, Sym>;

inline int direct_op(const std::string& op) {
    static const std::map<std::string, int> table = {
        {"bool.not", CATENA_MAP_BOOL_NOT}, {"bool.and", CATENA_MAP_BOOL_AND}, {"bool.or", CATENA_MAP_BOOL_OR},
        {"u64.add", CATENA_MAP_U64_ADD}, {"u64.sub", CATENA_MAP_U64_SUB}, {"u64.mul", CATENA_MAP_U64_MUL}, {"u64.eq", CATENA_MAP_U64_EQ},
        {"u64.ne", CATENA_MAP_U64_NE}, {"u64.lt", CATENA_MAP_U64_LT}, {"u64.lte", CATENA_MAP_U64_LTE}, {"u64.gt", CATENA_MAP_U64_GT},
        {"u64.gte", CATENA_MAP_U64_GTE}, {"u64.to-f32", CATENA_MAP_U64_TO_F32},
        {"u32.add", CATENA_MAP_U32_ADD}, {"u32.sub", CATENA_MAP_U32_SUB}, {"u32.mul", CATENA_MAP_U32_MUL}, {"u32.and", CATENA_MAP_U32_AND},
        {"u32.or", CATENA_MAP_U32_OR}, {"u32.xor", CATENA_MAP_U32_XOR}, {"u32.not", CATENA_MAP_U32_NOT}, {"u32.shl", CATENA_MAP_U32_SHL},
        {"u32.shr", CATENA_MAP_U32_SHR}, {"u32.eq", CATENA_MAP_U32_EQ}, {"u32.ne", CATENA_MAP_U32_NE}, {"u32.lt", CATENA_MAP_U32_LT},
        {"u32.lte", CATENA_MAP_U32_LTE}, {"u32.gt", CATENA_MAP_U32_GT}, {"u32.gte", CATENA_MAP_U32_GTE}, {"u32.to-f32", CATENA_MAP_U32_TO_F32},
        {"f32.add", CATENA_MAP_F32_ADD}, {"f32.sub", CATENA_MAP_F32_SUB}, {"f32.mul", CATENA_MAP_F32_MUL}, {"f32.div", CATENA_MAP_F32_DIV},
        {"f32.neg", CATENA_MAP_F32_NEG}, {"f32.fma", CATENA_MAP_F32_FMA}, {"f32.eq", CATENA_MAP_F32_EQ}, {"f32.ne", CATENA_MAP_F32_NE},
        {"f32.lt", CATENA_MAP_F32_LT}, {"f32.lte", CATENA_MAP_F32_LTE}, {"f32.gt", CATENA_MAP_F32_GT}, {"f32.gte", CATENA_MAP_F32_GTE},
        {"f32.round-to-u32", CATENA_MAP_F32_ROUND_TO_U32},
        {"f32.select", CATENA_MAP_SELECT32}, {"u32.select", CATENA_MAP_SELECT32}, {"u64.select", CATENA_MAP_SELECT}, {"bool.select", CATENA_MAP_SELECT32}};
    auto it = table.find(op);
    return it == table.end() ? -1 : it->second;
}
inline bool reads_b(int op) {
    switch (op) {
    case CATENA_MAP_HALT: case CATENA_MAP_MOV: case CATENA_MAP_MOV32: case CATENA_MAP_JMP: case CATENA_MAP_JZ: case CATENA_MAP_ASSERT: case CATENA_MAP_BOOL_NOT:
    case CATENA_MAP_U64_TO_F32: case CATENA_MAP_U32_NOT: case CATENA_MAP_U32_TO_F32: case CATENA_MAP_F32_NEG: case CATENA_MAP_F32_ROUND_TO_U32:
    case CATENA_MAP_LOAD_U64: case CATENA_MAP_LOAD_F32: return false;
    default: return true;
    }
}
inline bool reads_c(int op) {
    return op == CATENA_MAP_SELECT || op == CATENA_MAP_SELECT32 || op == CATENA_MAP_F32_FMA || op == CATENA_MAP_F32_MULADD ||
           op == CATENA_MAP_F32_MULSUB || op == CATENA_MAP_F32_SUBMUL;
}
// bool / u32 / f32 values live in the low half of a register: their moves leave the high half alone
inline int mov_for(const std::string& lowered) { return (lowered == "f32" || lowered == "u32" || lowered == "bool") ? CATENA_MAP_MOV32 : CATENA_MAP_MOV; }
inline bool writes(int op) { return op != CATENA_MAP_HALT && op != CATENA_MAP_JMP && op != CATENA_MAP_JZ && op != CATENA_MAP_ASSERT; }

class Builder {
public:
    Builder(const eval::Evaluator& ev, const std::map<Preset, uint32_t>* fixed, std::vector<Preset> presets, uint32_t first_reg)
        : ev_(ev), fixed_(fixed), presets_(std::move(presets)), next_reg_(first_reg) {}

    std::vector<catena_b200_map_insn_t> code;
    const std::vector<Preset>& presets() const { return presets_; }
    uint32_t next_reg() const { return next_reg_; }

    uint32_t preset(const Preset& p) {
        if (fixed_) return fixed_->at(p);
        auto it = discovered_.find(p);
        if (it != discovered_.end()) return it->second;
        const uint32_t k = (uint32_t)presets_.size();
        discovered_[p] = k;
        presets_.push_back(p);
        return k;
    }
    uint32_t constant(uint64_t v) { Preset p; p.kind = Preset::Const; p.value = v; return preset(p); }
    uint32_t fresh() {
        const uint32_t r = next_reg_++;
        if (fixed_ && next_reg_ > kMaxRegsCompiled) throw Unsupported("the producer needs more than 4096 registers");
        return r;
    }
    size_t emit(int op, uint32_t dst = 0, uint32_t a = 0, uint32_t b = 0, uint32_t c = 0, uint32_t target = 0) {
        if (code.size() >= kMaxInsns - 1) throw Unsupported("the producer needs more than 2048 instructions");
        code.push_back(catena_b200_map_insn_t{(uint16_t)op, (uint16_t)dst, (uint16_t)a, (uint16_t)b, (uint16_t)c, 0, target});
        return code.size() - 1;
    }

    std::vector<Sym> call(const std::string& name, const std::vector<Sym>& args) {
        const GpuModule* m = ev_.module(name);
        if (!m) throw Unsupported("no lowered module for `" + name + "`");
        if (depth_ > 64) throw Unsupported("`" + name + "`: calls nest deeper than 64");
        Env env;
        size_t k = 0;
        for (const Operand& s : m->entry.sources) {
            if (s.lowered == "erased") continue;
            if (k >= args.size()) throw Unsupported(m->entry.name + ": too few runtime inputs");
            env[s.name] = args[k++];
        }
        if (k != args.size()) throw Unsupported(m->entry.name + ": too many runtime inputs");
        ++depth_;
        for (const GpuAssign& a : m->entry.assignments) assign(env, a);
        --depth_;
        std::vector<Sym> out;
        for (const Operand& t : m->entry.targets)
            if (t.lowered != "erased") out.push_back(env.at(t.name));
        return out;
    }

    void assign_in(Env& env, const GpuAssign& a) { assign(env, a); }

    void apply(Env& env, const Sym& fn, const std::vector<Sym>& inputs, const std::vector<Operand>& outputs) {
        if (fn.kind != Sym::Fn) throw Unsupported("function application needs a function symbol");
        if (primitive(env, fn.fn, inputs, outputs, {})) return;
        bind(env, outputs, call(fn.fn, runtime(inputs)));
    }

private:
    const eval::Evaluator& ev_;
    const std::map<Preset, uint32_t>* fixed_;
    std::vector<Preset> presets_;
    std::map<Preset, uint32_t> discovered_;
    uint32_t next_reg_;
    int depth_ = 0;

    static Sym value(const Env& env, const Operand& o) {
        if (o.is_fn) { Sym s; s.kind = Sym::Fn; s.fn = o.name; return s; }
        if (o.lowered == "erased") return Sym();
        return env.at(o.name);
    }
    static std::vector<Sym> runtime(const std::vector<Sym>& vs) {
        std::vector<Sym> out;
        for (const Sym& v : vs)
            if (v.kind == Sym::Reg || v.kind == Sym::Buffer) out.push_back(v);
        return out;
    }
    static void bind(Env& env, const std::vector<Operand>& outputs, const std::vector<Sym>& values) {
        std::vector<const Operand*> slots;
        if (values.size() == outputs.size()) {
            for (const Operand& o : outputs) slots.push_back(&o);
        } else {
            for (const Operand& o : outputs)
                if (o.lowered != "erased") slots.push_back(&o);
            if (slots.size() != values.size()) throw Unsupported("value count does not match the runtime outputs");
        }
        for (size_t i = 0; i < slots.size(); ++i)
            if (slots[i]->lowered != "erased") env[slots[i]->name] = values[i];
    }
    static std::vector<std::vector<Sym>> components(const std::vector<size_t>& sizes, const std::vector<Sym>& items, const char* what) {
        size_t total = 0;
        for (size_t s : sizes) total += s;
        if (sizes.empty() || total != items.size()) throw Unsupported(std::string(what) + ": component sizes do not cover the inputs");
        std::vector<std::vector<Sym>> out;
        size_t off = 0;
        for (size_t s : sizes) {
            out.emplace_back(items.begin() + off, items.begin() + off + s);
            off += s;
        }
        return out;
    }
    static const Sym& single_fn(const std::vector<Sym>& comp) {
        const Sym* f = nullptr;
        for (const Sym& v : comp)
            if (v.kind == Sym::Fn) { if (f) throw Unsupported("more than one function symbol in a component"); f = &v; }
        if (!f) throw Unsupported("no function symbol in a component");
        return *f;
    }
    static uint32_t single_reg(const std::vector<Sym>& comp) {
        std::vector<Sym> r = runtime(comp);
        if (r.size() != 1 || r[0].kind != Sym::Reg) throw Unsupported("expected one scalar in a component");
        return r[0].reg;
    }
    static uint32_t reg_of(const Sym& s, const std::string& op) {
        if (s.kind != Sym::Reg) throw Unsupported("`" + op + "` applied to a buffer");
        return s.reg;
    }

    void assign(Env& env, const GpuAssign& a) {
        std::vector<Sym> ins;
        for (const Operand& o : a.inputs) ins.push_back(value(env, o));
        if (!a.call_symbol.empty()) {
            bind(env, a.outputs, call(a.call_symbol, runtime(ins)));
            return;
        }
        if (primitive(env, a.op, ins, a.outputs, a.input_sizes)) return;
        if (a.op == "bool.ifc") {
            auto c = components(a.input_sizes, ins, "bool.ifc");
            if (c.size() != 6) throw Unsupported("bool.ifc expects 6 input components");
            const uint32_t flag = single_reg(c[4]);
            std::vector<Operand> outs;
            for (const Operand& o : a.outputs)
                if (o.lowered != "erased") outs.push_back(o);
            std::vector<uint32_t> dst;
            for (size_t k = 0; k < outs.size(); ++k) dst.push_back(fresh());
            const size_t jz = emit(CATENA_MAP_JZ, 0, flag);
            branch(c[0], c[1], c[5], outs, dst);
            const size_t jmp = emit(CATENA_MAP_JMP);
            code[jz].target = (uint32_t)code.size();
            branch(c[2], c[3], c[5], outs, dst);
            code[jmp].target = (uint32_t)code.size();
            std::vector<Sym> bound;
            for (uint32_t d : dst) bound.push_back(Sym::r(d));
            bind(env, outs, bound);
        } else if (a.op == "eval") {
            if (ins.empty() || ins.back().kind != Sym::Fn) throw Unsupported("eval: the last input must be a function symbol");
            apply(env, ins.back(), std::vector<Sym>(ins.begin(), ins.end() - 1), a.outputs);
        } else if (a.op == "reducec") {
            auto c = components(a.input_sizes, ins, "reducec");
            if (c.size() != 6) throw Unsupported("reducec expects 6 input components");
            if (c[0].size() != a.outputs.size() || a.outputs.empty()) throw Unsupported("reducec: zero does not match the accumulator arity");
            const Sym& add_fn = single_fn(c[2]);
            const Sym& get_fn = single_fn(c[4]);
            const uint32_t count = single_reg(c[5]);
            std::vector<Sym> acc;
            for (size_t k = 0; k < c[0].size(); ++k) {
                const uint32_t d = fresh();
                emit(mov_for(a.outputs[k].lowered), d, reg_of(c[0][k], "reducec"));
                acc.push_back(Sym::r(d));
            }
            const uint32_t counter = fresh(), more = fresh();
            emit(CATENA_MAP_MOV, counter, constant(0));
            const size_t top = emit(CATENA_MAP_U64_LT, more, counter, count);
            const size_t leave = emit(CATENA_MAP_JZ, 0, more);
            std::vector<Operand> slots, nexts;
            for (const Operand& o : a.outputs) {
                slots.push_back(Operand::var("reduce_value_" + o.name, o.lowered));
                nexts.push_back(Operand::var("reduce_next_" + o.name, o.lowered));
            }
            Env scratch;
            std::vector<Sym> gi = c[3];
            gi.push_back(Sym::r(counter));
            apply(scratch, get_fn, gi, slots);
            std::vector<Sym> ai = c[1];
            ai.insert(ai.end(), acc.begin(), acc.end());
            for (const Operand& s : slots) ai.push_back(scratch.at(s.name));
            apply(scratch, add_fn, ai, nexts);
            for (size_t k = 0; k < nexts.size(); ++k) emit(mov_for(nexts[k].lowered), acc[k].reg, reg_of(scratch.at(nexts[k].name), "reducec"));
            emit(CATENA_MAP_U64_ADD, counter, counter, constant(1));
            emit(CATENA_MAP_JMP, 0, 0, 0, 0, (uint32_t)top);
            code[leave].target = (uint32_t)code.size();
            bind(env, a.outputs, acc);
        } else {
            throw Unsupported("`" + a.op + "` cannot run inside a map kernel");
        }
    }

    void branch(const std::vector<Sym>& env_values, const std::vector<Sym>& fn_values, const std::vector<Sym>& argument,
                const std::vector<Operand>& outs, const std::vector<uint32_t>& dst) {
        Env scratch;
        std::vector<Sym> inputs = env_values;
        inputs.insert(inputs.end(), argument.begin(), argument.end());
        apply(scratch, single_fn(fn_values), inputs, outs);
        for (size_t k = 0; k < outs.size(); ++k) emit(mov_for(outs[k].lowered), dst[k], reg_of(scratch.at(outs[k].name), "bool.ifc"));
    }

    bool const_value(uint32_t reg, uint64_t* v) const {
        if (reg >= presets_.size() || presets_[reg].kind != Preset::Const) return false;
        *v = presets_[reg].value;
        return true;
    }

    bool primitive(Env& env, const std::string& op, const std::vector<Sym>& in, const std::vector<Operand>& outputs,
                   const std::vector<size_t>& input_sizes) {
        if (op == "unit.intro" || op == "ax-mp" || op == "assert-then" || op == ":.param") return true;
        const std::vector<Sym> rt = runtime(in);
        const int direct = direct_op(op);
        if (direct >= 0) {
            uint32_t regs[3] = {0, 0, 0};
            if (rt.empty() || rt.size() > 3) throw Unsupported("`" + op + "`: operand count");
            std::vector<uint64_t> consts;
            for (size_t k = 0; k < rt.size(); ++k) {
                regs[k] = reg_of(rt[k], op);
                uint64_t v;
                if (const_value(regs[k], &v)) consts.push_back(v);
            }
            uint64_t folded;
            if (consts.size() == rt.size() && ev_.fold(op, consts, &folded)) {
                bind(env, outputs, {Sym::r(constant(folded))});
                return true;
            }
            const uint32_t d = fresh();
            emit(direct, d, regs[0], regs[1], regs[2]);
            bind(env, outputs, {Sym::r(d)});
            return true;
        }
        auto bind_const = [&](uint64_t v) { bind(env, outputs, {Sym::r(constant(v))}); return true; };
        if (op == "bool.t" || op == "u64.one" || op == "u32.one") return bind_const(1);
        if (op == "bool.f" || op == "u64.zero") return bind_const(0);
        if (op == "f32.one") return bind_const(0x3F800000u);
        if (op.rfind("const.u64.", 0) == 0 || op.rfind("const.u32.", 0) == 0) {
            uint64_t v;
            if (!ev_.fold(op, {}, &v)) throw Unsupported("invalid integer constant `" + op + "`");
            return bind_const(v);
        }
        if (op == "bool.id" || op == ":.forget" || op == "u64.name" || op == "ix.to-u64" || op == "u32.bitcast-f32" || op == "f32.bitcast-u32" ||
            op == ":.ty") {
            if (rt.size() != 1) throw Unsupported("`" + op + "`: expected one runtime input");
            for (const Operand& o : outputs)
                if (o.lowered != "erased") env[o.name] = rt[0];
            return true;
        }
        if (op == "bool.copy") { bind(env, outputs, {rt.at(0), rt.at(0)}); return true; }
        if (op == "assert") { emit(CATENA_MAP_ASSERT, 0, reg_of(rt.at(0), op)); return true; }
        if (op == "ix.zero") return bind_const(0);
        if (op == "u64.to-ix") {
            if (input_sizes.empty()) { bind(env, outputs, {rt.at(0)}); return true; }
            auto c = components(input_sizes, in, "u64.to-ix");
            bind(env, outputs, {Sym::r(single_reg(c.at(0)))});
            return true;
        }
        if (op == "row-major-index") {
            if (rt.size() != 3) throw Unsupported("row-major-index: expected (cols, row, col)");
            const uint32_t t = fresh(), d = fresh();
            emit(CATENA_MAP_U64_MUL, t, reg_of(rt[1], op), reg_of(rt[0], op));
            emit(CATENA_MAP_U64_ADD, d, t, reg_of(rt[2], op));
            bind(env, outputs, {Sym::r(d)});
            return true;
        }
        if (op == "row-major-row" || op == "row-major-col") {
            if (rt.size() != 2) throw Unsupported(op + ": expected (cols, flat)");
            const uint32_t d = fresh();
            emit(op == "row-major-row" ? CATENA_MAP_U64_DIV : CATENA_MAP_U64_REM, d, reg_of(rt[1], op), reg_of(rt[0], op));
            bind(env, outputs, {Sym::r(d)});
            return true;
        }
        if (op == "ix") {
            if (rt.size() != 2 || rt[1].kind != Sym::Buffer || (rt[1].lowered != "ptr<u64>" && rt[1].lowered != "ptr<f32>"))
                throw Unsupported("`ix` needs (index, typed buffer)");
            const uint32_t d = fresh();
            emit(rt[1].lowered == "ptr<u64>" ? CATENA_MAP_LOAD_U64 : CATENA_MAP_LOAD_F32, d, reg_of(rt[0], op), rt[1].reg);
            bind(env, outputs, {Sym::r(d)});
            return true;
        }
        if (op == "mem.cast.u64" || op == "mem.cast.f32") {
            if (rt.size() != 1 || rt[0].kind != Sym::Buffer) throw Unsupported("`" + op + "` of something that is not a buffer");
            Preset p;
            p.kind = Preset::BufLen;
            p.value = rt[0].reg;
            p.elem = op == "mem.cast.u64" ? 8 : 4;
            bind(env, outputs, {Sym::r(preset(p)), Sym::buf(rt[0].reg, op == "mem.cast.u64" ? "ptr<u64>" : "ptr<f32>")});
            return true;
        }
        if (op == "buf.u64.cast-same-length" || op == "buf.f32.cast-same-length") { bind(env, outputs, {rt.at(0)}); return true; }
        return false;
    }
};

inline std::vector<uint32_t> reads_of(const catena_b200_map_insn_t& c) {
    std::vector<uint32_t> out;
    if (c.op != CATENA_MAP_HALT && c.op != CATENA_MAP_JMP) out.push_back(c.a);
    if (reads_b(c.op)) out.push_back(c.b);
    if (reads_c(c.op)) out.push_back(c.c);
    return out;
}

// Straight-line code before register reuse (every register is written once): an F32_MUL whose only reader is an F32_ADD /
// F32_SUB sinks into it as one instruction (two roundings, as before: not an fma) — one dispatch and one round trip through the
// register file less.  A sum takes at most one product.
inline void fuse_mul_add(std::vector<catena_b200_map_insn_t>& code, uint32_t result_reg) {
    std::map<uint32_t, uint32_t> uses;
    std::map<uint32_t, size_t> reader;
    for (size_t k = 0; k < code.size(); ++k)
        for (uint32_t r : reads_of(code[k])) {
            ++uses[r];
            reader.emplace(r, k);
        }
    ++uses[result_reg];
    std::map<size_t, size_t> fused;               // index of the sum -> index of the product it takes
    for (size_t k = 0; k < code.size(); ++k) {
        const catena_b200_map_insn_t& c = code[k];
        if (c.op != CATENA_MAP_F32_MUL || uses[c.dst] != 1 || c.dst == result_reg) continue;
        const size_t j = reader.at(c.dst);
        const catena_b200_map_insn_t& n = code[j];
        if (j > k && !fused.count(j) && (n.op == CATENA_MAP_F32_ADD || n.op == CATENA_MAP_F32_SUB) && ((n.a == c.dst) != (n.b == c.dst))) fused[j] = k;
    }
    std::set<size_t> gone;
    for (const auto& kv : fused) gone.insert(kv.second);
    std::vector<catena_b200_map_insn_t> out;
    for (size_t k = 0; k < code.size(); ++k) {
        if (gone.count(k)) continue;
        auto it = fused.find(k);
        if (it == fused.end()) {
            out.push_back(code[k]);
            continue;
        }
        const catena_b200_map_insn_t &c = code[k], &m = code[it->second];
        const uint16_t other = c.a == m.dst ? c.b : c.a;
        const int op = c.op == CATENA_MAP_F32_ADD ? CATENA_MAP_F32_MULADD : (c.a == m.dst ? CATENA_MAP_F32_MULSUB : CATENA_MAP_F32_SUBMUL);
        out.push_back(catena_b200_map_insn_t{(uint16_t)op, c.dst, m.a, m.b, other, 0, 0});
    }
    code.swap(out);
}

// Straight-line code only: every temporary is written once, so a register is free again after its last read.
inline void reuse_registers(std::vector<catena_b200_map_insn_t>& code, uint32_t n_init, uint32_t index_reg, uint32_t* result_reg, uint32_t* n_regs) {
    auto reads = [](const catena_b200_map_insn_t& c) { return reads_of(c); };
    std::map<uint32_t, size_t> last;
    for (size_t k = 0; k < code.size(); ++k)
        for (uint32_t r : reads(code[k])) last[r] = k;
    last[*result_reg] = code.size();
    std::map<uint32_t, uint32_t> mapping = {{index_reg, index_reg}};
    std::vector<uint32_t> free_regs;
    uint32_t top = index_reg + 1;
    auto mapped = [&](uint32_t r) { auto it = mapping.find(r); return it == mapping.end() ? r : it->second; };
    for (size_t k = 0; k < code.size(); ++k) {
        catena_b200_map_insn_t c = code[k];
        const std::vector<uint32_t> used = reads(c);
        catena_b200_map_insn_t n = c;
        n.a = (c.op != CATENA_MAP_HALT && c.op != CATENA_MAP_JMP) ? (uint16_t)mapped(c.a) : 0;
        n.b = reads_b(c.op) ? (uint16_t)mapped(c.b) : c.b;
        n.c = reads_c(c.op) ? (uint16_t)mapped(c.c) : 0;
        for (uint32_t r : std::set<uint32_t>(used.begin(), used.end()))
            if (r >= n_init && r != index_reg && last[r] == k && mapping.count(r)) free_regs.push_back(mapping[r]);
        n.dst = 0;
        if (writes(c.op)) {
            uint32_t d;
            if (!free_regs.empty()) { d = free_regs.back(); free_regs.pop_back(); }
            else d = top++;
            mapping[c.dst] = d;
            n.dst = (uint16_t)d;
        }
        code[k] = n;
    }
    *result_reg = mapped(*result_reg);
    *n_regs = top;
}

}  // namespace detail

namespace detail {
// Shared driver: binds `env_vars` to preset registers / buffer slots, lets body(builder, args, index) emit the code and
// return the result, finishes with HALT, runs the two passes and the register reuse.
template <class Body>
inline Program compile(const std::vector<GpuModule>& modules, const std::string& name, const std::vector<Operand>& env_vars,
                       const std::string& elem_lowered, Body body) {
    Program prog;
    prog.producer = name;
    if (elem_lowered == "u64") prog.elem_bytes = 8;
    else if (elem_lowered == "f32" || elem_lowered == "u32" || elem_lowered == "bool") prog.elem_bytes = 4;
    else throw Unsupported("a buffer of `" + elem_lowered + "` elements");
    std::vector<int> slot_of(env_vars.size(), -1);
    uint32_t n_buffers = 0;
    for (size_t k = 0; k < env_vars.size(); ++k) {
        const std::string& l = env_vars[k].lowered;
        const bool buffer = l == "mem" || l == "ptr<u64>" || l == "ptr<f32>";
        if (!buffer && l != "f32" && l != "u32" && l != "u64" && l != "bool") throw Unsupported("environment value of type `" + l + "`");
        prog.env_is_buffer.push_back(buffer);
        if (buffer) slot_of[k] = (int)n_buffers++;
    }
    if (n_buffers > kMaxBuffers) throw Unsupported("more than 16 buffers in the environment");
    const eval::Evaluator ev(modules);
    uint32_t index = 0;
    Sym result;
    auto run = [&](Builder& b) {
        std::vector<Sym> args;
        for (size_t k = 0; k < env_vars.size(); ++k) {
            if (slot_of[k] >= 0) { args.push_back(Sym::buf((uint32_t)slot_of[k], env_vars[k].lowered)); continue; }
            Preset p;
            p.kind = Preset::Env;
            p.value = k;
            args.push_back(Sym::r(b.preset(p)));
        }
        index = b.fresh();
        result = body(b, args, index);
        b.emit(CATENA_MAP_HALT);
        if (result.kind != Sym::Reg) throw Unsupported("the producer returns a buffer");
    };
    // pass 1 discovers the presets (constants appear while walking), pass 2 emits with the registers behind them
    Builder first(ev, nullptr, {}, 1u << 20);
    run(first);
    std::vector<Preset> presets = first.presets();
    std::map<Preset, uint32_t> fixed;
    for (size_t k = 0; k < presets.size(); ++k) fixed[presets[k]] = (uint32_t)k;
    if (presets.size() >= kMaxRegsCompiled) throw Unsupported("the producer needs more than 4096 registers");
    Builder second(ev, &fixed, presets, (uint32_t)presets.size());
    run(second);
    prog.code = second.code;
    prog.n_regs = second.next_reg();
    prog.index_reg = index;
    prog.result_reg = result.reg;
    bool straight = true;
    for (const auto& c : prog.code) straight = straight && c.op != CATENA_MAP_JMP && c.op != CATENA_MAP_JZ;
    if (straight) {
        fuse_mul_add(prog.code, prog.result_reg);
        reuse_registers(prog.code, (uint32_t)presets.size(), prog.index_reg, &prog.result_reg, &prog.n_regs);
    }
    // BufLen presets name buffer slots; launches index the environment
    for (Preset& p : presets)
        if (p.kind == Preset::BufLen)
            for (size_t k = 0; k < slot_of.size(); ++k)
                if (slot_of[k] == (int)p.value) { p.value = k; break; }
    prog.presets = presets;
    return prog;
}
}  // namespace detail

// Register program for out[i] = producer(env_vars..., i).  `env_vars`: the runtime values of the materializec's environment
// component (their `lowered` types decide how a launch binds them); `elem_lowered`: element type of the buffer produced.
// Throws lowering::Unsupported for a producer a map kernel cannot run.
inline Program compile_producer(const std::vector<GpuModule>& modules, const std::string& producer, const std::vector<Operand>& env_vars,
                                const std::string& elem_lowered) {
    using namespace detail;
    if (elem_lowered == "bool") throw Unsupported("materializec of `bool` elements");
    return compile(modules, producer, env_vars, elem_lowered, [&](Builder& b, std::vector<Sym> args, uint32_t index) {
        args.push_back(Sym::r(index));
        Env scratch;
        Sym fn;
        fn.kind = Sym::Fn;
        fn.fn = producer;
        const std::vector<Operand> outs = {Operand::var("value", elem_lowered)};
        b.apply(scratch, fn, args, outs);
        return scratch.at("value");
    });
}

// The runtime inputs of a `reducec` assignment, in order: what a launch of its fold programs binds.
inline std::vector<Operand> fold_inputs(const GpuAssign& a) {
    std::vector<Operand> out;
    for (const Operand& o : a.inputs)
        if (!o.is_fn && o.lowered != "erased") out.push_back(o);
    return out;
}

// Register program whose ONE element is component `component` of a reducec's result: the sequential left fold
// acc = zero; for i < n: acc = add(add_env, acc, get(get_env, i)) (catena-lang/src/codegen/ops/reducec.rs:34-133) as a loop run
// by one thread — the reference runs the same loop on one host core.  Launch with length 1 and the values of fold_inputs(a).
inline Program compile_fold(const std::vector<GpuModule>& modules, const GpuAssign& a, size_t component) {
    using namespace detail;
    std::vector<Operand> outs;
    for (const Operand& o : a.outputs)
        if (o.lowered != "erased") outs.push_back(o);
    if (a.op != "reducec" || component >= outs.size()) throw Unsupported("reducec: no such accumulator component");
    return compile(modules, "reducec[" + std::to_string(component) + "]", fold_inputs(a), outs[component].lowered,
                   [&](Builder& b, std::vector<Sym> args, uint32_t) {
                       Env env;
                       size_t k = 0;
                       for (const Operand& o : a.inputs)
                           if (!o.is_fn && o.lowered != "erased") env[o.name] = args[k++];
                       b.assign_in(env, a);
                       return env.at(outs[component].name);
                   });
}

// How a reducec over device buffers that matches no fold kernel runs.  `sequential`: one program per accumulator component
// (bit-exact for every `add`).  `staged`: when `add` is a prebuilt fold's (u64.add-env, f32.add-env, f32.max-env) the getter's
// values are materialised by `getter` (launched with the getter's environment) and folded by the prebuilt kernel `kind`.
struct FoldPlan {
    std::vector<Program> sequential;
    bool staged = false;
    Program getter;
    size_t get_env_begin = 0, get_env_size = 0;    // the getter's environment component among the assignment's inputs
    std::string kind;                              // "sum_u64", "sum_f32", "max_f32"
};
inline FoldPlan fold_plan_for(const std::vector<GpuModule>& modules, const GpuAssign& a) {
    FoldPlan plan;
    std::vector<Operand> outs;
    for (const Operand& o : a.outputs)
        if (o.lowered != "erased") outs.push_back(o);
    if (a.op != "reducec" || outs.empty()) throw Unsupported("not a reducec");
    for (size_t k = 0; k < outs.size(); ++k) plan.sequential.push_back(compile_fold(modules, a, k));
    if (outs.size() == 1 && a.input_sizes.size() == 6) {
        static const char* adds[][3] = {{"u64.add-env", "u64", "sum_u64"}, {"f32.add-env", "f32", "sum_f32"}, {"f32.max-env", "f32", "max_f32"}};
        for (auto& ad : adds) {
            bool has = false;
            for (const Operand& o : a.inputs) has = has || (o.is_fn && o.name == ad[0]);
            if (!has || outs[0].lowered != ad[1]) continue;
            const size_t begin = a.input_sizes[0] + a.input_sizes[1] + a.input_sizes[2];
            std::vector<Operand> get_env;
            for (size_t k = begin; k < begin + a.input_sizes[3]; ++k)
                if (!a.inputs[k].is_fn && a.inputs[k].lowered != "erased") get_env.push_back(a.inputs[k]);
            const Operand* get_fn = nullptr;
            for (size_t k = begin + a.input_sizes[3]; k < begin + a.input_sizes[3] + a.input_sizes[4]; ++k)
                if (a.inputs[k].is_fn) get_fn = &a.inputs[k];
            if (!get_fn) break;
            try {
                plan.getter = compile_producer(modules, get_fn->name, get_env, outs[0].lowered);
                plan.staged = true;
                plan.get_env_begin = begin;
                plan.get_env_size = a.input_sizes[3];
                plan.kind = ad[2];
            } catch (const Unsupported&) {
            }
            break;
        }
    }
    return plan;
}

// The register program of a `materializec` assignment: inputs `len, env..., producer` (input_sizes {1, n, 1} when given).
inline Program for_assignment(const std::vector<GpuModule>& modules, const GpuAssign& a) {
    if (a.op != "materializec" || a.outputs.size() != 1 || a.outputs[0].lowered.rfind("ptr<", 0) != 0 || a.inputs.size() < 2)
        throw Unsupported("not a materializec of one buffer");
    size_t env_begin = 1, env_end = a.inputs.size() - 1;
    if (!a.input_sizes.empty()) {
        if (a.input_sizes.size() != 3 || a.input_sizes[0] != 1) throw Unsupported("materializec expects the components len, env, producer");
        env_end = 1 + a.input_sizes[1];
    }
    std::vector<Operand> env_vars;
    for (size_t k = env_begin; k < env_end && k < a.inputs.size(); ++k)
        if (!a.inputs[k].is_fn && a.inputs[k].lowered != "erased") env_vars.push_back(a.inputs[k]);
    const Operand* fn = nullptr;
    for (size_t k = env_end; k < a.inputs.size(); ++k)
        if (a.inputs[k].is_fn) fn = &a.inputs[k];
    if (!fn) throw Unsupported("materializec needs one producer symbol");
    const std::string& l = a.outputs[0].lowered;
    return compile_producer(modules, fn->name, env_vars, l.substr(4, l.size() - 5));
}

}  // namespace map_program
}  // namespace catena_b200

#endif  // CATENA_B200_MAP_PROGRAM_HPP
