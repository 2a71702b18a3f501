// Compiled map: a register program (the instruction set of map_program.cu) turned into an sm_100a kernel of its own.
//
// The reference renders C++ for every `materializec` and runs nvcc when the Runtime is built
// (catena-lang/src/codegen/ops/materializec.rs:36-145, catena-lang/src/runtime/artifact.rs:59-80).  This file is the
// counterpart for producers no prebuilt kernel matches: it writes PTX for the register program — one to three PTX
// instructions per program instruction, every f32 operation with an explicit `.rn` (PTX never contracts an explicitly
// rounded mul and add into an fma, which is the reference's --fmad=false), constants as immediates — and hands the text to
// the driver's own PTX compiler (cuModuleLoadDataEx; no nvcc, no NVRTC, no source files).  The interpreter of map_program.cu
// stays as the cross-check: both give the same bits and report the same faults.
//
// Kernel shape: 256 threads, a CTA walks tiles of V x 256 consecutive elements (grid-stride over tiles); element
// tile * V * 256 + v * 256 + thread, so every load of `buffer[index]` and every store is one contiguous 128-byte line per
// warp.  V = 4 independent elements per thread for programs without jumps (the loads of all four are in flight together),
// V = 1 for programs with `bool.ifc` branches or `reducec` loops.  Register k of the program is a pair of 32-bit PTX
// registers (low, high half) per element, exactly the interpreter's split: 32-bit instructions write the low half only.
// Preset registers are shared by the four elements; constants of the program are immediates, environment values are kernel
// parameters.  With four elements per thread the f32 sums, differences, products and fmas of elements (0, 1) and (2, 3) are one
// packed f32x2 instruction each (packed_pair below): half the arithmetic instructions of a kernel that is bound by issue.
//
// Nothing a compiled program does can fault or hang the GPU, for the same reasons as in the interpreter: the program is
// validated first; loads are predicated on the bounds check; taken backward jumps are counted against the same budget; the
// cases the reference leaves undefined yield 0 and a code in the shared error word.
#include <cuda.h>
#include <stdarg.h>
#include <string.h>

#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

namespace catena {
namespace mapjit {

constexpr uint32_t kThreads = 256;
// A compiled program's registers are PTX virtual registers (the assembler allocates the real ones), so the file may be larger
// than the interpreter's 256, which sit in shared memory: programs with branches get no register reuse from the host compilers.
constexpr uint32_t kMaxRegs = 4096;
constexpr uint32_t kBackJumpBudget = 1u << 22;      // as map_program.cu
enum Err : uint32_t { ERR_ASSERT = 1, ERR_RANGE = 2, ERR_UNDEFINED = 3, ERR_BUDGET = 4 };

struct Spec {
    const catena_b200_map_insn_t* code;
    uint32_t n_insn;
    const uint64_t* init;
    const uint8_t* is_const;
    uint32_t n_init, n_regs, index_reg, result_reg, n_buffers, elem_bytes;
};

static bool straight_line(const Spec& s) {
    for (uint32_t k = 0; k < s.n_insn; ++k)
        if (s.code[k].op == CATENA_MAP_JMP || s.code[k].op == CATENA_MAP_JZ) return false;
    return true;
}

// ---- PTX text -------------------------------------------------------------------------------------------------------
struct Emitter {
    const Spec& s;
    uint32_t lanes;
    std::string out;
    std::vector<uint32_t> dyn;          // preset registers read from the kernel parameters, in parameter order

    explicit Emitter(const Spec& spec) : s(spec), lanes(straight_line(spec) ? 4 : 1) {
        for (uint32_t k = 0; k < s.n_init; ++k)
            if (!(s.is_const && s.is_const[k])) dyn.push_back(k);
    }

    void line(const char* fmt, ...) __attribute__((format(printf, 2, 3))) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof(buf), fmt, ap);
        va_end(ap);
        out += "    ";
        out += buf;
        out += "\n";
    }
    // names of the halves of program register k for element v
    std::string lo(uint32_t v, uint32_t k) const { return k < s.n_init ? "%lc_" + std::to_string(k) : "%l" + std::to_string(v) + "_" + std::to_string(k); }
    std::string hi(uint32_t v, uint32_t k) const { return k < s.n_init ? "%hc_" + std::to_string(k) : "%h" + std::to_string(v) + "_" + std::to_string(k); }

    // low half of register k when it is a constant of the program
    bool constant(uint32_t k, uint32_t* bits) const {
        if (k >= s.n_init || !s.is_const || !s.is_const[k]) return false;
        *bits = (uint32_t)s.init[k];
        return true;
    }

    void fault(const char* pred, uint32_t code) { line("@%s max.u32 %%fault, %%fault, %u;", pred, code); }

    void pack(const char* rd, uint32_t v, uint32_t k) { line("mov.b64 %s, {%s, %s};", rd, lo(v, k).c_str(), hi(v, k).c_str()); }
    void unpack(uint32_t v, uint32_t k, const char* rd) { line("mov.b64 {%s, %s}, %s;", lo(v, k).c_str(), hi(v, k).c_str(), rd); }

    void u64_binary(const char* ins, uint32_t v, const catena_b200_map_insn_t& in) {
        pack("%rd0", v, in.a);
        pack("%rd1", v, in.b);
        line("%s %%rd2, %%rd0, %%rd1;", ins);
        unpack(v, in.dst, "%rd2");
    }
    void u64_divide(const char* ins, uint32_t v, const catena_b200_map_insn_t& in) {
        pack("%rd0", v, in.a);
        pack("%rd1", v, in.b);
        line("setp.eq.u64 %%p1, %%rd1, 0;");
        line("selp.b64 %%rd1, 1, %%rd1, %%p1;");
        line("%s %%rd2, %%rd0, %%rd1;", ins);
        line("selp.b64 %%rd2, 0, %%rd2, %%p1;");
        fault("%p1", ERR_UNDEFINED);
        unpack(v, in.dst, "%rd2");
    }
    void u64_compare(const char* cmp, uint32_t v, const catena_b200_map_insn_t& in) {
        pack("%rd0", v, in.a);
        pack("%rd1", v, in.b);
        line("setp.%s.u64 %%p1, %%rd0, %%rd1;", cmp);
        line("selp.u32 %s, 1, 0, %%p1;", lo(v, in.dst).c_str());
    }
    void w_binary(const char* ins, uint32_t v, const catena_b200_map_insn_t& in) {
        line("%s %s, %s, %s;", ins, lo(v, in.dst).c_str(), lo(v, in.a).c_str(), lo(v, in.b).c_str());
    }
    void w_compare(const char* cmp, uint32_t v, const catena_b200_map_insn_t& in) {
        line("setp.%s %%p1, %s, %s;", cmp, lo(v, in.a).c_str(), lo(v, in.b).c_str());
        line("selp.u32 %s, 1, 0, %%p1;", lo(v, in.dst).c_str());
    }
    void shift(const char* ins, uint32_t v, const catena_b200_map_insn_t& in) {
        line("setp.lt.u32 %%p1, %s, 32;", lo(v, in.b).c_str());
        line("%s %%r0, %s, %s;", ins, lo(v, in.a).c_str(), lo(v, in.b).c_str());
        line("selp.b32 %s, %%r0, 0, %%p1;", lo(v, in.dst).c_str());
        fault("!%p1", ERR_UNDEFINED);
    }
    void mul_then(const char* ins, bool product_first, uint32_t v, const catena_b200_map_insn_t& in) {
        line("mul.rn.f32 %%r0, %s, %s;", lo(v, in.a).c_str(), lo(v, in.b).c_str());
        if (product_first) line("%s %s, %%r0, %s;", ins, lo(v, in.dst).c_str(), lo(v, in.c).c_str());
        else line("%s %s, %s, %%r0;", ins, lo(v, in.dst).c_str(), lo(v, in.c).c_str());
    }
    void load(bool wide, uint32_t v, const catena_b200_map_insn_t& in) {
        pack("%rd0", v, in.a);
        line("setp.lt.u64 %%p1, %%rd0, %%bn%u_%u;", wide ? 8 : 4, in.b);
        line("shl.b64 %%rd1, %%rd0, %u;", wide ? 3 : 2);
        line("add.u64 %%rd1, %%rd1, %%bb_%u;", in.b);
        if (wide) {
            line("mov.b64 %%rd2, 0;");
            line("@%%p1 ld.global.nc.b64 %%rd2, [%%rd1];");
            unpack(v, in.dst, "%rd2");
        } else {
            line("mov.b32 %%r0, 0;");
            line("@%%p1 ld.global.nc.b32 %%r0, [%%rd1];");
            line("mov.b32 %s, %%r0;", lo(v, in.dst).c_str());
        }
        fault("!%p1", ERR_RANGE);
    }

    // f32 arithmetic of elements v and v + 1 as ONE packed f32x2 instruction (sm_100): each half is the scalar instruction's
    // separately rounded IEEE operation.  A product is fma(a, b, -0) with the -0 from a kernel parameter: ptxas merges a packed mul
    // with the packed add or sub that consumes it into one fma, explicit .rn notwithstanding (measured: csrc/gemm_f32.cu), and an
    // fma whose addend it cannot see stays an fma; a * b + (-0) is exactly the rounded product.  Returns false for other opcodes.
    bool packed_pair(uint32_t k, uint32_t v) {
        const catena_b200_map_insn_t& in = s.code[k];
        auto pair = [&](const char* rd, uint32_t reg) { line("mov.b64 %s, {%s, %s};", rd, lo(v, reg).c_str(), lo(v + 1, reg).c_str()); };
        auto result = [&](const char* rd) { line("mov.b64 {%s, %s}, %s;", lo(v, in.dst).c_str(), lo(v + 1, in.dst).c_str(), rd); };
        switch (in.op) {
        case CATENA_MAP_F32_ADD:
        case CATENA_MAP_F32_SUB:
            pair("%rd0", in.a);
            pair("%rd1", in.b);
            line("%s.rn.f32x2 %%rd2, %%rd0, %%rd1;", in.op == CATENA_MAP_F32_ADD ? "add" : "sub");
            result("%rd2");
            return true;
        case CATENA_MAP_F32_MUL:
            pair("%rd0", in.a);
            pair("%rd1", in.b);
            line("fma.rn.f32x2 %%rd2, %%rd0, %%rd1, %%nz2;");
            result("%rd2");
            return true;
        case CATENA_MAP_F32_FMA:
            pair("%rd0", in.a);
            pair("%rd1", in.b);
            pair("%rd2", in.c);
            line("fma.rn.f32x2 %%rd3, %%rd0, %%rd1, %%rd2;");
            result("%rd3");
            return true;
        case CATENA_MAP_F32_MULADD:
        case CATENA_MAP_F32_MULSUB:
        case CATENA_MAP_F32_SUBMUL:
            pair("%rd0", in.a);
            pair("%rd1", in.b);
            pair("%rd2", in.c);
            line("fma.rn.f32x2 %%rd3, %%rd0, %%rd1, %%nz2;");
            if (in.op == CATENA_MAP_F32_MULADD) line("add.rn.f32x2 %%rd3, %%rd3, %%rd2;");
            else if (in.op == CATENA_MAP_F32_MULSUB) line("sub.rn.f32x2 %%rd3, %%rd3, %%rd2;");
            else line("sub.rn.f32x2 %%rd3, %%rd2, %%rd3;");
            result("%rd3");
            return true;
        default: return false;
        }
    }
    // In a whole tile the elements of a thread are index0 + e0 + v * 256: a load of buffer[index] needs ONE address (the others are
    // constant offsets from it) and ONE bounds test (the last element's, indices ascend).  When that test fails the elements
    // are tested one by one, as everywhere else.  %idx0 holds index0 + e0.
    bool whole_tile = false;
    uint32_t tile_loads = 0;
    bool tile_load(uint32_t k) {
        const catena_b200_map_insn_t& in = s.code[k];
        const bool wide = in.op == CATENA_MAP_LOAD_U64;
        if (!whole_tile || (!wide && in.op != CATENA_MAP_LOAD_F32) || in.a != s.index_reg) return false;
        const uint32_t bytes = wide ? 8 : 4, id = tile_loads++;
        line("add.u64 %%rd0, %%idx0, %u;", (lanes - 1) * kThreads);
        line("setp.lt.u64 %%p1, %%rd0, %%bn%u_%u;", bytes, in.b);
        line("@!%%p1 bra TL_EACH_%u;", id);
        line("mad.lo.u64 %%rd1, %%idx0, %u, %%bb_%u;", bytes, in.b);
        for (uint32_t v = 0; v < lanes; ++v) {
            if (wide) {
                line("ld.global.nc.b64 %%rd2, [%%rd1+%u];", v * kThreads * bytes);
                unpack(v, in.dst, "%rd2");
            } else {
                line("ld.global.nc.b32 %s, [%%rd1+%u];", lo(v, in.dst).c_str(), v * kThreads * bytes);
            }
        }
        line("bra TL_DONE_%u;", id);
        out += "TL_EACH_" + std::to_string(id) + ":\n";
        for (uint32_t v = 0; v < lanes; ++v) load(wide, v, in);
        out += "TL_DONE_" + std::to_string(id) + ":\n";
        return true;
    }
    // instruction k for all elements of the thread
    void instruction_all(uint32_t k) {
        if (tile_load(k)) return;
        for (uint32_t v = 0; v < lanes; ++v) {
            if (v + 1 < lanes && packed_pair(k, v)) ++v;
            else instruction(k, v);
        }
    }

    // one program instruction for element v; `k` is its index (jump bookkeeping)
    void instruction(uint32_t k, uint32_t v) {
        const catena_b200_map_insn_t& in = s.code[k];
        const std::string d = lo(v, in.dst), a = lo(v, in.a), b = lo(v, in.b), c = lo(v, in.c);
        switch (in.op) {
        case CATENA_MAP_HALT: line("bra STORE;"); break;
        case CATENA_MAP_JMP:
        case CATENA_MAP_JZ:
            if (in.op == CATENA_MAP_JZ) {
                line("setp.ne.u32 %%p1, %s, 0;", a.c_str());
                line("@%%p1 bra SKIP_%u;", k);
            }
            if (in.target <= k) {           // a taken backward jump counts against the budget
                line("add.u32 %%back, %%back, 1;");
                line("setp.gt.u32 %%p2, %%back, %u;", kBackJumpBudget);
                line("@%%p2 bra GIVE_UP;");
            }
            line("bra L_%u;", in.target);
            if (in.op == CATENA_MAP_JZ) out += "SKIP_" + std::to_string(k) + ":\n";
            break;
        case CATENA_MAP_ASSERT:
            line("setp.eq.u32 %%p1, %s, 0;", a.c_str());
            fault("%p1", ERR_ASSERT);
            break;
        case CATENA_MAP_MOV:
            line("mov.b32 %%r0, %s;", hi(v, in.a).c_str());
            line("mov.b32 %s, %s;", d.c_str(), a.c_str());
            line("mov.b32 %s, %%r0;", hi(v, in.dst).c_str());
            break;
        case CATENA_MAP_MOV32: line("mov.b32 %s, %s;", d.c_str(), a.c_str()); break;
        case CATENA_MAP_SELECT:
            line("setp.ne.u32 %%p1, %s, 0;", a.c_str());
            line("selp.b32 %%r0, %s, %s, %%p1;", b.c_str(), c.c_str());
            line("selp.b32 %%r1, %s, %s, %%p1;", hi(v, in.b).c_str(), hi(v, in.c).c_str());
            line("mov.b32 %s, %%r0;", d.c_str());
            line("mov.b32 %s, %%r1;", hi(v, in.dst).c_str());
            break;
        case CATENA_MAP_SELECT32:
            line("setp.ne.u32 %%p1, %s, 0;", a.c_str());
            line("selp.b32 %s, %s, %s, %%p1;", d.c_str(), b.c_str(), c.c_str());
            break;
        case CATENA_MAP_BOOL_NOT:
            line("setp.eq.u32 %%p1, %s, 0;", a.c_str());
            line("selp.u32 %s, 1, 0, %%p1;", d.c_str());
            break;
        case CATENA_MAP_BOOL_AND:
        case CATENA_MAP_BOOL_OR:
            line("setp.ne.u32 %%p1, %s, 0;", a.c_str());
            line("setp.ne.u32 %%p2, %s, 0;", b.c_str());
            line("%s.pred %%p1, %%p1, %%p2;", in.op == CATENA_MAP_BOOL_AND ? "and" : "or");
            line("selp.u32 %s, 1, 0, %%p1;", d.c_str());
            break;
        case CATENA_MAP_U64_ADD: u64_binary("add.u64", v, in); break;
        case CATENA_MAP_U64_SUB: u64_binary("sub.u64", v, in); break;
        case CATENA_MAP_U64_MUL: u64_binary("mul.lo.u64", v, in); break;
        case CATENA_MAP_U64_DIV: u64_divide("div.u64", v, in); break;
        case CATENA_MAP_U64_REM: u64_divide("rem.u64", v, in); break;
        case CATENA_MAP_U64_EQ: u64_compare("eq", v, in); break;
        case CATENA_MAP_U64_NE: u64_compare("ne", v, in); break;
        case CATENA_MAP_U64_LT: u64_compare("lt", v, in); break;
        case CATENA_MAP_U64_LTE: u64_compare("le", v, in); break;
        case CATENA_MAP_U64_GT: u64_compare("gt", v, in); break;
        case CATENA_MAP_U64_GTE: u64_compare("ge", v, in); break;
        case CATENA_MAP_U64_TO_F32:
            pack("%rd0", v, in.a);
            line("cvt.rn.f32.u64 %s, %%rd0;", d.c_str());
            break;
        case CATENA_MAP_U32_ADD: w_binary("add.u32", v, in); break;
        case CATENA_MAP_U32_SUB: w_binary("sub.u32", v, in); break;
        case CATENA_MAP_U32_MUL: w_binary("mul.lo.u32", v, in); break;
        case CATENA_MAP_U32_AND: w_binary("and.b32", v, in); break;
        case CATENA_MAP_U32_OR: w_binary("or.b32", v, in); break;
        case CATENA_MAP_U32_XOR: w_binary("xor.b32", v, in); break;
        case CATENA_MAP_U32_NOT: line("not.b32 %s, %s;", d.c_str(), a.c_str()); break;
        case CATENA_MAP_U32_SHL: shift("shl.b32", v, in); break;
        case CATENA_MAP_U32_SHR: shift("shr.u32", v, in); break;
        case CATENA_MAP_U32_EQ: w_compare("eq.u32", v, in); break;
        case CATENA_MAP_U32_NE: w_compare("ne.u32", v, in); break;
        case CATENA_MAP_U32_LT: w_compare("lt.u32", v, in); break;
        case CATENA_MAP_U32_LTE: w_compare("le.u32", v, in); break;
        case CATENA_MAP_U32_GT: w_compare("gt.u32", v, in); break;
        case CATENA_MAP_U32_GTE: w_compare("ge.u32", v, in); break;
        case CATENA_MAP_U32_TO_F32: line("cvt.rn.f32.u32 %s, %s;", d.c_str(), a.c_str()); break;
        case CATENA_MAP_F32_ADD: w_binary("add.rn.f32", v, in); break;
        case CATENA_MAP_F32_SUB: w_binary("sub.rn.f32", v, in); break;
        case CATENA_MAP_F32_MUL: w_binary("mul.rn.f32", v, in); break;
        case CATENA_MAP_F32_DIV: {
            // two quotients that cost less and are the same IEEE result: 1 / x is the correctly rounded reciprocal, and x / 2^k
            // is x * 2^-k (one rounding of the same real number) while 2^-k is a normal number
            uint32_t num = 0, den = 0;
            if (constant(in.a, &num) && num == 0x3F800000u) {
                line("rcp.rn.f32 %s, %s;", d.c_str(), b.c_str());
            } else if (constant(in.b, &den) && (den & 0x007FFFFFu) == 0 && ((den >> 23) & 0xFFu) >= 1 && ((den >> 23) & 0xFFu) <= 253) {
                const uint32_t inverse = (den & 0x80000000u) | ((254u - ((den >> 23) & 0xFFu)) << 23);
                line("mul.rn.f32 %s, %s, 0f%08X;", d.c_str(), a.c_str(), inverse);
            } else {
                w_binary("div.rn.f32", v, in);
            }
            break;
        }
        case CATENA_MAP_F32_NEG: line("xor.b32 %s, %s, 0x80000000;", d.c_str(), a.c_str()); break;
        case CATENA_MAP_F32_FMA: line("fma.rn.f32 %s, %s, %s, %s;", d.c_str(), a.c_str(), b.c_str(), c.c_str()); break;
        case CATENA_MAP_F32_MULADD: mul_then("add.rn.f32", true, v, in); break;
        case CATENA_MAP_F32_MULSUB: mul_then("sub.rn.f32", true, v, in); break;
        case CATENA_MAP_F32_SUBMUL: mul_then("sub.rn.f32", false, v, in); break;
        // C comparisons: == < <= > >= are false on a NaN (ordered), != is true (unordered or not equal)
        case CATENA_MAP_F32_EQ: w_compare("eq.f32", v, in); break;
        case CATENA_MAP_F32_NE: w_compare("neu.f32", v, in); break;
        case CATENA_MAP_F32_LT: w_compare("lt.f32", v, in); break;
        case CATENA_MAP_F32_LTE: w_compare("le.f32", v, in); break;
        case CATENA_MAP_F32_GT: w_compare("gt.f32", v, in); break;
        case CATENA_MAP_F32_GTE: w_compare("ge.f32", v, in); break;
        case CATENA_MAP_F32_ROUND_TO_U32:
            line("setp.ge.f32 %%p1, %s, 0f00000000;", a.c_str());
            line("setp.lt.f32 %%p2, %s, 0f4F800000;", a.c_str());
            line("and.pred %%p1, %%p1, %%p2;");
            line("cvt.rni.u32.f32 %%r0, %s;", a.c_str());
            line("selp.b32 %s, %%r0, 0, %%p1;", d.c_str());
            fault("!%p1", ERR_UNDEFINED);
            break;
        case CATENA_MAP_LOAD_U64: load(true, v, in); break;
        case CATENA_MAP_LOAD_F32: load(false, v, in); break;
        default: break;          // unreachable: validated
        }
    }

    void emit() {
        const uint32_t nd = (uint32_t)dyn.size(), nb = s.n_buffers;
        out += "// generated by catena-b200 (map_jit.cu) from a register program of " + std::to_string(s.n_insn) + " instructions\n";
        out += ".version 8.6\n.target sm_100a\n.address_size 64\n\n";
        out += ".visible .entry catena_map_kernel(\n";
        line(".param .align 8 .b8 p_init[%u],", 8 * (nd ? nd : 1));
        line(".param .align 8 .b8 p_bufs[%u],", 16 * (nb ? nb : 1));
        line(".param .u64 p_out,");
        line(".param .u64 p_index0,");
        line(".param .u64 p_len,");
        line(".param .u64 p_err,");
        line(".param .u64 p_nz2)");
        out += ".reqntid " + std::to_string(kThreads) + ", 1, 1\n{\n";
        if (s.n_init) line(".reg .b32 %%lc_<%u>, %%hc_<%u>;", s.n_init, s.n_init);
        for (uint32_t v = 0; v < lanes; ++v) {
            line(".reg .b32 %%l%u_<%u>, %%h%u_<%u>;", v, s.n_regs, v, s.n_regs);
            line(".reg .b64 %%e%u;", v);
            line(".reg .pred %%ok%u;", v);
        }
        if (nb) line(".reg .b64 %%bb_<%u>, %%bn8_<%u>, %%bn4_<%u>;", nb, nb, nb);
        line(".reg .b64 %%rd<4>, %%out, %%index0, %%len, %%err, %%tile, %%tiles, %%step, %%tid64, %%nz2, %%idx0;");
        line(".reg .b32 %%r<4>, %%fault, %%back, %%gave;");
        line(".reg .pred %%p<4>;");
        out += "\n";
        line("ld.param.u64 %%out, [p_out];");
        line("cvta.to.global.u64 %%out, %%out;");
        line("ld.param.u64 %%err, [p_err];");
        line("cvta.to.global.u64 %%err, %%err;");
        line("ld.param.u64 %%index0, [p_index0];");
        line("ld.param.u64 %%nz2, [p_nz2];");
        line("ld.param.u64 %%len, [p_len];");
        for (uint32_t j = 0; j < nb; ++j) {
            line("ld.param.u64 %%bb_%u, [p_bufs+%u];", j, 16 * j);
            line("cvta.to.global.u64 %%bb_%u, %%bb_%u;", j, j);
            line("ld.param.u64 %%rd0, [p_bufs+%u];", 16 * j + 8);
            line("shr.u64 %%bn8_%u, %%rd0, 3;", j);
            line("shr.u64 %%bn4_%u, %%rd0, 2;", j);
        }
        uint32_t slot = 0;
        for (uint32_t k = 0; k < s.n_init; ++k) {
            if (s.is_const && s.is_const[k]) {
                line("mov.b32 %%lc_%u, 0x%08X;", k, (uint32_t)s.init[k]);
                line("mov.b32 %%hc_%u, 0x%08X;", k, (uint32_t)(s.init[k] >> 32));
            } else {
                line("ld.param.b32 %%lc_%u, [p_init+%u];", k, 8 * slot);
                line("ld.param.b32 %%hc_%u, [p_init+%u];", k, 8 * slot + 4);
                ++slot;
            }
        }
        // registers the program reads before it writes them are zero, as the interpreter's file is
        for (uint32_t v = 0; v < lanes; ++v)
            for (uint32_t k = s.n_init; k < s.n_regs; ++k) {
                line("mov.b32 %s, 0;", lo(v, k).c_str());
                line("mov.b32 %s, 0;", hi(v, k).c_str());
            }
        const uint32_t per_tile = lanes * kThreads;
        line("mov.b32 %%fault, 0;");
        line("mov.b32 %%r0, %%tid.x;");
        line("cvt.u64.u32 %%tid64, %%r0;");
        line("mov.b32 %%r0, %%ctaid.x;");
        line("cvt.u64.u32 %%tile, %%r0;");
        line("mov.b32 %%r0, %%nctaid.x;");
        line("cvt.u64.u32 %%step, %%r0;");
        line("add.u64 %%tiles, %%len, %u;", per_tile - 1);
        line("shr.u64 %%tiles, %%tiles, %u;", lanes == 4 ? 10 : 8);
        out += "TILE:\n";
        line("setp.ge.u64 %%p0, %%tile, %%tiles;");
        line("@%%p0 bra DONE;");
        // element v of this thread: tile * per_tile + v * 256 + thread
        line("mad.lo.u64 %%e0, %%tile, %u, %%tid64;", per_tile);
        // Straight-line programs are written twice: for a tile that lies wholly inside the range — no element needs a validity
        // test, the four indices are one sum plus constants, the stores are unconditional — and for the ragged last tile.
        const bool split = lanes > 1 && (uint64_t)s.n_insn * lanes <= 1024;
        if (split) {
            line("add.u64 %%rd0, %%tile, 1;");
            line("mul.lo.u64 %%rd0, %%rd0, %u;", per_tile);
            line("setp.gt.u64 %%p0, %%rd0, %%len;");
            line("@%%p0 bra RAGGED;");
            line("add.u64 %%idx0, %%e0, %%index0;");
            for (uint32_t v = 0; v < lanes; ++v) {
                if (v) line("add.u64 %%rd1, %%idx0, %u;", v * kThreads);
                unpack(v, s.index_reg, v ? "%rd1" : "%idx0");
            }
            whole_tile = true;
            for (uint32_t k = 0; k < s.n_insn && s.code[k].op != CATENA_MAP_HALT; ++k)
                instruction_all(k);
            whole_tile = false;
            line("mad.lo.u64 %%rd0, %%e0, %u, %%out;", s.elem_bytes);        // one address, constant offsets
            for (uint32_t v = 0; v < lanes; ++v) {
                if (s.elem_bytes == 8) {
                    line("mov.b64 %%rd1, {%s, %s};", lo(v, s.result_reg).c_str(), hi(v, s.result_reg).c_str());
                    line("st.global.b64 [%%rd0+%u], %%rd1;", v * kThreads * 8);
                } else {
                    line("st.global.b32 [%%rd0+%u], %s;", v * kThreads * 4, lo(v, s.result_reg).c_str());
                }
            }
            line("bra NEXT;");
            out += "RAGGED:\n";
        }
        // a thread whose first element is past the end has none
        line("setp.lt.u64 %%ok0, %%e0, %%len;");
        line("@!%%ok0 bra NEXT;");
        for (uint32_t v = 1; v < lanes; ++v) {
            line("add.u64 %%e%u, %%e0, %u;", v, v * kThreads);
            line("setp.lt.u64 %%ok%u, %%e%u, %%len;", v, v);
        }
        for (uint32_t v = 0; v < lanes; ++v) {
            // an element past the end repeats element 0 of the thread (valid) and is not stored
            if (v) line("selp.b64 %%rd0, %%e%u, %%e0, %%ok%u;", v, v);
            else line("mov.b64 %%rd0, %%e0;");
            line("add.u64 %%rd0, %%rd0, %%index0;");
            unpack(v, s.index_reg, "%rd0");
        }
        line("mov.b32 %%back, 0;");
        line("mov.b32 %%gave, 0;");
        // jump targets get labels
        std::vector<bool> target(s.n_insn + 1, false);
        for (uint32_t k = 0; k < s.n_insn; ++k)
            if (s.code[k].op == CATENA_MAP_JMP || s.code[k].op == CATENA_MAP_JZ) target[s.code[k].target] = true;
        for (uint32_t k = 0; k < s.n_insn; ++k) {
            if (target[k]) out += "L_" + std::to_string(k) + ":\n";
            if (lanes > 1 && s.code[k].op == CATENA_MAP_HALT) break;       // straight line: the first HALT ends the element
            instruction_all(k);
        }
        line("bra STORE;");
        out += "GIVE_UP:\n";
        line("max.u32 %%fault, %%fault, %u;", ERR_BUDGET);
        line("mov.b32 %%gave, 1;");
        out += "STORE:\n";
        line("setp.ne.u32 %%p1, %%gave, 0;");
        for (uint32_t v = 0; v < lanes; ++v) {
            line("selp.b32 %%r0, 0, %s, %%p1;", lo(v, s.result_reg).c_str());
            if (s.elem_bytes == 8) {
                line("selp.b32 %%r1, 0, %s, %%p1;", hi(v, s.result_reg).c_str());
                line("mov.b64 %%rd1, {%%r0, %%r1};");
                line("mad.lo.u64 %%rd0, %%e%u, 8, %%out;", v);
                line("@%%ok%u st.global.b64 [%%rd0], %%rd1;", v);
            } else {
                line("mad.lo.u64 %%rd0, %%e%u, 4, %%out;", v);
                line("@%%ok%u st.global.b32 [%%rd0], %%r0;", v);
            }
        }
        out += "NEXT:\n";
        line("add.u64 %%tile, %%tile, %%step;");
        line("bra TILE;");
        out += "DONE:\n";
        line("setp.ne.u32 %%p1, %%fault, 0;");
        line("@%%p1 red.global.max.u32 [%%err], %%fault;");
        line("ret;");
        out += "}\n";
    }
};

static catena_status_t check_spec(const Spec& s) {
    if (s.elem_bytes != 4 && s.elem_bytes != 8) return fail(CATENA_E_BAD_ARG, "map kernel: elements of 4 or 8 bytes");
    if (s.n_init && !s.init) return fail(CATENA_E_BAD_ARG, "map kernel: null argument");
    CATENA_TRY(map_program_validate(s.code, s.n_insn, s.n_init, s.n_regs, s.index_reg, s.result_reg, s.n_buffers, kMaxRegs));
    uint32_t dynamic = 0;
    for (uint32_t k = 0; k < s.n_init; ++k) dynamic += !(s.is_const && s.is_const[k]);
    if (dynamic > 256) return fail(CATENA_E_TOO_LARGE, "map kernel: more than 256 environment presets (they travel as kernel parameters)");
    return CATENA_OK;
}

// ---- driver entry points (looked up through the runtime: the library does not link libcuda) -------------------------
struct Driver {
    CUresult (*module_load)(CUmodule*, const void*, unsigned int, CUjit_option*, void**) = nullptr;
    CUresult (*module_unload)(CUmodule) = nullptr;
    CUresult (*module_function)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*launch)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void**, void**) = nullptr;
    CUresult (*occupancy)(int*, CUfunction, int, size_t) = nullptr;
    bool ok = false;
};

static const Driver& driver() {
    static Driver d;
    static std::once_flag once;
    std::call_once(once, [] {
        auto get = [](const char* name, void** fn) {
            cudaDriverEntryPointQueryResult r;
            return cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &r) == cudaSuccess && r == cudaDriverEntryPointSuccess && *fn;
        };
        d.ok = get("cuModuleLoadDataEx", (void**)&d.module_load) && get("cuModuleUnload", (void**)&d.module_unload) &&
               get("cuModuleGetFunction", (void**)&d.module_function) && get("cuLaunchKernel", (void**)&d.launch) &&
               get("cuOccupancyMaxActiveBlocksPerMultiprocessor", (void**)&d.occupancy);
    });
    return d;
}

}  // namespace mapjit
}  // namespace catena

using namespace catena;

struct catena_b200_map_kernel {
    int device;
    CUmodule module;
    CUfunction function;
    uint32_t lanes, n_init, n_buffers, elem_bytes, ctas_per_sm;
    std::vector<uint32_t> dyn;
};

extern "C" {

catena_status_t catena_b200_map_ptx_s(const catena_b200_map_insn_t* code, uint32_t n_insn, const uint64_t* init, const uint8_t* init_is_const,
                                      uint32_t n_init, uint32_t n_regs, uint32_t index_reg, uint32_t result_reg, uint32_t n_buffers,
                                      uint32_t elem_bytes, char* text, uint64_t capacity, uint64_t* length) {
    const mapjit::Spec spec = {code, n_insn, init, init_is_const, n_init, n_regs, index_reg, result_reg, n_buffers, elem_bytes};
    CATENA_TRY(mapjit::check_spec(spec));
    mapjit::Emitter em(spec);
    em.emit();
    if (length) *length = em.out.size() + 1;
    if (text && capacity) {
        const size_t n = em.out.size() + 1 <= capacity ? em.out.size() : (size_t)capacity - 1;
        memcpy(text, em.out.data(), n);
        text[n] = 0;
        if (n < em.out.size()) return fail(CATENA_E_TOO_LARGE, "map kernel: the text does not fit the buffer");
    }
    return CATENA_OK;
}

catena_status_t catena_b200_map_compile_s(const catena_b200_map_insn_t* code, uint32_t n_insn, const uint64_t* init, const uint8_t* init_is_const,
                                          uint32_t n_init, uint32_t n_regs, uint32_t index_reg, uint32_t result_reg, uint32_t n_buffers,
                                          uint32_t elem_bytes, catena_b200_map_kernel_t** kernel) {
    if (!kernel) return fail(CATENA_E_BAD_ARG, "map kernel: null output pointer");
    *kernel = nullptr;
    const mapjit::Spec spec = {code, n_insn, init, init_is_const, n_init, n_regs, index_reg, result_reg, n_buffers, elem_bytes};
    CATENA_TRY(mapjit::check_spec(spec));
    CATENA_TRY(ensure_device());
    const mapjit::Driver& drv = mapjit::driver();
    if (!drv.ok) return fail(CATENA_E_CUDA, "map kernel: the driver's module entry points are not available");
    mapjit::Emitter em(spec);
    em.emit();
    char log[2048];
    log[0] = 0;
    CUjit_option opts[2] = {CU_JIT_ERROR_LOG_BUFFER, CU_JIT_ERROR_LOG_BUFFER_SIZE_BYTES};
    void* vals[2] = {log, (void*)(uintptr_t)sizeof(log)};
    CUmodule mod = nullptr;
    if (drv.module_load(&mod, em.out.c_str(), 2, opts, vals) != CUDA_SUCCESS) {
        fprintf(stderr, "catena-b200: PTX of a map kernel rejected by the driver: %s\n", log);
        return fail(CATENA_E_CUDA, "map kernel: the driver rejected the generated PTX");
    }
    CUfunction fn = nullptr;
    if (drv.module_function(&fn, mod, "catena_map_kernel") != CUDA_SUCCESS) {
        drv.module_unload(mod);
        return fail(CATENA_E_CUDA, "map kernel: entry not found in the compiled module");
    }
    int per_sm = 0;
    if (drv.occupancy(&per_sm, fn, (int)mapjit::kThreads, 0) != CUDA_SUCCESS || per_sm < 1) per_sm = 1;
    catena_b200_map_kernel* k = new catena_b200_map_kernel();
    k->device = tls().device;
    k->module = mod;
    k->function = fn;
    k->lanes = em.lanes;
    k->n_init = n_init;
    k->n_buffers = n_buffers;
    k->elem_bytes = elem_bytes;
    k->ctas_per_sm = (uint32_t)per_sm;
    k->dyn = em.dyn;
    *kernel = k;
    return CATENA_OK;
}

catena_status_t catena_b200_map_kernel_launch_s(const catena_b200_map_kernel_t* kernel, const uint64_t* init, uint32_t n_init,
                                                const catena_mem_t* buffers, uint32_t n_buffers, uint64_t index0, uint64_t len,
                                                catena_mem_t* out) {
    if (!out) return fail(CATENA_E_BAD_ARG, "map kernel: null output pointer");
    out->data = nullptr;
    out->len = 0;
    if (!kernel) return fail(CATENA_E_BAD_ARG, "map kernel: null kernel");
    if (n_init != kernel->n_init || n_buffers != kernel->n_buffers || (n_init && !init) || (n_buffers && !buffers))
        return fail(CATENA_E_BAD_ARG, "map kernel: presets or buffers do not match the compiled program");
    uint64_t bufs[2 * 16] = {0};
    for (uint32_t k = 0; k < n_buffers; ++k) {
        if (buffers[k].len != 0 && !buffers[k].data) return fail(CATENA_E_BAD_ARG, "map kernel: null buffer");
        if ((uintptr_t)buffers[k].data & 7) return fail(CATENA_E_BAD_ARG, "map kernel: buffers must be 8-byte aligned");
        bufs[2 * k] = (uint64_t)(uintptr_t)buffers[k].data;
        bufs[2 * k + 1] = buffers[k].len;
    }
    if (len > (~0ull) / kernel->elem_bytes || index0 > ~0ull - len) return fail(CATENA_E_TOO_LARGE, "map kernel: length overflows");
    CATENA_TRY(ensure_device());
    if (tls().device != kernel->device) return fail(CATENA_E_BAD_ARG, "map kernel: compiled for another device");
    if (len == 0) return CATENA_OK;
    uint32_t* err = nullptr;
    CATENA_TRY(map_program_error_word(&err));
    std::vector<uint64_t> dyn(kernel->dyn.size() ? kernel->dyn.size() : 1, 0);
    for (size_t j = 0; j < kernel->dyn.size(); ++j) dyn[j] = init[kernel->dyn[j]];
    void* result = nullptr;
    CATENA_TRY(pool_alloc(len * kernel->elem_bytes, &result));
    const int sms = tls().sm_count > 0 ? tls().sm_count : 148;
    uint64_t blocks = ceil_div_u64(len, (uint64_t)mapjit::kThreads * kernel->lanes);
    if (blocks > (uint64_t)sms * kernel->ctas_per_sm) blocks = (uint64_t)sms * kernel->ctas_per_sm;
    uint64_t out_ptr = (uint64_t)(uintptr_t)result, err_ptr = (uint64_t)(uintptr_t)err;
    uint64_t neg_zero2 = 0x8000000080000000ull;        // two packed -0.0f: the addend that makes a packed fma a rounded product
    void* params[7] = {dyn.data(), bufs, &out_ptr, &index0, &len, &err_ptr, &neg_zero2};
    const CUresult r = mapjit::driver().launch(kernel->function, (unsigned)blocks, 1, 1, mapjit::kThreads, 1, 1, 0, (CUstream)tls().stream, params, nullptr);
    count_launch();
    catena_status_t s = CATENA_OK;
    if (r != CUDA_SUCCESS) s = fail(CATENA_E_CUDA, "map kernel: launch failed");
    if (s == CATENA_OK && tls().blocking) s = map_program_check_errors();
    if (s != CATENA_OK) {
        pool_free(result);
        return s;
    }
    out->data = result;
    out->len = len * kernel->elem_bytes;
    return CATENA_OK;
}

void catena_b200_map_kernel_release(catena_b200_map_kernel_t* kernel) {
    if (!kernel) return;
    if (mapjit::driver().ok && kernel->module) {
        // launches of the kernel may still be queued (non-blocking mode): the module goes only once its device is idle
        int current = -1;
        if (cudaGetDevice(&current) == cudaSuccess && cudaSetDevice(kernel->device) == cudaSuccess) {
            (void)cudaDeviceSynchronize();
            mapjit::driver().module_unload(kernel->module);
            if (current >= 0 && current != kernel->device) (void)cudaSetDevice(current);
        }
        (void)cudaGetLastError();
    }
    delete kernel;
}

}  // extern "C"
