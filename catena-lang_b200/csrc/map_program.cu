// Generic map kernel: out[i] = producer(env..., i) for a producer that no prebuilt kernel matches.
//
// The reference renders one kernel per `materializec` — `uint64_t i = blockIdx.x * blockDim.x + threadIdx.x; if (i >= len)
// return; T value; program_producer(env..., i, &value); out[i] = value;` — and compiles it with nvcc when the Runtime is
// built (catena-lang/src/codegen/ops/materializec.rs:36-82, host wrapper :84-145).  A backend that selects prebuilt kernels
// has no compiler at run time, so the producer arrives as a REGISTER PROGRAM — the producer's scalar assignments, calls
// inlined, one instruction per primitive of the table catena-lang/src/codegen/gpu.rs:322-447 — and this kernel interprets it
// for every index.  All threads run the same instruction stream (it lives in shared memory), so the interpreter's
// dispatch does not diverge; only `bool.ifc` branches and `reducec` loops of the program itself can.
//
// Values are 64-bit registers: bool as 0 / 1, u32 and the bit pattern of an f32 in the low half, u64 as is, so the bitcasts are
// moves.  f32 arithmetic goes through the explicitly rounded operations of catena_math.cuh (never contracted),
// `f32.fma` is one fused operation, `f32.round-to-u32` rounds to nearest even, `u64.to-f32` / `u32.to-f32` round once.
//
// Nothing a program does can fault or hang the GPU: the host checks every register number, buffer number and jump target
// before the launch; loads are bounds-checked against the buffer's length; backward jumps are counted against a budget.
// Where the reference's generated C would trap (`catena_assert`), read past a buffer or be undefined (a u32 shift by 32 or
// more, `f32.round-to-u32` outside [0, 2^32), a row-major division by zero columns) the element yields 0, the launch carries on
// and the entry point reports CATENA_E_ASSERT.
#include <string.h>

#include "catena_math.cuh"
#include "common.cuh"

namespace catena {

namespace mapvm {

constexpr uint32_t kMaxInsns = 2048;          // 32 KiB of shared memory
constexpr uint32_t kMaxRegs = 256;
constexpr uint32_t kMaxBuffers = 16;
constexpr uint32_t kBackJumpBudget = 1u << 22;   // taken backward jumps per element before the element is given up

enum Err : uint32_t { ERR_NONE = 0, ERR_ASSERT = 1, ERR_RANGE = 2, ERR_UNDEFINED = 3, ERR_BUDGET = 4 };

struct Buffers {
    const uint8_t* base[kMaxBuffers];
    uint64_t bytes[kMaxBuffers];
};

__device__ __forceinline__ float as_f32(uint64_t r) { return __uint_as_float((uint32_t)r); }
__device__ __forceinline__ uint64_t from_f32(float f) { return (uint64_t)__float_as_uint(f); }

// Small programs travel as kernel parameters (no copy, no scratch, and the constant cache broadcasts an instruction to the
// warp); larger ones are copied to the device and staged in shared memory.
#ifndef CATENA_MAP_PARAM_INSNS
#define CATENA_MAP_PARAM_INSNS 192
#endif
constexpr uint32_t kParamInsns = CATENA_MAP_PARAM_INSNS, kParamInit = 48;
struct ParamProgram {
    uint4 code[kParamInsns];
    uint64_t init[kParamInit];
};

// The register file.  Low halves: shared memory, [register][thread][lane] (conflict-free, and unlike a local-memory array it
// cannot be evicted: with the file in local memory an SM's resident threads touched several times the L1 and the spill to L2
// and HBM cost ten times the algorithmic traffic).  High halves: a local-memory array — bool / u32 / f32 instructions never
// touch them, so a program without u64 arithmetic uses them for the index only.  The high half of a register that holds a
// 32-bit value is stale; nothing reads it: flags are tested on the low half, and the type system never feeds a 32-bit value
// to a u64 instruction (the primitive table has no u32 -> u64 conversion).
// REGS: capacity of the high-half file.  V: elements a thread carries through the program in lockstep — one fetch, decode
// and dispatch per V elements; V > 1 only for programs without jumps (the host decides).  PARAM: the program sits in the
// kernel parameters instead of shared memory.  T: threads per CTA.
template <int REGS, int V, bool PARAM, int T>
__global__ void __launch_bounds__(T) map_program_kernel(const __grid_constant__ ParamProgram prm, const uint4* __restrict__ code,
                                                          uint32_t n_insn, const uint64_t* __restrict__ init, uint32_t n_init, uint32_t n_regs,
                                                          uint32_t index_reg, uint32_t result_reg, const __grid_constant__ Buffers bufs,
                                                          void* __restrict__ out, uint32_t elem_bytes, uint64_t index0, uint64_t len, uint32_t* err) {
    extern __shared__ uint4 s_dyn[];
    const uint4* s_code = s_dyn;
    // low halves: the V lanes of a register sit side by side, [register][thread][lane], so that one 16-byte access moves all
    // four (a warp's access is 512 contiguous bytes: four conflict-free wavefronts)
    uint32_t* s_lo = reinterpret_cast<uint32_t*>(s_dyn + (PARAM ? 0 : n_insn)) + threadIdx.x * V;
    if (!PARAM) {
        for (uint32_t k = threadIdx.x; k < n_insn; k += T) s_dyn[k] = code[k];
        __syncthreads();
    }
#define lo(R, v) s_lo[(R) * (V * T) + (v)]
    uint32_t hi[REGS][V];
#pragma unroll 1
    for (uint32_t k = 0; k < n_regs; ++k) {
        const uint64_t x = k < n_init ? (PARAM ? prm.init[k] : init[k]) : 0ull;
#pragma unroll
        for (int v = 0; v < V; ++v) {
            lo(k, v) = (uint32_t)x;
            hi[k][v] = (uint32_t)(x >> 32);
        }
    }
    uint32_t fault = ERR_NONE;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += stride * V) {
        // element v of this trip is i + v * stride; past the end it repeats element i (valid), and is not stored
#pragma unroll
        for (int v = 0; v < V; ++v) {
            const uint64_t e = index0 + (i + v * stride < len ? i + v * stride : i);     // out[j] is element index0 + j
            lo(index_reg, v) = (uint32_t)e;
            hi[index_reg][v] = (uint32_t)(e >> 32);
        }
        uint32_t pc = 0, back = 0;
        bool gave_up = false;
        while (true) {
            const uint4 w = PARAM ? prm.code[pc] : s_code[pc];
            ++pc;
            const uint32_t op = w.x & 0xFFFFu, dst = w.x >> 16, ra = w.y & 0xFFFFu, rb = w.y >> 16, rc = w.z & 0xFFFFu;
            if (op == CATENA_MAP_HALT) break;
            if (op == CATENA_MAP_JMP || op == CATENA_MAP_JZ) {          // V == 1 here
                if (op == CATENA_MAP_JMP || lo(ra, 0) == 0) {
                    if (w.w < pc && ++back > kBackJumpBudget) {
                        fault = max(fault, (uint32_t)ERR_BUDGET);
                        gave_up = true;
                        break;
                    }
                    pc = w.w;
                }
                continue;
            }
            // one dispatch per instruction; inside a case the V elements are independent
#define CATENA_R64(R, v) (((uint64_t)hi[R][v] << 32) | lo(R, v))
#define CATENA_W64(v, X)                       \
    do {                                       \
        const uint64_t x_ = (X);               \
        lo(dst, v) = (uint32_t)x_;             \
        hi[dst][v] = (uint32_t)(x_ >> 32);     \
    } while (0)
#define CATENA_LANES _Pragma("unroll") for (int v = 0; v < V; ++v)
// all lanes of a register's low half in one access (16 bytes for four lanes)
#define CATENA_LD(R, X)                                                                    \
    uint32_t X[V];                                                                         \
    if (V == 4) {                                                                          \
        const uint4 t_ = *reinterpret_cast<const uint4*>(&lo(R, 0));                       \
        X[0] = t_.x; X[V > 1 ? 1 : 0] = t_.y; X[V > 2 ? 2 : 0] = t_.z; X[V > 3 ? 3 : 0] = t_.w; \
    } else {                                                                               \
        CATENA_LANES X[v] = lo(R, v);                                                      \
    }
#define CATENA_ST(X)                                                                       \
    if (V == 4) *reinterpret_cast<uint4*>(&lo(dst, 0)) = make_uint4(X[0], X[V > 1 ? 1 : 0], X[V > 2 ? 2 : 0], X[V > 3 ? 3 : 0]); \
    else CATENA_LANES lo(dst, v) = X[v]
// 32-bit operands and result
#define CATENA_W(EXPR)      { CATENA_LD(ra, A_) CATENA_LD(rb, B_) uint32_t R_[V]; CATENA_LANES { const uint32_t a = A_[v], b = B_[v]; (void)b; R_[v] = (uint32_t)(EXPR); } CATENA_ST(R_); } break
#define CATENA_W1(EXPR)     { CATENA_LD(ra, A_) uint32_t R_[V]; CATENA_LANES { const uint32_t a = A_[v]; R_[v] = (uint32_t)(EXPR); } CATENA_ST(R_); } break
// 64-bit operands, 64-bit result
#define CATENA_D(EXPR)      CATENA_LANES { const uint64_t a = CATENA_R64(ra, v), b = CATENA_R64(rb, v); (void)b; CATENA_W64(v, EXPR); } break
// 64-bit operands, 32-bit result (compares, conversions)
#define CATENA_DW(EXPR)     CATENA_LANES { const uint64_t a = CATENA_R64(ra, v), b = CATENA_R64(rb, v); (void)b; lo(dst, v) = (uint32_t)(EXPR); } break
#define CATENA_DW1(EXPR)    CATENA_LANES { const uint64_t a = CATENA_R64(ra, v); lo(dst, v) = (uint32_t)(EXPR); } break
#define CATENA_F(EXPR)      { CATENA_LD(ra, A_) CATENA_LD(rb, B_) uint32_t R_[V]; CATENA_LANES { const float a = __uint_as_float(A_[v]), b = __uint_as_float(B_[v]); (void)b; R_[v] = __float_as_uint(EXPR); } CATENA_ST(R_); } break
#define CATENA_FC(EXPR)     { CATENA_LD(ra, A_) CATENA_LD(rb, B_) uint32_t R_[V]; CATENA_LANES { const float a = __uint_as_float(A_[v]), b = __uint_as_float(B_[v]); R_[v] = (EXPR) ? 1u : 0u; } CATENA_ST(R_); } break
#define CATENA_UNDEF        (fault = max(fault, (uint32_t)ERR_UNDEFINED), 0)
            switch (op) {
            case CATENA_MAP_ASSERT:
                CATENA_LANES { if (lo(ra, v) == 0) fault = max(fault, (uint32_t)ERR_ASSERT); }
                break;
            case CATENA_MAP_MOV:
                CATENA_LANES { lo(dst, v) = lo(ra, v); hi[dst][v] = hi[ra][v]; }
                break;
            case CATENA_MAP_SELECT:
                CATENA_LANES {
                    const bool t = lo(ra, v) != 0;
                    const uint32_t l = t ? lo(rb, v) : lo(rc, v), h = t ? hi[rb][v] : hi[rc][v];
                    lo(dst, v) = l;
                    hi[dst][v] = h;
                }
                break;
            case CATENA_MAP_MOV32: CATENA_W1(a);
            case CATENA_MAP_SELECT32: {
                CATENA_LD(ra, A_) CATENA_LD(rb, B_) CATENA_LD(rc, C_) uint32_t R_[V];
                CATENA_LANES R_[v] = A_[v] != 0 ? B_[v] : C_[v];
                CATENA_ST(R_);
                break;
            }
            case CATENA_MAP_BOOL_NOT: CATENA_W1(a ? 0u : 1u);
            case CATENA_MAP_BOOL_AND: CATENA_W((a && b) ? 1u : 0u);
            case CATENA_MAP_BOOL_OR: CATENA_W((a || b) ? 1u : 0u);
            case CATENA_MAP_U64_ADD: CATENA_D(a + b);
            case CATENA_MAP_U64_SUB: CATENA_D(a - b);
            case CATENA_MAP_U64_MUL: CATENA_D(a * b);
            case CATENA_MAP_U64_DIV: CATENA_D(b == 0 ? (uint64_t)CATENA_UNDEF : a / b);
            case CATENA_MAP_U64_REM: CATENA_D(b == 0 ? (uint64_t)CATENA_UNDEF : a % b);
            case CATENA_MAP_U64_EQ: CATENA_DW(a == b);
            case CATENA_MAP_U64_NE: CATENA_DW(a != b);
            case CATENA_MAP_U64_LT: CATENA_DW(a < b);
            case CATENA_MAP_U64_LTE: CATENA_DW(a <= b);
            case CATENA_MAP_U64_GT: CATENA_DW(a > b);
            case CATENA_MAP_U64_GTE: CATENA_DW(a >= b);
            case CATENA_MAP_U64_TO_F32: CATENA_DW1(__float_as_uint(cmath::u64_to_f32(a)));
            case CATENA_MAP_U32_ADD: CATENA_W(a + b);
            case CATENA_MAP_U32_SUB: CATENA_W(a - b);
            case CATENA_MAP_U32_MUL: CATENA_W(a * b);
            case CATENA_MAP_U32_AND: CATENA_W(a & b);
            case CATENA_MAP_U32_OR: CATENA_W(a | b);
            case CATENA_MAP_U32_XOR: CATENA_W(a ^ b);
            case CATENA_MAP_U32_NOT: CATENA_W1(~a);
            case CATENA_MAP_U32_SHL: CATENA_W(b >= 32u ? (uint32_t)CATENA_UNDEF : a << b);
            case CATENA_MAP_U32_SHR: CATENA_W(b >= 32u ? (uint32_t)CATENA_UNDEF : a >> b);
            case CATENA_MAP_U32_EQ: CATENA_W(a == b);
            case CATENA_MAP_U32_NE: CATENA_W(a != b);
            case CATENA_MAP_U32_LT: CATENA_W(a < b);
            case CATENA_MAP_U32_LTE: CATENA_W(a <= b);
            case CATENA_MAP_U32_GT: CATENA_W(a > b);
            case CATENA_MAP_U32_GTE: CATENA_W(a >= b);
            case CATENA_MAP_U32_TO_F32: CATENA_W1(__float_as_uint(cmath::u32_to_f32(a)));
            case CATENA_MAP_F32_ADD: CATENA_F(cmath::add(a, b));
            case CATENA_MAP_F32_SUB: CATENA_F(cmath::sub(a, b));
            case CATENA_MAP_F32_MUL: CATENA_F(cmath::mul(a, b));
            case CATENA_MAP_F32_DIV: CATENA_F(cmath::div(a, b));
            case CATENA_MAP_F32_NEG: CATENA_W1(a ^ 0x80000000u);
            case CATENA_MAP_F32_FMA: {
                CATENA_LD(ra, A_) CATENA_LD(rb, B_) CATENA_LD(rc, C_) uint32_t R_[V];
                CATENA_LANES R_[v] = __float_as_uint(__fmaf_rn(__uint_as_float(A_[v]), __uint_as_float(B_[v]), __uint_as_float(C_[v])));
                CATENA_ST(R_);
                break;
            }
#define CATENA_F3(EXPR)                                                                                            \
    {                                                                                                              \
        CATENA_LD(ra, A_) CATENA_LD(rb, B_) CATENA_LD(rc, C_) uint32_t R_[V];                                      \
        CATENA_LANES {                                                                                             \
            const float p = cmath::mul(__uint_as_float(A_[v]), __uint_as_float(B_[v])), c = __uint_as_float(C_[v]); \
            R_[v] = __float_as_uint(EXPR);                                                                         \
        }                                                                                                          \
        CATENA_ST(R_);                                                                                             \
    }                                                                                                              \
    break
            case CATENA_MAP_F32_MULADD: CATENA_F3(cmath::add(p, c));
            case CATENA_MAP_F32_MULSUB: CATENA_F3(cmath::sub(p, c));
            case CATENA_MAP_F32_SUBMUL: CATENA_F3(cmath::sub(c, p));
#undef CATENA_F3
            case CATENA_MAP_F32_EQ: CATENA_FC(a == b);
            case CATENA_MAP_F32_NE: CATENA_FC(a != b);
            case CATENA_MAP_F32_LT: CATENA_FC(a < b);
            case CATENA_MAP_F32_LTE: CATENA_FC(a <= b);
            case CATENA_MAP_F32_GT: CATENA_FC(a > b);
            case CATENA_MAP_F32_GTE: CATENA_FC(a >= b);
            case CATENA_MAP_F32_ROUND_TO_U32: CATENA_F(__uint_as_float(!(a >= 0.0f && a < 4294967296.0f) ? (uint32_t)CATENA_UNDEF : cmath::round_to_u32(a)));
            // loads: buffer rb [register ra]; rb is a buffer number (checked by the host), not a register
            case CATENA_MAP_LOAD_U64:
                CATENA_LANES {
                    const uint64_t a = CATENA_R64(ra, v);
                    uint64_t x = 0;
                    if (a >= (bufs.bytes[rb] >> 3)) fault = max(fault, (uint32_t)ERR_RANGE);
                    else x = __ldg(reinterpret_cast<const uint64_t*>(bufs.base[rb]) + a);
                    CATENA_W64(v, x);
                }
                break;
            case CATENA_MAP_LOAD_F32:
                CATENA_LANES {
                    const uint64_t a = CATENA_R64(ra, v);
                    uint32_t x = 0;
                    if (a >= (bufs.bytes[rb] >> 2)) fault = max(fault, (uint32_t)ERR_RANGE);
                    else x = __ldg(reinterpret_cast<const uint32_t*>(bufs.base[rb]) + a);
                    lo(dst, v) = x;
                }
                break;
            default: break;      // unreachable: the host validated every opcode
            }
#undef CATENA_R64
#undef CATENA_W64
#undef CATENA_LANES
#undef CATENA_LD
#undef CATENA_ST
#undef CATENA_W
#undef CATENA_W1
#undef CATENA_D
#undef CATENA_DW
#undef CATENA_DW1
#undef CATENA_F
#undef CATENA_FC
#undef CATENA_UNDEF
        }
#pragma unroll
        for (int v = 0; v < V; ++v) {
            const uint64_t e = i + v * stride;
            if (e < len) {
                if (elem_bytes == 8) static_cast<uint64_t*>(out)[e] = gave_up ? 0ull : (((uint64_t)hi[result_reg][v] << 32) | lo(result_reg, v));
                else static_cast<uint32_t*>(out)[e] = gave_up ? 0u : lo(result_reg, v);
            }
        }
    }
#undef lo
    if (fault != ERR_NONE) atomicMax(err, fault);
}

struct State {
    uint32_t* err = nullptr;        // device error word
    uint32_t* err_host = nullptr;   // pinned
};
static thread_local State g_state[kMaxDevices];

static catena_status_t state(State** out) {
    State& st = g_state[tls().device];
    if (!st.err) {
        CATENA_CUDA(cudaMalloc(&st.err, sizeof(uint32_t)));
        CATENA_CUDA(cudaMemset(st.err, 0, sizeof(uint32_t)));
        CATENA_CUDA(cudaMallocHost(&st.err_host, sizeof(uint32_t)));
        *st.err_host = 0;
    }
    *out = &st;
    return CATENA_OK;
}

// which operands of an opcode are registers: bit 0 = a, bit 1 = b, bit 2 = c, bit 3 = writes dst; 0xFF = unknown opcode
static uint32_t operand_mask(uint32_t op) {
    switch (op) {
    case CATENA_MAP_HALT: case CATENA_MAP_JMP: return 0;
    case CATENA_MAP_JZ: case CATENA_MAP_ASSERT: return 1;
    case CATENA_MAP_MOV: case CATENA_MAP_MOV32: case CATENA_MAP_BOOL_NOT: case CATENA_MAP_U64_TO_F32: case CATENA_MAP_U32_NOT:
    case CATENA_MAP_U32_TO_F32: case CATENA_MAP_F32_NEG: case CATENA_MAP_F32_ROUND_TO_U32: return 1 | 8;
    case CATENA_MAP_SELECT: case CATENA_MAP_SELECT32: case CATENA_MAP_F32_FMA: case CATENA_MAP_F32_MULADD: case CATENA_MAP_F32_MULSUB:
    case CATENA_MAP_F32_SUBMUL: return 1 | 2 | 4 | 8;
    case CATENA_MAP_LOAD_U64: case CATENA_MAP_LOAD_F32: return 1 | 8;      // b is a buffer number
    default: return op < CATENA_MAP_OP_COUNT ? (1 | 2 | 8) : 0xFF;
    }
}

static catena_status_t validate(const catena_b200_map_insn_t* code, uint32_t n_insn, uint32_t n_init, uint32_t n_regs, uint32_t index_reg,
                                uint32_t result_reg, uint32_t n_buffers, uint32_t max_regs = kMaxRegs) {
    if (!code || n_insn == 0 || n_insn > kMaxInsns) return fail(CATENA_E_BAD_ARG, "map program: between 1 and 2048 instructions");
    if (n_regs == 0 || n_regs > max_regs || n_init > n_regs)
        return fail(CATENA_E_BAD_ARG, "map program: too many registers (interpreted: 256, compiled: 4096; preset ones included)");
    if (index_reg < n_init || index_reg >= n_regs || result_reg >= n_regs) return fail(CATENA_E_BAD_ARG, "map program: index or result register out of range");
    if (n_buffers > kMaxBuffers) return fail(CATENA_E_BAD_ARG, "map program: more than 16 buffers");
    if (code[n_insn - 1].op != CATENA_MAP_HALT) return fail(CATENA_E_BAD_ARG, "map program: the last instruction must be HALT");
    for (uint32_t k = 0; k < n_insn; ++k) {
        const catena_b200_map_insn_t& in = code[k];
        const uint32_t mask = operand_mask(in.op);
        if (mask == 0xFF) return fail(CATENA_E_BAD_ARG, "map program: unknown opcode");
        // operands an opcode does not use are still read by the interpreter's common prologue: they must be registers too
        if (in.a >= n_regs || in.c >= n_regs) return fail(CATENA_E_BAD_ARG, "map program: register out of range");
        const bool load = in.op == CATENA_MAP_LOAD_U64 || in.op == CATENA_MAP_LOAD_F32;
        if (load ? in.b >= n_buffers : in.b >= n_regs) return fail(CATENA_E_BAD_ARG, "map program: register or buffer out of range");
        if ((mask & 8) && (in.dst < n_init || in.dst >= n_regs || in.dst == index_reg))
            return fail(CATENA_E_BAD_ARG, "map program: an instruction writes a preset register, the index register or past the register file");
        if ((in.op == CATENA_MAP_JMP || in.op == CATENA_MAP_JZ) && in.target >= n_insn) return fail(CATENA_E_BAD_ARG, "map program: jump target out of range");
    }
    return CATENA_OK;
}

}  // namespace mapvm

catena_status_t map_program_validate(const catena_b200_map_insn_t* code, uint32_t n_insn, uint32_t n_init, uint32_t n_regs, uint32_t index_reg,
                                     uint32_t result_reg, uint32_t n_buffers, uint32_t max_regs) {
    return mapvm::validate(code, n_insn, n_init, n_regs, index_reg, result_reg, n_buffers, max_regs);
}

catena_status_t map_program_error_word(uint32_t** err) {
    mapvm::State* st = nullptr;
    CATENA_TRY(mapvm::state(&st));
    *err = st->err;
    return CATENA_OK;
}

// Reports (and clears) what the programs of earlier launches ran into; synchronises the stream.
catena_status_t map_program_check_errors() {
    CATENA_TRY(ensure_device());
    mapvm::State& st = mapvm::g_state[tls().device];
    if (!st.err) return CATENA_OK;
    cudaStream_t s = tls().stream;
    CATENA_CUDA(cudaMemcpyAsync(st.err_host, st.err, sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    CATENA_CUDA(cudaStreamSynchronize(s));
    const uint32_t e = *st.err_host;
    if (e == mapvm::ERR_NONE) return CATENA_OK;
    *st.err_host = 0;
    cudaMemsetAsync(st.err, 0, sizeof(uint32_t), s);
    switch (e) {
    case mapvm::ERR_ASSERT: return fail(CATENA_E_ASSERT, "map program: catena assertion failed");
    case mapvm::ERR_RANGE: return fail(CATENA_E_ASSERT, "map program: an index reaches past its buffer");
    case mapvm::ERR_UNDEFINED: return fail(CATENA_E_ASSERT, "map program: an operation the reference's generated code leaves undefined (shift by 32 or more, round-to-u32 out of range, division by zero columns)");
    default: return fail(CATENA_E_ASSERT, "map program: loop budget exceeded");
    }
}

}  // namespace catena

using namespace catena;

extern "C" {

catena_status_t catena_b200_map_program_s(const catena_b200_map_insn_t* code, uint32_t n_insn, const uint64_t* init, uint32_t n_init,
                                          uint32_t n_regs, uint32_t index_reg, uint32_t result_reg, const catena_mem_t* buffers,
                                          uint32_t n_buffers, uint32_t elem_bytes, uint64_t len, catena_mem_t* out) {
    return catena_b200_map_program_range_s(code, n_insn, init, n_init, n_regs, index_reg, result_reg, buffers, n_buffers, elem_bytes, 0, len, out);
}

catena_status_t catena_b200_map_program_range_s(const catena_b200_map_insn_t* code, uint32_t n_insn, const uint64_t* init, uint32_t n_init,
                                                uint32_t n_regs, uint32_t index_reg, uint32_t result_reg, const catena_mem_t* buffers,
                                                uint32_t n_buffers, uint32_t elem_bytes, uint64_t index0, uint64_t len, catena_mem_t* out) {
    if (!out) return fail(CATENA_E_BAD_ARG, "map program: null output pointer");
    out->data = nullptr;
    out->len = 0;
    if (elem_bytes != 4 && elem_bytes != 8) return fail(CATENA_E_BAD_ARG, "map program: elements of 4 or 8 bytes");
    if ((n_init && !init) || (n_buffers && !buffers)) return fail(CATENA_E_BAD_ARG, "map program: null argument");
    CATENA_TRY(mapvm::validate(code, n_insn, n_init, n_regs, index_reg, result_reg, n_buffers));
    mapvm::Buffers bufs = {};
    for (uint32_t k = 0; k < n_buffers; ++k) {
        if (buffers[k].len != 0 && !buffers[k].data) return fail(CATENA_E_BAD_ARG, "map program: null buffer");
        if ((uintptr_t)buffers[k].data & 7) return fail(CATENA_E_BAD_ARG, "map program: buffers must be 8-byte aligned");
        bufs.base[k] = static_cast<const uint8_t*>(buffers[k].data);
        bufs.bytes[k] = buffers[k].len;
    }
    if (len > (~0ull) / elem_bytes || index0 > ~0ull - len) return fail(CATENA_E_TOO_LARGE, "map program: length overflows");
    CATENA_TRY(ensure_device());
    if (len == 0) return CATENA_OK;                        // no allocation, no launch (materializec.rs:108-116)
    mapvm::State* st = nullptr;
    CATENA_TRY(mapvm::state(&st));
    bool straight = true;                                  // no jumps: V elements per thread can run in lockstep
    for (uint32_t k = 0; k < n_insn; ++k) straight = straight && code[k].op != CATENA_MAP_JMP && code[k].op != CATENA_MAP_JZ;
    const bool by_param = n_insn <= mapvm::kParamInsns && n_init <= mapvm::kParamInit;
    const size_t code_bytes = (size_t)n_insn * sizeof(catena_b200_map_insn_t), init_bytes = (size_t)n_init * sizeof(uint64_t);
    void* scratch = nullptr;
    void* result = nullptr;
    catena_status_t s = pool_alloc(len * elem_bytes, &result);
    if (s != CATENA_OK) return s;
    cudaStream_t stream = tls().stream;
    cudaError_t e = cudaSuccess;
    static_assert(sizeof(catena_b200_map_insn_t) == sizeof(uint4), "instruction layout");
    mapvm::ParamProgram prm;
    memset(&prm, 0, sizeof(prm));
    if (by_param) {
        memcpy(prm.code, code, code_bytes);
        if (init_bytes) memcpy(prm.init, init, init_bytes);
    } else {
        // instructions and preset registers travel in one scratch block
        s = pool_alloc(code_bytes + init_bytes + 16, &scratch);
        if (s != CATENA_OK) {
            pool_free(result);
            return s;
        }
        e = cudaMemcpyAsync(scratch, code, code_bytes, cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess && init_bytes)
            e = cudaMemcpyAsync(static_cast<uint8_t*>(scratch) + code_bytes, init, init_bytes, cudaMemcpyHostToDevice, stream);
        // the host arrays are pageable and may change when this call returns: the copies must have read them
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    }
    if (e == cudaSuccess) {
        const int sms = tls().sm_count > 0 ? tls().sm_count : 148;
        // geometry: the low halves of the register file take n_regs x lanes x threads x 4 bytes of shared memory per CTA
        const size_t smem_limit = 200 * 1024, staged = by_param ? 0 : code_bytes;
        int lanes = straight && n_regs <= 128 ? 4 : 1, threads = 256;
        if ((size_t)n_regs * lanes * threads * 4 + staged > smem_limit) lanes = 1;
        if ((size_t)n_regs * lanes * threads * 4 + staged > smem_limit) threads = 128;
        const size_t smem = (size_t)n_regs * lanes * threads * 4 + staged;
        uint64_t per_sm = (227ull * 1024) / (smem + 1024);
        per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
        uint64_t blocks = ceil_div_u64(len, (uint64_t)threads * lanes);
        if (blocks > (uint64_t)sms * per_sm) blocks = (uint64_t)sms * per_sm;
        const uint4* dcode = static_cast<const uint4*>(scratch);
        const uint64_t* dinit = scratch ? reinterpret_cast<const uint64_t*>(static_cast<uint8_t*>(scratch) + code_bytes) : nullptr;
#define CATENA_MAP_LAUNCH(R, V, P, TT)                                                                                                 \
    do {                                                                                                                            \
        static thread_local size_t attr_[kMaxDevices] = {0};                                                                        \
        if (smem > 48 * 1024 && attr_[tls().device] < smem) {                                                                       \
            e = cudaFuncSetAttribute(mapvm::map_program_kernel<R, V, P, TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e == cudaSuccess) attr_[tls().device] = smem;                                                                       \
        }                                                                                                                           \
        if (e == cudaSuccess)                                                                                                       \
            mapvm::map_program_kernel<R, V, P, TT><<<(unsigned)blocks, TT, smem, stream>>>(                                         \
                prm, dcode, n_insn, dinit, n_init, n_regs, index_reg, result_reg, bufs, result, elem_bytes, index0, len, st->err);          \
    } while (0)
#define CATENA_MAP_PICK(R)                                                   \
    do {                                                                     \
        if (lanes == 4 && by_param) CATENA_MAP_LAUNCH(R, 4, true, 256);      \
        else if (lanes == 4) CATENA_MAP_LAUNCH(R, 4, false, 256);            \
        else if (by_param) CATENA_MAP_LAUNCH(R, 1, true, 256);               \
        else CATENA_MAP_LAUNCH(R, 1, false, 256);                            \
    } while (0)
        if (n_regs <= 32) CATENA_MAP_PICK(32);
        else if (n_regs <= 64) CATENA_MAP_PICK(64);
        else if (n_regs <= 128) CATENA_MAP_PICK(128);
        else if (threads == 256 && by_param) CATENA_MAP_LAUNCH(256, 1, true, 256);
        else if (threads == 256) CATENA_MAP_LAUNCH(256, 1, false, 256);
        else if (by_param) CATENA_MAP_LAUNCH(256, 1, true, 128);
        else CATENA_MAP_LAUNCH(256, 1, false, 128);
#undef CATENA_MAP_PICK
#undef CATENA_MAP_LAUNCH
        count_launch();
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) s = fail_cuda(e, "map program");
    if (s == CATENA_OK && tls().blocking) s = map_program_check_errors();
    if (scratch) pool_free(scratch);
    if (s != CATENA_OK) {
        pool_free(result);
        return s;
    }
    out->data = result;
    out->len = len * elem_bytes;
    return CATENA_OK;
}

}  // extern "C"
