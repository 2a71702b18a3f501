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
// Values are 64-bit registers: bool as 0 / 1, u32 zero-extended, f32 as its bit pattern in the low half, u64 as is, so the
// bitcasts are moves.  f32 arithmetic goes through the explicitly rounded operations of catena_math.cuh (never contracted),
// `f32.fma` is one fused operation, `f32.round-to-u32` rounds to nearest even, `u64.to-f32` / `u32.to-f32` round once.
//
// Nothing a program does can fault or hang the GPU: the host checks every register number, buffer number and jump target
// before the launch; loads are bounds-checked against the buffer's length; backward jumps are counted against a budget.
// Where the reference's generated C would trap (`catena_assert`), read past a buffer or be undefined (a u32 shift by 32 or
// more, `f32.round-to-u32` outside [0, 2^32), a row-major division by zero columns) the element yields 0, the launch carries on
// and the entry point reports CATENA_E_ASSERT.
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

template <int REGS>
__global__ void __launch_bounds__(256) map_program_kernel(const uint4* __restrict__ code, uint32_t n_insn, const uint64_t* __restrict__ init,
                                                          uint32_t n_init, uint32_t index_reg, uint32_t result_reg, const Buffers bufs,
                                                          void* __restrict__ out, uint32_t elem_bytes, uint64_t len, uint32_t* err) {
    extern __shared__ uint4 s_code[];
    for (uint32_t k = threadIdx.x; k < n_insn; k += blockDim.x) s_code[k] = code[k];
    __syncthreads();
    uint64_t r[REGS];
#pragma unroll 1
    for (uint32_t k = 0; k < (uint32_t)REGS; ++k) r[k] = k < n_init ? init[k] : 0ull;
    uint32_t fault = ERR_NONE;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += stride) {
        r[index_reg] = i;
        uint32_t pc = 0, back = 0;
        bool running = true;
        while (running) {
            const uint4 w = s_code[pc++];
            const uint32_t op = w.x & 0xFFFFu, dst = w.x >> 16, ra = w.y & 0xFFFFu, rb = w.y >> 16, rc = w.z & 0xFFFFu;
            const uint64_t a = r[ra], b = r[rb];
            uint64_t v = 0;
            bool write = true;
            switch (op) {
            case CATENA_MAP_HALT: running = false; write = false; break;
            case CATENA_MAP_MOV: v = a; break;
            case CATENA_MAP_JMP:
            case CATENA_MAP_JZ:
                write = false;
                if (op == CATENA_MAP_JMP || a == 0) {
                    if (w.w < pc && ++back > kBackJumpBudget) {
                        fault = max(fault, (uint32_t)ERR_BUDGET);
                        r[result_reg] = 0;
                        running = false;
                    } else {
                        pc = w.w;
                    }
                }
                break;
            case CATENA_MAP_ASSERT: write = false; if (a == 0) fault = max(fault, (uint32_t)ERR_ASSERT); break;
            case CATENA_MAP_SELECT: v = a ? b : r[rc]; break;
            case CATENA_MAP_BOOL_NOT: v = a ? 0 : 1; break;
            case CATENA_MAP_BOOL_AND: v = (a && b) ? 1 : 0; break;
            case CATENA_MAP_BOOL_OR: v = (a || b) ? 1 : 0; break;
            case CATENA_MAP_U64_ADD: v = a + b; break;
            case CATENA_MAP_U64_SUB: v = a - b; break;
            case CATENA_MAP_U64_MUL: v = a * b; break;
            case CATENA_MAP_U64_DIV:
            case CATENA_MAP_U64_REM:
                if (b == 0) fault = max(fault, (uint32_t)ERR_UNDEFINED);
                else v = op == CATENA_MAP_U64_DIV ? a / b : a % b;
                break;
            case CATENA_MAP_U64_EQ: v = a == b; break;
            case CATENA_MAP_U64_NE: v = a != b; break;
            case CATENA_MAP_U64_LT: v = a < b; break;
            case CATENA_MAP_U64_LTE: v = a <= b; break;
            case CATENA_MAP_U64_GT: v = a > b; break;
            case CATENA_MAP_U64_GTE: v = a >= b; break;
            case CATENA_MAP_U64_TO_F32: v = from_f32(cmath::u64_to_f32(a)); break;
            case CATENA_MAP_U32_ADD: v = (uint32_t)((uint32_t)a + (uint32_t)b); break;
            case CATENA_MAP_U32_SUB: v = (uint32_t)((uint32_t)a - (uint32_t)b); break;
            case CATENA_MAP_U32_MUL: v = (uint32_t)((uint32_t)a * (uint32_t)b); break;
            case CATENA_MAP_U32_AND: v = (uint32_t)a & (uint32_t)b; break;
            case CATENA_MAP_U32_OR: v = (uint32_t)a | (uint32_t)b; break;
            case CATENA_MAP_U32_XOR: v = (uint32_t)a ^ (uint32_t)b; break;
            case CATENA_MAP_U32_NOT: v = (uint32_t)~(uint32_t)a; break;
            case CATENA_MAP_U32_SHL:
            case CATENA_MAP_U32_SHR:
                if ((uint32_t)b >= 32u) fault = max(fault, (uint32_t)ERR_UNDEFINED);
                else v = op == CATENA_MAP_U32_SHL ? (uint32_t)((uint32_t)a << (uint32_t)b) : ((uint32_t)a >> (uint32_t)b);
                break;
            case CATENA_MAP_U32_EQ: v = (uint32_t)a == (uint32_t)b; break;
            case CATENA_MAP_U32_NE: v = (uint32_t)a != (uint32_t)b; break;
            case CATENA_MAP_U32_LT: v = (uint32_t)a < (uint32_t)b; break;
            case CATENA_MAP_U32_LTE: v = (uint32_t)a <= (uint32_t)b; break;
            case CATENA_MAP_U32_GT: v = (uint32_t)a > (uint32_t)b; break;
            case CATENA_MAP_U32_GTE: v = (uint32_t)a >= (uint32_t)b; break;
            case CATENA_MAP_U32_TO_F32: v = from_f32(cmath::u32_to_f32((uint32_t)a)); break;
            case CATENA_MAP_F32_ADD: v = from_f32(cmath::add(as_f32(a), as_f32(b))); break;
            case CATENA_MAP_F32_SUB: v = from_f32(cmath::sub(as_f32(a), as_f32(b))); break;
            case CATENA_MAP_F32_MUL: v = from_f32(cmath::mul(as_f32(a), as_f32(b))); break;
            case CATENA_MAP_F32_DIV: v = from_f32(cmath::div(as_f32(a), as_f32(b))); break;
            case CATENA_MAP_F32_NEG: v = (uint32_t)a ^ 0x80000000u; break;
            case CATENA_MAP_F32_FMA: v = from_f32(__fmaf_rn(as_f32(a), as_f32(b), as_f32(r[rc]))); break;
            case CATENA_MAP_F32_EQ: v = as_f32(a) == as_f32(b); break;
            case CATENA_MAP_F32_NE: v = as_f32(a) != as_f32(b); break;
            case CATENA_MAP_F32_LT: v = as_f32(a) < as_f32(b); break;
            case CATENA_MAP_F32_LTE: v = as_f32(a) <= as_f32(b); break;
            case CATENA_MAP_F32_GT: v = as_f32(a) > as_f32(b); break;
            case CATENA_MAP_F32_GTE: v = as_f32(a) >= as_f32(b); break;
            case CATENA_MAP_F32_ROUND_TO_U32: {
                const float x = as_f32(a);
                if (!(x >= 0.0f && x < 4294967296.0f)) fault = max(fault, (uint32_t)ERR_UNDEFINED);
                else v = cmath::round_to_u32(x);
                break;
            }
            case CATENA_MAP_LOAD_U64:
            case CATENA_MAP_LOAD_F32: {       // dst = buffer rb [a]; rb is a buffer number (checked by the host), not a register
                const uint32_t shift = op == CATENA_MAP_LOAD_U64 ? 3u : 2u;
                if (a >= (bufs.bytes[rb] >> shift)) fault = max(fault, (uint32_t)ERR_RANGE);
                else if (shift == 3u) v = __ldg(reinterpret_cast<const uint64_t*>(bufs.base[rb]) + a);
                else v = __ldg(reinterpret_cast<const uint32_t*>(bufs.base[rb]) + a);
                break;
            }
            default: running = false; write = false; break;      // unreachable: the host validated every opcode
            }
            if (write) r[dst] = v;
        }
        if (elem_bytes == 8) static_cast<uint64_t*>(out)[i] = r[result_reg];
        else static_cast<uint32_t*>(out)[i] = (uint32_t)r[result_reg];
    }
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
    case CATENA_MAP_MOV: case CATENA_MAP_BOOL_NOT: case CATENA_MAP_U64_TO_F32: case CATENA_MAP_U32_NOT: case CATENA_MAP_U32_TO_F32:
    case CATENA_MAP_F32_NEG: case CATENA_MAP_F32_ROUND_TO_U32: return 1 | 8;
    case CATENA_MAP_SELECT: case CATENA_MAP_F32_FMA: return 1 | 2 | 4 | 8;
    case CATENA_MAP_LOAD_U64: case CATENA_MAP_LOAD_F32: return 1 | 8;      // b is a buffer number
    default: return op < CATENA_MAP_OP_COUNT ? (1 | 2 | 8) : 0xFF;
    }
}

static catena_status_t validate(const catena_b200_map_insn_t* code, uint32_t n_insn, uint32_t n_init, uint32_t n_regs, uint32_t index_reg,
                                uint32_t result_reg, uint32_t n_buffers) {
    if (!code || n_insn == 0 || n_insn > kMaxInsns) return fail(CATENA_E_BAD_ARG, "map program: between 1 and 2048 instructions");
    if (n_regs == 0 || n_regs > kMaxRegs || n_init > n_regs) return fail(CATENA_E_BAD_ARG, "map program: at most 256 registers, preset ones included");
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
    if (len > (~0ull) / elem_bytes) return fail(CATENA_E_TOO_LARGE, "map program: length overflows");
    CATENA_TRY(ensure_device());
    if (len == 0) return CATENA_OK;                        // no allocation, no launch (materializec.rs:108-116)
    mapvm::State* st = nullptr;
    CATENA_TRY(mapvm::state(&st));
    // instructions and preset registers travel in one scratch block
    const size_t code_bytes = (size_t)n_insn * sizeof(catena_b200_map_insn_t), init_bytes = (size_t)n_init * sizeof(uint64_t);
    void* scratch = nullptr;
    void* result = nullptr;
    CATENA_TRY(pool_alloc(code_bytes + init_bytes + 16, &scratch));
    catena_status_t s = pool_alloc(len * elem_bytes, &result);
    if (s != CATENA_OK) {
        pool_free(scratch);
        return s;
    }
    cudaStream_t stream = tls().stream;
    cudaError_t e = cudaMemcpyAsync(scratch, code, code_bytes, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess && init_bytes)
        e = cudaMemcpyAsync(static_cast<uint8_t*>(scratch) + code_bytes, init, init_bytes, cudaMemcpyHostToDevice, stream);
    // the host arrays are pageable and may change when this call returns: the copies must have read them
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e == cudaSuccess) {
        const int sms = tls().sm_count > 0 ? tls().sm_count : 148;
        uint64_t blocks = ceil_div_u64(len, 256);
        if (blocks > (uint64_t)sms * 8) blocks = (uint64_t)sms * 8;
        const uint4* dcode = static_cast<const uint4*>(scratch);
        const uint64_t* dinit = reinterpret_cast<const uint64_t*>(static_cast<uint8_t*>(scratch) + code_bytes);
#define CATENA_MAP_LAUNCH(R)                                                                                                         \
    mapvm::map_program_kernel<R><<<(unsigned)blocks, 256, code_bytes, stream>>>(dcode, n_insn, dinit, n_init, index_reg, result_reg, bufs, \
                                                                                result, elem_bytes, len, st->err)
        if (n_regs <= 32) CATENA_MAP_LAUNCH(32);
        else if (n_regs <= 64) CATENA_MAP_LAUNCH(64);
        else if (n_regs <= 128) CATENA_MAP_LAUNCH(128);
        else CATENA_MAP_LAUNCH(256);
#undef CATENA_MAP_LAUNCH
        count_launch();
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) s = fail_cuda(e, "map program");
    if (s == CATENA_OK && tls().blocking) s = map_program_check_errors();
    pool_free(scratch);
    if (s != CATENA_OK) {
        pool_free(result);
        return s;
    }
    out->data = result;
    out->len = len * elem_bytes;
    return CATENA_OK;
}

}  // extern "C"
