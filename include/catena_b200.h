/* catena_b200.h — C ABI of libcatena_b200.so
 *
 * A prebuilt sm_100a kernel library behind the calling convention that catena-lang's code
 * generator gives every entry point (catena-lang/src/codegen/gpu.rs:235-261,
 * catena-lang/src/runtime/executor.rs:65-106):
 *
 *     extern "C" void program_<name>(<inputs by value, source order>..., <T>* out...)
 *
 * with `bool -> uint8_t`, `u32 -> uint32_t`, `u64 -> uint64_t`, `f32 -> float` and
 * `mem -> catena_mem_t` passed BY VALUE (catena-lang/src/codegen/lower_types.rs:84-137,
 * catena-lang/src/codegen/prelude.rs:28-31).  Symbol names follow
 * catena-lang/src/codegen/mod.rs:379-388 (`program_` + name, non-alphanumerics -> `_`).
 *
 * Differences from the generated code, all additive:
 *   - `catena_mem_t.data` is DEVICE memory from catena_b200_mem_alloc (cudaMalloc behind a
 *     size-class pool), not cudaMallocManaged (catena-lang/src/runtime/mem.rs:152-171); hosts
 *     read results with catena_b200_mem_download.  Managed pointers are accepted as inputs.
 *   - a failed assertion never traps the device (catena-lang/src/codegen/prelude.rs:38-55
 *     calls __builtin_trap): the `void` entry point records a status readable with
 *     catena_b200_last_status(), prints one line on stderr and returns `{NULL,0}` / zero
 *     outputs; every entry point also has a `_s` twin returning the status.
 *   - there is no CPU fallback: without a CUDA device every compute entry point fails with
 *     CATENA_E_NO_DEVICE.
 */
#ifndef CATENA_B200_H
#define CATENA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* catena-lang/src/codegen/prelude.rs:28-31, catena-lang/src/runtime/executor.rs:14-19 */
typedef struct {
    void* data;   /* device pointer (NULL when len == 0) */
    uint64_t len; /* BYTES */
} catena_mem_t;

typedef int32_t catena_status_t;
enum {
    CATENA_OK = 0,
    CATENA_E_ASSERT = 1,      /* a `catena_assert` of the program would have trapped        */
    CATENA_E_CUDA = 2,        /* a CUDA runtime/driver call failed (`catena_host_gpu_check`) */
    CATENA_E_NO_DEVICE = 3,   /* no CUDA device / not an sm_100 part                         */
    CATENA_E_BAD_ARG = 4,     /* null pointer, misaligned buffer, unsupported shape          */
    CATENA_E_TIMEOUT = 5,     /* a bounded device-side wait gave up                          */
    CATENA_E_TOO_LARGE = 6,   /* size beyond a stated maximum                                */
    CATENA_E_UNSUPPORTED = 7  /* e.g. GpuDialect::Hip                                        */
};

/* ---- runtime: device, stream, status ------------------------------------------------ */
/* Replaces the implicit "globally set device" of the generated code
 * (catena-lang/doc/CODEGEN.md:164-166): binds the calling thread's library state to `device`. */
catena_status_t catena_b200_init(int device);
int catena_b200_device_count(void);
/* the device the calling thread's library state is bound to, -1 before the first catena_b200_init / compute call */
int catena_b200_current_device(void);
/* Entry points launch on this stream (default: the legacy default stream, as the generated
 * code does).  `stream` is a cudaStream_t.
 * Threads and streams: device, stream, blocking flag, last status and the scratch that kernels share between launches
 * (attention exchange area, rotary tables, device error words) belong to the calling HOST THREAD, per device.  One thread
 * drives one stream at a time: set_stream waits (in non-blocking mode) for the work queued on the old stream before the
 * same scratch can be used from the new one.  Several host threads may drive one device on their own streams; they share
 * only the memory pool, which orders the reuse of a freed block after the freeing stream's queued work.  As in the
 * reference (a device-wide synchronisation after every launch, catena-lang/src/codegen/ops/materializec.rs:138-141) the
 * compute entry points are not re-entrant on one thread's state. */
catena_status_t catena_b200_set_stream(void* stream);
void* catena_b200_get_stream(void);
/* 1 (default): every entry point synchronises before returning, as the generated code's
 * cudaDeviceSynchronize does (catena-lang/src/codegen/ops/materializec.rs:138-141).
 * 0: entry points only enqueue; call catena_b200_sync() before reading results. */
void catena_b200_set_blocking(int blocking);
catena_status_t catena_b200_sync(void);
catena_status_t catena_b200_last_status(void);
void catena_b200_clear_status(void);
const char* catena_b200_status_string(catena_status_t s);
const char* catena_b200_version(void);
/* number of kernels this library launched since load (all threads) */
uint64_t catena_b200_launch_count(void);

/* ---- allocator (replaces GpuRuntime::{alloc,free}, catena-lang/src/runtime/mem.rs:152-190)
 * A size-class pool over cudaMalloc, per device, shared by the host threads of that device.  mem_free in non-blocking mode
 * records an event on the calling thread's stream; a later mem_alloc that reuses the block from another stream makes
 * that stream wait for the event, so kernels still queued on the freeing stream never see the block change under them. */
catena_status_t catena_b200_mem_alloc(uint64_t bytes, catena_mem_t* out);
catena_status_t catena_b200_mem_free(catena_mem_t mem);
/* Mem::from_slice (catena-lang/src/runtime/mem.rs:72-106): allocate + copy host bytes in */
catena_status_t catena_b200_mem_upload(const void* host, uint64_t bytes, catena_mem_t* out);
/* Mem::to_f32_vec / to_u64_vec (catena-lang/src/runtime/mem.rs:43-70): copy bytes out */
catena_status_t catena_b200_mem_download(catena_mem_t mem, void* host, uint64_t bytes);
/* copy host bytes into an existing allocation (no reallocation) */
catena_status_t catena_b200_mem_write(catena_mem_t mem, const void* host, uint64_t bytes);
/* return pooled blocks to the driver */
catena_status_t catena_b200_mem_trim(void);
/* CUDA-IPC export/import so another process (one per GPU) can map an allocation as peer
 * memory over NVLink.  `handle64` is a 64-byte cudaIpcMemHandle_t; `offset` is the byte
 * offset of `mem.data` inside the exported allocation.  No counterpart in the reference
 * (single device, catena-lang/doc/CODEGEN.md:164-166). */
catena_status_t catena_b200_ipc_export(catena_mem_t mem, void* handle64, uint64_t* offset);
catena_status_t catena_b200_ipc_import(const void* handle64, uint64_t offset, uint64_t bytes,
                                       catena_mem_t* out);
catena_status_t catena_b200_ipc_close(catena_mem_t mem, uint64_t offset);

/* ---- scalar stdlib programs (run on the host, like the reference's non-materialize code)
 * catena-lang/stdlib/math.hex:3,27,52,91,110,148,185,202,213,224,235; stdlib/nn.hex:2,15,24,38 */
void program_math_sin_approx(float x, float* out);
void program_math_cos_approx(float x, float* out);
void program_math_sin_approx_full_nonneg(float x, float* out);
void program_math_sin_approx_full(float x, float* out);
void program_math_log_approx(float x, float* out);
void program_math_exp_approx_nonneg(float x, float* out);
void program_math_exp_approx(float x, float* out);
void program_math_exp2_approx(float x, float* out);
void program_math_log2_approx(float x, float* out);
void program_math_powf(float x, float y, float* out);
void program_math_sqrt(float x, float* out);
void program_nn_sigmoid(float x, float* out);
void program_nn_silu(float x, float* out);
void program_nn_tanh(float x, float* out);
void program_nn_gelu_approx(float x, float* out);

/* ---- buffer programs ------------------------------------------------------------------ */
/* catena-lang/stdlib/nn.hex:93-122 and :154-182.  Bit-exact with the reference's sequential folds up to 65536 elements for
 * inputs without NaN: the reference's max fold keeps the accumulator when `acc >= v` (catena-lang/stdlib/sum.hex:73-84), so
 * with a NaN in the input its result depends on where the NaN stands, and the parallel maximum here does not reproduce
 * that.  A zero of either sign as the maximum gives the same output bits. */
void program_nn_softmax(catena_mem_t in, catena_mem_t* out);
void program_nn_rmsnorm(catena_mem_t in, catena_mem_t* out);
catena_status_t program_nn_softmax_s(catena_mem_t in, catena_mem_t* out);
catena_status_t program_nn_rmsnorm_s(catena_mem_t in, catena_mem_t* out);
/* catena-lang/stdlib/sum.hex:29-44, :47-67, :86-101 */
void program_sum_f32(catena_mem_t in, float* out);
void program_mean_f32(catena_mem_t in, float* out);
void program_max_f32(catena_mem_t in, float* out);
catena_status_t program_sum_f32_s(catena_mem_t in, float* out);
catena_status_t program_mean_f32_s(catena_mem_t in, float* out);
catena_status_t program_max_f32_s(catena_mem_t in, float* out);
/* catena-lang/stdlib/tensor.hex:10-21, :35-46, :70-82, :141-168, :204-227 */
void program_tensor_broadcast_f32(float v, uint64_t n, catena_mem_t* out);
void program_tensor_arange_f32(uint64_t n, catena_mem_t* out);
void program_tensor_slice_f32(catena_mem_t in, uint64_t start, uint64_t len, catena_mem_t* out);
void program_tensor_concat_f32(catena_mem_t l, catena_mem_t r, catena_mem_t* out);
void program_tensor_argmax_f32(catena_mem_t in, uint64_t* out);
catena_status_t program_tensor_broadcast_f32_s(float v, uint64_t n, catena_mem_t* out);
catena_status_t program_tensor_arange_f32_s(uint64_t n, catena_mem_t* out);
catena_status_t program_tensor_slice_f32_s(catena_mem_t in, uint64_t start, uint64_t len,
                                           catena_mem_t* out);
catena_status_t program_tensor_concat_f32_s(catena_mem_t l, catena_mem_t r, catena_mem_t* out);
catena_status_t program_tensor_argmax_f32_s(catena_mem_t in, uint64_t* out);
/* catena-lang/tests/cases/matrix/matmul.hex:2-63 (entry program of the f32 matmul chain,
 * catena-lang/stdlib/matrix.hex:210-327): row-major f32, bit-exact ascending-k left fold with
 * separately rounded mul/add.  Asserts a.len/4 == nk and b.len/4 == km. */
void program_matmul_2x2_via_mem(catena_mem_t a, catena_mem_t b, uint64_t n, uint64_t m, uint64_t k,
                                uint64_t nk, uint64_t km, uint64_t nm, catena_mem_t* out);
catena_status_t program_matmul_2x2_via_mem_s(catena_mem_t a, catena_mem_t b, uint64_t n, uint64_t m,
                                             uint64_t k, uint64_t nk, uint64_t km, uint64_t nm,
                                             catena_mem_t* out);
/* catena-lang/tests/cases/matrix/matmul.hex:66-149 (identity views, stdlib/matrix.hex:129-159) */
void program_matmul_right_identity_2x2_via_mem(catena_mem_t a, uint64_t n, uint64_t nn, catena_mem_t* out);
void program_matmul_left_identity_2x2_via_mem(catena_mem_t a, uint64_t n, uint64_t nn, catena_mem_t* out);

/* Integer programs of the reference's tests over `mem` buffers of u64.  catena-lang/tests/cases/reducec/basic.hex:27-58
 * (`sum-u64`: mem.cast.u64, then reducec with u64.add from 0), :60-122 (`dot-u64`: both buffers cast, lengths asserted equal,
 * reducec over the element products), catena-lang/tests/runtime.rs:713-726 (`array-head-u64`: mem.cast.u64, u64.assert-nz,
 * element 0; called directly by catena-lang/smoketest/src/array_head.cpp:37-43).  Arithmetic is modulo 2^64, so the
 * kernels' tree order gives the bits of the sequential fold for every length.  A length mismatch / an empty buffer is
 * CATENA_E_ASSERT. */
void program_sum_u64(catena_mem_t in, uint64_t* out);
void program_dot_u64(catena_mem_t lhs, catena_mem_t rhs, uint64_t* out);
void program_array_head_u64(catena_mem_t in, uint64_t* out);
catena_status_t program_sum_u64_s(catena_mem_t in, uint64_t* out);
catena_status_t program_dot_u64_s(catena_mem_t lhs, catena_mem_t rhs, uint64_t* out);
catena_status_t program_array_head_u64_s(catena_mem_t in, uint64_t* out);

/* elementwise application of a scalar stdlib program over an f32 buffer: the map kernel a
 * `materializec` with that producer lowers to (catena-lang/src/codegen/ops/materializec.rs:36-145).
 * `op` is the hexpr name, e.g. "nn.silu", "math.exp-approx". */
catena_status_t catena_b200_map_f32_s(const char* op, catena_mem_t in, catena_mem_t* out);

/* `gpu.materialize` (catena-lang/stdlib/gpu.hex:39-49, renderer catena-lang/src/codegen/gpu.rs:998-1065): the same map
 * with explicit launch parameters.  The types are the reference's (catena-lang/src/codegen/prelude.rs:13-26); the
 * buffer it materialises has catena_launch_len(params) elements (prelude.rs:59-62), element i being the kernel's
 * value for thread_id = i.  Here the kernel is one of the prebuilt scalar programs applied to the environment buffer
 * `in` at thread_id (arbitrary kernels would need the producer JIT, which this backend does not have); the launch
 * parameters fix only the length — the geometry that runs is the library's, and never enters the result.
 * CATENA_E_ASSERT when `in` holds fewer than catena_launch_len(params) floats. */
typedef struct { uint32_t x, y, z; } catena_dim3_t;
typedef struct { catena_dim3_t grid_dim, block_dim; } catena_launch_params_t;
uint64_t catena_b200_launch_len(catena_launch_params_t params);
catena_status_t catena_b200_gpu_materialize_f32_s(const char* op, catena_launch_params_t params, catena_mem_t in, catena_mem_t* out);

/* ---- generic map: `materializec` with a producer that no prebuilt kernel matches -------------------------------------
 * The reference renders and compiles one kernel per `materializec` — out[i] = producer(env..., i), one thread per element
 * (catena-lang/src/codegen/ops/materializec.rs:36-82).  This backend compiles nothing at run time: the lowering backend
 * (catena-lang_b200/map_program.py, include/catena_b200_map_program.hpp) turns the producer's scalar assignments into a
 * register program — calls inlined, one instruction per primitive of catena-lang/src/codegen/gpu.rs:322-447, `bool.ifc` as
 * a conditional jump, a `reducec` inside the producer as a loop — and one prebuilt kernel interprets it for every index.
 *
 * Registers hold 64 bits: bool 0 / 1, u32 zero-extended, f32 as its bit pattern in the low half (the bitcasts are MOV).
 * Registers 0 .. n_init-1 are preset from `init` (environment scalars, constants, buffer lengths) and read-only;
 * `index_reg` receives i; the element written is the low `elem_bytes` (4 or 8) of `result_reg` after HALT.  LOAD reads
 * buffers[b][register a], bounds-checked.  The program is validated before the launch (opcodes, register and buffer
 * numbers, jump targets, HALT last); a program cannot fault or hang the GPU.  Where the reference's generated code would
 * trap or be undefined — a failed assert, an index past its buffer, a u32 shift by 32 or more, round-to-u32 outside
 * [0, 2^32), division by zero columns, more than 2^22 loop iterations for one element — that element is 0 and the call returns
 * CATENA_E_ASSERT (in non-blocking mode: the next catena_b200_check_device_errors does).  len == 0: {NULL, 0}, no launch.
 * A program of up to 192 instructions and 48 preset registers travels in the kernel parameters; a longer one is copied to
 * the device first, and that copy synchronises the stream even in non-blocking mode (the host arrays are the caller's). */
enum catena_b200_map_op {
    CATENA_MAP_HALT = 0,
    CATENA_MAP_MOV,             /* dst = a */
    CATENA_MAP_JMP,             /* pc = target */
    CATENA_MAP_JZ,              /* if (a == 0) pc = target */
    CATENA_MAP_ASSERT,          /* `assert`: a != 0, else CATENA_E_ASSERT */
    CATENA_MAP_SELECT,          /* dst = a ? b : c   (bool / u32 / u64 / f32 .select) */
    CATENA_MAP_BOOL_NOT, CATENA_MAP_BOOL_AND, CATENA_MAP_BOOL_OR,
    CATENA_MAP_U64_ADD, CATENA_MAP_U64_SUB, CATENA_MAP_U64_MUL,
    CATENA_MAP_U64_DIV, CATENA_MAP_U64_REM,     /* row-major-row / row-major-col (catena-lang/src/codegen/ops/row_major.rs:30-68) */
    CATENA_MAP_U64_EQ, CATENA_MAP_U64_NE, CATENA_MAP_U64_LT, CATENA_MAP_U64_LTE, CATENA_MAP_U64_GT, CATENA_MAP_U64_GTE,
    CATENA_MAP_U64_TO_F32,
    CATENA_MAP_U32_ADD, CATENA_MAP_U32_SUB, CATENA_MAP_U32_MUL, CATENA_MAP_U32_AND, CATENA_MAP_U32_OR, CATENA_MAP_U32_XOR,
    CATENA_MAP_U32_NOT, CATENA_MAP_U32_SHL, CATENA_MAP_U32_SHR,
    CATENA_MAP_U32_EQ, CATENA_MAP_U32_NE, CATENA_MAP_U32_LT, CATENA_MAP_U32_LTE, CATENA_MAP_U32_GT, CATENA_MAP_U32_GTE,
    CATENA_MAP_U32_TO_F32,
    CATENA_MAP_F32_ADD, CATENA_MAP_F32_SUB, CATENA_MAP_F32_MUL, CATENA_MAP_F32_DIV, CATENA_MAP_F32_NEG,
    CATENA_MAP_F32_FMA,         /* dst = fmaf(a, b, c) */
    CATENA_MAP_F32_EQ, CATENA_MAP_F32_NE, CATENA_MAP_F32_LT, CATENA_MAP_F32_LTE, CATENA_MAP_F32_GT, CATENA_MAP_F32_GTE,
    CATENA_MAP_F32_ROUND_TO_U32,
    CATENA_MAP_LOAD_U64, CATENA_MAP_LOAD_F32,   /* `ix`: dst = buffers[b][register a]; b is a buffer number */
    CATENA_MAP_MOV32, CATENA_MAP_SELECT32,      /* MOV / SELECT of a bool, u32 or f32 value: only the low half of the register moves */
    /* an f32.mul whose only reader is the f32.add / f32.sub right behind it, as one instruction: the product and the sum are
     * rounded separately, exactly as the two instructions round them (this is not an fma) */
    CATENA_MAP_F32_MULADD,      /* dst = (a * b) + c */
    CATENA_MAP_F32_MULSUB,      /* dst = (a * b) - c */
    CATENA_MAP_F32_SUBMUL,      /* dst = c - (a * b) */
    CATENA_MAP_OP_COUNT
};
typedef struct {
    uint16_t op, dst, a, b, c, reserved;
    uint32_t target;            /* JMP / JZ: index of the next instruction */
} catena_b200_map_insn_t;
catena_status_t catena_b200_map_program_s(const catena_b200_map_insn_t* code, uint32_t n_insn, const uint64_t* init, uint32_t n_init,
                                          uint32_t n_regs, uint32_t index_reg, uint32_t result_reg, const catena_mem_t* buffers,
                                          uint32_t n_buffers, uint32_t elem_bytes, uint64_t len, catena_mem_t* out);
/* The same for the index range [index0, index0 + len): out[j] = producer(env..., index0 + j).  Elements are independent, so a
 * map shards over GPUs by contiguous index ranges (catena-lang_b200/shard.py: index_ranges); every rank runs the same program. */
catena_status_t catena_b200_map_program_range_s(const catena_b200_map_insn_t* code, uint32_t n_insn, const uint64_t* init, uint32_t n_init,
                                                uint32_t n_regs, uint32_t index_reg, uint32_t result_reg, const catena_mem_t* buffers,
                                                uint32_t n_buffers, uint32_t elem_bytes, uint64_t index0, uint64_t len, catena_mem_t* out);

/* ---- compiled map: the same register program as a kernel of its own -------------------------------------------------
 * What the reference does with nvcc when the Runtime is built (catena-lang/src/codegen/ops/materializec.rs:36-145,
 * catena-lang/src/runtime/artifact.rs:59-80), done without a compiler toolchain: the library writes PTX for the register
 * program (every f32 operation explicitly rounded, so nothing is contracted into an fma; program constants as immediates)
 * and the driver compiles it for the device (cuModuleLoadDataEx).  The compiled kernel gives the bits of the interpreter
 * above and reports the same faults through the same status, at the speed of a prebuilt map kernel.
 * `init_is_const[k] != 0` marks preset register k as a constant of the program (its value is taken from `init` now and
 * baked in); the other presets are environment values (at most 256), read from the `init` of every launch.  NULL = none is
 * constant.  A compiled program may use up to 4096 registers (the interpreter: 256).
 * catena_b200_map_ptx_s only writes the PTX text (`length` receives its size with the terminator; `text` may be NULL to
 * ask for the size) and needs no GPU.  A kernel belongs to the device that was current when it was compiled and may be
 * launched from any host thread bound to that device; releasing it waits for the device to be idle first. */
typedef struct catena_b200_map_kernel catena_b200_map_kernel_t;
catena_status_t catena_b200_map_ptx_s(const catena_b200_map_insn_t* code, uint32_t n_insn, const uint64_t* init, const uint8_t* init_is_const,
                                      uint32_t n_init, uint32_t n_regs, uint32_t index_reg, uint32_t result_reg, uint32_t n_buffers,
                                      uint32_t elem_bytes, char* text, uint64_t capacity, uint64_t* length);
catena_status_t catena_b200_map_compile_s(const catena_b200_map_insn_t* code, uint32_t n_insn, const uint64_t* init, const uint8_t* init_is_const,
                                          uint32_t n_init, uint32_t n_regs, uint32_t index_reg, uint32_t result_reg, uint32_t n_buffers,
                                          uint32_t elem_bytes, catena_b200_map_kernel_t** kernel);
/* out[j] = producer(env..., index0 + j), j < len; `init` / `buffers` as for catena_b200_map_program_range_s */
catena_status_t catena_b200_map_kernel_launch_s(const catena_b200_map_kernel_t* kernel, const uint64_t* init, uint32_t n_init,
                                                const catena_mem_t* buffers, uint32_t n_buffers, uint64_t index0, uint64_t len,
                                                catena_mem_t* out);
void catena_b200_map_kernel_release(catena_b200_map_kernel_t* kernel);

/* ---- programs with no counterpart in the reference (it has no bf16, int8 or attention);
 *      same calling convention; semantics composed from the reference's rules -------------- */
/* C[M,N] = A[M,K] * B, A row-major bf16, B column-major bf16 (stored [N,K]); fp32 accumulation in
 * ascending k (tcgen05 tiles, fixed order, no split-K), bf16 round-to-nearest-even output. */
void program_gemm_bf16_rc(catena_mem_t a, catena_mem_t b_colmajor, uint64_t m, uint64_t n, uint64_t k,
                          catena_mem_t* c);
catena_status_t program_gemm_bf16_rc_s(catena_mem_t a, catena_mem_t b_colmajor, uint64_t m, uint64_t n,
                                       uint64_t k, catena_mem_t* c);
/* int8 x int8 -> int32, same layouts, exact. */
void program_gemm_i8_rc(catena_mem_t a, catena_mem_t b_colmajor, uint64_t m, uint64_t n, uint64_t k,
                        catena_mem_t* c_i32);
catena_status_t program_gemm_i8_rc_s(catena_mem_t a, catena_mem_t b_colmajor, uint64_t m, uint64_t n,
                                     uint64_t k, catena_mem_t* c_i32);
/* Cached-attention decode, one new token: q [B,Hq,D] bf16, k/v cache [B,Hkv,L,D] bf16,
 * o [B,Hq,D] bf16; scale = 1/sqrt(D); softmax per catena-lang/stdlib/nn.hex:93-122 (global max,
 * math.exp-approx, fp32).  D must be 128; Hq a multiple of Hkv with Hq/Hkv <= 8. */
void program_attn_decode_bf16(catena_mem_t q, catena_mem_t k_cache, catena_mem_t v_cache, uint64_t batch,
                              uint64_t hq, uint64_t hkv, uint64_t d, uint64_t kv_len, catena_mem_t* o);
catena_status_t program_attn_decode_bf16_s(catena_mem_t q, catena_mem_t k_cache, catena_mem_t v_cache,
                                           uint64_t batch, uint64_t hq, uint64_t hkv, uint64_t d,
                                           uint64_t kv_len, catena_mem_t* o);

/* ---- launch-level API: caller-owned outputs, used for sharded (multi-GPU) execution ------ */
/* Same kernels as the programs above writing into caller memory; `ldc` is the row pitch of C in
 * elements so a rank can write its column block straight into a full-width matrix. */
catena_status_t catena_b200_gemm_bf16_into(const void* a, const void* b_colmajor, void* c, uint64_t m,
                                           uint64_t n, uint64_t k, uint64_t ldc);
catena_status_t catena_b200_gemm_i8_into(const void* a, const void* b_colmajor, void* c_i32, uint64_t m,
                                         uint64_t n, uint64_t k, uint64_t ldc);
/* GEMM fused with the gather of a row-sharded product: the epilogue stores every output tile to `c` and, with plain
 * stores over NVLink, to the same rows of up to 7 other GPUs' copies of C.  peer_c[i] are peer-mapped DEVICE pointers
 * (catena_b200_ipc_import of the peer's allocation, plus this rank's row offset), 16-byte aligned, same `ldc`.  The
 * stores are complete when the stream has drained; ranks then need one barrier before they read each other's rows.
 * Needs more than 128 rows (the CTA-pair kernel).  No counterpart in the reference. */
catena_status_t catena_b200_gemm_bf16_into_peers(const void* a, const void* b_colmajor, void* c, uint64_t m, uint64_t n,
                                                 uint64_t k, uint64_t ldc, void* const* peer_c, uint32_t n_peers);
catena_status_t catena_b200_gemm_i8_into_peers(const void* a, const void* b_colmajor, void* c_i32, uint64_t m, uint64_t n,
                                               uint64_t k, uint64_t ldc, void* const* peer_c, uint32_t n_peers);
catena_status_t catena_b200_matmul_f32_into(const void* a, const void* b, void* c, uint64_t n, uint64_t m,
                                            uint64_t k);
/* units [unit0, unit1) of the B*Hkv (batch, kv-head) pairs only; q/o are indexed by absolute
 * position, so disjoint unit ranges can be run by different launches (or GPUs) into one output. */
catena_status_t catena_b200_attn_decode_bf16_into(const void* q, const void* k_cache, const void* v_cache,
                                                  void* o, uint64_t batch, uint64_t hq, uint64_t hkv,
                                                  uint64_t d, uint64_t kv_len, uint64_t unit0, uint64_t unit1);
/* The same launch fused with the gather of a (batch, kv-head)-sharded decode: the warps that write a unit's outputs to
 * `o` also store them, with plain stores over NVLink, into up to 7 other GPUs' copies of O at the same offsets.  peer_o[i]
 * are peer-mapped DEVICE pointers to the start of the peer's O (catena_b200_ipc_import).  The stores are complete when
 * the stream has drained; ranks then need one barrier before they read each other's units.  Needs the tcgen05 kernel
 * (kv_len <= 7168, q 16-byte aligned): CATENA_E_UNSUPPORTED otherwise.  No counterpart in the reference. */
catena_status_t catena_b200_attn_decode_bf16_into_peers(const void* q, const void* k_cache, const void* v_cache, void* o,
                                                        uint64_t batch, uint64_t hq, uint64_t hkv, uint64_t d, uint64_t kv_len,
                                                        uint64_t unit0, uint64_t unit1, void* const* peer_o, uint32_t n_peers);
/* elementwise / fold kernels into caller memory (device pointers; `n` in elements) */
catena_status_t catena_b200_map_f32_into(const char* op, const void* in, void* out, uint64_t n);
catena_status_t catena_b200_softmax_f32_into(const void* in, void* out, uint64_t n);
catena_status_t catena_b200_rmsnorm_f32_into(const void* in, void* out, uint64_t n);
/* Sum of n f32 values without any allocation.  No counterpart in the reference (its sum-f32 folds
 * on the host).  For callers that cannot let the library allocate: a host that handed all of HBM to
 * its own arena at start-up, or a latency-critical loop that cannot take the device-wide
 * synchronisation of a cudaMalloc.  `in` (n floats) and `out` (1 float) are caller-owned DEVICE
 * pointers.  The reduction tree's partial sums live in a fixed 256 KiB array inside the library image
 * (resident on every GPU that loads the library), which limits n to 2^30 elements; larger inputs
 * return CATENA_E_TOO_LARGE.  The first call on a device resolves that array's device address: make
 * it before any stream capture begins.  Calls share the array, so calls whose kernels overlap on the
 * GPU race; calls issued on one stream are ordered.  The result is bit-identical to program_sum_f32. */
catena_status_t catena_b200_sum_f32_noalloc(const void* in, uint64_t n, void* out);
/* ---- Llama-style transformer block -----------------------------------------------------------
 * No counterpart in the reference (it has no bf16, attention or rotary embedding): the block is
 * composed from reference programs under the inherited rules — nn.rmsnorm without a gain vector
 * (catena-lang/stdlib/nn.hex:125-182), the matmul cell rule for every projection
 * (catena-lang/stdlib/matrix.hex:236-256), nn.softmax semantics with math.exp-approx for attention
 * (nn.hex:93-122, math.hex:148-199), nn.silu for SwiGLU (nn.hex:2-56), rotary angles from math.powf
 * and math.sin-approx-full (math.hex:91-103, 202-231; cos(x) = sin-approx-full(x + pi/2)).
 * Parity unpinned.  All pointers are DEVICE pointers, all matrices bf16 and row-major with the
 * contraction dimension contiguous ([out_features, in_features]); head_dim is 128.
 *   x = embedding[ids];  q,k,v = rmsnorm(x) W_qkv^T;  rotate q,k;  append k,v to the cache
 *   x2 = x + attention(q, cache) W_o^T;  out = x2 + (silu(g) * u) W_down^T with g,u = rmsnorm(x2) W_gate_up^T */
typedef struct catena_llama_block_t {
    uint64_t hidden, n_heads, n_kv_heads, ffn, vocab;
    uint64_t max_len;        /* rows per (sequence, kv head) of the caches */
    const void* embedding;   /* [vocab, hidden] */
    const void* w_qkv;       /* [(n_heads + 2 n_kv_heads) * 128, hidden]: query heads, key heads, value heads */
    const void* w_o;         /* [hidden, n_heads * 128] */
    const void* w_gate_up;   /* [2 ffn, hidden]: gate rows, then up rows */
    const void* w_down;      /* [hidden, ffn] */
    float rope_base;         /* e.g. 10000 */
} catena_llama_block_t;
/* bytes of scratch the two calls below need for `tokens` tokens in flight (batch * seq, or batch) */
uint64_t catena_b200_llama_workspace_bytes(const catena_llama_block_t* blk, uint64_t tokens);
/* Prefill: ids [batch * seq] int32 (sequence-major), positions 0..seq-1, causal attention; fills rows 0..seq-1 of
 * k_cache / v_cache [batch, n_kv_heads, max_len, 128] and writes out [batch * seq, hidden].  The workspace is
 * caller-owned, 256-byte aligned.  An id outside the vocabulary gives CATENA_E_ASSERT (never a trap). */
catena_status_t catena_b200_llama_prefill(const catena_llama_block_t* blk, const int32_t* ids, uint64_t batch, uint64_t seq,
                                          void* k_cache, void* v_cache, void* out, void* workspace, uint64_t workspace_bytes);
/* One decode step: ids [batch], every sequence at position `pos` (its cache rows 0..pos-1 are filled); appends
 * row `pos` and writes out [batch, hidden].  Cache rows past the visible length are never read. */
catena_status_t catena_b200_llama_decode(const catena_llama_block_t* blk, const int32_t* ids, uint64_t batch, uint64_t pos,
                                         void* k_cache, void* v_cache, void* out, void* workspace, uint64_t workspace_bytes);
/* The block's operators one by one (same kernels), for parity tests and other compositions. */
catena_status_t catena_b200_embed_bf16_into(const void* table, const int32_t* ids, void* out, uint64_t tokens, uint64_t hidden,
                                            uint64_t vocab);
catena_status_t catena_b200_rmsnorm_rows_bf16_into(const void* x, void* y, uint64_t rows, uint64_t hidden);
/* qkv [tokens, (n_heads + 2 n_kv_heads) * 128]; token t is sequence t / seq at position pos0 + t % seq; writes the rotated
 * queries to q_out [tokens, n_heads, 128] and row `position` of the caches [batch, n_kv_heads, cap, 128] */
catena_status_t catena_b200_rope_append_bf16_into(const void* qkv, void* q_out, void* k_cache, void* v_cache, uint64_t tokens,
                                                  uint64_t seq, uint64_t pos0, uint64_t n_heads, uint64_t n_kv_heads, uint64_t cap,
                                                  float rope_base);
/* causal attention of q [batch * seq, n_heads, 128] over cache rows 0..s of each sequence; out [batch * seq, n_heads * 128] */
catena_status_t catena_b200_attn_prefill_bf16_into(const void* q, const void* k_cache, const void* v_cache, void* out, uint64_t batch,
                                                   uint64_t seq, uint64_t n_heads, uint64_t n_kv_heads, uint64_t cap);
/* catena_b200_attn_decode_bf16_into on caches whose units own kv_cap rows of which the first kv_len are visible */
catena_status_t catena_b200_attn_decode_bf16_cache_into(const void* q, const void* k_cache, const void* v_cache, void* o, uint64_t batch,
                                                        uint64_t hq, uint64_t hkv, uint64_t d, uint64_t kv_len, uint64_t kv_cap);
/* gate_up [tokens, 2 ffn] -> out [tokens, ffn] = silu(gate) * up */
catena_status_t catena_b200_swiglu_bf16_into(const void* gate_up, void* out, uint64_t tokens, uint64_t ffn);
/* out [m, ffn] = silu(x w_gate^T) * (x w_up^T), w_gate_up [2 ffn, k] (gate rows, then up rows); bit-identical to
 * catena_b200_linear_bf16_into followed by catena_b200_swiglu_bf16_into.  m <= 16 is one launch and `scratch` is
 * unused; larger m needs scratch [m, 2 ffn] bf16 for the projection. */
catena_status_t catena_b200_linear_swiglu_bf16_into(const void* x, const void* w_gate_up, void* scratch, void* out, uint64_t m,
                                                    uint64_t ffn, uint64_t k);
/* out = x + y over n bf16 elements (n a multiple of 8; out may alias x or y) */
catena_status_t catena_b200_add_bf16_into(const void* x, const void* y, void* out, uint64_t n);
/* y [m, n] = x [m, k] w[n, k]^T (+ residual [m, n], added after the product is rounded to bf16).  m <= 16 runs a kernel
 * that streams w once (HBM-bound), larger m the tcgen05 GEMM. */
catena_status_t catena_b200_linear_bf16_into(const void* x, const void* w, const void* residual, void* y, uint64_t m, uint64_t n,
                                             uint64_t k);

/* test hook: cap the persistent grid of the tensor-core GEMM (0 = one CTA per SM); results must not
 * change with it.  No counterpart in the reference. */
void catena_b200_debug_set_cta_limit(int limit);
/* test hook: 1 = run tensor-core GEMMs on the CTA-pair (cta_group::2) kernel, 0 = single-CTA kernel;
 * both give bit-identical results.  No counterpart in the reference. */
void catena_b200_debug_set_gemm_pair(int on);
/* test hook: 1 = decode attention on the tcgen05 kernel, 0 = on the mma.sync kernel (same semantics).
 * No counterpart in the reference. */
void catena_b200_debug_set_attn_tc(int on);
/* test hook: which kernels a decode step of the Llama-style block uses, as bits (a negative value: back to the default).
 * 1 = everything after the attention (o projection, norm, gate/up + SwiGLU, down projection) as one persistent kernel with
 * grid barriers; 2 = everything before it (embedding, norm, q/k/v projection, rotation, cache append) likewise — both measured
 * slower than launches chained by programmatic dependent launch; 4 = rotation and cache append in the epilogue of the q/k/v
 * projection instead of a launch of their own.  Every combination gives bit-identical results.  No counterpart in the
 * reference. */
void catena_b200_debug_set_decode_fused(int mode);
/* test hook: 1 = prefill attention on the tcgen05 kernel (the default), 0 = on the mma.sync kernel (same semantics).
 * No counterpart in the reference. */
void catena_b200_debug_set_prefill_tc(int on);
/* test hook: geometry of the calling thread's last decode-attention launch: out[0] = kernel (0 mma.sync, 1 tcgen05),
 * out[1] = clusters of 8 CTAs that can be resident at once, out[2] = clusters launched, out[3] = dynamic shared
 * memory per CTA in bytes.  No counterpart in the reference. */
void catena_b200_debug_attn_last_launch(uint32_t out[4]);
/* test hook: the prefill attention kernel takes reciprocals by a short correctly-rounded sequence for arguments in
 * [0.5, 2^100); this compares that sequence with the IEEE reciprocal for EVERY float of the range on the device:
 * out[0] = values compared, out[1] = mismatches (must be 0).  No counterpart in the reference. */
catena_status_t catena_b200_debug_rcp_check(uint64_t out[2]);
/* test hook: the kernels that use sm_100's packed f32x2 arithmetic write a product as fma.rn.f32x2(a, b, -0) with the -0 hidden
 * from the assembler, because a packed mul is merged with the packed add behind it into one fma (which rounds once, against
 * the contract of catena-lang/src/runtime/artifact.rs:59-80).  Over pseudo-random operands on the device: out[0] = pairs
 * compared, out[1] = pairs where the fma form followed by a packed add differs from __fadd_rn(c, __fmul_rn(a, b)) (must be
 * 0), out[2] = pairs where a packed mul followed by a packed add differs (not 0 while the assembler merges them).  No
 * counterpart in the reference. */
catena_status_t catena_b200_debug_packed_f32x2_check(uint64_t out[3]);
/* test hooks for the give-up path of the bounded device-side waits (catena-lang/src/codegen/prelude.rs:38-55 traps
 * instead; here a wait that runs out makes the kernel drain its copies, free its tensor memory and return, and the host
 * reports CATENA_E_TIMEOUT).  set_wait_limit_ns: limit of every wait in the tcgen05 GEMM (CTA-pair kernel) and the
 * tcgen05 decode attention launched from now on (0 = the default, one second).  stall_next: the NEXT launch of that
 * family leaves one hand-over out on purpose — family 1 (CTA-pair GEMM): the TMA producers stop before k-block
 * `value - 1` of their first tile; family 2 (tcgen05 decode attention): item 0 never publishes its chunk maxima
 * (`value` non-zero).  Nothing faults or spins without bound: the waiting roles give up after the limit.  The output of
 * such a launch is undefined; the library stays usable.  No counterpart in the reference. */
void catena_b200_debug_set_wait_limit_ns(uint64_t ns);
void catena_b200_debug_stall_next(int family, uint32_t value);
/* after non-blocking launches: reports (and clears) a device-side bounded-wait expiry or what a map program ran into */
catena_status_t catena_b200_check_device_errors(void);

#ifdef __cplusplus
}
#endif
#endif /* CATENA_B200_H */
