// Shared declarations of the kernel library: status handling, per-thread runtime state,
// launch bookkeeping.  Internal — the public surface is include/catena_b200.h.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/catena_b200.h"

namespace catena {

// Per-host-thread library state.  The generated code of the reference uses the process-global
// current device and the default stream (catena-lang/doc/CODEGEN.md:164-166); here both are
// explicit so one process per GPU (or one thread per GPU) can drive the library.
// Per-device tables (pools, scratch, error words) hold this many devices; catena_b200_init refuses larger indices.
constexpr int kMaxDevices = 16;

struct ThreadState {
    int device = -1;           // -1: not initialised
    cudaStream_t stream = 0;   // legacy default stream unless set
    int blocking = 1;          // synchronise after each entry point
    catena_status_t last = CATENA_OK;
    int sm_count = 0;
    int cc_major = 0;
};

ThreadState& tls();

// Makes sure a device is bound (lazy init on device 0).  Returns CATENA_OK or an error.
catena_status_t ensure_device();

// Records a failure: remembers it for catena_b200_last_status and prints one line.
catena_status_t fail(catena_status_t s, const char* what);
catena_status_t fail_cuda(cudaError_t e, const char* what);

void count_launch(uint64_t n = 1);

// Test knobs of the bounded device-side waits (process-wide).  The limit applies to tcgen05 GEMM and decode-attention
// launches made after it is set; a stall request is taken (and cleared) by the next launch of that kernel family:
// 1 = CTA-pair GEMM (value = k-block + 1 at which the TMA producers stop), 2 = tcgen05 decode attention.
uint64_t debug_wait_limit_ns();
uint32_t debug_take_stall(int family);

// Pool allocator (mem.cu).
catena_status_t pool_alloc(uint64_t bytes, void** out);
catena_status_t pool_free(void* p);

// After enqueuing: check launch error, optionally synchronise.
catena_status_t finish(const char* what);

#define CATENA_CUDA(expr)                                                   \
    do {                                                                    \
        cudaError_t _e = (expr);                                            \
        if (_e != cudaSuccess) return ::catena::fail_cuda(_e, #expr);       \
    } while (0)

#define CATENA_TRY(expr)                                                    \
    do {                                                                    \
        catena_status_t _s = (expr);                                        \
        if (_s != CATENA_OK) return _s;                                     \
    } while (0)

static inline uint64_t ceil_div_u64(uint64_t a, uint64_t b) { return (a + b - 1) / b; }

// ---- launchers implemented by the kernel files (all enqueue on tls().stream) ------------
// gemm_f32.cu
catena_status_t launch_matmul_f32(const float* a, const float* b, float* c, uint64_t n, uint64_t m,
                                  uint64_t k);
catena_status_t launch_identity_matmul_f32(const float* a, float* c, uint64_t n, int identity_on_left);
catena_status_t packed_f32x2_check(uint64_t out[3]);
// gemm_tc.cu
catena_status_t launch_gemm_tc(const void* a, const void* b, void* c, uint64_t m, uint64_t n, uint64_t k,
                               uint64_t ldc, int is_i8);
// Where the epilogue of a q/k/v projection puts its output instead of a [tokens, (hq + 2 hkv) * 128] matrix: rotated
// queries into q_out [tokens, hq, 128], rotated keys and plain values into the caches [batch, hkv, cap, 128] at position
// pos0 + (token % seq); `table` holds (cos, sin) of the `seq` positions, [seq][64].
struct GemmRopeOut {
    const float2* table;
    void* q_out;
    void* k_cache;
    void* v_cache;
    uint32_t seq, pos0, hq, hkv, cap;
};
catena_status_t launch_gemm_tc_rope(const void* a, const void* b, uint64_t m, uint64_t n, uint64_t k, const GemmRopeOut& rope);
catena_status_t launch_gemm_tc_swiglu(const void* x, const void* w, void* act, uint64_t m, uint64_t ffn, uint64_t k);
bool gemm_tc_fuses_residual(uint64_t m);
catena_status_t launch_gemm_tc_residual(const void* a, const void* b, void* c, uint64_t m, uint64_t n, uint64_t k, uint64_t ldc,
                                        const void* residual);
catena_status_t launch_gemm_tc_peers(const void* a, const void* b, void* c, uint64_t m, uint64_t n, uint64_t k, uint64_t ldc,
                                     int is_i8, void* const* peer_c, uint32_t n_peers);
catena_status_t gemm_tc_check_errors();
void gemm_tc_set_cta_limit(int limit);
void gemm_tc_set_pair_mode(int on);
void attn_set_cluster_limit(int limit);
void attn_set_tc_mode(int on);
void attn_last_launch(uint32_t out[4]);
catena_status_t attn_prefill_rcp_check(uint64_t out[2]);
extern thread_local uint32_t g_attn_last_launch[4];
// attn_decode.cu
// Ranges of memory that the kernels queued after a decode-attention launch will stream: the tcgen05 kernel prefetches
// them into L2 from an idle warp while it runs (a hint; results never depend on it).
struct AttnPrefetch {
    const void* ptr[4];
    uint64_t bytes[4];
    uint32_t n;
    uint32_t pace_ns;
};
catena_status_t launch_attn_decode(const void* q, const void* kc, const void* vc, void* o, uint64_t batch,
                                   uint64_t hq, uint64_t hkv, uint64_t d, uint64_t kv_len, uint64_t kv_cap,
                                   uint64_t unit0, uint64_t unit1, void* const* peer_o = nullptr, uint32_t n_peers = 0,
                                   const AttnPrefetch* prefetch = nullptr);
catena_status_t attn_check_errors();
// llama_decode_fused.cu: the part of a decode step after its attention as one persistent kernel
int decode_fused_mode();      // bit 0: the tail kernel, bit 1: the head kernel, bit 2: rotation + cache append in the q/k/v projection's epilogue
void decode_fused_set_mode(int mode);
bool decode_tail_supported(uint64_t m, uint64_t hidden, uint64_t ko, uint64_t ffn);
catena_status_t launch_decode_tail(const void* att, const void* x, const void* w_o, const void* w_gate_up, const void* w_down, void* x2,
                                   void* act, void* out, uint64_t m, uint64_t hidden, uint64_t ko, uint64_t ffn);
bool decode_head_supported(uint64_t m, uint64_t hidden, uint64_t hq, uint64_t hkv);
catena_status_t launch_decode_head(const void* table, const int32_t* ids, const void* w_qkv, const float* inv_freq, uint32_t* bad, void* x,
                                   void* qkv, void* q_out, void* k_cache, void* v_cache, uint64_t m, uint64_t hidden, uint64_t vocab,
                                   uint64_t hq, uint64_t hkv, uint64_t cap, uint64_t pos);
catena_status_t decode_fused_check_errors();
// map_program.cu
catena_status_t map_program_check_errors();
catena_status_t map_program_validate(const catena_b200_map_insn_t* code, uint32_t n_insn, uint32_t n_init, uint32_t n_regs, uint32_t index_reg,
                                     uint32_t result_reg, uint32_t n_buffers, uint32_t max_regs);
catena_status_t map_program_error_word(uint32_t** err);     // the device error word the interpreter and the compiled kernels share
// map_reduce.cu
enum ReduceKind { RED_SUM = 0, RED_MAX = 1, RED_SUMSQ = 2 };
int map_op_from_name(const char* name);  // -1 if unknown
catena_status_t launch_map_unary(int op, const float* in, float* out, uint64_t n);
catena_status_t reduce_f32(int kind, const float* in, uint64_t n, float* host_out);
catena_status_t argmax_f32(const float* in, uint64_t n, uint64_t* host_out);
catena_status_t launch_softmax(const float* in, float* out, uint64_t n);
catena_status_t launch_rmsnorm(const float* in, float* out, uint64_t n);
catena_status_t launch_broadcast(float v, float* out, uint64_t n);
catena_status_t launch_arange(float* out, uint64_t n);
catena_status_t launch_slice(const float* in, uint64_t start, float* out, uint64_t n);
catena_status_t launch_concat(const float* l, uint64_t nl, const float* r, uint64_t nr, float* out);

}  // namespace catena
