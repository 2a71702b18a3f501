// One decode step of the Llama-style block in THREE launches instead of eight: two persistent kernels around the
// cached-attention kernel.
//   decode_head_kernel   x = embedding[ids];  n = rmsnorm(x) (every CTA, into shared memory);  qkv = n W_qkv^T     (phase 1)
//                        rotate q and k, append k and v to the caches at this step's position                      (phase 2)
//   (attention)          attn_decode_tc.cu
//   decode_tail_kernel   x2  = x + att W_o^T                                                                        (phase 1)
//                        n   = rmsnorm(x2) (every CTA, into shared memory);  act = silu(n W_gate^T) * (n W_up^T)    (phase 2)
//                        out = x2 + act W_down^T                                                                    (phase 3)
// The grid stays resident (cooperative launch, two CTAs per SM) and crosses its phase boundaries at a grid barrier; before a
// CTA waits at a barrier it has already issued the loads of its first batch of the NEXT phase's weights (weights do not
// depend on activations).
//
// MEASURED, and why this path is NOT the default: on the 2048-hidden block (4 tokens, 2048 - 2175 cache rows) a decode step
// takes 62.8 us as eight launches chained by programmatic dependent launch, 67.9 us with the tail kernel, 67.5 us with the
// head kernel, 71.8 us with both.  A grid barrier under a full HBM stream (fence, 296 arrivals on one word, acquire polls
// behind 32 KB of prefetched weights per CTA) plus the norm that every CTA then repeats costs about 5 us per boundary;
// a programmatic launch boundary costs about 3.5 us, and a cooperative launch cannot overlap its predecessor's tail at
// all.  The projections themselves are latency-bound at this size (8 - 67 MB over 296 CTAs is one to four batches per
// warp), which neither form changes.  The kernels stay selectable (CATENA_B200_DECODE_FUSED=1 tail, 2 head, 3 both, or the
// test hook) because they give the eight-launch path's bits with different kernels, which the tests use as a cross-check.
//
// Arithmetic: the projections are skinny.cuh's (the stand-alone skinny GEMM uses the same code), the norm reproduces the
// summation tree of rmsnorm_rows_kernel (llama.cu) — thread t of a 256-thread CTA adds the squares of its elements in
// ascending order, xor butterfly per warp, warps added in ascending order — with 64 threads per row playing the 256, the
// rotation is rope_append_small_kernel's: outputs and caches are bit-identical to the separate launches (tested).
//
// Grid barrier: a counter in global memory that only grows; the host passes every launch the count at which it starts
// (`base`), and barrier b of the launch waits for base + (b + 1) * gridDim.x.  Arrivals publish with a fence before the
// atomic increment, the poll is an acquire load; the wait is bounded (the debug wait limit, one second by default): on
// expiry the CTA records an error code and leaves, and the host resets the counter.  Activations written in one phase are
// read in the next with L2-coherent loads.
#include <cuda_bf16.h>

#include "catena_math.cuh"
#include "common.cuh"
#include "skinny.cuh"

namespace catena {

namespace llama {

constexpr uint32_t kFusedEpsBits = 0x3727C5ACu;      // 1e-5, catena-lang/stdlib/nn.hex:154-182

struct DecodeTail {
    const __nv_bfloat16* att;        // [M, KO]   attention output
    const __nv_bfloat16* x;          // [M, H]    residual stream
    const __nv_bfloat16* w_o;        // [H, KO]
    const __nv_bfloat16* w_gate_up;  // [2F, H]
    const __nv_bfloat16* w_down;     // [H, F]
    __nv_bfloat16* x2;               // [M, H]
    __nv_bfloat16* act;              // [M, F]
    __nv_bfloat16* out;              // [M, H]
    uint32_t M, H, KO, F;
    uint32_t* barrier;               // grid-barrier counter (monotonic)
    uint32_t base;                   // its value when this launch starts
    uint32_t* err;
    uint64_t wait_ns;
};
struct DecodeHead {
    const __nv_bfloat16* table;      // [vocab, H] embedding
    const int32_t* ids;              // [M]
    const __nv_bfloat16* w_qkv;      // [(Hq + 2 Hkv) * 128, H]
    const float* inv_freq;           // [64] base^(-2i/128)
    __nv_bfloat16* x;                // [M, H]    residual stream (written)
    __nv_bfloat16* qkv;              // [M, (Hq + 2 Hkv) * 128] scratch
    __nv_bfloat16* q_out;            // [M, Hq, 128]
    __nv_bfloat16* k_cache;          // [M, Hkv, cap, 128]
    __nv_bfloat16* v_cache;
    uint32_t M, H, Hq, Hkv, cap, pos, vocab;
    uint32_t* bad;                   // set when an id lies outside the table
    uint32_t* barrier;
    uint32_t base;
    uint32_t* err;
    uint64_t wait_ns;
};

__device__ __forceinline__ uint64_t fused_globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// All threads of all CTAs call this; false when the wait ran out (or another CTA already gave up).
__device__ __forceinline__ bool grid_barrier(uint32_t* counter, uint32_t target, uint32_t* err, uint64_t wait_ns, uint32_t* flag_smem) {
    __syncthreads();                                   // this CTA's stores of the phase are issued
    if (threadIdx.x == 0) {
        __threadfence();                               // ... and ordered before the arrival
        atomicAdd(counter, 1u);
        uint32_t ok = 1, seen;
        const uint64_t t0 = fused_globaltimer_ns();
        uint32_t spins = 0;
        while (true) {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
            if ((int32_t)(seen - target) >= 0) break;
            if ((++spins & 31u) == 0) {
                uint32_t e;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(e) : "l"(err) : "memory");
                if (e != 0 || fused_globaltimer_ns() - t0 > wait_ns) {
                    atomicCAS(err, 0u, 7u);
                    ok = 0;
                    break;
                }
            }
        }
        *flag_smem = ok;
    }
    __syncthreads();
    return *flag_smem != 0;
}

// n[r, :] = src_r / sqrt~(mean(src_r^2) + eps) for the M rows, into shared memory [M][H].  Row r is x2 + r H (written by
// other CTAs in the previous phase: L2-coherent loads), or, with `ids`, row ids[r] of the embedding table x2 — an id outside
// the table sets *bad and reads row 0 — which is also copied to x_out by CTA 0.  Four rows at a time, 64 threads (two warps)
// per row: lane l of the row's warp tw stands for the threads vw * 32 + l, vw = 4 tw .. 4 tw + 3, of a 256-thread CTA
// working on that row alone.
__device__ __forceinline__ void norm_rows_to_shared(const __nv_bfloat16* x2, uint32_t M, uint32_t H, __nv_bfloat16* n_smem, float (*wsum)[8],
                                                    float* rms_s, const int32_t* ids = nullptr, uint32_t vocab = 0, uint32_t* bad = nullptr,
                                                    __nv_bfloat16* x_out = nullptr) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t team = warp >> 1, tw = warp & 1u;                 // row team of this warp, its half of the virtual warps
    const uint32_t h8 = H / 8;
    for (uint32_t r0 = 0; r0 < M; r0 += 4) {
        const uint32_t row = r0 + team;
        size_t src_row = row;
        if (ids && row < M) {
            const int32_t id = ids[row];
            if (id < 0 || (uint32_t)id >= vocab) {
                if (lane == 0 && tw == 0) atomicExch(bad, 1u);
                src_row = 0;
            } else {
                src_row = (size_t)id;
            }
        }
        const uint4* xr = reinterpret_cast<const uint4*>(x2 + src_row * H);
        if (row < M) {
#pragma unroll
            for (uint32_t q = 0; q < 4; ++q) {
                const uint32_t vt = (4 * tw + q) * 32 + lane;       // the thread of rmsnorm_rows_kernel this lane stands for
                float acc = 0.0f;
                for (uint32_t i = vt; i < h8; i += 256) {
                    uint4 v;
                    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(xr + i));
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float a = __uint_as_float(w[e] << 16), b = __uint_as_float(w[e] & 0xFFFF0000u);
                        acc = cmath::add(acc, cmath::mul(a, a));
                        acc = cmath::add(acc, cmath::mul(b, b));
                    }
                }
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) acc = cmath::add(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, off));
                if (lane == 0) wsum[team][4 * tw + q] = acc;
            }
        }
        __syncthreads();
        if (row < M && tw == 0 && lane == 0) {
            float s = wsum[team][0];
            for (int w = 1; w < 8; ++w) s = cmath::add(s, wsum[team][w]);
            const float mean = cmath::div(s, cmath::u64_to_f32(H));
            rms_s[team] = cmath::sqrt_newton(cmath::add(mean, cmath::from_bits(kFusedEpsBits)));
        }
        __syncthreads();
        if (row < M) {
            const float rms = rms_s[team];
            uint4* nr = reinterpret_cast<uint4*>(n_smem + (size_t)row * H);
            for (uint32_t i = tw * 32 + lane; i < h8; i += 64) {
                uint4 v;
                asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(xr + i));
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float a = cmath::div(__uint_as_float(w[e] << 16), rms), b = cmath::div(__uint_as_float(w[e] & 0xFFFF0000u), rms);
                    o[e] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(a)) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(b)) << 16);
                }
                nr[i] = make_uint4(o[0], o[1], o[2], o[3]);
                if (x_out && blockIdx.x == 0) reinterpret_cast<uint4*>(x_out + (size_t)row * H)[i] = v;
            }
        }
        __syncthreads();
    }
}

// gridDim.x resident CTAs of 256 threads (cooperative launch); dynamic shared memory: M * H bf16 for the normalised rows.
__global__ void __launch_bounds__(256, 2) decode_tail_kernel(const DecodeTail p) {
    __shared__ float part[8][16][8];
    __shared__ float wsum[4][8];
    __shared__ float rms_s[4];
    __shared__ uint32_t barrier_ok;
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    __nv_bfloat16* n_smem = reinterpret_cast<__nv_bfloat16*>(dyn_smem);

    const SkinnyJob o_proj = {p.att, p.w_o, p.x, p.x2, p.M, p.H, p.KO, 0u};
    const SkinnyJob gate_up = {n_smem, p.w_gate_up, nullptr, p.act, p.M, 2 * p.F, p.H, p.F};
    const SkinnyJob down = {p.act, p.w_down, p.x2, p.out, p.M, p.H, p.F, 0u};
    const uint32_t base = p.base;
    uint4 cur[kSkinnyUnroll];

    {   // ---- phase 1: the o projection and the first residual
        const SkinnySchedule sc(o_proj, blockIdx.x, gridDim.x);
        if (sc.steps > 0) skinny_load_w(o_proj, sc, 0, cur);
        asm volatile("griddepcontrol.wait;" ::: "memory");     // the attention kernel's output (no-op without the launch attribute)
        skinny_run<A_READONLY>(o_proj, sc, part, cur);
    }
    {   // ---- phase 2: norm, gate / up projection, SwiGLU
        const SkinnySchedule sc(gate_up, blockIdx.x, gridDim.x);
        if (sc.steps > 0) skinny_load_w(gate_up, sc, 0, cur);  // in flight across the barrier
        if (!grid_barrier(p.barrier, base + gridDim.x, p.err, p.wait_ns, &barrier_ok)) return;
        norm_rows_to_shared(p.x2, p.M, p.H, n_smem, wsum, rms_s);
        skinny_run<A_SHARED>(gate_up, sc, part, cur);
    }
    {   // ---- phase 3: the down projection and the second residual
        const SkinnySchedule sc(down, blockIdx.x, gridDim.x);
        if (sc.steps > 0) skinny_load_w(down, sc, 0, cur);
        if (!grid_barrier(p.barrier, base + 2u * gridDim.x, p.err, p.wait_ns, &barrier_ok)) return;
        skinny_run<A_COHERENT>(down, sc, part, cur);
    }
}

// Rotary embedding + cache append of one decode step (every token is its own sequence at position `pos`): the arithmetic of
// rope_append_small_kernel (llama.cu), one (token, head, pair) per thread, reading the projection written in phase 1.
__device__ __forceinline__ float head_load_bf16(const __nv_bfloat16* p) {
    uint16_t h;
    asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(h) : "l"(p));
    return __uint_as_float((uint32_t)h << 16);
}
__global__ void __launch_bounds__(256, 2) decode_head_kernel(const DecodeHead p) {
    __shared__ float part[8][16][8];
    __shared__ float wsum[4][8];
    __shared__ float rms_s[4];
    __shared__ uint32_t barrier_ok;
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    __nv_bfloat16* n_smem = reinterpret_cast<__nv_bfloat16*>(dyn_smem);
    const uint32_t heads = p.Hq + 2 * p.Hkv;
    const SkinnyJob qkv = {n_smem, p.w_qkv, nullptr, p.qkv, p.M, heads * 128u, p.H, 0u};
    uint4 cur[kSkinnyUnroll];
    {   // ---- phase 1: embedding, norm, q/k/v projection
        const SkinnySchedule sc(qkv, blockIdx.x, gridDim.x);
        if (sc.steps > 0) skinny_load_w(qkv, sc, 0, cur);
        asm volatile("griddepcontrol.wait;" ::: "memory");
        norm_rows_to_shared(p.table, p.M, p.H, n_smem, wsum, rms_s, p.ids, p.vocab, p.bad, p.x);
        skinny_run<A_SHARED>(qkv, sc, part, cur);
    }
    if (!grid_barrier(p.barrier, p.base + gridDim.x, p.err, p.wait_ns, &barrier_ok)) return;
    // ---- phase 2: rotate q and k, append k and v at position p.pos
    const uint64_t total = (uint64_t)p.M * heads * 64;
    for (uint64_t idx = (uint64_t)blockIdx.x * 256 + threadIdx.x; idx < total; idx += (uint64_t)gridDim.x * 256) {
        const uint32_t i = (uint32_t)(idx % 64);
        const uint32_t head = (uint32_t)((idx / 64) % heads);
        const uint32_t t = (uint32_t)(idx / (64ull * heads));
        const __nv_bfloat16* src = p.qkv + ((size_t)t * heads + head) * 128;
        const float x1 = head_load_bf16(src + i), x2 = head_load_bf16(src + i + 64);
        if (head >= p.Hq + p.Hkv) {   // value head: plain copy
            __nv_bfloat16* dst = p.v_cache + (((size_t)t * p.Hkv + (head - p.Hq - p.Hkv)) * p.cap + p.pos) * 128;
            dst[i] = __float2bfloat16_rn(x1);
            dst[i + 64] = __float2bfloat16_rn(x2);
            continue;
        }
        const float angle = cmath::mul(cmath::u32_to_f32(p.pos), p.inv_freq[i]);
        const float cs = cmath::sin_full(cmath::add(angle, cmath::from_bits(0x3FC90FDBu))), sn = cmath::sin_full(angle);
        __nv_bfloat16* dst = head < p.Hq ? p.q_out + ((size_t)t * p.Hq + head) * 128
                                         : p.k_cache + (((size_t)t * p.Hkv + (head - p.Hq)) * p.cap + p.pos) * 128;
        dst[i] = __float2bfloat16_rn(cmath::sub(cmath::mul(x1, cs), cmath::mul(x2, sn)));
        dst[i + 64] = __float2bfloat16_rn(cmath::add(cmath::mul(x2, cs), cmath::mul(x1, sn)));
    }
}

}  // namespace llama

// ---- host side --------------------------------------------------------------------------------------------------------
struct FusedState {
    uint32_t* counter = nullptr;   // grid-barrier counter
    uint32_t* err = nullptr;       // device error word
    uint32_t* err_host = nullptr;  // pinned
    uint32_t count = 0;            // value of the counter once everything enqueued so far has run
    int grid[2] = {0, 0};          // resident CTAs of the tail / head kernel for the shared memory asked for last
    size_t grid_smem[2] = {~(size_t)0, ~(size_t)0};
};
static thread_local FusedState g_fused[kMaxDevices];

constexpr int kDecodeModeDefault = 4;   // rotation + cache append in the q/k/v projection's epilogue: 60.8 against 63.1 us per step
static int g_decode_fused_mode = -1;
// The persistent kernels are off by default (see the measurements at the top); CATENA_B200_DECODE_FUSED=0..7 (read once) or the
// test hook selects the bits: 1 tail kernel, 2 head kernel, 4 rotation + cache append in the q/k/v projection's epilogue (default).
int decode_fused_mode() {
    if (g_decode_fused_mode < 0) {
        const char* e = getenv("CATENA_B200_DECODE_FUSED");
        g_decode_fused_mode = (e && e[0] >= '0' && e[0] <= '7' && e[1] == 0) ? e[0] - '0' : kDecodeModeDefault;
    }
    return g_decode_fused_mode;
}
void decode_fused_set_mode(int mode) { g_decode_fused_mode = mode < 0 ? -1 : (mode & 7); }   // negative: back to the default

// True when launch_decode_tail takes this shape.
bool decode_tail_supported(uint64_t m, uint64_t hidden, uint64_t ko, uint64_t ffn) {
    return m >= 1 && m <= 16 && hidden % 8 == 0 && ko % 8 == 0 && ffn % 8 == 0 && hidden <= 0x3FFFFFFFull && ko <= 0x7FFFFFFFull &&
           ffn <= 0x3FFFFFFFull && m * hidden * 2 <= 160 * 1024;
}

// Counter, error word and grid of kernel `which` (0 tail, 1 head) for `smem` bytes of dynamic shared memory; reserves
// `barriers` grid barriers on the counter and returns the count at which the launch starts.
static catena_status_t fused_prepare(int which, size_t smem, uint32_t barriers, FusedState** out, uint32_t* base) {
    FusedState& st = g_fused[tls().device];
    if (!st.counter) {
        CATENA_CUDA(cudaMalloc(&st.counter, 2 * sizeof(uint32_t)));
        CATENA_CUDA(cudaMemset(st.counter, 0, 2 * sizeof(uint32_t)));
        st.err = st.counter + 1;
        CATENA_CUDA(cudaMallocHost(&st.err_host, sizeof(uint32_t)));
        *st.err_host = 0;
    }
    if (st.grid_smem[which] != smem) {
        int per_sm = 0;
        if (which == 0) {
            CATENA_CUDA(cudaFuncSetAttribute(llama::decode_tail_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            CATENA_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, llama::decode_tail_kernel, 256, smem));
        } else {
            CATENA_CUDA(cudaFuncSetAttribute(llama::decode_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            CATENA_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, llama::decode_head_kernel, 256, smem));
        }
        const int sms = tls().sm_count > 0 ? tls().sm_count : 148;
        if (per_sm < 1) return fail(CATENA_E_CUDA, "decode step: the fused kernel cannot be resident");
        st.grid[which] = (per_sm > 2 ? 2 : per_sm) * sms;
        st.grid_smem[which] = smem;
    }
    // the counter only grows: start again from zero (stream-ordered) well before it wraps
    if (st.count > 0x7F000000u) {
        CATENA_CUDA(cudaMemsetAsync(st.counter, 0, sizeof(uint32_t), tls().stream));
        st.count = 0;
    }
    *base = st.count;
    st.count += barriers * (uint32_t)st.grid[which];
    *out = &st;
    return CATENA_OK;
}

// x2 = x + att w_o^T; act = silu(rmsnorm(x2) w_gate^T) * (rmsnorm(x2) w_up^T); out = x2 + act w_down^T, one launch.
catena_status_t launch_decode_tail(const void* att, const void* x, const void* w_o, const void* w_gate_up, const void* w_down, void* x2,
                                   void* act, void* out, uint64_t m, uint64_t hidden, uint64_t ko, uint64_t ffn) {
    CATENA_TRY(ensure_device());
    if (!decode_tail_supported(m, hidden, ko, ffn)) return fail(CATENA_E_UNSUPPORTED, "decode tail: shape");
    if (((uintptr_t)att | (uintptr_t)x | (uintptr_t)w_o | (uintptr_t)w_gate_up | (uintptr_t)w_down | (uintptr_t)x2 | (uintptr_t)act | (uintptr_t)out) & 15)
        return fail(CATENA_E_BAD_ARG, "decode tail: operands must be 16-byte aligned");
    FusedState* stp = nullptr;
    uint32_t base = 0;
    CATENA_TRY(fused_prepare(0, (size_t)m * hidden * 2, 2, &stp, &base));
    FusedState& st = *stp;
    const size_t smem = (size_t)m * hidden * 2;
    llama::DecodeTail p = {};
    p.att = (const __nv_bfloat16*)att; p.x = (const __nv_bfloat16*)x; p.w_o = (const __nv_bfloat16*)w_o;
    p.w_gate_up = (const __nv_bfloat16*)w_gate_up; p.w_down = (const __nv_bfloat16*)w_down;
    p.x2 = (__nv_bfloat16*)x2; p.act = (__nv_bfloat16*)act; p.out = (__nv_bfloat16*)out;
    p.M = (uint32_t)m; p.H = (uint32_t)hidden; p.KO = (uint32_t)ko; p.F = (uint32_t)ffn;
    p.barrier = st.counter; p.base = base; p.err = st.err; p.wait_ns = debug_wait_limit_ns();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)st.grid[0]);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = tls().stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;      // every CTA resident: they wait for one another at the barriers
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    CATENA_CUDA(cudaLaunchKernelEx(&cfg, llama::decode_tail_kernel, p));
    count_launch();
    return CATENA_OK;
}

bool decode_head_supported(uint64_t m, uint64_t hidden, uint64_t hq, uint64_t hkv) {
    return m >= 1 && m <= 16 && hidden % 8 == 0 && hidden <= 0x3FFFFFFFull && (hq + 2 * hkv) * 128 <= 0x3FFFFFFFull && m * hidden * 2 <= 160 * 1024;
}

// x = table[ids]; qkv = rmsnorm(x) w_qkv^T; q_out = rotated queries; row `pos` of the caches = rotated keys, values.  One launch.
catena_status_t launch_decode_head(const void* table, const int32_t* ids, const void* w_qkv, const float* inv_freq, uint32_t* bad, void* x,
                                   void* qkv, void* q_out, void* k_cache, void* v_cache, uint64_t m, uint64_t hidden, uint64_t vocab,
                                   uint64_t hq, uint64_t hkv, uint64_t cap, uint64_t pos) {
    CATENA_TRY(ensure_device());
    if (!decode_head_supported(m, hidden, hq, hkv)) return fail(CATENA_E_UNSUPPORTED, "decode head: shape");
    if (pos >= cap) return fail(CATENA_E_BAD_ARG, "rope: positions beyond the cache capacity");
    if (((uintptr_t)table | (uintptr_t)w_qkv | (uintptr_t)x | (uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15)
        return fail(CATENA_E_BAD_ARG, "decode head: operands must be 16-byte aligned");
    FusedState* stp = nullptr;
    uint32_t base = 0;
    const size_t smem = (size_t)m * hidden * 2;
    CATENA_TRY(fused_prepare(1, smem, 1, &stp, &base));
    llama::DecodeHead p = {};
    p.table = (const __nv_bfloat16*)table; p.ids = ids; p.w_qkv = (const __nv_bfloat16*)w_qkv; p.inv_freq = inv_freq;
    p.x = (__nv_bfloat16*)x; p.qkv = (__nv_bfloat16*)qkv; p.q_out = (__nv_bfloat16*)q_out;
    p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache;
    p.M = (uint32_t)m; p.H = (uint32_t)hidden; p.Hq = (uint32_t)hq; p.Hkv = (uint32_t)hkv; p.cap = (uint32_t)cap; p.pos = (uint32_t)pos;
    p.vocab = (uint32_t)vocab; p.bad = bad;
    p.barrier = stp->counter; p.base = base; p.err = stp->err; p.wait_ns = debug_wait_limit_ns();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)stp->grid[1]);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = tls().stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    CATENA_CUDA(cudaLaunchKernelEx(&cfg, llama::decode_head_kernel, p));
    count_launch();
    return CATENA_OK;
}

// Reads (and clears) the fused kernels' error word; after an expired barrier the counter starts again from zero.
catena_status_t decode_fused_check_errors() {
    CATENA_TRY(ensure_device());
    FusedState& st = g_fused[tls().device];
    if (!st.counter) return CATENA_OK;
    cudaStream_t s = tls().stream;
    CATENA_CUDA(cudaMemcpyAsync(st.err_host, st.err, sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    CATENA_CUDA(cudaStreamSynchronize(s));
    if (*st.err_host != 0) {
        *st.err_host = 0;
        cudaMemsetAsync(st.counter, 0, 2 * sizeof(uint32_t), s);
        st.count = 0;
        return fail(CATENA_E_TIMEOUT, "decode step: grid barrier wait expired");
    }
    return CATENA_OK;
}

}  // namespace catena
