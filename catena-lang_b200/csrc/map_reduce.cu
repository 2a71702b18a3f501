// Elementwise map kernels and reductions: what the reference lowers to one-thread-per-element
// `materializec` kernels (catena-lang/src/codegen/ops/materializec.rs:36-145) and to sequential
// host-side `reducec` folds (catena-lang/src/codegen/ops/reducec.rs:75-131), rebuilt as
// vectorised, coalesced HBM-bound kernels.
//
// Numerics:
//   * map kernels are bit-exact with the reference formulas (catena_math.cuh);
//   * a fold over n <= kExactFoldMax elements is evaluated in the reference's own order
//     (acc = zero; for i in 0..n: acc = add(acc, get(i))) by one thread reading values that the
//     whole block produced into shared memory, so it is bit-exact too;
//   * a longer fold uses a tree whose shape is a function of n only (never of the grid, the SM
//     count or the GPU count): thread t of block b folds elements 4*(j*256+t)+{0..3} of chunk b
//     for ascending j, then a 5-step xor butterfly inside each warp, then the 8 warp results in
//     ascending order, then the block partials are reduced by the same rule.  Sums then differ
//     from the sequential fold by rounding only (tolerance stated in the tests); max and argmax
//     are order-free on finite data (argmax keeps the lowest index among equal maxima, like
//     the reference's `>=` rule, catena-lang/stdlib/tensor.hex:186-201).
#include <string.h>

#include "catena_math.cuh"
#include "common.cuh"

namespace catena {

static constexpr uint64_t kExactFoldMax = 65536;   // longest fold evaluated sequentially
static constexpr int kThreads = 256;
static constexpr uint64_t kChunk = 16384;          // elements per block in the tree (64 per thread)
static constexpr int kStage = 2048;                // staging buffer of the sequential fold

enum FoldKind { F_SUM = 0, F_MAX = 1, F_SUMSQ = 2, F_EXPSUM = 3 };

template <int KIND>
__device__ __forceinline__ float fold_identity() {
    return KIND == F_MAX ? __uint_as_float(0xFF800000u) : __uint_as_float(0u);
}
// value produced for element x (the `get` closure of the fold)
template <int KIND>
__device__ __forceinline__ float fold_get(float x, float shift) {
    if (KIND == F_SUMSQ) return cmath::mul(x, x);                        // nn.hex:125-136
    if (KIND == F_EXPSUM) return cmath::exp_approx(cmath::sub(x, shift)); // nn.hex:59-72
    return x;
}
// the `add` closure: f32.add-env (sum.hex:7-14) or f32.max-env (sum.hex:73-84)
template <int KIND>
__device__ __forceinline__ float fold_add(float acc, float v) {
    if (KIND == F_MAX) return acc >= v ? acc : v;
    return cmath::add(acc, v);
}

// ---- sequential (bit-exact) fold: one block ------------------------------------------------
template <int KIND>
__device__ float fold_exact_block(const float* __restrict__ in, uint64_t n, float shift, float* stage) {
    float acc = fold_identity<KIND>();
    for (uint64_t base = 0; base < n; base += kStage) {
        uint64_t cnt = n - base < (uint64_t)kStage ? n - base : (uint64_t)kStage;
        for (uint64_t i = threadIdx.x; i < cnt; i += blockDim.x) stage[i] = fold_get<KIND>(in[base + i], shift);
        __syncthreads();
        if (threadIdx.x == 0) {
            for (uint64_t i = 0; i < cnt; ++i) acc = fold_add<KIND>(acc, stage[i]);
        }
        __syncthreads();
    }
    return acc;  // valid in thread 0
}

template <int KIND>
__global__ void __launch_bounds__(kThreads) fold_exact_kernel(const float* __restrict__ in, uint64_t n,
                                                              const float* shift_ptr, float* out) {
    __shared__ float stage[kStage];
    float shift = shift_ptr ? *shift_ptr : 0.0f;
    float acc = fold_exact_block<KIND>(in, n, shift, stage);
    if (threadIdx.x == 0) *out = acc;
}

// ---- fixed-shape tree fold -------------------------------------------------------------------
template <int KIND>
__device__ __forceinline__ float block_tree(float acc, float* warp_part) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        float other = __shfl_xor_sync(0xFFFFFFFFu, acc, off);
        // lower lane's value on the left, so both lanes of a pair compute the same expression
        bool low = (threadIdx.x & off) == 0;
        acc = low ? fold_add<KIND>(acc, other) : fold_add<KIND>(other, acc);
    }
    int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) warp_part[warp] = acc;
    __syncthreads();
    float r = fold_identity<KIND>();
    if (threadIdx.x == 0) {
        r = warp_part[0];
        for (int w = 1; w < kThreads / 32; ++w) r = fold_add<KIND>(r, warp_part[w]);
    }
    return r;
}

// level 0 applies `get`; GETK is the transform kind, ADDK the combine kind
template <int GETK, int ADDK>
__global__ void __launch_bounds__(kThreads) fold_tree_kernel(const float* __restrict__ in, uint64_t n,
                                                             const float* shift_ptr,
                                                             float* __restrict__ partials) {
    __shared__ float warp_part[kThreads / 32];
    float shift = shift_ptr ? *shift_ptr : 0.0f;
    uint64_t base = (uint64_t)blockIdx.x * kChunk;
    float acc = fold_identity<ADDK>();
    bool vec = ((reinterpret_cast<uintptr_t>(in) & 15) == 0) && (base + kChunk <= n);
    if (vec) {
        const float4* in4 = reinterpret_cast<const float4*>(in + base);
#pragma unroll 4
        for (int j = 0; j < (int)(kChunk / 4 / kThreads); ++j) {
            float4 v = in4[j * kThreads + threadIdx.x];
            if (GETK == F_EXPSUM) {                       // the four exp~ side by side, added in the same order
                const float x[4] = {cmath::sub(v.x, shift), cmath::sub(v.y, shift), cmath::sub(v.z, shift), cmath::sub(v.w, shift)};
                float e[4];
                cmath::exp_approx_n<4>(x, e);
                v = make_float4(e[0], e[1], e[2], e[3]);
                acc = fold_add<ADDK>(fold_add<ADDK>(fold_add<ADDK>(fold_add<ADDK>(acc, v.x), v.y), v.z), v.w);
                continue;
            }
            acc = fold_add<ADDK>(acc, fold_get<GETK>(v.x, shift));
            acc = fold_add<ADDK>(acc, fold_get<GETK>(v.y, shift));
            acc = fold_add<ADDK>(acc, fold_get<GETK>(v.z, shift));
            acc = fold_add<ADDK>(acc, fold_get<GETK>(v.w, shift));
        }
    } else {
        for (int j = 0; j < (int)(kChunk / 4 / kThreads); ++j) {
            uint64_t i0 = base + ((uint64_t)j * kThreads + threadIdx.x) * 4;
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (i0 + e < n) acc = fold_add<ADDK>(acc, fold_get<GETK>(in[i0 + e], shift));
        }
    }
    float r = block_tree<ADDK>(acc, warp_part);
    if (threadIdx.x == 0) partials[blockIdx.x] = r;
}

// The second level of the tree inside a consumer kernel: what fold_tree_kernel<ADDK, ADDK> computes with ONE block over
// `count` <= kChunk partials — the same elements per thread in the same order, the same butterfly, the same order of
// the warps — evaluated by every CTA of the consumer for itself (the partials sit in L2), so the consumer needs no
// separate launch for it.  Returns the value in every thread.
template <int ADDK>
__device__ __forceinline__ float fold_level1(const float* __restrict__ partials, uint32_t count, float* warp_part, float* result) {
    float acc = fold_identity<ADDK>();
    for (int j = 0; j < (int)(kChunk / 4 / kThreads); ++j) {
        const uint32_t i0 = ((uint32_t)j * kThreads + threadIdx.x) * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (i0 + e < count) acc = fold_add<ADDK>(acc, partials[i0 + e]);
    }
    const float r = block_tree<ADDK>(acc, warp_part);
    if (threadIdx.x == 0) *result = r;
    __syncthreads();
    return *result;
}

// ---- argmax ------------------------------------------------------------------------------------
struct IdxVal { uint64_t i; float v; };
__device__ __forceinline__ IdxVal better(IdxVal a, IdxVal b) {
    // value first; among equal values the lower index (first occurrence wins)
    bool keep_a = (a.v > b.v) || (a.v == b.v && a.i < b.i);
    return keep_a ? a : b;
}

__global__ void __launch_bounds__(kThreads) argmax_exact_kernel(const float* __restrict__ in, uint64_t n,
                                                                uint64_t* out) {
    // tensor.hex:204-227: init = (0, x[0]); fold over i = 0..n-1 keeping acc when acc >= value
    __shared__ float stage[kStage];
    uint64_t pos = 0;
    float best = 0.0f;
    for (uint64_t base = 0; base < n; base += kStage) {
        uint64_t cnt = n - base < (uint64_t)kStage ? n - base : (uint64_t)kStage;
        for (uint64_t i = threadIdx.x; i < cnt; i += blockDim.x) stage[i] = in[base + i];
        __syncthreads();
        if (threadIdx.x == 0) {
            if (base == 0) best = stage[0];
            for (uint64_t i = 0; i < cnt; ++i) {
                float v = stage[i];
                bool keep = best >= v;
                pos = keep ? pos : base + i;
                best = keep ? best : v;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) *out = pos;
}

__global__ void __launch_bounds__(kThreads) argmax_tree_kernel(const float* __restrict__ in,
                                                               const IdxVal* __restrict__ prev, uint64_t n,
                                                               IdxVal* __restrict__ partials) {
    __shared__ IdxVal warp_part[kThreads / 32];
    uint64_t base = (uint64_t)blockIdx.x * kChunk;
    IdxVal acc{UINT64_MAX, __uint_as_float(0xFF800000u)};
    for (int j = 0; j < (int)(kChunk / kThreads); ++j) {
        uint64_t i = base + (uint64_t)j * kThreads + threadIdx.x;
        if (i < n) {
            IdxVal v = prev ? prev[i] : IdxVal{i, in[i]};
            acc = better(acc, v);
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        IdxVal o;
        o.i = __shfl_xor_sync(0xFFFFFFFFu, acc.i, off);
        o.v = __shfl_xor_sync(0xFFFFFFFFu, acc.v, off);
        acc = better(acc, o);
    }
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        IdxVal r = warp_part[0];
        for (int w = 1; w < kThreads / 32; ++w) r = better(r, warp_part[w]);
        partials[blockIdx.x] = r;
    }
}

__global__ void argmax_finish_kernel(const IdxVal* p, uint64_t* out) { *out = p->i; }

// ---- map kernels ----------------------------------------------------------------------------------
template <int OP>
__global__ void __launch_bounds__(kThreads) map_unary_kernel(const float* __restrict__ in,
                                                             float* __restrict__ out, uint64_t n) {
    uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    bool vec = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    uint64_t n4 = vec ? n / 4 : 0;
    const float4* in4 = reinterpret_cast<const float4*>(in);
    float4* out4 = reinterpret_cast<float4*>(out);
    // Four float4 per trip, all four loads issued before the first value is used (a thread with one 16-byte load in flight
    // per trip keeps only 32 KB per SM in flight, which caps the stream near 5 TB/s).  Eight values at a time go through
    // the batched form of the op (zeros pad missing ones).
    const float4 zero4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (uint64_t i = tid; i < n4; i += 4 * stride) {
        const bool h1 = i + stride < n4, h2 = i + 2 * stride < n4, h3 = i + 3 * stride < n4;
        const float4 a = in4[i], b = h1 ? in4[i + stride] : zero4, c = h2 ? in4[i + 2 * stride] : zero4, d = h3 ? in4[i + 3 * stride] : zero4;
        const float x[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        float y[8];
        cmath::apply_n<OP, 8>(x, y);
        out4[i] = make_float4(y[0], y[1], y[2], y[3]);
        if (h1) out4[i + stride] = make_float4(y[4], y[5], y[6], y[7]);
        if (h2) {
            const float x2[8] = {c.x, c.y, c.z, c.w, d.x, d.y, d.z, d.w};
            cmath::apply_n<OP, 8>(x2, y);
            out4[i + 2 * stride] = make_float4(y[0], y[1], y[2], y[3]);
            if (h3) out4[i + 3 * stride] = make_float4(y[4], y[5], y[6], y[7]);
        }
    }
    for (uint64_t i = n4 * 4 + tid; i < n; i += stride) out[i] = cmath::apply<OP>(in[i]);
}

// softmax-at (nn.hex:75-90): exp~(x_i - max) / denom
// With `chunks` > 0 denom_ptr holds the level-0 partials of the exp-shifted sum and every CTA finishes that tree itself
// (fold_level1); with chunks == 0 it points at the scalar.
__global__ void __launch_bounds__(kThreads) softmax_map_kernel(const float* __restrict__ in,
                                                               float* __restrict__ out, uint64_t n,
                                                               const float* max_ptr, const float* denom_ptr, uint32_t chunks) {
    __shared__ float warp_part[kThreads / 32];
    __shared__ float result;
    const float m = *max_ptr;
    const float d = chunks ? fold_level1<F_SUM>(denom_ptr, chunks, warp_part, &result) : *denom_ptr;
    uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    bool vec = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    uint64_t n4 = vec ? n / 4 : 0;
    const float4* in4 = reinterpret_cast<const float4*>(in);
    float4* out4 = reinterpret_cast<float4*>(out);
    const float4 m4 = make_float4(m, m, m, m);
    for (uint64_t i = tid; i < n4; i += 4 * stride) {       // four loads in flight per thread (see map_unary_kernel)
        const bool h1 = i + stride < n4, h2 = i + 2 * stride < n4, h3 = i + 3 * stride < n4;
        const float4 a = in4[i], b = h1 ? in4[i + stride] : m4, c = h2 ? in4[i + 2 * stride] : m4, f = h3 ? in4[i + 3 * stride] : m4;
        const float x[8] = {cmath::sub(a.x, m), cmath::sub(a.y, m), cmath::sub(a.z, m), cmath::sub(a.w, m),
                            cmath::sub(b.x, m), cmath::sub(b.y, m), cmath::sub(b.z, m), cmath::sub(b.w, m)};
        float e[8];
        cmath::exp_approx_n<8>(x, e);
        out4[i] = make_float4(cmath::div(e[0], d), cmath::div(e[1], d), cmath::div(e[2], d), cmath::div(e[3], d));
        if (h1) out4[i + stride] = make_float4(cmath::div(e[4], d), cmath::div(e[5], d), cmath::div(e[6], d), cmath::div(e[7], d));
        if (h2) {
            const float x2[8] = {cmath::sub(c.x, m), cmath::sub(c.y, m), cmath::sub(c.z, m), cmath::sub(c.w, m),
                                 cmath::sub(f.x, m), cmath::sub(f.y, m), cmath::sub(f.z, m), cmath::sub(f.w, m)};
            cmath::exp_approx_n<8>(x2, e);
            out4[i + 2 * stride] = make_float4(cmath::div(e[0], d), cmath::div(e[1], d), cmath::div(e[2], d), cmath::div(e[3], d));
            if (h3) out4[i + 3 * stride] = make_float4(cmath::div(e[4], d), cmath::div(e[5], d), cmath::div(e[6], d), cmath::div(e[7], d));
        }
    }
    for (uint64_t i = n4 * 4 + tid; i < n; i += stride)
        out[i] = cmath::div(cmath::exp_approx(cmath::sub(in[i], m)), d);
}

// Whole softmax for one short row in a single launch: parallel max (order-free), sequential
// denominator, parallel map.
__global__ void __launch_bounds__(kThreads) softmax_small_kernel(const float* __restrict__ in,
                                                                 float* __restrict__ out, uint64_t n) {
    __shared__ float stage[kStage];
    __shared__ float warp_part[kThreads / 32];
    __shared__ float sh_max, sh_denom;
    float m = fold_identity<F_MAX>();
    for (uint64_t i = threadIdx.x; i < n; i += blockDim.x) m = fold_add<F_MAX>(m, in[i]);
    float r = block_tree<F_MAX>(m, warp_part);
    if (threadIdx.x == 0) sh_max = r;
    __syncthreads();
    float mx = sh_max;
    float acc = fold_exact_block<F_EXPSUM>(in, n, mx, stage);
    if (threadIdx.x == 0) sh_denom = acc;
    __syncthreads();
    float d = sh_denom;
    for (uint64_t i = threadIdx.x; i < n; i += blockDim.x)
        out[i] = cmath::div(cmath::exp_approx(cmath::sub(in[i], mx)), d);
}

// rmsnorm-at (nn.hex:139-151) with rms = sqrt~(sumsq/len + eps) (nn.hex:169-174)
// With `chunks` > 0 sumsq_ptr holds the level-0 partials of the sum of squares and every CTA finishes the tree itself.
__global__ void __launch_bounds__(kThreads) rmsnorm_map_kernel(const float* __restrict__ in,
                                                               float* __restrict__ out, uint64_t n,
                                                               const float* sumsq_ptr, uint32_t chunks) {
    __shared__ float warp_part[kThreads / 32];
    __shared__ float result;
    const float sumsq = chunks ? fold_level1<F_SUM>(sumsq_ptr, chunks, warp_part, &result) : *sumsq_ptr;
    float mean_sq = cmath::div(sumsq, cmath::u64_to_f32(n));
    float rms = cmath::sqrt_newton(cmath::add(mean_sq, cmath::from_bits(0x3727C5ACu)));
    uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    bool vec = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    uint64_t n4 = vec ? n / 4 : 0;
    const float4* in4 = reinterpret_cast<const float4*>(in);
    float4* out4 = reinterpret_cast<float4*>(out);
    for (uint64_t i = tid; i < n4; i += 4 * stride) {       // four loads in flight per thread (see map_unary_kernel)
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i + u * stride < n4) v[u] = in4[i + u * stride];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (i + u * stride < n4) {
                v[u].x = cmath::div(v[u].x, rms);
                v[u].y = cmath::div(v[u].y, rms);
                v[u].z = cmath::div(v[u].z, rms);
                v[u].w = cmath::div(v[u].w, rms);
                out4[i + u * stride] = v[u];
            }
        }
    }
    for (uint64_t i = n4 * 4 + tid; i < n; i += stride) out[i] = cmath::div(in[i], rms);
}

// broadcast (tensor.hex:2-21), arange (tensor.hex:24-46): MODE 0 = constant, 1 = (float)i
template <int MODE>
__global__ void __launch_bounds__(kThreads) fill_kernel(float* __restrict__ out, uint64_t n, float v) {
    uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = tid; i < n; i += stride) out[i] = MODE == 0 ? v : cmath::u64_to_f32(i);
}

// slice (tensor.hex:49-82) and concat (tensor.hex:85-168): out[i] = i < nl ? l[i] : r[i - nl]
__global__ void __launch_bounds__(kThreads) concat_kernel(const float* __restrict__ l, uint64_t nl,
                                                          const float* __restrict__ r, uint64_t nr,
                                                          float* __restrict__ out) {
    uint64_t n = nl + nr;
    uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = tid; i < n; i += stride) out[i] = i < nl ? l[i] : r[i - nl];
}

// ---- host side ---------------------------------------------------------------------------------------
static int grid_for(uint64_t work_items) {
    // a multiple of the SM count, 8 resident blocks of 256 threads per SM at most
    int sms = tls().sm_count > 0 ? tls().sm_count : 148;
    uint64_t blocks = ceil_div_u64(work_items, kThreads);
    uint64_t cap = (uint64_t)sms * 8;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    return (int)blocks;
}

struct OpName { const char* name; int op; };
static const OpName kOps[] = {
    {"math.sin-approx", cmath::OP_SIN_APPROX}, {"math.cos-approx", cmath::OP_COS_APPROX},
    {"math.sin-approx-full-nonneg", cmath::OP_SIN_FULL_NONNEG}, {"math.sin-approx-full", cmath::OP_SIN_FULL},
    {"math.log-approx", cmath::OP_LOG}, {"math.exp-approx-nonneg", cmath::OP_EXP_NONNEG},
    {"math.exp-approx", cmath::OP_EXP}, {"math.exp2-approx", cmath::OP_EXP2},
    {"math.log2-approx", cmath::OP_LOG2}, {"math.sqrt", cmath::OP_SQRT}, {"nn.sigmoid", cmath::OP_SIGMOID},
    {"nn.silu", cmath::OP_SILU}, {"nn.tanh", cmath::OP_TANH}, {"nn.gelu-approx", cmath::OP_GELU}};

int map_op_from_name(const char* name) {
    if (!name) return -1;
    for (const OpName& o : kOps)
        if (strcmp(o.name, name) == 0) return o.op;
    return -1;
}

template <int OP>
static void launch_map_t(const float* in, float* out, uint64_t n) {
    map_unary_kernel<OP><<<grid_for(ceil_div_u64(n, 4)), kThreads, 0, tls().stream>>>(in, out, n);
}

catena_status_t launch_map_unary(int op, const float* in, float* out, uint64_t n) {
    if (n == 0) return CATENA_OK;
    switch (op) {
        case cmath::OP_SIN_APPROX: launch_map_t<cmath::OP_SIN_APPROX>(in, out, n); break;
        case cmath::OP_COS_APPROX: launch_map_t<cmath::OP_COS_APPROX>(in, out, n); break;
        case cmath::OP_SIN_FULL_NONNEG: launch_map_t<cmath::OP_SIN_FULL_NONNEG>(in, out, n); break;
        case cmath::OP_SIN_FULL: launch_map_t<cmath::OP_SIN_FULL>(in, out, n); break;
        case cmath::OP_LOG: launch_map_t<cmath::OP_LOG>(in, out, n); break;
        case cmath::OP_EXP_NONNEG: launch_map_t<cmath::OP_EXP_NONNEG>(in, out, n); break;
        case cmath::OP_EXP: launch_map_t<cmath::OP_EXP>(in, out, n); break;
        case cmath::OP_EXP2: launch_map_t<cmath::OP_EXP2>(in, out, n); break;
        case cmath::OP_LOG2: launch_map_t<cmath::OP_LOG2>(in, out, n); break;
        case cmath::OP_SQRT: launch_map_t<cmath::OP_SQRT>(in, out, n); break;
        case cmath::OP_SIGMOID: launch_map_t<cmath::OP_SIGMOID>(in, out, n); break;
        case cmath::OP_SILU: launch_map_t<cmath::OP_SILU>(in, out, n); break;
        case cmath::OP_TANH: launch_map_t<cmath::OP_TANH>(in, out, n); break;
        case cmath::OP_GELU: launch_map_t<cmath::OP_GELU>(in, out, n); break;
        default: return fail(CATENA_E_BAD_ARG, "map: unknown op");
    }
    count_launch();
    return CATENA_OK;
}

// Enqueues the fold of `in[0..n)` into the device scalar `d_out`.  `d_shift` feeds F_EXPSUM.
// Scratch for the tree comes from the pool; pool_free orders its reuse after the kernels queued here (core.cu).
template <int KIND>
static catena_status_t enqueue_fold(const float* in, uint64_t n, const float* d_shift, float* d_out) {
    cudaStream_t st = tls().stream;
    if (n <= kExactFoldMax) {
        fold_exact_kernel<KIND><<<1, kThreads, 0, st>>>(in, n, d_shift, d_out);
        count_launch();
        return CATENA_OK;
    }
    constexpr int ADDK = (KIND == F_MAX) ? F_MAX : F_SUM;
    uint64_t blocks = ceil_div_u64(n, kChunk);
    void* scratch = nullptr;
    // two ping-pong partial buffers
    uint64_t lvl1 = ceil_div_u64(blocks, kChunk);
    CATENA_TRY(pool_alloc((blocks + lvl1 + 2) * sizeof(float), &scratch));
    float* p0 = (float*)scratch;
    float* p1 = p0 + blocks;
    if (blocks > 0x7FFFFFFFull) { pool_free(scratch); return fail(CATENA_E_TOO_LARGE, "fold: too many elements"); }
    fold_tree_kernel<KIND, ADDK><<<(unsigned)blocks, kThreads, 0, st>>>(in, n, d_shift, blocks == 1 ? d_out : p0);
    count_launch();
    uint64_t cur = blocks;
    float* src = p0;
    float* dst = p1;
    while (cur > 1) {
        uint64_t nb = ceil_div_u64(cur, kChunk);
        fold_tree_kernel<ADDK, ADDK><<<(unsigned)nb, kThreads, 0, st>>>(src, cur, nullptr, nb == 1 ? d_out : dst);
        count_launch();
        float* t = src; src = dst; dst = t;
        cur = nb;
    }
    return pool_free(scratch);
}

static catena_status_t enqueue_fold_kind(int kind, const float* in, uint64_t n, const float* d_shift,
                                         float* d_out) {
    switch (kind) {
        case F_SUM: return enqueue_fold<F_SUM>(in, n, d_shift, d_out);
        case F_MAX: return enqueue_fold<F_MAX>(in, n, d_shift, d_out);
        case F_SUMSQ: return enqueue_fold<F_SUMSQ>(in, n, d_shift, d_out);
        case F_EXPSUM: return enqueue_fold<F_EXPSUM>(in, n, d_shift, d_out);
    }
    return fail(CATENA_E_BAD_ARG, "fold kind");
}

catena_status_t reduce_f32(int kind, const float* in, uint64_t n, float* host_out) {
    CATENA_TRY(ensure_device());
    if (n == 0) {  // empty fold returns the zero element (sum.hex:37, sum.hex:94)
        uint32_t bits = kind == RED_MAX ? 0xFF800000u : 0u;
        memcpy(host_out, &bits, 4);
        return CATENA_OK;
    }
    void* d = nullptr;
    CATENA_TRY(pool_alloc(sizeof(float), &d));
    int fk = kind == RED_SUM ? F_SUM : kind == RED_MAX ? F_MAX : F_SUMSQ;
    catena_status_t s = enqueue_fold_kind(fk, in, n, nullptr, (float*)d);
    if (s == CATENA_OK) {
        cudaError_t e = cudaMemcpyAsync(host_out, d, sizeof(float), cudaMemcpyDeviceToHost, tls().stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(tls().stream);
        if (e != cudaSuccess) s = fail_cuda(e, "reduce_f32");
    }
    pool_free(d);
    return s;
}

catena_status_t argmax_f32(const float* in, uint64_t n, uint64_t* host_out) {
    CATENA_TRY(ensure_device());
    if (n == 0) return fail(CATENA_E_ASSERT, "tensor.argmax-f32: empty input (u64.assert-nz)");
    cudaStream_t st = tls().stream;
    void* d = nullptr;
    uint64_t blocks = ceil_div_u64(n, kChunk);
    uint64_t lvl1 = ceil_div_u64(blocks, kChunk);
    CATENA_TRY(pool_alloc(sizeof(uint64_t) * 2 + (blocks + lvl1 + 2) * sizeof(IdxVal), &d));
    uint64_t* d_out = (uint64_t*)d;
    if (n <= kExactFoldMax) {
        argmax_exact_kernel<<<1, kThreads, 0, st>>>(in, n, d_out);
        count_launch();
    } else {
        IdxVal* p0 = (IdxVal*)(d_out + 2);
        IdxVal* p1 = p0 + blocks;
        argmax_tree_kernel<<<(unsigned)blocks, kThreads, 0, st>>>(in, nullptr, n, p0);
        count_launch();
        uint64_t cur = blocks;
        IdxVal* src = p0;
        IdxVal* dst = p1;
        while (cur > 1) {
            uint64_t nb = ceil_div_u64(cur, kChunk);
            argmax_tree_kernel<<<(unsigned)nb, kThreads, 0, st>>>(nullptr, src, cur, dst);
            count_launch();
            IdxVal* t = src; src = dst; dst = t;
            cur = nb;
        }
        argmax_finish_kernel<<<1, 1, 0, st>>>(src, d_out);
        count_launch();
    }
    catena_status_t s = CATENA_OK;
    cudaError_t e = cudaMemcpyAsync(host_out, d_out, sizeof(uint64_t), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) s = fail_cuda(e, "argmax_f32");
    pool_free(d);
    return s;
}

static catena_status_t launch_softmax_fused_levels(const float* in, float* out, uint64_t n);
catena_status_t launch_softmax(const float* in, float* out, uint64_t n) {
    if (n == 0) return CATENA_OK;
    cudaStream_t st = tls().stream;
    if (n <= kExactFoldMax) {
        softmax_small_kernel<<<1, kThreads, 0, st>>>(in, out, n);
        count_launch();
        return CATENA_OK;
    }
    if (ceil_div_u64(n, kChunk) <= kChunk) return launch_softmax_fused_levels(in, out, n);
    void* d = nullptr;
    CATENA_TRY(pool_alloc(2 * sizeof(float), &d));
    float* d_max = (float*)d;
    float* d_den = d_max + 1;
    catena_status_t s = enqueue_fold<F_MAX>(in, n, nullptr, d_max);
    if (s == CATENA_OK) s = enqueue_fold<F_EXPSUM>(in, n, d_max, d_den);
    if (s == CATENA_OK) {
        softmax_map_kernel<<<grid_for(ceil_div_u64(n, 4)), kThreads, 0, st>>>(in, out, n, d_max, d_den, 0u);
        count_launch();
    }
    pool_free(d);
    return s;
}

// Long rows whose level-0 partials fit one block of the second level (n <= kChunk^2 = 2^28): the map kernel's CTAs finish
// the tree of the denominator themselves, which saves one tiny dependent launch; same tree, same bits.  (The maximum
// keeps its own second-level launch: the exp-shifted sum needs it as a scalar in every one of its 4096 short-lived CTAs,
// and a persistent form of that kernel measured slower — 77 against 64 us at 64 Mi elements, it is bound by the exp~
// arithmetic and balances worse.)
static catena_status_t launch_softmax_fused_levels(const float* in, float* out, uint64_t n) {
    const uint64_t chunks = ceil_div_u64(n, kChunk);
    void* d = nullptr;
    CATENA_TRY(pool_alloc((2 * chunks + 1) * sizeof(float), &d));
    float* p_max = static_cast<float*>(d);
    float* p_sum = p_max + chunks;
    float* d_max = p_sum + chunks;
    cudaStream_t st = tls().stream;
    fold_tree_kernel<F_MAX, F_MAX><<<(unsigned)chunks, kThreads, 0, st>>>(in, n, nullptr, p_max);
    fold_tree_kernel<F_MAX, F_MAX><<<1, kThreads, 0, st>>>(p_max, chunks, nullptr, d_max);
    fold_tree_kernel<F_EXPSUM, F_SUM><<<(unsigned)chunks, kThreads, 0, st>>>(in, n, d_max, p_sum);
    softmax_map_kernel<<<grid_for(ceil_div_u64(n, 4)), kThreads, 0, st>>>(in, out, n, d_max, p_sum, (uint32_t)chunks);
    count_launch(4);
    cudaError_t e = cudaGetLastError();
    pool_free(d);
    return e == cudaSuccess ? CATENA_OK : fail_cuda(e, "softmax launch");
}

catena_status_t launch_rmsnorm(const float* in, float* out, uint64_t n) {
    if (n == 0) return CATENA_OK;
    const uint64_t chunks = ceil_div_u64(n, kChunk);
    if (n > kExactFoldMax && chunks <= kChunk) {
        // two launches: sum-of-squares partials, then the map whose CTAs finish the tree themselves (same bits)
        void* d = nullptr;
        CATENA_TRY(pool_alloc(chunks * sizeof(float), &d));
        fold_tree_kernel<F_SUMSQ, F_SUM><<<(unsigned)chunks, kThreads, 0, tls().stream>>>(in, n, nullptr, static_cast<float*>(d));
        rmsnorm_map_kernel<<<grid_for(ceil_div_u64(n, 4)), kThreads, 0, tls().stream>>>(in, out, n, static_cast<float*>(d), (uint32_t)chunks);
        count_launch(2);
        cudaError_t e = cudaGetLastError();
        pool_free(d);
        return e == cudaSuccess ? CATENA_OK : fail_cuda(e, "rmsnorm launch");
    }
    void* d = nullptr;
    CATENA_TRY(pool_alloc(sizeof(float), &d));
    catena_status_t s = enqueue_fold<F_SUMSQ>(in, n, nullptr, (float*)d);
    if (s == CATENA_OK) {
        rmsnorm_map_kernel<<<grid_for(ceil_div_u64(n, 4)), kThreads, 0, tls().stream>>>(in, out, n, (float*)d, 0u);
        count_launch();
    }
    pool_free(d);
    return s;
}

catena_status_t launch_broadcast(float v, float* out, uint64_t n) {
    if (n == 0) return CATENA_OK;
    fill_kernel<0><<<grid_for(n), kThreads, 0, tls().stream>>>(out, n, v);
    count_launch();
    return CATENA_OK;
}

catena_status_t launch_arange(float* out, uint64_t n) {
    if (n == 0) return CATENA_OK;
    fill_kernel<1><<<grid_for(n), kThreads, 0, tls().stream>>>(out, n, 0.0f);
    count_launch();
    return CATENA_OK;
}

catena_status_t launch_slice(const float* in, uint64_t start, float* out, uint64_t n) {
    if (n == 0) return CATENA_OK;
    concat_kernel<<<grid_for(n), kThreads, 0, tls().stream>>>(in + start, n, nullptr, 0, out);
    count_launch();
    return CATENA_OK;
}

catena_status_t launch_concat(const float* l, uint64_t nl, const float* r, uint64_t nr, float* out) {
    if (nl + nr == 0) return CATENA_OK;
    concat_kernel<<<grid_for(nl + nr), kThreads, 0, tls().stream>>>(l, nl, r, nr, out);
    count_launch();
    return CATENA_OK;
}

// ---- sum without any allocation ------------------------------------------------------------------
// Block partials of the tree sum live in this fixed array instead of a pool block.  It is part of the
// module image, so every GPU that loads the library carries these 256 KiB until the process exits.
// kNoAllocMaxPartials level-0 partials cover kNoAllocMaxElems = 2^30 elements; the few extra slots
// hold the partials of the upper tree levels.
static constexpr uint64_t kNoAllocMaxPartials = 65536;
static constexpr uint64_t kNoAllocMaxElems = kNoAllocMaxPartials * kChunk;
static __device__ __align__(256) float g_sum_scratch[kNoAllocMaxPartials + 64];

// In host code `g_sum_scratch` is only a handle for the symbol, never a pointer a kernel may use: the
// device address is looked up once per device (with that device current) and cached here.
static float* g_sum_scratch_dev[16] = {nullptr};

catena_status_t sum_f32_noalloc(const float* in, uint64_t n, float* d_out) {
    CATENA_TRY(ensure_device());
    if (!d_out || (n != 0 && !in)) return fail(CATENA_E_BAD_ARG, "sum_f32_noalloc: null pointer");
    if (n > kNoAllocMaxElems)
        return fail(CATENA_E_TOO_LARGE, "sum_f32_noalloc: more than 2^30 elements (fixed scratch array)");
    const int dev = tls().device;
    if (!g_sum_scratch_dev[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_sum_scratch);
        if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(g_sum_scratch)");
        g_sum_scratch_dev[dev] = static_cast<float*>(p);
    }
    float* scratch = g_sum_scratch_dev[dev];
    cudaStream_t st = tls().stream;
    if (n <= kExactFoldMax) {
        // short inputs (and the empty one, whose sum is +0) take the sequential fold: no scratch at all
        fold_exact_kernel<F_SUM><<<1, kThreads, 0, st>>>(in, n, nullptr, d_out);
        count_launch();
        return finish("sum_f32_noalloc");
    }
    // Same tree as the pooled path: level 0 writes every partial it will read back, so nothing in the
    // array needs clearing between calls.
    uint64_t blocks = ceil_div_u64(n, kChunk);
    float* src = scratch;
    float* dst = scratch + kNoAllocMaxPartials;          // upper levels: at most 4, then 1 partials
    fold_tree_kernel<F_SUM, F_SUM><<<(unsigned)blocks, kThreads, 0, st>>>(in, n, nullptr, blocks == 1 ? d_out : src);
    count_launch();
    uint64_t cur = blocks;
    while (cur > 1) {
        uint64_t nb = ceil_div_u64(cur, kChunk);
        fold_tree_kernel<F_SUM, F_SUM><<<(unsigned)nb, kThreads, 0, st>>>(src, cur, nullptr, nb == 1 ? d_out : dst);
        count_launch();
        float* t = src; src = dst; dst = t;
        cur = nb;
    }
    return finish("sum_f32_noalloc");
}

}  // namespace catena

// Sum of `n` f32 values for callers that must not allocate: a host that gave all of HBM to its own
// arena when it started (so a cudaMalloc inside the library would fail), or a latency-critical loop
// that cannot take the device-wide synchronisation an allocation implies.  `in` and `out` are device
// pointers owned by the caller (`out`: one float).  No cudaMalloc, cudaFree or pool call is made; the
// partial sums of the reduction tree go to a fixed 256 KiB array inside the library image, which
// bounds the input at 2^30 elements (CATENA_E_TOO_LARGE beyond).  The first call on each device looks
// up that array's device address; make it before starting any stream capture.  All calls on a device
// share the array, so two calls whose kernels overlap on the GPU (different streams or threads) race;
// calls on one stream are ordered and safe.  The value is bit-identical to program_sum_f32.
extern "C" catena_status_t catena_b200_sum_f32_noalloc(const void* in, uint64_t n, void* out) {
    return catena::sum_f32_noalloc(static_cast<const float*>(in), n, static_cast<float*>(out));
}
