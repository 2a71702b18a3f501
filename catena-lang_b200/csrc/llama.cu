// Llama-style transformer block (pre-norm, rotary positions, SwiGLU) wired from this library's kernels.
// The reference has no bf16, no attention and no rotary embedding; every formula here is composed from
// reference programs under the inherited rules:
//   * rmsnorm      nn.rmsnorm (catena-lang/stdlib/nn.hex:125-182): y = x / sqrt~(mean(x^2) + eps), NO gain vector
//   * projections  the matmul cell rule (catena-lang/stdlib/matrix.hex:236-256): fp32 accumulate, fixed k order
//   * rotary       angle = position * base^(-2i/128) with base^(..) = math.powf (catena-lang/stdlib/math.hex:202-231),
//                  sin = math.sin-approx-full (math.hex:91-103), cos(x) = sin-approx-full(x + pi/2) because the
//                  reference has no full-range cosine (math.hex:27-47 covers small |x| only)
//   * attention    nn.softmax semantics (nn.hex:93-122): global max, exp~, probabilities as bf16 hi + lo
//   * SwiGLU       nn.silu (nn.hex:2-56) of the gate times the up projection
//   * residuals    f32.add of the two bf16 values, rounded to bf16
// Activations are bf16 in HBM; every intermediate sum is fp32 with separately rounded multiply and add.
//
// Kernels in this file: embedding gather, row rmsnorm, rotary + KV-cache append, causal prefill attention
// (mma.sync, two passes over the keys: maxima, then probabilities), SwiGLU, residual add, and a skinny
// GEMM (at most 8 rows: the decode step streams each weight matrix once, HBM-bound).  The wide
// projections of the prefill use the tcgen05 GEMM, the decode attention the cached-attention kernel.
#include <cuda_bf16.h>

#include "catena_math.cuh"
#include "common.cuh"
#include "skinny.cuh"

namespace catena {

namespace llama {

constexpr int kHeadDim = 128;
constexpr uint32_t kEpsBits = 0x3727C5ACu;      // 1e-5, nn.hex:154-182
constexpr uint32_t kHalfPiBits = 0x3FC90FDBu;   // pi/2 rounded to f32

// Programmatic dependent launch: every kernel of this file lets the next launch in the stream begin at once
// (pdl_trigger) and itself waits for the complete results of everything launched before it (pdl_wait) only when it
// first touches data another kernel may have written — launch latency and, in the skinny GEMM, the first batch of
// weight loads overlap the predecessor's tail.  Both are no-ops for a launch without the attribute.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) { return f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16); }

// ---------------------------------------------------------------- embedding gather
// out[t, :] = table[ids[t], :]; one CTA per token, 16-byte pieces.  An id outside the table sets *bad.
__global__ void embed_rows_kernel(const uint4* __restrict__ table, const int32_t* __restrict__ ids, uint4* __restrict__ out,
                                  uint32_t hidden16, uint32_t vocab, uint32_t* bad) {
    pdl_trigger();
    pdl_wait();
    const uint32_t t = blockIdx.x;
    const int32_t id = ids[t];
    if (id < 0 || (uint32_t)id >= vocab) {
        if (threadIdx.x == 0) atomicExch(bad, 1u);
        return;
    }
    const uint4* src = table + (size_t)id * hidden16;
    uint4* dst = out + (size_t)t * hidden16;
    for (uint32_t i = threadIdx.x; i < hidden16; i += blockDim.x) dst[i] = src[i];
}

// ---------------------------------------------------------------- row rmsnorm (bf16 in / out)
// One CTA of 256 threads per row.  Sum of squares in a fixed shape: thread t adds its elements in ascending
// order (8 consecutive elements per 2048-element stride), xor butterfly per warp, warps added in ascending order.
// With `ids` the row is gathered from the embedding table `x` first (and copied to x_out): embedding + first norm
// of the block in one launch.
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ ids, uint32_t vocab,
                                                          uint32_t* bad, uint4* __restrict__ x_out, uint4* __restrict__ y, uint32_t hidden) {
    __shared__ float warp_sum[8];
    __shared__ float rms_s;
    pdl_trigger();
    pdl_wait();
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    size_t src_row = row;
    if (ids) {
        const int32_t id = ids[row];
        if (id < 0 || (uint32_t)id >= vocab) {
            if (tid == 0) atomicExch(bad, 1u);
            return;
        }
        src_row = (size_t)id;
    }
    const uint4* xr = x + src_row * (hidden / 8);
    float acc = 0.0f;
    for (uint32_t i = tid; i < hidden / 8; i += 256) {
        const uint4 v = xr[i];
        if (x_out) x_out[(size_t)row * (hidden / 8) + i] = v;
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float a = bf16_bits_to_f32(w[e] & 0xFFFFu), b = bf16_bits_to_f32(w[e] >> 16);
            acc = cmath::add(acc, cmath::mul(a, a));
            acc = cmath::add(acc, cmath::mul(b, b));
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc = cmath::add(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, off));
    if ((tid & 31) == 0) warp_sum[tid >> 5] = acc;
    __syncthreads();
    if (tid == 0) {
        float s = warp_sum[0];
        for (int w = 1; w < 8; ++w) s = cmath::add(s, warp_sum[w]);
        const float mean = cmath::div(s, cmath::u64_to_f32(hidden));
        rms_s = cmath::sqrt_newton(cmath::add(mean, cmath::from_bits(kEpsBits)));
    }
    __syncthreads();
    const float rms = rms_s;
    uint4* yr = y + (size_t)row * (hidden / 8);
    for (uint32_t i = tid; i < hidden / 8; i += 256) {
        const uint4 v = xr[i];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t r[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
            r[e] = pack_bf16(cmath::div(bf16_bits_to_f32(w[e] & 0xFFFFu), rms), cmath::div(bf16_bits_to_f32(w[e] >> 16), rms));
        yr[i] = make_uint4(r[0], r[1], r[2], r[3]);
    }
}

// ---------------------------------------------------------------- rotary embedding + KV-cache append
// cos / sin of angle = position * inv_freq[i] for positions pos0 .. pos0 + seq - 1, i < 64: the angle depends on
// neither head nor sequence, so it is evaluated once per (position, i) instead of once per (token, head, i).
__device__ __forceinline__ float2 rope_cos_sin(uint32_t pos, float inv_freq) {
    const float angle = cmath::mul(cmath::u32_to_f32(pos), inv_freq);
    return make_float2(cmath::sin_full(cmath::add(angle, cmath::from_bits(kHalfPiBits))), cmath::sin_full(angle));
}
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, float2* __restrict__ table, uint32_t pos0, uint32_t seq) {
    pdl_trigger();
    pdl_wait();
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < seq * 64) table[idx] = rope_cos_sin(pos0 + idx / 64, inv_freq[idx % 64]);
}

// qkv [T, (Hq + 2 Hkv) * 128] bf16 (one row per token: query heads, key heads, value heads).
// Token t belongs to sequence t / S at position pos0 + t % S.  Writes
//   q_out   [T, Hq, 128]                 rotated queries
//   k_cache [B, Hkv, cap, 128] at pos    rotated keys
//   v_cache [B, Hkv, cap, 128] at pos    values
// One thread per (token, head, 8 pairs): pair i is (i, i + 64) ("rotate half").  `table` [S][64] holds (cos, sin)
// per position; without it (few tokens) they are evaluated in place — the same function, the same bits — by
// rope_append_small_kernel below, one pair per thread (the evaluation is a long dependent chain).
// inv_freq[i] = base^(-2i/128), computed once on the host with the same bit-exact functions.
__global__ void rope_append_small_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                                         __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                         const float* __restrict__ inv_freq, uint32_t T, uint32_t S, uint32_t pos0, uint32_t Hq,
                                         uint32_t Hkv, uint32_t cap) {
    pdl_trigger();
    pdl_wait();
    const uint32_t heads = Hq + 2 * Hkv;
    const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)T * heads * 64) return;
    const uint32_t i = (uint32_t)(idx % 64);
    const uint32_t head = (uint32_t)((idx / 64) % heads);
    const uint32_t t = (uint32_t)(idx / (64ull * heads));
    const uint32_t b = t / S, pos = pos0 + t % S;
    const __nv_bfloat16* src = qkv + ((size_t)t * heads + head) * kHeadDim;
    if (head >= Hq + Hkv) {   // value head: plain copy
        __nv_bfloat16* dst = v_cache + (((size_t)b * Hkv + (head - Hq - Hkv)) * cap + pos) * kHeadDim;
        dst[i] = src[i];
        dst[i + 64] = src[i + 64];
        return;
    }
    const float x1 = __bfloat162float(src[i]), x2 = __bfloat162float(src[i + 64]);
    const float2 cs = rope_cos_sin(pos, inv_freq[i]);
    __nv_bfloat16* dst = head < Hq ? q_out + ((size_t)t * Hq + head) * kHeadDim
                                   : k_cache + (((size_t)b * Hkv + (head - Hq)) * cap + pos) * kHeadDim;
    dst[i] = __float2bfloat16_rn(cmath::sub(cmath::mul(x1, cs.x), cmath::mul(x2, cs.y)));
    dst[i + 64] = __float2bfloat16_rn(cmath::add(cmath::mul(x2, cs.x), cmath::mul(x1, cs.y)));
}
__global__ void rope_append_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                                   __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                   const float2* __restrict__ table, uint32_t T, uint32_t S, uint32_t pos0, uint32_t Hq, uint32_t Hkv,
                                   uint32_t cap) {
    pdl_trigger();
    pdl_wait();
    const uint32_t heads = Hq + 2 * Hkv;
    const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)T * heads * 8) return;
    const uint32_t i0 = (uint32_t)(idx % 8) * 8;
    const uint32_t head = (uint32_t)((idx / 8) % heads);
    const uint32_t t = (uint32_t)(idx / (8ull * heads));
    const uint32_t b = t / S, s = t % S, pos = pos0 + s;
    const __nv_bfloat16* src = qkv + ((size_t)t * heads + head) * kHeadDim;
    const uint4 lo = *reinterpret_cast<const uint4*>(src + i0), hi = *reinterpret_cast<const uint4*>(src + 64 + i0);
    if (head >= Hq + Hkv) {   // value head: plain copy
        __nv_bfloat16* dst = v_cache + (((size_t)b * Hkv + (head - Hq - Hkv)) * cap + pos) * kHeadDim;
        *reinterpret_cast<uint4*>(dst + i0) = lo;
        *reinterpret_cast<uint4*>(dst + 64 + i0) = hi;
        return;
    }
    const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
    uint32_t r1[4], r2[4];
#pragma unroll
    for (uint32_t e = 0; e < 4; ++e) {
        float o1[2], o2[2];
#pragma unroll
        for (uint32_t u = 0; u < 2; ++u) {
            const uint32_t i = i0 + 2 * e + u;
            const float x1 = bf16_bits_to_f32(u ? lw[e] >> 16 : lw[e] & 0xFFFFu), x2 = bf16_bits_to_f32(u ? hw[e] >> 16 : hw[e] & 0xFFFFu);
            const float2 cs = table[(size_t)s * 64 + i];
            o1[u] = cmath::sub(cmath::mul(x1, cs.x), cmath::mul(x2, cs.y));
            o2[u] = cmath::add(cmath::mul(x2, cs.x), cmath::mul(x1, cs.y));
        }
        r1[e] = pack_bf16(o1[0], o1[1]);
        r2[e] = pack_bf16(o2[0], o2[1]);
    }
    __nv_bfloat16* dst = head < Hq ? q_out + ((size_t)t * Hq + head) * kHeadDim
                                   : k_cache + (((size_t)b * Hkv + (head - Hq)) * cap + pos) * kHeadDim;
    *reinterpret_cast<uint4*>(dst + i0) = make_uint4(r1[0], r1[1], r1[2], r1[3]);
    *reinterpret_cast<uint4*>(dst + 64 + i0) = make_uint4(r2[0], r2[1], r2[2], r2[3]);
}

// ---------------------------------------------------------------- SwiGLU and residual add
// gu [T, 2F] bf16 (gate columns, then up columns) -> a [T, F] = silu(gate) * up
__global__ void swiglu_kernel(const uint4* __restrict__ gu, uint4* __restrict__ a, uint64_t T, uint32_t F8) {
    pdl_trigger();
    pdl_wait();
    const uint64_t n = T * F8;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t t = idx / F8, c = idx % F8;
        const uint4 g = gu[t * 2 * F8 + c], u = gu[t * 2 * F8 + F8 + c];
        const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
        float gx[8], sg[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            gx[2 * e] = bf16_bits_to_f32(gw[e] & 0xFFFFu);
            gx[2 * e + 1] = bf16_bits_to_f32(gw[e] >> 16);
        }
        cmath::silu_n<8>(gx, sg);                      // nn.silu of the eight gates side by side (catena_math.cuh)
        uint32_t r[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
            r[e] = pack_bf16(cmath::mul(sg[2 * e], bf16_bits_to_f32(uw[e] & 0xFFFFu)), cmath::mul(sg[2 * e + 1], bf16_bits_to_f32(uw[e] >> 16)));
        a[idx] = make_uint4(r[0], r[1], r[2], r[3]);
    }
}

// out = x + y (bf16, fp32 add, RNE); out may alias x or y
__global__ void add_rows_kernel(const uint4* x, const uint4* y, uint4* out, uint64_t n8) {
    pdl_trigger();
    pdl_wait();
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n8; idx += (uint64_t)gridDim.x * blockDim.x) {
        const uint4 a = x[idx], b = y[idx];
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
        uint32_t r[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
            r[e] = pack_bf16(cmath::add(bf16_bits_to_f32(aw[e] & 0xFFFFu), bf16_bits_to_f32(bw[e] & 0xFFFFu)),
                             cmath::add(bf16_bits_to_f32(aw[e] >> 16), bf16_bits_to_f32(bw[e] >> 16)));
        out[idx] = make_uint4(r[0], r[1], r[2], r[3]);
    }
}

// ---------------------------------------------------------------- skinny GEMM (M <= 16 rows): arithmetic in skinny.cuh
// CTAs are persistent and software-pipelined (skinny.cuh); the first batch of weight loads is issued before the wait for the
// predecessor's results.
__global__ void __launch_bounds__(256, kSkinnyCtasPerSm) skinny_gemm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                         const __nv_bfloat16* __restrict__ res, __nv_bfloat16* __restrict__ y,
                                                         uint32_t M, uint32_t N, uint32_t K, uint32_t swiglu_f) {
    __shared__ float part[8][16][8];    // [warp][token][weight row]
    const SkinnyJob job = {x, w, res, y, M, N, K, swiglu_f};
    const SkinnySchedule sc(job, blockIdx.x, gridDim.x);
    uint4 cur[kSkinnyUnroll];
    pdl_trigger();
    if (sc.steps > 0) skinny_load_w(job, sc, 0, cur);      // weights are never written by a kernel: they may be fetched before the wait
    pdl_wait();
    skinny_run<A_READONLY>(job, sc, part, cur);
}

// The q/k/v projection of a decode step with the rotation and the cache append in its epilogue (skinny.cuh: SkinnyRope): one
// launch instead of the projection followed by rope_append_small_kernel, the same bits.  The (cos, sin) of the CTA's pairs
// depend on the step's position only, so they are evaluated before the wait for the predecessor, like the first weights.
__global__ void __launch_bounds__(256, kSkinnyCtasPerSm) skinny_qkv_rope_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                                                uint32_t M, uint32_t N, uint32_t K, SkinnyRope rope,
                                                                                const float* __restrict__ inv_freq) {
    __shared__ float part[8][16][8];
    __shared__ float pairs[16][8];
    __shared__ float2 cs_tab[kSkinnyRopeGroups * 4];
    SkinnyJob job = {x, w, nullptr, nullptr, M, N, K, 0u, rope};
    job.rope.cs = cs_tab;
    const SkinnySchedule sc(job, blockIdx.x, gridDim.x);
    uint4 cur[kSkinnyUnroll];
    pdl_trigger();
    if (sc.steps > 0) skinny_load_w<true>(job, sc, 0, cur);
    const uint32_t my_groups = sc.steps / sc.batches;
    if (threadIdx.x < my_groups * 4 && threadIdx.x < kSkinnyRopeGroups * 4) {
        const uint32_t grp = blockIdx.x + (threadIdx.x >> 2) * gridDim.x, i = (grp & 15u) * 4 + (threadIdx.x & 3u);
        cs_tab[threadIdx.x] = rope_cos_sin(rope.pos, inv_freq[i]);
    }
    pdl_wait();
    skinny_run<A_READONLY, true>(job, sc, part, cur, pairs);
}

// ---------------------------------------------------------------- causal prefill attention (mma.sync)
// q [T, Hq, 128] bf16 (rotated), k/v cache [B, Hkv, cap, 128] bf16, out [T, Hq * 128] bf16; token t = b * S + s
// attends to cache positions 0..s of its sequence.  One CTA (4 warps) per 64 queries of one head; warp w owns
// 16 query rows.  exp~ is not multiplicative, so there is no online rescaling: pass 1 multiplies Q K^T over all
// visible key tiles for the row maxima only, pass 2 multiplies again, forms p = exp~(s - max) and accumulates
// O += P V with P as a bf16 hi + lo pair.  Sums are fixed-order: a thread adds its own columns in ascending
// key order, the four threads of a row combine by xor butterfly.
// Shared-memory tiles are [row][128 bf16] with the 16-byte chunk index xor-ed by (row & 7).
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t tile_off(uint32_t row, uint32_t chunk) { return row * 256u + ((chunk ^ (row & 7u)) << 4); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// not volatile: the instruction is a pure function of its operands, so the compiler may interleave independent ones
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// copies rows [row0, row0 + 64) of a [rows_total, 128] bf16 matrix (row pitch `pitch` elements) into a swizzled tile
// with cp.async (one commit group per call); rows past rows_total are filled with zeros
__device__ __forceinline__ void load_tile_async(uint8_t* tile, const __nv_bfloat16* base, size_t pitch, uint32_t row0, uint32_t rows_total) {
    for (uint32_t i = threadIdx.x; i < 64 * 16; i += 128) {
        const uint32_t r = i >> 4, c = i & 15;
        const bool ok = row0 + r < rows_total;
        const __nv_bfloat16* src = base + (size_t)(ok ? row0 + r : 0) * pitch + c * 8;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(tile + tile_off(r, c))), "l"(src), "r"(ok ? 16u : 0u)
                     : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// math.exp-approx (catena-lang/stdlib/math.hex:148-199) for x <= 0, bit-identical to cmath::exp_approx there, with the
// conversions taken off the slow pipe: round-to-nearest-even of t in [0, 2^22) through the 1.5 * 2^23 constant
// (the same integer and the same float as (uint32_t)nearbyintf(t) and its conversion back).
__device__ __forceinline__ float exp_approx_nonpos(float x) {
    const float mag = -x;
    const float t = cmath::mul(mag, cmath::from_bits(0x3FB8AA3Bu));
    const float shifted = cmath::add(t, 12582912.0f);
    const float kf = cmath::sub(shifted, 12582912.0f);
    const uint32_t k = __float_as_uint(shifted) - 0x4B400000u;
    float xr = cmath::sub(mag, cmath::mul(kf, cmath::from_bits(0x3F317200u)));
    xr = cmath::sub(xr, cmath::mul(kf, cmath::from_bits(0x35BFBE8Eu)));
    float p = cmath::add(cmath::from_bits(0x3EEF1187u), cmath::mul(xr, cmath::from_bits(0x3E738A8Bu)));
    p = cmath::add(cmath::from_bits(0x3F809C7Eu), cmath::mul(xr, p));
    p = cmath::add(cmath::from_bits(0x3F7FF8FCu), cmath::mul(xr, p));
    p = cmath::mul(p, cmath::from_bits((k + 0x7Fu) * 0x00800000u));
    return x < 0.0f ? cmath::recip(p) : p;
}
// two probabilities -> packed bf16 hi parts and packed bf16 lo parts (p - hi), one conversion instruction each
__device__ __forceinline__ void split_hi_lo(float p0, float p1, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    const float r0 = cmath::sub(p0, __uint_as_float(hi << 16)), r1 = cmath::sub(p1, __uint_as_float(hi & 0xFFFF0000u));
    const __nv_bfloat162 l = __floats2bfloat162_rn(r0, r1);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

// Tiles stream through three 16 KiB buffers with cp.async: the K tile of step kt+1 is in flight while step kt is
// multiplied (two K buffers, one of them the Q tile's once the query fragments sit in registers), the V tile of
// step kt is in flight during Q K^T and exp~ of step kt.
__global__ void __launch_bounds__(128, 3) attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                                                             const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out,
                                                             uint32_t S, uint32_t Hq, uint32_t Hkv, uint32_t cap, float scale) {
    extern __shared__ __align__(1024) uint8_t smem_pf[];
    uint8_t* kbuf[2] = {smem_pf, smem_pf + 16384};           // kbuf[0] first holds the Q tile
    uint8_t* v_tile = smem_pf + 32768;
    const uint32_t qt = gridDim.x - 1 - blockIdx.x;          // heavy tiles first
    const uint32_t h = blockIdx.y, b = blockIdx.z, kvh = h / (Hq / Hkv);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    const __nv_bfloat16* qb = q + ((size_t)b * S * Hq + h) * kHeadDim;               // row pitch Hq * 128
    const __nv_bfloat16* kb = k_cache + ((size_t)b * Hkv + kvh) * cap * kHeadDim;    // row pitch 128
    const __nv_bfloat16* vb = v_cache + ((size_t)b * Hkv + kvh) * cap * kHeadDim;
    const float ninf = __uint_as_float(0xFF800000u);
    pdl_trigger();
    pdl_wait();

    load_tile_async(kbuf[0], qb, (size_t)Hq * kHeadDim, qt * 64, S);
    load_tile_async(kbuf[1], kb, kHeadDim, 0, S);            // K tile 0 of pass 1 (step parity is shifted by one in pass 1)
    cp_async_wait<1>();
    __syncthreads();
    uint32_t qa[8][4];   // A fragments of this warp's 16 query rows, one per 16-d step
#pragma unroll
    for (uint32_t ks = 0; ks < 8; ++ks)
        ldsm_x4(smem_addr(kbuf[0]) + tile_off(warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), 2 * ks + (lane >> 4)), qa[ks]);
    const uint32_t row_a = qt * 64 + warp * 16 + g, row_b = row_a + 8;   // the two query rows of this thread
    __syncthreads();     // every warp holds its fragments: kbuf[0] may be overwritten

    // S tile = Q K^T for the 64 keys in `tile`: sacc[nb] covers keys 8 nb .. 8 nb + 7
    // Consecutive MMAs go to different accumulators (four key blocks side by side): a chain of dependent mma.sync
    // would wait out the result latency after every instruction.
    auto scores = [&](const uint8_t* tile, float (&sacc)[8][4]) {
#pragma unroll
        for (uint32_t nb = 0; nb < 8; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[nb][e] = 0.0f;
#pragma unroll
        for (uint32_t nb0 = 0; nb0 < 8; nb0 += 4) {
#pragma unroll
            for (uint32_t ks2 = 0; ks2 < 4; ++ks2) {   // two 16-d steps per ldmatrix.x4
                uint32_t kf[4][4];
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j)
                    ldsm_x4(smem_addr(tile) + tile_off((nb0 + j) * 8 + (lane & 7), 4 * ks2 + (lane >> 3)), kf[j]);
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) mma_bf16(sacc[nb0 + j], qa[2 * ks2], kf[j][0], kf[j][1]);
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) mma_bf16(sacc[nb0 + j], qa[2 * ks2 + 1], kf[j][2], kf[j][3]);
            }
        }
    };

    // ---- pass 1: row maxima over every visible key; K tile kt sits in kbuf[(kt + 1) & 1] ----
    float ma = ninf, mb = ninf;
    for (uint32_t kt = 0; kt <= qt; ++kt) {
        if (kt < qt) {
            load_tile_async(kbuf[kt & 1], kb, kHeadDim, (kt + 1) * 64, S);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        float sacc[8][4];
        scores(kbuf[(kt + 1) & 1], sacc);
#pragma unroll
        for (uint32_t nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (uint32_t e = 0; e < 2; ++e) {
                const uint32_t key = kt * 64 + nb * 8 + 2 * tq + e;
                if (key <= row_a) ma = fmaxf(ma, cmath::mul(sacc[nb][e], scale));
                if (key <= row_b) mb = fmaxf(mb, cmath::mul(sacc[nb][2 + e], scale));
            }
        }
        __syncthreads();     // the buffer read here is the target of the load issued at the top of the next step
    }
    ma = fmaxf(ma, __shfl_xor_sync(0xFFFFFFFFu, ma, 1));
    ma = fmaxf(ma, __shfl_xor_sync(0xFFFFFFFFu, ma, 2));
    mb = fmaxf(mb, __shfl_xor_sync(0xFFFFFFFFu, mb, 1));
    mb = fmaxf(mb, __shfl_xor_sync(0xFFFFFFFFu, mb, 2));

    // ---- pass 2: probabilities and O += P V; K tile kt sits in kbuf[kt & 1], V tile kt in v_tile ----
    float oacc[16][4];
#pragma unroll
    for (int db = 0; db < 16; ++db)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[db][e] = 0.0f;
    float la = 0.0f, lb = 0.0f;
    load_tile_async(kbuf[0], kb, kHeadDim, 0, S);
    load_tile_async(v_tile, vb, kHeadDim, 0, S);
    for (uint32_t kt = 0; kt <= qt; ++kt) {
        // groups in flight, oldest first: K(kt), V(kt) [, K(kt+1)]
        if (kt < qt) {
            load_tile_async(kbuf[(kt + 1) & 1], kb, kHeadDim, (kt + 1) * 64, S);
            cp_async_wait<2>();
        } else {
            cp_async_wait<1>();
        }
        __syncthreads();
        float sacc[8][4];
        scores(kbuf[kt & 1], sacc);
        // probabilities in place (masked keys: 0), denominators in ascending key order
#pragma unroll
        for (uint32_t nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (uint32_t e = 0; e < 2; ++e) {
                const uint32_t key = kt * 64 + nb * 8 + 2 * tq + e;
                const float pa = key <= row_a ? exp_approx_nonpos(cmath::sub(cmath::mul(sacc[nb][e], scale), ma)) : 0.0f;
                const float pb = key <= row_b ? exp_approx_nonpos(cmath::sub(cmath::mul(sacc[nb][2 + e], scale), mb)) : 0.0f;
                sacc[nb][e] = pa;
                sacc[nb][2 + e] = pb;
                la = cmath::add(la, pa);
                lb = cmath::add(lb, pb);
            }
        }
        if (kt < qt) cp_async_wait<1>(); else cp_async_wait<0>();     // V(kt) has landed (K(kt+1) may still fly)
        __syncthreads();
#pragma unroll
        for (uint32_t kk = 0; kk < 4; ++kk) {   // 16 keys per step
            uint32_t phi[4], plo[4];
#pragma unroll
            for (uint32_t half = 0; half < 2; ++half)         // n-blocks 2kk (keys 0..7) and 2kk+1 (keys 8..15)
#pragma unroll
                for (uint32_t rr = 0; rr < 2; ++rr)           // row g, row g + 8
                    split_hi_lo(sacc[2 * kk + half][2 * rr], sacc[2 * kk + half][2 * rr + 1], phi[half * 2 + rr], plo[half * 2 + rr]);
#pragma unroll
            for (uint32_t db0 = 0; db0 < 8; db0 += 4) {       // eight 8-d blocks at a time: hi parts into all, then lo parts
                uint32_t vf[4][4];
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j)              // two 8-d blocks per ldmatrix.x4.trans
                    ldsm_x4_trans(smem_addr(v_tile) + tile_off(kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), 2 * (db0 + j) + (lane >> 4)), vf[j]);
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) {
                    mma_bf16(oacc[2 * (db0 + j)], phi, vf[j][0], vf[j][1]);
                    mma_bf16(oacc[2 * (db0 + j) + 1], phi, vf[j][2], vf[j][3]);
                }
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) {
                    mma_bf16(oacc[2 * (db0 + j)], plo, vf[j][0], vf[j][1]);
                    mma_bf16(oacc[2 * (db0 + j) + 1], plo, vf[j][2], vf[j][3]);
                }
            }
        }
        __syncthreads();     // v_tile and kbuf[kt & 1] are free again
        if (kt < qt) load_tile_async(v_tile, vb, kHeadDim, (kt + 1) * 64, S);
    }
    la = cmath::add(la, __shfl_xor_sync(0xFFFFFFFFu, la, 1));
    la = cmath::add(la, __shfl_xor_sync(0xFFFFFFFFu, la, 2));
    lb = cmath::add(lb, __shfl_xor_sync(0xFFFFFFFFu, lb, 1));
    lb = cmath::add(lb, __shfl_xor_sync(0xFFFFFFFFu, lb, 2));

    __nv_bfloat16* ob = out + ((size_t)b * S * Hq + h) * kHeadDim;
#pragma unroll
    for (uint32_t db = 0; db < 16; ++db) {
        const uint32_t d = db * 8 + 2 * tq;
        if (row_a < S)
            *reinterpret_cast<uint32_t*>(ob + (size_t)row_a * Hq * kHeadDim + d) = pack_bf16(cmath::div(oacc[db][0], la), cmath::div(oacc[db][1], la));
        if (row_b < S)
            *reinterpret_cast<uint32_t*>(ob + (size_t)row_b * Hq * kHeadDim + d) = pack_bf16(cmath::div(oacc[db][2], lb), cmath::div(oacc[db][3], lb));
    }
}

}  // namespace llama

// ================================================================ host side
static int grid_for(uint64_t work_items, int threads) {
    int sms = tls().sm_count > 0 ? tls().sm_count : 148;
    uint64_t blocks = ceil_div_u64(work_items, (uint64_t)threads);
    uint64_t cap = (uint64_t)sms * 8;
    return (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
}
// Launch on the thread's stream with programmatic stream serialisation allowed (see pdl_trigger / pdl_wait).
template <class... KArgs, class... Args>
static catena_status_t launch_pdl(const char* what, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = tls().stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) return fail_cuda(e, what);
    count_launch();
    return CATENA_OK;
}
static catena_status_t launched(const char* what) {
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? CATENA_OK : fail_cuda(e, what);
}

// inverse frequencies base^(-2i/128), i < 64, on the device (one table per thread, device and base)
struct RopeTable {
    float* dev = nullptr;
    uint32_t base_bits = 0;
};
static thread_local RopeTable g_rope[16];
static thread_local uint32_t* g_embed_bad[16] = {nullptr};

static catena_status_t rope_table(float base, const float** out) {
    RopeTable& t = g_rope[tls().device];
    const uint32_t bits = cmath::to_bits(base);
    if (!t.dev) CATENA_CUDA(cudaMalloc(&t.dev, 64 * sizeof(float)));
    if (t.base_bits != bits) {
        float host[64];
        for (uint32_t i = 0; i < 64; ++i) {
            const float e = -cmath::div(cmath::u32_to_f32(2 * i), 128.0f);
            host[i] = cmath::powf_approx(base, e);
        }
        CATENA_CUDA(cudaMemcpyAsync(t.dev, host, sizeof(host), cudaMemcpyHostToDevice, tls().stream));
        CATENA_CUDA(cudaStreamSynchronize(tls().stream));   // `host` is a stack array
        t.base_bits = bits;
    }
    *out = t.dev;
    return CATENA_OK;
}

static catena_status_t launch_embed(const void* table, const int32_t* ids, void* out, uint64_t tokens, uint64_t hidden, uint64_t vocab) {
    if (hidden % 8) return fail(CATENA_E_BAD_ARG, "embed: hidden must be a multiple of 8");
    if (!tokens) return CATENA_OK;
    uint32_t*& bad = g_embed_bad[tls().device];
    if (!bad) {
        CATENA_CUDA(cudaMalloc(&bad, sizeof(uint32_t)));
        CATENA_CUDA(cudaMemset(bad, 0, sizeof(uint32_t)));
    }
    return launch_pdl("embed_rows_kernel", llama::embed_rows_kernel, dim3((unsigned)tokens), dim3(128), 0, (const uint4*)table, ids,
                      (uint4*)out, (uint32_t)(hidden / 8), (uint32_t)vocab, bad);
}
// reports (and clears) an out-of-range token id seen by an earlier embedding launch; synchronises the stream
static catena_status_t embed_check() {
    uint32_t*& bad = g_embed_bad[tls().device];
    if (!bad) return CATENA_OK;
    uint32_t h = 0;
    CATENA_CUDA(cudaMemcpyAsync(&h, bad, sizeof(h), cudaMemcpyDeviceToHost, tls().stream));
    CATENA_CUDA(cudaStreamSynchronize(tls().stream));
    if (h) {
        cudaMemsetAsync(bad, 0, sizeof(uint32_t), tls().stream);
        return fail(CATENA_E_ASSERT, "embed: token id outside the table");
    }
    return CATENA_OK;
}
static catena_status_t launch_rmsnorm_rows(const void* x, void* y, uint64_t rows, uint64_t hidden) {
    if (hidden % 8) return fail(CATENA_E_BAD_ARG, "rmsnorm: hidden must be a multiple of 8");
    if (!rows) return CATENA_OK;
    return launch_pdl("rmsnorm_rows_kernel", llama::rmsnorm_rows_kernel, dim3((unsigned)rows), dim3(256), 0, (const uint4*)x,
                      (const int32_t*)nullptr, 0u, (uint32_t*)nullptr, (uint4*)nullptr, (uint4*)y, (uint32_t)hidden);
}
// (cos, sin) table of one call, [seq][64], in a per-thread buffer that only grows
struct RopeAngles {
    float2* dev = nullptr;
    uint64_t positions = 0;
};
static thread_local RopeAngles g_rope_angles[16];

// x = table[ids], y = rmsnorm(x) in one launch
static catena_status_t launch_embed_rmsnorm(const void* table, const int32_t* ids, void* x, void* y, uint64_t tokens, uint64_t hidden,
                                            uint64_t vocab) {
    if (hidden % 8) return fail(CATENA_E_BAD_ARG, "embed: hidden must be a multiple of 8");
    if (!tokens) return CATENA_OK;
    uint32_t*& bad = g_embed_bad[tls().device];
    if (!bad) {
        CATENA_CUDA(cudaMalloc(&bad, sizeof(uint32_t)));
        CATENA_CUDA(cudaMemset(bad, 0, sizeof(uint32_t)));
    }
    return launch_pdl("rmsnorm_rows_kernel", llama::rmsnorm_rows_kernel, dim3((unsigned)tokens), dim3(256), 0, (const uint4*)table, ids,
                      (uint32_t)vocab, bad, (uint4*)x, (uint4*)y, (uint32_t)hidden);
}
// enqueues the (cos, sin) table of positions pos0 .. pos0 + seq - 1 into the thread's buffer
static catena_status_t launch_rope_angles(const float* inv, uint64_t seq, uint64_t pos0, const float2** table) {
    RopeAngles& ra = g_rope_angles[tls().device];
    if (ra.positions < seq) {
        if (ra.dev) {
            CATENA_CUDA(cudaStreamSynchronize(tls().stream));
            CATENA_CUDA(cudaFree(ra.dev));
            ra.dev = nullptr;
        }
        CATENA_CUDA(cudaMalloc(&ra.dev, seq * 64 * sizeof(float2)));
        ra.positions = seq;
    }
    CATENA_TRY(launch_pdl("rope_table_kernel", llama::rope_table_kernel, dim3((unsigned)ceil_div_u64(seq * 64, 256)), dim3(256), 0, inv,
                          ra.dev, (uint32_t)pos0, (uint32_t)seq));
    *table = ra.dev;
    return CATENA_OK;
}
// q/k/v projection of a prefill with the rotation and the cache append in the GEMM's epilogue (no [tokens, qkv] matrix,
// no separate pass over it); false when the shape has to take the projection followed by launch_rope_append
static bool qkv_rope_fusable(uint64_t tokens, uint64_t seq, uint64_t hq, uint64_t hkv) {
    return seq >= 16 && tokens / seq * (hq + hkv) >= 8 && gemm_tc_fuses_residual(tokens) && tokens <= 0xFFFFFFFFull;
}
static catena_status_t launch_qkv_rope(const void* x, const void* w_qkv, void* q_out, void* k_cache, void* v_cache, uint64_t tokens,
                                       uint64_t seq, uint64_t pos0, uint64_t hq, uint64_t hkv, uint64_t cap, uint64_t hidden, float base) {
    if (seq == 0 || tokens % seq) return fail(CATENA_E_BAD_ARG, "rope: tokens must be batch * seq");
    if (pos0 + seq > cap) return fail(CATENA_E_BAD_ARG, "rope: positions beyond the cache capacity");
    const float* inv = nullptr;
    CATENA_TRY(rope_table(base, &inv));
    GemmRopeOut ro = {};
    CATENA_TRY(launch_rope_angles(inv, seq, pos0, &ro.table));
    ro.q_out = q_out;
    ro.k_cache = k_cache;
    ro.v_cache = v_cache;
    ro.seq = (uint32_t)seq;
    ro.pos0 = (uint32_t)pos0;
    ro.hq = (uint32_t)hq;
    ro.hkv = (uint32_t)hkv;
    ro.cap = (uint32_t)cap;
    return launch_gemm_tc_rope(x, w_qkv, tokens, (hq + 2 * hkv) * llama::kHeadDim, hidden, ro);
}
static catena_status_t launch_rope_append(const void* qkv, void* q_out, void* k_cache, void* v_cache, uint64_t tokens, uint64_t seq,
                                          uint64_t pos0, uint64_t hq, uint64_t hkv, uint64_t cap, float base) {
    if (!tokens) return CATENA_OK;
    if (seq == 0 || tokens % seq) return fail(CATENA_E_BAD_ARG, "rope: tokens must be batch * seq");
    if (pos0 + seq > cap) return fail(CATENA_E_BAD_ARG, "rope: positions beyond the cache capacity");
    // the kernels take 32-bit token, position and head counts, and one thread per (token, head, pair)
    if (tokens > 0xFFFFFFFFull || cap > 0xFFFFFFFFull || hq + 2 * hkv > 0xFFFFull || tokens * (hq + 2 * hkv) > (1ull << 40))
        return fail(CATENA_E_TOO_LARGE, "rope: more tokens, cache rows or heads than the kernels index");
    const float* inv = nullptr;
    CATENA_TRY(rope_table(base, &inv));
    if (seq >= 16 && tokens / seq * (hq + hkv) >= 8) {   // many (sequence, head) pairs per position: evaluate each angle once
        const float2* table = nullptr;
        CATENA_TRY(launch_rope_angles(inv, seq, pos0, &table));
        const uint64_t work = tokens * (hq + 2 * hkv) * 8;
        return launch_pdl("rope_append_kernel", llama::rope_append_kernel, dim3((unsigned)ceil_div_u64(work, 256)), dim3(256), 0,
                          (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
                          table, (uint32_t)tokens, (uint32_t)seq, (uint32_t)pos0, (uint32_t)hq, (uint32_t)hkv, (uint32_t)cap);
    }
    const uint64_t work = tokens * (hq + 2 * hkv) * 64;
    return launch_pdl("rope_append_small_kernel", llama::rope_append_small_kernel, dim3((unsigned)ceil_div_u64(work, 128)), dim3(128), 0,
                      (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, inv,
                      (uint32_t)tokens, (uint32_t)seq, (uint32_t)pos0, (uint32_t)hq, (uint32_t)hkv, (uint32_t)cap);
}
// A decode step's q/k/v projection with rotation and cache append in the epilogue; false when the shape has to take the
// projection followed by launch_rope_append.
static bool qkv_rope_skinny_fusable(uint64_t tokens, uint64_t seq, uint64_t hq, uint64_t hkv, uint64_t hidden) {
    if (seq != 1 || tokens == 0 || tokens > 16 || hidden == 0 || hidden % 8 || hidden > 0x7FFFFFFFull || hq + 2 * hkv > 0xFFFFull) return false;
    const int sms = tls().sm_count > 0 ? tls().sm_count : 148;
    const uint64_t groups = (hq + 2 * hkv) * 16, slots = (uint64_t)sms * llama::kSkinnyCtasPerSm;
    return ceil_div_u64(groups, slots) <= (uint64_t)llama::kSkinnyRopeGroups;
}
static catena_status_t launch_qkv_rope_skinny(const void* x, const void* w_qkv, void* q_out, void* k_cache, void* v_cache, uint64_t tokens,
                                              uint64_t pos, uint64_t hq, uint64_t hkv, uint64_t cap, uint64_t hidden, float base) {
    if (pos >= cap || cap > 0xFFFFFFFFull) return fail(CATENA_E_BAD_ARG, "rope: positions beyond the cache capacity");
    if (((uintptr_t)x | (uintptr_t)w_qkv) & 15) return fail(CATENA_E_BAD_ARG, "linear: operands must be 16-byte aligned");
    const float* inv = nullptr;
    CATENA_TRY(rope_table(base, &inv));
    const int sms = tls().sm_count > 0 ? tls().sm_count : 148;
    const uint64_t groups = (hq + 2 * hkv) * 16, slots = (uint64_t)sms * llama::kSkinnyCtasPerSm;
    const uint64_t rounds = ceil_div_u64(groups, slots);
    llama::SkinnyRope rope = {(__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nullptr,
                              (uint32_t)hq, (uint32_t)hkv, (uint32_t)cap, (uint32_t)pos};
    return launch_pdl("skinny_qkv_rope_kernel", llama::skinny_qkv_rope_kernel, dim3((unsigned)ceil_div_u64(groups, rounds)), dim3(256), 0,
                      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w_qkv, (uint32_t)tokens, (uint32_t)((hq + 2 * hkv) * llama::kHeadDim),
                      (uint32_t)hidden, rope, inv);
}
// Kernel selection for the prefill attention: the tcgen05 kernel (attn_prefill_tc.cu) unless CATENA_B200_PREFILL_TC=0
// (read once) or the test hook asks for the mma.sync kernel of this file; both implement the same semantics.
bool attn_prefill_tc_supports(const void* q, const void* k_cache, const void* v_cache, uint64_t hq, uint64_t hkv);
catena_status_t enqueue_attn_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out, uint64_t batch,
                                        uint64_t seq, uint64_t hq, uint64_t hkv, uint64_t cap);
catena_status_t attn_prefill_tc_check_errors();
static int g_prefill_tc_mode = -1;
static bool prefill_tc_mode() {
    if (g_prefill_tc_mode < 0) {
        const char* e = getenv("CATENA_B200_PREFILL_TC");
        g_prefill_tc_mode = (e && e[0] == '0') ? 0 : 1;
    }
    return g_prefill_tc_mode == 1;
}
void attn_prefill_set_tc_mode(int on) { g_prefill_tc_mode = on ? 1 : 0; }

static catena_status_t launch_attn_prefill(const void* q, const void* k_cache, const void* v_cache, void* out, uint64_t batch,
                                           uint64_t seq, uint64_t hq, uint64_t hkv, uint64_t cap) {
    if (!batch || !seq) return CATENA_OK;
    if (hkv == 0 || hq % hkv) return fail(CATENA_E_UNSUPPORTED, "attn_prefill: Hq must be a multiple of Hkv");
    if (seq > cap) return fail(CATENA_E_BAD_ARG, "attn_prefill: sequence beyond the cache capacity");
    if (prefill_tc_mode() && attn_prefill_tc_supports(q, k_cache, v_cache, hq, hkv))
        return enqueue_attn_prefill_tc(q, k_cache, v_cache, out, batch, seq, hq, hkv, cap);
    static thread_local bool attr_set = false;
    if (!attr_set) {
        CATENA_CUDA(cudaFuncSetAttribute(llama::attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 49152));
        attr_set = true;
    }
    dim3 grid((unsigned)ceil_div_u64(seq, 64), (unsigned)hq, (unsigned)batch);
    return launch_pdl("attn_prefill_kernel", llama::attn_prefill_kernel, grid, dim3(128), 49152, (const __nv_bfloat16*)q,
                      (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out, (uint32_t)seq, (uint32_t)hq,
                      (uint32_t)hkv, (uint32_t)cap, 1.0f / sqrtf(128.0f));
}
static catena_status_t launch_swiglu(const void* gu, void* a, uint64_t tokens, uint64_t ffn) {
    if (ffn % 8) return fail(CATENA_E_BAD_ARG, "swiglu: ffn must be a multiple of 8");
    if (!tokens) return CATENA_OK;
    return launch_pdl("swiglu_kernel", llama::swiglu_kernel, dim3(grid_for(tokens * (ffn / 8), 256)), dim3(256), 0, (const uint4*)gu,
                      (uint4*)a, tokens, (uint32_t)(ffn / 8));
}
static catena_status_t launch_add(const void* x, const void* y, void* out, uint64_t n) {
    if (n % 8) return fail(CATENA_E_BAD_ARG, "add: length must be a multiple of 8");
    if (!n) return CATENA_OK;
    return launch_pdl("add_rows_kernel", llama::add_rows_kernel, dim3(grid_for(n / 8, 256)), dim3(256), 0, (const uint4*)x, (const uint4*)y,
                      (uint4*)out, n / 8);
}
// y[M,N] = x[M,K] w[N,K]^T (+ res): the skinny kernel for M <= 16, else the tcgen05 GEMM followed by the residual add
static catena_status_t launch_linear(const void* x, const void* w, const void* res, void* y, uint64_t m, uint64_t n, uint64_t k) {
    if (!m || !n) return CATENA_OK;
    if (k == 0 || k % 8) return fail(CATENA_E_BAD_ARG, "linear: K must be a positive multiple of 8");
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return fail(CATENA_E_BAD_ARG, "linear: operands must be 16-byte aligned");
    if (m <= 16) {
        if (n > 0x7FFFFFFFull || k > 0x7FFFFFFFull) return fail(CATENA_E_TOO_LARGE, "linear: dimension too large");
        int sms = tls().sm_count > 0 ? tls().sm_count : 148;
        // persistent CTAs (two per SM), the same number of row groups for each of them where possible
        const uint64_t groups = ceil_div_u64(n, 8), slots = (uint64_t)sms * llama::kSkinnyCtasPerSm;
        const uint64_t rounds = ceil_div_u64(groups, slots);
        const unsigned grid = (unsigned)ceil_div_u64(groups, rounds);
        return launch_pdl("skinny_gemm_kernel", llama::skinny_gemm_kernel, dim3(grid), dim3(256), 0, (const __nv_bfloat16*)x,
                          (const __nv_bfloat16*)w, (const __nv_bfloat16*)res, (__nv_bfloat16*)y, (uint32_t)m, (uint32_t)n, (uint32_t)k, 0u);
    }
    // the CTA-pair kernel adds the residual in its epilogue (the same two roundings as the GEMM followed by the add)
    if (res && gemm_tc_fuses_residual(m) && !(((uintptr_t)res | (uintptr_t)y) & 15)) return launch_gemm_tc_residual(x, w, y, m, n, k, n, res);
    CATENA_TRY(launch_gemm_tc(x, w, y, m, n, k, n, 0));
    if (res) CATENA_TRY(launch_add(y, res, y, m * n));
    return CATENA_OK;
}

// act [m, ffn] = silu(x w_gate^T) * (x w_up^T) with w = [2 ffn, k] (gate rows, then up rows): one launch for m <= 16,
// else the GEMM into `gu` [m, 2 ffn] followed by the SwiGLU kernel
static catena_status_t launch_linear_swiglu(const void* x, const void* w, void* gu, void* act, uint64_t m, uint64_t ffn, uint64_t k) {
    if (!m || !ffn) return CATENA_OK;
    if (ffn % 8) return fail(CATENA_E_BAD_ARG, "swiglu: ffn must be a multiple of 8");
    if (m <= 16 && k % 8 == 0 && k > 0 && ffn <= 0x3FFFFFFFull && k <= 0x7FFFFFFFull && !(((uintptr_t)x | (uintptr_t)w) & 15)) {
        int sms = tls().sm_count > 0 ? tls().sm_count : 148;
        const uint64_t groups = ffn / 8, slots = (uint64_t)sms * llama::kSkinnyCtasPerSm;
        const uint64_t rounds = ceil_div_u64(groups, slots);
        const unsigned grid = (unsigned)ceil_div_u64(groups, rounds);
        return launch_pdl("skinny_gemm_kernel", llama::skinny_gemm_kernel, dim3(grid), dim3(256), 0, (const __nv_bfloat16*)x,
                          (const __nv_bfloat16*)w, (const __nv_bfloat16*)nullptr, (__nv_bfloat16*)act, (uint32_t)m, (uint32_t)(2 * ffn),
                          (uint32_t)k, (uint32_t)ffn);
    }
    // the CTA-pair kernel applies the activation in its epilogue (gate and up rows of the same outputs side by side in one tile)
    if (gemm_tc_fuses_residual(m) && ffn % 128 == 0 && k % 8 == 0 && !(((uintptr_t)x | (uintptr_t)w | (uintptr_t)act) & 15))
        return launch_gemm_tc_swiglu(x, w, act, m, ffn, k);
    CATENA_TRY(launch_linear(x, w, nullptr, gu, m, 2 * ffn, k));
    return launch_swiglu(gu, act, m, ffn);
}

// Runs `body` with per-launch synchronisation switched off, then restores the mode and (when blocking) waits
// once and reports any device-side error of the kernels used.
template <class F>
static catena_status_t composite(F body) {
    CATENA_TRY(ensure_device());
    const int was_blocking = tls().blocking;
    tls().blocking = 0;
    catena_status_t s = body();
    tls().blocking = was_blocking;
    if (s != CATENA_OK) return s;
    if (was_blocking) {
        CATENA_CUDA(cudaStreamSynchronize(tls().stream));
        CATENA_TRY(gemm_tc_check_errors());
        CATENA_TRY(attn_check_errors());
        CATENA_TRY(attn_prefill_tc_check_errors());
        CATENA_TRY(decode_fused_check_errors());
        CATENA_TRY(embed_check());
    }
    return CATENA_OK;
}

struct BlockDims {
    uint64_t H, Hq, Hkv, F, qkv_cols;
};
static catena_status_t check_block(const catena_llama_block_t* blk, BlockDims* d) {
    if (!blk || !blk->embedding || !blk->w_qkv || !blk->w_o || !blk->w_gate_up || !blk->w_down)
        return fail(CATENA_E_BAD_ARG, "llama: null block or weights");
    d->H = blk->hidden; d->Hq = blk->n_heads; d->Hkv = blk->n_kv_heads; d->F = blk->ffn;
    if (d->H == 0 || d->H % 16 || d->F == 0 || d->F % 16) return fail(CATENA_E_BAD_ARG, "llama: hidden and ffn must be multiples of 16");
    if (d->Hkv == 0 || d->Hq % d->Hkv || d->Hq / d->Hkv > 8) return fail(CATENA_E_UNSUPPORTED, "llama: heads must be a multiple (<= 8) of kv heads");
    if (blk->max_len == 0 || blk->vocab == 0) return fail(CATENA_E_BAD_ARG, "llama: empty cache or vocabulary");
    d->qkv_cols = (d->Hq + 2 * d->Hkv) * llama::kHeadDim;
    return CATENA_OK;
}
// workspace (bf16 elements per token): x, n, q, attn, x2 [H or Hq*128 each], qkv, gu [2F], a [F]
static uint64_t workspace_elems_per_token(const BlockDims& d) {
    return 3 * d.H + 2 * d.Hq * llama::kHeadDim + d.qkv_cols + 3 * d.F;
}

static catena_status_t run_block(const catena_llama_block_t* blk, const int32_t* ids, uint64_t batch, uint64_t seq, uint64_t pos0,
                                 void* k_cache, void* v_cache, void* out, void* workspace, uint64_t workspace_bytes) {
    BlockDims d;
    CATENA_TRY(check_block(blk, &d));
    if (!ids || !k_cache || !v_cache || !out || !workspace) return fail(CATENA_E_BAD_ARG, "llama: null argument");
    const uint64_t T = batch * seq;
    if (!T) return CATENA_OK;
    if (pos0 + seq > blk->max_len) return fail(CATENA_E_BAD_ARG, "llama: positions beyond max_len");
    // token counts and per-token workspace offsets are 32-bit in the kernels
    if (T > 0xFFFFFFFFull || blk->max_len > 0xFFFFFFFFull || T * workspace_elems_per_token(d) > (1ull << 46))
        return fail(CATENA_E_TOO_LARGE, "llama: more tokens than the kernels index");
    if (workspace_bytes < T * workspace_elems_per_token(d) * 2) return fail(CATENA_E_BAD_ARG, "llama: workspace too small");
    if ((uintptr_t)workspace & 255) return fail(CATENA_E_BAD_ARG, "llama: workspace must be 256-byte aligned");
    __nv_bfloat16* ws = static_cast<__nv_bfloat16*>(workspace);
    __nv_bfloat16* x = ws;                                   ws += T * d.H;
    __nv_bfloat16* nrm = ws;                                 ws += T * d.H;
    __nv_bfloat16* x2 = ws;                                  ws += T * d.H;
    __nv_bfloat16* q = ws;                                   ws += T * d.Hq * llama::kHeadDim;
    __nv_bfloat16* att = ws;                                 ws += T * d.Hq * llama::kHeadDim;
    __nv_bfloat16* qkv = ws;                                 ws += T * d.qkv_cols;
    __nv_bfloat16* gu = ws;                                  ws += T * 2 * d.F;
    __nv_bfloat16* act = ws;
    return composite([&]() -> catena_status_t {
        const bool fused_step = seq == 1 && !((uintptr_t)out & 15);
        if (fused_step && (decode_fused_mode() & 2) && decode_head_supported(T, d.H, d.Hq, d.Hkv) && !(((uintptr_t)k_cache | (uintptr_t)v_cache) & 15)) {
            // a decode step, when asked for: embedding, norm, q/k/v projection, rotation and cache append in one persistent kernel
            const float* inv = nullptr;
            CATENA_TRY(rope_table(blk->rope_base, &inv));
            uint32_t*& bad = g_embed_bad[tls().device];
            if (!bad) {
                CATENA_CUDA(cudaMalloc(&bad, sizeof(uint32_t)));
                CATENA_CUDA(cudaMemset(bad, 0, sizeof(uint32_t)));
            }
            CATENA_TRY(launch_decode_head(blk->embedding, ids, blk->w_qkv, inv, bad, x, qkv, q, k_cache, v_cache, T, d.H, blk->vocab, d.Hq,
                                          d.Hkv, blk->max_len, pos0));
        } else {
        CATENA_TRY(launch_embed_rmsnorm(blk->embedding, ids, x, nrm, T, d.H, blk->vocab));
        if (qkv_rope_fusable(T, seq, d.Hq, d.Hkv) && !(((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15)) {
            CATENA_TRY(launch_qkv_rope(nrm, blk->w_qkv, q, k_cache, v_cache, T, seq, pos0, d.Hq, d.Hkv, blk->max_len, d.H, blk->rope_base));
        } else if ((decode_fused_mode() & 4) && qkv_rope_skinny_fusable(T, seq, d.Hq, d.Hkv, d.H)) {
            CATENA_TRY(launch_qkv_rope_skinny(nrm, blk->w_qkv, q, k_cache, v_cache, T, pos0, d.Hq, d.Hkv, blk->max_len, d.H, blk->rope_base));
        } else {
            CATENA_TRY(launch_linear(nrm, blk->w_qkv, nullptr, qkv, T, d.qkv_cols, d.H));
            CATENA_TRY(launch_rope_append(qkv, q, k_cache, v_cache, T, seq, pos0, d.Hq, d.Hkv, blk->max_len, blk->rope_base));
        }
        }
        if (seq == 1) {
            // While the attention runs (latency-bound for a cache of a few thousand rows) it prefetches into L2 what the
            // projections behind it will stream first: W_o, then the leading gate and up rows, then the leading down rows.
            static const uint64_t budget = [] { const char* v = getenv("CATENA_B200_DECODE_PREFETCH_MB"); return (uint64_t)(v ? atoi(v) : 0) << 20; }();
            static const uint32_t pace = [] { const char* v = getenv("CATENA_B200_DECODE_PREFETCH_PACE_NS"); return (uint32_t)(v ? atoi(v) : 400); }();
            AttnPrefetch pf = {};
            if (budget) {
                uint64_t left = budget;
                auto add = [&](const void* p, uint64_t bytes) {
                    const uint64_t take = bytes < left ? bytes : left;
                    if (take >= 16384 && pf.n < 4) { pf.ptr[pf.n] = p; pf.bytes[pf.n] = take; ++pf.n; left -= take; }
                };
                const uint64_t wo = d.H * d.Hq * llama::kHeadDim * 2, half = d.F * d.H * 2;
                add(blk->w_o, wo);
                const uint64_t gu = left / 2 < half ? left / 2 : half;
                add(blk->w_gate_up, gu);
                add(static_cast<const char*>(blk->w_gate_up) + half, gu);
                add(blk->w_down, d.H * d.F * 2);
                pf.pace_ns = pace;
            }
            CATENA_TRY(launch_attn_decode(q, k_cache, v_cache, att, batch, d.Hq, d.Hkv, llama::kHeadDim, pos0 + 1, blk->max_len, 0,
                                          batch * d.Hkv, nullptr, 0, pf.n ? &pf : nullptr));
        } else {
            if (pos0 != 0) return fail(CATENA_E_UNSUPPORTED, "llama: a multi-token step must start at position 0");
            CATENA_TRY(launch_attn_prefill(q, k_cache, v_cache, att, batch, seq, d.Hq, d.Hkv, blk->max_len));
        }
        if (fused_step && (decode_fused_mode() & 1) && decode_tail_supported(T, d.H, d.Hq * llama::kHeadDim, d.F)) {
            // a decode step, when asked for: everything after the attention in one persistent kernel (llama_decode_fused.cu), same bits
            return launch_decode_tail(att, x, blk->w_o, blk->w_gate_up, blk->w_down, x2, act, out, T, d.H, d.Hq * llama::kHeadDim, d.F);
        }
        CATENA_TRY(launch_linear(att, blk->w_o, x, x2, T, d.H, d.Hq * llama::kHeadDim));
        CATENA_TRY(launch_rmsnorm_rows(x2, nrm, T, d.H));
        CATENA_TRY(launch_linear_swiglu(nrm, blk->w_gate_up, gu, act, T, d.F, d.H));
        CATENA_TRY(launch_linear(act, blk->w_down, x2, out, T, d.H, d.F));
        return CATENA_OK;
    });
}

extern "C" {

uint64_t catena_b200_llama_workspace_bytes(const catena_llama_block_t* blk, uint64_t tokens) {
    BlockDims d;
    if (check_block(blk, &d) != CATENA_OK) return 0;
    return tokens * workspace_elems_per_token(d) * 2;
}
catena_status_t catena_b200_llama_prefill(const catena_llama_block_t* blk, const int32_t* ids, uint64_t batch, uint64_t seq,
                                          void* k_cache, void* v_cache, void* out, void* workspace, uint64_t workspace_bytes) {
    return run_block(blk, ids, batch, seq, 0, k_cache, v_cache, out, workspace, workspace_bytes);
}
catena_status_t catena_b200_llama_decode(const catena_llama_block_t* blk, const int32_t* ids, uint64_t batch, uint64_t pos,
                                         void* k_cache, void* v_cache, void* out, void* workspace, uint64_t workspace_bytes) {
    return run_block(blk, ids, batch, 1, pos, k_cache, v_cache, out, workspace, workspace_bytes);
}

catena_status_t catena_b200_embed_bf16_into(const void* table, const int32_t* ids, void* out, uint64_t tokens, uint64_t hidden,
                                            uint64_t vocab) {
    if (!table || !ids || !out) return fail(CATENA_E_BAD_ARG, "embed: null argument");
    return composite([&]() { return launch_embed(table, ids, out, tokens, hidden, vocab); });
}
catena_status_t catena_b200_rmsnorm_rows_bf16_into(const void* x, void* y, uint64_t rows, uint64_t hidden) {
    if (!x || !y) return fail(CATENA_E_BAD_ARG, "rmsnorm: null argument");
    return composite([&]() { return launch_rmsnorm_rows(x, y, rows, hidden); });
}
catena_status_t catena_b200_rope_append_bf16_into(const void* qkv, void* q_out, void* k_cache, void* v_cache, uint64_t tokens,
                                                  uint64_t seq, uint64_t pos0, uint64_t n_heads, uint64_t n_kv_heads, uint64_t cap,
                                                  float rope_base) {
    if (!qkv || !q_out || !k_cache || !v_cache) return fail(CATENA_E_BAD_ARG, "rope: null argument");
    return composite([&]() { return launch_rope_append(qkv, q_out, k_cache, v_cache, tokens, seq, pos0, n_heads, n_kv_heads, cap, rope_base); });
}
catena_status_t catena_b200_attn_prefill_bf16_into(const void* q, const void* k_cache, const void* v_cache, void* out, uint64_t batch,
                                                   uint64_t seq, uint64_t n_heads, uint64_t n_kv_heads, uint64_t cap) {
    if (!q || !k_cache || !v_cache || !out) return fail(CATENA_E_BAD_ARG, "attn_prefill: null argument");
    return composite([&]() { return launch_attn_prefill(q, k_cache, v_cache, out, batch, seq, n_heads, n_kv_heads, cap); });
}
catena_status_t catena_b200_attn_decode_bf16_cache_into(const void* q, const void* k_cache, const void* v_cache, void* o, uint64_t batch,
                                                        uint64_t hq, uint64_t hkv, uint64_t d, uint64_t kv_len, uint64_t kv_cap) {
    return composite([&]() { return launch_attn_decode(q, k_cache, v_cache, o, batch, hq, hkv, d, kv_len, kv_cap, 0, batch * hkv); });
}
void catena_b200_debug_set_prefill_tc(int on) { attn_prefill_set_tc_mode(on); }
catena_status_t catena_b200_swiglu_bf16_into(const void* gate_up, void* out, uint64_t tokens, uint64_t ffn) {
    if (!gate_up || !out) return fail(CATENA_E_BAD_ARG, "swiglu: null argument");
    return composite([&]() { return launch_swiglu(gate_up, out, tokens, ffn); });
}
catena_status_t catena_b200_linear_swiglu_bf16_into(const void* x, const void* w_gate_up, void* scratch, void* out, uint64_t m,
                                                    uint64_t ffn, uint64_t k) {
    if (!x || !w_gate_up || !out || (m > 16 && !scratch)) return fail(CATENA_E_BAD_ARG, "linear_swiglu: null argument");
    return composite([&]() { return launch_linear_swiglu(x, w_gate_up, scratch, out, m, ffn, k); });
}
catena_status_t catena_b200_add_bf16_into(const void* x, const void* y, void* out, uint64_t n) {
    if (!x || !y || !out) return fail(CATENA_E_BAD_ARG, "add: null argument");
    return composite([&]() { return launch_add(x, y, out, n); });
}
catena_status_t catena_b200_linear_bf16_into(const void* x, const void* w, const void* residual, void* y, uint64_t m, uint64_t n,
                                             uint64_t k) {
    if (!x || !w || !y) return fail(CATENA_E_BAD_ARG, "linear: null argument");
    return composite([&]() { return launch_linear(x, w, residual, y, m, n, k); });
}

}  // extern "C"

}  // namespace catena
