// Skinny GEMM (at most 16 activation rows) as device code shared by the stand-alone kernel (llama.cu) and the fused
// decode-step kernels (llama_decode_fused.cu): the arithmetic — which warp takes which k blocks, the order of the MMAs, the
// order in which the warps' partial sums are added, the roundings of the epilogues — lives here once, so every kernel
// that uses it produces the same bits.
//
// y[m, n] = sum_k x[m, k] * w[n, k], optionally + res[m, n]; x [M, K] bf16, w [N, K] bf16 (K contiguous), y [M, N] bf16.
// HBM-bound on w: every weight is read exactly once, 16 bytes per lane, and the few rows of x ride along as the other
// operand of mma.sync m16n8k16 (tokens = the 16 rows of A, 8 weight rows = the columns of B).  On CUDA cores the
// unfused multiply-adds of even 4 tokens would cost as many issue slots as the weights cost bandwidth.
// A CTA owns 8 weight rows at a time; its 8 warps take the 32-wide k blocks round-robin (warp v: blocks v, v+8, ...) and
// their partial sums are added in ascending warp order.  Inside a k block lane (g, t) holds k = 8t..8t+7 of weight row g
// and of tokens g, g+8: the MMA's k index is a permutation of the true one, the same for both operands.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

#include "catena_math.cuh"

namespace catena {
namespace llama {

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
#ifndef CATENA_SKINNY_UNROLL
#define CATENA_SKINNY_UNROLL 8
#endif
#ifndef CATENA_SKINNY_CTAS
#define CATENA_SKINNY_CTAS 2
#endif
constexpr int kSkinnyUnroll = CATENA_SKINNY_UNROLL;   // 16-byte weight loads per lane and batch (a batch is issued at once)
constexpr int kSkinnyCtasPerSm = CATENA_SKINNY_CTAS;  // resident CTAs per SM the stand-alone kernel is sized for

// How the activations (and the residual) are read: through the read-only path when no kernel in flight writes them, with
// L2-coherent loads when an earlier phase of the SAME kernel wrote them, with plain loads from shared memory.
enum SkinnyA { A_READONLY = 0, A_COHERENT = 1, A_SHARED = 2 };
template <int MODE>
__device__ __forceinline__ uint4 skinny_load_a(const __nv_bfloat16* p) {
    if (MODE == A_READONLY) return __ldg(reinterpret_cast<const uint4*>(p));
    if (MODE == A_SHARED) return *reinterpret_cast<const uint4*>(p);
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ float skinny_load_res(const __nv_bfloat16* p, bool coherent) {
    if (!coherent) return __bfloat162float(*p);
    uint16_t h;
    asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(h) : "l"(p));
    return __uint_as_float((uint32_t)h << 16);
}

// One product.  With swiglu_f = F > 0 the weights are the [2F, K] gate / up matrix and y [M, F] = silu(gate) * up: a CTA
// multiplies the 8 gate rows of a group, then the matching 8 up rows, and combines them in the epilogue (both products
// rounded to bf16 first, exactly what a separate SwiGLU pass reads back from memory).
// Where a q/k/v projection of a decode step (every token its own sequence, all at position `pos`) puts its output instead of
// y: rotated queries into q_out [M, hq, 128], rotated keys and plain values into row `pos` of the caches [M, hkv, cap, 128].
// "Rotate half": pair i of a head is (i, i + 64), so a row group of such a job is rows 4q .. 4q+3 and 64+4q .. 64+4q+3 of one
// head (four whole pairs) instead of eight consecutive rows.  `cs` holds (cos, sin) of the CTA's pairs, [group of the CTA][4].
struct SkinnyRope {
    __nv_bfloat16* q_out;
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    const float2* cs;
    uint32_t hq, hkv, cap, pos;
};
struct SkinnyJob {
    const __nv_bfloat16* x;
    const __nv_bfloat16* w;
    const __nv_bfloat16* res;
    __nv_bfloat16* y;
    uint32_t M, N, K, swiglu_f;
    SkinnyRope rope;          // used by skinny_run<.., true> only
};
constexpr int kSkinnyRopeGroups = 8;      // row groups per CTA a rope job may have (the CTA's cos / sin table)
// weight row of lane group g (0..7) in row group `grp` of a rope job
__device__ __forceinline__ uint32_t skinny_rope_row(uint32_t grp, uint32_t g) { return (grp >> 4) * 128u + (grp & 15u) * 4u + (g & 3u) + (g >> 2) * 64u; }
// Schedule of a job over `nblocks` persistent CTAs: CTA `bid` takes the row groups bid, bid + nblocks, ...; a step is one
// batch of 8 * kSkinnyUnroll k blocks of one group (of its gate rows, then of its up rows).
struct SkinnySchedule {
    uint32_t kblocks, batches, halves, groups, steps, bid, nblocks, swiglu_f;
    __device__ __forceinline__ SkinnySchedule(const SkinnyJob& j, uint32_t bid_, uint32_t nblocks_) {
        bid = bid_;
        nblocks = nblocks_;
        swiglu_f = j.swiglu_f;
        kblocks = (j.K + 31) / 32;
        batches = (kblocks + 8 * kSkinnyUnroll - 1) / (8 * kSkinnyUnroll);
        halves = j.swiglu_f ? 2u : 1u;
        groups = j.swiglu_f ? j.swiglu_f / 8 : (j.N + 7) / 8;
        const uint32_t my_groups = bid < groups ? (groups - bid + nblocks - 1) / nblocks : 0;
        steps = my_groups * halves * batches;
    }
    __device__ __forceinline__ uint32_t row0_of(uint32_t s) const {   // first weight row of step s
        const uint32_t grp = bid + (s / (halves * batches)) * nblocks;
        return ((s / batches) % halves) * swiglu_f + grp * 8;
    }
};
// weights of step s: rows row0_of(s) .. +7, k blocks warp + 8 (u + kSkinnyUnroll (s % batches))
template <bool ROPE = false>
__device__ __forceinline__ void skinny_load_w(const SkinnyJob& j, const SkinnySchedule& sc, uint32_t s, uint4 (&wv)[kSkinnyUnroll]) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t n0 = sc.row0_of(s);
    const uint32_t row = ROPE ? skinny_rope_row(n0 / 8, g) : n0 + g;
    const uint32_t kb0 = warp + 8 * kSkinnyUnroll * (s % sc.batches);
    const __nv_bfloat16* wr = j.w + (size_t)row * j.K + 8 * t;
#pragma unroll
    for (int u = 0; u < kSkinnyUnroll; ++u) {
        const uint32_t k = (kb0 + 8 * u) * 32;
        wv[u] = make_uint4(0, 0, 0, 0);
        if (row < j.N && k + 8 * t < j.K)   // volatile: the whole batch is issued here, ahead of the (volatile) MMAs
            asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(wv[u].x), "=r"(wv[u].y), "=r"(wv[u].z), "=r"(wv[u].w)
                         : "l"(wr + k));
    }
}
// Runs the job's steps of this CTA.  `cur` already holds the weights of step 0 (skinny_load_w, issued by the caller as early
// as it can: weights are never written by a kernel).  Software-pipelined: the loads of step s + 1 are issued before step
// s is multiplied and reduced, so the stream never drains.  `part` is 8 x 16 x 8 floats of shared memory.
template <int A_MODE, bool ROPE = false>
__device__ __forceinline__ void skinny_run(const SkinnyJob& j, const SkinnySchedule& sc, float (*part)[16][8], uint4 (&cur)[kSkinnyUnroll],
                                           float (*pairs)[8] = nullptr) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const __nv_bfloat16* xa = j.x + (size_t)g * j.K + 8 * t;
    const __nv_bfloat16* xb = j.x + (size_t)(g + 8) * j.K + 8 * t;
    const uint32_t M = j.M, N = j.N, K = j.K, swiglu_f = j.swiglu_f, batches = sc.batches;
    uint4 nxt[kSkinnyUnroll];
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float gate = 0.0f;                   // SwiGLU: the gate value of this thread's (token, row) until the up rows are done
    for (uint32_t s = 0; s < sc.steps; ++s) {
        if (s + 1 < sc.steps) skinny_load_w<ROPE>(j, sc, s + 1, nxt);
        const uint32_t kb0 = warp + 8 * kSkinnyUnroll * (s % batches);
#pragma unroll
        for (int u = 0; u < kSkinnyUnroll; ++u) {
            const uint32_t k = (kb0 + 8 * u) * 32;
            const bool ok = k + 8 * t < K;
            const uint4 av = ok && g < M ? skinny_load_a<A_MODE>(xa + k) : zero;
            const uint4 bv = ok && g + 8 < M ? skinny_load_a<A_MODE>(xb + k) : zero;
            mma_bf16_16816(acc, av.x, bv.x, av.y, bv.y, cur[u].x, cur[u].y);
            mma_bf16_16816(acc, av.z, bv.z, av.w, bv.w, cur[u].z, cur[u].w);
        }
        if (s % batches == batches - 1) {    // the group is complete: add the warps' partial sums in ascending order
            const uint32_t n0 = sc.row0_of(s);
            __syncthreads();                 // the previous group's partials have been read
            part[warp][g][2 * t] = acc[0];
            part[warp][g][2 * t + 1] = acc[1];
            part[warp][g + 8][2 * t] = acc[2];
            part[warp][g + 8][2 * t + 1] = acc[3];
            acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
            __syncthreads();
            if (threadIdx.x < 128) {
                const uint32_t m = threadIdx.x >> 3, r = threadIdx.x & 7;
                if (m < M && n0 + r < N) {
                    float v = part[0][m][r];
#pragma unroll
                    for (int wv2 = 1; wv2 < 8; ++wv2) v = cmath::add(v, part[wv2][m][r]);
                    if (ROPE) {
                        pairs[m][r] = __bfloat162float(__float2bfloat16_rn(v));     // what a separate rotation pass reads back
                    } else if (swiglu_f) {
                        const float rounded = __bfloat162float(__float2bfloat16_rn(v));
                        if (n0 < swiglu_f) gate = rounded;
                        else j.y[(size_t)m * swiglu_f + (n0 - swiglu_f) + r] = __float2bfloat16_rn(cmath::mul(cmath::silu(gate), rounded));
                    } else {
                        if (j.res) v = cmath::add(__bfloat162float(__float2bfloat16_rn(v)), skinny_load_res(j.res + (size_t)m * N + n0 + r, A_MODE == A_COHERENT));
                        j.y[(size_t)m * N + n0 + r] = __float2bfloat16_rn(v);
                    }
                }
            }
            if (ROPE) {
                // rows r and r + 4 of the group are the two halves of pair 4q + r of one head: rotate (query and key heads) or
                // copy (value heads) and store where the attention reads — the arithmetic of rope_append_small_kernel
                __syncthreads();
                if (threadIdx.x < 64) {
                    const uint32_t m = threadIdx.x >> 2, r = threadIdx.x & 3, grp = n0 / 8, head = grp >> 4, i = (grp & 15u) * 4 + r;
                    if (m < M && head < j.rope.hq + 2 * j.rope.hkv) {
                        const float x1 = pairs[m][r], x2 = pairs[m][r + 4];
                        if (head >= j.rope.hq + j.rope.hkv) {
                            __nv_bfloat16* dst = j.rope.v_cache + (((size_t)m * j.rope.hkv + (head - j.rope.hq - j.rope.hkv)) * j.rope.cap + j.rope.pos) * 128;
                            dst[i] = __float2bfloat16_rn(x1);
                            dst[i + 64] = __float2bfloat16_rn(x2);
                        } else {
                            const float2 cs = j.rope.cs[(s / batches) * 4 + r];
                            __nv_bfloat16* dst = head < j.rope.hq ? j.rope.q_out + ((size_t)m * j.rope.hq + head) * 128
                                                                  : j.rope.k_cache + (((size_t)m * j.rope.hkv + (head - j.rope.hq)) * j.rope.cap + j.rope.pos) * 128;
                            dst[i] = __float2bfloat16_rn(cmath::sub(cmath::mul(x1, cs.x), cmath::mul(x2, cs.y)));
                            dst[i + 64] = __float2bfloat16_rn(cmath::add(cmath::mul(x2, cs.x), cmath::mul(x1, cs.y)));
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kSkinnyUnroll; ++u) cur[u] = nxt[u];
    }
}

}  // namespace llama
}  // namespace catena
