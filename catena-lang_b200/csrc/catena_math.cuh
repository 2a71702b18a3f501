// Scalar arithmetic of the catena stdlib as `__host__ __device__` functions whose results are
// bit-identical on host and device and independent of compiler flags: every f32 operation is an
// explicitly rounded intrinsic on the device (`__fmul_rn`, `__fadd_rn`, ... are never contracted
// into FMAs, whatever -fmad says) and a plain operator on the host (the host objects are built
// with -ffp-contract=off).  This is the determinism contract the reference gets from
// `--fmad=false` (catena-lang/src/runtime/artifact.rs:59-80) and from `f32.mul`/`f32.add` being
// separate C expressions (catena-lang/src/codegen/gpu.rs:322-447).
//
// Formulas and constants: catena-lang/stdlib/math.hex and catena-lang/stdlib/nn.hex (cited per
// function).  The polynomials are the reference's own low-order approximations — they are part
// of the semantics (math.exp-approx(0) is 0x3F7FF8FC, not 1).
#pragma once

#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#define CM_HD __host__ __device__ __forceinline__

namespace cmath {

#ifdef __CUDA_ARCH__
CM_HD float mul(float a, float b) { return __fmul_rn(a, b); }
CM_HD float add(float a, float b) { return __fadd_rn(a, b); }
CM_HD float sub(float a, float b) { return __fsub_rn(a, b); }
CM_HD float div(float a, float b) { return __fdiv_rn(a, b); }
// 1.0f / x: the correctly rounded reciprocal IS the IEEE quotient of 1 and x, at a fraction of the cost
CM_HD float recip(float x) { return __frcp_rn(x); }
CM_HD float from_bits(uint32_t u) { return __uint_as_float(u); }
CM_HD uint32_t to_bits(float f) { return __float_as_uint(f); }
CM_HD uint32_t round_to_u32(float x) { return __float2uint_rn(x); }   // (uint32_t)nearbyintf(x), gpu.rs:642-655
CM_HD float u32_to_f32(uint32_t x) { return __uint2float_rn(x); }
CM_HD float u64_to_f32(uint64_t x) { return __ull2float_rn(x); }
#else
CM_HD float mul(float a, float b) { return a * b; }
CM_HD float add(float a, float b) { return a + b; }
CM_HD float sub(float a, float b) { return a - b; }
CM_HD float div(float a, float b) { return a / b; }
CM_HD float recip(float x) { return 1.0f / x; }
CM_HD float from_bits(uint32_t u) { union { uint32_t u; float f; } v; v.u = u; return v.f; }
CM_HD uint32_t to_bits(float f) { union { uint32_t u; float f; } v; v.f = f; return v.u; }
CM_HD uint32_t round_to_u32(float x) { return (uint32_t)nearbyintf(x); }
CM_HD float u32_to_f32(uint32_t x) { return (float)x; }
CM_HD float u64_to_f32(uint64_t x) { return (float)x; }
#endif

// math.hex:3-23
CM_HD float sin_approx(float x) {
    float x2 = mul(x, x), x3 = mul(x2, x), x5 = mul(x3, x2), x7 = mul(x5, x2);
    float p1 = sub(x, div(x3, 6.0f));
    float p2 = add(p1, div(x5, 120.0f));
    return sub(p2, div(x7, 5040.0f));
}

// math.hex:27-47
CM_HD float cos_approx(float x) {
    float x2 = mul(x, x), x4 = mul(x2, x2), x6 = mul(x4, x2);
    float p1 = sub(1.0f, div(x2, 2.0f));
    float p2 = add(p1, div(x4, 24.0f));
    return sub(p2, div(x6, 720.0f));
}

// math.hex:52-87 (Cody-Waite reduction by pi/2, quadrant select)
CM_HD float sin_full_nonneg(float x) {
    uint32_t n = round_to_u32(mul(x, from_bits(0x3F22F983u)));
    float nf = u32_to_f32(n);
    float r = sub(sub(x, mul(nf, from_bits(0x3FC90FDAu))), mul(nf, from_bits(0x33A22168u)));
    float s = sin_approx(r), c = cos_approx(r);
    uint32_t q = n & 3u;
    float q23 = (q == 2u) ? -s : -c;
    float q123 = (q == 1u) ? c : q23;
    return (q == 0u) ? s : q123;
}

// math.hex:91-103
CM_HD float sin_full(float x) {
    bool neg = x < 0.0f;
    float base = sin_full_nonneg(neg ? -x : x);
    return neg ? -base : base;
}

// math.hex:110-144
CM_HD float log_approx(float x) {
    uint32_t xb = to_bits(x);
    float m = from_bits((xb & 0x007FFFFFu) + 0x3F000000u);
    float e = sub(u32_to_f32(xb >> 23), 126.0f);
    float p2 = add(from_bits(0xC03AA687u), mul(m, from_bits(0x3F60A4E1u)));
    float p1 = add(from_bits(0x4087355Au), mul(m, p2));
    float poly = add(from_bits(0xC00BE629u), mul(m, p1));
    return add(poly, mul(e, from_bits(0x3F317218u)));
}

// math.hex:148-183
CM_HD float exp_nonneg(float x) {
    uint32_t k = round_to_u32(mul(x, from_bits(0x3FB8AA3Bu)));
    float kf = u32_to_f32(k);
    float xr = sub(sub(x, mul(kf, from_bits(0x3F317200u))), mul(kf, from_bits(0x35BFBE8Eu)));
    float p2 = add(from_bits(0x3EEF1187u), mul(xr, from_bits(0x3E738A8Bu)));
    float p1 = add(from_bits(0x3F809C7Eu), mul(xr, p2));
    float poly = add(from_bits(0x3F7FF8FCu), mul(xr, p1));
    uint32_t pow2_bits = (k + 0x7Fu) * 0x00800000u;  // wraps in u32, as in the reference
    return mul(poly, from_bits(pow2_bits));
}

// math.hex:185-199
CM_HD float exp_approx(float x) {
    bool neg = x < 0.0f;
    float base = exp_nonneg(neg ? -x : x);
    return neg ? recip(base) : base;
}

// math.hex:202-231
CM_HD float exp2_approx(float x) { return exp_approx(mul(x, from_bits(0x3F317218u))); }
CM_HD float log2_approx(float x) { return mul(log_approx(x), from_bits(0x3FB8AA3Bu)); }
CM_HD float powf_approx(float x, float y) { return exp2_approx(mul(y, log2_approx(x))); }

// math.hex:235-272 (six Newton steps from max(1, x); 0 for x <= 0)
CM_HD float sqrt_newton(float x) {
    float g = (x < 1.0f) ? 1.0f : x;
#pragma unroll
    for (int it = 0; it < 6; ++it) g = mul(add(g, div(x, g)), 0.5f);
    return (x <= 0.0f) ? 0.0f : g;
}

// nn.hex:2-56
CM_HD float sigmoid(float x) { return recip(add(1.0f, exp_approx(-x))); }
CM_HD float silu(float x) { return mul(x, sigmoid(x)); }
CM_HD float tanh_approx(float x) { return sub(mul(sigmoid(mul(x, 2.0f)), 2.0f), 1.0f); }
CM_HD float gelu_approx(float x) {
    float x3 = mul(mul(x, x), x);
    float inner = add(x, mul(x3, from_bits(0x3D372713u)));
    float shaped = tanh_approx(mul(inner, from_bits(0x3F4C422Au)));
    return mul(mul(x, add(1.0f, shaped)), 0.5f);
}

enum MapOp {
    OP_SIN_APPROX = 0, OP_COS_APPROX, OP_SIN_FULL_NONNEG, OP_SIN_FULL, OP_LOG, OP_EXP_NONNEG, OP_EXP,
    OP_EXP2, OP_LOG2, OP_SQRT, OP_SIGMOID, OP_SILU, OP_TANH, OP_GELU, OP_COUNT
};

template <int OP>
CM_HD float apply(float x) {
    if (OP == OP_SIN_APPROX) return sin_approx(x);
    if (OP == OP_COS_APPROX) return cos_approx(x);
    if (OP == OP_SIN_FULL_NONNEG) return sin_full_nonneg(x);
    if (OP == OP_SIN_FULL) return sin_full(x);
    if (OP == OP_LOG) return log_approx(x);
    if (OP == OP_EXP_NONNEG) return exp_nonneg(x);
    if (OP == OP_EXP) return exp_approx(x);
    if (OP == OP_EXP2) return exp2_approx(x);
    if (OP == OP_LOG2) return log2_approx(x);
    if (OP == OP_SQRT) return sqrt_newton(x);
    if (OP == OP_SIGMOID) return sigmoid(x);
    if (OP == OP_SILU) return silu(x);
    if (OP == OP_TANH) return tanh_approx(x);
    return gelu_approx(x);
}

#ifdef __CUDACC__
// Correctly rounded 1 / p for 0.5 <= p < 2^100 without the range checks and the call of the general routine: the
// hardware approximation, one Newton step, then one more whose residual is taken against the refined value
// (Markstein's final correction).  catena_b200_debug_rcp_check (attn_prefill_tc.cu) compares it with __frcp_rn over every float of that
// range; the caller takes the general routine when any argument of a batch is outside it.
constexpr float kRcpFastBelow = 1.2676506e30f;   // 2^100
__device__ __forceinline__ float rcp_fast(float p) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(p));
    float e = __fmaf_rn(-p, r, 1.0f);
    r = __fmaf_rn(r, e, r);
    e = __fmaf_rn(-p, r, 1.0f);
    return __fmaf_rn(r, e, r);
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// ---- the exp~ family for W values at once, stage by stage across them (W dependency chains in flight) -------------------
// When every |x| <= 64 the steps that carry range checks take short forms that are bit-identical there: the
// round-to-nearest-even of t = |x| * log2(e) < 2^22 goes through the 1.5 * 2^23 constant (same integer, same float),
// exp~(|x|) < 2^94 so its reciprocal and that of 1 + exp~(-x) in [1, 2^94] are rcp_fast's.  One larger magnitude
// sends the whole batch through the scalar functions above.  NaNs pass the test and come out as NaNs either way.
template <int W>
__device__ __forceinline__ bool all_within_64(const float (&x)[W]) {
    float big = fabsf(x[0]);
#pragma unroll
    for (int u = 1; u + 1 < W; u += 2) big = max3(big, fabsf(x[u]), fabsf(x[u + 1]));
    if (W % 2 == 0) big = fmaxf(big, fabsf(x[W - 1]));
    return big <= 64.0f;
}
// ---- packed f32x2 arithmetic (sm_100): one instruction, two separately rounded IEEE operations ---------------------------
// A PRODUCT is written as fma(a, b, -0) with the -0 read from constant memory: ptxas merges a packed mul with the packed add or
// sub that consumes it into one fma — explicit .rn and --fmad=false notwithstanding (measured: the results are those of
// fma.rn.f32x2) — which would round once.  An fma whose addend the assembler cannot see stays an fma, and a * b + (-0) is
// exactly the rounded product (a zero product keeps its sign).  Sums, differences and genuine fmas need no such care.
static __constant__ unsigned long long c_neg_zero2 = 0x8000000080000000ull;
__device__ __forceinline__ uint64_t pk2f(float lo, float hi) { uint64_t d; asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi)); return d; }
__device__ __forceinline__ uint64_t pk2u(uint32_t lo, uint32_t hi) { uint64_t d; asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi)); return d; }
__device__ __forceinline__ void unpk2f(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ void unpk2u(uint64_t v, uint32_t& lo, uint32_t& hi) { asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) { uint64_t d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) { uint64_t d; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) { uint64_t d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) { return fma2(a, b, c_neg_zero2); }
__host__ __device__ constexpr uint64_t twice(uint32_t bits) { return ((uint64_t)bits << 32) | bits; }
// rcp_fast for two values: the same approximation and the same four fused steps per value
__device__ __forceinline__ uint64_t rcp_fast2(uint64_t p) {
    float p0, p1, r0, r1;
    unpk2f(p, p0, p1);
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(p0));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r1) : "f"(p1));
    const uint64_t np = p ^ twice(0x80000000u);
    uint64_t r = pk2f(r0, r1);
    uint64_t e = fma2(np, r, twice(0x3F800000u));
    r = fma2(r, e, r);
    e = fma2(np, r, twice(0x3F800000u));
    return fma2(r, e, r);
}

// exp~(x) for a batch that passed all_within_64: two values per instruction when W is even (same operations, same order,
// same roundings as the scalar stages)
template <int W>
__device__ __forceinline__ void exp_fast_n(const float (&x)[W], float (&out)[W]) {
    if constexpr (W % 2 == 0) {
        constexpr int H = W / 2;
        uint64_t mag[H], sh[H], xr[H], p[H];
#pragma unroll
        for (int q = 0; q < H; ++q) mag[q] = pk2f(fabsf(x[2 * q]), fabsf(x[2 * q + 1]));
#pragma unroll
        for (int q = 0; q < H; ++q) sh[q] = add2(mul2(mag[q], twice(0x3FB8AA3Bu)), twice(0x4B400000u));     // + 12582912
#pragma unroll
        for (int q = 0; q < H; ++q) p[q] = sub2(sh[q], twice(0x4B400000u));                                   // kf
#pragma unroll
        for (int q = 0; q < H; ++q) xr[q] = sub2(mag[q], mul2(p[q], twice(0x3F317200u)));
#pragma unroll
        for (int q = 0; q < H; ++q) xr[q] = sub2(xr[q], mul2(p[q], twice(0x35BFBE8Eu)));
#pragma unroll
        for (int q = 0; q < H; ++q) p[q] = add2(twice(0x3EEF1187u), mul2(xr[q], twice(0x3E738A8Bu)));
#pragma unroll
        for (int q = 0; q < H; ++q) p[q] = add2(twice(0x3F809C7Eu), mul2(xr[q], p[q]));
#pragma unroll
        for (int q = 0; q < H; ++q) p[q] = add2(twice(0x3F7FF8FCu), mul2(xr[q], p[q]));
#pragma unroll
        for (int q = 0; q < H; ++q) {
            uint32_t s0, s1;
            unpk2u(sh[q], s0, s1);
            p[q] = mul2(p[q], pk2u((s0 - 0x4B400000u + 0x7Fu) * 0x00800000u, (s1 - 0x4B400000u + 0x7Fu) * 0x00800000u));
        }
#pragma unroll
        for (int q = 0; q < H; ++q) {
            float a, b, ra, rb;
            unpk2f(p[q], a, b);
            unpk2f(rcp_fast2(p[q]), ra, rb);
            out[2 * q] = x[2 * q] < 0.0f ? ra : a;
            out[2 * q + 1] = x[2 * q + 1] < 0.0f ? rb : b;
        }
    } else {
        float mag[W], sh[W], kf[W], xr[W], p[W];
#pragma unroll
        for (int u = 0; u < W; ++u) mag[u] = fabsf(x[u]);
#pragma unroll
        for (int u = 0; u < W; ++u) sh[u] = add(mul(mag[u], from_bits(0x3FB8AA3Bu)), 12582912.0f);
#pragma unroll
        for (int u = 0; u < W; ++u) kf[u] = sub(sh[u], 12582912.0f);
#pragma unroll
        for (int u = 0; u < W; ++u) xr[u] = sub(mag[u], mul(kf[u], from_bits(0x3F317200u)));
#pragma unroll
        for (int u = 0; u < W; ++u) xr[u] = sub(xr[u], mul(kf[u], from_bits(0x35BFBE8Eu)));
#pragma unroll
        for (int u = 0; u < W; ++u) p[u] = add(from_bits(0x3EEF1187u), mul(xr[u], from_bits(0x3E738A8Bu)));
#pragma unroll
        for (int u = 0; u < W; ++u) p[u] = add(from_bits(0x3F809C7Eu), mul(xr[u], p[u]));
#pragma unroll
        for (int u = 0; u < W; ++u) p[u] = add(from_bits(0x3F7FF8FCu), mul(xr[u], p[u]));
#pragma unroll
        for (int u = 0; u < W; ++u) p[u] = mul(p[u], from_bits((to_bits(sh[u]) - 0x4B400000u + 0x7Fu) * 0x00800000u));
#pragma unroll
        for (int u = 0; u < W; ++u) out[u] = x[u] < 0.0f ? rcp_fast(p[u]) : p[u];
    }
}
template <int W>
__device__ __forceinline__ void exp_approx_n(const float (&x)[W], float (&out)[W]) {
    if (all_within_64(x)) {
        exp_fast_n(x, out);
    } else {
#pragma unroll
        for (int u = 0; u < W; ++u) out[u] = exp_approx(x[u]);
    }
}
template <int W>
__device__ __forceinline__ void sigmoid_n(const float (&x)[W], float (&out)[W]) {
    if (all_within_64(x)) {
        float nx[W], e[W];
#pragma unroll
        for (int u = 0; u < W; ++u) nx[u] = -x[u];
        exp_fast_n(nx, e);
        if constexpr (W % 2 == 0) {
#pragma unroll
            for (int q = 0; q < W / 2; ++q)
                unpk2f(rcp_fast2(add2(twice(0x3F800000u), pk2f(e[2 * q], e[2 * q + 1]))), out[2 * q], out[2 * q + 1]);
        } else {
#pragma unroll
            for (int u = 0; u < W; ++u) out[u] = rcp_fast(add(1.0f, e[u]));
        }
    } else {
#pragma unroll
        for (int u = 0; u < W; ++u) out[u] = sigmoid(x[u]);
    }
}
template <int W>
__device__ __forceinline__ void silu_n(const float (&x)[W], float (&out)[W]) {
    float s[W];
    sigmoid_n(x, s);
#pragma unroll
    for (int u = 0; u < W; ++u) out[u] = mul(x[u], s[u]);
}
template <int W>
__device__ __forceinline__ void tanh_n(const float (&x)[W], float (&out)[W]) {
    float y[W], s[W];
#pragma unroll
    for (int u = 0; u < W; ++u) y[u] = mul(x[u], 2.0f);
    sigmoid_n(y, s);
#pragma unroll
    for (int u = 0; u < W; ++u) out[u] = sub(mul(s[u], 2.0f), 1.0f);
}
template <int W>
__device__ __forceinline__ void gelu_n(const float (&x)[W], float (&out)[W]) {
    float z[W], t[W];
#pragma unroll
    for (int u = 0; u < W; ++u) {
        const float x3 = mul(mul(x[u], x[u]), x[u]);
        z[u] = mul(add(x[u], mul(x3, from_bits(0x3D372713u))), from_bits(0x3F4C422Au));
    }
    tanh_n(z, t);
#pragma unroll
    for (int u = 0; u < W; ++u) out[u] = mul(mul(x[u], add(1.0f, t[u])), 0.5f);
}
// apply<OP> to W values: the exp~ family in its batched form, everything else value by value
template <int OP, int W>
__device__ __forceinline__ void apply_n(const float (&x)[W], float (&out)[W]) {
    if (OP == OP_EXP) {
        exp_approx_n(x, out);
    } else if (OP == OP_EXP2) {
        float y[W];
#pragma unroll
        for (int u = 0; u < W; ++u) y[u] = mul(x[u], from_bits(0x3F317218u));
        exp_approx_n(y, out);
    } else if (OP == OP_SIGMOID) {
        sigmoid_n(x, out);
    } else if (OP == OP_SILU) {
        silu_n(x, out);
    } else if (OP == OP_TANH) {
        tanh_n(x, out);
    } else if (OP == OP_GELU) {
        gelu_n(x, out);
    } else {
#pragma unroll
        for (int u = 0; u < W; ++u) out[u] = apply<OP>(x[u]);
    }
}
#endif

}  // namespace cmath
