// Causal prefill attention on tcgen05 — the semantics of llama::attn_prefill_kernel (global row maximum first, then
// p = exp~(s - max) with the reference's polynomial, probabilities as a bf16 hi + lo pair, fp32 sums), with both
// contractions on the 5th-generation tensor cores:
//   S[128 queries x 128 keys] = Q_tile[128 x 128 d] * K_tile^T      A = Q in shared memory, B = K tile (both K-major,
//                                                                   128B swizzle, as TMA wrote them), D in TMEM
//   O[128 queries x 128 d]   += P[128 x 128 keys] * V_tile           A = P in TENSOR MEMORY (written by the consumer
//                                                                   threads with tcgen05.st), B = the V tile read as an
//                                                                   MN-major operand (no transpose), hi then lo
// One CTA per 128 queries of one head; a consumer thread owns one query row = one TMEM lane, so row maxima and row sums
// need no cross-thread reduction.  exp~ admits no online rescaling, hence two passes over the key tiles: pass 1
// multiplies Q K^T for the row maxima only, pass 2 multiplies again and accumulates P V.  A kernel that allocates TMEM
// gets one CTA per SM, and the polynomial is the bulk of the instructions, so the CTA carries FOUR consumer warpgroups;
// group g takes keys 32 g .. 32 g + 31 of every 128-key tile, and the four parts of a row's maximum and of its sum
// meet in shared memory (sum = ((part 0 + part 1) + part 2) + part 3, a fixed order).
//   warps 4g .. 4g+3  consumer group g (warp w reads TMEM lanes 32 (w % 4) ..)
//   warp 16    TMA producer (Q once, then K tiles / K and V tiles through a 5-stage ring of 32 KiB)
//   warp 17    MMA issuer; allocates the CTA's 512 TMEM columns: three score buffers of 128 columns, used round robin
//              by the sequence of score tiles (both passes), and the outputs at [384, 512).  The probabilities of 16
//              keys replace their 16 score columns in place: 8 columns of packed bf16 hi parts, then 8 of lo parts, each
//              an A operand of one K = 16 MMA.
// Tile width: a tcgen05.mma of M = 128 costs the issuer about as many cycles at N = 64 as at N = 128 (measured with
// the cycle accounting below: ~80 per instruction either way), so 64-key tiles made the tensor pipe the bottleneck
// (consumers waited for scores half of pass 2); 128-key tiles halve the score instructions per key.
// Score tiles run two ahead of the probabilities.  All waits are bounded.
#include <cuda.h>
#include <cuda_bf16.h>

#include <type_traits>

#include "catena_math.cuh"
#include "common.cuh"

namespace catena {

namespace attn3 {

constexpr int kD = 128;
constexpr int kTile = 128;                   // queries per CTA
constexpr int kKeys = 128;                   // keys per ring stage / score buffer
constexpr int kGroups = 4;                   // consumer warpgroups; each takes kKeys / kGroups = 32 keys of every tile
constexpr int kBufs = 3;                     // score buffers
constexpr int kStages = 5;
constexpr int kQBytes = 2 * kTile * 128;     // [d-half 2][row 128][128 B]
constexpr int kKeyHalfBytes = kKeys * 128;   // 16 KiB: 128 keys x 64 d
constexpr int kStageBytes = 2 * kKeyHalfBytes;
constexpr int kConsumers = 128;              // per group
constexpr int kThreads = kGroups * kConsumers + 64;
constexpr int kTmemCols = 512;
constexpr int kOCol = kBufs * kKeys;         // 384
constexpr uint64_t kWaitNs = 1000000000ull;
constexpr uint32_t kSuspendHintNs = 20000;

struct __align__(16) Control {
    uint64_t q_full;
    uint64_t full[kStages], empty[kStages];
    uint64_t s_full[kBufs], s_free[kBufs];   // score buffers
    uint64_t p_ready[kBufs];         // probabilities of the buffer written to TMEM
    uint64_t o_full;
    float xch[kGroups][kTile];       // per-row partial maxima / sums of the consumer groups
    uint32_t tmem_base;
    volatile uint32_t abort_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when it expired (about one second) or another thread of the CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Control* ctl, uint32_t* err) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 255u) == 0) {
            if (ctl->abort_flag) return false;
            if (globaltimer_ns() - t0 > kWaitNs) {
                ctl->abort_flag = 1;
                atomicCAS(err, 0u, 5u);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void tc_mma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptors (128B swizzle, descriptor version 1): K-major for Q and K tiles, MN-major for the
// V tile (rows of 128 B along N = 64 d; consecutive K = keys are consecutive rows; 8-key groups 1024 B apart = SBO;
// the second 64-d block `lbo` bytes away = LBO).
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr, uint32_t lbo) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// instruction descriptors: fp32 accumulate, bf16 operands, M = 128; N = 128 keys for the scores, N = 128 d for the outputs,
// where bit 16 says that B (the V tile) is MN-major
constexpr uint32_t kIdescQK = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kIdescPV = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24) | (1u << 16);

// math.exp-approx (catena-lang/stdlib/math.hex:148-199) for x <= 0, bit-identical to cmath::exp_approx there; the
// round-to-nearest-even of t in [0, 2^22) goes through the 1.5 * 2^23 constant (same integer, same float).
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
using cmath::kRcpFastBelow;
using cmath::max3;
using cmath::rcp_fast;
// The same function for kExpW (16) arguments, written stage by stage across them: that many independent dependency chains are
// in flight, so an instruction rarely waits for the result of the one before it (four warps share a scheduler here).
// 16 = the keys of one trip of the inner loop (0.295 ms against 0.300 ms with 8 on the 4 x 2048 x 16-head prefill).
// Arguments of masked keys must still be <= 0 (the caller passes 0 and discards the result).
#ifndef CATENA_PF_EXPW
#define CATENA_PF_EXPW 16
#endif
constexpr int kExpW = CATENA_PF_EXPW;
__device__ __forceinline__ void exp_approx_nonpos_n(const float (&x)[kExpW], float (&out)[kExpW]) {
    float mag[kExpW], sh[kExpW], kf[kExpW], xr[kExpW], p[kExpW];
#pragma unroll
    for (int u = 0; u < kExpW; ++u) mag[u] = -x[u];
#pragma unroll
    for (int u = 0; u < kExpW; ++u) sh[u] = cmath::add(cmath::mul(mag[u], cmath::from_bits(0x3FB8AA3Bu)), 12582912.0f);
#pragma unroll
    for (int u = 0; u < kExpW; ++u) kf[u] = cmath::sub(sh[u], 12582912.0f);
#pragma unroll
    for (int u = 0; u < kExpW; ++u) xr[u] = cmath::sub(mag[u], cmath::mul(kf[u], cmath::from_bits(0x3F317200u)));
#pragma unroll
    for (int u = 0; u < kExpW; ++u) xr[u] = cmath::sub(xr[u], cmath::mul(kf[u], cmath::from_bits(0x35BFBE8Eu)));
#pragma unroll
    for (int u = 0; u < kExpW; ++u) p[u] = cmath::add(cmath::from_bits(0x3EEF1187u), cmath::mul(xr[u], cmath::from_bits(0x3E738A8Bu)));
#pragma unroll
    for (int u = 0; u < kExpW; ++u) p[u] = cmath::add(cmath::from_bits(0x3F809C7Eu), cmath::mul(xr[u], p[u]));
#pragma unroll
    for (int u = 0; u < kExpW; ++u) p[u] = cmath::add(cmath::from_bits(0x3F7FF8FCu), cmath::mul(xr[u], p[u]));
#pragma unroll
    for (int u = 0; u < kExpW; ++u) p[u] = cmath::mul(p[u], cmath::from_bits((__float_as_uint(sh[u]) - 0x4B400000u + 0x7Fu) * 0x00800000u));
    // p >= 0.5 always (a polynomial near 1 times 2^k, k >= 0); NaNs pass the test and stay NaNs either way
    float big = p[0];
#pragma unroll
    for (int u = 1; u + 1 < kExpW; u += 2) big = max3(big, p[u], p[u + 1]);
    if (kExpW % 2 == 0) big = fmaxf(big, p[kExpW - 1]);
    if (big < kRcpFastBelow) {
#pragma unroll
        for (int u = 0; u < kExpW; ++u) out[u] = x[u] < 0.0f ? rcp_fast(p[u]) : p[u];
    } else {
#pragma unroll
        for (int u = 0; u < kExpW; ++u) out[u] = x[u] < 0.0f ? cmath::recip(p[u]) : p[u];
    }
}
// two probabilities -> packed bf16 hi parts and packed bf16 lo parts (p - hi)
__device__ __forceinline__ void split_hi_lo(float p0, float p1, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    const float r0 = cmath::sub(p0, __uint_as_float(hi << 16)), r1 = cmath::sub(p1, __uint_as_float(hi & 0xFFFF0000u));
    const __nv_bfloat162 l = __floats2bfloat162_rn(r0, r1);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

// ---- packed f32x2 arithmetic (sm_100): one instruction, two separately rounded IEEE operations --------------------------
// A product is written as fma(a, b, -0) with the -0 taken from a kernel ARGUMENT: ptxas merges a packed mul with the packed
// add or sub that consumes it into one fma (explicit .rn and --fmad=false notwithstanding), which would round once; an
// fma whose addend it cannot see stays an fma, and a * b + (-0) is exactly the rounded product.
__device__ __forceinline__ uint64_t pk2(uint32_t lo, uint32_t hi) { uint64_t d; asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi)); return d; }
__device__ __forceinline__ uint64_t pk2f(float lo, float hi) { uint64_t d; asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi)); return d; }
__device__ __forceinline__ void unpk2(uint64_t v, uint32_t& lo, uint32_t& hi) { asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) { uint64_t d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) { uint64_t d; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) { uint64_t d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__host__ __device__ constexpr uint64_t twice(uint32_t bits) { return ((uint64_t)bits << 32) | bits; }

// p[u] = exp~(scale * score[u] - m) for the 16 scores of one trip of the inner loop, none of them masked, two keys per
// instruction: the arithmetic of exp_approx_nonpos_n stage by stage (same operations, same order, same roundings), with
// mag = m - scale * score in place of -(scale * score - m) (round-to-nearest is symmetric, so the two are the same float).
__device__ __forceinline__ void exp_scores_packed(const uint32_t (&v)[16], uint64_t scale2, uint64_t m2, uint64_t nz2, float (&out)[16]) {
    uint64_t mag[8], sh[8], xr[8], p[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) mag[q] = sub2(m2, fma2(pk2(v[2 * q], v[2 * q + 1]), scale2, nz2));
#pragma unroll
    for (int q = 0; q < 8; ++q) sh[q] = add2(fma2(mag[q], twice(0x3FB8AA3Bu), nz2), twice(0x4B400000u));      // + 12582912
#pragma unroll
    for (int q = 0; q < 8; ++q) p[q] = sub2(sh[q], twice(0x4B400000u));                                        // kf
#pragma unroll
    for (int q = 0; q < 8; ++q) xr[q] = sub2(mag[q], fma2(p[q], twice(0x3F317200u), nz2));
#pragma unroll
    for (int q = 0; q < 8; ++q) xr[q] = sub2(xr[q], fma2(p[q], twice(0x35BFBE8Eu), nz2));
#pragma unroll
    for (int q = 0; q < 8; ++q) p[q] = add2(twice(0x3EEF1187u), fma2(xr[q], twice(0x3E738A8Bu), nz2));
#pragma unroll
    for (int q = 0; q < 8; ++q) p[q] = add2(twice(0x3F809C7Eu), fma2(xr[q], p[q], nz2));
#pragma unroll
    for (int q = 0; q < 8; ++q) p[q] = add2(twice(0x3F7FF8FCu), fma2(xr[q], p[q], nz2));
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        uint32_t s0, s1;
        unpk2(sh[q], s0, s1);
        p[q] = fma2(p[q], pk2((s0 - 0x4B400000u + 0x7Fu) * 0x00800000u, (s1 - 0x4B400000u + 0x7Fu) * 0x00800000u), nz2);
    }
    float pf[16], mg[16];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        uint32_t a, b;
        unpk2(p[q], a, b);
        pf[2 * q] = __uint_as_float(a);
        pf[2 * q + 1] = __uint_as_float(b);
        unpk2(mag[q], a, b);
        mg[2 * q] = __uint_as_float(a);
        mg[2 * q + 1] = __uint_as_float(b);
    }
    // p >= 0.5 always (a polynomial near 1 times 2^k, k >= 0); NaNs pass the test and stay NaNs either way
    float big = pf[0];
#pragma unroll
    for (int u = 1; u + 1 < 16; u += 2) big = max3(big, pf[u], pf[u + 1]);
    big = fmaxf(big, pf[15]);
    if (big < kRcpFastBelow) {
        // rcp_fast for two values at once: r = rcp.approx(p); e = 1 - p r; r += r e; e = 1 - p r; r += r e (fused steps)
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            float r0, r1;
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(pf[2 * q]));
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r1) : "f"(pf[2 * q + 1]));
            const uint64_t np = p[q] ^ twice(0x80000000u);
            uint64_t r = pk2f(r0, r1);
            uint64_t e = fma2(np, r, twice(0x3F800000u));
            r = fma2(r, e, r);
            e = fma2(np, r, twice(0x3F800000u));
            r = fma2(r, e, r);
            uint32_t a, b;
            unpk2(r, a, b);
            out[2 * q] = mg[2 * q] > 0.0f ? __uint_as_float(a) : pf[2 * q];
            out[2 * q + 1] = mg[2 * q + 1] > 0.0f ? __uint_as_float(b) : pf[2 * q + 1];
        }
    } else {
#pragma unroll
        for (int u = 0; u < 16; ++u) out[u] = mg[u] > 0.0f ? cmath::recip(pf[u]) : pf[u];
    }
}

// Optional cycle accounting of the consumers (build with -DCATENA_PF_PROFILE; one lane per consumer warp adds up where
// its cycles go): [0] whole kernel, [1] pass 1, [2] pass 2, [3] pass 2 waiting for scores, [4] first TMEM load of a
// tile, [5] waiting for the TMEM stores, [6] waiting for the outputs, [7] set-up before the roles start.
#ifdef CATENA_PF_PROFILE
__device__ unsigned long long g_pf_prof[16];
#define PF_T(var) const long long var = clock64()
#define PF_ADD(slot, cycles) do { if (lane == 0) atomicAdd(&g_pf_prof[slot], (unsigned long long)(cycles)); } while (0)
#else
#define PF_T(var) do { } while (0)
#define PF_ADD(slot, cycles) do { } while (0)
#endif

// grid (ceil(S / 128), Hq, B), 576 threads, one CTA per SM.
__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, uint32_t S, uint32_t Hq,
                       uint32_t Hkv, float scale, uint32_t* err, uint64_t neg_zero2) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* q_tile = smem;                                   // 32 KiB
    uint8_t* ring = smem + kQBytes;                           // kStages x 16 KiB
    Control* ctl = reinterpret_cast<Control*>(ring + kStages * kStageBytes);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    PF_T(pf_start);
    const uint32_t qt = gridDim.x - 1 - blockIdx.x;           // heavy tiles first
    const uint32_t h = blockIdx.y, b = blockIdx.z, kvh = h / (Hq / Hkv);
    const uint32_t n = qt + 1;                                // visible key tiles; the last one holds masked keys
    const int kv_unit = (int)(b * Hkv + kvh);
    constexpr uint32_t kProducerWarp = kGroups * 4, kIssuerWarp = kGroups * 4 + 1;

    if (tid == 0) {
        mbar_init(&ctl->q_full, 1);
        for (int s = 0; s < kStages; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
        for (int i = 0; i < kBufs; ++i) {
            mbar_init(&ctl->s_full[i], 1);
            mbar_init(&ctl->s_free[i], kGroups * kConsumers);   // all groups share every tile
            mbar_init(&ctl->p_ready[i], kGroups * kConsumers);
        }
        mbar_init(&ctl->o_full, 1);
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kIssuerWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                     "r"((uint32_t)kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;

    if (warp == kProducerWarp) {
        // =============================== TMA producer ===============================
        // ring order = the issuer's consumption order: pass 1  K(0) .. K(n-1);  pass 2  K(0) K(1) V(0) K(2) V(1) .. V(n-1)
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_q)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
            mbar_expect_tx(&ctl->q_full, kQBytes);
            tma_load_5d(smem_u32(q_tile), &map_q, 0, (int)(qt * kTile), 0, (int)h, (int)b, &ctl->q_full);
            uint32_t g = 0;
            bool ok = true;
            auto issue = [&](const CUtensorMap* map, uint32_t kt) {
                if (!ok) return;
                const uint32_t st = g % kStages;
                if (!mbar_wait(&ctl->empty[st], ((g / kStages) & 1u) ^ 1u, ctl, err)) { ok = false; return; }
                mbar_expect_tx(&ctl->full[st], kStageBytes);
                tma_load_4d(smem_u32(ring + st * kStageBytes), map, 0, (int)(kt * kKeys), 0, kv_unit, &ctl->full[st]);
                ++g;
            };
            for (uint32_t kt = 0; kt < n; ++kt) issue(&map_k, kt);
            for (uint32_t kt = 0; kt < n && kt < (uint32_t)kBufs - 1; ++kt) issue(&map_k, kt);
            for (uint32_t kt = 0; kt < n; ++kt) {
                if (kt + kBufs - 1 < n) issue(&map_k, kt + kBufs - 1);
                issue(&map_v, kt);
            }
        }
    } else if (warp == kIssuerWarp) {
        // =============================== MMA issuer ===============================
        if (lane == 0) {
            uint32_t g = 0, j = 0, jbuf = 0, jround = 0;     // ring position; score tile sequence number, j % kBufs, j / kBufs
            bool ok = mbar_wait(&ctl->q_full, 0, ctl, err);
            const uint32_t qa = smem_u32(q_tile);
            // S[buffer j % kBufs] = Q K^T with the K tile at the head of the ring
            auto score_tile = [&]() {
                if (!ok) return;
                PF_T(pf_a);
                if (!mbar_wait(&ctl->s_free[jbuf], (jround & 1u) ^ 1u, ctl, err)) { ok = false; return; }
                PF_T(pf_b);
                if (!mbar_wait(&ctl->full[g % kStages], (g / kStages) & 1u, ctl, err)) { ok = false; return; }
                PF_T(pf_c);
                PF_ADD(j < n ? 8 : 10, pf_b - pf_a);       // issuer: waiting for a free score buffer (pass 1 / pass 2)
                PF_ADD(j < n ? 9 : 11, pf_c - pf_b);       // issuer: waiting for the K tile
                tc_fence_after();
                const uint32_t ka = smem_u32(ring + (g % kStages) * kStageBytes);
#pragma unroll
                for (uint32_t ks = 0; ks < 8; ++ks)      // 16 d per MMA: d-half ks/4, 32 B steps inside the row
                    tc_mma_ss(tmem + jbuf * kKeys, desc_kmajor(qa + (ks >> 2) * (kQBytes / 2) + (ks & 3u) * 32),
                              desc_kmajor(ka + (ks >> 2) * kKeyHalfBytes + (ks & 3u) * 32), kIdescQK, ks != 0 ? 1u : 0u);
                tc_commit(&ctl->empty[g % kStages]);
                tc_commit(&ctl->s_full[jbuf]);
                PF_ADD(j < n ? 15 : 7, clock64() - pf_c);   // issuer: issuing the score MMAs and commits (pass 1 / pass 2; slot 7 shared with set-up)
                ++g;
                ++j;
                if (++jbuf == (uint32_t)kBufs) { jbuf = 0; ++jround; }
            };
            // pass 1
            for (uint32_t kt = 0; kt < n; ++kt) score_tile();
            // pass 2: the scores run kBufs - 1 tiles ahead of the probabilities; tile kt sits in buffer (n + kt) % kBufs
            for (uint32_t kt = 0; kt < n && kt < (uint32_t)kBufs - 1; ++kt) score_tile();
            uint32_t pbuf = n % kBufs;
            for (uint32_t kt = 0; kt < n && ok; ++kt) {
                if (kt + kBufs - 1 < n) score_tile();
                if (!ok) break;
                PF_T(pf_d);
                if (!mbar_wait(&ctl->p_ready[pbuf], (kt / kBufs) & 1u, ctl, err)) { ok = false; break; }
                PF_T(pf_e);
                if (!mbar_wait(&ctl->full[g % kStages], (g / kStages) & 1u, ctl, err)) { ok = false; break; }
                PF_T(pf_f);
                PF_ADD(12, pf_e - pf_d);                   // issuer: waiting for the probabilities
                PF_ADD(13, pf_f - pf_e);                   // issuer: waiting for the V tile
                tc_fence_after();
                const uint32_t va = smem_u32(ring + (g % kStages) * kStageBytes);
#pragma unroll
                for (uint32_t kk = 0; kk < (uint32_t)kKeys / 16; ++kk) {     // 16 keys: hi parts in 8 columns, lo parts in the next 8
                    const uint64_t vdesc = desc_mnmajor(va + kk * 2048, kKeyHalfBytes);
                    tc_mma_ts(tmem + kOCol, tmem + pbuf * kKeys + kk * 16, vdesc, kIdescPV, (kt | kk) != 0 ? 1u : 0u);
                    tc_mma_ts(tmem + kOCol, tmem + pbuf * kKeys + kk * 16 + 8, vdesc, kIdescPV, 1u);
                }
                tc_commit(&ctl->empty[g % kStages]);
                ++g;
                if (++pbuf == (uint32_t)kBufs) pbuf = 0;
            }
            if (ok) tc_commit(&ctl->o_full);
            PF_ADD(14, clock64() - pf_start);          // issuer: whole
        }
    } else {
        // =============================== consumers: group wg, thread r = query row r ===============================
        // All groups work on the same tile, a quarter of its keys each, so two multiplied tiles wait behind the one in work.
        const uint32_t wg = warp >> 2, r = tid & 127u, part = wg * (kKeys / kGroups);   // first key of this group's share
        const uint32_t row = qt * kTile + r;                         // position of this query in its sequence
        const uint32_t lane_addr = tmem + (((warp & 3u) * 32u) << 16);
        const float ninf = __uint_as_float(0xFF800000u);
        bool aborted = false;
        PF_T(pf_roles);
        PF_ADD(7, pf_roles - pf_start);
        // ---- pass 1: row maximum over this group's tiles (of the raw scores: scaling by a positive constant is
        // monotonic, so max_i fl(s_i * scale) = fl((max_i s_i) * scale); only the last tile has masked keys) ----
        float m_raw = ninf;
        for (uint32_t kt = 0; kt < n; ++kt) {
            const uint32_t buf = kt % kBufs, par = (kt / kBufs) & 1u;    // score tile number kt
            if (aborted || !__all_sync(0xFFFFFFFFu, mbar_wait(&ctl->s_full[buf], par, ctl, err))) {
                aborted = true;
                continue;
            }
            tc_fence_after();
            const bool diag = kt + 1 == n;
            const uint32_t rel = part;                               // first key of the share relative to the query tile (diag only)
            uint32_t va[32];
            tmem_ld32(lane_addr + buf * kKeys + part, va);
            tmem_ld_wait();
            if (diag) {
#pragma unroll
                for (uint32_t e = 0; e < 32; ++e)
                    if (rel + e <= r) m_raw = fmaxf(m_raw, __uint_as_float(va[e]));
            } else {
#pragma unroll
                for (uint32_t e = 0; e < 32; e += 2) m_raw = cmath::max3(m_raw, __uint_as_float(va[e]), __uint_as_float(va[e + 1]));
            }
            tc_fence_before();
            mbar_arrive(&ctl->s_free[buf]);
        }
        ctl->xch[wg][r] = m_raw;
        asm volatile("bar.sync 1, %0;" ::"n"(kGroups * kConsumers) : "memory");
        float m = ctl->xch[0][r];
#pragma unroll
        for (int gI = 1; gI < kGroups; ++gI) m = fmaxf(m, ctl->xch[gI][r]);
        m = cmath::mul(m, scale);
        const uint64_t scale2 = pk2f(scale, scale), m2 = pk2f(m, m);
        asm volatile("bar.sync 1, %0;" ::"n"(kGroups * kConsumers) : "memory");   // all parts read before xch is reused for the sums
        // ---- pass 2: probabilities into TMEM, row sum ----
        PF_T(pf_p2);
        PF_ADD(1, pf_p2 - pf_roles);
        float l = 0.0f;
        for (uint32_t kt = 0; kt < n; ++kt) {
            const uint32_t buf = (n + kt) % kBufs, par = ((n + kt) / kBufs) & 1u;   // score tile number n + kt
            PF_T(pf_w0);
            if (aborted || !__all_sync(0xFFFFFFFFu, mbar_wait(&ctl->s_full[buf], par, ctl, err))) {
                aborted = true;
                continue;
            }
            tc_fence_after();
            PF_T(pf_w1);
            PF_ADD(3, pf_w1 - pf_w0);
            const uint32_t rel = part;                               // meaningful on the last tile only
            const uint32_t base = lane_addr + buf * kKeys + part;
            // 16 keys per trip, ascending; the next 16 scores are in flight meanwhile.  MASKED only on the last tile
            // (keys past the query's own position).  The loop stays rolled: four groups at four places of an unrolled
            // body do not fit the instruction cache.
            auto tile = [&](auto masked_tag) {
                constexpr bool MASKED = decltype(masked_tag)::value;
                uint32_t v[16];
                tmem_ld16(base, v);
#pragma unroll 1
                for (uint32_t c = 0; c < (uint32_t)kKeys / kGroups / 16; ++c) {
                    float sc[16];
                    uint32_t hi[8], lo[8];
                    PF_T(pf_l0);
                    tmem_ld_wait();
                    PF_T(pf_l1);
                    if (c == 0) PF_ADD(4, pf_l1 - pf_l0);
                    if (MASKED || kExpW != 16) {
#pragma unroll
                        for (uint32_t e = 0; e < 16; ++e) sc[e] = __uint_as_float(v[e]);
                        if (c + 1 < (uint32_t)kKeys / kGroups / 16) tmem_ld16(base + (c + 1) * 16, v);
                    }
                    if constexpr (!MASKED && kExpW == 16) {
                        // a whole trip of 16 unmasked keys, two per instruction
                        float ps[16];
                        exp_scores_packed(v, scale2, m2, neg_zero2, ps);
                        if (c + 1 < (uint32_t)kKeys / kGroups / 16) tmem_ld16(base + (c + 1) * 16, v);
#pragma unroll
                        for (uint32_t u = 0; u < 16; ++u) l = cmath::add(l, ps[u]);                // ascending key order
#pragma unroll
                        for (uint32_t u = 0; u < 16; u += 2) split_hi_lo(ps[u], ps[u + 1], hi[u >> 1], lo[u >> 1]);
                    } else {
#pragma unroll
                    for (uint32_t e = 0; e < 16; e += kExpW) {       // kExpW keys side by side
                        float xs[kExpW], ps[kExpW];
#pragma unroll
                        for (uint32_t u = 0; u < (uint32_t)kExpW; ++u) { // masked keys: argument 0, result discarded
                            xs[u] = cmath::sub(cmath::mul(sc[e + u], scale), m);
                            if (MASKED && rel + c * 16 + e + u > r) xs[u] = 0.0f;
                        }
                        exp_approx_nonpos_n(xs, ps);
#pragma unroll
                        for (uint32_t u = 0; u < (uint32_t)kExpW; ++u) {
                            if (MASKED && rel + c * 16 + e + u > r) ps[u] = 0.0f;
                            l = cmath::add(l, ps[u]);                // ascending key order
                        }
#pragma unroll
                        for (uint32_t u = 0; u < (uint32_t)kExpW; u += 2) split_hi_lo(ps[u], ps[u + 1], hi[(e + u) >> 1], lo[(e + u) >> 1]);
                    }
                    }
                    // in place: the 16 score columns just read become 8 columns of hi parts and 8 of lo parts
                    tmem_st8(base + c * 16, hi);
                    tmem_st8(base + c * 16 + 8, lo);
                }
            };
            if (kt + 1 == n) tile(std::true_type{});
            else tile(std::false_type{});
            PF_T(pf_s0);
            tmem_st_wait();
            PF_T(pf_s1);
            PF_ADD(5, pf_s1 - pf_s0);
            tc_fence_before();
            mbar_arrive(&ctl->p_ready[buf]);
            mbar_arrive(&ctl->s_free[buf]);
        }
        PF_T(pf_p2e);
        PF_ADD(2, pf_p2e - pf_p2);
        ctl->xch[wg][r] = l;
        asm volatile("bar.sync 1, %0;" ::"n"(kGroups * kConsumers) : "memory");
        l = ctl->xch[0][r];
#pragma unroll
        for (int gI = 1; gI < kGroups; ++gI) l = cmath::add(l, ctl->xch[gI][r]);
        // ---- outputs: O / l, group g takes d columns 32 g .. 32 g + 31 ----
        PF_T(pf_o0);
        if (!aborted && __all_sync(0xFFFFFFFFu, mbar_wait(&ctl->o_full, 0, ctl, err))) {
            tc_fence_after();
            PF_T(pf_o1);
            PF_ADD(6, pf_o1 - pf_o0);
            __nv_bfloat16* orow = out + (((size_t)b * S + row) * Hq + h) * kD;
            const uint32_t c = wg;
            uint32_t v[32];
            tmem_ld32(lane_addr + kOCol + c * 32, v);
            tmem_ld_wait();
            if (row < S && !ctl->abort_flag) {
                uint32_t pk[16];
#pragma unroll
                for (uint32_t e = 0; e < 32; e += 2) {
                    const __nv_bfloat162 hv = __floats2bfloat162_rn(cmath::div(__uint_as_float(v[e]), l), cmath::div(__uint_as_float(v[e + 1]), l));
                    pk[e >> 1] = *reinterpret_cast<const uint32_t*>(&hv);
                }
#pragma unroll
                for (uint32_t qd = 0; qd < 4; ++qd)
                    reinterpret_cast<uint4*>(orow + c * 32)[qd] = make_uint4(pk[4 * qd], pk[4 * qd + 1], pk[4 * qd + 2], pk[4 * qd + 3]);
            }
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
#ifdef CATENA_PF_PROFILE
    if (warp < kGroups * 4) PF_ADD(0, clock64() - pf_start);
#endif
    if (warp == kIssuerWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kTmemCols) : "memory");
    }
}

// every float in [0.5, 2^100): rcp_fast against __frcp_rn; counts[0] = values compared, counts[1] = mismatches
__global__ void rcp_check_kernel(unsigned long long* counts) {
    unsigned long long seen = 0, bad = 0;
    const uint32_t lo = 0x3F000000u, hi = __float_as_uint(kRcpFastBelow);
    for (uint64_t b = lo + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; b < hi; b += (uint64_t)gridDim.x * blockDim.x) {
        const float p = __uint_as_float((uint32_t)b);
        ++seen;
        if (__float_as_uint(rcp_fast(p)) != __float_as_uint(__frcp_rn(p))) ++bad;
    }
    atomicAdd(&counts[0], seen);
    atomicAdd(&counts[1], bad);
}
}  // namespace attn3

typedef CUresult (*EncodeTiledFnA3)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFnA3 attn3_encode_fn() {
    static EncodeTiledFnA3 fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFnA3)p;
    }
    return fn;
}

static thread_local uint32_t* g_attn3_err_dev[16] = {nullptr};

// True when the tcgen05 prefill kernel takes the problem (it needs TMA-aligned operands).
bool attn_prefill_tc_supports(const void* q, const void* k_cache, const void* v_cache, uint64_t hq, uint64_t hkv) {
    return hkv != 0 && hq % hkv == 0 && !(((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15);
}

// Reports (and clears) an expired wait of an earlier launch; synchronises the stream.
catena_status_t attn_prefill_tc_check_errors() {
    const int dev = tls().device;
    if (!g_attn3_err_dev[dev]) return CATENA_OK;
    uint32_t h = 0;
    CATENA_CUDA(cudaMemcpyAsync(&h, g_attn3_err_dev[dev], sizeof(h), cudaMemcpyDeviceToHost, tls().stream));
    CATENA_CUDA(cudaStreamSynchronize(tls().stream));
    if (h) {
        cudaMemsetAsync(g_attn3_err_dev[dev], 0, sizeof(uint32_t), tls().stream);
        return fail(CATENA_E_TIMEOUT, "attn_prefill: bounded wait expired");
    }
    return CATENA_OK;
}

// q [batch * seq, hq, 128] bf16, caches [batch, hkv, cap, 128] bf16, out [batch * seq, hq * 128] bf16.
catena_status_t enqueue_attn_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out, uint64_t batch,
                                        uint64_t seq, uint64_t hq, uint64_t hkv, uint64_t cap) {
    EncodeTiledFnA3 fn = attn3_encode_fn();
    if (!fn) return fail(CATENA_E_CUDA, "cuTensorMapEncodeTiled is unavailable");
    const int dev = tls().device;
    if (!g_attn3_err_dev[dev]) {
        CATENA_CUDA(cudaMalloc(&g_attn3_err_dev[dev], sizeof(uint32_t)));
        CATENA_CUDA(cudaMemset(g_attn3_err_dev[dev], 0, sizeof(uint32_t)));
    }
    CUtensorMap map_q, map_k, map_v;
    {
        // q as (64 d, seq tokens, 2 d-halves, hq heads, batch): one copy of box 64 x 128 x 2 x 1 x 1 brings 128 query rows of
        // one head as [d-half][row][128 B], 128B-swizzled; rows past seq read as zero
        cuuint64_t dims[5] = {64, seq, 2, hq, batch};
        cuuint64_t strides[4] = {hq * 256, 128, 256, seq * hq * 256};
        cuuint32_t box[5] = {64, (cuuint32_t)attn3::kTile, 2, 1, 1};
        cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        CUresult r = fn(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(q), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(CATENA_E_CUDA, "cuTensorMapEncodeTiled (queries) failed");
    }
    for (int which = 0; which < 2; ++which) {
        // cache as (64 d, seq visible rows, 2 d-halves, batch * hkv units owning `cap` rows each)
        cuuint64_t dims[4] = {64, seq, 2, batch * hkv};
        cuuint64_t strides[3] = {256, 128, cap * 256};
        cuuint32_t box[4] = {64, (cuuint32_t)attn3::kKeys, 2, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        CUresult r = fn(which ? &map_v : &map_k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(which ? v_cache : k_cache), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(CATENA_E_CUDA, "cuTensorMapEncodeTiled (kv cache) failed");
    }
    const size_t smem = 1024 + (size_t)attn3::kQBytes + (size_t)attn3::kStages * attn3::kStageBytes + sizeof(attn3::Control) + 16;
    static thread_local bool attr_done[16] = {false};
    if (!attr_done[dev]) {
        CATENA_CUDA(cudaFuncSetAttribute(attn3::attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_done[dev] = true;
    }
    dim3 grid((unsigned)ceil_div_u64(seq, attn3::kTile), (unsigned)hq, (unsigned)batch);
    attn3::attn_prefill_tc_kernel<<<grid, attn3::kThreads, smem, tls().stream>>>(map_q, map_k, map_v, (__nv_bfloat16*)out, (uint32_t)seq,
                                                                                (uint32_t)hq, (uint32_t)hkv, 1.0f / sqrtf(128.0f),
                                                                                g_attn3_err_dev[dev], 0x8000000080000000ull);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail_cuda(e, "attn_prefill_tc launch");
    return CATENA_OK;
}

#ifdef CATENA_PF_PROFILE
extern "C" void catena_b200_debug_pf_prof(unsigned long long* out) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, attn3::g_pf_prof, sizeof(unsigned long long) * 16);
    unsigned long long zero[16] = {0};
    cudaMemcpyToSymbol(attn3::g_pf_prof, zero, sizeof(zero));
}
#endif
// runs rcp_check_kernel over the whole range and returns {values compared, mismatches}
catena_status_t attn_prefill_rcp_check(uint64_t out[2]) {
    unsigned long long* dev = nullptr;
    CATENA_CUDA(cudaMalloc(&dev, 2 * sizeof(unsigned long long)));
    CATENA_CUDA(cudaMemset(dev, 0, 2 * sizeof(unsigned long long)));
    attn3::rcp_check_kernel<<<148 * 8, 256, 0, tls().stream>>>(dev);
    unsigned long long h[2] = {0, 0};
    cudaError_t e = cudaMemcpyAsync(h, dev, sizeof(h), cudaMemcpyDeviceToHost, tls().stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(tls().stream);
    cudaFree(dev);
    if (e != cudaSuccess) return fail_cuda(e, "rcp check");
    out[0] = h[0];
    out[1] = h[1];
    return CATENA_OK;
}

}  // namespace catena
