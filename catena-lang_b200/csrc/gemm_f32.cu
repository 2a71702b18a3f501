// f32 matrix product with the reference's exact semantics
// (catena-lang/stdlib/matrix.hex:210-327, entry catena-lang/tests/cases/matrix/matmul.hex:2-63):
//
//     C[i,j] = (((+0 + a_i0*b_0j) + a_i1*b_1j) + ... + a_i,K-1*b_K-1,j)
//
// with `*` and `+` rounded separately (never an FMA) and k strictly ascending.  The reference
// runs one thread per output with an untiled K loop; here A and B are staged through shared
// memory in k-slabs and every thread keeps a TM x TN register tile, but each output element
// still owns its own accumulation chain in the same order, so results are bit-identical for
// every tile shape.  The K loop never pads: a trailing partial slab stops at exactly K (adding
// `+0` terms could flip a `-0` accumulator to `+0`).  tcgen05 has no fp32 input mode and tensor
// cores do not accumulate as a sequential IEEE chain, so this kernel is CUDA-core work by design.  What sm_100 does add is
// packed f32x2 arithmetic (two separately rounded IEEE operations per instruction): the large tile uses it, see below.
#include "common.cuh"

namespace catena {

template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN), TM * TN >= 64 ? 2 : 1)
matmul_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int n, int m,
                  int k, uint64_t neg_zero2) {
    constexpr int THREADS = (BM / TM) * (BN / TN);
    __shared__ __align__(16) float As[BK][BM + 4];  // transposed: As[kk][row]; rows are 16-byte multiples apart
    __shared__ __align__(16) float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN);   // column group
    const int ty = tid / (BN / TN);   // row group
    const int row0 = blockIdx.y * BM;
    const int col0 = blockIdx.x * BN;
    // columns of this thread's register tile: TN consecutive ones, or — for the 8-wide tile — 4 + 4 half a tile apart, so that
    // a warp's 16-byte reads of a Bs row are contiguous (conflict-free) instead of 32 bytes apart (4-way conflicts)
    constexpr bool SPLIT = TN == 8;
    constexpr bool PACKED = TN % 2 == 0;      // pairs of neighbouring columns: packed f32x2 arithmetic
    auto col_of = [&](int j) { return SPLIT ? (j / 4) * (BN / 2) + tx * 4 + (j % 4) : tx * TN + j; };

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;  // bit pattern 0x00000000 (matrix.hex:249)
    // A register tile of even width keeps its accumulators as PAIRS of neighbouring columns and works on them with the packed
    // f32x2 arithmetic of sm_100: each half is the same separately rounded IEEE product and sum, so the bits do not change,
    // but a k step of the 8 x 8 tile is 64 arithmetic instructions instead of 128.
    uint64_t acc2[PACKED ? TM : 1][PACKED ? TN / 2 : 1];
#pragma unroll
    for (int i = 0; i < (PACKED ? TM : 1); ++i)
#pragma unroll
        for (int j = 0; j < (PACKED ? TN / 2 : 1); ++j) acc2[i][j] = 0ull;

    // The next k-slab travels from global memory into registers while the current one is multiplied out of shared
    // memory (small products are latency bound: eight exposed slab loads were most of a 256^3 launch).
    constexpr int PA = (BM * BK + THREADS - 1) / THREADS, PB = (BK * BN + THREADS - 1) / THREADS;
    float ra[PA], rb[PB];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int p = 0; p < PA; ++p) {
            const int idx = tid + p * THREADS, r = idx / BK, kk = idx % BK;
            const int gr = row0 + r, gk = k0 + kk;
            ra[p] = (idx < BM * BK && gr < n && gk < k) ? A[(size_t)gr * k + gk] : 0.0f;
        }
#pragma unroll
        for (int p = 0; p < PB; ++p) {
            const int idx = tid + p * THREADS, kk = idx / BN, c = idx % BN;
            const int gk = k0 + kk, gc = col0 + c;
            rb[p] = (idx < BK * BN && gk < k && gc < m) ? B[(size_t)gk * m + gc] : 0.0f;
        }
    };
    // A[row0.., k0..] transposed and B[k0.., col0..]
    auto stage = [&]() {
#pragma unroll
        for (int p = 0; p < PA; ++p) {
            const int idx = tid + p * THREADS;
            if (idx < BM * BK) As[idx % BK][idx / BK] = ra[p];
        }
#pragma unroll
        for (int p = 0; p < PB; ++p) {
            const int idx = tid + p * THREADS;
            if (idx < BK * BN) Bs[idx / BN][idx % BN] = rb[p];
        }
    };
    if (k > 0) fetch(0);
    for (int k0 = 0; k0 < k; k0 += BK) {
        const int kb = min(BK, k - k0);
        stage();
        if (k0 + BK < k) fetch(k0 + BK);
        __syncthreads();
        if constexpr (PACKED) {
            // one k step: the operands (for the 8 x 8 tile four 16-byte loads), then TM x TN / 2 packed products and sums
            auto step = [&](int kk) {
                float av[TM];
                uint64_t bv[TN / 2];          // column pairs of the register tile
                if constexpr (SPLIT) {
                    const ulonglong2 b0 = *reinterpret_cast<const ulonglong2*>(&Bs[kk][tx * 4]), b1 = *reinterpret_cast<const ulonglong2*>(&Bs[kk][BN / 2 + tx * 4]);
                    const float4 a0 = *reinterpret_cast<const float4*>(&As[kk][ty * TM]), a1 = *reinterpret_cast<const float4*>(&As[kk][ty * TM + 4]);
                    av[0] = a0.x; av[1] = a0.y; av[2] = a0.z; av[3] = a0.w; av[4] = a1.x; av[5] = a1.y; av[6] = a1.z; av[7] = a1.w;
                    bv[0] = b0.x; bv[1] = b0.y; bv[2] = b1.x; bv[3] = b1.y;     // columns (0,1) (2,3) | (4,5) (6,7)
                } else {
#pragma unroll
                    for (int i = 0; i < TM; ++i) av[i] = As[kk][ty * TM + i];
#pragma unroll
                    for (int j = 0; j < TN / 2; ++j) bv[j] = *reinterpret_cast<const uint64_t*>(&Bs[kk][tx * TN + 2 * j]);
                }
#pragma unroll
                for (int i = 0; i < TM; ++i) {
                    uint64_t aa;
                    asm("mov.b64 %0, {%1, %1};" : "=l"(aa) : "f"(av[i]));
#pragma unroll
                    for (int j = 0; j < TN / 2; ++j) {
                        // The product is a packed fma with -0 as its addend: a * b + (-0) is the rounded product (a zero product
                        // keeps its sign).  The -0 arrives as a kernel argument so that ptxas cannot turn the fma back into a
                        // mul: it merges a packed mul and the packed add behind it into ONE fma — explicit .rn and
                        // --fmad=false notwithstanding — and that rounds once (measured: the bits of fma.rn.f32x2).  The
                        // instructions themselves round like their scalar forms (checked against __fmul_rn / __fadd_rn).
                        uint64_t prod;
                        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(prod) : "l"(aa), "l"(bv[j]), "l"(neg_zero2));
                        asm("add.rn.f32x2 %0, %1, %2;" : "=l"(acc2[i][j]) : "l"(acc2[i][j]), "l"(prod));
                    }
                }
            };
            if (kb == BK) {
#pragma unroll(TM * TN >= 64 ? 4 : 16)
                for (int kk = 0; kk < BK; ++kk) step(kk);
            } else {
                for (int kk = 0; kk < kb; ++kk) step(kk);
            }
        } else if (kb == BK) {
#pragma unroll
            for (int kk = 0; kk < BK; ++kk) {
                float a[TM], b[TN];
#pragma unroll
                for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
                for (int j = 0; j < TN; ++j) b[j] = Bs[kk][col_of(j)];
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));
            }
        } else {
            for (int kk = 0; kk < kb; ++kk) {
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j)
                        acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(As[kk][ty * TM + i], Bs[kk][col_of(j)]));
            }
        }
        __syncthreads();
    }
    if constexpr (PACKED) {
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN / 2; ++j) {
                acc[i][2 * j] = __uint_as_float((uint32_t)acc2[i][j]);
                acc[i][2 * j + 1] = __uint_as_float((uint32_t)(acc2[i][j] >> 32));
            }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        int gr = row0 + ty * TM + i;
        if (gr >= n) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            int gc = col0 + col_of(j);
            if (gc < m) C[(size_t)gr * m + gc] = acc[i][j];
        }
    }
}

// A * I or I * A with the identity generated on the fly (catena-lang/stdlib/matrix.hex:129-159):
// every output is the same left fold, whose terms are a*1 and a*0.
__global__ void identity_matmul_kernel(const float* __restrict__ A, float* __restrict__ C, int n, int left) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n * n) return;
    int i = idx / n, j = idx % n;
    float acc = 0.0f;
    for (int kk = 0; kk < n; ++kk) {
        float a = left ? (i == kk ? 1.0f : 0.0f) : A[(size_t)i * n + kk];
        float b = left ? A[(size_t)kk * n + j] : (kk == j ? 1.0f : 0.0f);
        acc = __fadd_rn(acc, __fmul_rn(a, b));
    }
    C[idx] = acc;
}

// Check of the packed forms the kernels above (and catena_math.cuh, map_jit.cu) rely on, over `n` pseudo-random operand
// triples per thread: counts[0] = pairs compared; counts[1] = pairs where fma.rn.f32x2(a, b, z) followed by add.rn.f32x2
// (z = -0 from a kernel argument) differs from __fadd_rn(c, __fmul_rn(a, b)) — must be 0; counts[2] = pairs where
// mul.rn.f32x2 followed by add.rn.f32x2 differs — NOT 0 with CUDA 12.9: the assembler merges the two into one fma.
__global__ void packed_f32x2_check_kernel(unsigned long long* counts, uint32_t n, uint64_t neg_zero2) {
    uint32_t state = (blockIdx.x * blockDim.x + threadIdx.x) * 2654435761u + 12345u;
    auto next = [&]() {             // xorshift; floats in [-2, 2) with every mantissa pattern, a few exact zeros and tiny values
        state ^= state << 13; state ^= state >> 17; state ^= state << 5;
        const uint32_t pick = state & 63u;
        if (pick == 0) return (state & 0x80000000u);                               // +0 / -0
        if (pick == 1) return (state & 0x807FFFFFu) | 0x00800000u;                 // tiny normal
        return (state & 0x807FFFFFu) | (0x3F000000u + ((state >> 8) & 0x01000000u));
    };
    unsigned long long compared = 0, bad_fma_form = 0, bad_mul_form = 0;
    for (uint32_t k = 0; k < n; ++k) {
        const uint32_t a0 = next(), a1 = next(), b0 = next(), b1 = next(), c0 = next(), c1 = next();
        const uint64_t a = ((uint64_t)a1 << 32) | a0, b = ((uint64_t)b1 << 32) | b0, c = ((uint64_t)c1 << 32) | c0;
        uint64_t p, viaFma, viaMul;
        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(p) : "l"(a), "l"(b), "l"(neg_zero2));
        asm("add.rn.f32x2 %0, %1, %2;" : "=l"(viaFma) : "l"(c), "l"(p));
        asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(p) : "l"(a), "l"(b));
        asm("add.rn.f32x2 %0, %1, %2;" : "=l"(viaMul) : "l"(c), "l"(p));
        const uint32_t w0 = __float_as_uint(__fadd_rn(__uint_as_float(c0), __fmul_rn(__uint_as_float(a0), __uint_as_float(b0))));
        const uint32_t w1 = __float_as_uint(__fadd_rn(__uint_as_float(c1), __fmul_rn(__uint_as_float(a1), __uint_as_float(b1))));
        const uint64_t want = ((uint64_t)w1 << 32) | w0;
        ++compared;
        bad_fma_form += viaFma != want;
        bad_mul_form += viaMul != want;
    }
    atomicAdd(&counts[0], compared);
    atomicAdd(&counts[1], bad_fma_form);
    atomicAdd(&counts[2], bad_mul_form);
}

// two packed -0.0f: the addend that makes a packed fma a rounded product (passed as an argument: see the kernel)
static const uint64_t kNegZero2 = 0x8000000080000000ull;

catena_status_t launch_matmul_f32(const float* a, const float* b, float* c, uint64_t n, uint64_t m, uint64_t k) {
    if (n == 0 || m == 0) return CATENA_OK;
    if (n > 0x7FFFFFFFull || m > 0x7FFFFFFFull || k > 0x7FFFFFFFull)
        return fail(CATENA_E_TOO_LARGE, "matmul f32: dimension beyond 2^31-1");
    cudaStream_t st = tls().stream;
    int sms = tls().sm_count > 0 ? tls().sm_count : 148;
    uint64_t big_tiles = ceil_div_u64(n, 64) * ceil_div_u64(m, 64);
    const uint64_t huge_tiles = ceil_div_u64(n, 128) * ceil_div_u64(m, 128);
    // row tiles ride on grid.y (at most 65535): 4 194 240 rows with the 64-row tiles; taller products are refused, not mis-launched
    if (ceil_div_u64(n, 3 * big_tiles >= 2 * (uint64_t)sms ? 64 : 16) > 65535)
        return fail(CATENA_E_TOO_LARGE, "matmul f32: more than 65535 row tiles (4194240 rows)");
    if (huge_tiles >= 2 * (uint64_t)sms) {
        // large products are bound by instruction issue (two FP instructions per multiply-add, by contract): an 8 x 8 register
        // tile spends 4 shared-memory loads per 128 of them where the 4 x 4 tile spends 2 per 32
        dim3 grid((unsigned)ceil_div_u64(m, 128), (unsigned)ceil_div_u64(n, 128));
        matmul_f32_kernel<128, 128, 16, 8, 8><<<grid, 256, 0, st>>>(a, b, c, (int)n, (int)m, (int)k, kNegZero2);
    } else if (3 * big_tiles >= 2 * (uint64_t)sms) {          // from two thirds of a wave of 64 x 64 tiles on (768^3: 144 tiles)
        dim3 grid((unsigned)ceil_div_u64(m, 64), (unsigned)ceil_div_u64(n, 64));
        matmul_f32_kernel<64, 64, 16, 4, 4><<<grid, 256, 0, st>>>(a, b, c, (int)n, (int)m, (int)k, kNegZero2);
    } else if (ceil_div_u64(m, 32) * ceil_div_u64(n, 16) >= 64) {
        // small products are latency bound: more, smaller tiles to cover the SMs.  One element per thread reads two
        // shared-memory words per multiply-add, which made shared memory the limit (8192 wavefronts per SM at 256^3); a 2 x 2
        // register tile reads two 8-byte words per four (256^3: 8.1 against 10.3 us, 512^3: 28.7 against 45.3 us).
        dim3 grid((unsigned)ceil_div_u64(m, 32), (unsigned)ceil_div_u64(n, 16));
        matmul_f32_kernel<16, 32, 128, 2, 2><<<grid, 128, 0, st>>>(a, b, c, (int)n, (int)m, (int)k, kNegZero2);
    } else {
        // tiny products: one element per thread, as many CTAs as there are 16 x 16 tiles
        dim3 grid((unsigned)ceil_div_u64(m, 16), (unsigned)ceil_div_u64(n, 16));
        matmul_f32_kernel<16, 16, 128, 1, 1><<<grid, 256, 0, st>>>(a, b, c, (int)n, (int)m, (int)k, kNegZero2);
    }
    count_launch();
    return CATENA_OK;
}

catena_status_t packed_f32x2_check(uint64_t out[3]) {
    unsigned long long* dev = nullptr;
    CATENA_CUDA(cudaMalloc(&dev, 3 * sizeof(unsigned long long)));
    cudaMemsetAsync(dev, 0, 3 * sizeof(unsigned long long), tls().stream);
    packed_f32x2_check_kernel<<<148 * 4, 256, 0, tls().stream>>>(dev, 256, kNegZero2);
    count_launch();
    unsigned long long host[3] = {0, 0, 0};
    cudaError_t e = cudaMemcpyAsync(host, dev, sizeof(host), cudaMemcpyDeviceToHost, tls().stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(tls().stream);
    cudaFree(dev);
    if (e != cudaSuccess) return fail_cuda(e, "packed f32x2 check");
    for (int i = 0; i < 3; ++i) out[i] = host[i];
    return CATENA_OK;
}

catena_status_t launch_identity_matmul_f32(const float* a, float* c, uint64_t n, int identity_on_left) {
    if (n == 0) return CATENA_OK;
    if (n > 46340) return fail(CATENA_E_TOO_LARGE, "identity matmul: n*n beyond 2^31-1");
    unsigned total = (unsigned)(n * n);
    identity_matmul_kernel<<<(total + 255) / 256, 256, 0, tls().stream>>>(a, c, (int)n, identity_on_left);
    count_launch();
    return CATENA_OK;
}

}  // namespace catena
