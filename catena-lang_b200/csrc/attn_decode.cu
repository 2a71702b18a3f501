// Cached-attention decode (one new query token) for sm_100a — a bandwidth-bound stream of the
// bf16 KV cache.  The reference has no attention; the semantics are composed from its programs:
//   s_j = (q . k_j) * scale                          fp32            (matrix.hex cell-dot rule)
//   w   = nn.softmax(s): GLOBAL max, math.exp-approx, fp32 denominator (catena-lang/stdlib/nn.hex:93-122)
//   o   = sum_j w_j * v_j                            fp32 -> bf16 round-to-nearest-even
// Online-softmax rescaling is NOT used: with the reference's polynomial exp,
// exp~(x-m1)*exp~(m1-m2) != exp~(x-m2), so every probability here is exp~(s_j - m) with the one
// true row maximum m, exactly as nn.softmax computes it.
//
// Work decomposition (a function of the problem only, never of the GPU or SM count):
//   unit   = (batch, kv-head) with its G = Hq/Hkv query heads, so K and V are read once per group;
//   split  = the KV length is cut into kSplits = 8 contiguous chunks; the 8 CTAs of one unit form a
//            thread-block cluster.  Each CTA streams its K chunk (TMA, 128B-swizzled 64-position
//            tiles, 4-stage mbarrier ring), keeps raw scores in shared memory, the cluster exchanges
//            the chunk maxima over distributed shared memory, each CTA turns its scores into
//            probabilities with the global maximum and streams its V chunk (already prefetched
//            into the ring during the exchange), and the 8 partial (sum p*v, sum p) pairs are
//            combined in ascending chunk order through distributed shared memory.
// Math runs on `mma.sync.m16n8k16` bf16 (positions on the M axis, the <= 8 query heads on N);
// probabilities enter the P*V product as a bf16 hi + bf16 lo pair so no precision is lost to the
// operand format.  FLOPs are irrelevant here (4 FLOP per KV byte); the kernel is sized for HBM.
#include <cooperative_groups.h>
#include <cuda.h>
#include <cuda_bf16.h>

#include "catena_math.cuh"
#include "common.cuh"

namespace cg = cooperative_groups;

namespace catena {

namespace attn {

constexpr int kD = 128;
constexpr int kTile = 64;                    // positions per ring stage
constexpr int kStages = 4;
constexpr int kSplits = 8;                   // cluster size = KV chunks per unit
constexpr int kStageBytes = kTile * kD * 2;  // 16 KiB (two 8 KiB halves of 64 d each)
constexpr int kHalfBytes = kTile * 128;
constexpr int kThreads = 128;
constexpr int kMaxG = 8;
constexpr uint64_t kWaitNs = 1000000000ull;

struct __align__(16) Control {
    uint64_t full[kStages];
    float local_max[kMaxG];
    float denom_part[kMaxG];
    float gmax[kMaxG];
    float warp_part[4][kMaxG];
    volatile uint32_t abort_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
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
                atomicCAS(err, 0u, 1u);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// byte offset inside a stage of the 16-byte chunk `chunk` (0..15 over d) of position row `row`
__device__ __forceinline__ uint32_t tile_off(uint32_t row, uint32_t chunk) {
    uint32_t half = chunk >> 3, c = chunk & 7u;
    return half * kHalfBytes + row * 128u + ((c ^ (row & 7u)) << 4);
}

// grid.x = kSplits * (unit1 - unit0); cluster (kSplits,1,1); block 128 threads.
__global__ void __launch_bounds__(kThreads)
attn_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ o, uint32_t L, uint32_t G,
                   uint32_t Hq, uint32_t Hkv, uint32_t unit0, uint32_t chunk, float scale, uint32_t* err) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* ring = smem;
    float* scores = reinterpret_cast<float*>(smem + kStages * kStageBytes);       // [G][chunk]
    __nv_bfloat16* p_hi = reinterpret_cast<__nv_bfloat16*>(scores + (size_t)G * chunk);  // [G][chunk]
    __nv_bfloat16* p_lo = p_hi + (size_t)G * chunk;
    float* o_part = reinterpret_cast<float*>(p_lo + (size_t)G * chunk);            // [G][128]
    Control* ctl = reinterpret_cast<Control*>(o_part + (size_t)G * kD);

    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t rank = cluster.block_rank();
    const uint32_t unit = unit0 + blockIdx.x / kSplits;
    const uint32_t b = unit / Hkv, kvh = unit % Hkv;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const uint32_t pos_begin = rank * chunk;
    const uint32_t valid = pos_begin < L ? min(chunk, L - pos_begin) : 0u;   // positions of this CTA
    const uint32_t T = (valid + kTile - 1) / kTile;                          // K tiles (= V tiles)
    const uint32_t total = 2 * T;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&ctl->full[s])), "r"(1) : "memory");
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // tile g of this CTA: g < T -> K tile g, else V tile g - T
    auto issue = [&](uint32_t g) {
        uint32_t st = g % kStages;
        const CUtensorMap* map = g < T ? &map_k : &map_v;
        uint32_t pos = pos_begin + (g < T ? g : g - T) * kTile;
        uint64_t* bar = &ctl->full[st];
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"((uint32_t)kStageBytes)
                     : "memory");
        uint32_t dst = smem_u32(ring + st * kStageBytes);
        tma_load_3d(dst, map, 0, (int)pos, (int)unit, bar);
        tma_load_3d(dst + kHalfBytes, map, 64, (int)pos, (int)unit, bar);
    };
    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
        for (uint32_t g = 0; g < total && g < (uint32_t)kStages; ++g) issue(g);
    }

    // Q as B fragments of S^T = K * Q^T: lane holds Q[head = lane/4][d = 16*ks + 2*(lane%4) + {0,1}] and d + 8
    uint32_t qb[8][2];
    {
        const uint32_t head = lane >> 2;
        const __nv_bfloat16* qrow = q + ((size_t)b * Hq + (size_t)kvh * G + head) * kD;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t d = ks * 16 + (lane & 3u) * 2;
            qb[ks][0] = head < G ? *reinterpret_cast<const uint32_t*>(qrow + d) : 0u;
            qb[ks][1] = head < G ? *reinterpret_cast<const uint32_t*>(qrow + d + 8) : 0u;
        }
    }

    bool aborted = false;
    // Waits for tile g, makes the decision block-uniform, and refills the stage of tile g-1
    // (every warp finished reading it before reaching this barrier).
    auto acquire = [&](uint32_t g) -> bool {
        bool ok = mbar_wait(&ctl->full[g % kStages], (g / kStages) & 1u, ctl, err);
        if (__syncthreads_or(ok ? 0 : 1)) return false;
        if (tid == 0 && g >= 1 && g - 1 + kStages < total) issue(g - 1 + kStages);
        return true;
    };

    // ---------------- phase 1: scores of this chunk ----------------
    for (uint32_t g = 0; g < T && !aborted; ++g) {
        if (!acquire(g)) { aborted = true; break; }
        const uint32_t base = smem_u32(ring + (g % kStages) * kStageBytes);
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        const uint32_t row = warp * 16 + (lane & 7u) + ((lane >> 3) & 1u) * 8;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t a[4];
            ldsm_x4(base + tile_off(row, ks * 2 + (lane >> 4)), a);
            mma_bf16(c, a, qb[ks][0], qb[ks][1]);
        }
        // C fragment: rows (lane/4, lane/4+8) of this warp's 16 positions, heads 2*(lane%4)+{0,1}
        const uint32_t p0 = g * kTile + warp * 16 + (lane >> 2);
        const uint32_t h0 = (lane & 3u) * 2;
        if (h0 < G) {
            scores[(size_t)h0 * chunk + p0] = cmath::mul(c[0], scale);
            scores[(size_t)h0 * chunk + p0 + 8] = cmath::mul(c[2], scale);
        }
        if (h0 + 1 < G) {
            scores[(size_t)(h0 + 1) * chunk + p0] = cmath::mul(c[1], scale);
            scores[(size_t)(h0 + 1) * chunk + p0 + 8] = cmath::mul(c[3], scale);
        }
    }
    __syncthreads();

    // chunk maxima (order-free on finite data)
    for (uint32_t h = warp; h < G; h += 4) {
        float m = __uint_as_float(0xFF800000u);
        if (!aborted)
            for (uint32_t p = lane; p < valid; p += 32) m = fmaxf(m, scores[(size_t)h * chunk + p]);
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
        if (lane == 0) ctl->local_max[h] = m;
    }
    cluster.sync();   // #1: every CTA's local_max is visible cluster-wide
    if (tid < G) {
        float m = __uint_as_float(0xFF800000u);
        for (uint32_t r = 0; r < (uint32_t)kSplits; ++r) {
            const float* remote = cluster.map_shared_rank(ctl->local_max, r);
            m = fmaxf(m, remote[tid]);
        }
        ctl->gmax[tid] = m;
    }
    __syncthreads();

    // probabilities p = exp~(s - max) as bf16 hi + lo, and this chunk's denominator in a fixed order:
    // thread t sums positions t, t+128, ... ascending; xor butterfly per warp; warps 0..3 ascending.
    for (uint32_t h = 0; h < G; ++h) {
        const float m = ctl->gmax[h];
        float acc = 0.0f;
        for (uint32_t p = tid; p < chunk; p += kThreads) {
            float pv = 0.0f;
            if (p < valid && !aborted) pv = cmath::exp_approx(cmath::sub(scores[(size_t)h * chunk + p], m));
            __nv_bfloat16 hi = __float2bfloat16_rn(pv);
            __nv_bfloat16 lo = __float2bfloat16_rn(cmath::sub(pv, __bfloat162float(hi)));
            p_hi[(size_t)h * chunk + p] = hi;
            p_lo[(size_t)h * chunk + p] = lo;
            acc = cmath::add(acc, pv);
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) acc = cmath::add(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, off));
        if (lane == 0) ctl->warp_part[warp][h] = acc;
    }
    __syncthreads();
    if (tid < G) {
        float d = ctl->warp_part[0][tid];
        for (int w = 1; w < 4; ++w) d = cmath::add(d, ctl->warp_part[w][tid]);
        ctl->denom_part[tid] = d;
    }

    // ---------------- phase 2: O^T = V^T * P^T over this chunk ----------------
    float acc[2][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[mt][e] = 0.0f;
    for (uint32_t g = T; g < total && !aborted; ++g) {
        if (!acquire(g)) { aborted = true; break; }
        const uint32_t base = smem_u32(ring + (g % kStages) * kStageBytes);
        const uint32_t tile_pos = (g - T) * kTile;
        const uint32_t head = lane >> 2;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t bh0 = 0, bh1 = 0, bl0 = 0, bl1 = 0;
            if (head < G) {
                size_t off = (size_t)head * chunk + tile_pos + ks * 16 + (lane & 3u) * 2;
                bh0 = *reinterpret_cast<const uint32_t*>(p_hi + off);
                bh1 = *reinterpret_cast<const uint32_t*>(p_hi + off + 8);
                bl0 = *reinterpret_cast<const uint32_t*>(p_lo + off);
                bl1 = *reinterpret_cast<const uint32_t*>(p_lo + off + 8);
            }
            const uint32_t prow = ks * 16 + (lane & 7u) + (lane >> 4) * 8;
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                uint32_t a[4];
                ldsm_x4_trans(base + tile_off(prow, (warp * 2 + mt) * 2 + ((lane >> 3) & 1u)), a);
                mma_bf16(acc[mt], a, bh0, bh1);
                mma_bf16(acc[mt], a, bl0, bl1);
            }
        }
    }
    // partial outputs: C fragment rows d = 16*mtile + lane/4 (+8), heads 2*(lane%4)+{0,1}
    {
        const uint32_t h0 = (lane & 3u) * 2;
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            const uint32_t d0 = (warp * 2 + mt) * 16 + (lane >> 2);
            if (h0 < G) {
                o_part[h0 * kD + d0] = acc[mt][0];
                o_part[h0 * kD + d0 + 8] = acc[mt][2];
            }
            if (h0 + 1 < G) {
                o_part[(h0 + 1) * kD + d0] = acc[mt][1];
                o_part[(h0 + 1) * kD + d0 + 8] = acc[mt][3];
            }
        }
    }
    cluster.sync();   // #2: every CTA's o_part / denom_part is visible cluster-wide

    // ---------------- combine: ascending chunk order, one slice of the outputs per CTA ----------------
    {
        const uint32_t per_rank = G * kD / kSplits;   // G*16 <= 128
        if (tid < per_rank) {
            const uint32_t idx = rank * per_rank + tid;
            const uint32_t h = idx / kD, d = idx % kD;
            float num = 0.0f, den = 0.0f;
            for (uint32_t r = 0; r < (uint32_t)kSplits; ++r) {
                const float* ro = cluster.map_shared_rank(o_part, r);
                const float* rd = cluster.map_shared_rank(ctl->denom_part, r);
                num = cmath::add(num, ro[h * kD + d]);
                den = cmath::add(den, rd[h]);
            }
            if (!aborted)
                o[((size_t)b * Hq + (size_t)kvh * G + h) * kD + d] = __float2bfloat16_rn(cmath::div(num, den));
        }
    }
    if (ctl->abort_flag) {
        uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    cluster.sync();   // #3: nobody leaves while peers still read its shared memory
}

}  // namespace attn

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn attn_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// KV cache [units, L, 128] bf16 as a 3-D tensor: box = 64 d x 64 positions x 1 unit, 128B swizzle;
// positions past L read as zero, so a ragged last tile never touches the next unit's rows.
static catena_status_t make_kv_map(CUtensorMap* map, const void* base, uint64_t units, uint64_t L) {
    EncodeTiledFn fn = attn_encode_fn();
    if (!fn) return fail(CATENA_E_CUDA, "cuTensorMapEncodeTiled is unavailable");
    cuuint64_t dims[3] = {(cuuint64_t)attn::kD, L, units};
    cuuint64_t strides[2] = {(cuuint64_t)attn::kD * 2, L * (cuuint64_t)attn::kD * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)attn::kTile, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(CATENA_E_CUDA, "cuTensorMapEncodeTiled (kv cache) failed");
    return CATENA_OK;
}

static thread_local uint32_t* g_attn_err_dev[16] = {nullptr};
static thread_local uint32_t* g_attn_err_host[16] = {nullptr};

static uint32_t chunk_for(uint64_t L) {
    uint64_t c = ceil_div_u64(ceil_div_u64(L, attn::kSplits), attn::kTile) * attn::kTile;
    return (uint32_t)(c < (uint64_t)attn::kTile ? attn::kTile : c);
}
static size_t attn_smem_bytes(uint32_t G, uint32_t chunk) {
    return 1024 + (size_t)attn::kStages * attn::kStageBytes + (size_t)G * chunk * (4 + 2 + 2) + (size_t)G * attn::kD * 4 +
           sizeof(attn::Control) + 16;
}

catena_status_t launch_attn_decode(const void* q, const void* kc, const void* vc, void* o, uint64_t batch, uint64_t hq,
                                   uint64_t hkv, uint64_t d, uint64_t kv_len, uint64_t unit0, uint64_t unit1) {
    CATENA_TRY(ensure_device());
    if (!q || !kc || !vc || !o) return fail(CATENA_E_BAD_ARG, "attn_decode: null operand");
    if (d != (uint64_t)attn::kD) return fail(CATENA_E_UNSUPPORTED, "attn_decode: head_dim must be 128");
    if (hkv == 0 || hq % hkv != 0 || hq / hkv > (uint64_t)attn::kMaxG)
        return fail(CATENA_E_UNSUPPORTED, "attn_decode: Hq must be a multiple of Hkv with Hq/Hkv <= 8");
    if (kv_len == 0 || batch == 0) return fail(CATENA_E_BAD_ARG, "attn_decode: empty cache");
    uint64_t units = batch * hkv;
    if (unit1 > units || unit0 > unit1) return fail(CATENA_E_BAD_ARG, "attn_decode: unit range");
    if (unit0 == unit1) return CATENA_OK;
    if (((uintptr_t)kc & 15) || ((uintptr_t)vc & 15) || ((uintptr_t)q & 3)) return fail(CATENA_E_BAD_ARG, "attn_decode: alignment");
    if (kv_len > 0x7FFFFFFFull || units > 0x7FFFFFFFull) return fail(CATENA_E_TOO_LARGE, "attn_decode: size");
    const uint32_t G = (uint32_t)(hq / hkv);
    const uint32_t chunk = chunk_for(kv_len);
    const size_t smem = attn_smem_bytes(G, chunk);
    if (smem > 227 * 1024) return fail(CATENA_E_TOO_LARGE, "attn_decode: KV length beyond the shared-memory score buffer");

    CUtensorMap map_k, map_v;
    CATENA_TRY(make_kv_map(&map_k, kc, units, kv_len));
    CATENA_TRY(make_kv_map(&map_v, vc, units, kv_len));
    int dev = tls().device & 15;
    if (!g_attn_err_dev[dev]) {
        CATENA_CUDA(cudaMalloc(&g_attn_err_dev[dev], sizeof(uint32_t)));
        CATENA_CUDA(cudaMemset(g_attn_err_dev[dev], 0, sizeof(uint32_t)));
        CATENA_CUDA(cudaMallocHost(&g_attn_err_host[dev], sizeof(uint32_t)));
        *g_attn_err_host[dev] = 0;
    }
    CATENA_CUDA(cudaFuncSetAttribute(attn::attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((unit1 - unit0) * attn::kSplits));
    cfg.blockDim = dim3(attn::kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = tls().stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = attn::kSplits;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    float scale = 1.0f / sqrtf((float)attn::kD);
    CATENA_CUDA(cudaLaunchKernelEx(&cfg, attn::attn_decode_kernel, map_k, map_v, (const __nv_bfloat16*)q, (__nv_bfloat16*)o,
                                   (uint32_t)kv_len, G, (uint32_t)hq, (uint32_t)hkv, (uint32_t)unit0, chunk, scale,
                                   g_attn_err_dev[dev]));
    count_launch();
    if (tls().blocking) {
        cudaStream_t st = tls().stream;
        CATENA_CUDA(cudaMemcpyAsync(g_attn_err_host[dev], g_attn_err_dev[dev], sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
        CATENA_CUDA(cudaStreamSynchronize(st));
        if (*g_attn_err_host[dev] != 0) {
            *g_attn_err_host[dev] = 0;
            cudaMemsetAsync(g_attn_err_dev[dev], 0, sizeof(uint32_t), st);
            return fail(CATENA_E_TIMEOUT, "attn_decode: bounded wait expired");
        }
    }
    return CATENA_OK;
}

catena_status_t attn_check_errors() {
    CATENA_TRY(ensure_device());
    int dev = tls().device & 15;
    if (!g_attn_err_dev[dev]) return CATENA_OK;
    cudaStream_t st = tls().stream;
    CATENA_CUDA(cudaMemcpyAsync(g_attn_err_host[dev], g_attn_err_dev[dev], sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    CATENA_CUDA(cudaStreamSynchronize(st));
    if (*g_attn_err_host[dev] != 0) {
        *g_attn_err_host[dev] = 0;
        cudaMemsetAsync(g_attn_err_dev[dev], 0, sizeof(uint32_t), st);
        return fail(CATENA_E_TIMEOUT, "attn_decode: bounded wait expired");
    }
    return CATENA_OK;
}

}  // namespace catena
