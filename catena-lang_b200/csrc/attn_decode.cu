// Cached-attention decode (one new query token) for sm_100a — a bandwidth-bound stream of the
// bf16 KV cache.  The reference has no attention; the semantics are composed from its programs:
//   s_j = (q . k_j) * scale                          fp32            (matrix.hex cell-dot rule)
//   w   = nn.softmax(s): GLOBAL max, math.exp-approx, fp32 denominator (catena-lang/stdlib/nn.hex:93-122)
//   o   = sum_j w_j * v_j                            fp32 -> bf16 round-to-nearest-even
// Online-softmax rescaling is NOT used: with the reference's polynomial exp,
// exp~(x-m1)*exp~(m1-m2) != exp~(x-m2), so every probability here is exp~(s_j - m) with the one
// true row maximum m, exactly as nn.softmax computes it.
//
// Work decomposition (a function of the problem only, never of the GPU, SM or cluster count):
//   unit   = (batch, kv-head) with its G = Hq/Hkv query heads, so K and V are read once per group;
//   split  = the KV length is cut into kSplits = 8 contiguous chunks, one per CTA of a thread-block
//            cluster; partial results are combined in ascending chunk order.
// Execution: persistent clusters, each walking units first, first + #clusters, ...  Per CTA:
//   warp 4      producer: one 4-D `cp.async.bulk.tensor` (128B swizzle, no multicast) per 64-position
//               tile into a ring of mbarrier-guarded stages, running ahead of the consumers;
//   warps 0-3   consumers; consecutive units are software-pipelined so the cluster-wide exchanges
//               never idle the stream:
//     iteration i:  K tiles of unit i -> raw scores, chunk maxima pushed to the peers | barrier.cluster.arrive
//                   V tiles of unit i-1 -> partial sum p*v, pushed to the owning peer  | barrier.cluster.wait
//                   global max of unit i, p = exp~(s - max) (bf16 hi + lo), chunk denominator pushed
//                   combine unit i-2 in ascending chunk order, divide, round to bf16, store
// Everything a peer needs is PUSHED into its shared memory (distributed shared memory stores) before
// the barrier, so after the barrier all reads are local.  Pushed buffers are multi-buffered (maxima
// x2, partial outputs and denominators x3): a slot is rewritten only after a later cluster barrier
// has proved every reader done.
// Math runs on `mma.sync.m16n8k16` bf16 (positions or head-dim on M, the <= 8 query heads on N);
// FLOPs are irrelevant here (4 FLOP per KV byte); the kernel is sized for HBM.
#include <cooperative_groups.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdlib.h>

#include "catena_math.cuh"
#include "common.cuh"

namespace cg = cooperative_groups;

namespace catena {

namespace attn {

constexpr int kD = 128;
constexpr int kTile = 64;                    // positions per ring stage
#ifndef CATENA_ATTN_STAGES
#define CATENA_ATTN_STAGES 4
#endif
constexpr int kStages = CATENA_ATTN_STAGES;
constexpr int kSplits = 8;                   // cluster size = KV chunks per unit
constexpr int kStageBytes = kTile * kD * 2;  // 16 KiB: [d-half 2][position 64][128 B]
constexpr int kHalfBytes = kTile * 128;
constexpr int kConsumers = 128;              // warps 0..3
constexpr int kThreads = 160;                // + producer warp 4
constexpr int kMaxG = 8;
constexpr uint64_t kWaitNs = 1000000000ull;
// a waiting thread may be suspended by the hardware for up to this long (it is woken when the phase completes):
// without the hint the producer / issuer threads spin and take issue slots from the warps doing the work
constexpr uint32_t kSuspendHintNs = 20000;

struct __align__(16) Control {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    float lmax_all[2][kSplits][kMaxG];   // chunk maxima of every rank, written by the peers (push)
    float den_all[3][kSplits][kMaxG];    // chunk denominators of every rank, written by the peers
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
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when it expired (about one second) or another thread already gave up.
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
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
#ifdef CATENA_ATTN_RELAXED_ARRIVE
    asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
#else
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
#endif
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
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
// Split cluster barrier: every thread of every CTA of the cluster executes both halves, once per
// iteration; writes made before `arrive` are visible to peers after their `wait`.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// barrier among the four consumer warps only (the producer warp never joins it)
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// byte offset inside a stage of the 16-byte chunk `chunk` (0..15 over d) of position row `row`
__device__ __forceinline__ uint32_t tile_off(uint32_t row, uint32_t chunk) {
    uint32_t half = chunk >> 3, c = chunk & 7u;
    return half * kHalfBytes + row * 128u + ((c ^ (row & 7u)) << 4);
}

// grid.x = kSplits * #clusters; cluster (kSplits,1,1); block 160 threads.
__global__ void __launch_bounds__(kThreads)
attn_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ o, uint32_t L, uint32_t G,
                   uint32_t Hq, uint32_t Hkv, uint32_t unit0, uint32_t unit1, uint32_t chunk, float scale,
                   uint32_t* err) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* ring = smem;
    const size_t gc = (size_t)G * chunk;
    float* scores = reinterpret_cast<float*>(smem + kStages * kStageBytes);           // [2][G][chunk]
    __nv_bfloat16* p_hi = reinterpret_cast<__nv_bfloat16*>(scores + 2 * gc);          // [2][G][chunk]
    __nv_bfloat16* p_lo = p_hi + 2 * gc;                                              // [2][G][chunk]
    // partial outputs of every rank for THIS CTA's slice of the (head, d) outputs, written by the peers
    float* o_gather = reinterpret_cast<float*>(p_lo + 2 * gc);                        // [3][kSplits][G*16]
    float* o_stage = o_gather + 3 * (size_t)G * kD;                                  // [G][128] local staging
    Control* ctl = reinterpret_cast<Control*>(o_stage + (size_t)G * kD);
    const uint32_t per_rank = G * kD / kSplits;                                       // outputs combined per CTA

    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t rank = cluster.block_rank();
    const uint32_t nclusters = gridDim.x / kSplits;
    const uint32_t first = unit0 + blockIdx.x / kSplits;
    const uint32_t n = first < unit1 ? (unit1 - first + nclusters - 1) / nclusters : 0;   // units of this cluster
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const uint32_t pos_begin = rank * chunk;
    const uint32_t valid = pos_begin < L ? min(chunk, L - pos_begin) : 0u;   // positions of this CTA per unit
    const uint32_t T = (valid + kTile - 1) / kTile;                          // K tiles (= V tiles) per unit

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&ctl->full[s])), "r"(1) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&ctl->empty[s])), "r"(4) : "memory");
        }
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == 4) {
        // =============================== producer warp ===============================
        // Tile stream, in groups of T tiles:  K(0) | K(1) V(0) | K(2) V(1) | ... | V(n-1)   (consumption order).
        // Cluster-barrier schedule: arrive_i as early as possible, wait_i only after K(i+1) has been issued, so the
        // ring keeps filling across the exchange and no consumer ever waits for an arrival the producer owes.
        uint32_t g = 0;
        bool ok = true;
        auto issue_group = [&](bool is_v, uint32_t j) {
            if (lane != 0) return;
            const CUtensorMap* map = is_v ? &map_v : &map_k;
            const int unit = (int)(first + j * nclusters);
            for (uint32_t t = 0; t < T; ++t, ++g) {
                if (!ok) continue;
                const uint32_t st = g % kStages;
                if (!mbar_wait(&ctl->empty[st], ((g / kStages) & 1u) ^ 1u, ctl, err)) { ok = false; continue; }
                uint64_t* bar = &ctl->full[st];
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                             "r"((uint32_t)kStageBytes)
                             : "memory");
                tma_load_4d(smem_u32(ring + st * kStageBytes), map, 0, (int)(pos_begin + t * kTile), 0, unit, bar);
            }
        };
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
        }
        cluster_arrive();                                    // arrive_0
        if (n > 0) issue_group(false, 0);
        for (uint32_t i = 0; i <= n + 1; ++i) {
            if (i >= 1 && i <= n) issue_group(true, i - 1);
            if (i + 1 < n) issue_group(false, i + 1);
            __syncwarp();
            cluster_wait();                                  // wait_i
            if (i < n + 1) cluster_arrive();                 // arrive_{i+1}
        }
    } else {
        // =============================== consumer warps 0..3 ===============================
        bool aborted = false;
        uint32_t g = 0;   // tiles consumed so far
        // warp-uniform: wait for tile gg to land
        auto acquire = [&](uint32_t gg) -> bool {
            bool ok = mbar_wait(&ctl->full[gg % kStages], (gg / kStages) & 1u, ctl, err);
            return __all_sync(0xFFFFFFFFu, ok);
        };
        auto release = [&](uint32_t gg) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->empty[gg % kStages]);
        };

        // Q of unit j as B fragments of S^T = K * Q^T: lane holds Q[head = lane/4][d = 16*ks + 2*(lane%4) + {0,1}], d + 8
        auto load_q = [&](uint32_t j, uint32_t (&dst)[8][2]) {
            const uint32_t unit = first + j * nclusters;
            const uint32_t head = lane >> 2;
            const __nv_bfloat16* qrow = q + ((size_t)unit * G + head) * kD;   // (b*Hq + kvh*G + head) = unit*G + head
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t d = ks * 16 + (lane & 3u) * 2;
                dst[ks][0] = head < G ? *reinterpret_cast<const uint32_t*>(qrow + d) : 0u;
                dst[ks][1] = head < G ? *reinterpret_cast<const uint32_t*>(qrow + d + 8) : 0u;
            }
        };
        uint32_t qb[8][2], qn[8][2];
        if (n > 0) load_q(0, qn);

        for (uint32_t i = 0; i <= n + 1; ++i) {
            // ---------------- K tiles of unit i: raw scores ----------------
            if (i < n) {
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) { qb[ks][0] = qn[ks][0]; qb[ks][1] = qn[ks][1]; }
                if (i + 1 < n) load_q(i + 1, qn);     // lands while this unit streams
                float* sc = scores + (size_t)(i & 1u) * gc;
                for (uint32_t t = 0; t < T; ++t, ++g) {
                    if (aborted || !acquire(g)) { aborted = true; continue; }
                    const uint32_t base = smem_u32(ring + (g % kStages) * kStageBytes);
                    // The legacy MMA has a long result latency here, so the eight 16-wide d slices go to eight
                    // independent accumulators (no MMA waits on another) and are joined by a fixed fp32 tree.
                    float cs[8][4];
                    const uint32_t row = warp * 16 + (lane & 7u) + ((lane >> 3) & 1u) * 8;
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        uint32_t a[4];
                        ldsm_x4(base + tile_off(row, ks * 2 + (lane >> 4)), a);
                        cs[ks][0] = cs[ks][1] = cs[ks][2] = cs[ks][3] = 0.0f;
                        mma_bf16(cs[ks], a, qb[ks][0], qb[ks][1]);
                    }
                    release(g);
                    float c[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        c[e] = cmath::add(cmath::add(cmath::add(cs[0][e], cs[1][e]), cmath::add(cs[2][e], cs[3][e])),
                                          cmath::add(cmath::add(cs[4][e], cs[5][e]), cmath::add(cs[6][e], cs[7][e])));
                    // C fragment: rows (lane/4, lane/4+8) of this warp's 16 positions, heads 2*(lane%4)+{0,1}
                    const uint32_t p0 = t * kTile + warp * 16 + (lane >> 2);
                    const uint32_t h0 = (lane & 3u) * 2;
                    if (h0 < G) {
                        sc[(size_t)h0 * chunk + p0] = cmath::mul(c[0], scale);
                        sc[(size_t)h0 * chunk + p0 + 8] = cmath::mul(c[2], scale);
                    }
                    if (h0 + 1 < G) {
                        sc[(size_t)(h0 + 1) * chunk + p0] = cmath::mul(c[1], scale);
                        sc[(size_t)(h0 + 1) * chunk + p0 + 8] = cmath::mul(c[3], scale);
                    }
                }
                consumer_sync();
                // chunk maxima (order-free on finite data)
                for (uint32_t h = warp; h < G; h += 4) {
                    float m = __uint_as_float(0xFF800000u);
                    if (!ctl->abort_flag)
                        for (uint32_t p = lane; p < valid; p += 32) m = fmaxf(m, sc[(size_t)h * chunk + p]);
#pragma unroll
                    for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
                    // push: lane r stores this chunk's maximum into rank r's table, so after the barrier
                    // every CTA finds all eight maxima in its own shared memory
                    if (lane < (uint32_t)kSplits) *cluster.map_shared_rank(&ctl->lmax_all[i & 1u][rank][h], lane) = m;
                }
            }
            __syncwarp();
            cluster_arrive();

            // ---------------- V tiles of unit i-1: O^T = V^T * P^T over this chunk ----------------
            if (i >= 1 && i <= n) {
                const uint32_t j = i - 1;
                const __nv_bfloat16* ph = p_hi + (size_t)(j & 1u) * gc;
                const __nv_bfloat16* pl = p_lo + (size_t)(j & 1u) * gc;
                // one accumulator per (d tile, 16-position slice, hi/lo half of p): within a tile no MMA waits on
                // another; each accumulator only chains from tile to tile.  Joined by a fixed fp32 tree at the end.
                float acc[2][4][2][4];
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
                        for (int e = 0; e < 4; ++e) { acc[mt][ks][0][e] = 0.0f; acc[mt][ks][1][e] = 0.0f; }
                for (uint32_t t = 0; t < T; ++t, ++g) {
                    if (aborted || !acquire(g)) { aborted = true; continue; }
                    const uint32_t base = smem_u32(ring + (g % kStages) * kStageBytes);
                    const uint32_t tile_pos = t * kTile;
                    const uint32_t head = lane >> 2;
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        uint32_t bh0 = 0, bh1 = 0, bl0 = 0, bl1 = 0;
                        if (head < G) {
                            size_t off = (size_t)head * chunk + tile_pos + ks * 16 + (lane & 3u) * 2;
                            bh0 = *reinterpret_cast<const uint32_t*>(ph + off);
                            bh1 = *reinterpret_cast<const uint32_t*>(ph + off + 8);
                            bl0 = *reinterpret_cast<const uint32_t*>(pl + off);
                            bl1 = *reinterpret_cast<const uint32_t*>(pl + off + 8);
                        }
                        const uint32_t prow = ks * 16 + (lane & 7u) + (lane >> 4) * 8;
#pragma unroll
                        for (int mt = 0; mt < 2; ++mt) {
                            uint32_t a[4];
                            ldsm_x4_trans(base + tile_off(prow, (warp * 2 + mt) * 2 + ((lane >> 3) & 1u)), a);
                            mma_bf16(acc[mt][ks][0], a, bh0, bh1);
                            mma_bf16(acc[mt][ks][1], a, bl0, bl1);
                        }
                    }
                    release(g);
                }
                // partial outputs: C fragment rows d = 16*mtile + lane/4 (+8), heads 2*(lane%4)+{0,1},
                // staged as [head][d] in local shared memory ...
                const uint32_t h0 = (lane & 3u) * 2;
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    const uint32_t d0 = (warp * 2 + mt) * 16 + (lane >> 2);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const uint32_t h = h0 + (e & 1), d = d0 + (e >> 1) * 8;
                        if (h < G) {
                            const float hi = cmath::add(cmath::add(acc[mt][0][0][e], acc[mt][1][0][e]),
                                                        cmath::add(acc[mt][2][0][e], acc[mt][3][0][e]));
                            const float lo = cmath::add(cmath::add(acc[mt][0][1][e], acc[mt][1][1][e]),
                                                        cmath::add(acc[mt][2][1][e], acc[mt][3][1][e]));
                            o_stage[h * kD + d] = cmath::add(hi, lo);
                        }
                    }
                }
                consumer_sync();
                // ... then pushed 16 bytes at a time: outputs [idx, idx+4) belong to the slice of rank
                // idx / per_rank, which will combine them (per_rank is a multiple of 4)
                for (uint32_t v4 = tid; v4 < G * (kD / 4); v4 += kConsumers) {
                    const uint32_t idx = v4 * 4;
                    const uint32_t dst_rank = idx / per_rank;
                    float* og = o_gather + ((size_t)(j % 3u) * kSplits + rank) * per_rank + (idx - dst_rank * per_rank);
                    *reinterpret_cast<float4*>(cluster.map_shared_rank(og, dst_rank)) =
                        *reinterpret_cast<const float4*>(o_stage + idx);
                }
            }
            __syncwarp();
            cluster_wait();

            // ---------------- unit i: global max over the cluster, probabilities, chunk denominator ----------------
            if (i < n) {
                if (tid < G) {
                    float m = __uint_as_float(0xFF800000u);
#pragma unroll
                    for (uint32_t r = 0; r < (uint32_t)kSplits; ++r) m = fmaxf(m, ctl->lmax_all[i & 1u][r][tid]);
                    ctl->gmax[tid] = m;
                }
                consumer_sync();
                const float* sc = scores + (size_t)(i & 1u) * gc;
                __nv_bfloat16* ph = p_hi + (size_t)(i & 1u) * gc;
                __nv_bfloat16* pl = p_lo + (size_t)(i & 1u) * gc;
                const bool dead = ctl->abort_flag != 0;
                // fixed order: thread t sums positions t, t+128, ... ascending; xor butterfly per warp; warps 0..3 ascending
                for (uint32_t h = 0; h < G; ++h) {
                    const float m = ctl->gmax[h];
                    float acc = 0.0f;
                    for (uint32_t p = tid; p < chunk; p += kConsumers) {
                        float pv = 0.0f;
                        if (p < valid && !dead) pv = cmath::exp_approx(cmath::sub(sc[(size_t)h * chunk + p], m));
                        __nv_bfloat16 hi = __float2bfloat16_rn(pv);
                        __nv_bfloat16 lo = __float2bfloat16_rn(cmath::sub(pv, __bfloat162float(hi)));
                        ph[(size_t)h * chunk + p] = hi;
                        pl[(size_t)h * chunk + p] = lo;
                        acc = cmath::add(acc, pv);
                    }
#pragma unroll
                    for (int off = 16; off >= 1; off >>= 1) acc = cmath::add(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, off));
                    if (lane == 0) ctl->warp_part[warp][h] = acc;
                }
                consumer_sync();
                if (tid < G) {
                    float d = ctl->warp_part[0][tid];
                    for (int w = 1; w < 4; ++w) d = cmath::add(d, ctl->warp_part[w][tid]);
#pragma unroll
                    for (uint32_t r = 0; r < (uint32_t)kSplits; ++r)
                        *cluster.map_shared_rank(&ctl->den_all[i % 3u][rank][tid], r) = d;
                }
            }

            // ---------------- unit i-2: combine in ascending chunk order, one slice of the outputs per CTA ----------------
            if (i >= 2) {
                const uint32_t j = i - 2;
                if (tid < per_rank) {   // per_rank = G*16 <= 128
                    const uint32_t idx = rank * per_rank + tid;
                    const uint32_t h = idx / kD, d = idx % kD;
                    const float* og = o_gather + (size_t)(j % 3u) * kSplits * per_rank + tid;
                    float num = 0.0f, den = 0.0f;
#pragma unroll
                    for (uint32_t r = 0; r < (uint32_t)kSplits; ++r) {
                        num = cmath::add(num, og[r * per_rank]);
                        den = cmath::add(den, ctl->den_all[j % 3u][r][h]);
                    }
                    const uint32_t unit = first + j * nclusters;
                    if (!ctl->abort_flag)
                        o[((size_t)unit * G + h) * kD + d] = __float2bfloat16_rn(cmath::div(num, den));
                }
            }
        }
    }
    __syncwarp();
    if (ctl->abort_flag) {
        uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    // nobody leaves while peers may still write into its shared memory
    cluster_arrive();
    cluster_wait();
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

// KV cache [units, L, 128] bf16 viewed as a 4-D tensor (64 d, L positions, 2 d-halves, units) so that one
// copy of box 64 x 64 x 2 x 1 brings a whole 64-position tile as [d-half][position][128 B], 128B-swizzled;
// positions past L read as zero, so a ragged last tile never touches the next unit's rows.
static catena_status_t make_kv_map(CUtensorMap* map, const void* base, uint64_t units, uint64_t L, uint64_t cap) {
    EncodeTiledFn fn = attn_encode_fn();
    if (!fn) return fail(CATENA_E_CUDA, "cuTensorMapEncodeTiled is unavailable");
    cuuint64_t dims[4] = {64, L, 2, units};
    cuuint64_t strides[3] = {(cuuint64_t)attn::kD * 2, 128, cap * (cuuint64_t)attn::kD * 2};   // a unit owns `cap` rows
    cuuint32_t box[4] = {64, (cuuint32_t)attn::kTile, 2, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(CATENA_E_CUDA, "cuTensorMapEncodeTiled (kv cache) failed");
    return CATENA_OK;
}

static thread_local uint32_t* g_attn_err_dev[16] = {nullptr};
static thread_local uint32_t* g_attn_err_host[16] = {nullptr};
// Test hook shared with the GEMM: caps the number of resident clusters (0 = as many as fit).
static int g_attn_cluster_limit = 0;
void attn_set_cluster_limit(int limit) { g_attn_cluster_limit = limit > 0 ? limit : 0; }
// Geometry of this thread's last decode launch: {kernel (0 mma.sync, 1 tcgen05), clusters that fit, clusters launched,
// dynamic shared memory per CTA}.
thread_local uint32_t g_attn_last_launch[4] = {0, 0, 0, 0};
void attn_last_launch(uint32_t out[4]) { for (int i = 0; i < 4; ++i) out[i] = g_attn_last_launch[i]; }

// Kernel selection: the tcgen05 kernel (attn_decode_tc.cu) wherever it supports the problem, else the mma.sync
// kernel in this file.  CATENA_B200_ATTN_TC=0 (read once) or the test hook forces the mma.sync kernel; both
// implement the same semantics.
static int g_attn_tc_mode = -1;
static bool attn_tc_mode() {
    if (g_attn_tc_mode < 0) {
        const char* e = getenv("CATENA_B200_ATTN_TC");
        g_attn_tc_mode = (e && e[0] == '0') ? 0 : 1;
    }
    return g_attn_tc_mode == 1;
}
void attn_set_tc_mode(int on) { g_attn_tc_mode = on ? 1 : 0; }
bool attn_tc_supports(uint32_t G, uint64_t kv_len);
void attn_tc_reset_exchange();
catena_status_t enqueue_attn_decode_tc(const void* q, const void* kc, const void* vc, void* o, uint64_t units, uint32_t G,
                                       uint64_t kv_len, uint64_t kv_cap, uint64_t unit0, uint64_t unit1, int cluster_limit,
                                       uint32_t* err_dev, void* const* peer_o, uint32_t n_peers, const AttnPrefetch* prefetch);

// After enqueuing: in blocking mode wait and turn a device-side bounded-wait expiry into a status.
static catena_status_t attn_finish_launch(int dev) {
    if (tls().blocking) {
        cudaStream_t st = tls().stream;
        CATENA_CUDA(cudaMemcpyAsync(g_attn_err_host[dev], g_attn_err_dev[dev], sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
        CATENA_CUDA(cudaStreamSynchronize(st));
        if (*g_attn_err_host[dev] != 0) {
            *g_attn_err_host[dev] = 0;
            cudaMemsetAsync(g_attn_err_dev[dev], 0, sizeof(uint32_t), st);
            attn_tc_reset_exchange();
            return fail(CATENA_E_TIMEOUT, "attn_decode: bounded wait expired");
        }
    }
    return CATENA_OK;
}

static uint32_t chunk_for(uint64_t L) {
    uint64_t c = ceil_div_u64(ceil_div_u64(L, attn::kSplits), attn::kTile) * attn::kTile;
    return (uint32_t)(c < (uint64_t)attn::kTile ? attn::kTile : c);
}
static size_t attn_smem_bytes(uint32_t G, uint32_t chunk) {
    return 1024 + (size_t)attn::kStages * attn::kStageBytes + 2 * (size_t)G * chunk * (4 + 2 + 2) +
           4 * (size_t)G * attn::kD * 4 + sizeof(attn::Control) + 16;
}

catena_status_t launch_attn_decode(const void* q, const void* kc, const void* vc, void* o, uint64_t batch, uint64_t hq,
                                   uint64_t hkv, uint64_t d, uint64_t kv_len, uint64_t kv_cap, uint64_t unit0, uint64_t unit1,
                                   void* const* peer_o, uint32_t n_peers, const AttnPrefetch* prefetch) {
    CATENA_TRY(ensure_device());
    if (!q || !kc || !vc || !o) return fail(CATENA_E_BAD_ARG, "attn_decode: null operand");
    if (d != (uint64_t)attn::kD) return fail(CATENA_E_UNSUPPORTED, "attn_decode: head_dim must be 128");
    if (hkv == 0 || hq % hkv != 0 || hq / hkv > (uint64_t)attn::kMaxG)
        return fail(CATENA_E_UNSUPPORTED, "attn_decode: Hq must be a multiple of Hkv with Hq/Hkv <= 8");
    if (kv_len == 0 || batch == 0) return fail(CATENA_E_BAD_ARG, "attn_decode: empty cache");
    if (kv_cap < kv_len) return fail(CATENA_E_BAD_ARG, "attn_decode: cache capacity below the visible length");
    uint64_t units = batch * hkv;
    if (unit1 > units || unit0 > unit1) return fail(CATENA_E_BAD_ARG, "attn_decode: unit range");
    if (unit0 == unit1) return CATENA_OK;
    if (((uintptr_t)kc & 15) || ((uintptr_t)vc & 15) || ((uintptr_t)q & 3)) return fail(CATENA_E_BAD_ARG, "attn_decode: alignment");
    if (kv_len > 0x7FFFFFFFull || kv_cap > 0x7FFFFFFFull || units > 0x7FFFFFFFull) return fail(CATENA_E_TOO_LARGE, "attn_decode: size");
    const uint32_t G = (uint32_t)(hq / hkv);
    int dev = tls().device;
    if (!g_attn_err_dev[dev]) {
        CATENA_CUDA(cudaMalloc(&g_attn_err_dev[dev], sizeof(uint32_t)));
        CATENA_CUDA(cudaMemset(g_attn_err_dev[dev], 0, sizeof(uint32_t)));
        CATENA_CUDA(cudaMallocHost(&g_attn_err_host[dev], sizeof(uint32_t)));
        *g_attn_err_host[dev] = 0;
    }
    if (attn_tc_mode() && attn_tc_supports(G, kv_len) && ((uintptr_t)q & 15) == 0) {
        CATENA_TRY(enqueue_attn_decode_tc(q, kc, vc, o, units, G, kv_len, kv_cap, unit0, unit1, g_attn_cluster_limit, g_attn_err_dev[dev],
                                          peer_o, n_peers, prefetch));
        return attn_finish_launch(dev);
    }
    if (n_peers > 0) return fail(CATENA_E_UNSUPPORTED, "attn_decode: peer outputs need the tcgen05 kernel (at most 7168 cache rows, 16-byte aligned q)");
    const uint32_t chunk = chunk_for(kv_len);
    const size_t smem = attn_smem_bytes(G, chunk);
    if (smem > 227 * 1024) return fail(CATENA_E_TOO_LARGE, "attn_decode: KV length beyond the shared-memory score buffer");

    CUtensorMap map_k, map_v;
    CATENA_TRY(make_kv_map(&map_k, kc, units, kv_len, kv_cap));
    CATENA_TRY(make_kv_map(&map_v, vc, units, kv_len, kv_cap));
    CATENA_CUDA(cudaFuncSetAttribute(attn::attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));

    cudaLaunchConfig_t cfg = {};
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
    // persistent clusters: as many as can be resident at once, never more than there are units
    cfg.gridDim = dim3((unsigned)(attn::kSplits * (unit1 - unit0)));
    int max_clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&max_clusters, attn::attn_decode_kernel, &cfg) != cudaSuccess || max_clusters < 1) {
        (void)cudaGetLastError();
        max_clusters = 16;
    }
    uint64_t clusters = unit1 - unit0;
    if (clusters > (uint64_t)max_clusters) clusters = (uint64_t)max_clusters;
    if (g_attn_cluster_limit > 0 && clusters > (uint64_t)g_attn_cluster_limit) clusters = (uint64_t)g_attn_cluster_limit;
    cfg.gridDim = dim3((unsigned)(clusters * attn::kSplits));
    g_attn_last_launch[0] = 0; g_attn_last_launch[1] = (uint32_t)max_clusters;
    g_attn_last_launch[2] = (uint32_t)clusters; g_attn_last_launch[3] = (uint32_t)smem;
    float scale = 1.0f / sqrtf((float)attn::kD);
    CATENA_CUDA(cudaLaunchKernelEx(&cfg, attn::attn_decode_kernel, map_k, map_v, (const __nv_bfloat16*)q, (__nv_bfloat16*)o,
                                   (uint32_t)kv_len, G, (uint32_t)hq, (uint32_t)hkv, (uint32_t)unit0, (uint32_t)unit1, chunk,
                                   scale, g_attn_err_dev[dev]));
    count_launch();
    return attn_finish_launch(dev);
}

catena_status_t attn_check_errors() {
    CATENA_TRY(ensure_device());
    int dev = tls().device;
    if (!g_attn_err_dev[dev]) return CATENA_OK;
    cudaStream_t st = tls().stream;
    CATENA_CUDA(cudaMemcpyAsync(g_attn_err_host[dev], g_attn_err_dev[dev], sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    CATENA_CUDA(cudaStreamSynchronize(st));
    if (*g_attn_err_host[dev] != 0) {
        *g_attn_err_host[dev] = 0;
        cudaMemsetAsync(g_attn_err_dev[dev], 0, sizeof(uint32_t), st);
        attn_tc_reset_exchange();
        return fail(CATENA_E_TIMEOUT, "attn_decode: bounded wait expired");
    }
    return CATENA_OK;
}

}  // namespace catena
