// Tensor-core GEMM for sm_100a on CTA PAIRS: C[M,N] = A[M,K] * B^T, A row-major [M,K], B stored [N,K]
// (both K-major), bf16 -> fp32 -> bf16 or int8 -> int32 -> int32.  Same arithmetic contract as the
// single-CTA kernel in gemm_tc.cu: one TMEM accumulator per output tile, k-blocks issued in ascending
// order, no split-K, no atomics; tile -> CTA map and grid size never enter the arithmetic.
//
// Why pairs: with one CTA per 128x256 tile each SM must pull 48 KiB per 512 tensor-cycles (96 B/clk);
// at the measured L2 latency that needs more bytes in flight than shared memory can hold, so the
// tensor pipe waits on the ring.  `tcgen05.mma.cta_group::2` computes a 256x256 tile on two SMs with
// each CTA loading only its own 128 rows of A and its own 128 rows (half of N) of B — 32 KiB per
// k-block per SM (64 B/clk) — which a 6-stage ring covers.
//
// Structure (cluster of 2 CTAs = 2 SMs, persistent, 192 threads per CTA):
//   warp 0      TMA producer in BOTH CTAs: `cp.async.bulk.tensor.2d.cta_group::2` (no multicast) of its
//               A and B halves into its own 128B-swizzled ring; every load signals the LEADER CTA's
//               full barrier, which the leader arms with the byte count of both CTAs;
//   warp 1      both CTAs allocate TMEM together (`tcgen05.alloc.cta_group::2`); the LEADER's elected
//               thread issues `tcgen05.mma.cta_group::2` (M=256, N<=256) and `tcgen05.commit` with a
//               cluster multicast mask, releasing ring stages / publishing accumulators in both CTAs;
//   warps 2-5   epilogue in both CTAs: `tcgen05.ld` of the CTA's own 128 accumulator rows, convert,
//               store, then arrive on the leader's tmem-empty barrier (remote arrive for the peer).
// Every mbarrier wait is bounded (about one second); the cluster barriers at start and end are
// hardware barriers that every thread of both CTAs reaches unconditionally.
#include <cuda.h>
#include <cuda_bf16.h>

#include "catena_math.cuh"
#include "common.cuh"

namespace catena {

namespace tc2 {

constexpr int BM = 128;            // rows per CTA (pair tile: 256)
constexpr int BN = 256;            // pair-tile columns = TMEM columns per accumulator
constexpr int BK_BYTES = 128;
#ifndef CATENA_GEMM_STAGES
#define CATENA_GEMM_STAGES 7
#endif
constexpr int MAX_STAGES = 7;
// ring depth: the plain kernel fills shared memory with stages; the gather-fused one keeps 16 KiB for its transposes
constexpr int stages_for(bool has_peers) { return has_peers ? 6 : CATENA_GEMM_STAGES; }
constexpr int A_BYTES = BM * BK_BYTES;              // 16 KiB
constexpr int B_BYTES = (BN / 2) * BK_BYTES;        // 16 KiB: this CTA's half of N
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;      // 32 KiB
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;
constexpr int TMEM_COLS = 512;
#ifndef CATENA_GEMM_GROUP_M
#define CATENA_GEMM_GROUP_M 8
#endif
constexpr int GROUP_M = CATENA_GEMM_GROUP_M;   // rasterisation in pair-tile rows (8 x 256 rows)
constexpr int kMaxPeers = 7;       // other GPUs of an 8-GPU box

// Where the epilogue stores each output tile besides this GPU's C: peer-mapped pointers (CUDA IPC / P2P) to the same
// rows of the other GPUs' copies of C.  The gather of a row-sharded GEMM then rides on the epilogue's stores.
struct PeerOut {
    void* ptr[kMaxPeers];
    uint32_t n;
    const void* residual;         // EPI_RESIDUAL: bf16 [M, ldc] added to the rounded product
    GemmRopeOut rope;             // EPI_ROPE
};
// epilogue variants (separate instantiations: the plain kernel carries none of the others' code or registers)
constexpr int EPI_PLAIN = 0;      // C = round(A B^T)
constexpr int EPI_PEERS = 1;      // the same, also stored to peer-mapped copies of C (gather-fused)
constexpr int EPI_RESIDUAL = 2;   // bf16 only: C = round(round(A B^T) + residual), the sum taken in fp32
constexpr int EPI_SWIGLU = 4;     // bf16 only, B = [2 F, K] (gate rows, then up rows): C [M, F] = silu(round(gate)) * round(up).  The
                                  // leader CTA loads 128 gate rows, its peer the 128 up rows of the same outputs, so a 256-column
                                  // accumulator holds gate and up of 128 outputs side by side; N is 2 F in the tile arithmetic
constexpr int EPI_ROPE = 3;       // bf16 only, a q/k/v projection: the rounded product is rotated (q, k heads) and stored
                                  // straight into the query buffer and the KV caches (GemmRopeOut); C itself is not written

struct __align__(8) Control {
    uint64_t full[MAX_STAGES];       // used in the leader CTA
    uint64_t empty[MAX_STAGES];      // one per CTA, signalled by the leader's commit (multicast)
    uint64_t tmem_full[2];       // one per CTA, signalled by the leader's commit (multicast)
    uint64_t tmem_empty[2];      // used in the leader CTA: 2 x 128 epilogue threads arrive
    uint64_t wait_ns;            // limit of every bounded wait of this launch
    uint32_t tmem_base;
    volatile uint32_t abort_flag;
};
constexpr int PEER_STAGE_BYTES = 32 * 128;           // per epilogue warp: 32 rows x 32 int32 (or bf16) columns, for peer stores
constexpr int smem_bytes(bool has_peers) {
    return stages_for(has_peers) * STAGE_BYTES + 1024 + (int)((sizeof(Control) + 15) / 16 * 16) + (has_peers ? 4 * PEER_STAGE_BYTES : 0);
}
static_assert(smem_bytes(false) <= 232448 && smem_bytes(true) <= 232448, "shared memory per CTA");

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// arrive on a barrier anywhere in the cluster (address from mapa)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Control* ctl, uint32_t* err, uint32_t code) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 255u) == 0) {
            if (ctl->abort_flag) return false;
            if (globaltimer_ns() - t0 > ctl->wait_ns) {
                ctl->abort_flag = 1;
                atomicCAS(err, 0u, code);
                return false;
            }
        }
    }
}
// TMA load into this CTA's shared memory; completion bytes go to `bar_cluster_addr` (the leader's barrier)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// arrives (once the MMAs issued so far have completed) on the barrier at this shared-memory offset in
// every CTA of `mask`
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar, uint16_t mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask)
                 : "memory");
}
template <bool IS_I8>
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    if (IS_I8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0),
              "r"(0), "r"(0), "r"(0)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0),
              "r"(0), "r"(0), "r"(0)
            : "memory");
    }
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
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// K-major, 128 B rows, 128B swizzle: start >> 4, LBO field 1 (unused), SBO = 1024 B, version 1, SWIZZLE_128B
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// dense, K-major A and B; c_format F32 / S32; a,b format BF16 / signed int8; N >> 3 at [17,23); M >> 4 at [24,29), M = 256
template <bool IS_I8>
__device__ __forceinline__ uint32_t make_idesc(uint32_t n) {
    return ((IS_I8 ? 2u : 1u) << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

struct Work {
    uint32_t m_blk;   // pair-tile row block (256 rows)
    uint32_t col0;    // first column
    uint32_t width;   // columns: 256, or 128 / 64 for the units of the last partial round
};

// Static schedule over CTA pairs; the tiles of the last partial round are cut along N into `split` units
// (timing only: an element's k order does not depend on the unit width).
__device__ __forceinline__ bool get_work(uint32_t it, uint32_t pair, uint32_t pairs, uint32_t mb, uint32_t nb, uint32_t tiles,
                                         uint32_t split, Work& w) {
    const uint32_t full = (tiles / pairs) * pairs;
    const uint32_t idx = it * pairs + pair;
    uint32_t t, part = 0, width = BN;
    if (idx < full) {
        t = idx;
    } else {
        const uint32_t u = idx - full;
        if (u >= (tiles - full) * split) return false;
        t = full + u / split;
        part = u % split;
        width = BN / split;
    }
    const uint32_t per_group = GROUP_M * nb;
    const uint32_t g = t / per_group;
    const uint32_t first_m = g * GROUP_M;
    const uint32_t rows = min((uint32_t)GROUP_M, mb - first_m);
    const uint32_t in_g = t - g * per_group;
    w.m_blk = first_m + in_g % rows;
    w.col0 = (in_g / rows) * BN + part * width;
    w.width = width;
    return true;
}

template <bool IS_I8, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b128,
                const __grid_constant__ CUtensorMap map_b64, const __grid_constant__ CUtensorMap map_b32,
                void* __restrict__ c_out, PeerOut peers, uint32_t M, uint32_t N, uint32_t K, uint64_t ldc, uint32_t split, uint32_t* err,
                uint64_t wait_ns, uint32_t stall_kb) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr bool HAS_PEERS = EPI == EPI_PEERS;
    constexpr int STAGES = HAS_PEERS ? 6 : CATENA_GEMM_STAGES;
    Control* ctl = reinterpret_cast<Control*>(smem + STAGES * STAGE_BYTES);
    uint8_t* peer_stage = smem + STAGES * STAGE_BYTES + (sizeof(Control) + 15) / 16 * 16;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    constexpr uint32_t K_ELEMS = IS_I8 ? BK_BYTES : BK_BYTES / 2;
    constexpr uint32_t MMA_PER_BLOCK = BK_BYTES / 32;
    const uint32_t mb = (M + 2 * BM - 1) / (2 * BM), nb = (N + BN - 1) / BN;
    const uint32_t tiles = mb * nb;
    const uint32_t kblocks = (K + K_ELEMS - 1) / K_ELEMS;

    // Programmatic dependent launch: the next kernel of the stream may be scheduled as soon as every CTA of this grid
    // has got here, so its launch latency and set-up run under this grid's tail; this grid in turn does its own set-up
    // (barriers, TMEM, tensor maps) and then waits below for everything launched before it to complete.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b128)) : "memory");
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctl->tmem_full[b], 1);
            mbar_init(&ctl->tmem_empty[b], 2 * EPI_THREADS);
        }
        ctl->abort_flag = 0;
        ctl->wait_ns = wait_ns;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // both CTAs' barriers exist before anything in the pair signals them
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    asm volatile("griddepcontrol.wait;" ::: "memory");     // no global memory is read or written above this line

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer (both CTAs) ----------------
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            Work w;
            for (uint32_t it = 0; ok && get_work(it, pair, pairs, mb, nb, tiles, split, w); ++it) {
                const uint32_t half = w.width / 2;     // this CTA's rows of B
                const CUtensorMap* mapb = half == 128u ? &map_b128 : (half == 64u ? &map_b64 : &map_b32);
                const uint32_t bytes_pair = 2u * (A_BYTES + half * BK_BYTES);
                const int a_row = (int)(w.m_blk * 2 * BM + rank * BM);
                const int b_row = EPI == EPI_SWIGLU ? (int)(w.col0 / 2 + rank * (N / 2)) : (int)(w.col0 + rank * half);
                for (uint32_t kb = 0; kb < kblocks; ++kb) {
                    // test hook: the producers of both CTAs stop before k-block stall_kb - 1 of their first tile, so the
                    // issuer's wait for that stage runs out and the whole pair takes the give-up path
                    if (stall_kb != 0 && it == 0 && kb + 1 == stall_kb) { ok = false; break; }
                    if (!mbar_wait(&ctl->empty[stage], phase ^ 1u, ctl, err, 1u)) { ok = false; break; }
                    if (rank == 0) mbar_expect_tx(&ctl->full[stage], bytes_pair);
                    const uint32_t bar = mapa(smem_u32(&ctl->full[stage]), 0);
                    const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
                    tma_load_2d_pair(sa, &map_a, (int)(kb * K_ELEMS), a_row, bar);
                    tma_load_2d_pair(sa + A_BYTES, mapb, (int)(kb * K_ELEMS), b_row, bar);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---------------- MMA issuer (leader CTA only) ----------------
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            Work w;
            for (uint32_t it = 0; ok && get_work(it, pair, pairs, mb, nb, tiles, split, w); ++it) {
                const uint32_t idesc = make_idesc<IS_I8>(w.width);
                if (!mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1u, ctl, err, 2u)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (uint32_t kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(&ctl->full[stage], phase, ctl, err, 3u)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
                    const uint64_t da = make_smem_desc(sa);
                    const uint64_t db = make_smem_desc(sa + A_BYTES);
#pragma unroll
                    for (uint32_t kk = 0; kk < MMA_PER_BLOCK; ++kk)
                        tc_mma_pair<IS_I8>(tmem_d, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
                    tc_commit_pair(&ctl->empty[stage], 3);     // both CTAs may refill this stage
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc_commit_pair(&ctl->tmem_full[acc], 3);       // accumulator complete in both CTAs
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: warps 2..5 of both CTAs ----------------
        const uint32_t quad = warp & 3u;
        const uint32_t row_in_cta = quad * 32 + lane;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        Work w;
        for (uint32_t it = 0; ok && get_work(it, pair, pairs, mb, nb, tiles, split, w); ++it) {
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(&ctl->tmem_full[acc], acc_phase, ctl, err, 4u));
            if (!ok) break;
            tc_fence_after();
            const uint32_t row = w.m_blk * 2 * BM + rank * BM + row_in_cta;
            const uint32_t taddr = tmem_base + ((quad * 32u) << 16) + acc * BN;
            if (EPI == EPI_SWIGLU) {
                // columns 0..127 = gate, 128..255 = up of outputs col0 / 2 .. col0 / 2 + 127: both are rounded to bf16 as the
                // unfused projection would have stored them, then nn.silu(gate) * up, eight outputs side by side
                const uint32_t F = N / 2, out0 = w.col0 / 2;
#pragma unroll 1
                for (uint32_t c = 0; c < 128; c += 32) {
                    uint32_t vg[32], vu[32];
                    tmem_ld32(taddr + c, vg);
                    tmem_ld32(taddr + 128 + c, vu);
                    tmem_ld_wait();
                    if (row < M) {
                        uint32_t o[16];
#pragma unroll
                        for (int e = 0; e < 32; e += 8) {
                            float g[8], sg[8];
#pragma unroll
                            for (int u = 0; u < 8; ++u) g[u] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(vg[e + u])));
                            cmath::silu_n<8>(g, sg);
#pragma unroll
                            for (int u = 0; u < 8; u += 2) {
                                const float u0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(vu[e + u])));
                                const float u1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(vu[e + u + 1])));
                                const __nv_bfloat162 h = __floats2bfloat162_rn(__fmul_rn(sg[u], u0), __fmul_rn(sg[u + 1], u1));
                                o[(e + u) >> 1] = *reinterpret_cast<const uint32_t*>(&h);
                            }
                        }
                        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(c_out) + (uint64_t)row * ldc + out0 + c;
                        if (out0 + c + 32 <= F && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) reinterpret_cast<uint4*>(dst)[q] = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
                        } else {
                            for (int q = 0; q < 32; ++q)
                                if (out0 + c + q < F) reinterpret_cast<uint16_t*>(dst)[q] = (uint16_t)(q & 1 ? o[q >> 1] >> 16 : o[q >> 1] & 0xFFFFu);
                        }
                    }
                }
            }
            if (EPI == EPI_ROPE) {
                // A 256-column tile is two heads of 128.  Rotary pairs are (i, i + 64): the thread reads 32 columns of
                // each half of a head, rounds both to bf16 as the unfused projection would have stored them, rotates with
                // separately rounded products (llama::rope_append_kernel's arithmetic) and stores 64 B to either half.
                const GemmRopeOut& ro = peers.rope;
                const uint32_t seq_i = row / ro.seq, s_pos = row - seq_i * ro.seq, pos = ro.pos0 + s_pos;
                for (uint32_t hcol = 0; hcol < w.width && w.col0 + hcol < N; hcol += 128) {
                    const uint32_t head = (w.col0 + hcol) >> 7;
                    __nv_bfloat16* dst;
                    bool rotate = true;
                    if (head < ro.hq) {
                        dst = static_cast<__nv_bfloat16*>(ro.q_out) + ((uint64_t)row * ro.hq + head) * 128;
                    } else if (head < ro.hq + ro.hkv) {
                        dst = static_cast<__nv_bfloat16*>(ro.k_cache) + (((uint64_t)seq_i * ro.hkv + (head - ro.hq)) * ro.cap + pos) * 128;
                    } else {
                        dst = static_cast<__nv_bfloat16*>(ro.v_cache) + (((uint64_t)seq_i * ro.hkv + (head - ro.hq - ro.hkv)) * ro.cap + pos) * 128;
                        rotate = false;
                    }
#pragma unroll 1
                    for (uint32_t j = 0; j < 2; ++j) {
                        uint32_t va[32], vb[32];
                        tmem_ld32(taddr + hcol + 32 * j, va);
                        tmem_ld32(taddr + hcol + 64 + 32 * j, vb);
                        tmem_ld_wait();
                        if (row < M) {
                            const float4* tab = reinterpret_cast<const float4*>(ro.table + (uint64_t)s_pos * 64 + 32 * j);
                            uint32_t o1[16], o2[16];
#pragma unroll
                            for (int e = 0; e < 32; e += 2) {
                                const float x1a = __bfloat162float(__float2bfloat16_rn(__uint_as_float(va[e])));
                                const float x1b = __bfloat162float(__float2bfloat16_rn(__uint_as_float(va[e + 1])));
                                const float x2a = __bfloat162float(__float2bfloat16_rn(__uint_as_float(vb[e])));
                                const float x2b = __bfloat162float(__float2bfloat16_rn(__uint_as_float(vb[e + 1])));
                                float r1a = x1a, r1b = x1b, r2a = x2a, r2b = x2b;
                                if (rotate) {
                                    const float4 cs = tab[e >> 1];            // (cos, sin) of pairs e and e + 1
                                    r1a = __fsub_rn(__fmul_rn(x1a, cs.x), __fmul_rn(x2a, cs.y));
                                    r2a = __fadd_rn(__fmul_rn(x2a, cs.x), __fmul_rn(x1a, cs.y));
                                    r1b = __fsub_rn(__fmul_rn(x1b, cs.z), __fmul_rn(x2b, cs.w));
                                    r2b = __fadd_rn(__fmul_rn(x2b, cs.z), __fmul_rn(x1b, cs.w));
                                }
                                const __nv_bfloat162 h1 = __floats2bfloat162_rn(r1a, r1b), h2 = __floats2bfloat162_rn(r2a, r2b);
                                o1[e >> 1] = *reinterpret_cast<const uint32_t*>(&h1);
                                o2[e >> 1] = *reinterpret_cast<const uint32_t*>(&h2);
                            }
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                reinterpret_cast<uint4*>(dst + 32 * j)[q] = make_uint4(o1[4 * q], o1[4 * q + 1], o1[4 * q + 2], o1[4 * q + 3]);
                                reinterpret_cast<uint4*>(dst + 64 + 32 * j)[q] = make_uint4(o2[4 * q], o2[4 * q + 1], o2[4 * q + 2], o2[4 * q + 3]);
                            }
                        }
                    }
                }
            }
#pragma unroll 1
            for (uint32_t c = 0; EPI != EPI_ROPE && EPI != EPI_SWIGLU && c < w.width; c += 32) {
                uint32_t v[32];
                tmem_ld32(taddr + c, v);
                uint4 res[4];
                bool res_whole = false;
                if (EPI == EPI_RESIDUAL && row < M) {          // in flight together with the accumulator load
                    const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(peers.residual) + (uint64_t)row * ldc + w.col0 + c;
                    res_whole = w.col0 + c + 32 <= N && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
                    if (res_whole) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) res[q] = reinterpret_cast<const uint4*>(src)[q];
                    }
                }
                tmem_ld_wait();
                if (row < M) {
                    const uint32_t col = w.col0 + c;
                    uint4 out[8];
                    if (IS_I8) {
#pragma unroll
                        for (int q = 0; q < 8; ++q) out[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                    } else {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint32_t p[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 2 * e]),
                                                                         __uint_as_float(v[8 * q + 2 * e + 1]));
                                p[e] = *reinterpret_cast<uint32_t*>(&h);
                                if (EPI == EPI_RESIDUAL && res_whole) {
                                    const uint32_t rw = e == 0 ? res[q].x : (e == 1 ? res[q].y : (e == 2 ? res[q].z : res[q].w));
                                    h = __floats2bfloat162_rn(__fadd_rn(__uint_as_float(p[e] << 16), __uint_as_float(rw << 16)),
                                                              __fadd_rn(__uint_as_float(p[e] & 0xFFFF0000u), __uint_as_float(rw & 0xFFFF0000u)));
                                    p[e] = *reinterpret_cast<uint32_t*>(&h);
                                }
                            }
                            out[q] = make_uint4(p[0], p[1], p[2], p[3]);
                        }
                    }
                    // this GPU's C: each thread stores its own row (L2 merges the partial lines)
                    if (IS_I8) {
                        int32_t* dst = reinterpret_cast<int32_t*>(c_out) + (uint64_t)row * ldc + col;
                        if (col + 32 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
                            for (int q = 0; q < 8; ++q) reinterpret_cast<uint4*>(dst)[q] = out[q];
                        } else {
                            for (int q = 0; q < 32; ++q)
                                if (col + q < N) dst[q] = (int32_t)v[q];
                        }
                    } else {
                        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(c_out) + (uint64_t)row * ldc + col;
                        if (col + 32 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) reinterpret_cast<uint4*>(dst)[q] = out[q];
                        } else {
                            for (int q = 0; q < 32; ++q) {
                                if (col + q >= N) break;
                                __nv_bfloat16 o = __float2bfloat16_rn(__uint_as_float(v[q]));
                                if (EPI == EPI_RESIDUAL) {
                                    const __nv_bfloat16 r = (reinterpret_cast<const __nv_bfloat16*>(peers.residual) + (uint64_t)row * ldc + col)[q];
                                    o = __float2bfloat16_rn(__fadd_rn(__bfloat162float(o), __bfloat162float(r)));
                                }
                                dst[q] = o;
                            }
                        }
                    }
                }
                // peer copies: NVLink wants whole 128-byte lines, so the warp's block is transposed through shared memory (rows
                // of 128 B, the 16-byte chunk index xor-ed with the row) and written with lanes along the columns.  A row of
                // 32 int32 columns is one line; of bf16 it is half a line, so two consecutive 32-column steps share a row
                // of the stage and are written out together (64 B segments reached only 400 GB/s per rank, lines 650).
                if (HAS_PEERS && peers.n > 0) {
                    constexpr uint32_t EB = IS_I8 ? 4u : 2u;              // bytes per output element
                    constexpr uint32_t CH = IS_I8 ? 8u : 4u;              // 16-byte chunks this step adds to a stage row
                    const uint32_t half = IS_I8 ? 0u : ((c >> 5) & 1u);   // bf16: which half of the line this step is
                    const uint32_t col = w.col0 + c, col_line = col - half * 32u;
                    uint8_t* stage = peer_stage + quad * PEER_STAGE_BYTES;
                    const bool whole = col_line + (IS_I8 ? 32u : 64u) <= N && ((ldc * EB) & 15u) == 0 && ((col_line * EB) & 15u) == 0;
                    if (whole) {
                        uint4 out[8];
                        if (IS_I8) {
#pragma unroll
                            for (int q = 0; q < 8; ++q) out[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                        } else {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                uint32_t p[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 2 * e]),
                                                                             __uint_as_float(v[8 * q + 2 * e + 1]));
                                    p[e] = *reinterpret_cast<uint32_t*>(&h);
                                }
                                out[q] = make_uint4(p[0], p[1], p[2], p[3]);
                            }
                        }
#pragma unroll
                        for (uint32_t q = 0; q < CH; ++q)
                            *reinterpret_cast<uint4*>(stage + lane * 128u + (((q + half * 4u) ^ (lane & 7u)) << 4)) = out[q];
                        __syncwarp();
                        if (IS_I8 || half == 1u) {
                            const uint32_t row_base = w.m_blk * 2 * BM + rank * BM + quad * 32;
#pragma unroll
                            for (uint32_t j = 0; j < 8; ++j) {              // 4 rows of 128 B per instruction
                                const uint32_t r = j * 4 + lane / 8, q = lane % 8;
                                const uint4 val = *reinterpret_cast<const uint4*>(stage + r * 128u + ((q ^ (r & 7u)) << 4));
                                if (row_base + r < M) {
                                    const uint64_t off = ((uint64_t)(row_base + r) * ldc + col_line) * EB + q * 16;
#pragma unroll
                                    for (uint32_t pi = 0; pi < (uint32_t)kMaxPeers; ++pi)
                                        if (pi < peers.n) *reinterpret_cast<uint4*>(static_cast<uint8_t*>(peers.ptr[pi]) + off) = val;
                                }
                            }
                            __syncwarp();
                        }
                    } else if (row < M) {
#pragma unroll
                        for (uint32_t pi = 0; pi < (uint32_t)kMaxPeers; ++pi) {
                            if (pi >= peers.n) break;
                            for (int q = 0; q < 32; ++q) {
                                if (col + q >= N) break;
                                if (IS_I8) (reinterpret_cast<int32_t*>(peers.ptr[pi]) + (uint64_t)row * ldc + col)[q] = (int32_t)v[q];
                                else (reinterpret_cast<__nv_bfloat16*>(peers.ptr[pi]) + (uint64_t)row * ldc + col)[q] = __float2bfloat16_rn(__uint_as_float(v[q]));
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive_cluster(mapa(smem_u32(&ctl->tmem_empty[acc]), 0));   // the leader's barrier counts both CTAs
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
    }

    // ---------------- teardown ----------------
    __syncwarp();
    if (ctl->abort_flag) {
        uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before();
    // neither CTA frees TMEM or leaves while its peer can still signal or read it
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

}  // namespace tc2

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn2 encode_fn2() {
    static EncodeTiledFn2 fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn2)p;
    }
    return fn;
}
static catena_status_t make_map2(CUtensorMap* map, const void* base, uint64_t rows, uint64_t k_elems, int elem_bytes,
                                 uint32_t box_rows) {
    EncodeTiledFn2 fn = encode_fn2();
    if (!fn) return fail(CATENA_E_CUDA, "cuTensorMapEncodeTiled is unavailable");
    cuuint64_t dims[2] = {k_elems, rows};
    cuuint64_t strides[1] = {k_elems * (uint64_t)elem_bytes};
    cuuint32_t box[2] = {(cuuint32_t)(tc2::BK_BYTES / elem_bytes), box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                    const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(CATENA_E_CUDA, "cuTensorMapEncodeTiled failed");
    return CATENA_OK;
}

// Enqueues the CTA-pair GEMM.  `err_dev` is the device error word shared with the single-CTA kernel.
catena_status_t enqueue_gemm_tc2(const void* a, const void* b, void* c, uint64_t m, uint64_t n, uint64_t k, uint64_t ldc,
                                 int is_i8, int cta_limit, uint32_t* err_dev, void* const* peer_c, uint32_t n_peers, const void* residual,
                                 const GemmRopeOut* rope, int swiglu) {
    if (swiglu && (is_i8 || n_peers || residual || rope || n % 256)) return fail(CATENA_E_BAD_ARG, "gemm: bad SwiGLU epilogue");
    if ((residual || rope) && (is_i8 || n_peers)) return fail(CATENA_E_BAD_ARG, "gemm: a residual / rotary epilogue goes with the plain bf16 kernel only");
    if (rope && (residual || n % 128 || !rope->table || !rope->q_out || !rope->k_cache || !rope->v_cache || !rope->seq ||
                 n != (uint64_t)(rope->hq + 2 * rope->hkv) * 128))
        return fail(CATENA_E_BAD_ARG, "gemm: bad rotary epilogue");
    if (n_peers > (uint32_t)tc2::kMaxPeers) return fail(CATENA_E_BAD_ARG, "gemm: more than 7 peer outputs");
    tc2::PeerOut peers = {};
    peers.n = n_peers;
    peers.residual = residual;
    if (rope) peers.rope = *rope;
    for (uint32_t i = 0; i < n_peers; ++i) {
        if (!peer_c || !peer_c[i] || ((uintptr_t)peer_c[i] & 15)) return fail(CATENA_E_BAD_ARG, "gemm: null or unaligned peer output");
        peers.ptr[i] = peer_c[i];
    }
    const int eb = is_i8 ? 1 : 2;
    CUtensorMap map_a, map_b128, map_b64, map_b32;
    CATENA_TRY(make_map2(&map_a, a, m, k, eb, tc2::BM));
    CATENA_TRY(make_map2(&map_b128, b, n, k, eb, 128));
    CATENA_TRY(make_map2(&map_b64, b, n, k, eb, 64));
    CATENA_TRY(make_map2(&map_b32, b, n, k, eb, 32));
    typedef void (*KernelFn)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, void*, tc2::PeerOut, uint32_t,
                             uint32_t, uint32_t, uint64_t, uint32_t, uint32_t*, uint64_t, uint32_t);
    KernelFn kernel = is_i8 ? (n_peers ? tc2::gemm_tc2_kernel<true, tc2::EPI_PEERS> : tc2::gemm_tc2_kernel<true, tc2::EPI_PLAIN>)
                            : (n_peers ? tc2::gemm_tc2_kernel<false, tc2::EPI_PEERS>
                                       : swiglu ? tc2::gemm_tc2_kernel<false, tc2::EPI_SWIGLU>
                                       : (rope ? tc2::gemm_tc2_kernel<false, tc2::EPI_ROPE>
                                               : (residual ? tc2::gemm_tc2_kernel<false, tc2::EPI_RESIDUAL> : tc2::gemm_tc2_kernel<false, tc2::EPI_PLAIN>)));
    const int smem_bytes = tc2::smem_bytes(n_peers != 0);
    CATENA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    const uint64_t tiles = ceil_div_u64(m, 2 * tc2::BM) * ceil_div_u64(n, tc2::BN);
    const int sms = tls().sm_count > 0 ? tls().sm_count : 148;
    uint64_t pairs = (uint64_t)(sms / 2);
    if (cta_limit > 0 && pairs > (uint64_t)(cta_limit / 2 > 0 ? cta_limit / 2 : 1)) pairs = (uint64_t)(cta_limit / 2 > 0 ? cta_limit / 2 : 1);
    if (tiles < pairs) pairs = tiles;
    const uint64_t rem = tiles % pairs;
    // (the rotary epilogue needs whole heads in a unit: no cut along N)
    const uint32_t split = rem == 0 || rope || swiglu ? 1u : (rem * 4 <= pairs ? 4u : (rem * 2 <= pairs ? 2u : 1u));
    const unsigned grid = (unsigned)(pairs * 2);
    cudaStream_t st = tls().stream;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(tc2::NUM_THREADS);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    static const bool pdl = [] { const char* v = getenv("CATENA_B200_GEMM_PDL"); return !(v && v[0] == '0'); }();
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, map_a, map_b128, map_b64, map_b32, c, peers, (uint32_t)m, (uint32_t)n, (uint32_t)k, ldc,
                                       split, err_dev, debug_wait_limit_ns(), debug_take_stall(1));
    count_launch();
    if (e != cudaSuccess) return fail_cuda(e, "gemm_tc2 launch");
    return CATENA_OK;
}

}  // namespace catena
