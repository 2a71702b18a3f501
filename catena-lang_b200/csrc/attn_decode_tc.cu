// Cached-attention decode on tcgen05 — same semantics as attn_decode.cu (global max, the reference's exp
// polynomial, 8 KV chunks per unit combined in ascending order), with both contractions on the 5th-generation
// tensor cores and the accumulators in TMEM:
//   S^T[128 positions x 16 heads] = K_tile[128 x 128 d] * Q^T      A = K tile in shared memory (K-major,
//                                                                  128B swizzle, as TMA wrote it), B = Q
//   O^T[128 d x 16 heads]        += V_tile^T[128 d x 128 pos] * P^T A = the SAME V tile read as an
//                                                                  MN-major operand (no transpose),
//                                                                  B = probabilities (bf16 hi, then lo)
// Heads beyond G are padding columns that nobody reads.
//
// A kernel that allocates TMEM gets ONE resident CTA per SM from the driver, whatever its shared memory and
// registers, and clusters of 8 such CTAs cover only 120 of the 148 SMs.  So this kernel uses no clusters: it is
// a persistent grid of one CTA per SM (cooperative launch: every CTA is resident), and each CTA runs TWO
// independent pipelines ("pipes"), each with its own TMA producer warp, MMA issuer warp, four consumer warps,
// shared-memory ring, operand buffers and 256 TMEM columns.  The work item of a pipe is one KV chunk of one
// unit: item w = 8 * unit + chunk goes to pipe (w mod #pipes), round (w div #pipes).  #pipes is a multiple of
// 8, so the 8 chunks of a unit are always handled in the same round by 8 neighbouring pipes.
//
// What the 8 chunks of a unit exchange goes through global memory (L2):
//   * chunk maxima: one 8-byte word {launch epoch, float bits} per (item, head), published with a single store
//     and polled (bounded) by the unit's 8 pipes before the probabilities are computed;
//   * partial outputs and denominators: written per item and counted on a ticket per unit; when all 8 are
//     counted, each of the 8 pipes adds the 8 partials of its eighth of the unit's outputs in ascending chunk
//     order.  Values are never accumulated with atomics; the ticket only says that the partials are complete.
// A pipe publishes the maxima of round r before it waits for anything of round r, and its own progress never
// depends on another pipe otherwise, so the waits cannot form a cycle.
//
// Scores never go to shared memory: the (at most 7) score tiles of a chunk stay in TMEM (two sets, so the next
// item's K tiles are multiplied while this item's probabilities are computed) and are read twice with
// tcgen05.ld — once for the maxima, once for exp~.
//   warps 0-3 / 4-7   consumers of pipe 0 / 1 (warp w reads TMEM lanes 32*(w%4)..)
//   warps 8 / 9       TMA producers (one 4-D copy per 128-position tile, no multicast)
//   warps 10 / 11     MMA issuers; warp 10 also allocates and frees the CTA's 512 TMEM columns
//   warps 12 / 13     finishers: count every item the consumers hand over on the unit's ticket, wait for the unit's
//                     other chunks and combine — dependent L2 round trips that the consumers never wait for
// All waits (mbarrier and global polls) are bounded; an expiry sets the CTA's abort flag and the error word.
#include <cuda.h>
#include <cuda_bf16.h>

#include "catena_math.cuh"
#include "common.cuh"

namespace catena {

namespace attn2 {

constexpr int kD = 128;
constexpr int kTile = 128;                   // positions per ring stage
#ifndef CATENA_ATTN_TC_STAGES
#define CATENA_ATTN_TC_STAGES 3
#endif
constexpr int kStages = CATENA_ATTN_TC_STAGES;
constexpr int kSplits = 8;
constexpr int kHalfBytes = kTile * 128;      // 16 KiB: 128 positions x 64 d
constexpr int kStageBytes = 2 * kHalfBytes;  // [d-half 2][position 128][128 B]
constexpr int kPipes = 2;
constexpr int kConsumers = 128;              // per pipe
constexpr int kThreads = kPipes * (kConsumers + 96);   // + producer, issuer and finisher warp per pipe
constexpr int kMaxG = 8;
constexpr int kMaxTiles = 7;                 // score tiles of one chunk (kept in TMEM)
constexpr int kSBufs = 2 * kMaxTiles;        // two sets of score accumulators
constexpr int kPipeCols = 256;               // TMEM columns per pipe: score buffer b at [16b, 16b+16), outputs at kOCol
constexpr int kOCol = 16 * kSBufs;
constexpr int kQBytes = 2 * 16 * 128;        // Q as a UMMA B operand: [d-half 2][16 head rows][128 B]
constexpr int kPSlots = 2;                   // probability operands of single tiles, reused round-robin
constexpr int kPTileBytes = 2 * 2048;        // per 64-position atom 16 rows x 128 B: rows 0..7 = bf16 hi part of p per
                                             //   head, rows 8..15 = lo part
constexpr int kOpsBytes = 2 * kQBytes + kPSlots * kPTileBytes;   // operand bytes per pipe (Q double-buffered)
// a waiting thread may be suspended by the hardware for up to this long (it is woken when the phase completes)
constexpr uint32_t kSuspendHintNs = 20000;

struct __align__(16) Control {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t s_full[kSBufs], s_free[kSBufs];   // score accumulators in TMEM
    uint64_t o_full, o_free;                   // output accumulator in TMEM
    uint64_t q_ready[2];                       // Q operand written
    uint64_t p_ready[kPSlots], p_free[kPSlots];   // probability operand of a tile written / multiplied
    uint64_t fin_ready, fin_done;              // an item's partial outputs handed to / taken by the finisher warp
    float warp_max[4][kMaxG];
    float warp_part[4][kMaxG];
    float lmax[kSplits][kMaxG];
    float gmax[kMaxG];
};
struct __align__(16) Common {
    uint64_t wait_ns;              // limit of every bounded wait of this launch
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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Common* com, uint32_t* err) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 255u) == 0) {
            if (com->abort_flag) return false;
            if (globaltimer_ns() - t0 > com->wait_ns) {
                com->abort_flag = 1;
                atomicCAS(err, 0u, 2u);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// generic-proxy writes to shared memory -> visible to the tensor core's (async proxy) operand reads
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// named barrier of one pipe's 128 consumer threads
__device__ __forceinline__ void consumer_sync(uint32_t pipe) { asm volatile("bar.sync %0, 128;" ::"r"(pipe + 1u) : "memory"); }
__device__ __forceinline__ uint64_t ld_relaxed_u64(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_u64(uint64_t* p, uint64_t v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Shared-memory matrix descriptors (128B swizzle, descriptor version 1).
//   K-major  (rows of 128 B along K; 8-row groups 1024 B apart): K tile as A, Q and P as B.
//   MN-major (rows of 128 B along M = 64 d; consecutive K = positions are consecutive rows; 8-position groups
//            1024 B apart = SBO; the second 64-d block `lbo` bytes away = LBO): V tile as A.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr, uint32_t lbo) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// instruction descriptor: fp32 accumulate, bf16 operands, M = 128, N = 16; bit 15 = A is MN-major
constexpr uint32_t kIdescQK = (1u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kIdescPV = kIdescQK | (1u << 15);

// math.exp-approx (catena-lang/stdlib/math.hex:148-199) of four arguments at once, the same operations in the
// same order as cmath::exp_approx but written stage by stage across the four values so that four independent
// dependency chains are in flight.
__device__ __forceinline__ void exp_approx4(const float (&x)[4], float (&out)[4]) {
    float mag[4], kf[4], xr[4], p[4];
    uint32_t k[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) mag[u] = x[u] < 0.0f ? -x[u] : x[u];
#pragma unroll
    for (int u = 0; u < 4; ++u) k[u] = cmath::round_to_u32(cmath::mul(mag[u], cmath::from_bits(0x3FB8AA3Bu)));
#pragma unroll
    for (int u = 0; u < 4; ++u) kf[u] = cmath::u32_to_f32(k[u]);
#pragma unroll
    for (int u = 0; u < 4; ++u) xr[u] = cmath::sub(mag[u], cmath::mul(kf[u], cmath::from_bits(0x3F317200u)));
#pragma unroll
    for (int u = 0; u < 4; ++u) xr[u] = cmath::sub(xr[u], cmath::mul(kf[u], cmath::from_bits(0x35BFBE8Eu)));
#pragma unroll
    for (int u = 0; u < 4; ++u) p[u] = cmath::add(cmath::from_bits(0x3EEF1187u), cmath::mul(xr[u], cmath::from_bits(0x3E738A8Bu)));
#pragma unroll
    for (int u = 0; u < 4; ++u) p[u] = cmath::add(cmath::from_bits(0x3F809C7Eu), cmath::mul(xr[u], p[u]));
#pragma unroll
    for (int u = 0; u < 4; ++u) p[u] = cmath::add(cmath::from_bits(0x3F7FF8FCu), cmath::mul(xr[u], p[u]));
#pragma unroll
    for (int u = 0; u < 4; ++u) p[u] = cmath::mul(p[u], cmath::from_bits((k[u] + 0x7Fu) * 0x00800000u));
#pragma unroll
    for (int u = 0; u < 4; ++u) out[u] = x[u] < 0.0f ? cmath::recip(p[u]) : p[u];
}

// Byte offset of element (row, col) in a K-major 128B-swizzled operand whose rows hold 64 bf16 (one atom):
// used for Q (row = head, col = d % 64) and P (row = head, col = position % 64).
__device__ __forceinline__ uint32_t operand_off(uint32_t row, uint32_t col) {
    return row * 128u + ((((col >> 3) ^ (row & 7u)) & 7u) << 4) + (col & 7u) * 2u;
}

// Optional timeline of one CTA's pipe 0 (build with -DCATENA_ATTN_TRACE): lane 0 of the first consumer warp, of the
// producer and of the issuer stamp clock64() into a device array that a debug entry point copies out.
#ifdef CATENA_ATTN_TRACE
__device__ unsigned long long g_trace[4][1024];
__device__ unsigned int g_trace_n[4];
#define TR(role, tag)                                                                                              \
    do {                                                                                                           \
        if (trace_on && trn < 1024u)                                                                               \
            g_trace[role][trn++] = ((unsigned long long)(tag) << 48) | ((unsigned long long)clock64() & 0xFFFFFFFFFFFFull); \
    } while (0)
#else
#define TR(role, tag) do { } while (0)
#endif

// Global-memory exchange area of one launch stream (see the header comment).
struct Exchange {
    uint64_t* maxima;     // [items][8]  {epoch << 32 | float bits}
    float* partial;       // [items][G][128]
    float* denom;         // [items][8]
    uint32_t* tickets;    // [units]     arrivals, counted modulo 8 (cleared by the host after a failed launch)
    uint32_t epoch;
};

// Where a unit's outputs go besides this GPU's O: peer-mapped pointers (CUDA IPC) to the other GPUs' copies of O, same
// layout.  The gather of a (batch, kv-head)-sharded launch then rides on the finishers' stores (plain stores over NVLink).
constexpr int kMaxPeers = 7;
struct PeerO {
    __nv_bfloat16* ptr[kMaxPeers];
    uint32_t n;
};

// Optional L2 prefetch hint: ranges of this GPU's memory that the kernels launched AFTER this one will stream (weights of
// the projections that follow a decode step's attention).  This kernel is latency-bound for short caches and leaves HBM
// bandwidth unused; an otherwise idle warp per CTA (the finisher of pipe 0, before its first item can be ready) issues
// paced bulk prefetches into L2 for the CTA's share of the ranges.  A hint only: nothing waits for it, results never
// depend on it.
constexpr int kMaxPrefetch = 4;
struct PrefetchHint {
    const uint8_t* ptr[kMaxPrefetch];
    uint32_t chunks[kMaxPrefetch];          // 16 KiB chunks of each range
    uint32_t n;
    uint32_t pace_ns;                       // pause between two chunks of a CTA
};
constexpr uint32_t kPrefetchChunk = 16384;

// grid.x CTAs (all resident), 384 threads; npipes = 2 * gridDim.x is a multiple of 8 or at least `items`.
__global__ void __launch_bounds__(kThreads, 1)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ o, uint32_t L, uint32_t G,
                      uint32_t unit0, uint32_t items, uint32_t chunk, float scale, Exchange ex, uint32_t* err, uint64_t wait_ns,
                      uint32_t stall, PeerO peers, PrefetchHint pf) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // role and pipe of this warp
    const uint32_t pipe = warp < 8 ? (warp >> 2) : (warp & 1u);    // warps 8.. alternate between the pipes
    uint8_t* ring = smem + pipe * (kStages * kStageBytes);             // kStages x 32 KiB per pipe
    uint8_t* ops = smem + kPipes * (kStages * kStageBytes);
    uint8_t* q_op = ops + pipe * kOpsBytes;
    uint8_t* p_op = q_op + 2 * kQBytes;                                // kPSlots x kPTileBytes
    Control* ctl = reinterpret_cast<Control*>(ops + kPipes * kOpsBytes) + pipe;
    Common* com = reinterpret_cast<Common*>(reinterpret_cast<Control*>(ops + kPipes * kOpsBytes) + kPipes);

    const uint32_t npipes = kPipes * gridDim.x;
    const uint32_t vid = blockIdx.x * kPipes + pipe;
    const uint32_t n = vid < items ? (items - vid + npipes - 1) / npipes : 0;    // items of this pipe
    const uint32_t rank = vid % kSplits;                                         // the same for all of them
    const uint32_t pos_begin = rank * chunk;
    const uint32_t valid = pos_begin < L ? min(chunk, L - pos_begin) : 0u;
    const uint32_t T = (valid + kTile - 1) / kTile;

    if (tid < kPipes) {
        Control* c = reinterpret_cast<Control*>(ops + kPipes * kOpsBytes) + tid;
        for (int s = 0; s < kStages; ++s) { mbar_init(&c->full[s], 1); mbar_init(&c->empty[s], 1); }
        for (int b = 0; b < kSBufs; ++b) {
            mbar_init(&c->s_full[b], 1);
            mbar_init(&c->s_free[b], kConsumers);
        }
        for (int b = 0; b < 2; ++b) mbar_init(&c->q_ready[b], kConsumers);
        mbar_init(&c->o_full, 1);
        mbar_init(&c->o_free, kConsumers);
        for (int b = 0; b < kPSlots; ++b) {
            mbar_init(&c->p_ready[b], kConsumers);
            mbar_init(&c->p_free[b], 1);
        }
        mbar_init(&c->fin_ready, kConsumers);
        mbar_init(&c->fin_done, 1);
        if (tid == 0) {
            com->abort_flag = 0;
            com->wait_ns = wait_ns;
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // operand buffers start as zeros: head rows >= G of Q and P are never written
    for (uint32_t i = tid; i < kPipes * kOpsBytes / 16; i += kThreads)
        reinterpret_cast<uint4*>(ops)[i] = make_uint4(0, 0, 0, 0);
    if (warp == 10) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&com->tmem_base)),
                     "r"((uint32_t)(kPipes * kPipeCols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_pipe = com->tmem_base + pipe * kPipeCols;
#ifdef CATENA_ATTN_TRACE
    const bool trace_on = blockIdx.x == 8 && lane == 0 && (warp == 0 || warp == 8 || warp == 10 || warp == 12);
    unsigned int trn = 0;
#endif

    if (warp >= 12) {
        // =============================== finisher ===============================
        // Item j of the pipe: once its partial outputs and denominator are in global memory, count it on the unit's
        // ticket, wait until all 8 chunks of the unit are counted, then combine THIS pipe's eighth of the unit's outputs
        // in ascending chunk order.  (One pipe combining the whole unit would be slower than its seven mates, which
        // all wait for it at the next exchange of maxima.)
        const uint32_t per_rank = G * kD / kSplits;          // outputs per pipe and unit: G * 16
        if (warp == 12 && lane == 0 && pf.n != 0) {
            for (uint32_t r = 0; r < pf.n && r < (uint32_t)kMaxPrefetch; ++r) {
                for (uint32_t c = blockIdx.x; c < pf.chunks[r]; c += gridDim.x) {
                    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(pf.ptr[r] + (size_t)c * kPrefetchChunk), "r"(kPrefetchChunk)
                                 : "memory");
                    if (pf.pace_ns) __nanosleep(pf.pace_ns);
                }
            }
        }
        __syncwarp();
        for (uint32_t j = 0; j < n; ++j) {
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(&ctl->fin_ready, j & 1u, com, err))) break;
            TR(3, 1);
            const uint32_t wj = vid + j * npipes;
            uint32_t ok = 1;
            if (lane == 0) {
                mbar_arrive(&ctl->fin_done);
                uint32_t* tk = ex.tickets + wj / kSplits;
                __threadfence();       // the consumers' stores (ordered before this by the mbarrier) before the ticket
                atomicAdd(tk, 1u);
                // tickets count modulo 8 across launches: a multiple of 8 means every chunk of this launch is in
                uint32_t seen;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(tk) : "memory");
                if (seen & 7u) {
                    const uint64_t t0 = globaltimer_ns();
                    uint32_t spins = 0;
                    while (true) {
                        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(tk) : "memory");
                        if ((seen & 7u) == 0) break;
                        if ((++spins & 63u) == 0) {
                            if (com->abort_flag) { ok = 0; break; }
                            if (globaltimer_ns() - t0 > com->wait_ns) {
                                com->abort_flag = 1;
                                atomicCAS(err, 0u, 4u);
                                ok = 0;
                                break;
                            }
                        }
                    }
                }
                __threadfence();
            }
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
            TR(3, 2);
            if (!ok) break;
            const size_t base = (size_t)(wj / kSplits) * kSplits;
            const uint32_t unit = unit0 + wj / kSplits;
            float pr[4][kSplits], dn[4][kSplits];
#pragma unroll
            for (uint32_t x = 0; x < 4; ++x) {               // per_rank <= 128: at most 4 outputs per lane
                const uint32_t e = min(lane + 32 * x, per_rank - 1), idx = rank * per_rank + e;
                const uint32_t h = idx / kD, d = idx % kD;
#pragma unroll
                for (uint32_t r = 0; r < (uint32_t)kSplits; ++r) {
                    pr[x][r] = __ldcg(ex.partial + ((base + r) * G + h) * kD + d);
                    dn[x][r] = __ldcg(ex.denom + (base + r) * 8 + h);
                }
            }
#pragma unroll
            for (uint32_t x = 0; x < 4; ++x) {
                const uint32_t e = lane + 32 * x, idx = rank * per_rank + e;
                float num = 0.0f, den = 0.0f;
#pragma unroll
                for (uint32_t r = 0; r < (uint32_t)kSplits; ++r) {   // ascending chunk order
                    num = cmath::add(num, pr[x][r]);
                    den = cmath::add(den, dn[x][r]);
                }
                if (e < per_rank && !com->abort_flag) {
                    const __nv_bfloat16 val = __float2bfloat16_rn(cmath::div(num, den));
                    const size_t off = (size_t)unit * G * kD + idx;
                    o[off] = val;
#pragma unroll
                    for (uint32_t pi = 0; pi < (uint32_t)kMaxPeers; ++pi)
                        if (pi < peers.n) peers.ptr[pi][off] = val;
                }
            }
            TR(3, 3);
        }
    } else if (warp >= 10) {
        // =============================== MMA issuer ===============================
        // Issue order per pipe:  K(0) | K(1) V(0) | K(2) V(1) | ... | V(n-1)
        if (lane == 0) {
            uint32_t g = 0;        // ring tiles consumed
            uint32_t pt = 0;       // probability tiles consumed
            bool ok = true;
            for (uint32_t i = 0; i <= n && ok; ++i) {
                if (i < n) {
                    // ---- S^T = K * Q^T for the tiles of item i, into score set i & 1 ----
                    ok = mbar_wait(&ctl->q_ready[i & 1u], (i >> 1) & 1u, com, err);
                    const uint32_t qa = smem_u32(q_op + (i & 1u) * kQBytes);
                    for (uint32_t t = 0; t < T && ok; ++t, ++g) {
                        const uint32_t b = (i & 1u) * kMaxTiles + t;
                        if (!mbar_wait(&ctl->s_free[b], ((i >> 1) & 1u) ^ 1u, com, err)) { ok = false; break; }
                        TR(2, 5);
                        if (!mbar_wait(&ctl->full[g % kStages], (g / kStages) & 1u, com, err)) { ok = false; break; }
                        TR(2, 6);
                        tc_fence_after();
                        const uint32_t sa = smem_u32(ring + (g % kStages) * kStageBytes);
#pragma unroll
                        for (uint32_t ks = 0; ks < 8; ++ks) {   // 16 d per MMA: d-half ks/4, 32 B steps inside the row
                            const uint64_t da = desc_kmajor(sa + (ks >> 2) * kHalfBytes + (ks & 3u) * 32);
                            const uint64_t db = desc_kmajor(qa + (ks >> 2) * (16 * 128) + (ks & 3u) * 32);
                            tc_mma_bf16(tmem_pipe + b * 16, da, db, kIdescQK, ks != 0 ? 1u : 0u);
                        }
                        tc_commit(&ctl->empty[g % kStages]);
                        tc_commit(&ctl->s_full[b]);
                        TR(2, 1);
                    }
                }
                if (i >= 1 && ok) {
                    // ---- O^T += V^T * P^T for the tiles of item i-1 ----
                    const uint32_t j = i - 1;
                    TR(2, 3);
                    ok = mbar_wait(&ctl->o_free, (j & 1u) ^ 1u, com, err);
                    for (uint32_t t = 0; t < T && ok; ++t, ++g, ++pt) {
                        const uint32_t slot = pt % kPSlots;
                        if (!mbar_wait(&ctl->p_ready[slot], (pt / kPSlots) & 1u, com, err)) { ok = false; break; }
                        TR(2, 4);
                        TR(2, 7);
                        if (!mbar_wait(&ctl->full[g % kStages], (g / kStages) & 1u, com, err)) { ok = false; break; }
                        TR(2, 8);
                        tc_fence_after();
                        const uint32_t sa = smem_u32(ring + (g % kStages) * kStageBytes);
#pragma unroll
                        for (uint32_t kk = 0; kk < 8; ++kk) {   // 16 positions per MMA
                            const uint64_t da = desc_mnmajor(sa + kk * 2048, kHalfBytes);
                            const uint32_t pa = slot * kPTileBytes + (kk >> 2) * 2048 + (kk & 3u) * 32;
                            // columns 0..7 accumulate the hi parts, columns 8..15 the lo parts
                            tc_mma_bf16(tmem_pipe + kOCol, da, desc_kmajor(smem_u32(p_op) + pa), kIdescPV, (t | kk) != 0 ? 1u : 0u);
                        }
                        tc_commit(&ctl->empty[g % kStages]);
                        tc_commit(&ctl->p_free[slot]);
                        TR(2, 2);
                    }
                    if (ok) tc_commit(&ctl->o_full);
                }
            }
        }
    } else if (warp >= 8) {
        // =============================== TMA producer ===============================
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
            uint32_t g = 0;
            bool ok = true;
            for (uint32_t i = 0; i <= n && ok; ++i) {
                for (uint32_t kv = 0; kv < 2 && ok; ++kv) {      // K of item i, then V of item i-1
                    if (kv == 0 ? i >= n : i == 0) continue;
                    const uint32_t j = kv == 0 ? i : i - 1;
                    const CUtensorMap* map = kv == 0 ? &map_k : &map_v;
                    const int unit = (int)(unit0 + (vid + j * npipes) / kSplits);
                    for (uint32_t t = 0; t < T; ++t, ++g) {
                        const uint32_t st = g % kStages;
                        if (!mbar_wait(&ctl->empty[st], ((g / kStages) & 1u) ^ 1u, com, err)) { ok = false; break; }
                        uint64_t* bar = &ctl->full[st];
                        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                                     "r"((uint32_t)kStageBytes)
                                     : "memory");
                        TR(1, 1 + kv);
                        tma_load_4d(smem_u32(ring + st * kStageBytes), map, 0, (int)(pos_begin + t * kTile), 0, unit, bar);
                    }
                }
            }
        }
    } else {
        // =============================== consumer warps (4 per pipe) ===============================
        // thread ct owns TMEM lane ct: position ct of a score tile, head-dim element ct of the outputs
        const uint32_t ct = tid & 127u, cw = warp & 3u;
        const uint32_t lane_addr = tmem_pipe + ((cw * 32u) << 16);
        const float ninf = __uint_as_float(0xFF800000u);
        bool aborted = false;
        // Q of item j -> UMMA B operand [d-half][head row][128 B], 128B-swizzled; rows >= G stay zero.  One 16-byte
        // piece (8 d of one head) per thread; the global load is issued early and stored after other work.
        const bool q_mine = ct < G * (kD / 8);
        const uint32_t q_h = ct / (kD / 8), q_d0 = (ct % (kD / 8)) * 8;
        auto q_fetch = [&](uint32_t j) -> uint4 {
            const uint32_t unit = unit0 + (vid + j * npipes) / kSplits;
            return q_mine ? *reinterpret_cast<const uint4*>(q + ((size_t)unit * G + q_h) * kD + q_d0) : make_uint4(0, 0, 0, 0);
        };
        auto q_store = [&](uint32_t j, const uint4& v) {
            if (q_mine) *reinterpret_cast<uint4*>(q_op + (j & 1u) * kQBytes + (q_d0 >> 6) * (16 * 128) + operand_off(q_h, q_d0 & 63u)) = v;
            fence_async_smem();
            mbar_arrive(&ctl->q_ready[j & 1u]);
        };
        if (n > 0) q_store(0, q_fetch(0));
        uint32_t pt = 0;       // probability tiles written

        for (uint32_t i = 0; i <= n; ++i) {
            const uint32_t w = vid + i * npipes;              // item i of this pipe
            const uint32_t set = (i & 1u) * kMaxTiles;
            TR(0, 10);
            // ---------------- item i: chunk maxima straight from TMEM, published ----------------
            if (i < n) {
                // the other Q buffer was last read by the K tiles of item i-1, whose scores this pipe has read
                if (i + 1 < n) q_store(i + 1, q_fetch(i + 1));
                float m[kMaxG];
#pragma unroll
                for (int h = 0; h < kMaxG; ++h) m[h] = ninf;
                for (uint32_t t = 0; t < T; ++t) {
                    if (aborted || !__all_sync(0xFFFFFFFFu, mbar_wait(&ctl->s_full[set + t], (i >> 1) & 1u, com, err))) {
                        aborted = true;
                        continue;
                    }
                    tc_fence_after();
                    uint32_t v[8];
                    tmem_ld8(lane_addr + (set + t) * 16, v);
                    tmem_ld_wait();
                    TR(0, 11);
                    if (t * kTile + ct < valid) {
#pragma unroll
                        for (int h = 0; h < kMaxG; ++h) m[h] = fmaxf(m[h], cmath::mul(__uint_as_float(v[h]), scale));
                    }
                }
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) {
#pragma unroll
                    for (int h = 0; h < kMaxG; ++h)
                        if ((uint32_t)h < G) m[h] = fmaxf(m[h], __shfl_xor_sync(0xFFFFFFFFu, m[h], off));
                }
                if (lane == 0) {
#pragma unroll
                    for (int h = 0; h < kMaxG; ++h) ctl->warp_max[cw][h] = m[h];
                }
                consumer_sync(pipe);
                // (test hook `stall`: item 0 never publishes its maxima, so the polls of its unit's pipes run out)
                if (ct < G && !(stall != 0 && w == 0)) {
                    float mm = fmaxf(fmaxf(ctl->warp_max[0][ct], ctl->warp_max[1][ct]), fmaxf(ctl->warp_max[2][ct], ctl->warp_max[3][ct]));
                    st_relaxed_u64(ex.maxima + (size_t)w * 8 + ct, ((uint64_t)ex.epoch << 32) | (uint64_t)__float_as_uint(mm));
                }
                TR(0, 12);
            }

            // ---------------- item i-1: partial outputs TMEM -> global ----------------
            if (i >= 1) {
                const uint32_t j = i - 1, wj = vid + j * npipes;
                uint32_t v[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) v[e] = 0u;
                if (!aborted) {
                    if (__all_sync(0xFFFFFFFFu, mbar_wait(&ctl->o_full, j & 1u, com, err))) {
                        if (T > 0) {      // with no tile the accumulator holds nothing of this item
                            tc_fence_after();
                            tmem_ld16(lane_addr + kOCol, v);
                            tmem_ld_wait();
                            tc_fence_before();
                        }
                    } else {
                        aborted = true;
                    }
                }
                mbar_arrive(&ctl->o_free);
                TR(0, 13);
                float* part = ex.partial + (size_t)wj * G * kD;
#pragma unroll
                for (uint32_t h = 0; h < (uint32_t)kMaxG; ++h)
                    if (h < G) part[h * kD + ct] = cmath::add(__uint_as_float(v[h]), __uint_as_float(v[8 + h]));
                // hand the item to the finisher (its denominator was stored in the previous iteration)
                if (j >= 1 && !aborted && !__all_sync(0xFFFFFFFFu, mbar_wait(&ctl->fin_done, (j - 1) & 1u, com, err))) aborted = true;
                mbar_arrive(&ctl->fin_ready);
            }

            // ---------------- item i: global max, probabilities as a UMMA operand, chunk denominator ----------------
            if (i < n) {
                if (cw == 0) {
                    const uint64_t* slots = ex.maxima + (size_t)(w - w % kSplits) * 8;
                    for (uint32_t s = lane; s < kSplits * G; s += 32) {
                        const uint32_t r = s / G, h = s - r * G;
                        uint64_t val = ld_relaxed_u64(slots + r * 8 + h);
                        if ((uint32_t)(val >> 32) != ex.epoch) {
                            const uint64_t t0 = globaltimer_ns();
                            uint32_t spins = 0;
                            while ((uint32_t)((val = ld_relaxed_u64(slots + r * 8 + h)) >> 32) != ex.epoch) {
                                if ((++spins & 63u) == 0) {
                                    if (com->abort_flag) break;
                                    if (globaltimer_ns() - t0 > com->wait_ns) {
                                        com->abort_flag = 1;
                                        atomicCAS(err, 0u, 3u);
                                        break;
                                    }
                                }
                            }
                        }
                        ctl->lmax[r][h] = __uint_as_float((uint32_t)val);
                    }
                    __syncwarp();
                    if (lane < (uint32_t)kMaxG) {
                        float mm = ninf;
#pragma unroll
                        for (uint32_t r = 0; r < (uint32_t)kSplits; ++r) mm = fmaxf(mm, ctl->lmax[r][lane < G ? lane : 0]);
                        ctl->gmax[lane] = lane < G ? mm : 0.0f;     // padding heads: finite, never used
                    }
                }
                __syncwarp();
                TR(0, 17);
                consumer_sync(pipe);
                TR(0, 18);
                const bool dead = com->abort_flag != 0;
                float gm[kMaxG];
#pragma unroll
                for (int h = 0; h < kMaxG; ++h) gm[h] = ctl->gmax[h];
                // fixed order: thread ct sums positions ct, ct+128, ... ascending; xor butterfly per warp; warps 0..3
                // ascending.  The polynomial is one long dependent chain, so the heads are evaluated four at a time.
                float acc[kMaxG];
#pragma unroll
                for (int h = 0; h < kMaxG; ++h) acc[h] = 0.0f;
                for (uint32_t t = 0; t < T && !aborted; ++t, ++pt) {
                    uint32_t v[8];
                    tmem_ld8(lane_addr + (set + t) * 16, v);
                    tmem_ld_wait();
                    tc_fence_before();
                    mbar_arrive(&ctl->s_free[set + t]);
                    TR(0, 19);
                    const uint32_t p = t * kTile + ct;
                    const bool live = p < valid && !dead;
                    const uint32_t slot = pt % kPSlots;
                    uint8_t* prow = p_op + slot * kPTileBytes + (ct >> 6) * 2048;
                    // the tile that used this operand slot before has been multiplied
                    if (!__all_sync(0xFFFFFFFFu, mbar_wait(&ctl->p_free[slot], ((pt / kPSlots) & 1u) ^ 1u, com, err))) {
                        aborted = true;
                        break;
                    }
#pragma unroll
                    for (uint32_t hb = 0; hb < (uint32_t)kMaxG; hb += 4) {
                        if (hb < G) {
                            float xs[4], pv[4];
#pragma unroll
                            for (uint32_t u = 0; u < 4; ++u)   // padding heads have score 0 and are dropped below
                                xs[u] = cmath::sub(cmath::mul(__uint_as_float(v[hb + u]), scale), gm[hb + u]);
                            exp_approx4(xs, pv);
#pragma unroll
                            for (uint32_t u = 0; u < 4; ++u) {
                                const uint32_t h = hb + u;
                                if (h < G) {
                                    const float pe = live ? pv[u] : 0.0f;
                                    const __nv_bfloat16 hi = __float2bfloat16_rn(pe);
                                    const __nv_bfloat16 lo = __float2bfloat16_rn(cmath::sub(pe, __bfloat162float(hi)));
                                    const uint32_t off = operand_off(h, p & 63u);
                                    *reinterpret_cast<__nv_bfloat16*>(prow + off) = hi;
                                    *reinterpret_cast<__nv_bfloat16*>(prow + off + 1024) = lo;
                                    acc[h] = cmath::add(acc[h], pe);
                                }
                            }
                        }
                    }
                    fence_async_smem();
                    mbar_arrive(&ctl->p_ready[slot]);
                }
                TR(0, 20);
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) {
#pragma unroll
                    for (uint32_t h = 0; h < (uint32_t)kMaxG; ++h)
                        if (h < G) acc[h] = cmath::add(acc[h], __shfl_xor_sync(0xFFFFFFFFu, acc[h], off));
                }
                if (lane == 0) {
#pragma unroll
                    for (uint32_t h = 0; h < (uint32_t)kMaxG; ++h) ctl->warp_part[cw][h] = acc[h];
                }
                consumer_sync(pipe);
                if (ct < G) {
                    float d = ctl->warp_part[0][ct];
                    for (int x = 1; x < 4; ++x) d = cmath::add(d, ctl->warp_part[x][ct]);
                    ex.denom[(size_t)w * 8 + ct] = d;
                }
            }
        }
    }
#ifdef CATENA_ATTN_TRACE
    if (trace_on) g_trace_n[warp == 0 ? 0 : (warp - 6) / 2] = trn;
#endif
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 10) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(com->tmem_base),
                     "r"((uint32_t)(kPipes * kPipeCols))
                     : "memory");
    }
}

}  // namespace attn2

typedef CUresult (*EncodeTiledFnA2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFnA2 attn2_encode_fn() {
    static EncodeTiledFnA2 fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFnA2)p;
    }
    return fn;
}

// KV cache [units, cap, 128] bf16, L visible rows per unit, as a 4-D tensor (64 d, L positions, 2 d-halves, units): one copy of box
// 64 x 128 x 2 x 1 brings a 128-position tile as [d-half][position][128 B], 128B-swizzled; positions past L
// read as zero.
static catena_status_t make_kv_map2(CUtensorMap* map, const void* base, uint64_t units, uint64_t L, uint64_t cap) {
    EncodeTiledFnA2 fn = attn2_encode_fn();
    if (!fn) return fail(CATENA_E_CUDA, "cuTensorMapEncodeTiled is unavailable");
    cuuint64_t dims[4] = {64, L, 2, units};
    cuuint64_t strides[3] = {(cuuint64_t)attn2::kD * 2, 128, cap * (cuuint64_t)attn2::kD * 2};   // a unit owns `cap` rows
    cuuint32_t box[4] = {64, (cuuint32_t)attn2::kTile, 2, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(CATENA_E_CUDA, "cuTensorMapEncodeTiled (kv cache) failed");
    return CATENA_OK;
}

static uint32_t chunk_for2(uint64_t L) {
    uint64_t c = ceil_div_u64(ceil_div_u64(L, attn2::kSplits), attn2::kTile) * attn2::kTile;
    return (uint32_t)(c < (uint64_t)attn2::kTile ? attn2::kTile : c);
}
static size_t attn2_smem_bytes() {
    return 1024 + (size_t)attn2::kPipes * (attn2::kStages * attn2::kStageBytes + attn2::kOpsBytes + sizeof(attn2::Control)) +
           sizeof(attn2::Common) + 16;
}

// True when the tcgen05 kernel can take this problem: the score tiles of a chunk must fit its TMEM sets.
bool attn_tc_supports(uint32_t G, uint64_t kv_len) {
    const uint32_t chunk = chunk_for2(kv_len);
    return G >= 1 && G <= (uint32_t)attn2::kMaxG && chunk / attn2::kTile <= (uint32_t)attn2::kMaxTiles &&
           attn2_smem_bytes() <= 227 * 1024;
}

// Exchange area of the calling thread's stream, grown on demand and never shrunk.
struct AttnExchange {
    void* base = nullptr;          // maxima (epoch-tagged), denominators, partial outputs: laid out per launch
    size_t bytes = 0;
    uint32_t* tickets = nullptr;   // always at the same place: they carry their count (a multiple of 8) between launches
    size_t ticket_units = 0;
    uint32_t epoch = 0;
    size_t maxima_bytes = 0;       // extent of the last launch's epoch-tagged maxima (the whole area while it is all zeros):
                                   // bytes beyond it may hold raw floats of that launch's denominators / partial outputs
                                   // and are cleared before a later launch's maxima move onto them
};
static thread_local AttnExchange g_attn_exchange[16];
static thread_local int g_attn2_max_ctas[16] = {0};

static size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

// After a launch that reported an expired wait: its tickets may be left part-way, so the area is cleared (stream-ordered).
void attn_tc_reset_exchange() {
    AttnExchange& xa = g_attn_exchange[tls().device];
    if (xa.base) cudaMemsetAsync(xa.base, 0, xa.bytes, tls().stream);
    xa.maxima_bytes = xa.bytes;
    if (xa.tickets) cudaMemsetAsync(xa.tickets, 0, xa.ticket_units * sizeof(uint32_t), tls().stream);
    xa.epoch = 0;
}

// Enqueues the tcgen05 decode kernel (arguments already validated by launch_attn_decode).
catena_status_t enqueue_attn_decode_tc(const void* q, const void* kc, const void* vc, void* o, uint64_t units, uint32_t G,
                                       uint64_t kv_len, uint64_t kv_cap, uint64_t unit0, uint64_t unit1, int cluster_limit,
                                       uint32_t* err_dev, void* const* peer_o, uint32_t n_peers, const AttnPrefetch* prefetch) {
    attn2::PrefetchHint pf = {};
    if (prefetch) {
        for (uint32_t i = 0; i < prefetch->n && pf.n < (uint32_t)attn2::kMaxPrefetch; ++i) {
            const uint64_t chunks = prefetch->bytes[i] / attn2::kPrefetchChunk;          // whole chunks only: never past the end
            if (!prefetch->ptr[i] || ((uintptr_t)prefetch->ptr[i] & 15) || chunks == 0) continue;
            pf.ptr[pf.n] = static_cast<const uint8_t*>(prefetch->ptr[i]);
            pf.chunks[pf.n] = (uint32_t)(chunks > 0xFFFFFFFFull ? 0xFFFFFFFFull : chunks);
            ++pf.n;
        }
        pf.pace_ns = prefetch->pace_ns;
    }
    if (n_peers > (uint32_t)attn2::kMaxPeers) return fail(CATENA_E_BAD_ARG, "attn_decode: more than 7 peer outputs");
    attn2::PeerO peers = {};
    peers.n = n_peers;
    for (uint32_t i = 0; i < n_peers; ++i) {
        if (!peer_o || !peer_o[i] || ((uintptr_t)peer_o[i] & 1)) return fail(CATENA_E_BAD_ARG, "attn_decode: null or unaligned peer output");
        peers.ptr[i] = static_cast<__nv_bfloat16*>(peer_o[i]);
    }
    const uint32_t chunk = chunk_for2(kv_len);
    const size_t smem = attn2_smem_bytes();
    const int dev = tls().device;
    const uint64_t n_units = unit1 - unit0, items = n_units * attn2::kSplits;
    if (items > 0x7FFFFFFFull) return fail(CATENA_E_TOO_LARGE, "attn_decode: too many chunk items");
    CUtensorMap map_k, map_v;
    CATENA_TRY(make_kv_map2(&map_k, kc, units, kv_len, kv_cap));
    CATENA_TRY(make_kv_map2(&map_v, vc, units, kv_len, kv_cap));

    // resident CTAs (one per SM for a kernel that allocates TMEM), asked once per device
    if (g_attn2_max_ctas[dev] == 0) {
        CATENA_CUDA(cudaFuncSetAttribute(attn2::attn_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        int per_sm = 0, sms = 0;
        CATENA_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn2::attn_decode_tc_kernel, attn2::kThreads, smem));
        CATENA_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, tls().device));
        if (per_sm < 1 || sms < 1) return fail(CATENA_E_CUDA, "attn_decode: the tcgen05 kernel cannot be resident");
        g_attn2_max_ctas[dev] = per_sm * sms;
    }
    // #pipes = 2 * CTAs: all items in one round, or a multiple of 8 pipes (so a unit never straddles two rounds)
    uint64_t max_ctas = (uint64_t)g_attn2_max_ctas[dev];
    if (cluster_limit > 0 && max_ctas > (uint64_t)cluster_limit * 4) max_ctas = (uint64_t)cluster_limit * 4;
    uint64_t ctas = items / attn2::kPipes;                 // items is a multiple of 8
    if (ctas > max_ctas) ctas = max_ctas / 4 * 4;
    if (ctas < 1) return fail(CATENA_E_CUDA, "attn_decode: fewer than 4 resident CTAs");

    // exchange area: maxima [items][8] u64 | denominators [items][8] f32 | partials [items][G][128] f32
    const size_t off_denom = align256(items * 8 * sizeof(uint64_t));
    const size_t off_partial = off_denom + align256(items * 8 * sizeof(float));
    const size_t need = off_partial + align256(items * G * attn2::kD * sizeof(float));
    AttnExchange& xa = g_attn_exchange[dev];
    if (xa.bytes < need || xa.epoch == 0xFFFFFFFFu) {
        if (xa.base) {
            CATENA_CUDA(cudaStreamSynchronize(tls().stream));
            CATENA_CUDA(cudaFree(xa.base));
            xa.base = nullptr;
            xa.bytes = 0;
        }
        const size_t want = need + need / 2;
        CATENA_CUDA(cudaMalloc(&xa.base, want));
        CATENA_CUDA(cudaMemset(xa.base, 0, want));          // epoch 0 never matches a launch
        xa.bytes = want;
        xa.epoch = 0;
        xa.maxima_bytes = want;                             // all zeros: epoch 0 everywhere
    }
    if (off_denom > xa.maxima_bytes) {
        // the maxima of this launch reach into what earlier launches used for denominators and partial outputs: a stale
        // float there could by chance carry this launch's epoch in its upper half, so the new part is cleared first
        CATENA_CUDA(cudaMemsetAsync(static_cast<uint8_t*>(xa.base) + xa.maxima_bytes, 0, off_denom - xa.maxima_bytes, tls().stream));
    }
    xa.maxima_bytes = off_denom;
    if (xa.ticket_units < n_units) {
        if (xa.tickets) {
            CATENA_CUDA(cudaStreamSynchronize(tls().stream));
            CATENA_CUDA(cudaFree(xa.tickets));
            xa.tickets = nullptr;
            xa.ticket_units = 0;
        }
        const size_t want_units = n_units + n_units / 2 + 64;
        CATENA_CUDA(cudaMalloc(&xa.tickets, want_units * sizeof(uint32_t)));
        CATENA_CUDA(cudaMemset(xa.tickets, 0, want_units * sizeof(uint32_t)));
        xa.ticket_units = want_units;
    }
    attn2::Exchange ex;
    uint8_t* xb = static_cast<uint8_t*>(xa.base);
    ex.maxima = reinterpret_cast<uint64_t*>(xb);
    ex.tickets = xa.tickets;
    ex.denom = reinterpret_cast<float*>(xb + off_denom);
    ex.partial = reinterpret_cast<float*>(xb + off_partial);
    ex.epoch = ++xa.epoch;

    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(attn2::kThreads);
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = tls().stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;             // every CTA resident: pipes wait for one another
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    g_attn_last_launch[0] = 1; g_attn_last_launch[1] = (uint32_t)g_attn2_max_ctas[dev];
    g_attn_last_launch[2] = (uint32_t)ctas; g_attn_last_launch[3] = (uint32_t)smem;
    float scale = 1.0f / sqrtf((float)attn2::kD);
    CATENA_CUDA(cudaLaunchKernelEx(&cfg, attn2::attn_decode_tc_kernel, map_k, map_v, (const __nv_bfloat16*)q, (__nv_bfloat16*)o,
                                   (uint32_t)kv_len, G, (uint32_t)unit0, (uint32_t)items, chunk, scale, ex, err_dev,
                                   debug_wait_limit_ns(), debug_take_stall(2), peers, pf));
    count_launch();
    return CATENA_OK;
}

#ifdef CATENA_ATTN_TRACE
// Copies the timeline out (4 roles x 1024 stamps, counts) and clears the counts.
extern "C" void catena_b200_debug_attn_trace(unsigned long long* stamps, unsigned int* counts) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(stamps, attn2::g_trace, sizeof(unsigned long long) * 4 * 1024);
    cudaMemcpyFromSymbol(counts, attn2::g_trace_n, sizeof(unsigned int) * 4);
    unsigned int zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(attn2::g_trace_n, zero, sizeof(zero));
}
#endif

}  // namespace catena
