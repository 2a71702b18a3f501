// Tensor-core GEMM for sm_100a: C[M,N] = A[M,K] * B^T with A row-major [M,K] and B stored
// column-major, i.e. as [N,K] with K contiguous (both operands K-major: the natural UMMA case).
//   bf16 x bf16 -> fp32 accumulate in TMEM -> bf16 (round-to-nearest-even) output
//   int8 x int8 -> int32 accumulate in TMEM -> int32 output (exact)
// No counterpart in the reference (it has f32 CUDA-core code only); the rule inherited from its
// matmul (catena-lang/stdlib/matrix.hex:236-256) is a FIXED ascending-k accumulation order per
// output element: k-blocks of 64 (bf16) / 128 (int8) elements are issued to `tcgen05.mma` in
// ascending order into one TMEM accumulator.  There is no split-K, no stream-K and no atomics, and
// neither the tile -> CTA map nor the grid size enters the arithmetic, so results are bitwise
// identical across runs, SM counts and GPU partitionings.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: `cp.async.bulk.tensor.2d` (no multicast) of a 128x128B A box and a
//               256x128B B box per k-block into a 128B-swizzled 4-stage shared-memory ring,
//               completion on mbarriers;
//   warp 1      owns TMEM (512 columns = two 128x256 fp32/int32 accumulators) and issues
//               `tcgen05.mma.cta_group::1` (M=128, N=256, K=16|32) from one thread;
//               `tcgen05.commit` releases ring stages and publishes finished accumulators;
//   warps 2-5   epilogue: `tcgen05.ld` 32 lanes x 32 columns, convert, store; overlaps the next
//               tile's main loop through the second accumulator.
// Every mbarrier wait is bounded (about one second of %globaltimer); on expiry the kernel raises an
// error word that the host turns into CATENA_E_TIMEOUT, lets in-flight copies land, frees TMEM and
// returns — it never traps and never spins forever.
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdlib.h>

#include "common.cuh"

namespace catena {

namespace tc {

constexpr int BM = 128;            // tile rows  (TMEM lanes)
constexpr int BN = 256;            // tile cols  (TMEM columns per accumulator)
constexpr int BK_BYTES = 128;      // k-block width in bytes = one 128B swizzle row
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK_BYTES;              // 16 KiB
constexpr int B_BYTES = BN * BK_BYTES;              // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;      // 48 KiB
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 16;        // rasterisation: tiles walk 16 row-blocks before the next column block
constexpr uint64_t WAIT_NS = 1000000000ull;

struct __align__(8) Control {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    volatile uint32_t abort_flag;
};
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + (int)sizeof(Control);

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
// Bounded wait.  Returns false when the wait expired or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Control* ctl, uint32_t* err,
                                          uint32_t code) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 255u) == 0) {
            if (ctl->abort_flag) return false;
            if (globaltimer_ns() - t0 > WAIT_NS) {
                ctl->abort_flag = 1;
                atomicCAS(err, 0u, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
template <bool IS_I8>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       uint32_t accumulate) {
    if (IS_I8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
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

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 B wide and 128B-swizzled:
// start address >> 4 in [0,14), leading byte offset (unused for swizzled K-major, set to 1) in
// [16,30), stride byte offset = 8 rows * 128 B = 1024 B (>> 4) in [32,46), descriptor version 1 in
// [46,48), layout type 2 (SWIZZLE_128B) in [61,64).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}

// Instruction descriptor (dense, no negate, both operands K-major):
// c_format [4,6): 1 = F32, 2 = S32; a_format [7,10), b_format [10,13): 1 = BF16 (kind::f16) or
// 1 = signed int8 (kind::i8); n_dim = N >> 3 in [17,23); m_dim = M >> 4 in [24,29).
template <bool IS_I8>
__host__ __device__ constexpr uint32_t make_idesc(uint32_t n) {
    return ((IS_I8 ? 2u : 1u) << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void tile_coords(uint32_t t, uint32_t mb, uint32_t nb, uint32_t& m_blk, uint32_t& n_blk) {
    uint32_t per_group = GROUP_M * nb;
    uint32_t g = t / per_group;
    uint32_t first_m = g * GROUP_M;
    uint32_t rows = min((uint32_t)GROUP_M, mb - first_m);
    uint32_t in_g = t - g * per_group;
    m_blk = first_m + in_g % rows;
    n_blk = in_g / rows;
}

// One unit of work: a 128-row tile of `width` columns starting at column `col0`.
struct Work {
    uint32_t m_blk, col0, width;
};

// Static schedule.  Tiles are dealt round-robin to the persistent CTAs; the tiles of the last, partial
// round are cut along N into `split` (1, 2 or 4) narrower units so that (nearly) every SM has work in
// that round too.  An output element's k order does not depend on the width of the unit that owns it,
// so the split changes the timing only, never a bit of the result.
__device__ __forceinline__ bool get_work(uint32_t it, uint32_t mb, uint32_t nb, uint32_t tiles, uint32_t split, Work& w) {
    const uint32_t full = (tiles / gridDim.x) * gridDim.x;
    const uint32_t idx = it * gridDim.x + blockIdx.x;
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
    uint32_t m_blk, n_blk;
    tile_coords(t, mb, nb, m_blk, n_blk);
    w.m_blk = m_blk;
    w.col0 = n_blk * BN + part * width;
    w.width = width;
    return true;
}

template <bool IS_I8>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_b128, const __grid_constant__ CUtensorMap map_b64,
               void* __restrict__ c_out, uint32_t M, uint32_t N, uint32_t K, uint64_t ldc, uint32_t split,
               uint32_t* err) {
    extern __shared__ uint8_t smem_raw[];
    // 128B-swizzled tiles need 1024-byte alignment (descriptor base_offset = 0)
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    Control* ctl = reinterpret_cast<Control*>(smem + STAGES * STAGE_BYTES);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    constexpr uint32_t K_ELEMS = IS_I8 ? BK_BYTES : BK_BYTES / 2;     // elements per k-block
    constexpr uint32_t MMA_PER_BLOCK = BK_BYTES / 32;                 // each MMA consumes 32 B of K
    const uint32_t mb = (M + BM - 1) / BM, nb = (N + BN - 1) / BN;
    const uint32_t tiles = mb * nb;
    const uint32_t kblocks = (K + K_ELEMS - 1) / K_ELEMS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctl->tmem_full[b], 1);
            mbar_init(&ctl->tmem_empty[b], EPI_THREADS);
        }
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer ----------------
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            Work w;
            for (uint32_t it = 0; ok && get_work(it, mb, nb, tiles, split, w); ++it) {
                const CUtensorMap* mapb = w.width == (uint32_t)BN ? &map_b : (w.width == (uint32_t)BN / 2 ? &map_b128 : &map_b64);
                const uint32_t bytes = A_BYTES + w.width * BK_BYTES;
                for (uint32_t kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(&ctl->empty[stage], phase ^ 1u, ctl, err, 1u)) { ok = false; break; }
                    mbar_expect_tx(&ctl->full[stage], bytes);
                    uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
                    tma_load_2d(sa, &map_a, (int)(kb * K_ELEMS), (int)(w.m_blk * BM), &ctl->full[stage]);
                    tma_load_2d(sa + A_BYTES, mapb, (int)(kb * K_ELEMS), (int)w.col0, &ctl->full[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer ----------------
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            Work w;
            for (uint32_t it = 0; ok && get_work(it, mb, nb, tiles, split, w); ++it) {
                const uint32_t idesc = make_idesc<IS_I8>(w.width);
                if (!mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1u, ctl, err, 2u)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (uint32_t kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(&ctl->full[stage], phase, ctl, err, 3u)) { ok = false; break; }
                    tc_fence_after();
                    uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
                    uint64_t da = make_smem_desc(sa);
                    uint64_t db = make_smem_desc(sa + A_BYTES);
#pragma unroll
                    for (uint32_t kk = 0; kk < MMA_PER_BLOCK; ++kk) {
                        // advancing K by 32 B inside the swizzle row = +2 in the (addr >> 4) field
                        tc_mma<IS_I8>(tmem_d, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
                    }
                    tc_commit(&ctl->empty[stage]);   // stage reusable once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc_commit(&ctl->tmem_full[acc]);     // accumulator complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: warps 2..5 ----------------
        const uint32_t quad = warp & 3u;             // TMEM lane quadrant this warp may access
        const uint32_t row_in_tile = quad * 32 + lane;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        Work w;
        for (uint32_t it = 0; ok && get_work(it, mb, nb, tiles, split, w); ++it) {
            // warp-uniform decision: the tcgen05.ld below is .sync.aligned
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(&ctl->tmem_full[acc], acc_phase, ctl, err, 4u));
            if (!ok) break;
            tc_fence_after();
            const uint32_t row = w.m_blk * BM + row_in_tile;
            const uint32_t col0 = w.col0;
            const uint32_t taddr = tmem_base + ((quad * 32u) << 16) + acc * BN;
#pragma unroll 1
            for (uint32_t c = 0; c < w.width; c += 32) {
                uint32_t v[32];
                tmem_ld32(taddr + c, v);
                tmem_ld_wait();
                if (row < M) {
                    const uint32_t col = col0 + c;
                    if (IS_I8) {
                        int32_t* dst = reinterpret_cast<int32_t*>(c_out) + (uint64_t)row * ldc + col;
                        if (col + 32 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                reinterpret_cast<uint4*>(dst)[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                        } else {
                            for (int q = 0; q < 32; ++q)
                                if (col + q < N) dst[q] = (int32_t)v[q];
                        }
                    } else {
                        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(c_out) + (uint64_t)row * ldc + col;
                        if (col + 32 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                uint32_t p[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 2 * e]),
                                                                             __uint_as_float(v[8 * q + 2 * e + 1]));
                                    p[e] = *reinterpret_cast<uint32_t*>(&h);
                                }
                                reinterpret_cast<uint4*>(dst)[q] = make_uint4(p[0], p[1], p[2], p[3]);
                            }
                        } else {
                            for (int q = 0; q < 32; ++q)
                                if (col + q < N) dst[q] = __float2bfloat16_rn(__uint_as_float(v[q]));
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&ctl->tmem_empty[acc]);
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
    }

    // ---------------- teardown ----------------
    __syncwarp();
    if (ctl->abort_flag) {
        // error path: give copies and MMAs in flight time to land before shared memory and TMEM go away
        uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

}  // namespace tc

// ---- host side ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// 2-D K-major operand [rows, k_elems]: box = 128 B of K x `box_rows` rows, 128B swizzle, OOB -> 0.
static catena_status_t make_operand_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t k_elems,
                                        int elem_bytes, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(CATENA_E_CUDA, "cuTensorMapEncodeTiled is unavailable");
    cuuint64_t dims[2] = {k_elems, rows};
    cuuint64_t strides[1] = {k_elems * (uint64_t)elem_bytes};
    cuuint32_t box[2] = {(cuuint32_t)(tc::BK_BYTES / elem_bytes), box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                    const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(CATENA_E_CUDA, "cuTensorMapEncodeTiled failed");
    return CATENA_OK;
}

// Test hook: caps the number of persistent CTAs so tests can show that the grid size does not
// enter the arithmetic (0 = one CTA per SM).
static int g_cta_limit = 0;
void gemm_tc_set_cta_limit(int limit) { g_cta_limit = limit > 0 ? limit : 0; }

// Kernel selection.  The CTA-pair kernel (gemm_tc2.cu) is the default; the single-CTA kernel serves
// products of at most 128 rows (half of a pair tile would be idle) and stays selectable — environment
// variable CATENA_B200_GEMM_PAIR=0 (read once) or the test hook below — because the two independent
// implementations must agree bit for bit, which the tests check.
static int g_pair_mode = -1;
static bool gemm_pair_mode(uint64_t m) {
    if (g_pair_mode < 0) {
        const char* e = getenv("CATENA_B200_GEMM_PAIR");
        g_pair_mode = (e && e[0] == '0') ? 0 : 1;
    }
    return g_pair_mode == 1 && m > 128;
}
void gemm_tc_set_pair_mode(int on) { g_pair_mode = on ? 1 : 0; }
catena_status_t enqueue_gemm_tc2(const void* a, const void* b, void* c, uint64_t m, uint64_t n, uint64_t k, uint64_t ldc,
                                 int is_i8, int cta_limit, uint32_t* err_dev, void* const* peer_c, uint32_t n_peers, const void* residual,
                                 const GemmRopeOut* rope, int swiglu);

struct ErrWord {
    uint32_t* dev = nullptr;
    uint32_t* host = nullptr;  // pinned
};
static thread_local ErrWord g_err[16];

static catena_status_t err_word(ErrWord** out) {
    ErrWord& e = g_err[tls().device];
    if (!e.dev) {
        CATENA_CUDA(cudaMalloc(&e.dev, sizeof(uint32_t)));
        CATENA_CUDA(cudaMemset(e.dev, 0, sizeof(uint32_t)));
        CATENA_CUDA(cudaMallocHost(&e.host, sizeof(uint32_t)));
        *e.host = 0;
    }
    *out = &e;
    return CATENA_OK;
}

static catena_status_t launch_gemm_tc_any(const void* a, const void* b, void* c, uint64_t m, uint64_t n, uint64_t k, uint64_t ldc,
                                          int is_i8, void* const* peer_c, uint32_t n_peers, const void* residual,
                                          const GemmRopeOut* rope = nullptr, int swiglu = 0);
catena_status_t launch_gemm_tc(const void* a, const void* b, void* c, uint64_t m, uint64_t n, uint64_t k,
                               uint64_t ldc, int is_i8) {
    return launch_gemm_tc_any(a, b, c, m, n, k, ldc, is_i8, nullptr, 0, nullptr);
}
// true when launch_gemm_tc_residual can take this shape (the CTA-pair kernel does the sum in its epilogue)
bool gemm_tc_fuses_residual(uint64_t m) { return gemm_pair_mode(m); }
// bf16 C = round(round(A B^T) + residual): `residual` is bf16 [m, ldc] and may be C itself
catena_status_t launch_gemm_tc_residual(const void* a, const void* b, void* c, uint64_t m, uint64_t n, uint64_t k, uint64_t ldc,
                                        const void* residual) {
    if (!residual || !gemm_pair_mode(m)) return fail(CATENA_E_UNSUPPORTED, "gemm: residual epilogue needs the CTA-pair kernel");
    return launch_gemm_tc_any(a, b, c, m, n, k, ldc, 0, nullptr, 0, residual);
}
// act [m, ffn] = silu(round(x w_gate^T)) * round(x w_up^T) with w = [2 ffn, k] (gate rows, then up rows), the activation in the
// GEMM's epilogue (CTA-pair kernel only, ffn a multiple of 128)
catena_status_t launch_gemm_tc_swiglu(const void* x, const void* w, void* act, uint64_t m, uint64_t ffn, uint64_t k) {
    if (!gemm_pair_mode(m) || ffn % 128) return fail(CATENA_E_UNSUPPORTED, "gemm: SwiGLU epilogue needs the CTA-pair kernel and ffn % 128 == 0");
    return launch_gemm_tc_any(x, w, act, m, 2 * ffn, k, ffn, 0, nullptr, 0, nullptr, nullptr, 1);
}
// bf16 q/k/v projection whose epilogue rotates and scatters into the query buffer and the KV caches (CTA-pair kernel only)
catena_status_t launch_gemm_tc_rope(const void* a, const void* b, uint64_t m, uint64_t n, uint64_t k, const GemmRopeOut& rope) {
    if (!gemm_pair_mode(m)) return fail(CATENA_E_UNSUPPORTED, "gemm: rotary epilogue needs the CTA-pair kernel");
    return launch_gemm_tc_any(a, b, rope.q_out, m, n, k, n, 0, nullptr, 0, nullptr, &rope);
}

// The same GEMM whose epilogue also stores every output tile to `n_peers` peer-mapped copies of C (pair kernel only).
catena_status_t launch_gemm_tc_peers(const void* a, const void* b, void* c, uint64_t m, uint64_t n, uint64_t k, uint64_t ldc,
                                     int is_i8, void* const* peer_c, uint32_t n_peers) {
    return launch_gemm_tc_any(a, b, c, m, n, k, ldc, is_i8, peer_c, n_peers, nullptr);
}
static catena_status_t launch_gemm_tc_any(const void* a, const void* b, void* c, uint64_t m, uint64_t n, uint64_t k, uint64_t ldc,
                                          int is_i8, void* const* peer_c, uint32_t n_peers, const void* residual,
                                          const GemmRopeOut* rope, int swiglu) {
    CATENA_TRY(ensure_device());
    if (m == 0 || n == 0) return CATENA_OK;
    if (!a || !b || !c) return fail(CATENA_E_BAD_ARG, "gemm: null operand");
    const int eb = is_i8 ? 1 : 2;
    if (k == 0 || (k * eb) % 16 != 0)
        return fail(CATENA_E_BAD_ARG, "gemm: K must be a positive multiple of 16 bytes (TMA row pitch)");
    if (((uintptr_t)a & 15) || ((uintptr_t)b & 15)) return fail(CATENA_E_BAD_ARG, "gemm: operands must be 16-byte aligned");
    if (m > 0x7FFFFF00ull || n > 0x7FFFFF00ull || k > 0x7FFFFF00ull) return fail(CATENA_E_TOO_LARGE, "gemm: dimension too large");
    if (ldc < (swiglu ? n / 2 : n)) return fail(CATENA_E_BAD_ARG, "gemm: ldc < n");

    ErrWord* ew = nullptr;
    CATENA_TRY(err_word(&ew));
    cudaStream_t st = tls().stream;
    if (n_peers > 0 && !gemm_pair_mode(m))
        return fail(CATENA_E_UNSUPPORTED, "gemm: peer outputs need the CTA-pair kernel (more than 128 rows)");
    if (gemm_pair_mode(m)) {
        CATENA_TRY(enqueue_gemm_tc2(a, b, c, m, n, k, ldc, is_i8, g_cta_limit, ew->dev, peer_c, n_peers, residual, rope, swiglu));
    } else {
        CUtensorMap map_a, map_b, map_b128, map_b64;
        CATENA_TRY(make_operand_map(&map_a, a, m, k, eb, tc::BM));
        CATENA_TRY(make_operand_map(&map_b, b, n, k, eb, tc::BN));
        CATENA_TRY(make_operand_map(&map_b128, b, n, k, eb, tc::BN / 2));
        CATENA_TRY(make_operand_map(&map_b64, b, n, k, eb, tc::BN / 4));
        if (is_i8)
            CATENA_CUDA(cudaFuncSetAttribute(tc::gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES));
        else
            CATENA_CUDA(cudaFuncSetAttribute(tc::gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES));
        uint64_t tiles = ceil_div_u64(m, tc::BM) * ceil_div_u64(n, tc::BN);
        int sms = tls().sm_count > 0 ? tls().sm_count : 148;
        unsigned grid = (unsigned)(tiles < (uint64_t)sms ? tiles : (uint64_t)sms);
        if (g_cta_limit > 0 && grid > (unsigned)g_cta_limit) grid = (unsigned)g_cta_limit;
        // tiles of the last partial round are cut along N so that round keeps (nearly) all CTAs busy
        const uint64_t rem = tiles % grid;
        const uint32_t split = rem == 0 ? 1u : (rem * 4 <= grid ? 4u : (rem * 2 <= grid ? 2u : 1u));
        if (is_i8)
            tc::gemm_tc_kernel<true><<<grid, tc::NUM_THREADS, tc::SMEM_BYTES, st>>>(map_a, map_b, map_b128, map_b64, c, (uint32_t)m,
                                                                                   (uint32_t)n, (uint32_t)k, ldc, split, ew->dev);
        else
            tc::gemm_tc_kernel<false><<<grid, tc::NUM_THREADS, tc::SMEM_BYTES, st>>>(map_a, map_b, map_b128, map_b64, c, (uint32_t)m,
                                                                                    (uint32_t)n, (uint32_t)k, ldc, split, ew->dev);
        count_launch();
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return fail_cuda(e, "gemm_tc launch");
    }
    if (tls().blocking) {
        CATENA_CUDA(cudaMemcpyAsync(ew->host, ew->dev, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
        CATENA_CUDA(cudaStreamSynchronize(st));
        if (*ew->host != 0) {
            uint32_t code = *ew->host;
            *ew->host = 0;
            cudaMemsetAsync(ew->dev, 0, sizeof(uint32_t), st);
            char msg[96];
            snprintf(msg, sizeof msg, "gemm_tc: bounded wait expired (role code %u)", code);
            return fail(CATENA_E_TIMEOUT, msg);
        }
    }
    return CATENA_OK;
}

// Reads (and clears) the device error word after asynchronous launches.
catena_status_t gemm_tc_check_errors() {
    CATENA_TRY(ensure_device());
    ErrWord* ew = nullptr;
    CATENA_TRY(err_word(&ew));
    cudaStream_t st = tls().stream;
    CATENA_CUDA(cudaMemcpyAsync(ew->host, ew->dev, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    CATENA_CUDA(cudaStreamSynchronize(st));
    if (*ew->host != 0) {
        *ew->host = 0;
        cudaMemsetAsync(ew->dev, 0, sizeof(uint32_t), st);
        return fail(CATENA_E_TIMEOUT, "gemm_tc: bounded wait expired");
    }
    return CATENA_OK;
}

}  // namespace catena
