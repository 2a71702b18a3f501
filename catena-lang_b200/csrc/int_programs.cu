// Integer programs over `mem` buffers of u64: the reference's `reducec` examples and its buffer-head program, which
// its tests run through Runtime::exec on managed memory with the fold on the HOST
// (catena-lang/tests/cases/reducec/basic.hex: `sum-u64` :27-58, `dot-u64` :60-122; catena-lang/tests/runtime.rs:713-740
// `array-head-u64`; catena-lang/smoketest/src/array_head.cpp:37-43 calls `program_array_head_u64` directly).
//
// Here the buffers are device memory, so the folds are kernels.  u64 addition and multiplication are arithmetic modulo
// 2^64 (C unsigned wraparound, catena-lang/src/codegen/gpu.rs:383-389): the sum is associative and commutative, so a
// tree in any order gives the bits of the reference's sequential left fold, for every length.
#include "common.cuh"

namespace catena {

namespace {

constexpr int kThreads = 256;
constexpr int kPerThread = 8;      // u64 values per thread the grid is sized for (16-byte loads, grid-stride beyond 8 CTAs per SM)

__device__ __forceinline__ uint64_t block_sum(uint64_t v, uint64_t* smem) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    uint64_t t = 0;
    if (threadIdx.x < 32) {
        t = threadIdx.x < kThreads / 32 ? smem[threadIdx.x] : 0;
#pragma unroll
        for (int off = 4; off >= 1; off >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, off);
    }
    return t;      // valid in thread 0
}

// One launch folds the whole buffer: every CTA adds the sum of its grid-stride share of x[i] (* y[i] when DOT) to work[0]
// with one 64-bit atomic (addition modulo 2^64 is associative and commutative: any order gives the same bits), then takes a
// ticket from work[1]; the CTA that draws the last ticket reads the total, writes it to `result` — a word of pinned host
// memory, so that no copy follows the kernel — and puts both words back to zero for the next call.
template <bool DOT>
__global__ void __launch_bounds__(kThreads) fold_u64_kernel(const uint64_t* __restrict__ x, const uint64_t* __restrict__ y, uint64_t n,
                                                            unsigned long long* work, unsigned long long* result) {
    __shared__ uint64_t smem[kThreads / 32];
    uint64_t acc = 0;
    const uint64_t stride = (uint64_t)gridDim.x * kThreads * 2;
    const bool vec = ((reinterpret_cast<uintptr_t>(x) | (DOT ? reinterpret_cast<uintptr_t>(y) : 0)) & 15) == 0;
    uint64_t i = ((uint64_t)blockIdx.x * kThreads + threadIdx.x) * 2;
    if (vec) {
        for (; i + 1 < n; i += stride) {
            const ulonglong2 a = *reinterpret_cast<const ulonglong2*>(x + i);
            if (DOT) {
                const ulonglong2 b = *reinterpret_cast<const ulonglong2*>(y + i);
                acc += a.x * b.x + a.y * b.y;
            } else {
                acc += a.x + a.y;
            }
        }
        if (i < n) acc += DOT ? x[i] * y[i] : x[i];              // odd tail element
    } else {
        for (; i < n; i += stride) {
            acc += DOT ? x[i] * y[i] : x[i];
            if (i + 1 < n) acc += DOT ? x[i + 1] * y[i + 1] : x[i + 1];
        }
    }
    const uint64_t t = block_sum(acc, smem);
    if (threadIdx.x == 0) {
        atomicAdd(&work[0], (unsigned long long)t);
        __threadfence();                                          // the sum is visible before the ticket is
        if (atomicAdd(&work[1], 1ull) == (unsigned long long)gridDim.x - 1) {
            __threadfence();
            *result = atomicExch(&work[0], 0ull);                 // every CTA's sum is in: read the total and clear it
            work[1] = 0;
        }
    }
}

// Per host thread and device: the two device words of the kernel above (zero between calls) and the pinned host word
// the last CTA writes the total to.
struct FoldState {
    unsigned long long* work = nullptr;
    unsigned long long* result = nullptr;      // cudaHostAlloc: the same address on host and device
};
static thread_local FoldState g_fold_state[kMaxDevices];

static catena_status_t fold_state(FoldState** out) {
    FoldState& st = g_fold_state[tls().device];
    if (!st.work) {
        CATENA_CUDA(cudaMalloc(&st.work, 2 * sizeof(unsigned long long)));
        CATENA_CUDA(cudaMemset(st.work, 0, 2 * sizeof(unsigned long long)));
        CATENA_CUDA(cudaHostAlloc(&st.result, sizeof(unsigned long long), cudaHostAllocPortable | cudaHostAllocMapped));
        *st.result = 0;
    }
    *out = &st;
    return CATENA_OK;
}

catena_status_t fold_u64(const uint64_t* x, const uint64_t* y, uint64_t n, uint64_t* host_out) {
    if (!host_out) return fail(CATENA_E_BAD_ARG, "u64 fold: null output pointer");
    *host_out = 0;
    CATENA_TRY(ensure_device());
    if (n == 0) return CATENA_OK;                      // the fold's zero element, const.u64.0x0 (basic.hex:43, :107)
    const int sms = tls().sm_count > 0 ? tls().sm_count : 148;
    uint64_t blocks = ceil_div_u64(n, (uint64_t)kThreads * kPerThread);
    if (blocks > (uint64_t)sms * 8) blocks = (uint64_t)sms * 8;            // grid: at most 8 CTAs per SM, grid-stride beyond
    FoldState* fs = nullptr;
    CATENA_TRY(fold_state(&fs));
    cudaStream_t st = tls().stream;
    if (y) fold_u64_kernel<true><<<(unsigned)blocks, kThreads, 0, st>>>(x, y, n, fs->work, fs->result);
    else fold_u64_kernel<false><<<(unsigned)blocks, kThreads, 0, st>>>(x, nullptr, n, fs->work, fs->result);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        // a launch that did not complete may have left the words half way: clear them before the next call
        (void)cudaMemset(fs->work, 0, 2 * sizeof(unsigned long long));
        return fail_cuda(e, "u64 fold");
    }
    *host_out = *fs->result;
    return CATENA_OK;
}

inline catena_status_t check_u64_mem(catena_mem_t m, const char* what) {
    if (m.len != 0 && !m.data) return fail(CATENA_E_BAD_ARG, what);
    if ((uintptr_t)m.data & 7) return fail(CATENA_E_BAD_ARG, what);
    return CATENA_OK;
}

}  // namespace
}  // namespace catena

using namespace catena;

extern "C" {

// sum-u64 (basic.hex:27-58): mem.cast.u64 gives len = bytes / 8 (gpu.rs:752-766), then the fold of the elements
catena_status_t program_sum_u64_s(catena_mem_t in, uint64_t* out) {
    CATENA_TRY(check_u64_mem(in, "sum-u64: null or misaligned buffer"));
    return fold_u64(static_cast<const uint64_t*>(in.data), nullptr, in.len / sizeof(uint64_t), out);
}
void program_sum_u64(catena_mem_t in, uint64_t* out) { (void)program_sum_u64_s(in, out); }

// dot-u64 (basic.hex:60-122): both buffers cast, their lengths asserted equal (`mem.cast.u64.same-length`), then the
// fold of the element products
catena_status_t program_dot_u64_s(catena_mem_t lhs, catena_mem_t rhs, uint64_t* out) {
    if (out) *out = 0;
    CATENA_TRY(check_u64_mem(lhs, "dot-u64: null or misaligned buffer"));
    CATENA_TRY(check_u64_mem(rhs, "dot-u64: null or misaligned buffer"));
    if (lhs.len / sizeof(uint64_t) != rhs.len / sizeof(uint64_t)) return fail(CATENA_E_ASSERT, "dot-u64: the buffers differ in length");
    return fold_u64(static_cast<const uint64_t*>(lhs.data), static_cast<const uint64_t*>(rhs.data), lhs.len / sizeof(uint64_t), out);
}
void program_dot_u64(catena_mem_t lhs, catena_mem_t rhs, uint64_t* out) { (void)program_dot_u64_s(lhs, rhs, out); }

// array-head-u64 (tests/runtime.rs:713-726): mem.cast.u64, `u64.assert-nz` on the length, element 0
catena_status_t program_array_head_u64_s(catena_mem_t in, uint64_t* out) {
    if (!out) return fail(CATENA_E_BAD_ARG, "array-head-u64: null output pointer");
    *out = 0;
    CATENA_TRY(check_u64_mem(in, "array-head-u64: null or misaligned buffer"));
    if (in.len / sizeof(uint64_t) == 0) return fail(CATENA_E_ASSERT, "array-head-u64: empty buffer (u64.assert-nz)");
    CATENA_TRY(ensure_device());
    CATENA_CUDA(cudaMemcpyAsync(out, in.data, sizeof(uint64_t), cudaMemcpyDeviceToHost, tls().stream));
    CATENA_CUDA(cudaStreamSynchronize(tls().stream));
    return CATENA_OK;
}
void program_array_head_u64(catena_mem_t in, uint64_t* out) { (void)program_array_head_u64_s(in, out); }

}  // extern "C"
