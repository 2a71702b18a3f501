// Runtime core of the kernel library: device binding, stream, status, the device-memory pool
// and CUDA-IPC export/import.  Replaces what the reference resolves from libcudart at run time
// (cudaMallocManaged / cudaFree, catena-lang/src/runtime/mem.rs:128-191) and the process-global
// device assumption of the generated code (catena-lang/doc/CODEGEN.md:164-166).
#include <atomic>
#include <map>
#include <mutex>
#include <string.h>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace catena {

static thread_local ThreadState g_tls;
static std::atomic<uint64_t> g_launches{0};

static std::atomic<uint64_t> g_wait_limit_ns{1000000000ull};
static std::atomic<uint32_t> g_stall[3] = {{0}, {0}, {0}};

ThreadState& tls() { return g_tls; }
uint64_t debug_wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }
uint32_t debug_take_stall(int family) {
    if (family < 1 || family > 2) return 0;
    return g_stall[family].exchange(0u, std::memory_order_relaxed);
}
void count_launch(uint64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

catena_status_t fail(catena_status_t s, const char* what) {
    g_tls.last = s;
    fprintf(stderr, "catena_b200: %s: %s\n", catena_b200_status_string(s), what ? what : "");
    fflush(stderr);
    return s;
}

catena_status_t fail_cuda(cudaError_t e, const char* what) {
    g_tls.last = CATENA_E_CUDA;
    fprintf(stderr, "catena_b200: CUDA error %d (%s) in %s\n", (int)e, cudaGetErrorString(e),
            what ? what : "");
    fflush(stderr);
    return CATENA_E_CUDA;
}

static catena_status_t bind_device(int device) {
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count <= 0) {
        (void)cudaGetLastError();
        return fail(CATENA_E_NO_DEVICE, "no CUDA device is visible (this library has no CPU path)");
    }
    if (device < 0 || device >= count) return fail(CATENA_E_BAD_ARG, "device index out of range");
    if (device >= kMaxDevices) return fail(CATENA_E_UNSUPPORTED, "device index beyond the 16 devices the per-device tables hold");
    CATENA_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    CATENA_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(CATENA_E_NO_DEVICE, "kernels are built for sm_100a only (Blackwell B200)");
    g_tls.device = device;
    g_tls.sm_count = prop.multiProcessorCount;
    g_tls.cc_major = prop.major;
    return CATENA_OK;
}

catena_status_t ensure_device() {
    if (g_tls.device >= 0) {
        int cur = -1;
        if (cudaGetDevice(&cur) == cudaSuccess && cur != g_tls.device) cudaSetDevice(g_tls.device);
        return CATENA_OK;
    }
    return bind_device(0);
}

catena_status_t finish(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail_cuda(e, what);
    if (g_tls.blocking) {
        e = cudaStreamSynchronize(g_tls.stream);
        if (e != cudaSuccess) return fail_cuda(e, what);
    }
    return CATENA_OK;
}

// ---- device-memory pool ---------------------------------------------------------------
// Every entry point of the reference allocates its output (materializec.rs:117-122), so the
// allocator sits on the hot path.  Blocks are rounded up to a size class (256 B granules up to
// 1 MiB, then 2 MiB granules), cached per device on free and handed back without touching the
// driver; cudaMalloc/cudaFree only run on a miss or on catena_b200_mem_trim.
//
// Reuse is ordered after the work that may still read or write a freed block.  In blocking mode every
// entry point has synchronised its stream before it returns, so a block is idle when it is freed.  In
// non-blocking mode pool_free records an event on the freeing thread's stream; pool_alloc on the same
// stream needs nothing more (stream order), pool_alloc on another stream makes that stream wait for the
// event first.  The pool is shared by all host threads of a device.
struct FreeBlock {
    void* ptr;
    cudaStream_t stream;   // stream the block was freed on
    cudaEvent_t idle;      // nullptr: nothing was in flight when the block was freed
};
struct Pool {
    std::mutex mu;
    std::multimap<uint64_t, FreeBlock> free_blocks;   // size class -> block
    std::unordered_map<void*, uint64_t> live;         // block -> size class
    std::vector<cudaEvent_t> spare_events;
};
static Pool g_pools[kMaxDevices];

static uint64_t size_class(uint64_t bytes) {
    if (bytes <= (1ull << 20)) return (bytes + 255) & ~255ull;
    return (bytes + (2ull << 20) - 1) & ~((2ull << 20) - 1);
}

catena_status_t pool_alloc(uint64_t bytes, void** out) {
    *out = nullptr;
    if (bytes == 0) return CATENA_OK;
    CATENA_TRY(ensure_device());
    Pool& p = g_pools[g_tls.device];
    uint64_t cls = size_class(bytes);
    {
        std::unique_lock<std::mutex> lk(p.mu);
        auto it = p.free_blocks.find(cls);
        if (it != p.free_blocks.end()) {
            FreeBlock fb = it->second;
            p.free_blocks.erase(it);
            p.live[fb.ptr] = cls;
            lk.unlock();
            if (fb.idle) {
                cudaError_t e = cudaSuccess;
                if (fb.stream != g_tls.stream) e = cudaStreamWaitEvent(g_tls.stream, fb.idle, 0);
                lk.lock();
                p.spare_events.push_back(fb.idle);
                lk.unlock();
                if (e != cudaSuccess) return fail_cuda(e, "cudaStreamWaitEvent (pool reuse)");
            }
            *out = fb.ptr;
            return CATENA_OK;
        }
    }
    void* ptr = nullptr;
    cudaError_t e = cudaMalloc(&ptr, cls);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        catena_b200_mem_trim();
        e = cudaMalloc(&ptr, cls);
        if (e != cudaSuccess) return fail_cuda(e, "cudaMalloc");
    }
    std::lock_guard<std::mutex> lk(p.mu);
    p.live[ptr] = cls;
    *out = ptr;
    return CATENA_OK;
}

catena_status_t pool_free(void* ptr) {
    if (!ptr) return CATENA_OK;
    CATENA_TRY(ensure_device());
    Pool& p = g_pools[g_tls.device];
    uint64_t cls = 0;
    cudaEvent_t ev = nullptr;
    {
        std::lock_guard<std::mutex> lk(p.mu);
        auto it = p.live.find(ptr);
        if (it == p.live.end()) return fail(CATENA_E_BAD_ARG, "mem_free: pointer was not allocated by this library");
        cls = it->second;
        p.live.erase(it);
        if (!g_tls.blocking && !p.spare_events.empty()) {
            ev = p.spare_events.back();
            p.spare_events.pop_back();
        }
    }
    if (!g_tls.blocking) {
        // kernels that use the block may still be queued on this thread's stream
        cudaError_t e = ev ? cudaSuccess : cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventRecord(ev, g_tls.stream);
        if (e != cudaSuccess) {
            // no event: fall back to waiting here, so the block is idle when it goes back on the list
            (void)cudaGetLastError();
            if (ev) cudaEventDestroy(ev);
            ev = nullptr;
            cudaStreamSynchronize(g_tls.stream);
        }
    }
    std::lock_guard<std::mutex> lk(p.mu);
    p.free_blocks.emplace(cls, FreeBlock{ptr, g_tls.stream, ev});
    return CATENA_OK;
}

}  // namespace catena

using namespace catena;

extern "C" {

catena_status_t catena_b200_init(int device) { return bind_device(device); }

int catena_b200_current_device(void) { return tls().device; }

int catena_b200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return n;
}

catena_status_t catena_b200_set_stream(void* stream) {
    // The thread's scratch (attention exchange area, rotary table, error words) is ordered by its stream: work still
    // queued on the old stream must be done before the same scratch is used from the new one.
    if ((cudaStream_t)stream != tls().stream && tls().device >= 0 && !tls().blocking) {
        CATENA_TRY(ensure_device());
        CATENA_CUDA(cudaStreamSynchronize(tls().stream));
    }
    tls().stream = (cudaStream_t)stream;
    return CATENA_OK;
}
void* catena_b200_get_stream(void) { return (void*)tls().stream; }
void catena_b200_set_blocking(int blocking) { tls().blocking = blocking ? 1 : 0; }

catena_status_t catena_b200_sync(void) {
    CATENA_TRY(ensure_device());
    CATENA_CUDA(cudaStreamSynchronize(tls().stream));
    return CATENA_OK;
}

catena_status_t catena_b200_last_status(void) { return tls().last; }
void catena_b200_clear_status(void) { tls().last = CATENA_OK; }

const char* catena_b200_status_string(catena_status_t s) {
    switch (s) {
        case CATENA_OK: return "ok";
        case CATENA_E_ASSERT: return "catena assertion failed";
        case CATENA_E_CUDA: return "CUDA error";
        case CATENA_E_NO_DEVICE: return "no usable CUDA device";
        case CATENA_E_BAD_ARG: return "bad argument";
        case CATENA_E_TIMEOUT: return "device-side wait timed out";
        case CATENA_E_TOO_LARGE: return "size beyond the supported maximum";
        case CATENA_E_UNSUPPORTED: return "unsupported";
        default: return "unknown status";
    }
}

const char* catena_b200_version(void) { return "catena_b200 0.1 (sm_100a)"; }
uint64_t catena_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

void catena_b200_debug_set_wait_limit_ns(uint64_t ns) {
    g_wait_limit_ns.store(ns ? ns : 1000000000ull, std::memory_order_relaxed);
}
void catena_b200_debug_stall_next(int family, uint32_t value) {
    if (family >= 1 && family <= 2) g_stall[family].store(value, std::memory_order_relaxed);
}

catena_status_t catena_b200_mem_alloc(uint64_t bytes, catena_mem_t* out) {
    if (!out) return fail(CATENA_E_BAD_ARG, "mem_alloc: null out");
    out->data = nullptr;
    out->len = 0;
    void* p = nullptr;
    CATENA_TRY(pool_alloc(bytes, &p));
    out->data = p;
    out->len = bytes;
    return CATENA_OK;
}

catena_status_t catena_b200_mem_free(catena_mem_t mem) { return pool_free(mem.data); }

catena_status_t catena_b200_mem_write(catena_mem_t mem, const void* host, uint64_t bytes) {
    if (bytes == 0) return CATENA_OK;
    if (!host || !mem.data || bytes > mem.len) return fail(CATENA_E_BAD_ARG, "mem_write");
    CATENA_TRY(ensure_device());
    CATENA_CUDA(cudaMemcpyAsync(mem.data, host, bytes, cudaMemcpyHostToDevice, tls().stream));
    if (tls().blocking) CATENA_CUDA(cudaStreamSynchronize(tls().stream));
    return CATENA_OK;
}

catena_status_t catena_b200_mem_upload(const void* host, uint64_t bytes, catena_mem_t* out) {
    CATENA_TRY(catena_b200_mem_alloc(bytes, out));
    if (bytes == 0) return CATENA_OK;
    catena_status_t s = catena_b200_mem_write(*out, host, bytes);
    if (s != CATENA_OK) {
        pool_free(out->data);
        out->data = nullptr;
        out->len = 0;
    }
    return s;
}

catena_status_t catena_b200_mem_download(catena_mem_t mem, void* host, uint64_t bytes) {
    if (bytes == 0) return CATENA_OK;
    if (!host || !mem.data || bytes > mem.len) return fail(CATENA_E_BAD_ARG, "mem_download");
    CATENA_TRY(ensure_device());
    CATENA_CUDA(cudaMemcpyAsync(host, mem.data, bytes, cudaMemcpyDeviceToHost, tls().stream));
    CATENA_CUDA(cudaStreamSynchronize(tls().stream));
    return CATENA_OK;
}

catena_status_t catena_b200_mem_trim(void) {
    CATENA_TRY(ensure_device());
    Pool& p = g_pools[tls().device];
    std::vector<FreeBlock> blocks;
    std::vector<cudaEvent_t> events;
    {
        std::lock_guard<std::mutex> lk(p.mu);
        for (auto& kv : p.free_blocks) blocks.push_back(kv.second);
        p.free_blocks.clear();
        events.swap(p.spare_events);
    }
    if (!blocks.empty()) cudaDeviceSynchronize();
    for (FreeBlock& b : blocks) {
        cudaFree(b.ptr);
        if (b.idle) cudaEventDestroy(b.idle);
    }
    for (cudaEvent_t ev : events) cudaEventDestroy(ev);
    return CATENA_OK;
}

catena_status_t catena_b200_ipc_export(catena_mem_t mem, void* handle64, uint64_t* offset) {
    if (!mem.data || !handle64 || !offset) return fail(CATENA_E_BAD_ARG, "ipc_export");
    CATENA_TRY(ensure_device());
    // IPC handles name whole allocations.  Blocks of the pool are whole cudaMalloc allocations,
    // so a `mem` returned by catena_b200_mem_alloc starts at offset 0 of the exported base.
    {
        Pool& p = g_pools[tls().device];
        std::lock_guard<std::mutex> lk(p.mu);
        if (p.live.find(mem.data) == p.live.end())
            return fail(CATENA_E_BAD_ARG, "ipc_export: not the start of an allocation of this library");
    }
    cudaIpcMemHandle_t h;
    CATENA_CUDA(cudaIpcGetMemHandle(&h, mem.data));
    memcpy(handle64, &h, sizeof(h));
    *offset = 0;
    return CATENA_OK;
}

catena_status_t catena_b200_ipc_import(const void* handle64, uint64_t offset, uint64_t bytes,
                                       catena_mem_t* out) {
    if (!handle64 || !out) return fail(CATENA_E_BAD_ARG, "ipc_import");
    CATENA_TRY(ensure_device());
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void* base = nullptr;
    CATENA_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
    out->data = (char*)base + offset;
    out->len = bytes;
    return CATENA_OK;
}

catena_status_t catena_b200_ipc_close(catena_mem_t mem, uint64_t offset) {
    if (!mem.data) return CATENA_OK;
    CATENA_TRY(ensure_device());
    CATENA_CUDA(cudaIpcCloseMemHandle((char*)mem.data - offset));
    return CATENA_OK;
}

}  // extern "C"
