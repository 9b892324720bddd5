// Device memory of the library goes through a small cache: a block that is released (handle destroyed, inference call
// done) is kept and handed to the next request of about the same size instead of going back to the driver.
// cudaMalloc / cudaFree take driver-wide locks; on a machine whose other GPUs are busy a single cudaFree of a few GB was
// measured anywhere between 5 ms and 2 s, which is a multiple of a whole `fit`.  With the cache a second `fit` (or
// predict call) of the same shape makes no allocator call at all.  Blocks are whole cudaMalloc allocations (never
// sub-allocated), so they stay valid for cudaIpcGetMemHandle.  The cache gives everything back when an allocation fails
// (then it retries once) and on evb_trim_cache(); it never keeps more than half of the device's memory
// (EVB_CACHE_MAX_GB sets another limit); EVB_CACHE=0 turns it off.
#include "evb_internal.cuh"
#include <mutex>
#include <stdlib.h>
#include <unordered_map>
#include <vector>

namespace {

struct Block { void *p; size_t bytes; };
struct DevCache {
    std::mutex mu;
    std::vector<Block> free_blocks;
    std::unordered_map<void *, size_t> live; // blocks handed out by evb_dev_alloc
    size_t cached_bytes = 0;
    size_t cap = 0; // most bytes the cache keeps: half of the device's memory unless EVB_CACHE_MAX_GB says otherwise
};
DevCache g_cache[64];

bool cache_on() {
    static const bool on = [] { const char *e = getenv("EVB_CACHE"); return e ? atoi(e) != 0 : true; }();
    return on;
}

size_t round_size(size_t bytes) {
    if (bytes < 512) return 512;
    if (bytes < ((size_t)1 << 20)) return (bytes + 511) & ~(size_t)511;
    return (bytes + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1); // whole MB: shapes that differ a little share blocks
}

void release_all(DevCache &c) {
    for (const Block &b : c.free_blocks) cudaFree(b.p);
    c.free_blocks.clear();
    c.cached_bytes = 0;
}

} // namespace

// cudaMalloc semantics (the current device); *p is null on failure
cudaError_t evb_dev_alloc(void **p, size_t bytes) {
    *p = nullptr;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const size_t want = round_size(bytes);
    if (!cache_on() || dev < 0 || dev >= 64) return cudaMalloc(p, want);
    DevCache &c = g_cache[dev];
    std::lock_guard<std::mutex> lock(c.mu);
    // best fit among the cached blocks that are not much larger than the request
    size_t best = (size_t)-1;
    const size_t limit = want + want / 8 + ((size_t)1 << 20);
    for (size_t i = 0; i < c.free_blocks.size(); ++i) {
        const size_t b = c.free_blocks[i].bytes;
        if (b >= want && b <= limit && (best == (size_t)-1 || b < c.free_blocks[best].bytes)) best = i;
    }
    if (best != (size_t)-1) {
        const Block b = c.free_blocks[best];
        c.free_blocks[best] = c.free_blocks.back();
        c.free_blocks.pop_back();
        c.cached_bytes -= b.bytes;
        c.live[b.p] = b.bytes;
        *p = b.p;
        return cudaSuccess;
    }
    e = cudaMalloc(p, want);
    if (e != cudaSuccess && !c.free_blocks.empty()) { // out of memory with blocks in the cache: give them back, try again
        cudaGetLastError();
        release_all(c);
        e = cudaMalloc(p, want);
    }
    if (e != cudaSuccess) { *p = nullptr; return e; }
    c.live[*p] = want;
    return cudaSuccess;
}

// `really`: hand the block back to the driver (blocks that other processes may have mapped through CUDA IPC)
void evb_dev_free(void *p, bool really) {
    if (!p) return;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || !cache_on() || dev < 0 || dev >= 64) { cudaFree(p); return; }
    DevCache &c = g_cache[dev];
    std::lock_guard<std::mutex> lock(c.mu);
    auto it = c.live.find(p);
    if (it == c.live.end()) { cudaFree(p); return; } // not one of ours (allocated on another device, or before a fork)
    const size_t bytes = it->second;
    c.live.erase(it);
    if (c.cap == 0) {
        size_t free_b = 0, total_b = 0;
        c.cap = cudaMemGetInfo(&free_b, &total_b) == cudaSuccess ? total_b / 2 : (size_t)16 << 30;
        if (const char *e = getenv("EVB_CACHE_MAX_GB")) { const double gb = atof(e); if (gb >= 0.0) c.cap = (size_t)(gb * 1073741824.0); }
    }
    if (really || c.cached_bytes + bytes > c.cap) { cudaFree(p); return; }
    c.free_blocks.push_back({p, bytes});
    c.cached_bytes += bytes;
}

// ---- the same for what else a handle takes from the driver: pinned host blocks, its stream, its two events ------------
namespace {
struct HostCache {
    std::mutex mu;
    std::vector<Block> free_blocks;
    std::unordered_map<void *, size_t> live;
    std::vector<cudaStream_t> streams[64];
    std::vector<cudaEvent_t> events[64];
};
HostCache g_host;
} // namespace

cudaError_t evb_host_alloc(void **p, size_t bytes) {
    *p = nullptr;
    const size_t want = (bytes + 4095) & ~(size_t)4095;
    if (!cache_on()) return cudaMallocHost(p, want);
    std::lock_guard<std::mutex> lock(g_host.mu);
    for (size_t i = 0; i < g_host.free_blocks.size(); ++i) {
        if (g_host.free_blocks[i].bytes == want) {
            *p = g_host.free_blocks[i].p;
            g_host.free_blocks[i] = g_host.free_blocks.back();
            g_host.free_blocks.pop_back();
            g_host.live[*p] = want;
            return cudaSuccess;
        }
    }
    const cudaError_t e = cudaMallocHost(p, want);
    if (e != cudaSuccess) { *p = nullptr; return e; }
    g_host.live[*p] = want;
    return cudaSuccess;
}
void evb_host_free(void *p) {
    if (!p) return;
    if (!cache_on()) { cudaFreeHost(p); return; }
    std::lock_guard<std::mutex> lock(g_host.mu);
    auto it = g_host.live.find(p);
    if (it == g_host.live.end()) { cudaFreeHost(p); return; }
    const size_t bytes = it->second;
    g_host.live.erase(it);
    if (bytes > ((size_t)64 << 20) || g_host.free_blocks.size() >= 64) { cudaFreeHost(p); return; } // small blocks only: tree and column-sample buffers
    g_host.free_blocks.push_back({p, bytes});
}
// a non-blocking stream / an event without timing of the current device
cudaError_t evb_stream_get(cudaStream_t *st) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (cache_on() && dev >= 0 && dev < 64) {
        std::lock_guard<std::mutex> lock(g_host.mu);
        if (!g_host.streams[dev].empty()) { *st = g_host.streams[dev].back(); g_host.streams[dev].pop_back(); return cudaSuccess; }
    }
    return cudaStreamCreateWithFlags(st, cudaStreamNonBlocking);
}
void evb_stream_put(cudaStream_t st) { // the stream is idle (the caller has synchronised it)
    if (!st) return;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || !cache_on() || dev < 0 || dev >= 64) { cudaStreamDestroy(st); return; }
    std::lock_guard<std::mutex> lock(g_host.mu);
    if (g_host.streams[dev].size() >= 16) { cudaStreamDestroy(st); return; }
    g_host.streams[dev].push_back(st);
}
cudaError_t evb_event_get(cudaEvent_t *ev) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (cache_on() && dev >= 0 && dev < 64) {
        std::lock_guard<std::mutex> lock(g_host.mu);
        if (!g_host.events[dev].empty()) { *ev = g_host.events[dev].back(); g_host.events[dev].pop_back(); return cudaSuccess; }
    }
    return cudaEventCreateWithFlags(ev, cudaEventDisableTiming);
}
void evb_event_put(cudaEvent_t ev) {
    if (!ev) return;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || !cache_on() || dev < 0 || dev >= 64) { cudaEventDestroy(ev); return; }
    std::lock_guard<std::mutex> lock(g_host.mu);
    if (g_host.events[dev].size() >= 64) { cudaEventDestroy(ev); return; }
    g_host.events[dev].push_back(ev);
}

extern "C" int32_t evb_trim_cache(int32_t device) {
    if (device < 0 || device >= 64) { evb_set_error("evb_trim_cache: device %d out of range", device); return EVB_ERR_ARG; }
    int prev = 0;
    EVB_CUDA(cudaGetDevice(&prev));
    EVB_CUDA(cudaSetDevice(device));
    {
        DevCache &c = g_cache[device];
        std::lock_guard<std::mutex> lock(c.mu);
        release_all(c);
    }
    {
        std::lock_guard<std::mutex> lock(g_host.mu);
        for (cudaStream_t st : g_host.streams[device]) cudaStreamDestroy(st);
        for (cudaEvent_t ev : g_host.events[device]) cudaEventDestroy(ev);
        g_host.streams[device].clear();
        g_host.events[device].clear();
        for (const Block &b : g_host.free_blocks) cudaFreeHost(b.p);
        g_host.free_blocks.clear();
    }
    EVB_CUDA(cudaSetDevice(prev));
    return EVB_OK;
}
