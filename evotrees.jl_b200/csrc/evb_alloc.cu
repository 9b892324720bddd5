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
    EVB_CUDA(cudaSetDevice(prev));
    return EVB_OK;
}
