// Host-to-device copies of ordinary (pageable) host memory at pinned-memory speed: the data goes through a small ring
// of pinned buffers that several host threads fill while the copy engine drains the previous one.  A plain
// cudaMemcpy from pageable memory does the same staging inside the driver with one thread, which caps a 4 GB feature
// matrix at a fraction of the PCIe rate.  The ring and the worker threads are created on first use and kept for the
// life of the process.
#include "evb_internal.cuh"
#include <condition_variable>
#include <mutex>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <thread>
#if defined(__x86_64__)
#include <emmintrin.h>
#endif
#include <stdint.h>

namespace {

constexpr int STAGE_NB = 3;
constexpr size_t STAGE_BYTES = (size_t)64 << 20;

struct StageRing {
    void *buf[STAGE_NB] = {nullptr, nullptr, nullptr};
    cudaEvent_t ev[STAGE_NB] = {nullptr, nullptr, nullptr};
    bool used[STAGE_NB] = {false, false, false};
    int next = 0;
    bool ready = false;
    std::mutex mu;
};
StageRing g_rings[64]; // one ring per device (events belong to a device)

int stage_threads() {
    static const int n = [] {
        if (const char *e = getenv("EVB_STAGE_THREADS")) { const int v = atoi(e); if (v >= 1 && v <= 64) return v; }
        const unsigned hc = std::thread::hardware_concurrency();
        int v = hc ? (int)hc * 3 / 4 : 4;
        return v < 1 ? 1 : v > 12 ? 12 : v;
    }();
    return n;
}

// Copy into the pinned ring with streaming stores: the destination is read next by the copy engine, not by this core,
// so it should not be pulled into the cache first (a plain memcpy reads every destination line before writing it,
// and the host's memory bandwidth is what limits the whole upload).
#if defined(__x86_64__)
void stream_copy(char *dst, const char *src, size_t n) {
    size_t head = (16 - ((uintptr_t)dst & 15)) & 15;
    if (head > n) head = n;
    if (head) { memcpy(dst, src, head); dst += head; src += head; n -= head; }
    const size_t blocks = n / 64;
    for (size_t i = 0; i < blocks; ++i) {
        const __m128i a = _mm_loadu_si128((const __m128i *)(src) + 0), b = _mm_loadu_si128((const __m128i *)(src) + 1);
        const __m128i c = _mm_loadu_si128((const __m128i *)(src) + 2), d = _mm_loadu_si128((const __m128i *)(src) + 3);
        _mm_stream_si128((__m128i *)(dst) + 0, a); _mm_stream_si128((__m128i *)(dst) + 1, b);
        _mm_stream_si128((__m128i *)(dst) + 2, c); _mm_stream_si128((__m128i *)(dst) + 3, d);
        src += 64; dst += 64;
    }
    _mm_sfence();
    if (n & 63) memcpy(dst, src, n & 63);
}
#else
void stream_copy(char *dst, const char *src, size_t n) { memcpy(dst, src, n); }
#endif

// copies bytes [off, off + len) of the packed sequence (nseg segments of seg_bytes, segment k starting at src + k * stride)
void gather_copy(char *dst, const char *src, size_t seg_bytes, size_t stride, size_t off, size_t len) {
    size_t p = off;
    const size_t end = off + len;
    while (p < end) {
        const size_t seg = p / seg_bytes, within = p - seg * seg_bytes;
        const size_t n = seg_bytes - within < end - p ? seg_bytes - within : end - p;
        stream_copy(dst + (p - off), src + seg * stride + within, n);
        p += n;
    }
}

// Worker threads that live as long as the process: a chunk is cut into one slice per worker.  (Starting threads for
// every 32 MB chunk cost about as much as copying it.)  The pool is never destroyed: its threads may still be
// waiting when the process exits.
struct GatherPool {
    std::mutex m;
    std::condition_variable cv_go, cv_done;
    unsigned long long gen = 0;
    int nworkers = 0, pending = 0;
    char *dst = nullptr;
    const char *src = nullptr;
    size_t seg_bytes = 0, stride = 0, off = 0, bytes = 0, per = 0;
    void worker(int id) {
        unsigned long long seen = 0;
        for (;;) {
            std::unique_lock<std::mutex> lk(m);
            cv_go.wait(lk, [&] { return gen != seen; });
            seen = gen;
            char *d = dst; const char *s = src;
            const size_t sb = seg_bytes, st = stride, o0 = off, total = bytes, slice = per;
            lk.unlock();
            const size_t o = (size_t)id * slice;
            if (o < total) gather_copy(d + o, s, sb, st, o0 + o, total - o < slice ? total - o : slice);
            lk.lock();
            if (--pending == 0) cv_done.notify_one();
        }
    }
    void run(char *d, const char *s, size_t sb, size_t st, size_t o0, size_t total) {
        std::unique_lock<std::mutex> lk(m);
        if (nworkers == 0) {
            nworkers = stage_threads();
            for (int t = 0; t < nworkers; ++t) std::thread([this, t] { worker(t); }).detach();
        }
        dst = d; src = s; seg_bytes = sb; stride = st; off = o0; bytes = total;
        per = ((total + nworkers - 1) / nworkers + 4095) & ~(size_t)4095;
        pending = nworkers;
        ++gen;
        cv_go.notify_all();
        cv_done.wait(lk, [&] { return pending == 0; });
    }
};
GatherPool *g_pool = new GatherPool; // callers hold their ring's lock; rings of different devices share the pool through its own lock
// a forked child has none of the parent's threads: it starts with a pool of its own
const int g_atfork = pthread_atfork(nullptr, nullptr, [] { g_pool = new GatherPool; });

void parallel_gather(char *dst, const char *src, size_t seg_bytes, size_t stride, size_t off, size_t bytes) {
    if (bytes < ((size_t)4 << 20) || stage_threads() == 1) { gather_copy(dst, src, seg_bytes, stride, off, bytes); return; }
    static std::mutex one_job; // one chunk at a time through the pool
    std::lock_guard<std::mutex> g(one_job);
    g_pool->run(dst, src, seg_bytes, stride, off, bytes);
}

} // namespace

// Copies nseg segments of seg_bytes (segment k at src_host + k * stride) of pageable host memory to the device, packed
// back to back at dst_dev, on stream `st`: a block of rows of a column-major matrix, or (nseg = 1) a plain range.
// Returns when the host memory has been read (the caller may reuse or free it); with `drain` also the copies have
// completed.  Without it the last chunks may still be on their way from the pinned ring (in stream order on `st`), and a
// later call continues with the next ring buffer: a sequence of calls then streams without a gap.  One copy at a time
// per device (the ring is shared); concurrent callers wait for each other.
int32_t evb_h2d_staged_strided(void *dst_dev, const void *src_host, size_t seg_bytes, size_t nseg, size_t stride, cudaStream_t st, bool drain) {
    const size_t bytes = seg_bytes * nseg;
    if (bytes == 0) return EVB_OK;
    int dev = 0;
    EVB_CUDA(cudaGetDevice(&dev));
    if (bytes < ((size_t)1 << 20) || getenv("EVB_STAGE_OFF") || dev < 0 || dev >= 64) { // small: the driver's own staging is as good
        if (nseg == 1) EVB_CUDA(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, st));
        else EVB_CUDA(cudaMemcpy2DAsync(dst_dev, seg_bytes, src_host, stride, seg_bytes, nseg, cudaMemcpyHostToDevice, st));
        return EVB_OK;
    }
    StageRing &g_ring = g_rings[dev];
    std::lock_guard<std::mutex> lock(g_ring.mu);
    if (!g_ring.ready) {
        for (int b = 0; b < STAGE_NB; ++b) {
            EVB_CUDA(cudaHostAlloc(&g_ring.buf[b], STAGE_BYTES, cudaHostAllocDefault));
            EVB_CUDA(cudaEventCreateWithFlags(&g_ring.ev[b], cudaEventDisableTiming));
        }
        g_ring.ready = true;
    }
    const char *src = static_cast<const char *>(src_host);
    char *dst = static_cast<char *>(dst_dev);
    for (size_t off = 0; off < bytes; off += STAGE_BYTES) {
        const int b = g_ring.next;
        g_ring.next = (b + 1) % STAGE_NB;
        const size_t len = bytes - off < STAGE_BYTES ? bytes - off : STAGE_BYTES;
        if (g_ring.used[b]) EVB_CUDA(cudaEventSynchronize(g_ring.ev[b])); // the copy that last used this buffer has left it
        parallel_gather(static_cast<char *>(g_ring.buf[b]), src, seg_bytes, stride, off, len);
        EVB_CUDA(cudaMemcpyAsync(dst + off, g_ring.buf[b], len, cudaMemcpyHostToDevice, st));
        EVB_CUDA(cudaEventRecord(g_ring.ev[b], st));
        g_ring.used[b] = true;
    }
    if (drain)
        for (int q = 0; q < STAGE_NB; ++q)
            if (g_ring.used[q]) { EVB_CUDA(cudaEventSynchronize(g_ring.ev[q])); g_ring.used[q] = false; }
    return EVB_OK;
}

int32_t evb_h2d_staged(void *dst_dev, const void *src_host, size_t bytes, cudaStream_t st, bool drain) {
    return evb_h2d_staged_strided(dst_dev, src_host, bytes, 1, bytes, st, drain);
}
