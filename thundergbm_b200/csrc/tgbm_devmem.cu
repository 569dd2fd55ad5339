// Device memory of the library's buffers.
//
// A training call allocates and frees a few dozen buffers of up to several GB.  With cudaMalloc / cudaFree that costs
// 10-30 ms per call on one GPU and several times that when the host threads of an n_device = N call contend for the
// driver (cudaFree also unmaps the memory from every peer NCCL opened).  Released blocks are therefore kept, per
// device, and handed out again to the next request of (nearly) the same size: a call that follows another of the same
// shape allocates nothing.  The blocks are plain cudaMalloc memory, so whatever holds for cudaMalloc'ed buffers (peer
// access between the GPUs of one process, which NCCL relies on) holds for them.  A stream-ordered memory pool
// (cudaMallocFromPoolAsync) opened to the peer GPUs was measured too: with it the set-up of a call on 4 GPUs took
// 400 ms instead of 150 ms, every growth of such a pool being mapped on every peer.
//
// The interface keeps the meaning of cudaMalloc / cudaFree: dev_free waits for the device before the block goes back
// to the cache, so a block is never handed out again while work that was queued before its release still runs.
//
// What the cache holds between calls is bounded: at the end of every entry point of the C ABI (dev_trim) it is cut
// back to TGBM_POOL_KEEP_MB megabytes per device (default 16384; 0 = keep nothing), largest blocks first.
// TGBM_NO_POOL=1 selects plain cudaMalloc / cudaFree.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <iterator>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "tgbm_common.h"
#include "tgbm_device.cuh"

namespace tgbm {
namespace {

constexpr int MAX_DEVICES = 64;
constexpr size_t GRANULE = 512;   // request sizes are rounded up to this

struct DeviceCache {
    std::mutex mutex;
    std::multimap<size_t, void *> free_blocks;       // size -> block
    std::unordered_map<void *, size_t> live;         // blocks handed out -> size
    size_t cached_bytes = 0;
    bool dirty = false;                               // something was released since the last trim
};

// never destroyed: a buffer may be released while the process exits (a binding's finaliser, a static object of the
// host program), after the static destructors of this file would have run
DeviceCache *const g_cache = new DeviceCache[MAX_DEVICES];

bool cache_enabled() {
    static const bool on = getenv("TGBM_NO_POOL") == nullptr;
    return on;
}

size_t keep_bytes() {
    static const size_t keep = [] {
        const char *e = getenv("TGBM_POOL_KEEP_MB");
        const double mb = e ? atof(e) : 16384.0;
        return mb > 0 ? (size_t)(mb * 1048576.0) : (size_t)0;
    }();
    return keep;
}

// a cached block may serve a request when it wastes at most an eighth of it (or 64 KB)
bool fits(size_t block, size_t want) { return block >= want && block - want <= std::max<size_t>(want / 8, 65536); }

// gives cached blocks of device `dev` (the current device) back to the driver until at most `keep` bytes remain
void release_down_to(DeviceCache &c, size_t keep) {
    std::vector<void *> victims;
    {
        std::lock_guard<std::mutex> lock(c.mutex);
        while (c.cached_bytes > keep && !c.free_blocks.empty()) {
            auto it = std::prev(c.free_blocks.end());
            c.cached_bytes -= it->first;
            victims.push_back(it->second);
            c.free_blocks.erase(it);
        }
    }
    for (void *p : victims) cudaFree(p);
}

[[noreturn]] void fail(cudaError_t e, size_t bytes) {
    cudaGetLastError();
    throw Error(std::string("CUDA error: ") + cudaGetErrorString(e) + " allocating " + std::to_string(bytes) + " bytes of device memory");
}

}  // namespace

void *dev_alloc(size_t bytes) {
    if (bytes == 0) return nullptr;
    void *p = nullptr;
    int dev = 0;
    if (!cache_enabled() || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        const cudaError_t e = cudaMalloc(&p, bytes);
        if (e != cudaSuccess) fail(e, bytes);
        return p;
    }
    DeviceCache &c = g_cache[dev];
    const size_t want = (bytes + GRANULE - 1) / GRANULE * GRANULE;
    {
        std::lock_guard<std::mutex> lock(c.mutex);
        auto it = c.free_blocks.lower_bound(want);
        if (it != c.free_blocks.end() && fits(it->first, want)) {
            p = it->second;
            c.live[p] = it->first;
            c.cached_bytes -= it->first;
            c.free_blocks.erase(it);
            return p;
        }
    }
    cudaError_t e = cudaMalloc(&p, want);
    if (e == cudaErrorMemoryAllocation) {   // the cache may hold what is missing
        cudaGetLastError();
        release_down_to(c, 0);
        e = cudaMalloc(&p, want);
    }
    if (e != cudaSuccess) fail(e, bytes);
    std::lock_guard<std::mutex> lock(c.mutex);
    c.live[p] = want;
    return p;
}

void dev_free(void *p) noexcept {
    if (!p) return;
    int owner = -1, cur = 0;
    cudaPointerAttributes attr = {};
    if (cudaPointerGetAttributes(&attr, p) == cudaSuccess) owner = attr.device;
    else cudaGetLastError();
    cudaGetDevice(&cur);
    if (!cache_enabled() || owner < 0 || owner >= MAX_DEVICES) { cudaFree(p); return; }
    DeviceCache &c = g_cache[owner];
    size_t size = 0;
    {
        std::lock_guard<std::mutex> lock(c.mutex);
        auto it = c.live.find(p);
        if (it != c.live.end()) { size = it->second; c.live.erase(it); }
    }
    if (size == 0) { cudaFree(p); return; }              // not one of ours
    if (owner != cur) cudaSetDevice(owner);               // a buffer may be released by another thread than the one that made it
    cudaDeviceSynchronize();                              // cudaFree's promise: nothing queued before the release still uses the block
    if (owner != cur) cudaSetDevice(cur);
    std::lock_guard<std::mutex> lock(c.mutex);
    c.free_blocks.emplace(size, p);
    c.cached_bytes += size;
    c.dirty = true;
}

static void trim_all(size_t keep, bool only_dirty) noexcept {
    if (!cache_enabled()) return;
    int cur = -1;
    for (int dev = 0; dev < MAX_DEVICES; ++dev) {
        DeviceCache &c = g_cache[dev];
        {
            std::lock_guard<std::mutex> lock(c.mutex);
            if ((only_dirty && !c.dirty) || c.cached_bytes <= keep) { c.dirty = false; continue; }
            c.dirty = false;
        }
        if (cur < 0 && cudaGetDevice(&cur) != cudaSuccess) { cudaGetLastError(); return; }
        cudaSetDevice(dev);
        release_down_to(c, keep);
    }
    if (cur >= 0) cudaSetDevice(cur);
}

// ---- large host -> device copies ---------------------------------------------------------------------------------
// cudaMemcpyAsync from pageable memory (what a NumPy caller hands over) is staged by the driver through one small
// pinned buffer: 10.8 GB/s measured for the 2.4 GB of a Higgs-sized CSR, a fifth of what the link carries from pinned
// memory (page-locking the caller's arrays in place with cudaHostRegister runs at 11 GB/s too).  upload_h2d does the staging itself: a few host threads copy 8 MB pieces into page-locked slots (two per
// thread, kept for the next call) and send each slot on with cudaMemcpyAsync on the thread's own stream.  Page-locked
// or registered sources, and small copies, go to cudaMemcpyAsync directly.
namespace {

constexpr size_t STAGE_BYTES = 8u << 20;
constexpr int STAGE_KEEP = 16;   // slots that stay allocated between calls (128 MB)

std::mutex &g_stage_mutex = *new std::mutex;
std::vector<void *> &g_stage_free = *new std::vector<void *>;

void *stage_acquire() {
    {
        std::lock_guard<std::mutex> lock(g_stage_mutex);
        if (!g_stage_free.empty()) { void *p = g_stage_free.back(); g_stage_free.pop_back(); return p; }
    }
    void *p = nullptr;
    if (cudaHostAlloc(&p, STAGE_BYTES, cudaHostAllocPortable) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return p;
}

void stage_release(void *p) {
    if (!p) return;
    {
        std::lock_guard<std::mutex> lock(g_stage_mutex);
        if ((int)g_stage_free.size() < STAGE_KEEP) { g_stage_free.push_back(p); return; }
    }
    cudaFreeHost(p);
}

bool host_is_pageable(const void *p) {
    cudaPointerAttributes attr = {};
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) { cudaGetLastError(); return true; }
    return attr.type == cudaMemoryTypeUnregistered;
}

}  // namespace

int upload_threads() {
    static const int n = [] {
        if (const char *e = getenv("TGBM_UPLOAD_THREADS")) return std::max(1, std::min(STAGE_KEEP / 2, atoi(e)));
        const int hw = (int)std::thread::hardware_concurrency();
        return std::max(1, std::min(8, hw / 2));   // 16 cores: 4 / 6 / 8 threads bring 2.4 GB over in 100 / 82 / 65 ms, 12 and more in 0.2-1.2 s
    }();
    return n;
}

void upload_h2d(void *dst, const void *src, size_t bytes, cudaStream_t stream, int n_threads) {
    if (bytes == 0) return;
    static const bool staged = getenv("TGBM_NO_STAGED_UPLOAD") == nullptr;
    if (!staged || bytes < 4 * STAGE_BYTES || n_threads < 1 || !host_is_pageable(src)) {
        TGBM_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream));
        return;
    }
    int dev = 0;
    TGBM_CUDA(cudaGetDevice(&dev));
    const size_t n_chunks = (bytes + STAGE_BYTES - 1) / STAGE_BYTES;
    const int T = (int)std::min<size_t>((size_t)n_threads, n_chunks);
    std::vector<std::string> errors(T);
    std::vector<std::thread> workers;
    for (int t = 0; t < T; ++t)
        workers.emplace_back([&, t] {
            void *slot[2] = {nullptr, nullptr};
            cudaEvent_t done[2] = {nullptr, nullptr};
            bool busy[2] = {false, false};
            cudaStream_t st = nullptr;
            auto check = [&](cudaError_t e, const char *what) {
                if (e != cudaSuccess) { cudaGetLastError(); throw Error(std::string("CUDA error: ") + cudaGetErrorString(e) + " in " + what); }
            };
            try {
                check(cudaSetDevice(dev), "cudaSetDevice");
                check(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking), "cudaStreamCreate");
                for (int k = 0; k < 2; ++k) {
                    slot[k] = stage_acquire();
                    if (!slot[k]) throw Error("no page-locked memory for the upload");
                    check(cudaEventCreateWithFlags(&done[k], cudaEventDisableTiming), "cudaEventCreate");
                }
                int k = 0;
                for (size_t c = t; c < n_chunks; c += T, k ^= 1) {
                    const size_t off = c * STAGE_BYTES, len = std::min(STAGE_BYTES, bytes - off);
                    if (busy[k]) check(cudaEventSynchronize(done[k]), "cudaEventSynchronize");
                    memcpy(slot[k], static_cast<const char *>(src) + off, len);
                    check(cudaMemcpyAsync(static_cast<char *>(dst) + off, slot[k], len, cudaMemcpyHostToDevice, st), "cudaMemcpyAsync");
                    check(cudaEventRecord(done[k], st), "cudaEventRecord");
                    busy[k] = true;
                }
                check(cudaStreamSynchronize(st), "cudaStreamSynchronize");
            } catch (const std::exception &e) {
                errors[t] = e.what();
                if (st) cudaStreamSynchronize(st);   // nothing may still read the slots when they go back
            }
            for (int k = 0; k < 2; ++k) {
                if (done[k]) cudaEventDestroy(done[k]);
                stage_release(slot[k]);
            }
            if (st) cudaStreamDestroy(st);
        });
    for (auto &w : workers) w.join();
    for (const auto &e : errors)
        if (!e.empty()) throw Error(e);
    (void)stream;   // the pieces are on the device when the workers return: whatever is queued next sees them
}

void dev_trim() noexcept { trim_all(keep_bytes(), true); }
void dev_release_all() noexcept {
    trim_all(0, false);
    std::vector<void *> slots;
    {
        std::lock_guard<std::mutex> lock(g_stage_mutex);
        slots.swap(g_stage_free);
    }
    for (void *p : slots) cudaFreeHost(p);
}

}  // namespace tgbm
