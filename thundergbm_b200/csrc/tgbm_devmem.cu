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
#include <iterator>
#include <map>
#include <mutex>
#include <string>
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

DeviceCache g_cache[MAX_DEVICES];

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

void dev_trim() noexcept { trim_all(keep_bytes(), true); }
void dev_release_all() noexcept { trim_all(0, false); }

}  // namespace tgbm
