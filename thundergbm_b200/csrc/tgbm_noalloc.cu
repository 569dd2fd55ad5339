// tgbm_metric_score_noalloc: the training metric on device-resident scores without any allocation.
//
// Who needs this.  Some hosts of this library may not ask the CUDA runtime for memory while they run: a serving
// or training process whose own pool has already claimed the whole device (a cudaMalloc there fails, or succeeds
// only by fragmenting what the pool manages), and a monitoring hook called between the steps of somebody else's
// step loop, where the implicit device-wide synchronisation of cudaMalloc / cudaFree would stall work queued on other
// streams.  tgbm_metric_score allocates device copies of its inputs plus the scratch of its two-stage
// reduction on every call, so such callers cannot use it.
//
// What is different here.  Inputs and the one-float result are device pointers owned by the caller.  The only
// scratch the reduction needs -- one partial sum per thread block and the grand total -- lives in a fixed array in
// device memory that is part of the loaded library image: every GPU that loads the library carries those 8.2 KB
// until the process exits, whether or not this function is ever called.  No cudaMalloc, cudaFree or allocating
// library routine is called.
//
// Limits and rules.
//  * At most TGBM_NOALLOC_MAX_ROWS rows (2^30) and TGBM_NOALLOC_MAX_CLASSES score columns; more is refused with a
//    message in tgbm_last_error().  The ranking objectives are refused (their metric needs per-query sort buffers).
//  * The first call on each device looks the scratch array's device address up (cudaGetSymbolAddress).  The name of
//    the array in host code is only a handle, not an address the GPU can use, so that lookup is mandatory; its result
//    is cached per device.  Make this first call outside any stream capture.  The cache does not survive
//    cudaDeviceReset (or any other re-creation of the device's primary context): a process that resets a device
//    must not call this function on it afterwards.
//  * All calls on a device share the one scratch array.  Two calls whose kernels overlap on the GPU (different
//    streams without an ordering between them) race on it; calls on the same stream are ordered and safe.  Nothing in
//    the array has to start at zero: every slot that is read is written earlier in the same call.
#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>
#include <string>

#include "../../include/thundergbm.h"
#include "tgbm_kernels.cuh"

namespace {

constexpr int kMaxBlocks = 1024;  // thread blocks of the first reduction stage = partial sums kept
static __device__ __align__(256) double g_noalloc_scratch[kMaxBlocks + 1];  // [0, kMaxBlocks): partials, [kMaxBlocks]: total

constexpr int kMaxDevices = 64;
double *g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

// device address of the scratch array on the current device (looked up once per device)
double *scratch_on_current_device() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) throw tgbm::Error(std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) throw tgbm::Error("device index out of range for the no-allocation entry point");
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr)
            throw tgbm::Error(std::string("cudaGetSymbolAddress(scratch) failed: ") + cudaGetErrorString(e));
        g_scratch_addr[dev] = static_cast<double *>(p);
    }
    return g_scratch_addr[dev];
}

}  // namespace

extern "C" {

int tgbm_metric_score_noalloc(const char *objective, int n_rows, int trees_per_round, const float *d_label,
                              const float *d_raw, float *d_out, void *cuda_stream) {
    try {
        tgbm::set_last_error("");
        const int o = tgbm::objective_from_name(objective ? objective : "");
        TGBM_CHECK(o != tgbm::OBJ_UNKNOWN, std::string("undefined objective ") + (objective ? objective : "(null)"));
        TGBM_CHECK(!tgbm::need_group_file(o), "ranking metrics need per-query buffers; use tgbm_metric_score");
        TGBM_CHECK(d_label && d_raw && d_out, "null device pointer");
        TGBM_CHECK(n_rows >= 1 && n_rows <= TGBM_NOALLOC_MAX_ROWS,
                   "n_rows outside [1, " + std::to_string(TGBM_NOALLOC_MAX_ROWS) + "] for the no-allocation entry point");
        TGBM_CHECK(trees_per_round >= 1 && trees_per_round <= TGBM_NOALLOC_MAX_CLASSES,
                   "trees_per_round outside [1, " + std::to_string(TGBM_NOALLOC_MAX_CLASSES) + "] for the no-allocation entry point");
        double *scratch = scratch_on_current_device();
        cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
        // same two-stage, fixed-order reduction and the same grid as tgbm_metric_score, so the results are bit-identical
        const int blocks = std::max(1, std::min((n_rows + 255) / 256, kMaxBlocks));
        tgbm::k_metric_partial<<<blocks, 256, 0, st>>>(o, d_label, d_raw, n_rows, trees_per_round, scratch);
        tgbm::k_metric_sum<<<1, 32, 0, st>>>(scratch, blocks, scratch + kMaxBlocks);
        tgbm::k_metric_final<<<1, 32, 0, st>>>(o, scratch + kMaxBlocks, (long long)n_rows, d_out);
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) throw tgbm::Error(std::string("kernel launch failed: ") + cudaGetErrorString(e));
        return 0;
    } catch (const std::exception &e) {
        tgbm::set_last_error(e.what());
        return 1;
    }
}

}  // extern "C"
