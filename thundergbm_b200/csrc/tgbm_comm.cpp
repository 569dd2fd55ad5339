#include "tgbm_comm.h"

#include <dlfcn.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>

#include "tgbm_common.h"

namespace tgbm {
namespace {

// the handful of NCCL entry points used, declared here so that nccl.h is not a build dependency
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { ncclInt8 = 0, ncclUint8 = 1, ncclInt32 = 2, ncclUint32 = 3, ncclInt64 = 4, ncclUint64 = 5, ncclFloat32 = 7, ncclFloat64 = 8 };
enum { ncclSum = 0, ncclProd = 1, ncclMax = 2, ncclMin = 3 };

struct Api {
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    void *lib = nullptr;
};

Api &api() {
    static Api a;
    static std::once_flag once;
    std::call_once(once, [] {
        // RTLD_NOLOAD first: reuse the copy a host framework (e.g. torch) already mapped
        a.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
        if (!a.lib) a.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!a.lib) a.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!a.lib) return;
        a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(a.lib, "ncclGetUniqueId");
        a.CommInitRank = (decltype(a.CommInitRank))dlsym(a.lib, "ncclCommInitRank");
        a.CommDestroy = (decltype(a.CommDestroy))dlsym(a.lib, "ncclCommDestroy");
        a.AllReduce = (decltype(a.AllReduce))dlsym(a.lib, "ncclAllReduce");
        a.AllGather = (decltype(a.AllGather))dlsym(a.lib, "ncclAllGather");
        a.GetErrorString = (decltype(a.GetErrorString))dlsym(a.lib, "ncclGetErrorString");
        a.CommGetAsyncError = (decltype(a.CommGetAsyncError))dlsym(a.lib, "ncclCommGetAsyncError");
        a.CommAbort = (decltype(a.CommAbort))dlsym(a.lib, "ncclCommAbort");
    });
    TGBM_CHECK(a.lib && a.GetUniqueId && a.CommInitRank && a.AllReduce && a.AllGather,
               "multi-GPU training needs NCCL (libnccl.so.2 could not be loaded)");
    return a;
}

void check(ncclResult_t r, const char *what) {
    if (r != 0) {
        const char *s = api().GetErrorString ? api().GetErrorString(r) : "?";
        throw Error(std::string("NCCL error in ") + what + ": " + s);
    }
}

int nccl_type(Comm::DType t) {
    switch (t) {
    case Comm::I32: return ncclInt32;
    case Comm::I64: return ncclInt64;
    case Comm::U32: return ncclUint32;
    case Comm::F64: return ncclFloat64;
    case Comm::U8: return ncclUint8;
    case Comm::F32: return ncclFloat32;
    }
    return ncclInt32;
}

}  // namespace

void Comm::allreduce(void *buf, size_t count, DType t, Op op, cudaStream_t stream) const {
    if (world <= 1 || count == 0) return;
    check(api().AllReduce(buf, buf, count, nccl_type(t), op == SUM ? ncclSum : ncclMax, (ncclComm_t)nccl_comm, stream),
          "ncclAllReduce");
}

void Comm::allgather(const void *in, void *out, size_t count, DType t, cudaStream_t stream) const {
    if (world <= 1) {
        size_t es = (t == I64 || t == F64) ? 8 : (t == U8 ? 1 : 4);
        if (in != out) cudaMemcpyAsync(out, in, count * es, cudaMemcpyDeviceToDevice, stream);
        return;
    }
    check(api().AllGather(in, out, count, nccl_type(t), (ncclComm_t)nccl_comm, stream), "ncclAllGather");
}

void Comm::agree(const std::string &local_error, const char *phase, cudaStream_t stream) const {
    bool all_ok = local_error.empty();
    if (world > 1) {
        if (host) {
            all_ok = host->agree(local_error.empty());
        } else {
            int h = local_error.empty() ? 0 : 1;
            cudaMemcpyAsync(d_flag, &h, sizeof(int), cudaMemcpyHostToDevice, stream);
            allreduce(d_flag, 1, I32, MAX, stream);
            cudaMemcpyAsync(&h, d_flag, sizeof(int), cudaMemcpyDeviceToHost, stream);
            wait(stream);
            all_ok = h == 0;
        }
    }
    if (all_ok) return;
    if (!local_error.empty()) throw Error(local_error);
    throw Error(std::string("another rank failed while ") + phase + "; this rank stops with it");
}

void Comm::wait(cudaStream_t stream) const {
    if (world <= 1 || !nccl_comm) {
        const cudaError_t e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) throw Error(std::string("CUDA error: ") + cudaGetErrorString(e));
        return;
    }
    const auto t0 = std::chrono::steady_clock::now();
    for (long spin = 0;; ++spin) {
        const cudaError_t q = cudaStreamQuery(stream);
        if (q == cudaSuccess) return;
        if (q != cudaErrorNotReady) throw Error(std::string("CUDA error: ") + cudaGetErrorString(q));
        ncclResult_t async = 0;
        const bool have = api().CommGetAsyncError != nullptr;
        if (have && (spin & 63) == 0) check(api().CommGetAsyncError((ncclComm_t)nccl_comm, &async), "ncclCommGetAsyncError");
        const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        const bool group_broken = host && (spin & 63) == 0 && host->broken();
        if ((async != 0 && async != 7 /* ncclInProgress */) || waited > timeout_s || group_broken) {
            if (api().CommAbort) api().CommAbort((ncclComm_t)nccl_comm);
            const_cast<Comm *>(this)->nccl_comm = nullptr;
            if (host) host->abandon();
            throw Error(async != 0 && async != 7 ? std::string("NCCL reported an asynchronous error: ") + (api().GetErrorString ? api().GetErrorString(async) : "?")
                        : group_broken ? std::string("another rank of the group failed; its collectives were aborted")
                                       : "a collective did not finish within " + std::to_string((int)timeout_s) +
                                             " s (a rank is missing?); the communicator was aborted");
        }
        if (spin < 2000) std::this_thread::yield();
        else std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

void comm_get_unique_id(unsigned char id[128]) {
    ncclUniqueId u;
    check(api().GetUniqueId(&u), "ncclGetUniqueId");
    memcpy(id, u.internal, 128);
}

Comm *comm_create(const unsigned char id[128], int rank, int world) {
    Comm *c = new Comm;
    c->rank = rank;
    c->world = world;
    if (world > 1) {
        ncclUniqueId u;
        memcpy(u.internal, id, 128);
        ncclComm_t nc = nullptr;
        check(api().CommInitRank(&nc, world, u, rank), "ncclCommInitRank");
        c->nccl_comm = nc;
        if (cudaMalloc((void **)&c->d_flag, sizeof(int)) != cudaSuccess) {
            api().CommDestroy(nc);
            delete c;
            throw Error("cudaMalloc of the communicator's status word failed");
        }
        if (const char *e = getenv("TGBM_COMM_TIMEOUT_S")) c->timeout_s = atof(e) > 0 ? atof(e) : c->timeout_s;
    }
    return c;
}

void comm_destroy(Comm *c) {
    if (!c) return;
    if (c->nccl_comm) api().CommDestroy((ncclComm_t)c->nccl_comm);
    if (c->d_flag) cudaFree(c->d_flag);
    delete c;
}

}  // namespace tgbm
