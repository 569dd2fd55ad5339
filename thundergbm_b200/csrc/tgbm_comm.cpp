#include "tgbm_comm.h"

#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <string>

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
    }
    return c;
}

void comm_destroy(Comm *c) {
    if (!c) return;
    if (c->nccl_comm) api().CommDestroy((ncclComm_t)c->nccl_comm);
    delete c;
}

}  // namespace tgbm
