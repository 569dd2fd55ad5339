// Collective layer for row-sharded training: one process per GPU, NCCL over NVLink.
// The reference has no collective library: it shards by columns and exchanges split points and
// ins2node_id through host memory and cudaMemcpyPeer (src/thundergbm/builder/tree_builder.cu:94-145).
// Here rows are sharded and the per-level node histograms are sum-reduced, so every rank runs
// the same split selection on identical integers.
//
// NCCL is bound at run time (dlopen of libnccl.so.2) so that a single-GPU process never needs it.
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>

#include "tgbm_hostgroup.h"

namespace tgbm {

struct Comm {
    int rank = 0;
    int world = 1;
    void *nccl_comm = nullptr;
    // ranks that are threads of one process (n_device > 1 through the reference's entry points) also meet on the host
    std::shared_ptr<HostGroup> host;
    int *d_flag = nullptr;  // one device word for agree() between processes
    double timeout_s = 600;  // wait(): how long a stream with collectives in flight may stay busy (TGBM_COMM_TIMEOUT_S)

    enum DType { I32, I64, U32, F64, U8, F32 };
    enum Op { SUM, MAX };

    bool active() const { return world > 1; }
    // in-place all-reduce on `stream`
    void allreduce(void *buf, size_t count, DType t, Op op, cudaStream_t stream) const;
    // out must hold world*count elements
    void allgather(const void *in, void *out, size_t count, DType t, cudaStream_t stream) const;

    // Every rank reports whether its last local phase succeeded (`local_error` empty) before anyone enqueues the next
    // collective; throws on EVERY rank when some rank failed: the failing rank its own message, the others a note
    // naming the phase.  In-process groups meet on the host (HostGroup); process groups all-reduce one word.
    void agree(const std::string &local_error, const char *phase, cudaStream_t stream) const;
    // cudaStreamSynchronize for a stream that carries collectives: polls the stream and the communicator's asynchronous
    // error state, and gives up (aborting the communicator, then throwing) after `timeout_s` or on a reported error --
    // a rank that left between steps must not keep this host thread waiting for ever.
    void wait(cudaStream_t stream) const;
};

// 128-byte NCCL unique id, created by rank 0 and handed to every rank by the caller
void comm_get_unique_id(unsigned char id[128]);
Comm *comm_create(const unsigned char id[128], int rank, int world);
void comm_destroy(Comm *c);

}  // namespace tgbm
