// Row-sharded randomized SVD over several GPUs (one process per GPU): the tall matrix A is split by
// rows, A = [A_0; ...; A_{P-1}], every rank keeps its A_p (m_p x n), the small factors are replicated.
// What crosses NVLink per call: the k x k Gram matrix of every tall-panel QR pass, the n x k partial
// products A_p^T Q_p of every power iteration and of the final projection -- all through NCCL
// all-reduce on the caller's stream, nothing else.  The reference has no multi-GPU mode; this is the
// sharded counterpart of svd_lowrank_cuda (modules/svd_lowrank_cuda/src/svd_lowrank_cuda.cu:569-581).
//
// NCCL is bound at run time (dlopen of libnccl.so.2), so the library loads on hosts without it and
// shares the copy a host application (for instance PyTorch) has already loaded.
#include <bitsqz_llm_c.h>

#include "bsq_internal.hpp"

#include <dlfcn.h>

#include <cstring>
#include <mutex>

namespace {

using namespace bsq;

struct NcclApi {
    // the five entry points used, with the signatures of nccl.h (ncclResult_t is an int enum, 0 = success;
    // ncclUniqueId is 128 opaque bytes; ncclFloat = 7, ncclSum = 0)
    int (*GetUniqueId)(void *id) = nullptr;
    int (*CommInitRank)(void **comm, int nranks, struct UniqueId128 id, int rank) = nullptr;
    int (*AllReduce)(const void *send, void *recv, size_t count, int dtype, int op, void *comm, cudaStream_t stream) = nullptr;
    int (*CommDestroy)(void *comm) = nullptr;
    bool ok = false;
};
struct UniqueId128 {
    char bytes[128];
};

NcclApi &nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(h, "ncclAllReduce"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
        api.ok = api.GetUniqueId && api.CommInitRank && api.AllReduce && api.CommDestroy;
    });
    return api;
}

struct ShardComm {
    void *comm = nullptr;
    int rank = 0, world = 1;
};

cudaError_t allreduce_sum(void *ctx, float *buf, size_t count, cudaStream_t stream) {
    ShardComm *c = static_cast<ShardComm *>(ctx);
    if (!c || !c->comm) return cudaErrorInvalidValue;
    return nccl().AllReduce(buf, buf, count, /*ncclFloat*/ 7, /*ncclSum*/ 0, c->comm, stream) == 0 ? cudaSuccess
                                                                                                    : cudaErrorUnknown;
}

}  // namespace

extern "C" {

int bsq_shard_unique_id(void *out, size_t bytes) {
    if (!out || bytes < 128 || !nccl().ok) return 1;
    UniqueId128 id;
    std::memset(&id, 0, sizeof(id));
    if (nccl().GetUniqueId(&id) != 0) return 1;
    std::memcpy(out, &id, 128);
    return 0;
}

void *bsq_shard_comm_create(const void *unique_id, int rank, int world) {
    if (!unique_id || world < 1 || rank < 0 || rank >= world || !nccl().ok) return nullptr;
    UniqueId128 id;
    std::memcpy(&id, unique_id, 128);
    ShardComm *c = new ShardComm();
    c->rank = rank;
    c->world = world;
    if (nccl().CommInitRank(&c->comm, world, id, rank) != 0) {
        delete c;
        return nullptr;
    }
    return c;
}

void bsq_shard_comm_destroy(void *comm) {
    ShardComm *c = static_cast<ShardComm *>(comm);
    if (!c) return;
    if (c->comm) nccl().CommDestroy(c->comm);
    delete c;
}

int bsq_svd_lowrank_sharded(void *comm, const float *d_A_local, int m_local, int m_total, int n, int k, int niter,
                            unsigned long long seed, float *d_U_local, float *d_S, float *d_V, void *stream) {
    ShardComm *c = static_cast<ShardComm *>(comm);
    if (!c || !d_A_local || !d_U_local || !d_S || !d_V || m_local <= 0 || m_total < m_local || n <= 0 || k <= 0 || niter < 0)
        return 1;
    if (m_total < n) return 1;       // the sharded dimension must be the tall one
    SvdWorkspace *ws = svd_workspace_create_sharded(m_local, n, k, niter, device_sm_count(), allreduce_sum, c, m_total);
    if (!ws) return 1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const cudaError_t e = svd_lowrank(ws, d_A_local, d_U_local, d_S, d_V, seed, nullptr, st);
    const cudaError_t s = svd_workspace_finish(ws, st);
    svd_workspace_destroy(ws);
    if (e != cudaSuccess || s != cudaSuccess) {
        cudaGetLastError();
        return 1;
    }
    return 0;
}

}  // extern "C"
