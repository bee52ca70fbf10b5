// Row-sharded randomized SVD over several GPUs (one process per GPU): the tall matrix A is split by
// rows, A = [A_0; ...; A_{P-1}], every rank keeps its A_p (m_p x n), the small factors are replicated.
// What crosses NVLink per call: the k x k Gram matrix of every tall-panel QR pass, the n x k partial
// products A_p^T Q_p of every power iteration and of the final projection -- all through NCCL
// all-reduce on the caller's stream, nothing else.  The reference has no multi-GPU mode; this is the
// sharded counterpart of svd_lowrank_cuda (modules/svd_lowrank_cuda/src/svd_lowrank_cuda.cu:569-581).
//
// NCCL is bound at run time (dlopen of libnccl.so.2), so the library loads on hosts without it and
// shares the copy a host application (for instance PyTorch) has already loaded.
#include <bitsqz_llm.hpp>
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

struct bsq_shard_svd {
    ShardComm *comm = nullptr;
    SvdWorkspace *ws = nullptr;
    int m_local = 0, m_total = 0, n = 0, k = 0, niter = 0;
    float *u = nullptr, *s = nullptr, *v = nullptr;        // factor buffers of bsq_shard_compress
};

// The workspace (about twenty device allocations, a random-number generator, a solver handle) is made once per
// communicator and shape and serves any number of calls.
bsq_shard_svd *bsq_shard_svd_create(void *comm, int m_local, int m_total, int n, int k, int niter) {
    ShardComm *c = static_cast<ShardComm *>(comm);
    if (!c || m_local <= 0 || m_total < m_local || n <= 0 || k <= 0 || niter < 0) return nullptr;
    if (m_total < n) return nullptr;       // the sharded dimension must be the tall one
    bsq_shard_svd *h = new bsq_shard_svd();
    h->comm = c;
    h->m_local = m_local; h->m_total = m_total; h->n = n; h->niter = niter;
    h->k = k < n ? k : n;
    h->ws = svd_workspace_create_sharded(m_local, n, k, niter, device_sm_count(), allreduce_sum, c, m_total);
    if (!h->ws) {
        delete h;
        return nullptr;
    }
    return h;
}

void bsq_shard_svd_destroy(bsq_shard_svd *h) {
    if (!h) return;
    if (h->ws) svd_workspace_destroy(h->ws);
    if (h->u) cudaFree(h->u);
    if (h->s) cudaFree(h->s);
    if (h->v) cudaFree(h->v);
    cudaGetLastError();
    delete h;
}

int bsq_shard_svd_run(bsq_shard_svd *h, const float *d_A_local, unsigned long long seed, float *d_U_local, float *d_S, float *d_V,
                      void *stream) {
    if (!h || !d_A_local || !d_U_local || !d_S || !d_V) return 1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const cudaError_t e = svd_lowrank(h->ws, d_A_local, d_U_local, d_S, d_V, seed, nullptr, st);
    const cudaError_t s = svd_workspace_finish(h->ws, st);
    if (e != cudaSuccess || s != cudaSuccess) {
        cudaGetLastError();
        return 1;
    }
    return 0;
}

int bsq_shard_svd_profile(bsq_shard_svd *h, int on) { return (h && svd_workspace_profile(h->ws, on != 0) == cudaSuccess) ? 0 : 1; }
int bsq_shard_svd_profile_read(bsq_shard_svd *h, float *ms, int *kinds, int capacity) {
    return (h && capacity >= 0) ? svd_workspace_spans(h->ws, ms, kinds, capacity) : 0;
}

// This rank's shard as an ordinary packed object: its m_local rows of U, and S and V, as FP32 sections of an
// m_local x n matrix of rank k.  bitsqz_llm_decompress, initialised for that shape and rank with FP32 factors,
// reconstructs the shard's rows from it; no rank needs any other rank's object.
int bsq_shard_compress(bsq_shard_svd *h, const float *d_A_local, unsigned long long seed, struct bitsqz_llm_array **out, void *stream) {
    if (!h || !d_A_local || !out || *out) return 1;
    if (h->m_local > 65535 || h->n > 65535) return 1;      // one object holds at most 65 535 rows: use more shards
    const size_t ub = (size_t)h->m_local * h->k * 4, sb = (size_t)h->k * 4, vb = (size_t)h->n * h->k * 4;
    if (!h->u && (cudaMalloc(reinterpret_cast<void **>(&h->u), ub) != cudaSuccess || cudaMalloc(reinterpret_cast<void **>(&h->s), sb) != cudaSuccess ||
                  cudaMalloc(reinterpret_cast<void **>(&h->v), vb) != cudaSuccess)) {
        cudaGetLastError();
        return 1;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t total = sizeof(bitsqz_llm_array_t) + ub + sb + vb;
    uint8_t *block = static_cast<uint8_t *>(host_block_take(total));
    if (!block) return 1;
    uint8_t *payload = block + sizeof(bitsqz_llm_array_t);
    cudaError_t e = svd_lowrank(h->ws, d_A_local, h->u, h->s, h->v, seed, nullptr, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(payload, h->u, ub, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(payload + ub, h->s, sb, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(payload + ub + sb, h->v, vb, cudaMemcpyDeviceToHost, st);
    const cudaError_t f = svd_workspace_finish(h->ws, st);
    if (e != cudaSuccess || f != cudaSuccess) {
        cudaGetLastError();
        bitsqz_llm_free(reinterpret_cast<bitsqz_llm_array_t *>(block));
        return 1;
    }
    bitsqz_llm_array_t *a = reinterpret_cast<bitsqz_llm_array_t *>(block);
    std::memset(a, 0, sizeof(*a));
    a->num_rows = (uint16_t)h->m_local;
    a->num_columns = (uint16_t)h->n;
    a->num_elements = (uint32_t)h->m_local * (uint32_t)h->n;
    a->svd_ranks = (int16_t)h->k;
    a->svd_niters = (int16_t)(h->niter < 1 ? 1 : h->niter);
    a->effective_rank = (int16_t)h->k;
    a->svd_uv_format = a->svd_s_format = a->quantization_only_format = quantization_NONE;
    a->flags = 1u;                                          // SVD sections
    a->section_u.offset = 0;        a->section_u.size = ub; a->section_u.storage = BITSQZ_SECTION_FP32;
    a->section_s.offset = ub;       a->section_s.size = sb; a->section_s.storage = BITSQZ_SECTION_FP32;
    a->section_v.offset = ub + sb;  a->section_v.size = vb; a->section_v.storage = BITSQZ_SECTION_FP32;
    a->payload = payload;
    *out = a;
    return 0;
}

int bsq_svd_lowrank_sharded(void *comm, const float *d_A_local, int m_local, int m_total, int n, int k, int niter,
                            unsigned long long seed, float *d_U_local, float *d_S, float *d_V, void *stream) {
    bsq_shard_svd *h = bsq_shard_svd_create(comm, m_local, m_total, n, k, niter);
    if (!h) return 1;
    const int rc = bsq_shard_svd_run(h, d_A_local, seed, d_U_local, d_S, d_V, stream);
    bsq_shard_svd_destroy(h);
    return rc;
}

}  // extern "C"
