// Row-sharded randomized SVD over several GPUs (one process per GPU): the tall matrix A is split by
// rows, A = [A_0; ...; A_{P-1}], every rank keeps its A_p (m_p x n), the small factors are replicated.
// What crosses NVLink per call: the k x k Gram matrix of every tall-panel QR pass -- one kernel per rank that
// sends, waits and adds over peer memory (below; NCCL where the ranks cannot map each other's memory) --
// and the n x k partial products A_p^T Q_p of every power iteration and of the final projection, through NCCL
// all-reduce on the caller's stream; nothing else.  The reference has no multi-GPU mode; this is the
// sharded counterpart of svd_lowrank_cuda (modules/svd_lowrank_cuda/src/svd_lowrank_cuda.cu:569-581).
//
// NCCL is bound at run time (dlopen of libnccl.so.2), so the library loads on hosts without it and
// shares the copy a host application (for instance PyTorch) has already loaded.
#include <bitsqz_llm.hpp>
#include <bitsqz_llm_c.h>

#include "bsq_internal.hpp"

#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

namespace {

using namespace bsq;

struct NcclApi {
    // the five entry points used, with the signatures of nccl.h (ncclResult_t is an int enum, 0 = success;
    // ncclUniqueId is 128 opaque bytes; ncclFloat = 7, ncclSum = 0)
    int (*GetUniqueId)(void *id) = nullptr;
    int (*CommInitRank)(void **comm, int nranks, struct UniqueId128 id, int rank) = nullptr;
    int (*AllReduce)(const void *send, void *recv, size_t count, int dtype, int op, void *comm, cudaStream_t stream) = nullptr;
    int (*AllGather)(const void *send, void *recv, size_t sendcount, int dtype, void *comm, cudaStream_t stream) = nullptr;
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
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(h, "ncclAllGather"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
        api.ok = api.GetUniqueId && api.CommInitRank && api.AllReduce && api.CommDestroy;
    });
    return api;
}

// ---- one-shot all-reduce of a small matrix over peer memory ------------------------------------------------------
// The k x k Gram matrix of a tall-panel QR pass is 64-256 KiB: an exchange whose cost is latency, not bandwidth.  Every
// rank keeps an exchange area that all other ranks of the node have mapped (CUDA IPC; the handles travel through one
// NCCL all-gather at set-up): per call parity one slot of 256 x 256 floats PER SOURCE RANK, and one flag word per rank.
// One kernel per rank does the whole all-reduce: it stores its matrix into its slot in every rank's area (posted
// stores over NVLink: nobody waits for a round trip), fences, tells every peer (the call's sequence number into the
// peer's flag word for this rank), waits -- with a limit -- until every rank's number has arrived here, and adds the
// slots, now all in local memory, in rank order, so that every rank gets the same bits.  Two parities are enough: a
// rank starts call n + 1 only after every rank's call n contribution has arrived, so when it overwrites the parity of
// call n (with call n + 2) every peer has finished reading call n: a peer sends call n + 1 only after its sums of call
// n are done, and this rank needs that contribution before it can get to call n + 2.  No multicast, no TMA from peer
// memory.
constexpr int kPeerMaxWorld = 16;
constexpr size_t kPeerSlotFloats = 256 * 256;
constexpr int kPeerCtas = 8, kPeerThreads = 256;
constexpr unsigned kPeerSpinLimit = 1u << 24;        // polls with a short sleep in between: seconds (ranks may start a call apart)

struct PeerControl {                                  // behind the slots of a rank's area
    unsigned flags[64];                               // flags[r]: sequence number of rank r's last contribution
    unsigned counter;                                 // CTAs of the running kernel that have sent their slice
    unsigned status;                                  // 1: a wait ran out
};
// area: float slot[2][world][kPeerSlotFloats], then PeerControl
__host__ __device__ inline size_t peer_area_bytes(int world) { return (size_t)2 * world * kPeerSlotFloats * sizeof(float) + sizeof(PeerControl); }
__device__ __forceinline__ float *peer_slot(unsigned char *area, int world, unsigned parity, int source) {
    return reinterpret_cast<float *>(area) + ((size_t)parity * world + source) * kPeerSlotFloats;
}
__host__ __device__ inline PeerControl *peer_control(unsigned char *area, int world) {
    return reinterpret_cast<PeerControl *>(area + (size_t)2 * world * kPeerSlotFloats * sizeof(float));
}

struct PeerTable {                                    // device-side copy of the mapped addresses
    unsigned char *area[kPeerMaxWorld];
};

struct PeerExchange {
    unsigned char *mine = nullptr;
    unsigned char *mapped[kPeerMaxWorld] = {};
    PeerTable *d_table = nullptr;
    unsigned seq = 0;
    int world = 0, rank = 0;
    bool ok = false;
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(kPeerThreads) peer_allreduce_kernel(float *buf, int count, const PeerTable *table, int rank, int world,
                                                                     unsigned seq) {
    unsigned char *mine = table->area[rank];
    PeerControl *ctl = peer_control(mine, world);
    const unsigned parity = seq & 1u;
    const int per_cta = ((count + (int)gridDim.x - 1) / (int)gridDim.x + 3) & ~3;
    const int lo = blockIdx.x * per_cta, hi = min(count, lo + per_cta);
    // this CTA's slice of the local matrix into this rank's slot on every rank
    const bool vec = (count & 3) == 0 && (reinterpret_cast<uintptr_t>(buf) & 15) == 0;
    for (int p = 0; p < world; ++p) {
        float *dst = peer_slot(table->area[p], world, parity, rank);
        if (vec) {
            for (int i = lo + 4 * (int)threadIdx.x; i < hi; i += 4 * (int)blockDim.x)
                *reinterpret_cast<float4 *>(dst + i) = *reinterpret_cast<const float4 *>(buf + i);
        } else {
            for (int i = lo + (int)threadIdx.x; i < hi; i += (int)blockDim.x) dst[i] = buf[i];
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(&ctl->counter, 1u);
        if (prev == gridDim.x - 1) {                  // the last CTA to have sent its slice: the whole matrix is out
            ctl->counter = 0;
            __threadfence_system();
            for (int p = 0; p < world; ++p) st_release_sys(&peer_control(table->area[p], world)->flags[rank], seq);
        }
    }
    bool ok = true;
    if ((int)threadIdx.x < world) {
        unsigned spins = 0;
        while (ld_acquire_sys(&ctl->flags[threadIdx.x]) < seq) {
            if (++spins > kPeerSpinLimit) { ok = false; break; }
            __nanosleep(40);
        }
    }
    ok = __syncthreads_and(ok) != 0;
    if (!ok) {                                        // give up: say so, leave buf as it is
        if (threadIdx.x == 0) ctl->status = 1u;
        return;
    }
    // all contributions are in local memory now (L2: the peers' stores never went through this SM's L1)
    if (vec) {
        for (int i = lo + 4 * (int)threadIdx.x; i < hi; i += 4 * (int)blockDim.x) {
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int p = 0; p < world; ++p) {
                const float4 v = __ldcg(reinterpret_cast<const float4 *>(peer_slot(mine, world, parity, p) + i));
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
            }
            *reinterpret_cast<float4 *>(buf + i) = sum;
        }
    } else {
        for (int i = lo + (int)threadIdx.x; i < hi; i += (int)blockDim.x) {
            float sum = 0.0f;
            for (int p = 0; p < world; ++p) sum += __ldcg(peer_slot(mine, world, parity, p) + i);
            buf[i] = sum;
        }
    }
}

struct ShardComm {
    void *comm = nullptr;
    int rank = 0, world = 1;
    PeerExchange px;
};

bool peer_enabled() {
    const char *e = getenv("BSQ_SHARD_PEER");         // 0: NCCL for the small all-reduces too
    return !(e && e[0] == '0');
}

// Every rank allocates its area, the IPC handles go round through NCCL, every rank maps the others' areas; the
// exchange is used only if that worked on every rank (a sum over the ranks of "it worked here").
void peer_setup(ShardComm *c) {
    PeerExchange &px = c->px;
    px.world = c->world;
    px.rank = c->rank;
    if (!peer_enabled() || c->world < 2 || c->world > kPeerMaxWorld || !nccl().AllGather) return;
    bool fine = cudaMalloc(reinterpret_cast<void **>(&px.mine), peer_area_bytes(c->world)) == cudaSuccess &&
                cudaMemset(px.mine, 0, peer_area_bytes(c->world)) == cudaSuccess;
    cudaIpcMemHandle_t handle;
    std::memset(&handle, 0, sizeof(handle));
    fine = fine && cudaIpcGetMemHandle(&handle, px.mine) == cudaSuccess;
    unsigned char *d_send = nullptr, *d_recv = nullptr;
    float *d_vote = nullptr;
    const size_t hb = sizeof(cudaIpcMemHandle_t);
    if (cudaMalloc(reinterpret_cast<void **>(&d_send), hb) != cudaSuccess || cudaMalloc(reinterpret_cast<void **>(&d_recv), hb * c->world) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void **>(&d_vote), sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        return;                                       // (every rank takes part in the collectives below or none: an allocation of a few bytes does not fail on one rank alone)
    }
    std::vector<cudaIpcMemHandle_t> all(c->world);
    cudaMemcpy(d_send, &handle, hb, cudaMemcpyHostToDevice);
    if (nccl().AllGather(d_send, d_recv, hb, /*ncclInt8*/ 0, c->comm, nullptr) != 0) fine = false;
    if (cudaStreamSynchronize(nullptr) != cudaSuccess) fine = false;
    cudaMemcpy(all.data(), d_recv, hb * c->world, cudaMemcpyDeviceToHost);
    for (int p = 0; p < c->world && fine; ++p) {
        if (p == c->rank) { px.mapped[p] = px.mine; continue; }
        void *ptr = nullptr;
        if (cudaIpcOpenMemHandle(&ptr, all[p], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); fine = false; break; }
        px.mapped[p] = static_cast<unsigned char *>(ptr);
    }
    PeerTable table;
    std::memset(&table, 0, sizeof(table));
    for (int p = 0; p < c->world; ++p) table.area[p] = px.mapped[p];
    fine = fine && cudaMalloc(reinterpret_cast<void **>(&px.d_table), sizeof(PeerTable)) == cudaSuccess &&
           cudaMemcpy(px.d_table, &table, sizeof(table), cudaMemcpyHostToDevice) == cudaSuccess;
    // agreement: the exchange is on only if it is on everywhere
    const float vote = fine ? 1.0f : 0.0f;
    float total = 0.0f;
    cudaMemcpy(d_vote, &vote, sizeof(float), cudaMemcpyHostToDevice);
    const bool voted = nccl().AllReduce(d_vote, d_vote, 1, /*ncclFloat*/ 7, /*ncclSum*/ 0, c->comm, nullptr) == 0 &&
                       cudaStreamSynchronize(nullptr) == cudaSuccess &&
                       cudaMemcpy(&total, d_vote, sizeof(float), cudaMemcpyDeviceToHost) == cudaSuccess;
    px.ok = voted && total == (float)c->world;
    cudaFree(d_send);
    cudaFree(d_recv);
    cudaFree(d_vote);
    cudaGetLastError();
}

void peer_teardown(ShardComm *c) {
    PeerExchange &px = c->px;
    for (int p = 0; p < px.world; ++p)
        if (p != px.rank && px.mapped[p]) cudaIpcCloseMemHandle(px.mapped[p]);
    if (px.d_table) cudaFree(px.d_table);
    if (px.mine) cudaFree(px.mine);
    cudaGetLastError();
    px = PeerExchange{};
}

cudaError_t allreduce_sum(void *ctx, float *buf, size_t count, cudaStream_t stream) {
    ShardComm *c = static_cast<ShardComm *>(ctx);
    if (!c || !c->comm) return cudaErrorInvalidValue;
    if (c->px.ok && count <= kPeerSlotFloats) {       // the k x k matrices: one kernel over peer memory
        peer_allreduce_kernel<<<kPeerCtas, kPeerThreads, 0, stream>>>(buf, (int)count, c->px.d_table, c->rank, c->world, ++c->px.seq);
        return cudaGetLastError();
    }
    return nccl().AllReduce(buf, buf, count, /*ncclFloat*/ 7, /*ncclSum*/ 0, c->comm, stream) == 0 ? cudaSuccess
                                                                                                    : cudaErrorUnknown;
}

// 0 = fine; 1 = a wait of the peer exchange ran out since the last check (the word is cleared)
int peer_status(ShardComm *c, cudaStream_t stream) {
    if (!c->px.ok) return 0;
    unsigned h = 0;
    unsigned *word = &peer_control(c->px.mine, c->world)->status;
    if (cudaMemcpyAsync(&h, word, sizeof(unsigned), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess)
        return 1;
    if (h) cudaMemsetAsync(word, 0, sizeof(unsigned), stream);
    return h ? 1 : 0;
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
    peer_setup(c);                                    // optional: without it the small all-reduces go through NCCL too
    return c;
}

void bsq_shard_comm_destroy(void *comm) {
    ShardComm *c = static_cast<ShardComm *>(comm);
    if (!c) return;
    peer_teardown(c);
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
    const int px = peer_status(h->comm, st);
    if (e != cudaSuccess || s != cudaSuccess || px != 0) {
        cudaGetLastError();
        return 1;
    }
    return 0;
}

// 1 if this communicator's small all-reduces run as one kernel over peer memory, 0 if they go through NCCL
int bsq_shard_uses_peer_exchange(void *comm) {
    ShardComm *c = static_cast<ShardComm *>(comm);
    return (c && c->px.ok) ? 1 : 0;
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
    if (e != cudaSuccess || f != cudaSuccess || peer_status(h->comm, st) != 0) {
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
