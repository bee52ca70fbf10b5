// Host side of the drop-in library: the nine functions of include/bitsqz_llm.hpp.
//
// Mirrors the observable behaviour of the reference orchestrator (src/bitsqz_llm.cu): the
// same argument checks and 0/1 return codes (:785-885, :891-975), the same stage order
// (:981-1302, :1304-1393), the same section order and byte layout of the returned object
// (:1237-1277) and the same compatibility rules on decompress (:654-761).  What differs is
// how the work is issued: every stage is enqueued on one stream without intermediate
// synchronisation, results are copied straight from the device buffers into their final place
// inside one pinned, pooled host block, and the call synchronises once at the end.  There is
// one compress and one decompress runtime per CUDA device (the reference keeps one pair per
// process); a host thread per GPU can therefore drive several devices through this interface.
#include <bitsqz_llm.hpp>
#include <bitsqz_llm_c.h>

#include "bsq_internal.hpp"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

using namespace bsq;

enum : uint32_t { kFlagSvd = 1u << 0, kFlagOutlier = 1u << 1, kFlagError = 1u << 2 };
constexpr int kMaxDevices = 64;
constexpr uint32_t kQuantMagic = 0x51544355u;      // quantization_cuda.cuh:12

// 48-byte header in front of every quantised section (quantization_cuda.cuh:15-26)
struct QuantHeader {
    uint32_t magic;
    uint16_t version;
    uint16_t reserved0;
    int32_t method;
    uint32_t reserved1;
    uint64_t num_elements;
    uint64_t num_blocks;
    uint64_t block_size;
    float dq_scale;
    uint32_t reserved2;
};
static_assert(sizeof(QuantHeader) == 48, "quantiser section header is 48 bytes");

// 8-byte header in front of every top-k section (topk_cuda.cuh:16-21)
struct TopkHeader {
    uint16_t num_rows, num_columns, num_topk_columns, reserved;
};
static_assert(sizeof(TopkHeader) == 8, "top-k section header is 8 bytes");

bool ratio_ok(float r) { return std::isfinite(r) && r >= 0.0f && r <= 1.0f; }
bool method_ok(int m) { return m == quantization_NONE || m == NF4 || m == NF4_DQ; }
uint64_t quant_section_bytes(int method, uint64_t n) {
    const uint64_t nb = (n + 63) / 64;
    return sizeof(QuantHeader) + (method == NF4 ? nb * 4 : nb) + (n + 1) / 2;
}
uint64_t topk_section_bytes(uint32_t rows, uint32_t k) { return sizeof(TopkHeader) + (uint64_t)rows * k * 6; }

// ---- pinned host blocks ------------------------------------------------------------------------
// compress returns one contiguous block (header + payload) that the caller releases with
// bitsqz_llm_free, so the block can come from a pool of page-locked memory: device-to-host
// copies then land directly in the object that is handed out.
class HostPool {
  public:
    void *take(size_t bytes) {
        const size_t cap = round_up(bytes);
        {
            std::lock_guard<std::mutex> g(mu_);
            auto it = free_.find(cap);
            if (it != free_.end() && !it->second.empty()) {
                void *p = it->second.back();
                it->second.pop_back();
                cached_ -= cap;
                live_[p] = cap;
                return p;
            }
        }
        void *p = nullptr;
        if (cudaHostAlloc(&p, cap, cudaHostAllocPortable) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        std::lock_guard<std::mutex> g(mu_);
        live_[p] = cap;
        return p;
    }
    // true if p was a pool block (and is now recycled)
    bool give_back(void *p) {
        size_t cap = 0;
        {
            std::lock_guard<std::mutex> g(mu_);
            auto it = live_.find(p);
            if (it == live_.end()) return false;
            cap = it->second;
            live_.erase(it);
            if (cached_ + cap <= kCacheLimit) {
                free_[cap].push_back(p);
                cached_ += cap;
                return true;
            }
        }
        cudaFreeHost(p);
        return true;
    }

    // release every cached (not handed-out) block; blocks still owned by callers stay valid
    void trim() {
        std::vector<void *> doomed;
        {
            std::lock_guard<std::mutex> g(mu_);
            for (auto &kv : free_)
                for (void *p : kv.second) doomed.push_back(p);
            free_.clear();
            cached_ = 0;
        }
        for (void *p : doomed) cudaFreeHost(p);
        cudaGetLastError();
    }

  private:
    static size_t round_up(size_t b) { return (b + (1u << 16) - 1) & ~(size_t)((1u << 16) - 1); }
    static constexpr size_t kCacheLimit = (size_t)1 << 30;
    std::mutex mu_;
    std::unordered_map<size_t, std::vector<void *>> free_;
    std::unordered_map<void *, size_t> live_;
    size_t cached_ = 0;
};
HostPool &host_pool() {
    static HostPool *pool = new HostPool();      // never destroyed: blocks may outlive static teardown
    return *pool;
}

}  // namespace

void *bsq::host_block_take(size_t bytes) {
    void *p = host_pool().take(bytes);
    return p ? p : std::malloc(bytes);
}

namespace {

// ---- device buffers ----------------------------------------------------------------------------
struct DevBuf {
    void *p = nullptr;
    bool alloc(size_t bytes) {
        release();
        if (bytes == 0) return true;
        if (cudaMalloc(&p, bytes) != cudaSuccess) {
            cudaGetLastError();
            p = nullptr;
            return false;
        }
        return true;
    }
    void release() {
        if (p) cudaFree(p);
        p = nullptr;
    }
    template <typename T>
    T *as() const { return static_cast<T *>(p); }
};

// Device-side pieces of one quantised section
struct QuantBufs {
    uint64_t n = 0, cap = 0;
    DevBuf scales_f32, scale_codes, data, dq;
    bool alloc(uint64_t count) {
        n = cap = count;
        const uint64_t nb = (count + 63) / 64;
        return scales_f32.alloc(nb * 4) && scale_codes.alloc(nb) && data.alloc((count + 1) / 2) && dq.alloc(16);
    }
    void release() {
        scales_f32.release(); scale_codes.release(); data.release(); dq.release();
        n = cap = 0;
    }
};

struct TopkBufs {
    uint32_t k = 0;
    DevBuf idx, val;
    bool alloc(uint32_t rows, uint32_t kk) {
        k = kk;
        if (kk == 0) return true;
        return idx.alloc((size_t)rows * kk * 2) && val.alloc((size_t)rows * kk * 4);
    }
    void release() { idx.release(); val.release(); k = 0; }
};

struct SectionPlan {
    uint64_t offset = 0, size = 0;
    uint8_t storage = BITSQZ_SECTION_NONE;
};

// What a compress call has in flight between its "begin" (everything enqueued) and its "end" (stream waited for,
// status read, header written).
struct CompressJob {
    bool active = false;
    bool to_device = false;               // packed object goes to a device buffer instead of a pinned host block
    uint8_t *block = nullptr;             // host: header + payload (pool block or malloc); device: the caller's buffer
    bool pooled = false;
    uint64_t total = 0;                   // header + payload bytes if every planned section is present
    SectionPlan sec_u, sec_s, sec_v, sec_direct, sec_out, sec_err;
    bool has_svd = false, error_path = false;
    bool prof = false;
    int nev = 0, ev_svd = -1, ev_quant = -1, ev_recon = -1, ev_err = -1;
    std::chrono::steady_clock::time_point t_begin;
};

constexpr size_t kStageBytes = 4096;      // pinned staging for the small headers of a device-resident object

struct Runtime {
    bool initialized = false;
    bool is_compress = false;
    uint16_t rows = 0, cols = 0;
    float outlier_ratio = 0.0f, error_ratio = 0.0f;
    int svd_ranks = -1, svd_niters = 1, rank = 0;       // rank: allocated (effective) rank, 0 without SVD
    int uv_format = quantization_NONE, s_format = quantization_NONE, q_format = quantization_NONE;
    int input_location = BITSQZ_LLM_INPUT_DEVICE;
    bool uses_quant = false;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev[8] = {};
    DevBuf input_stage, residual, recon, error, u, s, v, scratch, status, recon_ws;
    size_t recon_ws_bytes = 0;
    QuantBufs q_direct, q_u, q_s, q_v;
    TopkBufs outlier, err;
    SvdWorkspace *svd = nullptr;
    unsigned *h_status = nullptr;                        // pinned mirror of the device status words
    uint8_t *h_stage = nullptr;                          // pinned: section headers on their way to / from a device-resident object
    size_t stage_used = 0;
    CompressJob job;
    bool decompress_active = false;
    unsigned inject_status = 0;                          // test hook: OR-ed into the status word of the next call

    void release() {
        if (stream) cudaStreamSynchronize(stream);
        input_stage.release(); residual.release(); recon.release(); error.release();
        u.release(); s.release(); v.release(); scratch.release(); status.release(); recon_ws.release();
        q_direct.release(); q_u.release(); q_s.release(); q_v.release();
        outlier.release(); err.release();
        if (svd) { svd_workspace_destroy(svd); svd = nullptr; }
        for (auto &e : ev) { if (e) cudaEventDestroy(e); e = nullptr; }
        if (h_status) { cudaFreeHost(h_status); h_status = nullptr; }
        if (h_stage) { cudaFreeHost(h_stage); h_stage = nullptr; }
        if (job.active && !job.to_device && job.block) {
            if (job.pooled) host_pool().give_back(job.block); else std::free(job.block);
        }
        if (stream) { cudaStreamDestroy(stream); stream = nullptr; }
        cudaGetLastError();
        *this = Runtime{};
    }
};

struct DeviceSlot {
    std::mutex mu;
    Runtime compress, decompress;
};
DeviceSlot *slot_for_current_device() {
    static DeviceSlot slots[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        return nullptr;
    }
    return &slots[dev];
}

bool common_setup(Runtime &rt) {
    rt.sm_count = device_sm_count();
    if (cudaStreamCreateWithFlags(&rt.stream, cudaStreamNonBlocking) != cudaSuccess) return false;
    for (auto &e : rt.ev)
        if (cudaEventCreate(&e) != cudaSuccess) return false;
    if (!rt.status.alloc(64)) return false;
    if (cudaMemset(rt.status.p, 0, 64) != cudaSuccess) return false;
    if (cudaHostAlloc(reinterpret_cast<void **>(&rt.h_status), 64, cudaHostAllocPortable) != cudaSuccess) return false;
    std::memset(rt.h_status, 0, 64);
    if (cudaHostAlloc(reinterpret_cast<void **>(&rt.h_stage), kStageBytes, cudaHostAllocPortable) != cudaSuccess) return false;
    return true;
}

}  // namespace

// ================================================================================================
// initialise / release
// ================================================================================================
namespace {

// Shared part of both initialisers.  Returns false on any allocation failure.
bool setup_runtime(Runtime &rt, bool compress, uint16_t rows, uint16_t cols, float outlier_ratio, float error_ratio,
                   int svd_ranks, int svd_niters, int uv, int s, int q, int input_location) {
    rt.is_compress = compress;
    rt.rows = rows;
    rt.cols = cols;
    rt.outlier_ratio = outlier_ratio;
    rt.error_ratio = error_ratio;
    rt.svd_ranks = svd_ranks;
    rt.svd_niters = svd_niters;
    rt.uv_format = uv;
    rt.s_format = s;
    rt.q_format = q;
    rt.input_location = input_location;
    rt.uses_quant = uv != quantization_NONE || s != quantization_NONE || q != quantization_NONE;
    const bool has_svd = svd_ranks >= 1;
    const size_t n = (size_t)rows * cols;
    // compress clamps the rank (src/bitsqz_llm.cu:820-822); decompress takes it as given (:929,948)
    rt.rank = !has_svd ? 0 : (compress ? std::max(1, std::min(svd_ranks, (int)std::min(rows, cols))) : svd_ranks);
    if (!common_setup(rt)) return false;

    const int ko = outlier_ratio > 0.0f ? topk_num_columns(cols, outlier_ratio) : 0;
    const int ke = error_ratio > 0.0f ? topk_num_columns(cols, error_ratio) : 0;
    if (ko < 0 || ke < 0) return false;
    if (!rt.outlier.alloc(rows, (uint32_t)ko) || !rt.err.alloc(rows, (uint32_t)ke)) return false;

    if (compress) {
        if (input_location == BITSQZ_LLM_INPUT_HOST && !rt.input_stage.alloc(n * 4)) return false;
        if (!rt.residual.alloc(n * 4)) return false;
        if (ke > 0 && (!rt.recon.alloc(n * 4) || !rt.error.alloc(n * 4))) return false;
    }
    if (has_svd) {
        const size_t r = (size_t)rt.rank;
        if (!rt.u.alloc((size_t)rows * r * 4) || !rt.s.alloc(r * 4) || !rt.v.alloc((size_t)cols * r * 4)) return false;
        if (!compress || ke > 0) {                      // the reconstruction runs on decompress and for the error stage
            rt.recon_ws_bytes = reconstruct_workspace_bytes(rows, cols, rt.rank);
            if (rt.recon_ws_bytes && !rt.recon_ws.alloc(rt.recon_ws_bytes)) return false;
        }
        if (compress) {
            if (uv != quantization_NONE && (!rt.q_u.alloc((uint64_t)rows * r) || !rt.q_v.alloc((uint64_t)cols * r))) return false;
            if (s != quantization_NONE && !rt.q_s.alloc(r)) return false;
            rt.svd = svd_workspace_create(rows, cols, rt.rank, svd_niters, rt.sm_count);
            if (!rt.svd) return false;
        }
    } else if (compress && q != quantization_NONE) {
        if (!rt.q_direct.alloc(n)) return false;
    }
    // decompress decodes its sections one after the other on one stream, so one set of quantiser
    // buffers sized for the largest section serves them all; which method a section uses is read
    // from the object, not from this runtime (src/bitsqz_llm.cu:731-738)
    if (!compress && rt.uses_quant) {
        const uint64_t r = (uint64_t)std::max(rt.rank, 0);
        const uint64_t biggest = std::max<uint64_t>(std::max<uint64_t>(n, (uint64_t)rows * r), (uint64_t)cols * r);
        if (!rt.q_direct.alloc(biggest)) return false;
    }
    if (rt.uses_quant) {
        size_t scratch = nf4dq_scratch_bytes(n);
        scratch = std::max(scratch, frontend_scratch_bytes(rows, cols));
        if (!rt.scratch.alloc(scratch)) return false;
        if (cudaMemset(rt.scratch.p, 0, 16) != cudaSuccess) return false;      // the front end's carried selection bound starts empty
    }
    rt.initialized = true;
    return true;
}

}  // namespace

int bitsqz_llm_compress_initialize(uint16_t num_rows, uint16_t num_columns, float outlier_topk_ratio,
                                   float error_correction_topk_ratio, int svd_ranks, int svd_niters,
                                   quantization_method_t svd_uv_format, quantization_method_t svd_s_format,
                                   quantization_method_t quantization_only_format,
                                   bitsqz_llm_input_location_t input_location) {
    try {
        if (num_rows == 0 || num_columns == 0) return 1;
        if (!ratio_ok(outlier_topk_ratio) || !ratio_ok(error_correction_topk_ratio)) return 1;
        if (!method_ok(svd_uv_format) || !method_ok(svd_s_format) || !method_ok(quantization_only_format)) return 1;
        if (input_location != BITSQZ_LLM_INPUT_HOST && input_location != BITSQZ_LLM_INPUT_DEVICE) return 1;
        if (svd_niters < 1) return 1;
        DeviceSlot *slot = slot_for_current_device();
        if (!slot) return 1;
        std::lock_guard<std::mutex> g(slot->mu);
        slot->compress.release();
        if (!setup_runtime(slot->compress, true, num_rows, num_columns, outlier_topk_ratio, error_correction_topk_ratio,
                           svd_ranks, svd_niters, svd_uv_format, svd_s_format, quantization_only_format,
                           input_location)) {
            slot->compress.release();
            return 1;
        }
        return 0;
    } catch (...) {
        return 1;
    }
}

void bitsqz_llm_compress_release() {
    try {
        DeviceSlot *slot = slot_for_current_device();
        if (!slot) return;
        {
            std::lock_guard<std::mutex> g(slot->mu);
            slot->compress.release();
        }
        host_pool().trim();               // cached result blocks go back to the system; blocks callers still hold stay valid
    } catch (...) {
    }
}

int bitsqz_llm_decompress_initialize(uint16_t num_rows, uint16_t num_columns, float outlier_topk_ratio,
                                     float error_correction_topk_ratio, int svd_ranks,
                                     quantization_method_t svd_uv_format, quantization_method_t svd_s_format,
                                     quantization_method_t quantization_only_format) {
    try {
        if (num_rows == 0 || num_columns == 0) return 1;
        if (!ratio_ok(outlier_topk_ratio) || !ratio_ok(error_correction_topk_ratio)) return 1;
        if (!method_ok(svd_uv_format) || !method_ok(svd_s_format) || !method_ok(quantization_only_format)) return 1;
        DeviceSlot *slot = slot_for_current_device();
        if (!slot) return 1;
        std::lock_guard<std::mutex> g(slot->mu);
        slot->decompress.release();
        if (!setup_runtime(slot->decompress, false, num_rows, num_columns, outlier_topk_ratio,
                           error_correction_topk_ratio, svd_ranks, 1, svd_uv_format, svd_s_format,
                           quantization_only_format, BITSQZ_LLM_INPUT_DEVICE)) {
            slot->decompress.release();
            return 1;
        }
        return 0;
    } catch (...) {
        return 1;
    }
}

void bitsqz_llm_decompress_release() {
    try {
        DeviceSlot *slot = slot_for_current_device();
        if (!slot) return;
        std::lock_guard<std::mutex> g(slot->mu);
        slot->decompress.release();
    } catch (...) {
    }
}

// ================================================================================================
// compress
// ================================================================================================
namespace {

// Where the bytes of a packed object go: `base` is the start of the payload, in a pinned host block or in a device
// buffer.  Device-produced bytes are copied there by the stream either way; host-known bytes (section headers) are
// written directly into a host block and travel through the runtime's pinned staging area into a device buffer.
bool put_small(Runtime &rt, const CompressJob &job, uint8_t *dst, const void *src, size_t bytes) {
    if (!job.to_device) {
        std::memcpy(dst, src, bytes);
        return true;
    }
    const size_t need = (bytes + 15) & ~(size_t)15;
    if (rt.stage_used + need > kStageBytes) return false;
    uint8_t *stage = rt.h_stage + rt.stage_used;
    rt.stage_used += need;
    std::memcpy(stage, src, bytes);
    return cudaMemcpyAsync(dst, stage, bytes, cudaMemcpyHostToDevice, rt.stream) == cudaSuccess;
}
bool put_device(Runtime &rt, uint8_t *dst, const void *d_src, size_t bytes) {
    return cudaMemcpyAsync(dst, d_src, bytes, cudaMemcpyDefault, rt.stream) == cudaSuccess;
}

// One quantised section into its final place: the host-known 48-byte header (quantization_cuda.cu:736-807), then
// the scales and nibbles from the device buffers.
bool emit_quant_section(Runtime &rt, const CompressJob &job, const QuantBufs &q, int method, uint8_t *dst) {
    const uint64_t n = q.n, nb = (n + 63) / 64;
    QuantHeader h{};
    h.magic = kQuantMagic;
    h.version = 1;
    h.method = method;
    h.num_elements = n;
    h.num_blocks = nb;
    h.block_size = 64;
    if (!put_small(rt, job, dst, &h, sizeof(h))) return false;
    uint8_t *scales_dst = dst + sizeof(h);
    if (method == NF4) {
        if (!put_device(rt, scales_dst, q.scales_f32.p, nb * 4)) return false;
        scales_dst += nb * 4;
    } else {
        if (!put_device(rt, dst + offsetof(QuantHeader, dq_scale), q.dq.p, 4)) return false;
        if (!put_device(rt, scales_dst, q.scale_codes.p, nb)) return false;
        scales_dst += nb;
    }
    return put_device(rt, scales_dst, q.data.p, (n + 1) / 2);
}

bool emit_topk_section(Runtime &rt, const CompressJob &job, const TopkBufs &t, uint8_t *dst) {
    TopkHeader h{rt.rows, rt.cols, (uint16_t)t.k, 0};
    if (!put_small(rt, job, dst, &h, sizeof(h))) return false;
    const size_t cnt = (size_t)rt.rows * t.k;
    return put_device(rt, dst + 8, t.idx.p, cnt * 2) && put_device(rt, dst + 8 + cnt * 2, t.val.p, cnt * 4);
}

// Quantise `d_src` (n elements) into q; d_deq (nullable, may alias d_src) receives the dequantised values.
bool run_quantize(Runtime &rt, int method, const float *d_src, QuantBufs &q, float *d_deq) {
    cudaError_t err;
    if (method == NF4)
        err = nf4_quantize(d_src, q.n, q.scales_f32.as<float>(), q.data.as<uint8_t>(), d_deq, rt.sm_count, rt.stream);
    else
        err = nf4dq_quantize(d_src, q.n, q.dq.as<float>(), q.scale_codes.as<uint8_t>(), q.data.as<uint8_t>(), d_deq,
                             rt.scratch.p, rt.sm_count, rt.stream);
    return err == cudaSuccess;
}

double ms_between(cudaEvent_t a, cudaEvent_t b) {
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, a, b) != cudaSuccess) { cudaGetLastError(); return 0.0; }
    return (double)ms;
}

// Bytes of the packed object of this runtime's configuration when every planned section is present.
uint64_t plan_sections(const Runtime &rt, CompressJob &job) {
    const uint16_t rows = rt.rows, cols = rt.cols;
    const uint64_t n = (uint64_t)rows * cols;
    const uint32_t ko = rt.outlier.k, ke = rt.err.k, rank = (uint32_t)rt.rank;
    job.has_svd = rt.svd_ranks >= 1;
    uint64_t off = 0;
    auto plan = [&](SectionPlan &s, uint64_t size, uint8_t storage) {
        s.offset = off; s.size = size; s.storage = storage; off += size;
    };
    job.sec_u = job.sec_s = job.sec_v = job.sec_direct = job.sec_out = job.sec_err = SectionPlan{};
    // section order U, S, V | direct, outlier, error; unpadded (src/bitsqz_llm.cu:1237-1277)
    if (job.has_svd) {
        if (rt.uv_format != quantization_NONE) plan(job.sec_u, quant_section_bytes(rt.uv_format, (uint64_t)rows * rank), BITSQZ_SECTION_QUANT);
        else plan(job.sec_u, (uint64_t)rows * rank * 4, BITSQZ_SECTION_FP32);
        if (rt.s_format != quantization_NONE) plan(job.sec_s, quant_section_bytes(rt.s_format, rank), BITSQZ_SECTION_QUANT);
        else plan(job.sec_s, (uint64_t)rank * 4, BITSQZ_SECTION_FP32);
        if (rt.uv_format != quantization_NONE) plan(job.sec_v, quant_section_bytes(rt.uv_format, (uint64_t)cols * rank), BITSQZ_SECTION_QUANT);
        else plan(job.sec_v, (uint64_t)cols * rank * 4, BITSQZ_SECTION_FP32);
    } else if (rt.q_format != quantization_NONE) {
        plan(job.sec_direct, quant_section_bytes(rt.q_format, n), BITSQZ_SECTION_QUANT);
    } else {
        plan(job.sec_direct, n * 4, BITSQZ_SECTION_FP32);
    }
    job.error_path = ke > 0 && (job.has_svd || rt.q_format != quantization_NONE);
    if (ko > 0) plan(job.sec_out, topk_section_bytes(rows, ko), BITSQZ_SECTION_TOPK);
    if (job.error_path) plan(job.sec_err, topk_section_bytes(rows, ke), BITSQZ_SECTION_TOPK);
    return sizeof(bitsqz_llm_array_t) + off;
}

void abandon_job(Runtime &rt) {
    CompressJob &job = rt.job;
    cudaStreamSynchronize(rt.stream);
    cudaGetLastError();
    if (!job.to_device && job.block) {
        if (job.pooled) host_pool().give_back(job.block); else std::free(job.block);
    }
    job = CompressJob{};
}

// Enqueue one compress call on the runtime's stream: staging of a host input, every stage, and the copies of the
// results into their final place.  d_packed == nullptr: the object goes to a pinned host block; otherwise into the
// caller's device buffer of `capacity` bytes.  Returns without waiting; compress_end finishes the call.
int compress_begin(Runtime &rt, const float *x, int input_location, uint8_t *d_packed, uint64_t capacity, bool want_profile) {
    if (rt.job.active || rt.decompress_active) return 1;
    CompressJob &job = rt.job;
    job = CompressJob{};
    job.t_begin = std::chrono::steady_clock::now();
    const uint16_t rows = rt.rows, cols = rt.cols;
    const uint32_t n = (uint32_t)rows * cols;
    const uint32_t ko = rt.outlier.k, ke = rt.err.k;
    const uint32_t rank = (uint32_t)rt.rank;
    cudaStream_t st = rt.stream;
    unsigned *d_status = rt.status.as<unsigned>();      // [0] kernel status bits, [1] error-nonzero flag
    if (input_location == BITSQZ_LLM_INPUT_HOST && !rt.input_stage.p) return 1;

    job.total = plan_sections(rt, job);
    const bool has_svd = job.has_svd, error_path = job.error_path;
    job.to_device = d_packed != nullptr;
    if (job.to_device) {
        if (capacity < job.total) return 1;
        job.block = d_packed;
    } else {
        job.pooled = true;
        job.block = static_cast<uint8_t *>(host_pool().take(job.total));
        if (!job.block) {
            job.pooled = false;
            job.block = static_cast<uint8_t *>(std::malloc(job.total));
            if (!job.block) return 1;
        }
        std::memset(job.block, 0, sizeof(bitsqz_llm_array_t));
    }
    job.active = true;
    rt.stage_used = 0;
    auto fail = [&]() {
        abandon_job(rt);
        return 1;
    };
    uint8_t *payload = job.block + sizeof(bitsqz_llm_array_t);
    job.prof = want_profile;
    auto mark = [&]() { if (job.prof && job.nev < 8) cudaEventRecord(rt.ev[job.nev++], st); };

    if (cudaMemsetAsync(d_status, 0, 64, st) != cudaSuccess) return fail();
    if (rt.inject_status) {                                             // test hook: as if a kernel had reported these bits
        rt.h_status[8] = rt.inject_status;
        rt.inject_status = 0;
        if (cudaMemcpyAsync(d_status, rt.h_status + 8, 4, cudaMemcpyHostToDevice, st) != cudaSuccess) return fail();
    }
    const float *d_input = x;
    if (input_location == BITSQZ_LLM_INPUT_HOST) {
        if (cudaMemcpyAsync(rt.input_stage.p, x, (size_t)n * 4, cudaMemcpyHostToDevice, st) != cudaSuccess) return fail();
        d_input = rt.input_stage.as<float>();
    }
    mark();                                                               // ev0: input staged

    // ---- stages ----
    const float *d_src = d_input;          // what SVD / the quantiser sees (outliers zeroed)
    bool fused_front = false;
    bool residual_bound = false;                                        // d_status[8] holds an upper bound of |residual|
    if (!has_svd && rt.q_format != quantization_NONE && ko > 0 && !error_path && frontend_supported(rows, cols, ko) &&
        (reinterpret_cast<uintptr_t>(d_input) % 16) == 0) {
        fused_front = true;
        if (frontend_quantize(rt.q_format, d_input, rows, cols, ko, rt.outlier.idx.as<uint16_t>(), rt.outlier.val.as<float>(),
                              rt.q_direct.scales_f32.as<float>(), rt.q_direct.dq.as<float>(),
                              rt.q_direct.scale_codes.as<uint8_t>(), rt.q_direct.data.as<uint8_t>(), rt.scratch.p, d_status,
                              rt.sm_count, st) != cudaSuccess)
            return fail();
    } else if (ko > 0) {
        // (the largest k-th |x| bounds what is left in the residual: the SVD's products take their FP16 scale from it)
        if (topk_rows(d_input, rt.residual.as<float>(), rows, cols, ko, rt.outlier.idx.as<uint16_t>(),
                      rt.outlier.val.as<float>(), d_status, rt.sm_count, st, d_status + 8, &residual_bound) != cudaSuccess)
            return fail();
        d_src = rt.residual.as<float>();
    }
    mark();                                                               // ev1: outlier separation done
    if (has_svd) {
        // The random matrix of the range finder is the one the reference's FIRST compress call after initialisation
        // uses: its generator is seeded once, with 1234 (src/bitsqz_llm.cu:841-859), its warm-up run draws the first
        // N_work x k normals of that XORWOW sequence, and its captured graph goes on from there, whatever seed the call
        // passes (:1069-1074) -- so call c works with block c of the sequence, and block 1 is the only one a caller
        // can count on.  Every call here uses block 1: same singular values as that first reference call to ~5e-5
        // relative, and the same object for the same input on every call.
        const unsigned long long omega_offset = (unsigned long long)std::min(rows, cols) * rank;
        if (svd_lowrank(rt.svd, d_src, rt.u.as<float>(), rt.s.as<float>(), rt.v.as<float>(), 1234ULL, d_status, st, omega_offset,
                        residual_bound ? d_status + 8 : nullptr) != cudaSuccess)
            return fail();
        mark(); job.ev_svd = job.nev - 1;
        // quantised factors replace U, S, V in place for the error stage (src/bitsqz_llm.cu:1078-1139)
        if (rt.uv_format != quantization_NONE) {
            if (!run_quantize(rt, rt.uv_format, rt.u.as<float>(), rt.q_u, error_path ? rt.u.as<float>() : nullptr)) return fail();
            if (!run_quantize(rt, rt.uv_format, rt.v.as<float>(), rt.q_v, error_path ? rt.v.as<float>() : nullptr)) return fail();
        }
        if (rt.s_format != quantization_NONE)
            if (!run_quantize(rt, rt.s_format, rt.s.as<float>(), rt.q_s, error_path ? rt.s.as<float>() : nullptr)) return fail();
        mark(); job.ev_quant = job.nev - 1;
        if (error_path) {
            if (reconstruct_lowrank(rt.u.as<float>(), rt.s.as<float>(), rt.v.as<float>(), rows, cols, (int)rank, d_src,
                                    rt.error.as<float>(), d_status + 1, d_status, rt.recon_ws.as<float>(), rt.recon_ws_bytes, rt.sm_count,
                                    st) != cudaSuccess)
                return fail();
            mark(); job.ev_recon = job.nev - 1;
        }
    } else if (rt.q_format != quantization_NONE && !fused_front) {
        if (!run_quantize(rt, rt.q_format, d_src, rt.q_direct, error_path ? rt.recon.as<float>() : nullptr)) return fail();
        mark(); job.ev_quant = job.nev - 1;
        if (error_path)
            if (residual_error(d_src, rt.recon.as<float>(), n, rt.error.as<float>(), d_status + 1, rt.sm_count, st) != cudaSuccess)
                return fail();
    }
    if (error_path) {
        if (topk_rows(rt.error.as<float>(), nullptr, rows, cols, ke, rt.err.idx.as<uint16_t>(), rt.err.val.as<float>(),
                      d_status, rt.sm_count, st) != cudaSuccess)
            return fail();
        mark(); job.ev_err = job.nev - 1;
    }

    // ---- results straight into the object ----
    bool ok = true;
    if (has_svd) {
        const size_t ub = (size_t)rows * rank * 4, sb = (size_t)rank * 4, vb = (size_t)cols * rank * 4;
        // FP32 factors are stored as computed; when they were quantised the device copies now hold
        // the dequantised values and the payload takes the quantised form instead
        if (rt.uv_format != quantization_NONE) ok = ok && emit_quant_section(rt, job, rt.q_u, rt.uv_format, payload + job.sec_u.offset);
        else ok = ok && put_device(rt, payload + job.sec_u.offset, rt.u.p, ub);
        if (rt.s_format != quantization_NONE) ok = ok && emit_quant_section(rt, job, rt.q_s, rt.s_format, payload + job.sec_s.offset);
        else ok = ok && put_device(rt, payload + job.sec_s.offset, rt.s.p, sb);
        if (rt.uv_format != quantization_NONE) ok = ok && emit_quant_section(rt, job, rt.q_v, rt.uv_format, payload + job.sec_v.offset);
        else ok = ok && put_device(rt, payload + job.sec_v.offset, rt.v.p, vb);
    } else if (rt.q_format != quantization_NONE) {
        ok = ok && emit_quant_section(rt, job, rt.q_direct, rt.q_format, payload + job.sec_direct.offset);
    } else {
        ok = ok && put_device(rt, payload + job.sec_direct.offset, d_src, (size_t)n * 4);
    }
    if (ko > 0) ok = ok && emit_topk_section(rt, job, rt.outlier, payload + job.sec_out.offset);
    if (error_path) ok = ok && emit_topk_section(rt, job, rt.err, payload + job.sec_err.offset);
    ok = ok && cudaMemcpyAsync(rt.h_status, d_status, 64, cudaMemcpyDeviceToHost, st) == cudaSuccess;
    mark();                                                               // last event: copies done
    if (!ok) return fail();
    return 0;
}

// Wait for the call begun by compress_begin and finish the object: status check, header (src/bitsqz_llm.cu:1253-1271).
// Host object: *out receives the block.  Device object: the 200-byte header is copied to the front of the caller's
// buffer and into *header_out (nullable), whose `payload` is then a DEVICE pointer.
int compress_end(Runtime &rt, bitsqz_llm_array_t **out, bitsqz_llm_array_t *header_out, uint64_t *packed_size,
                 bitsqz_llm_compress_profile_t *profile) {
    CompressJob &job = rt.job;
    if (!job.active) return 1;
    cudaStream_t st = rt.stream;
    if (cudaStreamSynchronize(st) != cudaSuccess || rt.h_status[0] != 0) {
        abandon_job(rt);
        return 1;
    }
    const bool has_svd = job.has_svd;
    const bool has_error_topk = job.error_path && rt.h_status[1] != 0;      // src/bitsqz_llm.cu:1160-1178
    bitsqz_llm_array_t hdr;
    std::memset(&hdr, 0, sizeof(hdr));
    hdr.num_rows = rt.rows;
    hdr.num_columns = rt.cols;
    hdr.num_elements = (uint32_t)rt.rows * rt.cols;
    hdr.outlier_topk_ratio = rt.outlier_ratio;
    hdr.error_correction_topk_ratio = rt.error_ratio;
    hdr.svd_ranks = (int16_t)rt.svd_ranks;
    hdr.svd_niters = (int16_t)rt.svd_niters;
    hdr.effective_rank = (int16_t)(has_svd ? rt.rank : 0);
    hdr.svd_uv_format = (quantization_method_t)rt.uv_format;
    hdr.svd_s_format = (quantization_method_t)rt.s_format;
    hdr.quantization_only_format = (quantization_method_t)rt.q_format;
    hdr.flags = (has_svd ? kFlagSvd : 0u) | (rt.outlier.k > 0 ? kFlagOutlier : 0u) | (has_error_topk ? kFlagError : 0u);
    auto put = [](bitsqz_section_t &dst, const SectionPlan &s) {
        dst.offset = s.offset; dst.size = s.size; dst.storage = s.storage;
    };
    put(hdr.section_u, job.sec_u);
    put(hdr.section_s, job.sec_s);
    put(hdr.section_v, job.sec_v);
    put(hdr.section_direct, job.sec_direct);
    put(hdr.section_outlier_topk, job.sec_out);
    if (has_error_topk) put(hdr.section_error_topk, job.sec_err);
    hdr.payload = job.block + sizeof(bitsqz_llm_array_t);
    if (job.to_device) {
        std::memcpy(rt.h_stage, &hdr, sizeof(hdr));
        if (cudaMemcpyAsync(job.block, rt.h_stage, sizeof(hdr), cudaMemcpyHostToDevice, st) != cudaSuccess ||
            cudaStreamSynchronize(st) != cudaSuccess) {
            abandon_job(rt);
            return 1;
        }
        if (header_out) *header_out = hdr;
    } else {
        std::memcpy(job.block, &hdr, sizeof(hdr));
        if (out) *out = reinterpret_cast<bitsqz_llm_array_t *>(job.block);
    }
    if (packed_size) *packed_size = bitsqz_llm_get_packed_size(&hdr);

    if (job.prof && profile) {
        // Stage buckets from stream events (stages are not separated by host synchronisation here);
        // fused work is booked under the stage that contains it.
        const double total_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - job.t_begin).count();
        int prev = 1;
        profile->topk_separation_latency_ms = ms_between(rt.ev[0], rt.ev[1]);
        if (job.ev_svd >= 0) { profile->svd_lowrank_cuda_latency_ms = ms_between(rt.ev[prev], rt.ev[job.ev_svd]); prev = job.ev_svd; }
        if (job.ev_quant >= 0) { profile->quantization_compress_latency_ms = ms_between(rt.ev[prev], rt.ev[job.ev_quant]); prev = job.ev_quant; }
        if (job.ev_recon >= 0) { profile->reconstruct_svd_latency_ms = ms_between(rt.ev[prev], rt.ev[job.ev_recon]); prev = job.ev_recon; }
        if (job.ev_err >= 0) { profile->error_extraction_latency_ms = ms_between(rt.ev[prev], rt.ev[job.ev_err]); prev = job.ev_err; }
        const double accounted = profile->topk_separation_latency_ms + profile->svd_lowrank_cuda_latency_ms +
                                 profile->quantization_compress_latency_ms + profile->reconstruct_svd_latency_ms +
                                 profile->error_extraction_latency_ms;
        profile->other_latency_ms = std::max(0.0, total_ms - accounted);
    }
    job = CompressJob{};
    return 0;
}

}  // namespace

int bitsqz_llm_compress(const float *row_major_matrix_float_data, bitsqz_llm_array_t **out,
                        bitsqz_llm_compress_profile_t *profile) {
    try {
        DeviceSlot *slot = slot_for_current_device();
        if (!slot) return 1;
        std::lock_guard<std::mutex> g(slot->mu);
        Runtime &rt = slot->compress;
        if (!rt.initialized) return 1;
        if (!row_major_matrix_float_data || !out || *out) return 1;
        if (profile) *profile = bitsqz_llm_compress_profile_t{};
        if (compress_begin(rt, row_major_matrix_float_data, rt.input_location, nullptr, 0, profile != nullptr) != 0) return 1;
        return compress_end(rt, out, nullptr, nullptr, profile);
    } catch (...) {
        return 1;
    }
}

// ================================================================================================
// decompress, (de)serialisation
// ================================================================================================
namespace {

int section_bounds_ok(const bitsqz_section_t &s, uint64_t payload_size) {        // src/bitsqz_llm.cu:319-332
    if (s.storage == BITSQZ_SECTION_NONE) return s.size == 0;
    if (s.size == 0 || s.offset > payload_size || s.size > payload_size - s.offset) return 0;
    return s.storage == BITSQZ_SECTION_FP32 || s.storage == BITSQZ_SECTION_QUANT || s.storage == BITSQZ_SECTION_TOPK;
}

bool section_method_ok(const bitsqz_section_t &s, int method) {                  // src/bitsqz_llm.cu:617-630
    if (s.storage == BITSQZ_SECTION_NONE) return true;
    if (s.storage == BITSQZ_SECTION_FP32) return method == quantization_NONE;
    if (s.storage == BITSQZ_SECTION_QUANT) return method != quantization_NONE && method_ok(method);
    return false;
}

// The small headers that sit inside the payload, fetched before anything is decided from them: straight reads for a
// host payload, one batch of small device-to-host copies (and one wait) for a device-resident payload.
struct SectionHeads {
    QuantHeader u, s, v, direct;
    TopkHeader outlier, err;
};

bool fetch_heads(Runtime &rt, const bitsqz_llm_array_t *c, bool payload_on_device, SectionHeads *heads) {
    std::memset(heads, 0, sizeof(*heads));
    const uint8_t *payload = static_cast<const uint8_t *>(c->payload);
    struct Want { const bitsqz_section_t *sec; void *dst; size_t bytes; uint8_t storage; };
    const Want wants[6] = {
        {&c->section_u, &heads->u, sizeof(QuantHeader), BITSQZ_SECTION_QUANT},
        {&c->section_s, &heads->s, sizeof(QuantHeader), BITSQZ_SECTION_QUANT},
        {&c->section_v, &heads->v, sizeof(QuantHeader), BITSQZ_SECTION_QUANT},
        {&c->section_direct, &heads->direct, sizeof(QuantHeader), BITSQZ_SECTION_QUANT},
        {&c->section_outlier_topk, &heads->outlier, sizeof(TopkHeader), BITSQZ_SECTION_TOPK},
        {&c->section_error_topk, &heads->err, sizeof(TopkHeader), BITSQZ_SECTION_TOPK},
    };
    size_t used = 0;
    uint8_t *staged[6] = {};
    for (int i = 0; i < 6; ++i) {
        const Want &w = wants[i];
        if (w.sec->storage != w.storage || w.sec->size < w.bytes) continue;     // absent, FP32, or too short (rejected later)
        if (!payload_on_device) {
            std::memcpy(w.dst, payload + w.sec->offset, w.bytes);
            continue;
        }
        staged[i] = rt.h_stage + used;
        used += 64;
        if (cudaMemcpyAsync(staged[i], payload + w.sec->offset, w.bytes, cudaMemcpyDeviceToHost, rt.stream) != cudaSuccess) return false;
    }
    if (payload_on_device) {
        if (cudaStreamSynchronize(rt.stream) != cudaSuccess) return false;
        for (int i = 0; i < 6; ++i)
            if (staged[i]) std::memcpy(wants[i].dst, staged[i], wants[i].bytes);
    }
    return true;
}

// topk_validate_packed_buffer (topk_cuda.cu:271-297) + runtime capacity check (src/bitsqz_llm.cu:632-652)
bool topk_section_ok(const TopkBufs &cap, const bitsqz_llm_array_t *c, const bitsqz_section_t &s, const TopkHeader &h) {
    if (cap.k == 0 || s.size < sizeof(TopkHeader)) return false;
    if (h.num_rows == 0 || h.num_columns == 0 || h.num_topk_columns > h.num_columns) return false;
    if (s.size != topk_section_bytes(h.num_rows, h.num_topk_columns)) return false;
    if (h.num_rows != c->num_rows || h.num_columns != c->num_columns) return false;
    return h.num_topk_columns <= cap.k;
}

// Everything that can be decided from the 200-byte header alone (src/bitsqz_llm.cu:654-761).
bool validate_header(const Runtime &rt, const bitsqz_llm_array_t *c) {
    if (!c->payload || c->num_rows == 0 || c->num_columns == 0 || c->num_elements == 0) return false;
    if (rt.rows != c->num_rows || rt.cols != c->num_columns) return false;
    if (c->num_elements != (uint32_t)c->num_rows * c->num_columns) return false;
    const uint64_t packed = bitsqz_llm_get_packed_size(c);
    if (packed < sizeof(bitsqz_llm_array_t)) return false;
    const uint64_t payload_size = packed - sizeof(bitsqz_llm_array_t);
    const bitsqz_section_t *all[6] = {&c->section_u, &c->section_s, &c->section_v,
                                      &c->section_direct, &c->section_outlier_topk, &c->section_error_topk};
    for (const bitsqz_section_t *s : all)
        if (!section_bounds_ok(*s, payload_size)) return false;
    if (!section_method_ok(c->section_u, c->svd_uv_format) || !section_method_ok(c->section_s, c->svd_s_format) ||
        !section_method_ok(c->section_v, c->svd_uv_format) || !section_method_ok(c->section_direct, c->quantization_only_format))
        return false;
    const bool has_svd = c->flags & kFlagSvd;
    auto present = [](const bitsqz_section_t &s) { return s.storage != BITSQZ_SECTION_NONE; };
    if (has_svd) {
        const uint16_t rank = (uint16_t)c->effective_rank;
        if (rank == 0 || rt.svd_ranks != (int)rank || rt.rank != (int)rank) return false;
        if (!present(c->section_u) || !present(c->section_s) || !present(c->section_v) || present(c->section_direct)) return false;
    } else {
        if (c->effective_rank != 0) return false;
        if (!present(c->section_direct) || present(c->section_u) || present(c->section_s) || present(c->section_v)) return false;
    }
    const bool needs_quant = c->section_u.storage == BITSQZ_SECTION_QUANT || c->section_s.storage == BITSQZ_SECTION_QUANT ||
                             c->section_v.storage == BITSQZ_SECTION_QUANT || c->section_direct.storage == BITSQZ_SECTION_QUANT;
    if (needs_quant && !rt.uses_quant) return false;
    if (c->flags & kFlagOutlier) {
        if (c->section_outlier_topk.storage != BITSQZ_SECTION_TOPK) return false;
    } else if (present(c->section_outlier_topk)) {
        return false;
    }
    if (c->flags & kFlagError) {
        if (c->section_error_topk.storage != BITSQZ_SECTION_TOPK) return false;
    } else if (present(c->section_error_topk)) {
        return false;
    }
    return true;
}

// Checks of one quantised section against its 48-byte header (quantization_cuda.cu:691-734,809-876); uploads its
// scales and nibbles into the runtime's aligned buffers.
bool upload_quant(Runtime &rt, const bitsqz_llm_array_t *c, const bitsqz_section_t &s, const QuantHeader &h, int method,
                  uint64_t expected_count, QuantBufs *q) {
    if (s.storage != BITSQZ_SECTION_QUANT || method == quantization_NONE || !q || q->cap < expected_count) return false;
    q->n = expected_count;
    if (s.size < sizeof(QuantHeader)) return false;
    const uint64_t nb = (expected_count + 63) / 64;
    if (h.magic != kQuantMagic || h.version != 1 || h.method != method || h.num_elements != expected_count ||
        h.block_size != 64 || h.num_blocks != nb || s.size != quant_section_bytes(method, expected_count))
        return false;
    const uint8_t *src = static_cast<const uint8_t *>(c->payload) + s.offset;
    const uint8_t *scales = src + sizeof(QuantHeader);
    cudaStream_t st = rt.stream;
    if (method == NF4) {
        return cudaMemcpyAsync(q->scales_f32.p, scales, nb * 4, cudaMemcpyDefault, st) == cudaSuccess &&
               cudaMemcpyAsync(q->data.p, scales + nb * 4, (expected_count + 1) / 2, cudaMemcpyDefault, st) == cudaSuccess;
    }
    return cudaMemcpyAsync(q->dq.p, src + offsetof(QuantHeader, dq_scale), 4, cudaMemcpyDefault, st) == cudaSuccess &&
           cudaMemcpyAsync(q->scale_codes.p, scales, nb, cudaMemcpyDefault, st) == cudaSuccess &&
           cudaMemcpyAsync(q->data.p, scales + nb, (expected_count + 1) / 2, cudaMemcpyDefault, st) == cudaSuccess;
}

// One section -> `d_out` (expected_count floats).  FP32: plain copy.  QUANT: upload, then the dequantise kernel.
bool decode_section(Runtime &rt, const bitsqz_llm_array_t *c, const bitsqz_section_t &s, const QuantHeader &h, int method,
                    uint64_t expected_count, QuantBufs *q, float *d_out) {
    const uint8_t *src = static_cast<const uint8_t *>(c->payload) + s.offset;
    if (s.storage == BITSQZ_SECTION_FP32) {
        if (s.size != expected_count * 4) return false;
        return cudaMemcpyAsync(d_out, src, s.size, cudaMemcpyDefault, rt.stream) == cudaSuccess;
    }
    if (!upload_quant(rt, c, s, h, method, expected_count, q)) return false;
    if (method == NF4)
        return nf4_dequantize(q->scales_f32.as<float>(), q->data.as<uint8_t>(), expected_count, d_out, rt.sm_count, rt.stream) == cudaSuccess;
    return nf4dq_dequantize(q->dq.as<float>(), q->scale_codes.as<uint8_t>(), q->data.as<uint8_t>(), expected_count, d_out,
                            rt.sm_count, rt.stream) == cudaSuccess;
}

bool upload_topk(Runtime &rt, const bitsqz_llm_array_t *c, const bitsqz_section_t &s, const TopkHeader &h, TopkBufs &bufs) {
    const uint8_t *src = static_cast<const uint8_t *>(c->payload) + s.offset;
    const size_t cnt = (size_t)h.num_rows * h.num_topk_columns;
    if (cnt == 0) return true;
    return cudaMemcpyAsync(bufs.idx.p, src + 8, cnt * 2, cudaMemcpyDefault, rt.stream) == cudaSuccess &&
           cudaMemcpyAsync(bufs.val.p, src + 8 + cnt * 2, cnt * 4, cudaMemcpyDefault, rt.stream) == cudaSuccess;
}

bool apply_topk_section(Runtime &rt, const bitsqz_llm_array_t *c, const bitsqz_section_t &s, const TopkHeader &h, TopkBufs &bufs,
                        float *d_dst) {
    if ((size_t)h.num_rows * h.num_topk_columns == 0) return true;
    if (!upload_topk(rt, c, s, h, bufs)) return false;
    return topk_apply(bufs.idx.as<uint16_t>(), bufs.val.as<float>(), h.num_rows, h.num_columns, h.num_topk_columns, d_dst,
                      rt.status.as<unsigned>(), rt.stream) == cudaSuccess;
}

// Enqueue one decompress call (src/bitsqz_llm.cu:1304-1393).  `c` is the 200-byte header in host memory; its payload
// pointer may be host memory (the reference's objects) or, with payload_on_device, device memory.
int decompress_begin(Runtime &rt, const bitsqz_llm_array_t *c, bool payload_on_device, float *d_dst) {
    if (rt.decompress_active || rt.job.active) return 1;
    if (!validate_header(rt, c)) return 1;
    cudaStream_t st = rt.stream;
    auto fail = [&]() {
        cudaStreamSynchronize(st);
        cudaGetLastError();
        return 1;
    };
    SectionHeads heads;
    if (!fetch_heads(rt, c, payload_on_device, &heads)) return fail();
    const bool has_out = c->flags & kFlagOutlier, has_err = c->flags & kFlagError;
    if (has_out && !topk_section_ok(rt.outlier, c, c->section_outlier_topk, heads.outlier)) return 1;
    if (has_err && !topk_section_ok(rt.err, c, c->section_error_topk, heads.err)) return 1;
    if (cudaMemsetAsync(rt.status.p, 0, 64, st) != cudaSuccess) return fail();
    if (rt.inject_status) {
        rt.h_status[8] = rt.inject_status;
        rt.inject_status = 0;
        if (cudaMemcpyAsync(rt.status.p, rt.h_status + 8, 4, cudaMemcpyHostToDevice, st) != cudaSuccess) return fail();
    }
    unsigned *d_status = rt.status.as<unsigned>();
    bool lists_done = false;
    if (c->flags & kFlagSvd) {
        const uint32_t rank = (uint16_t)c->effective_rank;
        if (!decode_section(rt, c, c->section_u, heads.u, c->svd_uv_format, (uint64_t)c->num_rows * rank, &rt.q_direct, rt.u.as<float>())) return fail();
        if (!decode_section(rt, c, c->section_s, heads.s, c->svd_s_format, rank, &rt.q_direct, rt.s.as<float>())) return fail();
        if (!decode_section(rt, c, c->section_v, heads.v, c->svd_uv_format, (uint64_t)c->num_columns * rank, &rt.q_direct, rt.v.as<float>())) return fail();
        if (reconstruct_lowrank(rt.u.as<float>(), rt.s.as<float>(), rt.v.as<float>(), c->num_rows, c->num_columns, (int)rank,
                                nullptr, d_dst, nullptr, d_status, rt.recon_ws.as<float>(), rt.recon_ws_bytes, rt.sm_count, st) != cudaSuccess)
            return fail();
    } else if (c->section_direct.storage == BITSQZ_SECTION_QUANT && (has_out != has_err)) {
        // quantised matrix with exactly one list: dequantise and add the list in one pass over the output
        // (with one list the reference's order "error list first, outliers second" has nothing to order)
        const TopkHeader &th = has_out ? heads.outlier : heads.err;
        TopkBufs &tb = has_out ? rt.outlier : rt.err;
        const bitsqz_section_t &ts = has_out ? c->section_outlier_topk : c->section_error_topk;
        const int method = c->quantization_only_format;
        if (!upload_quant(rt, c, c->section_direct, heads.direct, method, c->num_elements, &rt.q_direct)) return fail();
        if ((size_t)th.num_rows * th.num_topk_columns == 0) {
            if (!decode_section(rt, c, c->section_direct, heads.direct, method, c->num_elements, &rt.q_direct, d_dst)) return fail();
        } else {
            if (!upload_topk(rt, c, ts, th, tb)) return fail();
            QuantBufs &q = rt.q_direct;
            if (nf4_dequantize_add_topk(method == NF4 ? q.scales_f32.as<float>() : nullptr, method == NF4 ? nullptr : q.dq.as<float>(),
                                        method == NF4 ? nullptr : q.scale_codes.as<uint8_t>(), q.data.as<uint8_t>(), c->num_rows,
                                        c->num_columns, tb.idx.as<uint16_t>(), tb.val.as<float>(), th.num_topk_columns, d_dst,
                                        d_status, rt.sm_count, st) != cudaSuccess)
                return fail();
        }
        lists_done = true;
    } else {
        if (!decode_section(rt, c, c->section_direct, heads.direct, c->quantization_only_format, c->num_elements, &rt.q_direct, d_dst)) return fail();
    }
    if (!lists_done) {
        // error first, outliers second (src/bitsqz_llm.cu:1372-1387)
        if (has_err && !apply_topk_section(rt, c, c->section_error_topk, heads.err, rt.err, d_dst)) return fail();
        if (has_out && !apply_topk_section(rt, c, c->section_outlier_topk, heads.outlier, rt.outlier, d_dst)) return fail();
    }
    if (cudaMemcpyAsync(rt.h_status, rt.status.p, 64, cudaMemcpyDeviceToHost, st) != cudaSuccess) return fail();
    rt.decompress_active = true;
    return 0;
}

int decompress_end(Runtime &rt) {
    if (!rt.decompress_active) return 1;
    rt.decompress_active = false;
    if (cudaStreamSynchronize(rt.stream) != cudaSuccess) {
        cudaGetLastError();
        return 1;
    }
    return rt.h_status[0] == 0 ? 0 : 1;
}

}  // namespace

int bitsqz_llm_decompress(const bitsqz_llm_array_t *compressed, float *d_dst, uint32_t dst_num_elements) {
    try {
        DeviceSlot *slot = slot_for_current_device();
        if (!slot) return 1;
        std::lock_guard<std::mutex> g(slot->mu);
        Runtime &rt = slot->decompress;
        if (!rt.initialized) return 1;
        if (!compressed || !d_dst || !compressed->payload) return 1;
        if (dst_num_elements < compressed->num_elements) return 1;
        if (decompress_begin(rt, compressed, false, d_dst) != 0) return 1;
        return decompress_end(rt);
    } catch (...) {
        return 1;
    }
}

uint64_t bitsqz_llm_get_packed_size(const bitsqz_llm_array_t *compressed) {
    if (!compressed) return 0;
    const bitsqz_section_t *all[6] = {&compressed->section_u, &compressed->section_s, &compressed->section_v,
                                      &compressed->section_direct, &compressed->section_outlier_topk,
                                      &compressed->section_error_topk};
    uint64_t payload = 0;
    for (const bitsqz_section_t *s : all) {
        if (s->storage == BITSQZ_SECTION_NONE) continue;
        payload = std::max(payload, s->offset + s->size);
    }
    return sizeof(bitsqz_llm_array_t) + payload;
}

// The loaded copy lives in a page-locked pool block when one can be had (plain heap memory otherwise), so that
// bitsqz_llm_decompress uploads its sections at full PCIe speed without a staging copy inside the driver.
bitsqz_llm_array_t *load_bitsqz_llm_from_buffer(const void *buffer, uint64_t buffer_size) {
    if (!buffer || buffer_size < sizeof(bitsqz_llm_array_t)) return nullptr;
    bool pooled = true;
    bitsqz_llm_array_t *c = static_cast<bitsqz_llm_array_t *>(host_pool().take((size_t)buffer_size));
    if (!c) {
        pooled = false;
        c = static_cast<bitsqz_llm_array_t *>(std::malloc((size_t)buffer_size));
        if (!c) return nullptr;
    }
    std::memcpy(c, buffer, (size_t)buffer_size);
    c->payload = reinterpret_cast<uint8_t *>(c) + sizeof(bitsqz_llm_array_t);
    const uint64_t packed = bitsqz_llm_get_packed_size(c);
    bool ok = packed != 0 && buffer_size >= packed;
    if (ok) {
        const uint64_t payload_size = packed - sizeof(bitsqz_llm_array_t);
        const bitsqz_section_t *all[6] = {&c->section_u, &c->section_s, &c->section_v,
                                          &c->section_direct, &c->section_outlier_topk, &c->section_error_topk};
        for (const bitsqz_section_t *s : all) ok = ok && section_bounds_ok(*s, payload_size);
    }
    if (!ok) {
        if (pooled) host_pool().give_back(c); else std::free(c);
        return nullptr;
    }
    return c;
}

void bitsqz_llm_free(bitsqz_llm_array_t *compressed) {
    if (!compressed) return;
    if (!host_pool().give_back(compressed)) std::free(compressed);
}

// The reference's integration tests and walkthrough also call this helper of its top-k module
// (modules/topk_cuda/include/topk_cuda.cuh:47, topk_cuda.cu:53-69); exported under the same C++ name so that they
// link against this library unchanged.
uint16_t topk_compute_num_topk_columns(uint16_t num_columns, float topk_ratio) {
    return (uint16_t)bsq::topk_num_columns(num_columns, topk_ratio);
}

// ================================================================================================
// lanes and batches (include/bitsqz_llm_c.h): several independent matrices in flight on one device
// ================================================================================================
// A lane is a compress runtime and a decompress runtime of one configuration with a stream of their own.  Its calls
// come in two halves: "begin" enqueues everything and returns, "end" waits for the lane's stream and finishes the
// result.  Work begun on different lanes overlaps on the GPU: the host-to-device copy of one matrix, the tensor-core
// products of a second and the few-SM stages (k x k factorisations) of a third.  A batch is a set of lanes that a
// list of matrices is dealt over in turn.
struct bsq_lane {
    int device = 0;
    Runtime compress, decompress;
};

namespace {

bool lane_setup(bsq_lane *lane, uint16_t rows, uint16_t cols, float outlier, float error, int svd_ranks, int svd_niters, int uv,
                int s, int q) {
    if (rows == 0 || cols == 0 || !ratio_ok(outlier) || !ratio_ok(error) || !method_ok(uv) || !method_ok(s) || !method_ok(q) ||
        svd_niters < 1)
        return false;
    if (cudaGetDevice(&lane->device) != cudaSuccess) return false;
    // a lane takes host and device inputs alike: its compress runtime always has the staging buffer of a host input
    if (!setup_runtime(lane->compress, true, rows, cols, outlier, error, svd_ranks, svd_niters, uv, s, q, BITSQZ_LLM_INPUT_HOST))
        return false;
    const int eff_rank = lane->compress.rank;          // decompress demands exactly the effective rank
    return setup_runtime(lane->decompress, false, rows, cols, outlier, error, svd_ranks >= 1 ? eff_rank : svd_ranks, 1, uv, s, q,
                         BITSQZ_LLM_INPUT_DEVICE);
}

}  // namespace

extern "C" {

bsq_lane *bsq_lane_create(uint16_t rows, uint16_t cols, float outlier_topk_ratio, float error_correction_topk_ratio,
                          int svd_ranks, int svd_niters, int svd_uv_format, int svd_s_format, int quantization_only_format) {
    try {
        bsq_lane *lane = new bsq_lane();
        if (!lane_setup(lane, rows, cols, outlier_topk_ratio, error_correction_topk_ratio, svd_ranks, svd_niters, svd_uv_format,
                        svd_s_format, quantization_only_format)) {
            lane->compress.release();
            lane->decompress.release();
            delete lane;
            cudaGetLastError();
            return nullptr;
        }
        return lane;
    } catch (...) {
        return nullptr;
    }
}

void bsq_lane_destroy(bsq_lane *lane) {
    if (!lane) return;
    try {
        lane->compress.release();
        lane->decompress.release();
        delete lane;
    } catch (...) {
    }
}

uint64_t bsq_lane_packed_capacity(bsq_lane *lane) {
    if (!lane) return 0;
    CompressJob tmp;
    return plan_sections(lane->compress, tmp);
}

void *bsq_lane_stream(bsq_lane *lane, int decompress_side) {
    if (!lane) return nullptr;
    return decompress_side ? lane->decompress.stream : lane->compress.stream;
}

int bsq_lane_compress_begin(bsq_lane *lane, const float *matrix, int input_location, void *d_packed, uint64_t capacity) {
    try {
        if (!lane || !matrix) return 1;
        if (input_location != BITSQZ_LLM_INPUT_HOST && input_location != BITSQZ_LLM_INPUT_DEVICE) return 1;
        return compress_begin(lane->compress, matrix, input_location, static_cast<uint8_t *>(d_packed), capacity, false);
    } catch (...) {
        return 1;
    }
}

int bsq_lane_compress_end(bsq_lane *lane, struct bitsqz_llm_array **out, struct bitsqz_llm_array *device_header, uint64_t *packed_size) {
    try {
        if (!lane || !lane->compress.job.active) return 1;
        if (!lane->compress.job.to_device && (!out || *out)) {
            abandon_job(lane->compress);
            return 1;
        }
        return compress_end(lane->compress, out, device_header, packed_size, nullptr);
    } catch (...) {
        return 1;
    }
}

int bsq_lane_decompress_begin(bsq_lane *lane, const struct bitsqz_llm_array *header, int payload_on_device, float *d_dst,
                              uint64_t dst_num_elements) {
    try {
        if (!lane || !header || !d_dst || !header->payload) return 1;
        if (dst_num_elements < header->num_elements) return 1;
        return decompress_begin(lane->decompress, header, payload_on_device != 0, d_dst);
    } catch (...) {
        return 1;
    }
}

int bsq_lane_profile(bsq_lane *lane, int on) {
    if (!lane || !lane->compress.svd) return 1;
    return svd_workspace_profile(lane->compress.svd, on != 0) == cudaSuccess ? 0 : 1;
}

int bsq_lane_profile_read(bsq_lane *lane, float *ms, int *kinds, int capacity) {
    if (!lane || !lane->compress.svd || capacity < 0) return 0;
    return svd_workspace_spans(lane->compress.svd, ms, kinds, capacity);
}

int bsq_lane_decompress_end(bsq_lane *lane) {
    try {
        if (!lane) return 1;
        return decompress_end(lane->decompress);
    } catch (...) {
        return 1;
    }
}

// Test hook: the next compress (which = 0) or decompress (which = 1) call on this device's runtimes of the public
// interface starts with `bits` already set in its status word, as if a kernel had reported them.
void bsq_test_inject_status(int which, uint32_t bits) {
    DeviceSlot *slot = slot_for_current_device();
    if (!slot) return;
    std::lock_guard<std::mutex> g(slot->mu);
    (which ? slot->decompress : slot->compress).inject_status = bits;
}

}  // extern "C"

struct bsq_batch {
    std::vector<bsq_lane *> lanes;
};

extern "C" {

bsq_batch *bsq_batch_create(uint16_t rows, uint16_t cols, float outlier_topk_ratio, float error_correction_topk_ratio, int svd_ranks,
                            int svd_niters, int svd_uv_format, int svd_s_format, int quantization_only_format, int lanes) {
    try {
        if (lanes < 1 || lanes > 16) return nullptr;
        bsq_batch *b = new bsq_batch();
        for (int i = 0; i < lanes; ++i) {
            bsq_lane *lane = bsq_lane_create(rows, cols, outlier_topk_ratio, error_correction_topk_ratio, svd_ranks, svd_niters,
                                             svd_uv_format, svd_s_format, quantization_only_format);
            if (!lane) {
                for (bsq_lane *l : b->lanes) bsq_lane_destroy(l);
                delete b;
                return nullptr;
            }
            b->lanes.push_back(lane);
        }
        return b;
    } catch (...) {
        return nullptr;
    }
}

void bsq_batch_destroy(bsq_batch *b) {
    if (!b) return;
    for (bsq_lane *l : b->lanes) bsq_lane_destroy(l);
    delete b;
}

int bsq_batch_lanes(bsq_batch *b) { return b ? (int)b->lanes.size() : 0; }
bsq_lane *bsq_batch_lane(bsq_batch *b, int i) { return (b && i >= 0 && i < (int)b->lanes.size()) ? b->lanes[i] : nullptr; }

// Matrix i runs on lane i % lanes; a lane's previous matrix is finished just before its next one is begun, so up to
// `lanes` matrices are in flight.  On failure every lane is drained, the objects made so far are released and the
// output arrays are left null.
int bsq_batch_compress(bsq_batch *b, const float *const *matrices, int count, int input_location, void *const *d_packed,
                       uint64_t capacity, struct bitsqz_llm_array **outs, struct bitsqz_llm_array *device_headers,
                       uint64_t *packed_sizes) {
    if (!b || !matrices || count < 0) return 1;
    const bool to_device = d_packed != nullptr;
    if (!to_device && !outs) return 1;
    const int L = (int)b->lanes.size();
    int rc = 0;
    if (!to_device)
        for (int i = 0; i < count; ++i) outs[i] = nullptr;
    auto finish = [&](int i) {
        bsq_lane *lane = b->lanes[i % L];
        return bsq_lane_compress_end(lane, to_device ? nullptr : &outs[i], (to_device && device_headers) ? &device_headers[i] : nullptr,
                                     packed_sizes ? &packed_sizes[i] : nullptr);
    };
    int begun = 0;
    for (int i = 0; i < count && rc == 0; ++i) {
        if (i >= L) rc |= finish(i - L);
        if (rc == 0) {
            rc |= bsq_lane_compress_begin(b->lanes[i % L], matrices[i], input_location, to_device ? d_packed[i] : nullptr, capacity);
            if (rc == 0) begun = i + 1;
        }
    }
    for (int i = std::max(0, begun - L); i < begun; ++i) {
        if (b->lanes[i % L]->compress.job.active) rc |= finish(i);
    }
    if (rc != 0 && !to_device) {
        for (int i = 0; i < count; ++i) {
            if (outs[i]) bitsqz_llm_free(outs[i]);
            outs[i] = nullptr;
        }
    }
    return rc ? 1 : 0;
}

int bsq_batch_decompress(bsq_batch *b, const struct bitsqz_llm_array *const *headers, int count, int payload_on_device,
                         float *const *d_dsts, uint64_t dst_num_elements) {
    if (!b || !headers || !d_dsts || count < 0) return 1;
    const int L = (int)b->lanes.size();
    int rc = 0, begun = 0;
    for (int i = 0; i < count && rc == 0; ++i) {
        if (i >= L) rc |= bsq_lane_decompress_end(b->lanes[i % L]);
        if (rc == 0) {
            rc |= bsq_lane_decompress_begin(b->lanes[i % L], headers[i], payload_on_device, d_dsts[i], dst_num_elements);
            if (rc == 0) begun = i + 1;
        }
    }
    for (int i = std::max(0, begun - L); i < begun; ++i)
        if (b->lanes[i % L]->decompress.decompress_active) rc |= bsq_lane_decompress_end(b->lanes[i % L]);
    return rc ? 1 : 0;
}

}  // extern "C"
