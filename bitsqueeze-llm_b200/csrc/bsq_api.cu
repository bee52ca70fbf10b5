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

  private:
    static size_t round_up(size_t b) { return (b + (1u << 16) - 1) & ~(size_t)((1u << 16) - 1); }
    static constexpr size_t kCacheLimit = (size_t)2 << 30;
    std::mutex mu_;
    std::unordered_map<size_t, std::vector<void *>> free_;
    std::unordered_map<void *, size_t> live_;
    size_t cached_ = 0;
};
HostPool &host_pool() {
    static HostPool *pool = new HostPool();      // never destroyed: blocks may outlive static teardown
    return *pool;
}

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
    DevBuf input_stage, residual, recon, error, u, s, v, scratch, status;
    QuantBufs q_direct, q_u, q_s, q_v;
    TopkBufs outlier, err;
    SvdWorkspace *svd = nullptr;
    unsigned *h_status = nullptr;                        // pinned mirror of the device status words

    void release() {
        if (stream) cudaStreamSynchronize(stream);
        input_stage.release(); residual.release(); recon.release(); error.release();
        u.release(); s.release(); v.release(); scratch.release(); status.release();
        q_direct.release(); q_u.release(); q_s.release(); q_v.release();
        outlier.release(); err.release();
        if (svd) { svd_workspace_destroy(svd); svd = nullptr; }
        for (auto &e : ev) { if (e) cudaEventDestroy(e); e = nullptr; }
        if (h_status) { cudaFreeHost(h_status); h_status = nullptr; }
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
        std::lock_guard<std::mutex> g(slot->mu);
        slot->compress.release();
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

struct SectionPlan {
    uint64_t offset = 0, size = 0;
    uint8_t storage = BITSQZ_SECTION_NONE;
};

// Enqueue the device-to-host copies of one quantised section into its final place and write the
// host-known part of its 48-byte header (quantization_cuda.cu:736-807).
bool emit_quant_section(const Runtime &rt, const QuantBufs &q, int method, uint8_t *dst) {
    const uint64_t n = q.n, nb = (n + 63) / 64;
    QuantHeader h{};
    h.magic = kQuantMagic;
    h.version = 1;
    h.method = method;
    h.num_elements = n;
    h.num_blocks = nb;
    h.block_size = 64;
    std::memcpy(dst, &h, sizeof(h));
    uint8_t *scales_dst = dst + sizeof(h);
    cudaError_t err;
    if (method == NF4) {
        err = cudaMemcpyAsync(scales_dst, q.scales_f32.p, nb * 4, cudaMemcpyDeviceToHost, rt.stream);
        if (err != cudaSuccess) return false;
        scales_dst += nb * 4;
    } else {
        err = cudaMemcpyAsync(dst + offsetof(QuantHeader, dq_scale), q.dq.p, 4, cudaMemcpyDeviceToHost, rt.stream);
        if (err != cudaSuccess) return false;
        err = cudaMemcpyAsync(scales_dst, q.scale_codes.p, nb, cudaMemcpyDeviceToHost, rt.stream);
        if (err != cudaSuccess) return false;
        scales_dst += nb;
    }
    return cudaMemcpyAsync(scales_dst, q.data.p, (n + 1) / 2, cudaMemcpyDeviceToHost, rt.stream) == cudaSuccess;
}

bool emit_topk_section(const Runtime &rt, const TopkBufs &t, uint8_t *dst) {
    TopkHeader h{rt.rows, rt.cols, (uint16_t)t.k, 0};
    std::memcpy(dst, &h, sizeof(h));
    const size_t cnt = (size_t)rt.rows * t.k;
    if (cudaMemcpyAsync(dst + 8, t.idx.p, cnt * 2, cudaMemcpyDeviceToHost, rt.stream) != cudaSuccess) return false;
    return cudaMemcpyAsync(dst + 8 + cnt * 2, t.val.p, cnt * 4, cudaMemcpyDeviceToHost, rt.stream) == cudaSuccess;
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

int compress_locked(Runtime &rt, const float *x, bitsqz_llm_array_t **out, bitsqz_llm_compress_profile_t *profile) {
    using Clock = std::chrono::steady_clock;
    const auto t_begin = Clock::now();
    const uint16_t rows = rt.rows, cols = rt.cols;
    const uint32_t n = (uint32_t)rows * cols;
    const uint32_t ko = rt.outlier.k, ke = rt.err.k;
    const bool has_svd = rt.svd_ranks >= 1;
    const uint32_t rank = (uint32_t)rt.rank;
    cudaStream_t st = rt.stream;
    unsigned *d_status = rt.status.as<unsigned>();      // [0] kernel status bits, [1] error-nonzero flag

    // ---- plan the payload (section order U, S, V | direct, outlier, error; unpadded) ----
    SectionPlan sec_u, sec_s, sec_v, sec_direct, sec_out, sec_err;
    uint64_t off = 0;
    auto plan = [&](SectionPlan &s, uint64_t size, uint8_t storage) {
        s.offset = off; s.size = size; s.storage = storage; off += size;
    };
    if (has_svd) {
        if (rt.uv_format != quantization_NONE) plan(sec_u, quant_section_bytes(rt.uv_format, (uint64_t)rows * rank), BITSQZ_SECTION_QUANT);
        else plan(sec_u, (uint64_t)rows * rank * 4, BITSQZ_SECTION_FP32);
        if (rt.s_format != quantization_NONE) plan(sec_s, quant_section_bytes(rt.s_format, rank), BITSQZ_SECTION_QUANT);
        else plan(sec_s, (uint64_t)rank * 4, BITSQZ_SECTION_FP32);
        if (rt.uv_format != quantization_NONE) plan(sec_v, quant_section_bytes(rt.uv_format, (uint64_t)cols * rank), BITSQZ_SECTION_QUANT);
        else plan(sec_v, (uint64_t)cols * rank * 4, BITSQZ_SECTION_FP32);
    } else if (rt.q_format != quantization_NONE) {
        plan(sec_direct, quant_section_bytes(rt.q_format, n), BITSQZ_SECTION_QUANT);
    } else {
        plan(sec_direct, (uint64_t)n * 4, BITSQZ_SECTION_FP32);
    }
    const bool error_path = ke > 0 && (has_svd || rt.q_format != quantization_NONE);
    if (ko > 0) plan(sec_out, topk_section_bytes(rows, ko), BITSQZ_SECTION_TOPK);
    if (error_path) plan(sec_err, topk_section_bytes(rows, ke), BITSQZ_SECTION_TOPK);
    const uint64_t total = sizeof(bitsqz_llm_array_t) + off;

    bool pooled = true;
    uint8_t *block = static_cast<uint8_t *>(host_pool().take(total));
    if (!block) {
        pooled = false;
        block = static_cast<uint8_t *>(std::malloc(total));
        if (!block) return 1;
    }
    auto fail = [&]() {
        cudaStreamSynchronize(st);
        cudaGetLastError();
        if (pooled) host_pool().give_back(block); else std::free(block);
        return 1;
    };
    std::memset(block, 0, sizeof(bitsqz_llm_array_t));
    uint8_t *payload = block + sizeof(bitsqz_llm_array_t);
    const bool prof = profile != nullptr;
    int nev = 0;
    auto mark = [&]() { if (prof && nev < 8) cudaEventRecord(rt.ev[nev++], st); };

    if (cudaMemsetAsync(d_status, 0, 64, st) != cudaSuccess) return fail();
    const float *d_input = x;
    if (rt.input_location == BITSQZ_LLM_INPUT_HOST) {
        if (cudaMemcpyAsync(rt.input_stage.p, x, (size_t)n * 4, cudaMemcpyHostToDevice, st) != cudaSuccess) return fail();
        d_input = rt.input_stage.as<float>();
    }
    mark();                                                               // ev0: input staged

    // ---- stages ----
    const float *d_src = d_input;          // what SVD / the quantiser sees (outliers zeroed)
    bool fused_front = false;
    if (!has_svd && rt.q_format != quantization_NONE && ko > 0 && !error_path && frontend_supported(rows, cols, ko) &&
        (reinterpret_cast<uintptr_t>(d_input) % 16) == 0) {
        fused_front = true;
        if (frontend_quantize(rt.q_format, d_input, rows, cols, ko, rt.outlier.idx.as<uint16_t>(), rt.outlier.val.as<float>(),
                              rt.q_direct.scales_f32.as<float>(), rt.q_direct.dq.as<float>(),
                              rt.q_direct.scale_codes.as<uint8_t>(), rt.q_direct.data.as<uint8_t>(), rt.scratch.p, d_status,
                              rt.sm_count, st) != cudaSuccess)
            return fail();
    } else if (ko > 0) {
        if (topk_rows(d_input, rt.residual.as<float>(), rows, cols, ko, rt.outlier.idx.as<uint16_t>(),
                      rt.outlier.val.as<float>(), d_status, rt.sm_count, st) != cudaSuccess)
            return fail();
        d_src = rt.residual.as<float>();
    }
    mark();                                                               // ev1: outlier separation done
    int ev_svd = -1, ev_quant = -1, ev_recon = -1, ev_err = -1;
    if (has_svd) {
        if (svd_lowrank(rt.svd, d_src, rt.u.as<float>(), rt.s.as<float>(), rt.v.as<float>(), 1241ULL, d_status, st) != cudaSuccess)
            return fail();
        mark(); ev_svd = nev - 1;
        // quantised factors replace U, S, V in place for the error stage (src/bitsqz_llm.cu:1078-1139)
        if (rt.uv_format != quantization_NONE) {
            if (!run_quantize(rt, rt.uv_format, rt.u.as<float>(), rt.q_u, error_path ? rt.u.as<float>() : nullptr)) return fail();
            if (!run_quantize(rt, rt.uv_format, rt.v.as<float>(), rt.q_v, error_path ? rt.v.as<float>() : nullptr)) return fail();
        }
        if (rt.s_format != quantization_NONE)
            if (!run_quantize(rt, rt.s_format, rt.s.as<float>(), rt.q_s, error_path ? rt.s.as<float>() : nullptr)) return fail();
        mark(); ev_quant = nev - 1;
        if (error_path) {
            if (reconstruct_lowrank(rt.u.as<float>(), rt.s.as<float>(), rt.v.as<float>(), rows, cols, (int)rank, d_src,
                                    rt.error.as<float>(), d_status + 1, rt.sm_count, st) != cudaSuccess)
                return fail();
            mark(); ev_recon = nev - 1;
        }
    } else if (rt.q_format != quantization_NONE && !fused_front) {
        if (!run_quantize(rt, rt.q_format, d_src, rt.q_direct, error_path ? rt.recon.as<float>() : nullptr)) return fail();
        mark(); ev_quant = nev - 1;
        if (error_path)
            if (residual_error(d_src, rt.recon.as<float>(), n, rt.error.as<float>(), d_status + 1, rt.sm_count, st) != cudaSuccess)
                return fail();
    }
    if (error_path) {
        if (topk_rows(rt.error.as<float>(), nullptr, rows, cols, ke, rt.err.idx.as<uint16_t>(), rt.err.val.as<float>(),
                      d_status, rt.sm_count, st) != cudaSuccess)
            return fail();
        mark(); ev_err = nev - 1;
    }

    // ---- results straight into the returned block ----
    bool ok = true;
    if (has_svd) {
        const size_t ub = (size_t)rows * rank * 4, sb = (size_t)rank * 4, vb = (size_t)cols * rank * 4;
        // FP32 factors are stored as computed; when they were quantised the device copies now hold
        // the dequantised values and the payload takes the quantised form instead
        if (rt.uv_format != quantization_NONE) ok = ok && emit_quant_section(rt, rt.q_u, rt.uv_format, payload + sec_u.offset);
        else ok = ok && cudaMemcpyAsync(payload + sec_u.offset, rt.u.p, ub, cudaMemcpyDeviceToHost, st) == cudaSuccess;
        if (rt.s_format != quantization_NONE) ok = ok && emit_quant_section(rt, rt.q_s, rt.s_format, payload + sec_s.offset);
        else ok = ok && cudaMemcpyAsync(payload + sec_s.offset, rt.s.p, sb, cudaMemcpyDeviceToHost, st) == cudaSuccess;
        if (rt.uv_format != quantization_NONE) ok = ok && emit_quant_section(rt, rt.q_v, rt.uv_format, payload + sec_v.offset);
        else ok = ok && cudaMemcpyAsync(payload + sec_v.offset, rt.v.p, vb, cudaMemcpyDeviceToHost, st) == cudaSuccess;
    } else if (rt.q_format != quantization_NONE) {
        ok = ok && emit_quant_section(rt, rt.q_direct, rt.q_format, payload + sec_direct.offset);
    } else {
        ok = ok && cudaMemcpyAsync(payload + sec_direct.offset, d_src, (size_t)n * 4, cudaMemcpyDeviceToHost, st) == cudaSuccess;
    }
    if (ko > 0) ok = ok && emit_topk_section(rt, rt.outlier, payload + sec_out.offset);
    if (error_path) ok = ok && emit_topk_section(rt, rt.err, payload + sec_err.offset);
    ok = ok && cudaMemcpyAsync(rt.h_status, d_status, 64, cudaMemcpyDeviceToHost, st) == cudaSuccess;
    mark();                                                               // last event: copies done
    if (!ok) return fail();
    if (cudaStreamSynchronize(st) != cudaSuccess) return fail();
    if (rt.h_status[0] != 0) return fail();
    const bool has_error_topk = error_path && rt.h_status[1] != 0;      // src/bitsqz_llm.cu:1160-1178

    // ---- header (src/bitsqz_llm.cu:1253-1271) ----
    bitsqz_llm_array_t *arr = reinterpret_cast<bitsqz_llm_array_t *>(block);
    arr->num_rows = rows;
    arr->num_columns = cols;
    arr->num_elements = n;
    arr->outlier_topk_ratio = rt.outlier_ratio;
    arr->error_correction_topk_ratio = rt.error_ratio;
    arr->svd_ranks = (int16_t)rt.svd_ranks;
    arr->svd_niters = (int16_t)rt.svd_niters;
    arr->effective_rank = (int16_t)(has_svd ? rank : 0);
    arr->svd_uv_format = (quantization_method_t)rt.uv_format;
    arr->svd_s_format = (quantization_method_t)rt.s_format;
    arr->quantization_only_format = (quantization_method_t)rt.q_format;
    arr->flags = (has_svd ? kFlagSvd : 0u) | (ko > 0 ? kFlagOutlier : 0u) | (has_error_topk ? kFlagError : 0u);
    auto put = [](bitsqz_section_t &dst, const SectionPlan &s) {
        dst.offset = s.offset; dst.size = s.size; dst.storage = s.storage;
    };
    put(arr->section_u, sec_u);
    put(arr->section_s, sec_s);
    put(arr->section_v, sec_v);
    put(arr->section_direct, sec_direct);
    put(arr->section_outlier_topk, sec_out);
    if (has_error_topk) put(arr->section_error_topk, sec_err);
    arr->payload = payload;
    *out = arr;

    if (prof) {
        // Stage buckets from stream events (stages are not separated by host synchronisation here);
        // fused work is booked under the stage that contains it.
        const double total_ms = std::chrono::duration<double, std::milli>(Clock::now() - t_begin).count();
        int prev = 1;
        profile->topk_separation_latency_ms = ms_between(rt.ev[0], rt.ev[1]);
        if (ev_svd >= 0) { profile->svd_lowrank_cuda_latency_ms = ms_between(rt.ev[prev], rt.ev[ev_svd]); prev = ev_svd; }
        if (ev_quant >= 0) { profile->quantization_compress_latency_ms = ms_between(rt.ev[prev], rt.ev[ev_quant]); prev = ev_quant; }
        if (ev_recon >= 0) { profile->reconstruct_svd_latency_ms = ms_between(rt.ev[prev], rt.ev[ev_recon]); prev = ev_recon; }
        if (ev_err >= 0) { profile->error_extraction_latency_ms = ms_between(rt.ev[prev], rt.ev[ev_err]); prev = ev_err; }
        const double accounted = profile->topk_separation_latency_ms + profile->svd_lowrank_cuda_latency_ms +
                                 profile->quantization_compress_latency_ms + profile->reconstruct_svd_latency_ms +
                                 profile->error_extraction_latency_ms;
        profile->other_latency_ms = std::max(0.0, total_ms - accounted);
    }
    return 0;
}

}  // namespace

int bitsqz_llm_compress(const float *row_major_matrix_float_data, bitsqz_llm_array_t **out,
                        bitsqz_llm_compress_profile_t *profile) {
    try {
        DeviceSlot *slot = slot_for_current_device();
        if (!slot) return 1;
        std::lock_guard<std::mutex> g(slot->mu);
        if (!slot->compress.initialized) return 1;
        if (!row_major_matrix_float_data || !out || *out) return 1;
        if (profile) *profile = bitsqz_llm_compress_profile_t{};
        return compress_locked(slot->compress, row_major_matrix_float_data, out, profile);
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

// topk_validate_packed_buffer (topk_cuda.cu:271-297) + runtime capacity check (src/bitsqz_llm.cu:632-652)
bool topk_section_ok(const Runtime &rt, const TopkBufs &cap, const bitsqz_llm_array_t *c, const bitsqz_section_t &s,
                     TopkHeader *hdr) {
    if (cap.k == 0 || s.size < sizeof(TopkHeader)) return false;
    TopkHeader h;
    std::memcpy(&h, static_cast<const uint8_t *>(c->payload) + s.offset, sizeof(h));
    if (h.num_rows == 0 || h.num_columns == 0 || h.num_topk_columns > h.num_columns) return false;
    if (s.size != topk_section_bytes(h.num_rows, h.num_topk_columns)) return false;
    if (h.num_rows != c->num_rows || h.num_columns != c->num_columns) return false;
    if (h.num_topk_columns > cap.k) return false;
    (void)rt;
    *hdr = h;
    return true;
}

bool validate_for_decompress(const Runtime &rt, const bitsqz_llm_array_t *c) {   // src/bitsqz_llm.cu:654-761
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
    TopkHeader h;
    if (c->flags & kFlagOutlier) {
        if (c->section_outlier_topk.storage != BITSQZ_SECTION_TOPK || !topk_section_ok(rt, rt.outlier, c, c->section_outlier_topk, &h))
            return false;
    } else if (present(c->section_outlier_topk)) {
        return false;
    }
    if (c->flags & kFlagError) {
        if (c->section_error_topk.storage != BITSQZ_SECTION_TOPK || !topk_section_ok(rt, rt.err, c, c->section_error_topk, &h))
            return false;
    } else if (present(c->section_error_topk)) {
        return false;
    }
    return true;
}

// One section -> `d_out` (expected_count floats).  FP32: plain copy.  QUANT: header check
// (quantization_cuda.cu:691-734,809-876), copy of scales and nibbles, dequantise kernel.
bool decode_section(Runtime &rt, const bitsqz_llm_array_t *c, const bitsqz_section_t &s, int method, uint64_t expected_count,
                    QuantBufs *q, float *d_out) {
    const uint8_t *src = static_cast<const uint8_t *>(c->payload) + s.offset;
    if (s.storage == BITSQZ_SECTION_FP32) {
        if (s.size != expected_count * 4) return false;
        return cudaMemcpyAsync(d_out, src, s.size, cudaMemcpyHostToDevice, rt.stream) == cudaSuccess;
    }
    if (s.storage != BITSQZ_SECTION_QUANT || method == quantization_NONE || !q || q->cap < expected_count) return false;
    q->n = expected_count;
    if (s.size < sizeof(QuantHeader)) return false;
    QuantHeader h;
    std::memcpy(&h, src, sizeof(h));
    const uint64_t nb = (expected_count + 63) / 64;
    if (h.magic != kQuantMagic || h.version != 1 || h.method != method || h.num_elements != expected_count ||
        h.block_size != 64 || h.num_blocks != nb || s.size != quant_section_bytes(method, expected_count))
        return false;
    const uint8_t *scales = src + sizeof(h);
    if (method == NF4) {
        if (cudaMemcpyAsync(q->scales_f32.p, scales, nb * 4, cudaMemcpyHostToDevice, rt.stream) != cudaSuccess) return false;
        if (cudaMemcpyAsync(q->data.p, scales + nb * 4, (expected_count + 1) / 2, cudaMemcpyHostToDevice, rt.stream) != cudaSuccess) return false;
        return nf4_dequantize(q->scales_f32.as<float>(), q->data.as<uint8_t>(), expected_count, d_out, rt.sm_count, rt.stream) == cudaSuccess;
    }
    if (cudaMemcpyAsync(q->dq.p, src + offsetof(QuantHeader, dq_scale), 4, cudaMemcpyHostToDevice, rt.stream) != cudaSuccess) return false;
    if (cudaMemcpyAsync(q->scale_codes.p, scales, nb, cudaMemcpyHostToDevice, rt.stream) != cudaSuccess) return false;
    if (cudaMemcpyAsync(q->data.p, scales + nb, (expected_count + 1) / 2, cudaMemcpyHostToDevice, rt.stream) != cudaSuccess) return false;
    return nf4dq_dequantize(q->dq.as<float>(), q->scale_codes.as<uint8_t>(), q->data.as<uint8_t>(), expected_count, d_out,
                            rt.sm_count, rt.stream) == cudaSuccess;
}

bool apply_topk_section(Runtime &rt, const bitsqz_llm_array_t *c, const bitsqz_section_t &s, TopkBufs &bufs, float *d_dst) {
    const uint8_t *src = static_cast<const uint8_t *>(c->payload) + s.offset;
    TopkHeader h;
    std::memcpy(&h, src, sizeof(h));
    const size_t cnt = (size_t)h.num_rows * h.num_topk_columns;
    if (cnt == 0) return true;
    if (cudaMemcpyAsync(bufs.idx.p, src + 8, cnt * 2, cudaMemcpyHostToDevice, rt.stream) != cudaSuccess) return false;
    if (cudaMemcpyAsync(bufs.val.p, src + 8 + cnt * 2, cnt * 4, cudaMemcpyHostToDevice, rt.stream) != cudaSuccess) return false;
    return topk_apply(bufs.idx.as<uint16_t>(), bufs.val.as<float>(), h.num_rows, h.num_columns, h.num_topk_columns, d_dst,
                      rt.status.as<unsigned>(), rt.stream) == cudaSuccess;
}

int decompress_locked(Runtime &rt, const bitsqz_llm_array_t *c, float *d_dst) {
    if (!validate_for_decompress(rt, c)) return 1;
    cudaStream_t st = rt.stream;
    auto fail = [&]() {
        cudaStreamSynchronize(st);
        cudaGetLastError();
        return 1;
    };
    if (cudaMemsetAsync(rt.status.p, 0, 64, st) != cudaSuccess) return fail();
    if (c->flags & kFlagSvd) {
        const uint32_t rank = (uint16_t)c->effective_rank;
        if (!decode_section(rt, c, c->section_u, c->svd_uv_format, (uint64_t)c->num_rows * rank, &rt.q_direct, rt.u.as<float>())) return fail();
        if (!decode_section(rt, c, c->section_s, c->svd_s_format, rank, &rt.q_direct, rt.s.as<float>())) return fail();
        if (!decode_section(rt, c, c->section_v, c->svd_uv_format, (uint64_t)c->num_columns * rank, &rt.q_direct, rt.v.as<float>())) return fail();
        if (reconstruct_lowrank(rt.u.as<float>(), rt.s.as<float>(), rt.v.as<float>(), c->num_rows, c->num_columns, (int)rank,
                                nullptr, d_dst, nullptr, rt.sm_count, st) != cudaSuccess)
            return fail();
    } else {
        if (!decode_section(rt, c, c->section_direct, c->quantization_only_format, c->num_elements, &rt.q_direct, d_dst)) return fail();
    }
    // error first, outliers second (src/bitsqz_llm.cu:1372-1387)
    if ((c->flags & kFlagError) && !apply_topk_section(rt, c, c->section_error_topk, rt.err, d_dst)) return fail();
    if ((c->flags & kFlagOutlier) && !apply_topk_section(rt, c, c->section_outlier_topk, rt.outlier, d_dst)) return fail();
    if (cudaMemcpyAsync(rt.h_status, rt.status.p, 64, cudaMemcpyDeviceToHost, st) != cudaSuccess) return fail();
    if (cudaStreamSynchronize(st) != cudaSuccess) return fail();
    return rt.h_status[0] == 0 ? 0 : 1;
}

}  // namespace

int bitsqz_llm_decompress(const bitsqz_llm_array_t *compressed, float *d_dst, uint32_t dst_num_elements) {
    try {
        DeviceSlot *slot = slot_for_current_device();
        if (!slot) return 1;
        std::lock_guard<std::mutex> g(slot->mu);
        if (!slot->decompress.initialized) return 1;
        if (!compressed || !d_dst || !compressed->payload) return 1;
        if (dst_num_elements < compressed->num_elements) return 1;
        return decompress_locked(slot->decompress, compressed, d_dst);
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

bitsqz_llm_array_t *load_bitsqz_llm_from_buffer(const void *buffer, uint64_t buffer_size) {
    if (!buffer || buffer_size < sizeof(bitsqz_llm_array_t)) return nullptr;
    bitsqz_llm_array_t *c = static_cast<bitsqz_llm_array_t *>(std::calloc(1, (size_t)buffer_size));
    if (!c) return nullptr;
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
        std::free(c);
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
