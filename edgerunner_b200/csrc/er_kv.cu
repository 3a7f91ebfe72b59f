// Host side of the C ABI declared in include/er_kv.h: the KV cache object (device slabs, ring /
// block-table bookkeeping, scratch) and the launch code of every kernel.  The cache mirrors the public
// surface of the reference's KVCache (Sources/EdgeRunnerMetal/KVCache.swift:12-1138); storage layout and
// kernels are this library's own.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <chrono>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/er_kv.h"
#include "append.cuh"
#include "er_common.cuh"
#include "launchers.h"
#include "prefill.cuh"
#include "q8.cuh"
#include "turboquant.cuh"
#include "turboquant_outlier.cuh"
#include "turboquant_outlier_cache.cuh"

using namespace er;

namespace {

thread_local std::string g_last_error;
std::atomic<uint64_t> g_launches{0};

int32_t fail(int32_t code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

#define ER_CUDA(expr)                                                                              \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess) return fail(ER_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

inline int32_t check_launch(const char* what) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ER_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return ER_OK;
}

// inv_freq[pair] = 1.0f / powr(theta, float(2*pair)/float(headDim))   (Shaders/RoPE.metal:83-84),
// powr evaluated through double and rounded once.
template <typename TABLE>
void fill_inv_freq(TABLE& t, int capacity, float theta, uint32_t head_dim) {
    const uint32_t half = head_dim / 2;
    for (uint32_t d = 0; d < static_cast<uint32_t>(capacity); ++d) {
        if (d < half) {
            const float exponent = static_cast<float>(2u * d) / static_cast<float>(head_dim);
            const float pw = static_cast<float>(std::pow(static_cast<double>(theta), static_cast<double>(exponent)));
            t.f[d] = 1.0f / pw;
        } else {
            t.f[d] = 0.f;
        }
    }
}

// Scratch shared by the raw-buffer operators (no cache object): one per device, created on first use.
struct Workspace {
    int device = -1;
    int num_sms = 0;
    float* scratch = nullptr;
    int* counters = nullptr;   // [0] done counter, [1] status, [16..] item counters
    size_t counter_ints = 0;
};

constexpr int kMaxDevices = 64;
std::mutex g_ws_mu;
Workspace g_ws[kMaxDevices];   // one per device ordinal; never moves, so returned pointers stay valid

constexpr size_t kScratchFloatsPerCta = 2 * 8 * 130;   // two slots, up to 8 q heads per kv head

int32_t make_workspace(Workspace& w, int device, size_t item_counters) {
    w.device = device;
    ER_CUDA(cudaDeviceGetAttribute(&w.num_sms, cudaDevAttrMultiProcessorCount, device));
    ER_CUDA(cudaMalloc(&w.scratch, sizeof(float) * kScratchFloatsPerCta * w.num_sms));
    w.counter_ints = 16 + item_counters;
    ER_CUDA(cudaMalloc(&w.counters, sizeof(int) * w.counter_ints));
    ER_CUDA(cudaMemset(w.counters, 0, sizeof(int) * w.counter_ints));
    return ER_OK;
}

int32_t get_workspace(Workspace** out) {
    int device = 0;
    ER_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return fail(ER_ERR_UNSUPPORTED, "device ordinal %d beyond %d", device, kMaxDevices - 1);
    std::lock_guard<std::mutex> lock(g_ws_mu);
    Workspace& w = g_ws[device];
    if (w.device != device) {
        Workspace fresh;
        int32_t rc = make_workspace(fresh, device, static_cast<size_t>(kMaxPairs) * 16);
        if (rc != ER_OK) {
            cudaFree(fresh.scratch); cudaFree(fresh.counters); cudaGetLastError();
            return rc;
        }
        w = fresh;
    }
    *out = &w;
    return ER_OK;
}

// The raw-buffer operators read q with 16-byte loads and copy K / V rows with bulk copies that need 16-byte global
// addresses: a misaligned sub-buffer is refused here instead of faulting on the device.
int32_t check_raw_pointers(const void* q, const void* k, const void* v, const void* out) {
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out)) & 15u)
        return fail(ER_ERR_INVALID_ARGUMENT, "q, k, v and out must be 16-byte aligned device addresses");
    return ER_OK;
}

int32_t decode_status(int rc, int group, int kbits, int vbits) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (rc == 0) return ER_OK;
    if (rc == kNotBuilt)
        return fail(ER_ERR_UNSUPPORTED, "decode kernel for GQA group %d (key bits %d, value bits %d) is not built; groups 1, 2, 4, 8 and presets turbo2/turbo3/turbo4 are",
                    group, kbits, vbits);
    return fail(ER_ERR_CUDA, "flash_decode_kernel: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
}

// Chunked prefill: the tcgen05 kernel when the chunk fills at least one 128-row CTA tile and the layout is covered, else
// the mma.sync kernel; force_legacy (er_kv_config.prefill_kernel == ER_PREFILL_KERNEL_MMA_SYNC) always takes the latter.
int launch_prefill(int group, const PrefillParams& pp, uint64_t outer_extent, int num_kv_heads, int* status, cudaStream_t stream,
                   bool force_legacy = false) {
    if (!force_legacy && status != nullptr && static_cast<int64_t>(pp.seq_len) * group >= 128) {
        const int rc = launch_prefill_umma(group, pp, outer_extent, num_kv_heads, status, stream);
        if (rc != kNotBuilt) return rc;
    }
    return launch_prefill_f16(group, pp, num_kv_heads, stream);
}

int32_t dispatch_decode_f16(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    return decode_status(launch_decode_dense(group, p, grid, stream), group, 16, 16);
}

}  // namespace

namespace er {
// Hooks for the library's other translation units.
int32_t report_error(int32_t code, const char* message) { return fail(code, "%s", message); }
void count_kernel_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
}  // namespace er

// ------------------------------------------------------------------------------------------------ cache object

struct er_kv {
    er_kv_config cfg{};
    int device = 0;
    int num_sms = 0;
    bool turbo = false;
    int elem_bytes = 0;           // dense element size
    int k_row_bytes = 0;          // bytes of one (token, kv head) row
    int v_row_bytes = 0;
    int norm_bytes = 0;           // TurboQuant: bytes of one stored norm
    int page_tokens = 0;          // tokens per page (HEAD_MAJOR: padded ring length)
    int pool_pages = 0;           // pages per layer
    int pages_per_seq = 0;        // block-table stride (0 = identity addressing)
    bool token_major = false;
    bool q8 = false;              // q8_0 rows: int8 part in the K / V slabs, four fp16 scales per row in the side slabs
    bool outlier = false;         // balanced / aggressive TurboQuant rows: codes + mask + signs + two norms in one block per row
    OutlierFormat ofmt{};
    float* d_simt_partial = nullptr;   // split partials of the SIMT decode kernel
    float* d_prefill_partial = nullptr;   // partial rows of the tcgen05 prefill kernel's split tail tiles
    size_t simt_partial_floats = 0;
    uint8_t* k_slab = nullptr;
    uint8_t* v_slab = nullptr;
    uint8_t* kn_slab = nullptr;
    uint8_t* vn_slab = nullptr;
    int64_t k_layer_stride = 0, v_layer_stride = 0, n_layer_stride = 0;
    int32_t* d_lengths = nullptr;          // [layers][batch] tokens written (device copy is authoritative)
    std::vector<int32_t> h_lengths;
    int32_t* d_block_table = nullptr;
    std::vector<int32_t> h_block_table;    // [batch][pages_per_seq], -1 = unassigned
    std::vector<uint32_t> h_block_count;
    float* d_scratch = nullptr;
    int* d_counters = nullptr;             // [0] done, [1] status, [16..] item counters
    uint8_t* d_stage = nullptr;            // staging for host-facing calls
    size_t stage_bytes = 0;
    float* d_head_norm[2] = {nullptr, nullptr};   // normalised copies of a call's q and k rows (er_step_params norm weights)
    size_t head_norm_floats[2] = {0, 0};
    float cached_theta = 0.f;
    InvFreqTable inv_freq{};
    uint32_t out_heads_total = 0;            // er_kv_set_output_sharding: 0 = outputs are [layers][batch][num_heads][128]
    uint32_t out_head_offset = 0;
    uint32_t num_peers = 0;
    float* peer_out[8] = {};
    uint32_t probe_wait_limit_us = 0;        // er_kv_debug_wait_probe: patience of the next decode launches' waits
    int probe_withhold_tiles = 0;
    int* h_status = nullptr;                 // pinned, device-mapped host words: [0] the device status copied by er_kv_decode_step_host;
                                             // [2], [3] = {epoch, status} written by the last CTA of a host-buffer decode launch
    int* d_host_done = nullptr;              // device alias of h_status + 2 (nullptr: memory not mapped)
    int host_epoch = 0;
    const float* hostio_q = nullptr;         // set by er_kv_decode_step_host around its launch: the step's rows in mapped host memory
    const float* hostio_k = nullptr;
    const float* hostio_v = nullptr;
    bool hostio_used = false;                // the launch took the rows from there and will signal h_status[2]
    unsigned long long* d_trace = nullptr;   // caller-owned diagnostics buffer (er_kv_set_trace)
    uint32_t trace_ctas = 0;
    std::mutex mu;

    KVAddressing addressing() const {
        KVAddressing a;
        a.token_major = token_major ? 1 : 0;
        a.num_kv_heads = static_cast<int>(cfg.num_kv_heads);
        a.max_seq_len = static_cast<int>(cfg.max_seq_len);
        a.page_size = page_tokens;
        a.pages_per_seq = pages_per_seq;
        a.block_table = d_block_table;
        a.status = pages_per_seq > 0 ? d_counters + 1 : nullptr;
        return a;
    }
    const InvFreqTable& freq(float theta) {
        if (theta != cached_theta) {
            fill_inv_freq(inv_freq, kHalfDim, theta, cfg.head_dim);
            cached_theta = theta;
        }
        return inv_freq;
    }
};

namespace {

int32_t ensure_stage(er_kv* kv, size_t bytes) {
    if (kv->stage_bytes >= bytes) return ER_OK;
    if (kv->d_stage) cudaFree(kv->d_stage);
    kv->d_stage = nullptr;
    kv->stage_bytes = 0;
    size_t want = std::max<size_t>(bytes, 1 << 20);
    if (cudaMalloc(&kv->d_stage, want) != cudaSuccess) {
        cudaGetLastError();
        return fail(ER_ERR_ALLOCATION_FAILED, "staging buffer of %zu bytes", want);
    }
    kv->stage_bytes = want;
    return ER_OK;
}

int32_t pull_lengths(er_kv* kv) {
    ER_CUDA(cudaMemcpy(kv->h_lengths.data(), kv->d_lengths, kv->h_lengths.size() * sizeof(int32_t),
                       cudaMemcpyDeviceToHost));
    return ER_OK;
}
int32_t push_lengths(er_kv* kv) {
    ER_CUDA(cudaMemcpy(kv->d_lengths, kv->h_lengths.data(), kv->h_lengths.size() * sizeof(int32_t),
                       cudaMemcpyHostToDevice));
    return ER_OK;
}

int32_t check_layers(const er_kv* kv, uint32_t b, uint32_t e) {
    if (b >= e || e > kv->cfg.num_layers) return fail(ER_ERR_INVALID_LAYER, "layer range [%u, %u) of %u", b, e, kv->cfg.num_layers);
    return ER_OK;
}

// Every launch of a cache's kernels must go to the GPU that holds its slabs: with another device current the launch
// would carry foreign pointers (a fault, or peer loads where peer access is on).
int32_t check_device(const er_kv* kv) {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess) { cudaGetLastError(); return fail(ER_ERR_CUDA, "cudaGetDevice"); }
    if (device != kv->device)
        return fail(ER_ERR_INVALID_ARGUMENT, "cache lives on device %d but device %d is current", kv->device, device);
    return ER_OK;
}

// Paged layout: rows [0, end_row) of `seq` must lie in pages the block table has been given (host copy; kv->mu held).
int32_t check_page_coverage(const er_kv* kv, uint32_t seq, uint64_t end_row) {
    if (kv->pages_per_seq == 0) return ER_OK;
    const uint64_t need = std::min<uint64_t>(end_row, kv->cfg.max_seq_len);
    const uint64_t have = static_cast<uint64_t>(kv->h_block_count[seq]) * static_cast<uint64_t>(kv->page_tokens);
    if (need > have)
        return fail(ER_ERR_OUT_OF_PAGES, "sequence %u needs pages for %llu rows but its block table covers %llu", seq,
                    static_cast<unsigned long long>(need), static_cast<unsigned long long>(have));
    return ER_OK;
}

int32_t device_status_to_code(int status) {
    if (status == kStatusTimeout) return fail(ER_ERR_DEVICE_TIMEOUT, "a bounded wait inside a kernel gave up");
    if (status == kStatusOutOfPages) return fail(ER_ERR_OUT_OF_PAGES, "a row fell into a block-table entry without a page (the row was dropped)");
    if (status == kStatusBadLayout) return fail(ER_ERR_UNSUPPORTED, "a decode kernel could not place its tables in this device's shared-memory window");
    return status == 0 ? ER_OK : fail(ER_ERR_CUDA, "device status word %d", status);
}

bool is_dense(const er_kv* kv) { return kv->cfg.precision == ER_KV_FLOAT32 || kv->cfg.precision == ER_KV_FLOAT16; }

int32_t step_defaults(const er_kv* kv, const er_step_params* in, er_step_params& out) {
    if (in) out = *in; else { std::memset(&out, 0, sizeof(out)); out.rope_theta = 10000.f; }
    if (out.rope_scaling == 0.f) out.rope_scaling = 1.f;
    if (out.softmax_scale == 0.f) out.softmax_scale = 1.0f / std::sqrt(static_cast<float>(kv->cfg.head_dim));
    if (out.apply_rope && !(out.rope_theta > 0.f)) return fail(ER_ERR_INVALID_ARGUMENT, "rope_theta must be > 0");
    if (out.rms_eps == 0.f) out.rms_eps = 1e-6f;
    return ER_OK;
}

// Per-head RMS norm of `rows` head rows (rows_per_group consecutive rows share the weight vector of one layer) into the
// cache's scratch slot `which` (0 = queries, 1 = keys); *rows_io is replaced by the normalised copy.  No-op for a null
// weight pointer.
int32_t apply_head_norm(er_kv* kv, int which, const float** rows_io, size_t rows, size_t rows_per_group, const float* weight,
                        uint32_t first_group, const er_step_params& s, cudaStream_t stream) {
    if (weight == nullptr || rows == 0) return ER_OK;
    if (kv->cfg.head_dim != kHeadDim) return fail(ER_ERR_UNSUPPORTED, "head norm is built for head_dim 128");
    {
        std::lock_guard<std::mutex> lock(kv->mu);
        const size_t need = rows * kHeadDim;
        if (kv->head_norm_floats[which] < need) {
            if (kv->d_head_norm[which]) cudaFree(kv->d_head_norm[which]);
            kv->d_head_norm[which] = nullptr;
            kv->head_norm_floats[which] = 0;
            if (cudaMalloc(&kv->d_head_norm[which], need * sizeof(float)) != cudaSuccess) {
                cudaGetLastError();
                return fail(ER_ERR_ALLOCATION_FAILED, "head-norm scratch of %zu floats", need);
            }
            kv->head_norm_floats[which] = need;
        }
    }
    HeadNormParams hp{};
    hp.in = *rows_io; hp.out = kv->d_head_norm[which];
    hp.weight = weight + static_cast<size_t>(first_group) * s.norm_weight_layer_stride;
    hp.rows = static_cast<int>(rows); hp.rows_per_group = static_cast<int>(rows_per_group);
    hp.weight_stride = static_cast<int>(s.norm_weight_layer_stride);
    hp.eps = s.rms_eps;
    head_rms_norm_kernel<<<static_cast<unsigned>(std::min<size_t>((rows + 7) / 8, 4096)), 256, 0, stream>>>(hp);
    *rows_io = kv->d_head_norm[which];
    return check_launch("head_rms_norm_kernel");
}

int32_t launch_append(er_kv* kv, AppendParams& ap, cudaStream_t stream) {
    ap.k_base = kv->k_slab;
    ap.v_base = kv->v_slab;
    ap.k_layer_stride_bytes = kv->k_layer_stride;
    ap.v_layer_stride_bytes = kv->v_layer_stride;
    ap.addr = kv->addressing();
    if (ap.rows <= 0) return ER_OK;
    if (kv->turbo) {
        TurboAppendParams tp;
        tp.base = ap;
        tp.kn_base = kv->kn_slab;
        tp.vn_base = kv->vn_slab;
        tp.n_layer_stride_bytes = kv->n_layer_stride;
        tp.norm_fp16 = kv->cfg.norm_format == ER_TQ_NORM_FLOAT16;
        return launch_turbo_append(tp, static_cast<int>(kv->cfg.key_type), static_cast<int>(kv->cfg.value_type), stream,
                                   check_launch);
    }
    if (kv->outlier) {
        OutlierAppendParams op;
        op.base = ap;
        op.fmt = kv->ofmt;
        op.k_use_benefit = kv->cfg.key_type == ER_TQ_SELECT_QUANTIZATION_BENEFIT ? 1 : 0;                 // default: magnitude
        op.v_use_benefit = kv->cfg.value_type == ER_TQ_SELECT_MAGNITUDE ? 0 : 1;                          // default: benefit
        const int64_t jobs = 2 * static_cast<int64_t>(ap.rows) * kv->cfg.num_kv_heads;
        const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((jobs + kOutlierWarps - 1) / kOutlierWarps, 1 << 16));
        tq_outlier_append_kernel<<<blocks, kOutlierWarps * 32, 0, stream>>>(op);
        return check_launch("tq_outlier_append_kernel");
    }
    if (kv->q8) {
        Q8AppendParams qp;
        qp.base = ap;
        qp.ks_base = kv->kn_slab;
        qp.vs_base = kv->vn_slab;
        qp.s_layer_stride_bytes = kv->n_layer_stride;
        const int64_t jobs = 2 * static_cast<int64_t>(ap.rows) * kv->cfg.num_kv_heads;
        q8_append_kernel<<<static_cast<unsigned>((jobs + 7) / 8), 256, 0, stream>>>(qp);
        return check_launch("q8_append_kernel");
    }
    if (kv->cfg.precision == ER_KV_FLOAT16)
        append_rope_dense_kernel<__half><<<ap.rows, 128, 0, stream>>>(ap);
    else
        append_rope_dense_kernel<float><<<ap.rows, 128, 0, stream>>>(ap);
    return check_launch("append_rope_dense_kernel");
}

}  // namespace

extern "C" {

const char* er_status_string(int32_t s) {
    switch (s) {
        case ER_OK: return "ok";
        case ER_ERR_ALLOCATION_FAILED: return "allocationFailed";
        case ER_ERR_INVALID_LAYER: return "invalidLayer";
        case ER_ERR_PRECISION_MISMATCH: return "precisionMismatch";
        case ER_ERR_UNSUPPORTED_STORAGE: return "unsupportedStorage";
        case ER_ERR_COMPRESSED_RETRIEVE_REQUIRES_DECODED_API: return "compressedRetrieveRequiresDecodedAPI";
        case ER_ERR_COMPRESSED_BUFFER_ACCESS_REQUIRES_TURBOQUANT_API: return "compressedBufferAccessRequiresTurboQuantAPI";
        case ER_ERR_SHAPE: return "shape";
        case ER_ERR_CUDA: return "cuda";
        case ER_ERR_INVALID_ARGUMENT: return "invalidArgument";
        case ER_ERR_OUT_OF_PAGES: return "outOfPages";
        case ER_ERR_UNSUPPORTED: return "unsupported";
        case ER_ERR_DEVICE_TIMEOUT: return "deviceTimeout";
        default: return "unknown";
    }
}

const char* er_last_error_string(void) { return g_last_error.c_str(); }

int32_t er_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

uint64_t er_kernel_launch_count(void) { return g_launches.load(); }

int32_t er_host_alloc(void** out, size_t bytes) {
    if (!out) return fail(ER_ERR_INVALID_ARGUMENT, "null out");
    ER_CUDA(cudaHostAlloc(out, bytes, cudaHostAllocDefault));
    return ER_OK;
}
int32_t er_host_free(void* ptr) {
    ER_CUDA(cudaFreeHost(ptr));
    return ER_OK;
}

int32_t er_kv_create(const er_kv_config* c, er_kv** out) {
    if (!c || !out) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    if (c->max_seq_len == 0 || c->num_layers == 0 || c->num_kv_heads == 0 || c->head_dim == 0)
        return fail(ER_ERR_SHAPE, "zero-sized cache dimension");
    switch (c->precision) {
        case ER_KV_FLOAT32: case ER_KV_FLOAT16: case ER_KV_TURBOQUANT_V2: case ER_KV_Q8_0:
        case ER_KV_TURBOQUANT_BALANCED: case ER_KV_TURBOQUANT_AGGRESSIVE: break;
        case ER_KV_FLOAT8:
            return fail(ER_ERR_UNSUPPORTED_STORAGE, "precision %u is outside this backend's scope", c->precision);
        default: return fail(ER_ERR_INVALID_ARGUMENT, "unknown precision %u", c->precision);
    }
    if (c->prefill_kernel > ER_PREFILL_KERNEL_MMA_SYNC) return fail(ER_ERR_INVALID_ARGUMENT, "unknown prefill_kernel %u", c->prefill_kernel);
    if (c->decode_kernel > ER_DECODE_KERNEL_SIMT) return fail(ER_ERR_INVALID_ARGUMENT, "unknown decode_kernel %u", c->decode_kernel);
    if (er_device_count() <= 0) return fail(ER_ERR_CUDA, "no CUDA device: this backend has no CPU fallback");
    er_kv* kv = new er_kv();
    kv->cfg = *c;
    if (kv->cfg.max_batch == 0) kv->cfg.max_batch = 1;
    if (static_cast<uint64_t>(kv->cfg.num_layers) * kv->cfg.max_batch > 1u << 20) { delete kv; return fail(ER_ERR_SHAPE, "layers*batch too large"); }
    kv->turbo = c->precision == ER_KV_TURBOQUANT_V2;
    kv->q8 = c->precision == ER_KV_Q8_0;
    kv->outlier = c->precision == ER_KV_TURBOQUANT_BALANCED || c->precision == ER_KV_TURBOQUANT_AGGRESSIVE;
    auto bail = [&](int32_t rc) { er_kv_destroy(kv); return rc; };
    if (cudaGetDevice(&kv->device) != cudaSuccess) return bail(fail(ER_ERR_CUDA, "cudaGetDevice"));
    cudaDeviceGetAttribute(&kv->num_sms, cudaDevAttrMultiProcessorCount, kv->device);
    if (kv->turbo) {
        if (c->head_dim != kHeadDim) return bail(fail(ER_ERR_SHAPE, "TurboQuant storage needs head_dim 128 (TurboQuantLayout.supportedDimension)"));
        for (uint32_t t : {c->key_type, c->value_type})
            if (t != ER_TQ_TURBO2 && t != ER_TQ_TURBO3 && t != ER_TQ_TURBO4)
                return bail(fail(ER_ERR_INVALID_ARGUMENT, "TurboQuant type %u (expected 2, 3 or 4 bits)", t));
        kv->k_row_bytes = tq_code_words(static_cast<int>(c->key_type)) * 4;
        kv->v_row_bytes = tq_code_words(static_cast<int>(c->value_type)) * 4;
        kv->norm_bytes = c->norm_format == ER_TQ_NORM_FLOAT16 ? 2 : 4;
        if (kv->cfg.layout == ER_KV_LAYOUT_TOKEN_MAJOR) kv->cfg.layout = ER_KV_LAYOUT_HEAD_MAJOR;
    } else if (kv->outlier) {
        // TurboQuantPreset.balanced / .aggressive descriptors (TurboQuant.swift:267-327): 3 / 5 bits and 2 / 3 bits, 32 channels
        if (c->head_dim != kHeadDim) return bail(fail(ER_ERR_SHAPE, "TurboQuant storage needs head_dim 128 (TurboQuantLayout.supportedDimension)"));
        for (uint32_t t : {c->key_type, c->value_type})
            if (t > ER_TQ_SELECT_QUANTIZATION_BENEFIT)
                return bail(fail(ER_ERR_INVALID_ARGUMENT, "outlier selection %u (expected ER_TQ_SELECT_*)", t));
        kv->ofmt = c->precision == ER_KV_TURBOQUANT_BALANCED ? outlier_format(3, 5, 32) : outlier_format(2, 3, 32);
        kv->k_row_bytes = kv->v_row_bytes = kv->ofmt.row_words * 4;
        kv->norm_bytes = 0;
        if (kv->cfg.layout == ER_KV_LAYOUT_TOKEN_MAJOR) kv->cfg.layout = ER_KV_LAYOUT_HEAD_MAJOR;
    } else if (kv->q8) {
        // KVCache.resolvedStorageKind: headDim % 32 == 0 (KVCache.swift:764-768); the kernels here are built for 128
        if (c->head_dim != kHeadDim) return bail(fail(ER_ERR_UNSUPPORTED_STORAGE, "q8_0 storage is built for head_dim 128"));
        kv->k_row_bytes = kv->v_row_bytes = kQ8RowBytes;
        kv->norm_bytes = kQ8ScaleBytes;
        if (kv->cfg.layout == ER_KV_LAYOUT_TOKEN_MAJOR) kv->cfg.layout = ER_KV_LAYOUT_HEAD_MAJOR;
    } else {
        kv->elem_bytes = c->precision == ER_KV_FLOAT32 ? 4 : 2;
        kv->k_row_bytes = kv->v_row_bytes = static_cast<int>(c->head_dim) * kv->elem_bytes;
    }
    const uint32_t B = kv->cfg.max_batch;
    switch (kv->cfg.layout) {
        case ER_KV_LAYOUT_TOKEN_MAJOR:
            kv->token_major = true;
            kv->page_tokens = static_cast<int>(c->max_seq_len);
            kv->pool_pages = static_cast<int>(B);
            kv->pages_per_seq = 0;
            break;
        case ER_KV_LAYOUT_HEAD_MAJOR:
            kv->page_tokens = static_cast<int>((c->max_seq_len + 15u) & ~15u);
            kv->pool_pages = static_cast<int>(B);
            kv->pages_per_seq = 0;
            break;
        case ER_KV_LAYOUT_PAGED:
            if (c->page_size == 0 || c->page_size % 16 != 0 || c->num_pages == 0)
                return bail(fail(ER_ERR_INVALID_ARGUMENT, "paged layout needs page_size %% 16 == 0 and num_pages > 0"));
            kv->page_tokens = static_cast<int>(c->page_size);
            kv->pool_pages = static_cast<int>(c->num_pages);
            kv->pages_per_seq = static_cast<int>((c->max_seq_len + c->page_size - 1) / c->page_size);
            break;
        default: return bail(fail(ER_ERR_INVALID_ARGUMENT, "unknown layout %u", kv->cfg.layout));
    }
    const int64_t rows_per_layer = static_cast<int64_t>(kv->pool_pages) * c->num_kv_heads * kv->page_tokens;
    kv->k_layer_stride = rows_per_layer * kv->k_row_bytes;
    kv->v_layer_stride = rows_per_layer * kv->v_row_bytes;
    kv->n_layer_stride = rows_per_layer * kv->norm_bytes;
    auto alloc = [&](uint8_t** p, int64_t bytes) -> bool {
        if (bytes == 0) return true;
        if (cudaMalloc(p, static_cast<size_t>(bytes)) != cudaSuccess) { cudaGetLastError(); *p = nullptr; return false; }
        return cudaMemset(*p, 0, static_cast<size_t>(bytes)) == cudaSuccess;
    };
    if (!alloc(&kv->k_slab, kv->k_layer_stride * c->num_layers) || !alloc(&kv->v_slab, kv->v_layer_stride * c->num_layers) ||
        !alloc(&kv->kn_slab, kv->n_layer_stride * c->num_layers + (kv->n_layer_stride ? 256 : 0)) ||
        !alloc(&kv->vn_slab, kv->n_layer_stride * c->num_layers + (kv->n_layer_stride ? 256 : 0)))
        return bail(fail(ER_ERR_ALLOCATION_FAILED, "KV slabs (%lld + %lld bytes per layer, %u layers)",
                         static_cast<long long>(kv->k_layer_stride), static_cast<long long>(kv->v_layer_stride), c->num_layers));
    kv->h_lengths.assign(static_cast<size_t>(c->num_layers) * B, 0);
    if (cudaMalloc(&kv->d_lengths, kv->h_lengths.size() * sizeof(int32_t)) != cudaSuccess ||
        cudaMemset(kv->d_lengths, 0, kv->h_lengths.size() * sizeof(int32_t)) != cudaSuccess)
        return bail(fail(ER_ERR_ALLOCATION_FAILED, "length table"));
    if (kv->pages_per_seq > 0) {
        kv->h_block_table.assign(static_cast<size_t>(B) * kv->pages_per_seq, -1);   // -1 = no page assigned
        kv->h_block_count.assign(B, 0);
        if (cudaMalloc(&kv->d_block_table, kv->h_block_table.size() * sizeof(int32_t)) != cudaSuccess ||
            cudaMemset(kv->d_block_table, 0xFF, kv->h_block_table.size() * sizeof(int32_t)) != cudaSuccess)
            return bail(fail(ER_ERR_ALLOCATION_FAILED, "block table"));
    }
    const size_t counters = 16 + static_cast<size_t>(c->num_layers) * B * c->num_kv_heads;
    if (cudaMalloc(&kv->d_scratch, sizeof(float) * kScratchFloatsPerCta * std::max(kv->num_sms, 1)) != cudaSuccess ||
        cudaMalloc(&kv->d_counters, sizeof(int) * counters) != cudaSuccess ||
        cudaMemset(kv->d_counters, 0, sizeof(int) * counters) != cudaSuccess)
        return bail(fail(ER_ERR_ALLOCATION_FAILED, "scratch"));
    if (cudaHostAlloc(reinterpret_cast<void**>(&kv->h_status), 4 * sizeof(int), cudaHostAllocMapped) != cudaSuccess)
        return bail(fail(ER_ERR_ALLOCATION_FAILED, "pinned status word"));
    for (int i = 0; i < 4; ++i) kv->h_status[i] = 0;
    {
        void* alias = nullptr;
        if (cudaHostGetDevicePointer(&alias, kv->h_status, 0) == cudaSuccess) kv->d_host_done = static_cast<int*>(alias) + 2; else cudaGetLastError();
    }
    if (cudaDeviceSynchronize() != cudaSuccess) return bail(fail(ER_ERR_CUDA, "cache initialisation"));
    *out = kv;
    return ER_OK;
}

void er_kv_destroy(er_kv* kv) {
    if (!kv) return;
    cudaFree(kv->k_slab); cudaFree(kv->v_slab); cudaFree(kv->kn_slab); cudaFree(kv->vn_slab);
    cudaFree(kv->d_lengths); cudaFree(kv->d_block_table); cudaFree(kv->d_scratch); cudaFree(kv->d_counters);
    cudaFree(kv->d_head_norm[0]); cudaFree(kv->d_head_norm[1]);
    cudaFree(kv->d_stage); cudaFree(kv->d_simt_partial); cudaFree(kv->d_prefill_partial);
    if (kv->h_status) cudaFreeHost(kv->h_status);
    cudaGetLastError();
    delete kv;
}

int32_t er_kv_get_config(const er_kv* kv, er_kv_config* out) {
    if (!kv || !out) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    *out = kv->cfg;
    return ER_OK;
}

int32_t er_kv_current_length(er_kv* kv) {
    if (!kv) return fail(ER_ERR_INVALID_ARGUMENT, "null cache");
    std::lock_guard<std::mutex> lock(kv->mu);
    int32_t rc = pull_lengths(kv);
    if (rc != ER_OK) return rc;
    int32_t best = 0;
    for (int32_t n : kv->h_lengths) best = std::max(best, std::min<int32_t>(n, static_cast<int32_t>(kv->cfg.max_seq_len)));
    return best;
}

int64_t er_kv_total_written(er_kv* kv, uint32_t layer, uint32_t seq) {
    if (!kv) return fail(ER_ERR_INVALID_ARGUMENT, "null cache");
    if (layer >= kv->cfg.num_layers) return fail(ER_ERR_INVALID_LAYER, "layer %u", layer);
    if (seq >= kv->cfg.max_batch) return fail(ER_ERR_INVALID_ARGUMENT, "sequence %u", seq);
    std::lock_guard<std::mutex> lock(kv->mu);
    int32_t rc = pull_lengths(kv);
    if (rc != ER_OK) return rc;
    return kv->h_lengths[static_cast<size_t>(layer) * kv->cfg.max_batch + seq];
}

int32_t er_kv_cache_params(er_kv* kv, uint32_t layer, uint32_t seq, ERKVCacheParams* out) {
    if (!kv || !out) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (layer >= kv->cfg.num_layers) return fail(ER_ERR_INVALID_LAYER, "layer %u", layer);
    if (seq >= kv->cfg.max_batch) return fail(ER_ERR_INVALID_ARGUMENT, "sequence %u", seq);
    std::lock_guard<std::mutex> lock(kv->mu);
    int32_t rc = pull_lengths(kv);
    if (rc != ER_OK) return rc;
    const int32_t total = kv->h_lengths[static_cast<size_t>(layer) * kv->cfg.max_batch + seq];
    out->maxSeqLen = kv->cfg.max_seq_len;
    out->currentLen = static_cast<uint32_t>(std::min<int64_t>(total, kv->cfg.max_seq_len));
    out->writePos = static_cast<uint32_t>(total % static_cast<int32_t>(kv->cfg.max_seq_len));
    out->numKVHeads = kv->cfg.num_kv_heads;
    out->headDim = kv->cfg.head_dim;
    out->precision = kv->cfg.precision;
    return ER_OK;
}

int32_t er_kv_reset(er_kv* kv) {
    if (!kv) return fail(ER_ERR_INVALID_ARGUMENT, "null cache");
    std::lock_guard<std::mutex> lock(kv->mu);
    std::fill(kv->h_lengths.begin(), kv->h_lengths.end(), 0);
    return push_lengths(kv);
}

int32_t er_kv_advance_write_position(er_kv* kv, uint32_t layer, uint32_t seq, uint32_t count) {
    if (!kv) return fail(ER_ERR_INVALID_ARGUMENT, "null cache");
    if (layer >= kv->cfg.num_layers) return fail(ER_ERR_INVALID_LAYER, "layer %u", layer);
    std::lock_guard<std::mutex> lock(kv->mu);
    int32_t rc = pull_lengths(kv);
    if (rc != ER_OK) return rc;
    for (uint32_t s = 0; s < kv->cfg.max_batch; ++s)
        if (seq == UINT32_MAX || seq == s) kv->h_lengths[static_cast<size_t>(layer) * kv->cfg.max_batch + s] += static_cast<int32_t>(count);
    return push_lengths(kv);
}

int32_t er_kv_set_position(er_kv* kv, uint32_t seq, uint32_t position) {
    if (!kv) return fail(ER_ERR_INVALID_ARGUMENT, "null cache");
    std::lock_guard<std::mutex> lock(kv->mu);
    int32_t rc = pull_lengths(kv);
    if (rc != ER_OK) return rc;
    for (uint32_t l = 0; l < kv->cfg.num_layers; ++l)
        for (uint32_t s = 0; s < kv->cfg.max_batch; ++s)
            if (seq == UINT32_MAX || seq == s) kv->h_lengths[static_cast<size_t>(l) * kv->cfg.max_batch + s] = static_cast<int32_t>(position);
    return push_lengths(kv);
}

int32_t er_kv_set_block_table(er_kv* kv, uint32_t seq, const int32_t* pages, uint32_t count) {
    if (!kv || (!pages && count)) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (kv->pages_per_seq == 0) return fail(ER_ERR_UNSUPPORTED_STORAGE, "cache is not paged");
    if (seq >= kv->cfg.max_batch) return fail(ER_ERR_INVALID_ARGUMENT, "sequence %u", seq);
    if (count > static_cast<uint32_t>(kv->pages_per_seq)) return fail(ER_ERR_SHAPE, "%u pages exceed the %d a sequence can hold", count, kv->pages_per_seq);
    for (uint32_t i = 0; i < count; ++i)
        if (pages[i] < 0 || pages[i] >= kv->pool_pages) return fail(ER_ERR_INVALID_ARGUMENT, "page id %d outside the pool of %d", pages[i], kv->pool_pages);
    std::lock_guard<std::mutex> lock(kv->mu);
    int32_t* row = kv->h_block_table.data() + static_cast<size_t>(seq) * kv->pages_per_seq;
    std::copy(pages, pages + count, row);
    std::fill(row + count, row + kv->pages_per_seq, -1);
    kv->h_block_count[seq] = count;
    ER_CUDA(cudaMemcpy(kv->d_block_table + static_cast<size_t>(seq) * kv->pages_per_seq, row,
                       sizeof(int32_t) * kv->pages_per_seq, cudaMemcpyHostToDevice));
    return ER_OK;
}

int32_t er_kv_get_block_table(er_kv* kv, uint32_t seq, int32_t* pages, uint32_t capacity, uint32_t* count) {
    if (!kv || !count) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (kv->pages_per_seq == 0) return fail(ER_ERR_UNSUPPORTED_STORAGE, "cache is not paged");
    if (seq >= kv->cfg.max_batch) return fail(ER_ERR_INVALID_ARGUMENT, "sequence %u", seq);
    std::lock_guard<std::mutex> lock(kv->mu);
    *count = kv->h_block_count[seq];
    for (uint32_t i = 0; i < std::min(capacity, *count); ++i) pages[i] = kv->h_block_table[static_cast<size_t>(seq) * kv->pages_per_seq + i];
    return ER_OK;
}

int32_t er_kv_device_buffers(er_kv* kv, uint32_t layer, er_kv_buffers* out) {
    if (!kv || !out) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (layer >= kv->cfg.num_layers) return fail(ER_ERR_INVALID_LAYER, "layer %u", layer);
    out->keys = kv->k_slab + layer * kv->k_layer_stride;
    out->values = kv->v_slab + layer * kv->v_layer_stride;
    out->key_norms = kv->kn_slab ? kv->kn_slab + layer * kv->n_layer_stride : nullptr;
    out->value_norms = kv->vn_slab ? kv->vn_slab + layer * kv->n_layer_stride : nullptr;
    out->key_bytes = static_cast<uint64_t>(kv->k_layer_stride);
    out->value_bytes = static_cast<uint64_t>(kv->v_layer_stride);
    out->key_row_bytes = static_cast<uint32_t>(kv->k_row_bytes);
    out->value_row_bytes = static_cast<uint32_t>(kv->v_row_bytes);
    return ER_OK;
}

// ---- host-facing append / retrieve ----

static int32_t host_append(er_kv* kv, uint32_t layer, uint32_t seq, const void* hk, const void* hv, size_t count,
                           int src_elem_bytes) {
    const size_t per_token = static_cast<size_t>(kv->cfg.num_kv_heads) * kv->cfg.head_dim;
    if (count != per_token) return fail(ER_ERR_SHAPE, "expected %zu elements per token, got %zu", per_token, count);
    if (seq >= kv->cfg.max_batch) return fail(ER_ERR_INVALID_ARGUMENT, "sequence %u", seq);
    int32_t rc = check_device(kv);
    if (rc != ER_OK) return rc;
    std::lock_guard<std::mutex> lock(kv->mu);
    rc = pull_lengths(kv);
    if (rc != ER_OK) return rc;
    int32_t& total = kv->h_lengths[static_cast<size_t>(layer) * kv->cfg.max_batch + seq];
    // the row goes to ring slot total % maxSeqLen: that slot's page must exist
    rc = check_page_coverage(kv, seq, static_cast<uint64_t>(total % static_cast<int32_t>(kv->cfg.max_seq_len)) + 1);
    if (rc != ER_OK) return rc;
    const size_t bytes = per_token * src_elem_bytes;
    rc = ensure_stage(kv, 2 * bytes);
    if (rc != ER_OK) return rc;
    ER_CUDA(cudaMemcpy(kv->d_stage, hk, bytes, cudaMemcpyHostToDevice));
    ER_CUDA(cudaMemcpy(kv->d_stage + bytes, hv, bytes, cudaMemcpyHostToDevice));
    if (kv->turbo || kv->q8 || kv->outlier) {
        AppendParams ap{};
        ap.k = reinterpret_cast<const float*>(kv->d_stage);
        ap.v = reinterpret_cast<const float*>(kv->d_stage + bytes);
        ap.bulk = 1; ap.fixed_layer = static_cast<int>(layer); ap.fixed_seq = static_cast<int>(seq);
        ap.start_pos = total; ap.rows = 1; ap.batch = static_cast<int>(kv->cfg.max_batch);
        ap.apply_rope = 0; ap.rope_scaling = 1.f;
        rc = launch_append(kv, ap, nullptr);
        if (rc != ER_OK) return rc;
    } else {
        const int slot = total % static_cast<int32_t>(kv->cfg.max_seq_len);
        const KVAddressing a = kv->addressing();
        scatter_row_kernel<<<4, 256>>>(kv->d_stage, kv->k_slab + layer * kv->k_layer_stride, a, static_cast<int>(seq), slot,
                                       static_cast<int>(kv->cfg.head_dim), kv->elem_bytes);
        if ((rc = check_launch("scatter_row_kernel")) != ER_OK) return rc;
        scatter_row_kernel<<<4, 256>>>(kv->d_stage + bytes, kv->v_slab + layer * kv->v_layer_stride, a, static_cast<int>(seq), slot,
                                       static_cast<int>(kv->cfg.head_dim), kv->elem_bytes);
        if ((rc = check_launch("scatter_row_kernel")) != ER_OK) return rc;
    }
    total += 1;
    rc = push_lengths(kv);
    if (rc != ER_OK) return rc;
    ER_CUDA(cudaDeviceSynchronize());
    return ER_OK;
}

int32_t er_kv_append_f32(er_kv* kv, uint32_t layer, uint32_t seq, const float* hk, const float* hv, size_t count) {
    if (!kv || !hk || !hv) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (layer >= kv->cfg.num_layers) return fail(ER_ERR_INVALID_LAYER, "layer %u", layer);
    // KVCache.append: float32, q8_0 and TurboQuant precisions; everything else is precisionMismatch (KVCache.swift:436-452).
    if (kv->cfg.precision != ER_KV_FLOAT32 && !kv->turbo && !kv->q8 && !kv->outlier) return fail(ER_ERR_PRECISION_MISMATCH, "append of Float rows into precision %u", kv->cfg.precision);
    return host_append(kv, layer, seq, hk, hv, count, 4);
}

int32_t er_kv_append_f16(er_kv* kv, uint32_t layer, uint32_t seq, const uint16_t* hk, const uint16_t* hv, size_t count) {
    if (!kv || !hk || !hv) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (layer >= kv->cfg.num_layers) return fail(ER_ERR_INVALID_LAYER, "layer %u", layer);
    if (kv->cfg.precision != ER_KV_FLOAT16) return fail(ER_ERR_PRECISION_MISMATCH, "appendF16 needs a float16 cache");
    return host_append(kv, layer, seq, hk, hv, count, 2);
}

// Logical order of KVCache.orderedRowIndices (KVCache.swift:1130-1138).
static void logical_window(const er_kv* kv, int32_t total, int& first_slot, int& tokens) {
    const int32_t maxn = static_cast<int32_t>(kv->cfg.max_seq_len);
    tokens = std::min(total, maxn);
    first_slot = total <= maxn ? 0 : total % maxn;
}

int32_t er_kv_retrieve(er_kv* kv, uint32_t layer, uint32_t seq, uint32_t element_bytes, void* hk, void* hv,
                       size_t capacity, uint32_t* token_count) {
    if (!kv || !token_count) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (layer >= kv->cfg.num_layers) return fail(ER_ERR_INVALID_LAYER, "layer %u", layer);
    if (seq >= kv->cfg.max_batch) return fail(ER_ERR_INVALID_ARGUMENT, "sequence %u", seq);
    // validateRequestedType (KVCache.swift:866-883)
    if (kv->turbo || kv->outlier) return fail(ER_ERR_COMPRESSED_RETRIEVE_REQUIRES_DECODED_API, "TurboQuant cache");
    if (kv->q8) return fail(ER_ERR_COMPRESSED_RETRIEVE_REQUIRES_DECODED_API, "q8_0 cache");
    if (static_cast<int>(element_bytes) != kv->elem_bytes) return fail(ER_ERR_PRECISION_MISMATCH, "requested %u-byte elements from a %d-byte cache", element_bytes, kv->elem_bytes);
    int32_t rc = check_device(kv);
    if (rc != ER_OK) return rc;
    std::lock_guard<std::mutex> lock(kv->mu);
    if ((rc = pull_lengths(kv)) != ER_OK) return rc;
    int first_slot, tokens;
    logical_window(kv, kv->h_lengths[static_cast<size_t>(layer) * kv->cfg.max_batch + seq], first_slot, tokens);
    *token_count = static_cast<uint32_t>(tokens);
    if (tokens == 0) return ER_OK;
    const size_t elems = static_cast<size_t>(tokens) * kv->cfg.num_kv_heads * kv->cfg.head_dim;
    if (!hk || !hv || capacity < elems) return fail(ER_ERR_SHAPE, "output capacity %zu < %zu elements", capacity, elems);
    const size_t bytes = elems * kv->elem_bytes;
    rc = ensure_stage(kv, 2 * bytes);
    if (rc != ER_OK) return rc;
    const KVAddressing a = kv->addressing();
    const int blocks = static_cast<int>(std::min<size_t>((bytes + 255) / 256, 4096));
    gather_rows_kernel<<<blocks, 256>>>(kv->k_slab + layer * kv->k_layer_stride, kv->d_stage, a, static_cast<int>(seq), first_slot, tokens, kv->k_row_bytes);
    if ((rc = check_launch("gather_rows_kernel")) != ER_OK) return rc;
    gather_rows_kernel<<<blocks, 256>>>(kv->v_slab + layer * kv->v_layer_stride, kv->d_stage + bytes, a, static_cast<int>(seq), first_slot, tokens, kv->v_row_bytes);
    if ((rc = check_launch("gather_rows_kernel")) != ER_OK) return rc;
    ER_CUDA(cudaMemcpy(hk, kv->d_stage, bytes, cudaMemcpyDeviceToHost));
    ER_CUDA(cudaMemcpy(hv, kv->d_stage + bytes, bytes, cudaMemcpyDeviceToHost));
    return ER_OK;
}

int32_t er_kv_retrieve_turboquant_rows(er_kv* kv, uint32_t layer, uint32_t seq, int is_value, uint32_t* h_codes,
                                       uint32_t* h_signs, uint32_t* h_mask, float* h_meta, size_t capacity_rows,
                                       uint32_t* row_count) {
    if (!kv || !row_count) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (layer >= kv->cfg.num_layers) return fail(ER_ERR_INVALID_LAYER, "layer %u", layer);
    if (seq >= kv->cfg.max_batch) return fail(ER_ERR_INVALID_ARGUMENT, "sequence %u", seq);
    if (!kv->turbo && !kv->outlier) return fail(ER_ERR_PRECISION_MISMATCH, "not a TurboQuant cache");
    int32_t rc = check_device(kv);
    if (rc != ER_OK) return rc;
    std::lock_guard<std::mutex> lock(kv->mu);
    if ((rc = pull_lengths(kv)) != ER_OK) return rc;
    int first_slot, tokens;
    logical_window(kv, kv->h_lengths[static_cast<size_t>(layer) * kv->cfg.max_batch + seq], first_slot, tokens);
    const size_t rows = static_cast<size_t>(tokens) * kv->cfg.num_kv_heads;
    *row_count = static_cast<uint32_t>(rows);
    if (rows == 0) return ER_OK;
    if (capacity_rows < rows || !h_codes || !h_meta) return fail(ER_ERR_SHAPE, "output capacity %zu < %zu rows", capacity_rows, rows);
    if (kv->outlier) {   // codes | signs | mask | meta, split out of the cached blocks on the device
        const size_t code_bytes = rows * kv->ofmt.wpr * 4;
        const size_t o_signs = (code_bytes + 255) & ~size_t(255), o_mask = o_signs + rows * 16, o_meta = o_mask + rows * 16;
        rc = ensure_stage(kv, o_meta + rows * 8);
        if (rc != ER_OK) return rc;
        OutlierExportParams ep;
        ep.rows = (is_value ? kv->v_slab : kv->k_slab) + layer * (is_value ? kv->v_layer_stride : kv->k_layer_stride);
        ep.codes = reinterpret_cast<uint32_t*>(kv->d_stage); ep.signs = reinterpret_cast<uint32_t*>(kv->d_stage + o_signs);
        ep.mask = reinterpret_cast<uint32_t*>(kv->d_stage + o_mask); ep.meta = reinterpret_cast<float*>(kv->d_stage + o_meta);
        ep.fmt = kv->ofmt; ep.addr = kv->addressing();
        ep.seq = static_cast<int>(seq); ep.first_slot = first_slot; ep.tokens = tokens;
        tq_outlier_export_rows_kernel<<<static_cast<unsigned>(std::min<size_t>((rows + 7) / 8, 8192)), 256>>>(ep);
        if ((rc = check_launch("tq_outlier_export_rows_kernel")) != ER_OK) return rc;
        ER_CUDA(cudaMemcpy(h_codes, ep.codes, code_bytes, cudaMemcpyDeviceToHost));
        ER_CUDA(cudaMemcpy(h_meta, ep.meta, rows * 8, cudaMemcpyDeviceToHost));
        if (h_signs) ER_CUDA(cudaMemcpy(h_signs, ep.signs, rows * 16, cudaMemcpyDeviceToHost));
        if (h_mask) ER_CUDA(cudaMemcpy(h_mask, ep.mask, rows * 16, cudaMemcpyDeviceToHost));
        return ER_OK;
    }
    const int row_bytes = is_value ? kv->v_row_bytes : kv->k_row_bytes;
    const size_t code_bytes = rows * row_bytes, norm_bytes = rows * kv->norm_bytes;
    const size_t norm_off = (code_bytes + 255) & ~size_t(255);
    const size_t meta_off = norm_off + ((norm_bytes + 255) & ~size_t(255));
    rc = ensure_stage(kv, meta_off + rows * 8);
    if (rc != ER_OK) return rc;
    const KVAddressing a = kv->addressing();
    const uint8_t* codes = (is_value ? kv->v_slab : kv->k_slab) + layer * (is_value ? kv->v_layer_stride : kv->k_layer_stride);
    const uint8_t* norms = (is_value ? kv->vn_slab : kv->kn_slab) + layer * kv->n_layer_stride;
    const int blocks = static_cast<int>(std::min<size_t>((code_bytes + 255) / 256, 4096));
    gather_rows_kernel<<<blocks, 256>>>(codes, kv->d_stage, a, static_cast<int>(seq), first_slot, tokens, row_bytes);
    if ((rc = check_launch("gather_rows_kernel")) != ER_OK) return rc;
    gather_rows_kernel<<<blocks, 256>>>(norms, kv->d_stage + norm_off, a, static_cast<int>(seq), first_slot, tokens, kv->norm_bytes);
    if ((rc = check_launch("gather_rows_kernel")) != ER_OK) return rc;
    float* d_meta = reinterpret_cast<float*>(kv->d_stage + meta_off);
    widen_norms_kernel<<<static_cast<int>((rows + 255) / 256), 256>>>(kv->d_stage + norm_off, d_meta, static_cast<int>(rows), kv->norm_bytes == 2);
    if ((rc = check_launch("widen_norms_kernel")) != ER_OK) return rc;
    ER_CUDA(cudaMemcpy(h_codes, kv->d_stage, code_bytes, cudaMemcpyDeviceToHost));
    ER_CUDA(cudaMemcpy(h_meta, d_meta, rows * 8, cudaMemcpyDeviceToHost));
    if (h_signs) std::memset(h_signs, 0, rows * 16);
    if (h_mask) std::memset(h_mask, 0, rows * 16);
    return ER_OK;
}

int32_t er_kv_retrieve_decoded_turboquant(er_kv* kv, uint32_t layer, uint32_t seq, float* hk, float* hv, size_t capacity,
                                          uint32_t* token_count) {
    if (!kv || !token_count) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (layer >= kv->cfg.num_layers) return fail(ER_ERR_INVALID_LAYER, "layer %u", layer);
    if (seq >= kv->cfg.max_batch) return fail(ER_ERR_INVALID_ARGUMENT, "sequence %u", seq);
    if (!kv->turbo && !kv->outlier) return fail(ER_ERR_PRECISION_MISMATCH, "not a TurboQuant cache");
    int32_t rc = check_device(kv);
    if (rc != ER_OK) return rc;
    std::lock_guard<std::mutex> lock(kv->mu);
    if ((rc = pull_lengths(kv)) != ER_OK) return rc;
    int first_slot, tokens;
    logical_window(kv, kv->h_lengths[static_cast<size_t>(layer) * kv->cfg.max_batch + seq], first_slot, tokens);
    *token_count = static_cast<uint32_t>(tokens);
    if (tokens == 0) return ER_OK;
    const size_t rows = static_cast<size_t>(tokens) * kv->cfg.num_kv_heads;
    const size_t elems = rows * kHeadDim;
    if (!hk || !hv || capacity < elems) return fail(ER_ERR_SHAPE, "output capacity %zu < %zu elements", capacity, elems);
    rc = ensure_stage(kv, 2 * elems * 4);
    if (rc != ER_OK) return rc;
    if (kv->outlier) {
        // approximateDecode: keys with the default residualWeight 1, values with the contract's valueResidualScale
        // (KVCache.swift:556-581)
        OutlierDecodeRowsParams dp;
        dp.fmt = kv->ofmt; dp.addr = kv->addressing();
        dp.seq = static_cast<int>(seq); dp.first_slot = first_slot; dp.tokens = tokens;
        for (int is_v = 0; is_v < 2; ++is_v) {
            dp.rows = (is_v ? kv->v_slab : kv->k_slab) + layer * (is_v ? kv->v_layer_stride : kv->k_layer_stride);
            dp.out = reinterpret_cast<float*>(kv->d_stage) + is_v * elems;
            dp.residual_weight = is_v ? kv->cfg.value_residual_scale : 1.0f;
            tq_outlier_decode_rows_kernel<<<static_cast<unsigned>(std::min<size_t>((rows + 7) / 8, 8192)), 256>>>(dp);
            if ((rc = check_launch("tq_outlier_decode_rows_kernel")) != ER_OK) return rc;
        }
        ER_CUDA(cudaMemcpy(hk, kv->d_stage, elems * 4, cudaMemcpyDeviceToHost));
        ER_CUDA(cudaMemcpy(hv, kv->d_stage + elems * 4, elems * 4, cudaMemcpyDeviceToHost));
        return ER_OK;
    }
    TurboDecodeRowsParams dp;
    dp.addr = kv->addressing();
    dp.seq = static_cast<int>(seq); dp.first_slot = first_slot; dp.tokens = tokens;
    dp.norm_fp16 = kv->norm_bytes == 2;
    for (int is_v = 0; is_v < 2; ++is_v) {
        dp.codes = (is_v ? kv->v_slab : kv->k_slab) + layer * (is_v ? kv->v_layer_stride : kv->k_layer_stride);
        dp.norms = (is_v ? kv->vn_slab : kv->kn_slab) + layer * kv->n_layer_stride;
        dp.out = reinterpret_cast<float*>(kv->d_stage) + is_v * elems;
        rc = launch_turbo_decode_rows(dp, static_cast<int>(is_v ? kv->cfg.value_type : kv->cfg.key_type), nullptr, check_launch);
        if (rc != ER_OK) return rc;
    }
    ER_CUDA(cudaMemcpy(hk, kv->d_stage, elems * 4, cudaMemcpyDeviceToHost));
    ER_CUDA(cudaMemcpy(hv, kv->d_stage + elems * 4, elems * 4, cudaMemcpyDeviceToHost));
    return ER_OK;
}

// Shared body of the two q8_0 retrieves: rows in ring order -> decoded floats and / or 34-byte blocks.
static int32_t q8_export(er_kv* kv, uint32_t layer, uint32_t seq, float* hk_values, float* hv_values, uint8_t* hk_blocks, uint8_t* hv_blocks,
                         size_t capacity, uint32_t* token_count) {
    if (!kv || !token_count) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (layer >= kv->cfg.num_layers) return fail(ER_ERR_INVALID_LAYER, "layer %u", layer);
    if (seq >= kv->cfg.max_batch) return fail(ER_ERR_INVALID_ARGUMENT, "sequence %u", seq);
    if (!kv->q8) return fail(ER_ERR_PRECISION_MISMATCH, "not a q8_0 cache");
    const bool blocks = hk_blocks != nullptr || hv_blocks != nullptr;
    int32_t rc = check_device(kv);
    if (rc != ER_OK) return rc;
    std::lock_guard<std::mutex> lock(kv->mu);
    if ((rc = pull_lengths(kv)) != ER_OK) return rc;
    int first_slot, tokens;
    logical_window(kv, kv->h_lengths[static_cast<size_t>(layer) * kv->cfg.max_batch + seq], first_slot, tokens);
    *token_count = static_cast<uint32_t>(tokens);
    if (tokens == 0) return ER_OK;
    const size_t rows = static_cast<size_t>(tokens) * kv->cfg.num_kv_heads;
    const size_t unit = blocks ? kQ8PackedRowBytes : kHeadDim * sizeof(float);
    const size_t need = blocks ? rows * kQ8PackedRowBytes : rows * kHeadDim;
    if ((blocks ? (!hk_blocks || !hv_blocks) : (!hk_values || !hv_values)) || capacity < need)
        return fail(ER_ERR_SHAPE, "output capacity %zu < %zu", capacity, need);
    rc = ensure_stage(kv, 2 * rows * unit);
    if (rc != ER_OK) return rc;
    Q8ExportParams ep{};
    ep.addr = kv->addressing();
    ep.seq = static_cast<int>(seq); ep.tokens = tokens; ep.first_slot = first_slot;
    for (int is_v = 0; is_v < 2; ++is_v) {
        ep.rows = (is_v ? kv->v_slab : kv->k_slab) + layer * (is_v ? kv->v_layer_stride : kv->k_layer_stride);
        ep.scales = (is_v ? kv->vn_slab : kv->kn_slab) + layer * kv->n_layer_stride;
        ep.out_blocks = blocks ? kv->d_stage + is_v * rows * unit : nullptr;
        ep.out_values = blocks ? nullptr : reinterpret_cast<float*>(kv->d_stage + is_v * rows * unit);
        q8_export_rows_kernel<<<static_cast<unsigned>(std::min<size_t>((rows + 7) / 8, 8192)), 256>>>(ep);
        if ((rc = check_launch("q8_export_rows_kernel")) != ER_OK) return rc;
    }
    ER_CUDA(cudaMemcpy(blocks ? static_cast<void*>(hk_blocks) : static_cast<void*>(hk_values), kv->d_stage, rows * unit, cudaMemcpyDeviceToHost));
    ER_CUDA(cudaMemcpy(blocks ? static_cast<void*>(hv_blocks) : static_cast<void*>(hv_values), kv->d_stage + rows * unit, rows * unit,
                       cudaMemcpyDeviceToHost));
    return ER_OK;
}

int32_t er_kv_retrieve_decoded_q8_0(er_kv* kv, uint32_t layer, uint32_t seq, float* hk, float* hv, size_t capacity, uint32_t* token_count) {
    return q8_export(kv, layer, seq, hk, hv, nullptr, nullptr, capacity, token_count);
}

int32_t er_kv_retrieve_q8_0_rows(er_kv* kv, uint32_t layer, uint32_t seq, uint8_t* hk, uint8_t* hv, size_t capacity_bytes, uint32_t* token_count) {
    if (!hk || !hv) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    return q8_export(kv, layer, seq, nullptr, nullptr, hk, hv, capacity_bytes, token_count);
}

// ---- stand-alone operators ----

int32_t er_quantize_q8_0_rows(const float* source, uint32_t row_count, uint32_t source_row_stride, uint32_t destination_row_base,
                              uint8_t* destination_blocks, void* stream) {
    if (!source || !destination_blocks) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (source_row_stride < kHeadDim) return fail(ER_ERR_SHAPE, "source_row_stride %u < 128", source_row_stride);
    if (row_count == 0) return ER_OK;
    q8_quantize_rows_packed_kernel<<<(row_count + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(source, row_count, source_row_stride,
                                                                                                    destination_row_base, destination_blocks);
    return check_launch("q8_quantize_rows_packed_kernel");
}

static int32_t rope_common(const float* in, void* out, const ERRoPEParams* p, bool to_f16, void* stream) {
    if (!in || !out || !p) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (p->headDim == 0 || p->headDim % 2 != 0 || p->headDim > 512) return fail(ER_ERR_SHAPE, "headDim %u (even, <= 512)", p->headDim);
    if (!(p->theta > 0.f)) return fail(ER_ERR_INVALID_ARGUMENT, "theta must be > 0");
    const uint64_t total = static_cast<uint64_t>(p->seqLen) * p->numHeads * (p->headDim / 2);
    if (total == 0) return ER_OK;
    WideInvFreqTable table;
    fill_inv_freq(table, 256, p->theta, p->headDim);
    const float scaling = p->scalingFactor == 0.f ? 1.f : p->scalingFactor;
    const int blocks = static_cast<int>(std::min<uint64_t>((total + 255) / 256, 1u << 16));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (to_f16)
        rope_neox_kernel<__half><<<blocks, 256, 0, s>>>(in, static_cast<__half*>(out), p->seqLen, p->numHeads, p->headDim, p->startPos, scaling, p->partialRotaryFactor, table);
    else
        rope_neox_kernel<float><<<blocks, 256, 0, s>>>(in, static_cast<float*>(out), p->seqLen, p->numHeads, p->headDim, p->startPos, scaling, p->partialRotaryFactor, table);
    return check_launch("rope_neox_kernel");
}

int32_t er_rope_neox_f32(const float* in, float* out, const ERRoPEParams* p, void* stream) { return rope_common(in, out, p, false, stream); }
int32_t er_rope_neox_f32_to_f16(const float* in, uint16_t* out, const ERRoPEParams* p, void* stream) { return rope_common(in, out, p, true, stream); }

int32_t er_turboquant_quantize_rows(const float* source, uint32_t row_count, uint32_t source_row_stride, uint32_t dst_row_base,
                                    uint32_t bits, uint32_t* out_codes, uint32_t* out_signs, uint32_t* out_mask, float* out_meta,
                                    void* stream) {
    if (!source || !out_codes || !out_meta) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (bits < 2 || bits > 4) return fail(ER_ERR_INVALID_ARGUMENT, "bits %u (fixed presets: 2, 3, 4)", bits);
    if (source_row_stride < kHeadDim) return fail(ER_ERR_SHAPE, "source_row_stride %u < 128", source_row_stride);
    if (row_count == 0) return ER_OK;
    return launch_turbo_quantize_rows(source, row_count, source_row_stride, dst_row_base, static_cast<int>(bits), out_codes, out_signs,
                                      out_mask, out_meta, static_cast<cudaStream_t>(stream), check_launch);
}

int32_t er_turboquant_quantize_rows_outliers(const float* source, uint32_t row_count, uint32_t source_row_stride, uint32_t dst_row_base,
                                             uint32_t regular_bits, uint32_t high_bits, uint32_t high_count, uint32_t use_quantization_benefit,
                                             uint32_t* out_codes, uint32_t* out_signs, uint32_t* out_mask, float* out_meta, void* stream) {
    if (!source || !out_codes || !out_signs || !out_mask || !out_meta) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (regular_bits < 2 || regular_bits > 4 || high_bits <= regular_bits || high_bits > 5 || high_count == 0 || high_count > kHeadDim)
        return fail(ER_ERR_INVALID_ARGUMENT, "regular bits %u (2..4), high-precision bits %u (regular < high <= 5), channel count %u (1..128)",
                    regular_bits, high_bits, high_count);
    if (source_row_stride < kHeadDim || source_row_stride % 4 != 0) return fail(ER_ERR_SHAPE, "source_row_stride %u (>= 128, multiple of 4)", source_row_stride);
    if (reinterpret_cast<uintptr_t>(source) & 15u) return fail(ER_ERR_INVALID_ARGUMENT, "source must be 16-byte aligned");
    if (row_count == 0) return ER_OK;
    TurboOutlierParams op{};
    op.source = source; op.rows = row_count; op.stride = source_row_stride; op.dst_row_base = dst_row_base;
    op.regular_bits = static_cast<int>(regular_bits); op.high_bits = static_cast<int>(high_bits); op.high_count = static_cast<int>(high_count);
    op.use_benefit = use_quantization_benefit ? 1 : 0;
    // TurboQuantLayout (TurboQuant.swift:275-319): base plane + side band, each rounded up to words
    op.words_per_row = (kHeadDim * op.regular_bits + 31) / 32 + (op.high_count * (op.high_bits - op.regular_bits) + 31) / 32;
    op.out_codes = out_codes; op.out_signs = out_signs; op.out_mask = out_mask; op.out_meta = out_meta;
    const unsigned blocks = std::min<unsigned>((row_count + kOutlierWarps - 1) / kOutlierWarps, 148u * 8u);
    tq_quantize_rows_outlier_kernel<<<blocks, kOutlierWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(op);
    return check_launch("tq_quantize_rows_outlier_kernel");
}

// Shapes the persistent flash-decode / tensor-core prefill kernels are built for; everything else on raw buffers goes
// through generic_decode_kernel.
static bool flash_shape(uint32_t head_dim, uint32_t heads, uint32_t kv_heads) {
    const uint32_t g = heads / kv_heads;
    return head_dim == kHeadDim && kv_heads <= 16 && (g == 1 || g == 2 || g == 4 || g == 8);
}

// One query row against ring rows (start + i) % capacity, i < count, of token-major fp16 buffers (count > 0).
static int32_t generic_decode_row(Workspace* ws, const float* q, const uint16_t* k, const uint16_t* v, float* out, uint32_t heads,
                                  uint32_t kv_heads, uint32_t head_dim, uint32_t start, uint32_t count, uint32_t capacity, float scale,
                                  cudaStream_t stream) {
    GenericDecodeParams p{};
    p.q = q; p.out = out;
    p.k = reinterpret_cast<const __half*>(k);
    p.v = reinterpret_cast<const __half*>(v);
    p.num_heads = static_cast<int>(heads); p.num_kv_heads = static_cast<int>(kv_heads); p.head_dim = static_cast<int>(head_dim);
    p.start = static_cast<int>(start); p.count = static_cast<int>(count); p.capacity = static_cast<int>(capacity);
    p.scale_log2 = scale * 1.4426950408889634f;
    p.scratch = ws->scratch; p.counters = ws->counters + 16;
    const int rc = launch_decode_generic(p, ws->num_sms, kScratchFloatsPerCta * static_cast<size_t>(ws->num_sms), ws->counter_ints - 16, stream);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (rc == kNotBuilt)
        return fail(ER_ERR_UNSUPPORTED, "attention on raw buffers: headDim %u must be even and <= 512, numHeads %u <= %zu", head_dim, heads,
                    ws->counter_ints - 16);
    if (rc != 0) return fail(ER_ERR_CUDA, "generic_decode_kernel: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    return ER_OK;
}

int32_t er_gqa_attention_f16kv(const float* q, const uint16_t* k, const uint16_t* v, float* out, const ERGQAParams* gp, void* stream) {
    if (!q || !k || !v || !out || !gp) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (gp->numKVHeads == 0 || gp->numHeads % gp->numKVHeads != 0) return fail(ER_ERR_SHAPE, "numHeads %u not divisible by numKVHeads %u", gp->numHeads, gp->numKVHeads);
    if (check_raw_pointers(q, k, v, out) != ER_OK) return ER_ERR_INVALID_ARGUMENT;
    const uint32_t kv_seq = gp->kvSeqLen > 0 ? gp->kvSeqLen : gp->seqLen;
    if (gp->seqLen == 0 || kv_seq == 0) return ER_OK;
    if (!flash_shape(gp->headDim, gp->numHeads, gp->numKVHeads)) {
        // other head sizes / groups: one launch of the generic kernel per query row (row r sees keys 0 .. r + qOffset)
        Workspace* gws = nullptr;
        int32_t grc = get_workspace(&gws);
        if (grc != ER_OK) return grc;
        const float sc = gp->scale != 0.f ? gp->scale : 1.0f / std::sqrt(static_cast<float>(gp->headDim));
        const size_t row_elems = static_cast<size_t>(gp->numHeads) * gp->headDim;
        for (uint32_t r = 0; r < gp->seqLen; ++r) {
            const uint64_t visible = gp->causal ? std::min<uint64_t>(kv_seq, static_cast<uint64_t>(r) + gp->qOffset + 1) : kv_seq;
            grc = generic_decode_row(gws, q + r * row_elems, k, v, out + r * row_elems, gp->numHeads, gp->numKVHeads, gp->headDim, 0,
                                     static_cast<uint32_t>(visible), kv_seq, sc, static_cast<cudaStream_t>(stream));
            if (grc != ER_OK) return grc;
        }
        return ER_OK;
    }
    if (gp->seqLen > 1) {   // prompt / chunk: tensor-core kernel
        PrefillParams pp{};
        pp.q = q; pp.out = out;
        pp.k_layer = reinterpret_cast<const uint8_t*>(k);
        pp.v_layer = reinterpret_cast<const uint8_t*>(v);
        pp.addr.token_major = 1; pp.addr.num_kv_heads = static_cast<int>(gp->numKVHeads);
        pp.addr.max_seq_len = static_cast<int>(kv_seq); pp.addr.page_size = static_cast<int>(kv_seq);
        pp.seq = 0; pp.seq_len = static_cast<int>(gp->seqLen); pp.kv_len = static_cast<int>(kv_seq);
        pp.q_offset = static_cast<int>(gp->qOffset); pp.causal = gp->causal ? 1 : 0;
        pp.num_q_heads = static_cast<int>(gp->numHeads);
        const float sc = gp->scale != 0.f ? gp->scale : 1.0f / std::sqrt(static_cast<float>(gp->headDim));
        pp.scale_log2 = sc * 1.4426950408889634f;
        pp.rope_scaling = 1.f;
        Workspace* pws = nullptr;
        int32_t prc = get_workspace(&pws);
        if (prc != ER_OK) return prc;
        const int rcl = launch_prefill(static_cast<int>(gp->numHeads / gp->numKVHeads), pp, 1, static_cast<int>(gp->numKVHeads),
                                       pws->counters + 1, static_cast<cudaStream_t>(stream));
        g_launches.fetch_add(1, std::memory_order_relaxed);
        if (rcl == -1) return fail(ER_ERR_UNSUPPORTED, "prefill kernel is built for GQA groups 1, 2, 4, 8");
        if (rcl != 0) return fail(ER_ERR_CUDA, "prefill_f16_kernel: %s", cudaGetErrorString(static_cast<cudaError_t>(rcl)));
        return ER_OK;
    }
    Workspace* ws = nullptr;
    int32_t rc = get_workspace(&ws);
    if (rc != ER_OK) return rc;
    DecodeParams p{};
    p.k_base = reinterpret_cast<const uint8_t*>(k);
    p.v_base = reinterpret_cast<const uint8_t*>(v);
    p.k_layer_stride_bytes = 0; p.v_layer_stride_bytes = 0;
    p.lengths = nullptr;
    p.layer_begin = 0; p.num_layers = 1; p.batch = 1;
    p.num_q_heads = static_cast<int>(gp->numHeads);
    p.pending = 0; p.advance = 0;
    const float scale = gp->scale != 0.f ? gp->scale : 1.0f / std::sqrt(static_cast<float>(gp->headDim));
    p.scale_log2 = scale * 1.4426950408889634f;
    p.apply_rope = 0; p.rope_scaling = 1.f;
    p.addr.token_major = 1; p.addr.num_kv_heads = static_cast<int>(gp->numKVHeads);
    p.addr.max_seq_len = static_cast<int>(kv_seq); p.addr.page_size = static_cast<int>(kv_seq);
    p.addr.pages_per_seq = 0; p.addr.block_table = nullptr;
    p.scratch = ws->scratch; p.done_counter = ws->counters; p.status = ws->counters + 1; p.item_counters = ws->counters + 16;
    const int group = static_cast<int>(gp->numHeads / gp->numKVHeads);
    encode_token_major_maps(p, group, 1, 1, kv_seq, gp->numKVHeads);
    // One launch per query row: row r sees keys 0 .. r + qOffset (Shaders/GQA.metal:345).
    for (uint32_t r = 0; r < gp->seqLen; ++r) {
        uint64_t visible = gp->causal ? std::min<uint64_t>(kv_seq, static_cast<uint64_t>(r) + gp->qOffset + 1) : kv_seq;
        p.fixed_kv_len = static_cast<int>(visible);
        p.fixed_q_pos = 0;
        p.q = q + static_cast<size_t>(r) * gp->numHeads * kHeadDim;
        p.out = out + static_cast<size_t>(r) * gp->numHeads * kHeadDim;
        rc = dispatch_decode_f16(group, p, ws->num_sms, static_cast<cudaStream_t>(stream));
        if (rc != ER_OK) return rc;
    }
    return ER_OK;
}

int32_t er_gqa_attention_f16kv_windowed(const float* q, const uint16_t* k, const uint16_t* v, float* out, const ERWindowedGQAParams* wp,
                                        void* stream) {
    if (!q || !k || !v || !out || !wp) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (wp->numKVHeads == 0 || wp->numHeads % wp->numKVHeads != 0) return fail(ER_ERR_SHAPE, "numHeads %u not divisible by numKVHeads %u", wp->numHeads, wp->numKVHeads);
    if (wp->kvCount > wp->kvCapacity) return fail(ER_ERR_SHAPE, "kvCount %u > kvCapacity %u", wp->kvCount, wp->kvCapacity);
    if (check_raw_pointers(q, k, v, out) != ER_OK) return ER_ERR_INVALID_ARGUMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (wp->kvCount == 0 || wp->kvCapacity == 0) {   // the shader's rule: no rows -> zeros
        const cudaError_t e = cudaMemsetAsync(out, 0, static_cast<size_t>(wp->numHeads) * wp->headDim * sizeof(float), s);
        return e == cudaSuccess ? ER_OK : fail(ER_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    }
    Workspace* ws = nullptr;
    int32_t rc = get_workspace(&ws);
    if (rc != ER_OK) return rc;
    if (!flash_shape(wp->headDim, wp->numHeads, wp->numKVHeads))   // the reference's Gemma 4 head sizes (256 / 512) land here
        return generic_decode_row(ws, q, k, v, out, wp->numHeads, wp->numKVHeads, wp->headDim, wp->kvStart % wp->kvCapacity, wp->kvCount,
                                  wp->kvCapacity, wp->attentionScale != 0.f ? wp->attentionScale : 1.0f / std::sqrt(static_cast<float>(wp->headDim)), s);
    DecodeParams p{};
    p.q = q; p.out = out;
    p.k_base = reinterpret_cast<const uint8_t*>(k);
    p.v_base = reinterpret_cast<const uint8_t*>(v);
    p.lengths = nullptr;
    p.num_layers = 1; p.batch = 1;
    p.num_q_heads = static_cast<int>(wp->numHeads);
    const float scale = wp->attentionScale != 0.f ? wp->attentionScale : 1.0f / std::sqrt(static_cast<float>(wp->headDim));
    p.scale_log2 = scale * 1.4426950408889634f;
    p.rope_scaling = 1.f;
    p.addr.token_major = 1; p.addr.num_kv_heads = static_cast<int>(wp->numKVHeads);
    p.addr.max_seq_len = static_cast<int>(wp->kvCapacity); p.addr.page_size = static_cast<int>(wp->kvCapacity);
    p.scratch = ws->scratch; p.done_counter = ws->counters; p.status = ws->counters + 1; p.item_counters = ws->counters + 16;
    p.fixed_kv_len = static_cast<int>(wp->kvCount);
    p.fixed_start = static_cast<int>(wp->kvStart % wp->kvCapacity);
    const int group = static_cast<int>(wp->numHeads / wp->numKVHeads);
    encode_token_major_maps(p, group, 1, 1, wp->kvCapacity, wp->numKVHeads);   // used when the range starts at slot 0
    return dispatch_decode_f16(group, p, ws->num_sms, s);
}

int32_t er_gqa_attention_f32(const float* q, const float* k, const float* v, float* out, const float* additive_mask,
                             const ERGQAParams* gp, void* stream) {
    if (!q || !k || !v || !out || !gp) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    // GQAKernel.encode's preconditions (GQAKernel.swift:123-125)
    if (gp->numKVHeads == 0 || gp->numHeads % gp->numKVHeads != 0) return fail(ER_ERR_SHAPE, "numHeads %u not divisible by numKVHeads %u", gp->numHeads, gp->numKVHeads);
    if (gp->headDim == 0 || gp->headDim > 512 || gp->headDim % 4 != 0) return fail(ER_ERR_SHAPE, "headDim %u (1...512, divisible by 4)", gp->headDim);
    const uint32_t kv_seq = gp->kvSeqLen > 0 ? gp->kvSeqLen : gp->seqLen;
    if (gp->seqLen == 0) return ER_OK;
    AttentionF32Params fp{};
    fp.q = q; fp.out = out; fp.k = k; fp.v = v;
    fp.mask = additive_mask; fp.mask_stride = static_cast<int>(kv_seq);
    fp.seq_len = static_cast<int>(gp->seqLen); fp.head_dim = static_cast<int>(gp->headDim);
    fp.num_heads = static_cast<int>(gp->numHeads); fp.num_kv_heads = static_cast<int>(gp->numKVHeads);
    fp.causal = gp->causal ? 1 : 0; fp.q_offset = static_cast<int>(gp->qOffset); fp.kv_len = static_cast<int>(kv_seq);
    fp.scale = gp->scale != 0.f ? gp->scale : 1.0f / std::sqrt(static_cast<float>(gp->headDim));
    fp.addr.token_major = 1; fp.addr.num_kv_heads = static_cast<int>(gp->numKVHeads);
    fp.addr.max_seq_len = static_cast<int>(std::max<uint32_t>(kv_seq, 1)); fp.addr.page_size = fp.addr.max_seq_len;
    const int rc = launch_attention_f32(fp, 1, static_cast<cudaStream_t>(stream));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (rc == kNotBuilt) return fail(ER_ERR_UNSUPPORTED, "attention_f32_kernel: numHeads %u beyond the grid limit", gp->numHeads);
    if (rc != 0) return fail(ER_ERR_CUDA, "attention_f32_kernel: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    return ER_OK;
}

// ---- cache-level device operators ----

int32_t er_kv_append_rope_kv(er_kv* kv, uint32_t lb, uint32_t le, const float* k, const float* v, const er_step_params* sp, void* stream) {
    if (!kv || !k || !v) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    int32_t rc = check_layers(kv, lb, le);
    if (rc != ER_OK) return rc;
    if (kv->cfg.head_dim != kHeadDim) return fail(ER_ERR_UNSUPPORTED, "device append is built for head_dim 128");
    er_step_params s;
    if ((rc = step_defaults(kv, sp, s)) != ER_OK) return rc;
    if ((rc = check_device(kv)) != ER_OK) return rc;
    rc = apply_head_norm(kv, 1, &k, static_cast<size_t>(le - lb) * kv->cfg.max_batch * kv->cfg.num_kv_heads,
                         static_cast<size_t>(kv->cfg.max_batch) * kv->cfg.num_kv_heads, s.k_norm_weight, lb, s, static_cast<cudaStream_t>(stream));
    if (rc != ER_OK) return rc;
    std::lock_guard<std::mutex> lock(kv->mu);
    AppendParams ap{};
    ap.k = k; ap.v = v;
    ap.lengths = kv->d_lengths;
    ap.bulk = 0; ap.layer_begin = static_cast<int>(lb); ap.batch = static_cast<int>(kv->cfg.max_batch);
    ap.rows = static_cast<int>((le - lb) * kv->cfg.max_batch);
    ap.apply_rope = s.apply_rope ? 1 : 0; ap.rope_scaling = s.rope_scaling;
    if (ap.apply_rope) ap.inv_freq = kv->freq(s.rope_theta);
    return launch_append(kv, ap, static_cast<cudaStream_t>(stream));
}

int32_t er_kv_write_rows(er_kv* kv, uint32_t layer, uint32_t seq, uint32_t start, uint32_t count, const float* k, const float* v,
                         const er_step_params* sp, void* stream) {
    if (!kv || !k || !v) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (layer >= kv->cfg.num_layers) return fail(ER_ERR_INVALID_LAYER, "layer %u", layer);
    if (seq >= kv->cfg.max_batch) return fail(ER_ERR_INVALID_ARGUMENT, "sequence %u", seq);
    if (kv->cfg.head_dim != kHeadDim) return fail(ER_ERR_UNSUPPORTED, "device append is built for head_dim 128");
    if (static_cast<uint64_t>(start) + count > kv->cfg.max_seq_len) return fail(ER_ERR_SHAPE, "rows [%u, %u) exceed max_seq_len %u", start, start + count, kv->cfg.max_seq_len);
    er_step_params s;
    int32_t rc = step_defaults(kv, sp, s);
    if (rc != ER_OK) return rc;
    if ((rc = check_device(kv)) != ER_OK) return rc;
    {
        std::lock_guard<std::mutex> lock(kv->mu);
        if ((rc = check_page_coverage(kv, seq, static_cast<uint64_t>(start) + count)) != ER_OK) return rc;
    }
    rc = apply_head_norm(kv, 1, &k, static_cast<size_t>(count) * kv->cfg.num_kv_heads, static_cast<size_t>(count) * kv->cfg.num_kv_heads,
                         s.k_norm_weight, layer, s, static_cast<cudaStream_t>(stream));
    if (rc != ER_OK) return rc;
    std::lock_guard<std::mutex> lock(kv->mu);
    AppendParams ap{};
    ap.k = k; ap.v = v;
    ap.bulk = 1; ap.fixed_layer = static_cast<int>(layer); ap.fixed_seq = static_cast<int>(seq);
    ap.start_pos = static_cast<int>(start); ap.rows = static_cast<int>(count); ap.batch = static_cast<int>(kv->cfg.max_batch);
    ap.apply_rope = s.apply_rope ? 1 : 0; ap.rope_scaling = s.rope_scaling;
    if (ap.apply_rope) ap.inv_freq = kv->freq(s.rope_theta);
    rc = launch_append(kv, ap, static_cast<cudaStream_t>(stream));
    if (rc != ER_OK) return rc;
    set_min_length_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(kv->d_lengths + static_cast<size_t>(layer) * kv->cfg.max_batch + seq,
                                                                          static_cast<int>(start + count));
    return check_launch("set_min_length_kernel");
}

// One side (keys or values) of a cache as the SIMT attention kernel reads it.
static int32_t row_source(const er_kv* kv, bool is_value, RowSource& s) {
    s = RowSource{};
    s.rows = is_value ? kv->v_slab : kv->k_slab;
    s.layer_stride_bytes = is_value ? kv->v_layer_stride : kv->k_layer_stride;
    s.side = is_value ? kv->vn_slab : kv->kn_slab;
    s.side_layer_stride_bytes = kv->n_layer_stride;
    s.addr = kv->addressing();
    if (kv->cfg.head_dim != kHeadDim) return fail(ER_ERR_UNSUPPORTED, "attention kernels are built for head_dim 128");
    if (kv->outlier) {
        s.format = kRowsOutlier; s.ofmt = kv->ofmt;
        s.res_coef = kQjlScale * (is_value ? kv->cfg.value_residual_scale : kv->cfg.key_residual_scale);
    } else if (kv->turbo) {
        s.format = kRowsTurbo; s.bits = static_cast<int>(is_value ? kv->cfg.value_type : kv->cfg.key_type); s.norm_fp16 = kv->norm_bytes == 2;
    } else if (kv->q8) {
        s.format = kRowsQ8;
    } else if (kv->cfg.precision == ER_KV_FLOAT16 && !kv->token_major) {
        s.format = kRowsF16;
    } else {
        return fail(ER_ERR_UNSUPPORTED, "this kernel reads float16 (head-major or paged), q8_0 and TurboQuant rows");
    }
    return ER_OK;
}

// Attention of `rows_per_pair` query rows per (layer, sequence) with the K rows of `kk` and the V rows of `vv` (the same cache,
// or two caches of the same geometry holding the two sides of layers whose keys and values use different formats).
// kk->mu is held by the caller when kk == vv; otherwise both are taken here.
static int32_t simt_attention(er_kv* kk, er_kv* vv, uint32_t lb, uint32_t le, const float* q, float* out, uint32_t num_heads, uint32_t pending,
                              int rows_per_pair, int q_pos0, int fixed_seq, const er_step_params& s, cudaStream_t stream) {
    if (num_heads == 0 || num_heads % kk->cfg.num_kv_heads != 0) return fail(ER_ERR_SHAPE, "num_heads %u not divisible by num_kv_heads %u", num_heads, kk->cfg.num_kv_heads);
    const int group = static_cast<int>(num_heads / kk->cfg.num_kv_heads);
    const int pairs = fixed_seq >= 0 ? static_cast<int>(le - lb) : static_cast<int>((le - lb) * kk->cfg.max_batch);
    const int64_t problems = static_cast<int64_t>(pairs) * rows_per_pair;
    if (problems > 65535) return fail(ER_ERR_UNSUPPORTED, "%lld attention problems in one call; at most 65535", static_cast<long long>(problems));
    const int items = static_cast<int>(problems) * static_cast<int>(kk->cfg.num_kv_heads);
    int splits = std::max(1, (4 * std::max(kk->num_sms, 1) + items - 1) / items);
    splits = std::min(splits, std::max(1, static_cast<int>((kk->cfg.max_seq_len + 63) / 64)));
    const size_t need = static_cast<size_t>(items) * splits * group * kSimtPartialStride;
    if (kk->simt_partial_floats < need) {
        if (kk->d_simt_partial) cudaFree(kk->d_simt_partial);
        kk->d_simt_partial = nullptr;
        kk->simt_partial_floats = 0;
        if (cudaMalloc(&kk->d_simt_partial, need * sizeof(float)) != cudaSuccess) {
            cudaGetLastError();
            return fail(ER_ERR_ALLOCATION_FAILED, "split partials of %zu floats", need);
        }
        kk->simt_partial_floats = need;
    }
    SimtDecodeParams op{};
    int32_t rc = row_source(kk, false, op.k);
    if (rc != ER_OK) return rc;
    if ((rc = row_source(vv, true, op.v)) != ER_OK) return rc;
    op.q = q; op.out = out;
    op.lengths = kk->d_lengths; op.layer_begin = static_cast<int>(lb); op.batch = static_cast<int>(kk->cfg.max_batch);
    op.num_q_heads = static_cast<int>(num_heads); op.pending = static_cast<int>(pending); op.splits = splits;
    op.fixed_seq = fixed_seq; op.rows_per_pair = rows_per_pair; op.q_pos0 = q_pos0;
    op.window = static_cast<int>(std::min<uint32_t>(s.sliding_window, 0x7fffffffu));
    op.scale_log2 = s.softmax_scale * 1.4426950408889634f;
    op.apply_rope = s.apply_rope ? 1 : 0; op.rope_scaling = s.rope_scaling;
    if (op.apply_rope) op.inv_freq = kk->freq(s.rope_theta);
    op.partial = kk->d_simt_partial;
    if (kk->out_heads_total > 0) {
        if (kk->num_peers > 0) return fail(ER_ERR_UNSUPPORTED, "peer outputs are built for the flash-decode kernels");
        if (kk->out_head_offset + num_heads > kk->out_heads_total) return fail(ER_ERR_SHAPE, "output sharding: heads exceed %u", kk->out_heads_total);
        op.out_heads_total = static_cast<int>(kk->out_heads_total); op.out_head_offset = static_cast<int>(kk->out_head_offset);
    }
    const int orc = launch_simt_decode(group, op, pairs, stream);
    g_launches.fetch_add(2, std::memory_order_relaxed);
    if (orc != 0) return fail(orc == kNotBuilt ? ER_ERR_UNSUPPORTED : ER_ERR_CUDA, "simt_decode_kernel: %s",
                              orc == kNotBuilt ? "GQA groups 1, 2, 4, 8 are built" : cudaGetErrorString(static_cast<cudaError_t>(orc)));
    return ER_OK;
}

// float16 caches: launches over a small amount of rows (one layer of a small batch) skip the persistent kernel
static bool uses_slim_kernel(const er_kv* kv, uint32_t layers) {
    const uint64_t capacity_bytes = static_cast<uint64_t>(layers) * kv->cfg.max_batch * kv->cfg.num_kv_heads * kv->cfg.max_seq_len * 2 * kRowBytesF16;
    const bool automatic = kv->cfg.decode_kernel == ER_DECODE_KERNEL_AUTO || kv->cfg.decode_kernel == ER_DECODE_KERNEL_SIMT;
    return kv->cfg.decode_kernel == ER_DECODE_KERNEL_SLIM || (automatic && capacity_bytes <= (128ull << 20));
}

static int32_t attention_locked(er_kv* kv, uint32_t lb, uint32_t le, const float* q, float* out, uint32_t num_heads, uint32_t pending,
                                uint32_t advance, const er_step_params& s, cudaStream_t stream, const float* k_new = nullptr,
                                const float* v_new = nullptr) {
    if (kv->cfg.head_dim != kHeadDim) return fail(ER_ERR_UNSUPPORTED, "attention kernels are built for head_dim 128");
    if (num_heads == 0 || num_heads % kv->cfg.num_kv_heads != 0) return fail(ER_ERR_SHAPE, "num_heads %u not divisible by num_kv_heads %u", num_heads, kv->cfg.num_kv_heads);
    if (kv->cfg.precision == ER_KV_FLOAT32) {
        // float32 rows: the fp32 operator's kernel (gqa_attention_f32, Shaders/GQA.metal:18-143) reading the cache in place
        if (s.sliding_window > 0) return fail(ER_ERR_UNSUPPORTED, "sliding_window is built for float16 caches");
        AttentionF32Params fp{};
        fp.q = q; fp.out = out;
        fp.k = reinterpret_cast<const float*>(kv->k_slab); fp.v = reinterpret_cast<const float*>(kv->v_slab);
        fp.layer_stride_elems = kv->k_layer_stride / 4;
        fp.seq_len = 1; fp.head_dim = kHeadDim; fp.num_heads = static_cast<int>(num_heads); fp.num_kv_heads = static_cast<int>(kv->cfg.num_kv_heads);
        fp.causal = 0; fp.scale = s.softmax_scale;
        fp.lengths = kv->d_lengths; fp.layer_begin = static_cast<int>(lb); fp.batch = static_cast<int>(kv->cfg.max_batch); fp.pending = static_cast<int>(pending);
        fp.apply_rope = s.apply_rope ? 1 : 0; fp.rope_scaling = s.rope_scaling;
        if (fp.apply_rope) fp.inv_freq = kv->freq(s.rope_theta);
        fp.addr = kv->addressing();
        const int problems = static_cast<int>((le - lb) * kv->cfg.max_batch);
        const int frc = launch_attention_f32(fp, problems, stream);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        if (frc != 0) return fail(frc == kNotBuilt ? ER_ERR_UNSUPPORTED : ER_ERR_CUDA, "attention_f32_kernel: %s",
                                  frc == kNotBuilt ? "shape not covered" : cudaGetErrorString(static_cast<cudaError_t>(frc)));
        if (advance != 0) {
            add_lengths_kernel<<<(problems + 255) / 256, 256, 0, stream>>>(kv->d_lengths, static_cast<int>(lb * kv->cfg.max_batch), problems, static_cast<int>(advance));
            return check_launch("add_lengths_kernel");
        }
        return ER_OK;
    }
    const int group = static_cast<int>(num_heads / kv->cfg.num_kv_heads);
    // The SIMT kernel serves: balanced / aggressive rows (the general form of gqa_attention_turboquant_decode,
    // Shaders/TurboQuant.metal:1794-2001) with eight heads per kv head (OutlierMmaPolicy packs hi and lo parts into one n-tile:
    // up to four), sliding windows over q8_0 / TurboQuant rows (a window start that is not a multiple of 8 tokens breaks the
    // 16-byte alignment the bulk copies of the side arrays need), and TurboQuant caches created with ER_DECODE_KERNEL_SIMT.
    const bool outlier_simt = kv->outlier && (group > 4 || kv->cfg.decode_kernel == ER_DECODE_KERNEL_SIMT);
    const bool turbo_simt = kv->turbo && kv->cfg.decode_kernel == ER_DECODE_KERNEL_SIMT;
    if (outlier_simt || turbo_simt || (s.sliding_window > 0 && kv->cfg.precision != ER_KV_FLOAT16)) {
        const int32_t src = simt_attention(kv, kv, lb, le, q, out, num_heads, pending, 1, -1, -1, s, stream);
        if (src != ER_OK) return src;
        if (advance != 0) {
            const int pairs = static_cast<int>((le - lb) * kv->cfg.max_batch);
            add_lengths_kernel<<<(pairs + 255) / 256, 256, 0, stream>>>(kv->d_lengths, static_cast<int>(lb * kv->cfg.max_batch), pairs, static_cast<int>(advance));
            return check_launch("add_lengths_kernel");
        }
        return ER_OK;
    }
    // (layer, sequence) pairs are scheduled kMaxPairs at a time.
    const uint32_t layers_per_launch = std::max<uint32_t>(1, kMaxPairs / kv->cfg.max_batch);
    if (kv->cfg.max_batch > static_cast<uint32_t>(kMaxPairs)) return fail(ER_ERR_UNSUPPORTED, "max_batch %u > %d", kv->cfg.max_batch, kMaxPairs);
    for (uint32_t l0 = lb; l0 < le; l0 += layers_per_launch) {
        const uint32_t l1 = std::min(le, l0 + layers_per_launch);
        const size_t off = static_cast<size_t>(l0 - lb) * kv->cfg.max_batch * num_heads * kHeadDim;
        int32_t rc;
        DecodeParams p{};
        p.q = q + off; p.out = out + off;
        if (kv->out_heads_total > 0) {   // kv-head sharding: rows of out_heads_total heads, this cache's heads at an offset
            if (kv->out_head_offset + num_heads > kv->out_heads_total)
                return fail(ER_ERR_SHAPE, "output sharding: heads [%u, %u) exceed %u", kv->out_head_offset, kv->out_head_offset + num_heads, kv->out_heads_total);
            const size_t out_off = static_cast<size_t>(l0 - lb) * kv->cfg.max_batch * kv->out_heads_total * kHeadDim;
            p.out = out + out_off;
            p.out_heads_total = static_cast<int>(kv->out_heads_total); p.out_head_offset = static_cast<int>(kv->out_head_offset);
            p.num_peers = static_cast<int>(kv->num_peers);
            for (uint32_t r = 0; r < kv->num_peers; ++r) p.peer_out[r] = kv->peer_out[r] + out_off;
        }
        p.k_base = kv->k_slab; p.v_base = kv->v_slab;
        p.k_layer_stride_bytes = kv->k_layer_stride; p.v_layer_stride_bytes = kv->v_layer_stride;
        p.kn_base = kv->kn_slab; p.vn_base = kv->vn_slab; p.n_layer_stride_bytes = kv->n_layer_stride;
        p.norm_fp16 = kv->norm_bytes == 2;
        p.lengths = kv->d_lengths; p.layer_begin = static_cast<int>(l0); p.num_layers = static_cast<int>(l1 - l0);
        p.batch = static_cast<int>(kv->cfg.max_batch); p.num_q_heads = static_cast<int>(num_heads);
        p.pending = static_cast<int>(pending); p.advance = static_cast<int>(advance);
        if (k_new != nullptr) {
            const size_t kv_off = static_cast<size_t>(l0 - lb) * kv->cfg.max_batch * kv->cfg.num_kv_heads * kHeadDim;
            p.k_new = k_new + kv_off; p.v_new = v_new + kv_off; p.fused_append = 1;
        }
        p.trace = (kv->d_trace != nullptr && kv->trace_ctas >= static_cast<uint32_t>(kv->num_sms)) ? kv->d_trace : nullptr;
        p.scale_log2 = s.softmax_scale * 1.4426950408889634f;
        p.apply_rope = s.apply_rope ? 1 : 0; p.rope_scaling = s.rope_scaling;
        if (p.apply_rope) p.inv_freq = kv->freq(s.rope_theta);
        // only the fused fp16 step reaches here with weights set (the other entry points normalise beforehand)
        p.q_norm_w = s.q_norm_weight; p.k_norm_w = s.k_norm_weight;
        p.norm_stride = static_cast<int>(s.norm_weight_layer_stride); p.rms_eps = s.rms_eps;
        p.addr = kv->addressing();
        p.window = static_cast<int>(std::min<uint32_t>(s.sliding_window, 0x7fffffffu));
        p.wait_limit_us = kv->probe_wait_limit_us; p.withhold_tiles = kv->probe_withhold_tiles;
        p.scratch = kv->d_scratch; p.done_counter = kv->d_counters; p.status = kv->d_counters + 1; p.item_counters = kv->d_counters + 16;
        if (kv->outlier) {
            p.k_res_coef = kQjlScale * kv->cfg.key_residual_scale;
            p.v_res_coef = kQjlScale * kv->cfg.value_residual_scale;
            rc = decode_status(launch_decode_outlier(group, kv->ofmt.rb, kv->ofmt.hb, p, kv->num_sms, stream), group, kv->ofmt.rb, kv->ofmt.rb);
        } else if (kv->turbo)
            rc = decode_status(launch_decode_turbo(group, static_cast<int>(kv->cfg.key_type), static_cast<int>(kv->cfg.value_type), p, kv->num_sms, stream),
                               group, static_cast<int>(kv->cfg.key_type), static_cast<int>(kv->cfg.value_type));
        else if (kv->q8)
            rc = decode_status(launch_decode_q8(group, p, kv->num_sms, stream), group, 8, 8);
        else {
            // small launches (one layer of a small batch) skip the persistent kernel's staging pipeline
            const bool want_slim = uses_slim_kernel(kv, l1 - l0);
            int src = kNotBuilt;
            if (want_slim && kv->probe_withhold_tiles == 0) {
                const int items = static_cast<int>((l1 - l0) * kv->cfg.max_batch * kv->cfg.num_kv_heads);
                const int splits = decode_slim_splits(group, items, static_cast<int>((kv->cfg.max_seq_len + 15) / 16), kv->num_sms,
                                                      kScratchFloatsPerCta * static_cast<size_t>(std::max(kv->num_sms, 1)));
                // diagnostics buffer: one row of stamps per CTA of this grid
                p.trace = (kv->d_trace != nullptr && kv->trace_ctas >= static_cast<uint32_t>(items) * static_cast<uint32_t>(std::max(splits, 1))) ? kv->d_trace : nullptr;
                if (splits > 0) src = launch_decode_slim(group, p, splits, stream);
                if (src == kNotBuilt) p.trace = (kv->d_trace != nullptr && kv->trace_ctas >= static_cast<uint32_t>(kv->num_sms)) ? kv->d_trace : nullptr;
            }
            if (src != kNotBuilt) {
                rc = decode_status(src, group, 16, 16);
            } else {
                if (kv->token_major)
                    encode_token_major_maps(p, group, kv->cfg.num_layers, kv->cfg.max_batch, kv->cfg.max_seq_len, kv->cfg.num_kv_heads);
                if (kv->hostio_q != nullptr && p.fused_append && l0 == lb && l1 == le && kv->d_host_done != nullptr) {
                    // host-buffer step in one launch: the kernel pulls the rows itself and reports to the host word
                    p.host_q = kv->hostio_q; p.host_k = kv->hostio_k; p.host_v = kv->hostio_v;
                    p.host_done = kv->d_host_done; p.host_epoch = ++kv->host_epoch;
                    kv->hostio_used = true;
                }
                rc = dispatch_decode_f16(group, p, kv->num_sms, stream);
            }
        }
        if (rc != ER_OK) return rc;
    }
    return ER_OK;
}

int32_t er_kv_attention_decode(er_kv* kv, uint32_t lb, uint32_t le, const float* q, float* out, uint32_t num_heads, uint32_t pending,
                               const er_step_params* sp, void* stream) {
    if (!kv || !q || !out) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    int32_t rc = check_layers(kv, lb, le);
    if (rc != ER_OK) return rc;
    er_step_params s;
    if ((rc = step_defaults(kv, sp, s)) != ER_OK) return rc;
    if ((rc = check_device(kv)) != ER_OK) return rc;
    rc = apply_head_norm(kv, 0, &q, static_cast<size_t>(le - lb) * kv->cfg.max_batch * num_heads, static_cast<size_t>(kv->cfg.max_batch) * num_heads,
                         s.q_norm_weight, lb, s, static_cast<cudaStream_t>(stream));
    if (rc != ER_OK) return rc;
    s.q_norm_weight = nullptr;     // applied above; the kernel must not apply them again
    s.k_norm_weight = nullptr;
    std::lock_guard<std::mutex> lock(kv->mu);
    return attention_locked(kv, lb, le, q, out, num_heads, pending ? 1 : 0, 0, s, static_cast<cudaStream_t>(stream));
}

// ---- layers whose keys and values use different row formats: the two sides live in two caches of the same geometry ----

static int32_t check_pair(const er_kv* kk, const er_kv* vv) {
    if (kk->cfg.max_seq_len != vv->cfg.max_seq_len || kk->cfg.max_batch != vv->cfg.max_batch || kk->cfg.num_kv_heads != vv->cfg.num_kv_heads ||
        kk->cfg.num_layers != vv->cfg.num_layers || kk->device != vv->device)
        return fail(ER_ERR_SHAPE, "the key cache and the value cache of a pair must agree in max_seq_len, max_batch, num_kv_heads, num_layers and device");
    return ER_OK;
}

// q8_0 or float16 keys with TurboQuant values of a fixed preset (TurboValuesPolicy) and TurboQuant keys of a fixed preset with
// float16 or q8_0 values (TurboKeysPolicy) and q8_0 with float16 rows (PlainPairPolicy) run the persistent kernel; every other pair, sliding windows, sharded outputs and caches created with
// ER_DECODE_KERNEL_SIMT run the SIMT kernel.
static bool pair_has_tensor_core_policy(const er_kv* kk, const er_kv* vv, uint32_t num_heads, const er_step_params& s) {
    if (kk->cfg.head_dim != kHeadDim || vv->cfg.head_dim != kHeadDim) return false;
    if (s.sliding_window != 0 || kk->out_heads_total > 0) return false;
    if (kk->cfg.decode_kernel == ER_DECODE_KERNEL_SIMT || vv->cfg.decode_kernel == ER_DECODE_KERNEL_SIMT) return false;
    if (num_heads == 0 || num_heads % kk->cfg.num_kv_heads != 0) return false;
    const uint32_t group = num_heads / kk->cfg.num_kv_heads;
    if (group != 1 && group != 2 && group != 4 && group != 8) return false;
    if (kk->q8 && vv->turbo) return true;
    if (kk->turbo && vv->cfg.precision == ER_KV_FLOAT16 && !vv->token_major) return !(kk->cfg.key_type == ER_TQ_TURBO4 && group == 8);
    if (kk->turbo && vv->q8) return true;
    if (kk->cfg.precision == ER_KV_FLOAT16 && !kk->token_major && vv->turbo) return !(vv->cfg.value_type == ER_TQ_TURBO4 && group == 8);
    if (kk->q8 && vv->cfg.precision == ER_KV_FLOAT16 && !vv->token_major) return true;
    if (kk->cfg.precision == ER_KV_FLOAT16 && !kk->token_major && vv->q8) return true;
    return false;
}

// kk->mu is held by the caller; positions, scratch and counters are the key cache's.
static int32_t pair_attention_tensor_core(er_kv* kk, er_kv* vv, uint32_t lb, uint32_t le, const float* q, float* out, uint32_t num_heads,
                                          uint32_t pending, const er_step_params& s, cudaStream_t stream) {
    const int group = static_cast<int>(num_heads / kk->cfg.num_kv_heads);
    const uint32_t layers_per_launch = std::max<uint32_t>(1, kMaxPairs / kk->cfg.max_batch);
    if (kk->cfg.max_batch > static_cast<uint32_t>(kMaxPairs)) return fail(ER_ERR_UNSUPPORTED, "max_batch %u > %d", kk->cfg.max_batch, kMaxPairs);
    for (uint32_t l0 = lb; l0 < le; l0 += layers_per_launch) {
        const uint32_t l1 = std::min(le, l0 + layers_per_launch);
        const size_t off = static_cast<size_t>(l0 - lb) * kk->cfg.max_batch * num_heads * kHeadDim;
        DecodeParams p{};
        p.q = q + off; p.out = out + off;
        p.k_base = kk->k_slab; p.k_layer_stride_bytes = kk->k_layer_stride;
        p.kn_base = kk->kn_slab; p.n_layer_stride_bytes = kk->n_layer_stride;
        p.v_base = vv->v_slab; p.v_layer_stride_bytes = vv->v_layer_stride;
        p.vn_base = vv->vn_slab; p.vn_layer_stride_bytes = vv->n_layer_stride;
        p.norm_fp16 = (kk->turbo ? kk->norm_bytes : vv->norm_bytes) == 2;   // the TurboQuant side's stored norms
        p.lengths = kk->d_lengths; p.layer_begin = static_cast<int>(l0); p.num_layers = static_cast<int>(l1 - l0);
        p.batch = static_cast<int>(kk->cfg.max_batch); p.num_q_heads = static_cast<int>(num_heads);
        p.pending = static_cast<int>(pending);
        p.trace = nullptr;
        p.scale_log2 = s.softmax_scale * 1.4426950408889634f;
        p.apply_rope = s.apply_rope ? 1 : 0; p.rope_scaling = s.rope_scaling;
        if (p.apply_rope) p.inv_freq = kk->freq(s.rope_theta);
        p.addr = kk->addressing();
        p.addr_v = vv->addressing();
        p.wait_limit_us = kk->probe_wait_limit_us; p.withhold_tiles = kk->probe_withhold_tiles;
        p.scratch = kk->d_scratch; p.done_counter = kk->d_counters; p.status = kk->d_counters + 1; p.item_counters = kk->d_counters + 16;
        const bool plain = !kk->turbo && !vv->turbo;   // q8_0 with float16 rows
        const int32_t rc = plain ? decode_status(launch_decode_q8_dense_pair(group, kk->q8 ? 1 : 0, p, kk->num_sms, stream), group, kk->q8 ? 8 : 16, kk->q8 ? 16 : 8)
                         : kk->q8 ? decode_status(launch_decode_q8k_turbov(group, static_cast<int>(vv->cfg.value_type), p, kk->num_sms, stream), group, 8,
                                                  static_cast<int>(vv->cfg.value_type))
                         : !kk->turbo ? decode_status(launch_decode_densek_turbov(group, static_cast<int>(vv->cfg.value_type), p, kk->num_sms, stream), group, 16,
                                                      static_cast<int>(vv->cfg.value_type))
                         : vv->q8 ? decode_status(launch_decode_turbok_q8v(group, static_cast<int>(kk->cfg.key_type), p, kk->num_sms, stream), group,
                                                  static_cast<int>(kk->cfg.key_type), 8)
                                  : decode_status(launch_decode_turbok_densev(group, static_cast<int>(kk->cfg.key_type), p, kk->num_sms, stream), group,
                                                  static_cast<int>(kk->cfg.key_type), 16);
        if (rc != ER_OK) return rc;
    }
    return ER_OK;
}

int32_t er_kv_attention_decode_pair(er_kv* key_cache, er_kv* value_cache, uint32_t lb, uint32_t le, const float* q, float* out, uint32_t num_heads,
                                    uint32_t pending, const er_step_params* sp, void* stream) {
    if (!key_cache || !value_cache || !q || !out) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    int32_t rc = check_layers(key_cache, lb, le);
    if (rc != ER_OK) return rc;
    if ((rc = check_pair(key_cache, value_cache)) != ER_OK) return rc;
    er_step_params s;
    if ((rc = step_defaults(key_cache, sp, s)) != ER_OK) return rc;
    if ((rc = check_device(key_cache)) != ER_OK) return rc;
    rc = apply_head_norm(key_cache, 0, &q, static_cast<size_t>(le - lb) * key_cache->cfg.max_batch * num_heads,
                         static_cast<size_t>(key_cache->cfg.max_batch) * num_heads, s.q_norm_weight, lb, s, static_cast<cudaStream_t>(stream));
    if (rc != ER_OK) return rc;
    std::lock_guard<std::mutex> lock(key_cache->mu);
    if (pair_has_tensor_core_policy(key_cache, value_cache, num_heads, s))
        return pair_attention_tensor_core(key_cache, value_cache, lb, le, q, out, num_heads, pending ? 1 : 0, s, static_cast<cudaStream_t>(stream));
    return simt_attention(key_cache, value_cache, lb, le, q, out, num_heads, pending ? 1 : 0, 1, -1, -1, s, static_cast<cudaStream_t>(stream));
}

// One side of a (layer, sequence) as fp16 hi + lo rows, head-major [kv head][tpad][128], for the chunked-prefill kernels: what the
// single-cache prefill does for its own two sides, for a side taken from either cache of a pair.
static int32_t expand_side_for_prefill(er_kv* src, bool is_v, uint32_t layer, uint32_t seq, const int32_t* len_ptr, __half* dst, __half* dst_lo,
                                       int tpad, cudaStream_t cs) {
    const uint8_t* rows = (is_v ? src->v_slab : src->k_slab) + layer * (is_v ? src->v_layer_stride : src->k_layer_stride);
    const int64_t max_rows = static_cast<int64_t>(src->cfg.max_seq_len) * src->cfg.num_kv_heads;
    const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((max_rows + 7) / 8, 16384));
    if (src->outlier) {
        OutlierExpandParams ep{};
        ep.rows = rows; ep.out = dst; ep.out_lo = dst_lo; ep.fmt = src->ofmt; ep.addr = src->addressing(); ep.len_ptr = len_ptr;
        ep.seq = static_cast<int>(seq); ep.out_stride_rows = tpad;
        ep.res_coef = kQjlScale * (is_v ? src->cfg.value_residual_scale : src->cfg.key_residual_scale);
        tq_outlier_expand_rows_kernel<<<blocks, 256, 0, cs>>>(ep);
        return check_launch("tq_outlier_expand_rows_kernel");
    }
    if (src->turbo) {
        TurboExpandParams ep{};
        ep.codes = rows; ep.norms = (is_v ? src->vn_slab : src->kn_slab) + layer * src->n_layer_stride;
        ep.out = dst; ep.out_lo = dst_lo; ep.addr = src->addressing(); ep.len_ptr = len_ptr;
        ep.seq = static_cast<int>(seq); ep.out_stride_rows = tpad; ep.norm_fp16 = src->norm_bytes == 2;
        return launch_turbo_expand_rows(ep, static_cast<int>(is_v ? src->cfg.value_type : src->cfg.key_type), static_cast<int>(max_rows), cs, check_launch);
    }
    if (src->q8) {
        Q8ExpandParams ep{};
        ep.rows = rows; ep.scales = (is_v ? src->vn_slab : src->kn_slab) + layer * src->n_layer_stride;
        ep.out = dst; ep.out_lo = dst_lo; ep.addr = src->addressing(); ep.len_ptr = len_ptr;
        ep.seq = static_cast<int>(seq); ep.out_stride_rows = tpad;
        q8_expand_rows_f16_kernel<<<blocks, 256, 0, cs>>>(ep);
        return check_launch("q8_expand_rows_f16_kernel");
    }
    F16ExpandParams ep{};
    ep.rows = rows; ep.out = reinterpret_cast<uint8_t*>(dst); ep.out_lo = reinterpret_cast<uint8_t*>(dst_lo); ep.addr = src->addressing();
    ep.len_ptr = len_ptr; ep.seq = static_cast<int>(seq); ep.out_stride_rows = tpad;
    f16_expand_rows_kernel<<<blocks, 256, 0, cs>>>(ep);
    return check_launch("f16_expand_rows_kernel");
}

static bool prefill_side_is_expandable(const er_kv* c) {
    return c->cfg.head_dim == kHeadDim && (c->turbo || c->outlier || c->q8 || (c->cfg.precision == ER_KV_FLOAT16 && !c->token_major));
}

// Chunked prefill of a layer whose two sides live in two caches, on the tensor-core prefill kernels: both sides expanded to fp16
// hi + lo rows in the key cache's scratch (scores in the keys' space, outputs transformed back from the values' space).
// kk->mu is held by the caller.
static int32_t pair_prefill_tensor_core(er_kv* kk, er_kv* vv, uint32_t layer, uint32_t seq, const float* q, float* out, uint32_t num_heads,
                                        uint32_t seq_len, uint32_t q_offset, er_step_params s, cudaStream_t cs) {
    const int tpad = (static_cast<int>(kk->cfg.max_seq_len) + 15) & ~15;
    const size_t rows_bytes = static_cast<size_t>(kk->cfg.num_kv_heads) * tpad * kHeadDim * 2;
    const int n_qrows = static_cast<int>(seq_len * num_heads);
    const size_t q_bytes = static_cast<size_t>(n_qrows) * kHeadDim * 4;
    int32_t rc = ensure_stage(kk, 4 * rows_bytes + q_bytes + 256);
    if (rc != ER_OK) return rc;
    __half* ek = reinterpret_cast<__half*>(kk->d_stage);
    __half* ev = reinterpret_cast<__half*>(kk->d_stage + rows_bytes);
    __half* ekl = reinterpret_cast<__half*>(kk->d_stage + 2 * rows_bytes);
    __half* evl = reinterpret_cast<__half*>(kk->d_stage + 3 * rows_bytes);
    float* qrot = reinterpret_cast<float*>(kk->d_stage + 4 * rows_bytes);
    const int32_t* len_ptr = kk->d_lengths + static_cast<size_t>(layer) * kk->cfg.max_batch + seq;
    if ((rc = expand_side_for_prefill(kk, false, layer, seq, len_ptr, ek, ekl, tpad, cs)) != ER_OK) return rc;
    if ((rc = expand_side_for_prefill(vv, true, layer, seq, len_ptr, ev, evl, tpad, cs)) != ER_OK) return rc;
    PrefillParams pp{};
    pp.q = q; pp.out = out;
    if (kk->turbo || kk->outlier) {   // rotated keys: [RoPE ->] randomizedHadamard on the queries
        TurboRotateParams rp{};
        rp.in = q; rp.out = qrot; rp.rows = n_qrows; rp.heads = static_cast<int>(num_heads); rp.inverse = 0;
        rp.apply_rope = s.apply_rope ? 1 : 0; rp.rope_scaling = s.rope_scaling;
        if (rp.apply_rope) rp.inv_freq = kk->freq(s.rope_theta);
        rp.pos_from_len = q_offset == UINT32_MAX ? 1 : 0; rp.pos0 = q_offset == UINT32_MAX ? 0u : q_offset;
        rp.seq_len = static_cast<int>(seq_len); rp.len_ptr = len_ptr; rp.max_len = static_cast<int>(kk->cfg.max_seq_len);
        tq_rotate_rows_kernel<<<std::min((n_qrows + 7) / 8, 4096), 256, 0, cs>>>(rp);
        if ((rc = check_launch("tq_rotate_rows_kernel")) != ER_OK) return rc;
        pp.q = qrot;
        s.apply_rope = 0;
    }
    pp.k_layer = reinterpret_cast<const uint8_t*>(ek); pp.v_layer = reinterpret_cast<const uint8_t*>(ev);
    pp.k_lo_layer = reinterpret_cast<const uint8_t*>(ekl); pp.v_lo_layer = reinterpret_cast<const uint8_t*>(evl);
    pp.addr = kk->addressing();
    pp.addr.token_major = 0; pp.addr.pages_per_seq = 0; pp.addr.page_size = tpad; pp.addr.block_table = nullptr;
    pp.seq = 0; pp.seq_len = static_cast<int>(seq_len);
    pp.kv_len_ptr = len_ptr;
    {
        const size_t want = prefill_split_partial_floats(kk->num_sms);
        if (kk->d_prefill_partial == nullptr && cudaMalloc(&kk->d_prefill_partial, want * sizeof(float)) != cudaSuccess) {
            cudaGetLastError();
            kk->d_prefill_partial = nullptr;     // the kernel runs unsplit
        }
        pp.split_partial = kk->d_prefill_partial;
        pp.split_partial_floats = kk->d_prefill_partial ? want : 0;
    }
    pp.q_offset_from_end = q_offset == UINT32_MAX ? 1 : 0;
    pp.q_offset = static_cast<int>(q_offset == UINT32_MAX ? 0 : q_offset);
    pp.causal = 1;
    pp.window = 0;
    pp.num_q_heads = static_cast<int>(num_heads);
    pp.scale_log2 = s.softmax_scale * 1.4426950408889634f;
    pp.apply_rope = s.apply_rope ? 1 : 0; pp.rope_scaling = s.rope_scaling;
    if (pp.apply_rope) pp.inv_freq = kk->freq(s.rope_theta);
    const int rcl = launch_prefill(static_cast<int>(num_heads / kk->cfg.num_kv_heads), pp, 1u, static_cast<int>(kk->cfg.num_kv_heads), kk->d_counters + 1, cs,
                                   kk->cfg.prefill_kernel == ER_PREFILL_KERNEL_MMA_SYNC);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (rcl == -1) return fail(ER_ERR_UNSUPPORTED, "prefill kernel is built for GQA groups 1, 2, 4, 8");
    if (rcl != 0) return fail(ER_ERR_CUDA, "prefill_f16_kernel: %s", cudaGetErrorString(static_cast<cudaError_t>(rcl)));
    if (vv->turbo || vv->outlier) {   // rotated values: outputs back to the original space
        TurboRotateParams rp{};
        rp.in = out; rp.out = out; rp.rows = n_qrows; rp.heads = static_cast<int>(num_heads); rp.inverse = 1;
        tq_rotate_rows_kernel<<<std::min((n_qrows + 7) / 8, 4096), 256, 0, cs>>>(rp);
        if ((rc = check_launch("tq_rotate_rows_kernel")) != ER_OK) return rc;
    }
    return ER_OK;
}

int32_t er_kv_attention_prefill_pair(er_kv* key_cache, er_kv* value_cache, uint32_t layer, uint32_t seq, const float* q, float* out,
                                     uint32_t num_heads, uint32_t seq_len, uint32_t q_offset, const er_step_params* sp, void* stream) {
    if (!key_cache || !value_cache || !q || !out) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (layer >= key_cache->cfg.num_layers) return fail(ER_ERR_INVALID_LAYER, "layer %u", layer);
    if (seq >= key_cache->cfg.max_batch) return fail(ER_ERR_INVALID_ARGUMENT, "sequence %u", seq);
    if (seq_len == 0) return ER_OK;
    int32_t rc = check_pair(key_cache, value_cache);
    if (rc != ER_OK) return rc;
    er_step_params s;
    if ((rc = step_defaults(key_cache, sp, s)) != ER_OK) return rc;
    if ((rc = check_device(key_cache)) != ER_OK) return rc;
    rc = apply_head_norm(key_cache, 0, &q, static_cast<size_t>(seq_len) * num_heads, static_cast<size_t>(seq_len) * num_heads, s.q_norm_weight, layer, s,
                         static_cast<cudaStream_t>(stream));
    if (rc != ER_OK) return rc;
    std::lock_guard<std::mutex> lock(key_cache->mu);
    {   // the tensor-core prefill kernels take a chunk anywhere in the sequence
        const uint32_t group = num_heads / std::max<uint32_t>(key_cache->cfg.num_kv_heads, 1);
        if (s.sliding_window == 0 && key_cache->out_heads_total == 0 && num_heads % key_cache->cfg.num_kv_heads == 0 &&
            (group == 1 || group == 2 || group == 4 || group == 8) && prefill_side_is_expandable(key_cache) && prefill_side_is_expandable(value_cache) &&
            key_cache->cfg.decode_kernel != ER_DECODE_KERNEL_SIMT && value_cache->cfg.decode_kernel != ER_DECODE_KERNEL_SIMT)
            return pair_prefill_tensor_core(key_cache, value_cache, layer, seq, q, out, num_heads, seq_len, q_offset, s, static_cast<cudaStream_t>(stream));
    }
    // query row r sits at position q_offset + r (UINT32_MAX: the chunk's rows are the newest rows) and sees the keys up to it
    const int q_pos0 = q_offset == UINT32_MAX ? -1 : static_cast<int>(q_offset);
    if (q_pos0 >= 0) {
        // rows_per_pair counts back from the cache length: the chunk must end at the newest row
        if ((rc = pull_lengths(key_cache)) != ER_OK) return rc;
        const int32_t total = key_cache->h_lengths[static_cast<size_t>(layer) * key_cache->cfg.max_batch + seq];
        if (static_cast<int64_t>(q_offset) + seq_len != total)
            return fail(ER_ERR_UNSUPPORTED, "pair prefill: the chunk [%u, %u) must end at the sequence's %d rows", q_offset, q_offset + seq_len, total);
    }
    return simt_attention(key_cache, value_cache, layer, layer + 1, q, out, num_heads, 0, static_cast<int>(seq_len), q_pos0, static_cast<int>(seq), s,
                          static_cast<cudaStream_t>(stream));
}

int32_t er_kv_attention_prefill(er_kv* kv, uint32_t layer, uint32_t seq, const float* q, float* out, uint32_t num_heads,
                                uint32_t seq_len, uint32_t q_offset, const er_step_params* sp, void* stream) {
    if (!kv || !q || !out) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (layer >= kv->cfg.num_layers) return fail(ER_ERR_INVALID_LAYER, "layer %u", layer);
    if (seq >= kv->cfg.max_batch) return fail(ER_ERR_INVALID_ARGUMENT, "sequence %u", seq);
    if ((kv->cfg.precision != ER_KV_FLOAT16 && !kv->turbo && !kv->q8 && !kv->outlier) || kv->cfg.head_dim != kHeadDim)
        return fail(ER_ERR_UNSUPPORTED, "chunked prefill attention is built for float16, q8_0 and TurboQuant caches with head_dim 128");
    if (num_heads == 0 || num_heads % kv->cfg.num_kv_heads != 0) return fail(ER_ERR_SHAPE, "num_heads %u not divisible by num_kv_heads %u", num_heads, kv->cfg.num_kv_heads);
    if (seq_len == 0) return ER_OK;
    er_step_params s;
    int32_t rc = step_defaults(kv, sp, s);
    if (rc != ER_OK) return rc;
    if ((rc = check_device(kv)) != ER_OK) return rc;
    rc = apply_head_norm(kv, 0, &q, static_cast<size_t>(seq_len) * num_heads, static_cast<size_t>(seq_len) * num_heads, s.q_norm_weight, layer, s,
                         static_cast<cudaStream_t>(stream));
    if (rc != ER_OK) return rc;
    std::lock_guard<std::mutex> lock(kv->mu);
    if (s.sliding_window > 0 && kv->cfg.precision != ER_KV_FLOAT16) {
        // windowed chunks over q8_0 / TurboQuant rows: the SIMT kernel, a problem per query row (the chunk ends at the newest row)
        const int q_pos0 = q_offset == UINT32_MAX ? -1 : static_cast<int>(q_offset);
        if (q_pos0 >= 0) {
            if ((rc = pull_lengths(kv)) != ER_OK) return rc;
            const int32_t total = kv->h_lengths[static_cast<size_t>(layer) * kv->cfg.max_batch + seq];
            if (static_cast<int64_t>(q_offset) + seq_len != total)
                return fail(ER_ERR_UNSUPPORTED, "windowed prefill on this cache: the chunk [%u, %u) must end at the sequence's %d rows", q_offset, q_offset + seq_len, total);
        }
        return simt_attention(kv, kv, layer, layer + 1, q, out, num_heads, 0, static_cast<int>(seq_len), q_pos0, static_cast<int>(seq), s,
                              static_cast<cudaStream_t>(stream));
    }
    PrefillParams pp{};
    pp.q = q; pp.out = out;
    pp.k_layer = kv->k_slab + layer * kv->k_layer_stride;
    pp.v_layer = kv->v_slab + layer * kv->v_layer_stride;
    pp.addr = kv->addressing();
    pp.seq = static_cast<int>(seq); pp.seq_len = static_cast<int>(seq_len);
    pp.kv_len_ptr = kv->d_lengths + static_cast<size_t>(layer) * kv->cfg.max_batch + seq;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const int n_qrows = static_cast<int>(seq_len * num_heads);
    const bool rotated = kv->turbo || kv->outlier;
    if (rotated) {
        // Rotated-space formulation: expand the sequence's codes to fp16 rows norm*centroid, rotate the queries, run the
        // same tensor-core kernel, rotate the outputs back.
        const int tpad = (static_cast<int>(kv->cfg.max_seq_len) + 15) & ~15;
        const size_t rows_bytes = static_cast<size_t>(kv->cfg.num_kv_heads) * tpad * kHeadDim * 2;
        const size_t q_bytes = static_cast<size_t>(n_qrows) * kHeadDim * 4;
        rc = ensure_stage(kv, 4 * rows_bytes + q_bytes + 256);
        if (rc != ER_OK) return rc;
        __half* ek = reinterpret_cast<__half*>(kv->d_stage);
        __half* ev = reinterpret_cast<__half*>(kv->d_stage + rows_bytes);
        __half* ekl = reinterpret_cast<__half*>(kv->d_stage + 2 * rows_bytes);   // keys and values keep their fp16 rounding residue
        __half* evl = reinterpret_cast<__half*>(kv->d_stage + 3 * rows_bytes);
        float* qrot = reinterpret_cast<float*>(kv->d_stage + 4 * rows_bytes);
        for (int is_v = 0; is_v < 2 && kv->outlier; ++is_v) {   // effective coordinates: centroid + residual term, times rowNorm
            OutlierExpandParams ep{};
            ep.rows = (is_v ? kv->v_slab : kv->k_slab) + layer * (is_v ? kv->v_layer_stride : kv->k_layer_stride);
            ep.out = is_v ? ev : ek;
            ep.out_lo = is_v ? evl : ekl;
            ep.fmt = kv->ofmt; ep.addr = kv->addressing();
            ep.len_ptr = pp.kv_len_ptr;
            ep.seq = static_cast<int>(seq); ep.out_stride_rows = tpad;
            ep.res_coef = kQjlScale * (is_v ? kv->cfg.value_residual_scale : kv->cfg.key_residual_scale);
            const int64_t max_rows = static_cast<int64_t>(kv->cfg.max_seq_len) * kv->cfg.num_kv_heads;
            tq_outlier_expand_rows_kernel<<<static_cast<unsigned>(std::min<int64_t>((max_rows + 7) / 8, 16384)), 256, 0, cs>>>(ep);
            if ((rc = check_launch("tq_outlier_expand_rows_kernel")) != ER_OK) return rc;
        }
        for (int is_v = 0; is_v < 2 && kv->turbo; ++is_v) {
            TurboExpandParams ep{};
            ep.codes = (is_v ? kv->v_slab : kv->k_slab) + layer * (is_v ? kv->v_layer_stride : kv->k_layer_stride);
            ep.norms = (is_v ? kv->vn_slab : kv->kn_slab) + layer * kv->n_layer_stride;
            ep.out = is_v ? ev : ek;
            ep.out_lo = is_v ? evl : ekl;
            ep.addr = kv->addressing();
            ep.len_ptr = pp.kv_len_ptr;
            ep.seq = static_cast<int>(seq); ep.out_stride_rows = tpad; ep.norm_fp16 = kv->norm_bytes == 2;
            rc = launch_turbo_expand_rows(ep, static_cast<int>(is_v ? kv->cfg.value_type : kv->cfg.key_type),
                                          static_cast<int>(kv->cfg.max_seq_len * kv->cfg.num_kv_heads), cs, check_launch);
            if (rc != ER_OK) return rc;
        }
        TurboRotateParams rp{};
        rp.in = q; rp.out = qrot; rp.rows = n_qrows; rp.heads = static_cast<int>(num_heads); rp.inverse = 0;
        rp.apply_rope = s.apply_rope ? 1 : 0; rp.rope_scaling = s.rope_scaling;
        if (rp.apply_rope) rp.inv_freq = kv->freq(s.rope_theta);
        rp.pos_from_len = q_offset == UINT32_MAX ? 1 : 0; rp.pos0 = q_offset == UINT32_MAX ? 0u : q_offset;
        rp.seq_len = static_cast<int>(seq_len); rp.len_ptr = pp.kv_len_ptr; rp.max_len = static_cast<int>(kv->cfg.max_seq_len);
        tq_rotate_rows_kernel<<<std::min((n_qrows + 7) / 8, 4096), 256, 0, cs>>>(rp);
        if ((rc = check_launch("tq_rotate_rows_kernel")) != ER_OK) return rc;
        pp.q = qrot;
        pp.k_layer = reinterpret_cast<const uint8_t*>(ek);
        pp.v_layer = reinterpret_cast<const uint8_t*>(ev);
        pp.k_lo_layer = reinterpret_cast<const uint8_t*>(ekl);
        pp.v_lo_layer = reinterpret_cast<const uint8_t*>(evl);
        pp.addr.token_major = 0; pp.addr.pages_per_seq = 0; pp.addr.page_size = tpad; pp.addr.block_table = nullptr;
        pp.seq = 0;
        s.apply_rope = 0;
    }
    if (kv->q8) {
        // gqa_attention_q8kv with seqLen > 1 (Shaders/GQA.metal:409-522): rows expanded to scale * q as fp16 hi + lo (exact:
        // 11 + 7 significant bits), same tensor-core kernel
        const int tpad = (static_cast<int>(kv->cfg.max_seq_len) + 15) & ~15;
        const size_t rows_bytes = static_cast<size_t>(kv->cfg.num_kv_heads) * tpad * kHeadDim * 2;
        rc = ensure_stage(kv, 4 * rows_bytes + 256);
        if (rc != ER_OK) return rc;
        __half* ek = reinterpret_cast<__half*>(kv->d_stage);
        __half* ev = reinterpret_cast<__half*>(kv->d_stage + rows_bytes);
        __half* ekl = reinterpret_cast<__half*>(kv->d_stage + 2 * rows_bytes);
        __half* evl = reinterpret_cast<__half*>(kv->d_stage + 3 * rows_bytes);
        for (int is_v = 0; is_v < 2; ++is_v) {
            Q8ExpandParams ep{};
            ep.rows = (is_v ? kv->v_slab : kv->k_slab) + layer * (is_v ? kv->v_layer_stride : kv->k_layer_stride);
            ep.scales = (is_v ? kv->vn_slab : kv->kn_slab) + layer * kv->n_layer_stride;
            ep.out = is_v ? ev : ek;
            ep.out_lo = is_v ? evl : ekl;
            ep.addr = kv->addressing();
            ep.len_ptr = pp.kv_len_ptr;
            ep.seq = static_cast<int>(seq); ep.out_stride_rows = tpad;
            const int64_t max_rows = static_cast<int64_t>(kv->cfg.max_seq_len) * kv->cfg.num_kv_heads;
            q8_expand_rows_f16_kernel<<<static_cast<unsigned>(std::min<int64_t>((max_rows + 7) / 8, 16384)), 256, 0, cs>>>(ep);
            if ((rc = check_launch("q8_expand_rows_f16_kernel")) != ER_OK) return rc;
        }
        pp.k_layer = reinterpret_cast<const uint8_t*>(ek);
        pp.v_layer = reinterpret_cast<const uint8_t*>(ev);
        pp.k_lo_layer = reinterpret_cast<const uint8_t*>(ekl);
        pp.v_lo_layer = reinterpret_cast<const uint8_t*>(evl);
        pp.addr.token_major = 0; pp.addr.pages_per_seq = 0; pp.addr.page_size = tpad; pp.addr.block_table = nullptr;
        pp.seq = 0;
    }
    {   // scratch that lets the tcgen05 kernel cut the tail of its grid along the keys
        const size_t want = prefill_split_partial_floats(kv->num_sms);
        if (kv->d_prefill_partial == nullptr && cudaMalloc(&kv->d_prefill_partial, want * sizeof(float)) != cudaSuccess) {
            cudaGetLastError();
            kv->d_prefill_partial = nullptr;     // the kernel runs unsplit
        }
        pp.split_partial = kv->d_prefill_partial;
        pp.split_partial_floats = kv->d_prefill_partial ? want : 0;
    }
    pp.q_offset_from_end = q_offset == UINT32_MAX ? 1 : 0;
    pp.q_offset = static_cast<int>(q_offset == UINT32_MAX ? 0 : q_offset);
    pp.causal = 1;
    pp.window = static_cast<int>(std::min<uint32_t>(s.sliding_window, 0x7fffffffu));
    pp.num_q_heads = static_cast<int>(num_heads);
    pp.scale_log2 = s.softmax_scale * 1.4426950408889634f;
    pp.apply_rope = s.apply_rope ? 1 : 0; pp.rope_scaling = s.rope_scaling;
    if (pp.apply_rope) pp.inv_freq = kv->freq(s.rope_theta);
    const uint64_t outer_extent = (rotated || kv->q8) ? 1u : static_cast<uint64_t>(kv->pool_pages);
    const int rcl = launch_prefill(static_cast<int>(num_heads / kv->cfg.num_kv_heads), pp, outer_extent, static_cast<int>(kv->cfg.num_kv_heads),
                                   kv->d_counters + 1, static_cast<cudaStream_t>(stream), kv->cfg.prefill_kernel == ER_PREFILL_KERNEL_MMA_SYNC);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (rcl == -1) return fail(ER_ERR_UNSUPPORTED, "prefill kernel is built for GQA groups 1, 2, 4, 8");
    if (rcl != 0) return fail(ER_ERR_CUDA, "prefill_f16_kernel: %s", cudaGetErrorString(static_cast<cudaError_t>(rcl)));
    if (rotated) {
        TurboRotateParams rp{};
        rp.in = out; rp.out = out; rp.rows = n_qrows; rp.heads = static_cast<int>(num_heads); rp.inverse = 1;
        tq_rotate_rows_kernel<<<std::min((n_qrows + 7) / 8, 4096), 256, 0, cs>>>(rp);
        if ((rc = check_launch("tq_rotate_rows_kernel")) != ER_OK) return rc;
    }
    return ER_OK;
}

int32_t er_kv_advance(er_kv* kv, uint32_t lb, uint32_t le, uint32_t count, void* stream) {
    if (!kv) return fail(ER_ERR_INVALID_ARGUMENT, "null cache");
    int32_t rc = check_layers(kv, lb, le);
    if (rc != ER_OK) return rc;
    if ((rc = check_device(kv)) != ER_OK) return rc;
    const int n = static_cast<int>((le - lb) * kv->cfg.max_batch);
    add_lengths_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(kv->d_lengths, static_cast<int>(lb * kv->cfg.max_batch), n, static_cast<int>(count));
    return check_launch("add_lengths_kernel");
}

int32_t er_kv_decode_step(er_kv* kv, uint32_t lb, uint32_t le, const float* q, const float* k, const float* v, float* out,
                          uint32_t num_heads, const er_step_params* sp, void* stream) {
    if (!kv || !q || !k || !v || !out) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    int32_t rc = check_layers(kv, lb, le);
    if (rc != ER_OK) return rc;
    er_step_params s;
    if ((rc = step_defaults(kv, sp, s)) != ER_OK) return rc;
    if ((rc = check_device(kv)) != ER_OK) return rc;
    const uint32_t layers_per_launch = std::max<uint32_t>(1, kMaxPairs / kv->cfg.max_batch);
    const bool simt_rows = kv->outlier || (kv->turbo && kv->cfg.decode_kernel == ER_DECODE_KERNEL_SIMT) ||
                           (s.sliding_window > 0 && kv->cfg.precision != ER_KV_FLOAT16 && kv->cfg.precision != ER_KV_FLOAT32);
    const bool one_launch = le - lb <= layers_per_launch || kv->cfg.precision == ER_KV_FLOAT32 || simt_rows;
    // fp16 rows: the attention kernel appends the new row itself (one launch per step).  TurboQuant rows are
    // quantised by the append kernel first.
    const bool fused = kv->cfg.precision == ER_KV_FLOAT16 && kv->cfg.head_dim == kHeadDim;
    // Q / K head norms: the fp16 kernel applies them itself while it prepares Q and the new K row; the other formats run
    // one small launch per tensor first, and everything below sees normalised rows and no weights
    if (!fused) {
        rc = apply_head_norm(kv, 0, &q, static_cast<size_t>(le - lb) * kv->cfg.max_batch * num_heads, static_cast<size_t>(kv->cfg.max_batch) * num_heads,
                             s.q_norm_weight, lb, s, static_cast<cudaStream_t>(stream));
        if (rc != ER_OK) return rc;
        rc = apply_head_norm(kv, 1, &k, static_cast<size_t>(le - lb) * kv->cfg.max_batch * kv->cfg.num_kv_heads,
                             static_cast<size_t>(kv->cfg.max_batch) * kv->cfg.num_kv_heads, s.k_norm_weight, lb, s, static_cast<cudaStream_t>(stream));
        if (rc != ER_OK) return rc;
        s.q_norm_weight = nullptr;
        s.k_norm_weight = nullptr;
        rc = er_kv_append_rope_kv(kv, lb, le, k, v, &s, stream);
        if (rc != ER_OK) return rc;
    }
    std::lock_guard<std::mutex> lock(kv->mu);
    // The launch commits the appended row (lengths += 1) when its last CTA drains.
    rc = attention_locked(kv, lb, le, q, out, num_heads, 1, one_launch ? 1 : 0, s, static_cast<cudaStream_t>(stream),
                          fused ? k : nullptr, fused ? v : nullptr);
    if (rc != ER_OK || one_launch) return rc;
    const int n = static_cast<int>((le - lb) * kv->cfg.max_batch);
    add_lengths_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(kv->d_lengths, static_cast<int>(lb * kv->cfg.max_batch), n, 1);
    return check_launch("add_lengths_kernel");
}

// Device alias of a host pointer when the memory is pinned and mapped (cudaHostAlloc / cudaHostRegister under
// unified addressing), else nullptr.
static void* mapped_device_pointer(const void* host) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, host) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (attr.type != cudaMemoryTypeHost) return nullptr;
    return attr.devicePointer;
}

static bool is_device_pointer(const void* p) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return attr.type == cudaMemoryTypeDevice;
}

int32_t er_kv_decode_step_host(er_kv* kv, uint32_t lb, uint32_t le, const float* hq, const float* hk, const float* hv, float* hout,
                               uint32_t num_heads, const er_step_params* sp, void* stream) {
    if (!kv || !hq || !hk || !hv || !hout) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    int32_t rc = check_layers(kv, lb, le);
    if (rc != ER_OK) return rc;
    if ((rc = check_device(kv)) != ER_OK) return rc;
    const size_t rows = static_cast<size_t>(le - lb) * kv->cfg.max_batch;
    const size_t q_bytes = rows * num_heads * kv->cfg.head_dim * 4, kv_bytes = rows * kv->cfg.num_kv_heads * kv->cfg.head_dim * 4;
    {
        std::lock_guard<std::mutex> lock(kv->mu);
        rc = ensure_stage(kv, 2 * q_bytes + 2 * kv_bytes);
        if (rc != ER_OK) return rc;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint8_t* dq = kv->d_stage; uint8_t* dk = dq + q_bytes; uint8_t* dv = dk + kv_bytes; uint8_t* dout = dv + kv_bytes;
    const void* mq = mapped_device_pointer(hq);
    const void* mk = mapped_device_pointer(hk);
    const void* mv = mapped_device_pointer(hv);
    void* mout = mapped_device_pointer(hout);
    // `hout` may also name device memory (a kv-head shard's step writes into the gathered buffer): the rows then stay on the
    // device and the call returns as soon as its work is enqueued -- the host buffers must stay untouched until the stream
    // has passed the step, and the status word is read with er_kv_device_status.
    const bool out_on_device = mout == nullptr && is_device_pointer(hout);
    const bool mapped_in = mq && mk && mv && q_bytes % 16 == 0 && kv_bytes % 16 == 0;
    // float16 rows, one persistent launch for the whole call, everything pinned: no gather launch, no copy, no stream
    // synchronisation -- the decode kernel's producer warps pull the rows of their own item visits from the mapped buffers
    // while earlier tiles stream, its merging warps store the output rows into host memory, and its last CTA writes
    // {epoch, status} to a mapped host word this thread polls.
    bool in_kernel = false;
    if (mapped_in && (mout || out_on_device) && kv->cfg.precision == ER_KV_FLOAT16 && kv->cfg.head_dim == kHeadDim && kv->d_host_done != nullptr &&
        !uses_slim_kernel(kv, le - lb) && le - lb <= std::max<uint32_t>(1, kMaxPairs / kv->cfg.max_batch)) {
        std::lock_guard<std::mutex> lock(kv->mu);
        kv->hostio_q = static_cast<const float*>(mq); kv->hostio_k = static_cast<const float*>(mk); kv->hostio_v = static_cast<const float*>(mv);
        kv->hostio_used = false;
        in_kernel = true;
    }
    if (!in_kernel) {
        if (mapped_in) {
            // pinned inputs: one gather launch reads them over the bus
            const int nq4 = static_cast<int>(q_bytes / 16), nkv4 = static_cast<int>(kv_bytes / 16);
            const int blocks = std::min(2 * std::max(kv->num_sms, 1), (nq4 + 2 * nkv4 + 255) / 256);
            gather_host_inputs_kernel<<<blocks, 256, 0, s>>>(static_cast<const float4*>(mq), static_cast<const float4*>(mk),
                                                             static_cast<const float4*>(mv), reinterpret_cast<float4*>(dq),
                                                             reinterpret_cast<float4*>(dk), reinterpret_cast<float4*>(dv), nq4, nkv4);
            if ((rc = check_launch("gather_host_inputs_kernel")) != ER_OK) return rc;
        } else {
            ER_CUDA(cudaMemcpyAsync(dq, hq, q_bytes, cudaMemcpyHostToDevice, s));
            ER_CUDA(cudaMemcpyAsync(dk, hk, kv_bytes, cudaMemcpyHostToDevice, s));
            ER_CUDA(cudaMemcpyAsync(dv, hv, kv_bytes, cudaMemcpyHostToDevice, s));
        }
    }
    // pinned output: the merging warps store the rows straight into host memory
    float* step_out = out_on_device ? hout : (mout ? static_cast<float*>(mout) : reinterpret_cast<float*>(dout));
    rc = er_kv_decode_step(kv, lb, le, reinterpret_cast<const float*>(dq), reinterpret_cast<const float*>(dk), reinterpret_cast<const float*>(dv),
                           step_out, num_heads, sp, stream);
    bool signalled = false;
    int epoch = 0;
    if (in_kernel) {
        std::lock_guard<std::mutex> lock(kv->mu);
        kv->hostio_q = kv->hostio_k = kv->hostio_v = nullptr;
        signalled = kv->hostio_used;
        epoch = kv->host_epoch;
        kv->hostio_used = false;
    }
    if (rc != ER_OK) return rc;
    if (in_kernel && !signalled) return fail(ER_ERR_CUDA, "host-buffer step: the decode launch did not take the mapped rows");
    if (out_on_device) return ER_OK;
    if (signalled) {
        // the launch reports by itself; poll its word (its patience for device waits is 2 s, so well past that means a lost launch)
        volatile int* done = kv->h_status + 2;
        const auto t0 = std::chrono::steady_clock::now();
        uint32_t spins = 0;
        while (done[0] != epoch) {
            if ((++spins & 0xFFFu) == 0u && std::chrono::steady_clock::now() - t0 > std::chrono::seconds(10)) {
                ER_CUDA(cudaStreamSynchronize(s));
                if (done[0] != epoch) return fail(ER_ERR_CUDA, "host-buffer step: the launch ended without reporting");
            }
        }
        std::atomic_thread_fence(std::memory_order_acquire);
        return device_status_to_code(done[1]);
    }
    if (!mout) ER_CUDA(cudaMemcpyAsync(hout, dout, q_bytes, cudaMemcpyDeviceToHost, s));
    // the step's device status travels back with the results: a bounded wait that gave up, or a row without a page,
    // is this call's error and not garbage returned as success
    ER_CUDA(cudaMemcpyAsync(kv->h_status, kv->d_counters + 1, sizeof(int), cudaMemcpyDeviceToHost, s));
    ER_CUDA(cudaStreamSynchronize(s));
    return device_status_to_code(*kv->h_status);
}

// ---- pages as bytes: prefix reuse across sequences and caches of the same shape ----

namespace {
struct PageGeometry { size_t k, v, n; };   // bytes of one page of one layer in the K / V slabs and in each side slab
PageGeometry page_geometry(const er_kv* kv) {
    const size_t rows = static_cast<size_t>(kv->cfg.num_kv_heads) * static_cast<size_t>(kv->page_tokens);
    return {rows * kv->k_row_bytes, rows * kv->v_row_bytes, rows * kv->norm_bytes};
}
int32_t move_pages(er_kv* kv, const int32_t* page_ids, uint32_t count, uint8_t* buffer, size_t buffer_bytes, bool to_buffer, void* stream) {
    if (!kv || (!page_ids && count) || (!buffer && count)) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    if (kv->token_major) return fail(ER_ERR_UNSUPPORTED, "page export / import needs the head-major or the paged layout");
    int32_t rc = check_device(kv);
    if (rc != ER_OK) return rc;
    const PageGeometry g = page_geometry(kv);
    const size_t L = kv->cfg.num_layers, per_page = L * (g.k + g.v + 2 * g.n);
    if (buffer_bytes < per_page * count) return fail(ER_ERR_INVALID_ARGUMENT, "buffer of %zu bytes for %u pages of %zu bytes", buffer_bytes, count, per_page);
    for (uint32_t i = 0; i < count; ++i)
        if (page_ids[i] < 0 || page_ids[i] >= kv->pool_pages) return fail(ER_ERR_INVALID_ARGUMENT, "page %d of a pool of %d", page_ids[i], kv->pool_pages);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    std::lock_guard<std::mutex> lock(kv->mu);
    for (uint32_t i = 0; i < count; ++i) {
        uint8_t* at = buffer + per_page * i;
        // one strided copy per slab: `layers` runs of a page's bytes, a layer stride apart in the cache, packed in the buffer
        auto slab = [&](uint8_t* base, int64_t layer_stride, size_t bytes) -> cudaError_t {
            if (bytes == 0) return cudaSuccess;
            uint8_t* in_cache = base + static_cast<size_t>(page_ids[i]) * bytes;
            const cudaError_t e = to_buffer ? cudaMemcpy2DAsync(at, bytes, in_cache, static_cast<size_t>(layer_stride), bytes, L, cudaMemcpyDefault, s)
                                            : cudaMemcpy2DAsync(in_cache, static_cast<size_t>(layer_stride), at, bytes, bytes, L, cudaMemcpyDefault, s);
            at += bytes * L;
            return e;
        };
        ER_CUDA(slab(kv->k_slab, kv->k_layer_stride, g.k));
        ER_CUDA(slab(kv->v_slab, kv->v_layer_stride, g.v));
        ER_CUDA(slab(kv->kn_slab, kv->n_layer_stride, g.n));
        ER_CUDA(slab(kv->vn_slab, kv->n_layer_stride, g.n));
    }
    return ER_OK;
}
}  // namespace

int64_t er_kv_page_bytes(er_kv* kv) {
    if (!kv) return fail(ER_ERR_INVALID_ARGUMENT, "null cache");
    if (kv->token_major) return fail(ER_ERR_UNSUPPORTED, "page export / import needs the head-major or the paged layout");
    const PageGeometry g = page_geometry(kv);
    return static_cast<int64_t>(kv->cfg.num_layers * (g.k + g.v + 2 * g.n));
}
int32_t er_kv_export_pages(er_kv* kv, const int32_t* page_ids, uint32_t count, void* buffer, size_t buffer_bytes, void* stream) {
    return move_pages(kv, page_ids, count, static_cast<uint8_t*>(buffer), buffer_bytes, true, stream);
}
int32_t er_kv_import_pages(er_kv* kv, const int32_t* page_ids, uint32_t count, const void* buffer, size_t buffer_bytes, void* stream) {
    return move_pages(kv, page_ids, count, static_cast<uint8_t*>(const_cast<void*>(buffer)), buffer_bytes, false, stream);
}

int32_t er_kv_set_trace(er_kv* kv, uint64_t* device_buffer, uint32_t capacity_ctas) {
    if (!kv) return fail(ER_ERR_INVALID_ARGUMENT, "null cache");
    std::lock_guard<std::mutex> lock(kv->mu);
    kv->d_trace = reinterpret_cast<unsigned long long*>(device_buffer);
    kv->trace_ctas = device_buffer ? capacity_ctas : 0;
    return kv->num_sms;
}

int32_t er_kv_device_status(er_kv* kv) {
    if (!kv) return fail(ER_ERR_INVALID_ARGUMENT, "null cache");
    int status = 0;
    ER_CUDA(cudaMemcpy(&status, kv->d_counters + 1, sizeof(int), cudaMemcpyDeviceToHost));
    return device_status_to_code(status);
}

int32_t er_kv_set_output_sharding(er_kv* kv, uint32_t heads_total, uint32_t head_offset, float* const* peer_outputs, uint32_t num_peers) {
    if (!kv) return fail(ER_ERR_INVALID_ARGUMENT, "null cache");
    if (num_peers > 8 || (num_peers > 0 && (!peer_outputs || heads_total == 0))) return fail(ER_ERR_INVALID_ARGUMENT, "at most 8 peer buffers, and peers need heads_total > 0");
    if (kv->cfg.precision == ER_KV_FLOAT32 && heads_total > 0) return fail(ER_ERR_UNSUPPORTED, "output sharding is built for the flash-decode kernels (fp16, q8_0, TurboQuant rows)");
    for (uint32_t r = 0; r < num_peers; ++r)
        if (!peer_outputs[r] || (reinterpret_cast<uintptr_t>(peer_outputs[r]) & 15u)) return fail(ER_ERR_INVALID_ARGUMENT, "peer output %u is null or not 16-byte aligned", r);
    std::lock_guard<std::mutex> lock(kv->mu);
    kv->out_heads_total = heads_total; kv->out_head_offset = heads_total ? head_offset : 0; kv->num_peers = heads_total ? num_peers : 0;
    for (uint32_t r = 0; r < 8; ++r) kv->peer_out[r] = r < kv->num_peers ? peer_outputs[r] : nullptr;
    return ER_OK;
}

// ---- device buffers other processes on this node can map (CUDA IPC) ----

int32_t er_peer_buffer_create(size_t bytes, void** device_ptr, uint8_t* handle_out) {
    if (!device_ptr || !handle_out || bytes == 0) return fail(ER_ERR_INVALID_ARGUMENT, "null argument or zero size");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return fail(ER_ERR_ALLOCATION_FAILED, "peer buffer of %zu bytes", bytes); }
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) { cudaFree(p); cudaGetLastError(); return fail(ER_ERR_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e)); }
    ER_CUDA(cudaMemset(p, 0, bytes));
    std::memcpy(handle_out, &h, sizeof(h));
    *device_ptr = p;
    return ER_OK;
}

int32_t er_peer_buffer_open(const uint8_t* handle, void** device_ptr) {
    if (!handle || !device_ptr) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    const cudaError_t e = cudaIpcOpenMemHandle(device_ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(ER_ERR_CUDA, "cudaIpcOpenMemHandle: %s", cudaGetErrorString(e)); }
    return ER_OK;
}

int32_t er_peer_buffer_close(void* opened_ptr) {
    if (!opened_ptr) return ER_OK;
    ER_CUDA(cudaIpcCloseMemHandle(opened_ptr));
    return ER_OK;
}

int32_t er_peer_buffer_destroy(void* device_ptr) {
    if (!device_ptr) return ER_OK;
    ER_CUDA(cudaFree(device_ptr));
    return ER_OK;
}

int32_t er_relayout_head_shards(const float* gathered, float* full, uint32_t world, uint32_t pairs, uint32_t local_heads, void* stream) {
    if (!gathered || !full) return fail(ER_ERR_INVALID_ARGUMENT, "null argument");
    const uint64_t vec = static_cast<uint64_t>(world) * pairs * local_heads * (kHeadDim / 4);
    if (vec == 0) return ER_OK;
    relayout_head_shards_kernel<<<static_cast<unsigned>(std::min<uint64_t>((vec + 255) / 256, 148 * 16)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float4*>(gathered), reinterpret_cast<float4*>(full), world, pairs, local_heads);
    return check_launch("relayout_head_shards_kernel");
}

int32_t er_kv_debug_wait_probe(er_kv* kv, uint32_t wait_limit_us, int withhold_tiles) {
    if (!kv) return fail(ER_ERR_INVALID_ARGUMENT, "null cache");
    if (withhold_tiles && (wait_limit_us == 0 || wait_limit_us > 100000))
        return fail(ER_ERR_INVALID_ARGUMENT, "withholding the tiles needs a wait limit of 1 .. 100000 microseconds");
    std::lock_guard<std::mutex> lock(kv->mu);
    kv->probe_wait_limit_us = wait_limit_us;
    kv->probe_withhold_tiles = withhold_tiles ? 1 : 0;
    return ER_OK;
}

int32_t er_kv_clear_device_status(er_kv* kv) {
    if (!kv) return fail(ER_ERR_INVALID_ARGUMENT, "null cache");
    ER_CUDA(cudaMemset(kv->d_counters + 1, 0, sizeof(int)));
    return ER_OK;
}

int32_t er_workspace_status(void) {
    int device = 0;
    ER_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return ER_OK;
    int status = 0;
    {
        std::lock_guard<std::mutex> lock(g_ws_mu);
        if (g_ws[device].device != device) return ER_OK;   // no raw-buffer operator has run on this device yet
        ER_CUDA(cudaMemcpy(&status, g_ws[device].counters + 1, sizeof(int), cudaMemcpyDeviceToHost));
        if (status != 0) ER_CUDA(cudaMemset(g_ws[device].counters + 1, 0, sizeof(int)));
    }
    return device_status_to_code(status);
}

}  // extern "C"
