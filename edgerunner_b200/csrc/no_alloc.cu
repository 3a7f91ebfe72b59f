// er_gqa_attention_f16kv_static: the raw-buffer GQA attention operator for callers that must not allocate.
//
// The regular operator (er_gqa_attention_f16kv) keeps its split-K partials and counters in a workspace it
// cudaMalloc's on first use.  Some hosts cannot allow that: an inference server that has handed every free byte
// of the GPU to its own memory pool (a later cudaMalloc simply fails), or a runtime that forbids the implicit
// device synchronisation and driver locks an allocation takes in its latency-critical thread.  For them this
// file carries the workspace inside the library image: one file-scope device array, reserved on every GPU that
// loads the library for as long as the process lives.  Nothing in this translation unit allocates or frees
// device or pinned memory.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <mutex>

#include "../../include/er_kv.h"
#include "launchers.h"

namespace er {
int32_t report_error(int32_t code, const char* message);   // er_kv.cu: records the thread's last-error text
void count_kernel_launch();                                 // er_kv.cu: bumps er_kernel_launch_count()
}  // namespace er

namespace {

// Limits of the static workspace.
constexpr int kStaticMaxCtas = 256;        // CTAs of one launch (one per SM; a B200 has 148)
constexpr int kStaticMaxGroup = 4;         // query heads per kv head
constexpr int kStaticMaxKVHeads = 16;      // kv heads of one call
constexpr int kStaticCounterBytes = 1024;  // [0] CTAs done, [16 .. 16+kv heads) per-head counters, [255] device status
constexpr int kStaticStatusIndex = 255;    // outside the range each call re-zeroes: sticky until read
constexpr int kStaticPartialBytes = kStaticMaxCtas * 2 * kStaticMaxGroup * 130 * 4;   // two partial slots per CTA
constexpr int kStaticScratchBytes = kStaticCounterBytes + kStaticPartialBytes;        // 1 065 984 bytes (~1.02 MiB)

// The workspace itself.  In host code this name is only a handle for the runtime, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
unsigned char* g_device_scratch[kMaxDevices] = {};   // per device: device address of g_static_scratch

// First call on a device: resolve the array's device address with that device current.
int32_t static_scratch_for_current_device(unsigned char** out) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return er::report_error(ER_ERR_CUDA, cudaGetErrorString(e));
    if (device < 0 || device >= kMaxDevices) return er::report_error(ER_ERR_UNSUPPORTED, "device ordinal beyond 63");
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (g_device_scratch[device] == nullptr) {
        unsigned char* ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            char msg[160];
            std::snprintf(msg, sizeof(msg), "cudaGetSymbolAddress(static scratch) on device %d: %s", device, cudaGetErrorString(e));
            return er::report_error(ER_ERR_CUDA, msg);
        }
        g_device_scratch[device] = ptr;
    }
    *out = g_device_scratch[device];
    return ER_OK;
}

}  // namespace

extern "C" int32_t er_gqa_attention_f16kv_static(const float* q, const uint16_t* k, const uint16_t* v, float* out,
                                                 const ERGQAParams* gp, void* stream) {
    using namespace er;
    if (!q || !k || !v || !out || !gp) return report_error(ER_ERR_INVALID_ARGUMENT, "null argument");
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out)) & 15u)
        return report_error(ER_ERR_INVALID_ARGUMENT, "q, k, v and out must be 16-byte aligned device addresses");
    if (gp->headDim != kHeadDim) return report_error(ER_ERR_UNSUPPORTED, "headDim must be 128");
    if (gp->numKVHeads == 0 || gp->numHeads % gp->numKVHeads != 0) return report_error(ER_ERR_SHAPE, "numHeads must be a multiple of numKVHeads");
    const int group = static_cast<int>(gp->numHeads / gp->numKVHeads);
    char msg[200];
    if (gp->numKVHeads > static_cast<uint32_t>(kStaticMaxKVHeads) || group > kStaticMaxGroup) {
        std::snprintf(msg, sizeof(msg), "static workspace holds at most %d kv heads and %d query heads per kv head (got %u, %d); "
                      "use er_gqa_attention_f16kv", kStaticMaxKVHeads, kStaticMaxGroup, gp->numKVHeads, group);
        return report_error(ER_ERR_UNSUPPORTED, msg);
    }
    const uint32_t kv_seq = gp->kvSeqLen > 0 ? gp->kvSeqLen : gp->seqLen;
    if (gp->seqLen == 0 || kv_seq == 0) return ER_OK;
    unsigned char* scratch = nullptr;
    int32_t rc = static_scratch_for_current_device(&scratch);
    if (rc != ER_OK) return rc;
    int device = 0, num_sms = 0;
    cudaGetDevice(&device);
    cudaError_t e = cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return report_error(ER_ERR_CUDA, cudaGetErrorString(e));
    if (num_sms > kStaticMaxCtas) {
        std::snprintf(msg, sizeof(msg), "static workspace is sized for %d CTAs, the device has %d SMs", kStaticMaxCtas, num_sms);
        return report_error(ER_ERR_UNSUPPORTED, msg);
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left: the counters must start at zero (the status word stays).
    e = cudaMemsetAsync(scratch, 0, kStaticStatusIndex * sizeof(int), s);
    if (e != cudaSuccess) return report_error(ER_ERR_CUDA, cudaGetErrorString(e));

    int* counters = reinterpret_cast<int*>(scratch);
    DecodeParams p{};
    p.k_base = reinterpret_cast<const uint8_t*>(k);
    p.v_base = reinterpret_cast<const uint8_t*>(v);
    p.lengths = nullptr;
    p.layer_begin = 0; p.num_layers = 1; p.batch = 1;
    p.num_q_heads = static_cast<int>(gp->numHeads);
    const float scale = gp->scale != 0.f ? gp->scale : 1.0f / std::sqrt(static_cast<float>(gp->headDim));
    p.scale_log2 = scale * 1.4426950408889634f;
    p.rope_scaling = 1.f;
    p.addr.token_major = 1; p.addr.num_kv_heads = static_cast<int>(gp->numKVHeads);
    p.addr.max_seq_len = static_cast<int>(kv_seq); p.addr.page_size = static_cast<int>(kv_seq);
    p.scratch = reinterpret_cast<float*>(scratch + kStaticCounterBytes);
    p.done_counter = counters; p.status = counters + kStaticStatusIndex; p.item_counters = counters + 16;
    encode_token_major_maps(p, group, 1, 1, kv_seq, gp->numKVHeads);   // host-side descriptor encoding: no device allocation
    for (uint32_t r = 0; r < gp->seqLen; ++r) {   // row r sees keys 0 .. r + qOffset (Shaders/GQA.metal:345)
        const uint64_t visible = gp->causal ? (static_cast<uint64_t>(r) + gp->qOffset + 1 < kv_seq ? static_cast<uint64_t>(r) + gp->qOffset + 1 : kv_seq) : kv_seq;
        p.fixed_kv_len = static_cast<int>(visible);
        p.q = q + static_cast<size_t>(r) * gp->numHeads * kHeadDim;
        p.out = out + static_cast<size_t>(r) * gp->numHeads * kHeadDim;
        const int lrc = launch_decode_dense(group, p, num_sms, s);
        count_kernel_launch();
        if (lrc == kNotBuilt) return report_error(ER_ERR_UNSUPPORTED, "GQA group size is not built (1, 2, 4 are)");
        if (lrc != 0) return report_error(ER_ERR_CUDA, cudaGetErrorString(static_cast<cudaError_t>(lrc)));
    }
    return ER_OK;
}

// Reads (and clears) the status word the kernels of er_gqa_attention_f16kv_static leave in the built-in workspace of the
// current device: ER_ERR_DEVICE_TIMEOUT when a bounded wait inside one of them gave up.  Synchronises with the device;
// like the operator itself it allocates nothing.
extern "C" int32_t er_gqa_attention_f16kv_static_status(void) {
    using namespace er;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return report_error(ER_ERR_CUDA, cudaGetErrorString(e));
    unsigned char* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_setup_mu);
        if (device < 0 || device >= kMaxDevices || g_device_scratch[device] == nullptr) return ER_OK;   // never used here
        scratch = g_device_scratch[device];
    }
    int status = 0;
    int* word = reinterpret_cast<int*>(scratch) + kStaticStatusIndex;
    e = cudaMemcpy(&status, word, sizeof(int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && status != 0) e = cudaMemset(word, 0, sizeof(int));
    if (e != cudaSuccess) return report_error(ER_ERR_CUDA, cudaGetErrorString(e));
    if (status == kStatusTimeout) return report_error(ER_ERR_DEVICE_TIMEOUT, "a bounded wait inside a kernel gave up");
    return status == 0 ? ER_OK : report_error(ER_ERR_CUDA, "unexpected device status");
}
