// EdgeRunnerCUDA.hpp -- C++17 host-side mirror of the reference's Swift classes for the KV-cache path, written
// over the C ABI of er_kv.h (header-only; link against liber_kv.so).
//
// The reference is compiled Swift; no Swift toolchain exists in this build environment, so the host layer a Swift
// `EdgeRunnerCUDA` target would contain is written here in C++ with the same names, argument meaning and error
// behaviour:
//
//   edgerunner::KVCache            Sources/EdgeRunnerMetal/KVCache.swift:12-1138
//   edgerunner::KVCacheError       Sources/EdgeRunnerMetal/KVCache.swift:1141-1148  (thrown, like Swift `throws`)
//   edgerunner::GQAKernel          Sources/EdgeRunnerMetal/GQAKernel.swift:4-187
//   edgerunner::RoPEKernel         Sources/EdgeRunnerMetal/RoPEKernel.swift:4-307
//   edgerunner::TurboQuantKernel   Sources/EdgeRunnerMetal/TurboQuantKernel.swift:13-112
//   edgerunner::BlockTableAllocator  (new: the reference has no paging; the allocator lives on the host side)
//
// MTLBuffer arguments become raw device pointers, MTLCommandBuffer becomes a cudaStream_t passed as void*.
#pragma once

#include <algorithm>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "er_kv.h"

namespace edgerunner {

// KVCacheError cases (KVCache.swift:1141-1148) plus the statuses that have no Swift counterpart.
class KVCacheError : public std::runtime_error {
public:
    enum Case {
        allocationFailed = ER_ERR_ALLOCATION_FAILED,
        invalidLayer = ER_ERR_INVALID_LAYER,
        precisionMismatch = ER_ERR_PRECISION_MISMATCH,
        unsupportedStorage = ER_ERR_UNSUPPORTED_STORAGE,
        compressedRetrieveRequiresDecodedAPI = ER_ERR_COMPRESSED_RETRIEVE_REQUIRES_DECODED_API,
        compressedBufferAccessRequiresTurboQuantAPI = ER_ERR_COMPRESSED_BUFFER_ACCESS_REQUIRES_TURBOQUANT_API,
        shape = ER_ERR_SHAPE,
        cuda = ER_ERR_CUDA,
        invalidArgument = ER_ERR_INVALID_ARGUMENT,
        outOfPages = ER_ERR_OUT_OF_PAGES,
        unsupported = ER_ERR_UNSUPPORTED,
        deviceTimeout = ER_ERR_DEVICE_TIMEOUT
    };
    explicit KVCacheError(int32_t code)
        : std::runtime_error(std::string(er_status_string(code)) + ": " + er_last_error_string()), code_(code) {}
    Case which() const { return static_cast<Case>(code_); }
    int32_t code() const { return code_; }

private:
    int32_t code_;
};

inline int32_t check(int32_t status) {
    if (status < 0) throw KVCacheError(status);
    return status;
}

struct TurboQuantRuntimeRows {   // retrieveTurboQuantRuntimeRows, KVCache.swift:588-629
    std::vector<uint32_t> codes, residualSigns, outlierMask;
    std::vector<float> metadata;   // (rowNorm, residualNorm) pairs
    uint32_t rowCount = 0;
    uint32_t codeWordsPerRow = 0;
};

class KVCache {
public:
    enum class Precision : uint32_t {   // KVCache.Precision raw values, KVCache.swift:39-49
        float32 = ER_KV_FLOAT32, float16 = ER_KV_FLOAT16, float8 = ER_KV_FLOAT8, q8_0 = ER_KV_Q8_0,
        turboquantV2 = ER_KV_TURBOQUANT_V2, turboQuantBalanced = ER_KV_TURBOQUANT_BALANCED,
        turboQuantAggressive = ER_KV_TURBOQUANT_AGGRESSIVE
    };
    enum class Layout : uint32_t { tokenMajor = ER_KV_LAYOUT_TOKEN_MAJOR, headMajor = ER_KV_LAYOUT_HEAD_MAJOR, paged = ER_KV_LAYOUT_PAGED };

    struct Options {
        uint32_t keyType = ER_TQ_TURBO3, valueType = ER_TQ_TURBO3;   // TurboQuantV2Contract defaults, TurboQuant.swift:343-355
        uint32_t normFormat = ER_TQ_NORM_FLOAT32;
        uint32_t maxBatch = 1;
        Layout layout = Layout::headMajor;
        uint32_t pageSize = 0, numPages = 0;
        uint32_t prefillKernel = ER_PREFILL_KERNEL_AUTO, decodeKernel = ER_DECODE_KERNEL_AUTO;   // A/B switches, er_kv_config
        float keyResidualScale = 0.f, valueResidualScale = 0.f;   // balanced / aggressive rows: TurboQuantV2Contract's residual scales
    };

    // KVCache.init(device:maxSeqLen:numLayers:numKVHeads:headDim:precision:) throws, KVCache.swift:192-275
    KVCache(int maxSeqLen, int numLayers, int numKVHeads, int headDim, Precision precision, const Options& opt)
        : maxSeqLen(maxSeqLen), numLayers(numLayers), numKVHeads(numKVHeads), headDim(headDim), precision(precision) {
        er_kv_config c{};
        c.max_seq_len = static_cast<uint32_t>(maxSeqLen);
        c.num_layers = static_cast<uint32_t>(numLayers);
        c.num_kv_heads = static_cast<uint32_t>(numKVHeads);
        c.head_dim = static_cast<uint32_t>(headDim);
        c.precision = static_cast<uint32_t>(precision);
        c.key_type = opt.keyType;
        c.value_type = opt.valueType;
        c.norm_format = opt.normFormat;
        c.max_batch = opt.maxBatch;
        c.layout = static_cast<uint32_t>(opt.layout);
        c.page_size = opt.pageSize;
        c.num_pages = opt.numPages;
        c.prefill_kernel = opt.prefillKernel;
        c.decode_kernel = opt.decodeKernel;
        c.key_residual_scale = opt.keyResidualScale;
        c.value_residual_scale = opt.valueResidualScale;
        if (precision == Precision::turboQuantBalanced || precision == Precision::turboQuantAggressive) {
            // key_type / value_type name the channel-selection rules there; 0 = the contract's (magnitude / quantisation benefit)
            if (c.key_type > ER_TQ_SELECT_QUANTIZATION_BENEFIT) c.key_type = ER_TQ_SELECT_DEFAULT;
            if (c.value_type > ER_TQ_SELECT_QUANTIZATION_BENEFIT) c.value_type = ER_TQ_SELECT_DEFAULT;
        }
        check(er_kv_create(&c, &handle_));
        options_ = opt;
    }
    KVCache(int maxSeqLen, int numLayers, int numKVHeads, int headDim, Precision precision)
        : KVCache(maxSeqLen, numLayers, numKVHeads, headDim, precision, Options()) {}
    ~KVCache() { er_kv_destroy(handle_); }
    KVCache(const KVCache&) = delete;
    KVCache& operator=(const KVCache&) = delete;

    const int maxSeqLen, numLayers, numKVHeads, headDim;
    const Precision precision;

    int elementsPerToken() const { return numKVHeads * headDim; }
    bool isTurboQuant() const {   // KVCache.Precision.isTurboQuant
        return precision == Precision::turboquantV2 || precision == Precision::turboQuantBalanced || precision == Precision::turboQuantAggressive;
    }
    int currentLength() const { return check(er_kv_current_length(handle_)); }
    er_kv* handle() const { return handle_; }

    // append(layer:keys:values:) / appendF16, KVCache.swift:410-476
    void append(int layer, const std::vector<float>& keys, const std::vector<float>& values, uint32_t seq = 0) {
        if (keys.size() != values.size()) throw KVCacheError(ER_ERR_SHAPE);
        check(er_kv_append_f32(handle_, static_cast<uint32_t>(layer), seq, keys.data(), values.data(), keys.size()));
    }
    void appendF16(int layer, const std::vector<uint16_t>& keys, const std::vector<uint16_t>& values, uint32_t seq = 0) {
        if (keys.size() != values.size()) throw KVCacheError(ER_ERR_SHAPE);
        check(er_kv_append_f16(handle_, static_cast<uint32_t>(layer), seq, keys.data(), values.data(), keys.size()));
    }

    // retrieve(layer:asType:), KVCache.swift:478-522.  T = float or uint16_t (fp16 bits).
    template <typename T>
    std::pair<std::vector<T>, std::vector<T>> retrieve(int layer, uint32_t seq = 0) const {
        const size_t cap = static_cast<size_t>(maxSeqLen) * elementsPerToken();
        std::vector<T> k(cap), v(cap);
        uint32_t tokens = 0;
        check(er_kv_retrieve(handle_, static_cast<uint32_t>(layer), seq, sizeof(T), k.data(), v.data(), cap, &tokens));
        k.resize(static_cast<size_t>(tokens) * elementsPerToken());
        v.resize(k.size());
        return {std::move(k), std::move(v)};
    }

    // retrieveDecodedTurboQuant, KVCache.swift:524-586
    std::pair<std::vector<float>, std::vector<float>> retrieveDecodedTurboQuant(int layer, uint32_t seq = 0) const {
        const size_t cap = static_cast<size_t>(maxSeqLen) * elementsPerToken();
        std::vector<float> k(cap), v(cap);
        uint32_t tokens = 0;
        check(er_kv_retrieve_decoded_turboquant(handle_, static_cast<uint32_t>(layer), seq, k.data(), v.data(), cap, &tokens));
        k.resize(static_cast<size_t>(tokens) * elementsPerToken());
        v.resize(k.size());
        return {std::move(k), std::move(v)};
    }

    // retrieveDecodedQ8_0, KVCache.swift:882-908
    std::pair<std::vector<float>, std::vector<float>> retrieveDecodedQ8_0(int layer, uint32_t seq = 0) const {
        const size_t cap = static_cast<size_t>(maxSeqLen) * elementsPerToken();
        std::vector<float> k(cap), v(cap);
        uint32_t tokens = 0;
        check(er_kv_retrieve_decoded_q8_0(handle_, static_cast<uint32_t>(layer), seq, k.data(), v.data(), cap, &tokens));
        k.resize(static_cast<size_t>(tokens) * elementsPerToken());
        v.resize(k.size());
        return {std::move(k), std::move(v)};
    }

    // retrieveTurboQuantRuntimeRows, KVCache.swift:588-629
    TurboQuantRuntimeRows retrieveTurboQuantRuntimeRows(int layer, bool values, uint32_t seq = 0) const {
        TurboQuantRuntimeRows r;
        const uint32_t bits = values ? options_.valueType : options_.keyType;
        r.codeWordsPerRow = (128 * bits + 31) / 32;
        if (precision == Precision::turboQuantBalanced) r.codeWordsPerRow = 14;    // TurboQuantReferenceTests.swift:112-143
        if (precision == Precision::turboQuantAggressive) r.codeWordsPerRow = 9;
        const size_t cap = static_cast<size_t>(maxSeqLen) * numKVHeads;
        r.codes.resize(cap * r.codeWordsPerRow);
        r.residualSigns.resize(cap * 4);
        r.outlierMask.resize(cap * 4);
        r.metadata.resize(cap * 2);
        check(er_kv_retrieve_turboquant_rows(handle_, static_cast<uint32_t>(layer), seq, values ? 1 : 0, r.codes.data(),
                                             r.residualSigns.data(), r.outlierMask.data(), r.metadata.data(), cap, &r.rowCount));
        r.codes.resize(static_cast<size_t>(r.rowCount) * r.codeWordsPerRow);
        r.residualSigns.resize(static_cast<size_t>(r.rowCount) * 4);
        r.outlierMask.resize(static_cast<size_t>(r.rowCount) * 4);
        r.metadata.resize(static_cast<size_t>(r.rowCount) * 2);
        return r;
    }

    // metalBuffers(layer:): dense-path accessor, throws compressedBufferAccessRequiresTurboQuantAPI on TurboQuant
    // storage (KVCache.swift:631-634, 836-848).  Returns (key, value) device pointers.
    std::pair<void*, void*> metalBuffers(int layer) const {
        er_kv_buffers b{};
        check(er_kv_device_buffers(handle_, static_cast<uint32_t>(layer), &b));
        if (isTurboQuant()) throw KVCacheError(ER_ERR_COMPRESSED_BUFFER_ACCESS_REQUIRES_TURBOQUANT_API);
        return {b.keys, b.values};
    }
    // turboQuantMetalBuffers(layer:), KVCache.swift:647-667
    er_kv_buffers turboQuantMetalBuffers(int layer) const {
        er_kv_buffers b{};
        check(er_kv_device_buffers(handle_, static_cast<uint32_t>(layer), &b));
        if (!isTurboQuant()) throw KVCacheError(ER_ERR_PRECISION_MISMATCH);
        return b;
    }

    ERKVCacheParams cacheParams(int layer, uint32_t seq = 0) const {   // KVCache.swift:691-703
        ERKVCacheParams p{};
        check(er_kv_cache_params(handle_, static_cast<uint32_t>(layer), seq, &p));
        return p;
    }
    void reset() { check(er_kv_reset(handle_)); }                                               // KVCache.swift:705-711
    void advanceWritePosition(int layer, int count, uint32_t seq = UINT32_MAX) {                // KVCache.swift:713-720
        check(er_kv_advance_write_position(handle_, static_cast<uint32_t>(layer), seq, static_cast<uint32_t>(count)));
    }
    void setPosition(int position, uint32_t seq = UINT32_MAX) {                                 // KVCache.swift:722-729
        check(er_kv_set_position(handle_, seq, static_cast<uint32_t>(position)));
    }
    void setBlockTable(uint32_t seq, const std::vector<int32_t>& pages) {
        check(er_kv_set_block_table(handle_, seq, pages.data(), static_cast<uint32_t>(pages.size())));
    }

    // One decode step of layers [layerBegin, layerEnd): append + attention + advance (the body of fusedDecodePass
    // steps 2-5, Sources/EdgeRunner/Models/LlamaLanguageModel.swift:3649-3941).  Device pointers.
    void decodeStep(int layerBegin, int layerEnd, const float* q, const float* k, const float* v, float* out, int numHeads,
                    const er_step_params& params, void* stream = nullptr) {
        check(er_kv_decode_step(handle_, static_cast<uint32_t>(layerBegin), static_cast<uint32_t>(layerEnd), q, k, v, out,
                                static_cast<uint32_t>(numHeads), &params, stream));
    }
    // Same with host buffers.
    void decodeStepHost(int layerBegin, int layerEnd, const float* q, const float* k, const float* v, float* out, int numHeads,
                        const er_step_params& params, void* stream = nullptr) {
        check(er_kv_decode_step_host(handle_, static_cast<uint32_t>(layerBegin), static_cast<uint32_t>(layerEnd), q, k, v, out,
                                     static_cast<uint32_t>(numHeads), &params, stream));
    }

    // The pieces of a step (LlamaLanguageModel.swift:3649-3941): append without advancing, attention over the rows plus
    // `pending` uncommitted ones, advance.
    void appendRoPEKV(int layerBegin, int layerEnd, const float* k, const float* v, const er_step_params& params, void* stream = nullptr) {
        check(er_kv_append_rope_kv(handle_, static_cast<uint32_t>(layerBegin), static_cast<uint32_t>(layerEnd), k, v, &params, stream));
    }
    void attentionDecode(int layerBegin, int layerEnd, const float* q, float* out, int numHeads, int pending, const er_step_params& params,
                         void* stream = nullptr) {
        check(er_kv_attention_decode(handle_, static_cast<uint32_t>(layerBegin), static_cast<uint32_t>(layerEnd), q, out,
                                     static_cast<uint32_t>(numHeads), static_cast<uint32_t>(pending), &params, stream));
    }
    void advance(int layerBegin, int layerEnd, int count = 1, void* stream = nullptr) {
        check(er_kv_advance(handle_, static_cast<uint32_t>(layerBegin), static_cast<uint32_t>(layerEnd), static_cast<uint32_t>(count), stream));
    }
    // Prefill: rows [start, start + count) of one (layer, sequence) from device float [count][numKVHeads][headDim], then
    // causal attention of a chunk of query rows (prefill dispatch, LlamaLanguageModel.swift:2286, 2940-2957).
    void writeRows(int layer, uint32_t seq, int start, int count, const float* k, const float* v, const er_step_params& params,
                   void* stream = nullptr) {
        check(er_kv_write_rows(handle_, static_cast<uint32_t>(layer), seq, static_cast<uint32_t>(start), static_cast<uint32_t>(count), k, v,
                               &params, stream));
    }
    void attentionPrefill(int layer, uint32_t seq, const float* q, float* out, int numHeads, int seqLen, int qOffset,
                          const er_step_params& params, void* stream = nullptr) {
        check(er_kv_attention_prefill(handle_, static_cast<uint32_t>(layer), seq, q, out, static_cast<uint32_t>(numHeads),
                                      static_cast<uint32_t>(seqLen), static_cast<uint32_t>(qOffset), &params, stream));
    }
    // Layers whose keys and values use different row formats: attention with THIS cache's K rows and `values`' V rows.
    void attentionDecodeWithValuesOf(const KVCache& values, int layerBegin, int layerEnd, const float* q, float* out, int numHeads,
                                     int pending, const er_step_params& params, void* stream = nullptr) {
        check(er_kv_attention_decode_pair(handle_, values.handle_, static_cast<uint32_t>(layerBegin), static_cast<uint32_t>(layerEnd), q, out,
                                          static_cast<uint32_t>(numHeads), static_cast<uint32_t>(pending), &params, stream));
    }
    void attentionPrefillWithValuesOf(const KVCache& values, int layer, uint32_t seq, const float* q, float* out, int numHeads, int seqLen,
                                      int qOffset, const er_step_params& params, void* stream = nullptr) {
        check(er_kv_attention_prefill_pair(handle_, values.handle_, static_cast<uint32_t>(layer), seq, q, out, static_cast<uint32_t>(numHeads),
                                           static_cast<uint32_t>(seqLen), static_cast<uint32_t>(qOffset), &params, stream));
    }
    int64_t totalWritten(int layer, uint32_t seq = 0) const { return er_kv_total_written(handle_, static_cast<uint32_t>(layer), seq); }
    er_kv_config config() const {
        er_kv_config c{};
        check(er_kv_get_config(handle_, &c));
        return c;
    }
    std::vector<int32_t> blockTable(uint32_t seq) const {
        std::vector<int32_t> pages(static_cast<size_t>(maxSeqLen) / 16 + 1);
        uint32_t n = 0;
        check(er_kv_get_block_table(handle_, seq, pages.data(), static_cast<uint32_t>(pages.size()), &n));
        pages.resize(n);
        return pages;
    }
    // The stored 34-byte q8_0 blocks (KVCache.swift:175-184, 1007-1038), rows in logical order.
    std::pair<std::vector<uint8_t>, std::vector<uint8_t>> retrieveQ8_0Rows(int layer, uint32_t seq = 0) const {
        const size_t cap = static_cast<size_t>(maxSeqLen) * numKVHeads * (headDim / 32) * 34;
        std::vector<uint8_t> k(cap), v(cap);
        uint32_t tokens = 0;
        check(er_kv_retrieve_q8_0_rows(handle_, static_cast<uint32_t>(layer), seq, k.data(), v.data(), cap, &tokens));
        k.resize(static_cast<size_t>(tokens) * numKVHeads * (headDim / 32) * 34);
        v.resize(k.size());
        return {std::move(k), std::move(v)};
    }
    // Device status word of this cache's kernels: throws ER_ERR_DEVICE_TIMEOUT / ER_ERR_OUT_OF_PAGES when one was left.
    void checkDeviceStatus() const { check(er_kv_device_status(handle_)); }
    void clearDeviceStatus() { check(er_kv_clear_device_status(handle_)); }
    // kv heads split over GPUs: decode launches write this cache's heads into rows of headsTotal heads (own buffer + peers').
    void setOutputSharding(int headsTotal, int headOffset, const std::vector<float*>& peerOutputs = {}) {
        check(er_kv_set_output_sharding(handle_, static_cast<uint32_t>(headsTotal), static_cast<uint32_t>(headOffset),
                                        peerOutputs.empty() ? nullptr : peerOutputs.data(), static_cast<uint32_t>(peerOutputs.size())));
    }
    // Pages as bytes (prefix reuse): size of a page over all layers; pack pages into / write pages from a device or host buffer.
    size_t pageBytes() const {
        const int64_t n = er_kv_page_bytes(handle_);
        if (n < 0) throw KVCacheError(static_cast<int32_t>(n));
        return static_cast<size_t>(n);
    }
    void exportPages(const std::vector<int32_t>& pages, void* buffer, size_t bufferBytes, void* stream = nullptr) const {
        check(er_kv_export_pages(handle_, pages.data(), static_cast<uint32_t>(pages.size()), buffer, bufferBytes, stream));
    }
    void importPages(const std::vector<int32_t>& pages, const void* buffer, size_t bufferBytes, void* stream = nullptr) {
        check(er_kv_import_pages(handle_, pages.data(), static_cast<uint32_t>(pages.size()), buffer, bufferBytes, stream));
    }
    int setTrace(uint64_t* deviceBuffer, uint32_t capacityCtas) { return check(er_kv_set_trace(handle_, deviceBuffer, capacityCtas)); }

private:
    er_kv* handle_ = nullptr;
    Options options_;
};

// A device buffer other processes of the node can map (CUDA IPC) -- the peers' output buffers of a kv-head-sharded step.
class PeerBuffer {
public:
    explicit PeerBuffer(size_t bytes) : owner_(true) { check(er_peer_buffer_create(bytes, &ptr_, handle_)); }
    explicit PeerBuffer(const uint8_t* handle64) : owner_(false) { check(er_peer_buffer_open(handle64, &ptr_)); }
    ~PeerBuffer() { if (ptr_) { if (owner_) er_peer_buffer_destroy(ptr_); else er_peer_buffer_close(ptr_); } }
    PeerBuffer(const PeerBuffer&) = delete;
    PeerBuffer& operator=(const PeerBuffer&) = delete;
    float* data() const { return static_cast<float*>(ptr_); }
    const uint8_t* handle() const { return handle_; }   // 64 bytes, meaningful on the creating side

private:
    void* ptr_ = nullptr;
    uint8_t handle_[64] = {};
    bool owner_;
};
// After an NCCL all-gather of [world][pairs][localHeads][128]: rows of world * localHeads heads.
inline void relayoutHeadShards(const float* gathered, float* full, int world, int pairs, int localHeads, void* stream = nullptr) {
    check(er_relayout_head_shards(gathered, full, static_cast<uint32_t>(world), static_cast<uint32_t>(pairs), static_cast<uint32_t>(localHeads), stream));
}

class RoPEKernel {
public:
    // encodeNeoX(commandBuffer:inputBuffer:outputBuffer:seqLen:numHeads:headDim:startPos:theta:scalingFactor:
    // partialRotaryFactor:), RoPEKernel.swift:240-260
    void encodeNeoX(void* stream, const float* inputBuffer, float* outputBuffer, int seqLen, int numHeads, int headDim,
                    int startPos = 0, float theta = 10000.f, float scalingFactor = 1.f, float partialRotaryFactor = 1.f) const {
        ERRoPEParams p{static_cast<uint32_t>(seqLen), static_cast<uint32_t>(numHeads), static_cast<uint32_t>(headDim),
                       static_cast<uint32_t>(startPos), theta, scalingFactor, partialRotaryFactor};
        check(er_rope_neox_f32(inputBuffer, outputBuffer, &p, stream));
    }
    // rope_neox_f32_to_f16 (Shaders/RoPE.metal:498-531): the K row of a step, rotated and rounded to fp16
    void encodeNeoXToF16(void* stream, const float* inputBuffer, uint16_t* outputBuffer, int seqLen, int numHeads, int headDim,
                         int startPos = 0, float theta = 10000.f, float scalingFactor = 1.f, float partialRotaryFactor = 1.f) const {
        ERRoPEParams p{static_cast<uint32_t>(seqLen), static_cast<uint32_t>(numHeads), static_cast<uint32_t>(headDim),
                       static_cast<uint32_t>(startPos), theta, scalingFactor, partialRotaryFactor};
        check(er_rope_neox_f32_to_f16(inputBuffer, outputBuffer, &p, stream));
    }
};

class GQAKernel {
public:
    static constexpr int blockSize = 16;              // GQAKernel.swift:13
    static constexpr int maxOptimizedHeadDim = 128;   // GQAKernel.swift:14
    // encode(commandBuffer:qBuffer:kBuffer:vBuffer:outputBuffer:seqLen:headDim:numHeads:numKVHeads:causal:kvSeqLen:
    // qOffset:) on fp16 K/V (pipelineF16KV), GQAKernel.swift:113-172
    void encode(void* stream, const float* qBuffer, const uint16_t* kBuffer, const uint16_t* vBuffer, float* outputBuffer,
                int seqLen, int headDim, int numHeads, int numKVHeads, bool causal, int kvSeqLen = 0, int qOffset = 0) const {
        const ERGQAParams p = params(seqLen, headDim, numHeads, numKVHeads, causal, kvSeqLen, qOffset);
        check(er_gqa_attention_f16kv(qBuffer, kBuffer, vBuffer, outputBuffer, &p, stream));
    }
    // The fp32 pipelines of the same holder (gqa_attention_f32 / _masked_wide, Shaders/GQA.metal:18-276): K / V float,
    // additiveMaskBuffer [seqLen][kvSeqLen] float or null (GQAKernel.swift:122).
    void encodeF32(void* stream, const float* qBuffer, const float* kBuffer, const float* vBuffer, float* outputBuffer,
                   int seqLen, int headDim, int numHeads, int numKVHeads, bool causal, int kvSeqLen = 0, int qOffset = 0,
                   const float* additiveMaskBuffer = nullptr) const {
        const ERGQAParams p = params(seqLen, headDim, numHeads, numKVHeads, causal, kvSeqLen, qOffset);
        check(er_gqa_attention_f32(qBuffer, kBuffer, vBuffer, outputBuffer, additiveMaskBuffer, &p, stream));
    }
    // fp16 K/V with the split-K workspace built into the library (no device allocation by the call); no reference counterpart.
    void encodeStaticWorkspace(void* stream, const float* qBuffer, const uint16_t* kBuffer, const uint16_t* vBuffer, float* outputBuffer,
                               int seqLen, int headDim, int numHeads, int numKVHeads, bool causal, int kvSeqLen = 0, int qOffset = 0) const {
        const ERGQAParams p = params(seqLen, headDim, numHeads, numKVHeads, causal, kvSeqLen, qOffset);
        check(er_gqa_attention_f16kv_static(qBuffer, kBuffer, vBuffer, outputBuffer, &p, stream));
    }
    static void checkStaticWorkspaceStatus() { check(er_gqa_attention_f16kv_static_status()); }
    static void checkWorkspaceStatus() { check(er_workspace_status()); }

private:
    static ERGQAParams params(int seqLen, int headDim, int numHeads, int numKVHeads, bool causal, int kvSeqLen, int qOffset) {
        ERGQAParams p{};
        p.seqLen = static_cast<uint32_t>(seqLen);
        p.headDim = static_cast<uint32_t>(headDim);
        p.numHeads = static_cast<uint32_t>(numHeads);
        p.numKVHeads = static_cast<uint32_t>(numKVHeads);
        p.groupSize = static_cast<uint32_t>(numKVHeads ? numHeads / numKVHeads : 0);
        p.scale = 0.f;   // 0 -> 1/sqrt(headDim)
        p.causal = causal ? 1u : 0u;
        p.kvBlockSize = p.qBlockSize = blockSize;
        p.kvSeqLen = static_cast<uint32_t>(kvSeqLen);
        p.qOffset = static_cast<uint32_t>(qOffset);
        return p;
    }
};

// Gemma4DecodeKernels (Sources/EdgeRunnerMetal/Gemma4DecodeKernels.swift): the sliding-window decode attention only.
class Gemma4DecodeKernels {
public:
    // encodeDecodeGQAF16KVWindowed: ring rows (kvStart + i) % kvCapacity, i < kvCount; attentionScale 0 -> 1/sqrt(headDim)
    void encodeDecodeGQAF16KVWindowed(void* stream, const float* qBuffer, const uint16_t* keyCacheBuffer, const uint16_t* valueCacheBuffer,
                                      float* outputBuffer, int numHeads, int numKVHeads, int headDim, int kvStart, int kvCount,
                                      int kvCapacity, float attentionScale = 0.f) const {
        ERWindowedGQAParams p{};
        p.numHeads = static_cast<uint32_t>(numHeads);
        p.numKVHeads = static_cast<uint32_t>(numKVHeads);
        p.headDim = static_cast<uint32_t>(headDim);
        p.kvStart = static_cast<uint32_t>(kvStart);
        p.kvCount = static_cast<uint32_t>(kvCount);
        p.kvCapacity = static_cast<uint32_t>(kvCapacity);
        p.attentionScale = attentionScale;
        check(er_gqa_attention_f16kv_windowed(qBuffer, keyCacheBuffer, valueCacheBuffer, outputBuffer, &p, stream));
    }
};

class TurboQuantKernel {
public:
    // turboquant_quantize_rows dispatch (encodeTurboQuantRows, LlamaLanguageModel.swift:1754-1818)
    void encodeQuantizeRows(void* stream, const float* source, int rowCount, int sourceRowStride, int destinationRowBase, int bits,
                            uint32_t* codes, uint32_t* residualSigns, uint32_t* outlierMask, float* metadata) const {
        check(er_turboquant_quantize_rows(source, static_cast<uint32_t>(rowCount), static_cast<uint32_t>(sourceRowStride),
                                          static_cast<uint32_t>(destinationRowBase), static_cast<uint32_t>(bits), codes,
                                          residualSigns, outlierMask, metadata, stream));
    }
    // The same dispatch for presets with high-precision channels and a QJL residual (balanced: 3 / 5 bits, aggressive: 2 / 3,
    // 32 channels): preferQuantizationBenefitSelection chooses the values' selection rule (TurboQuant.swift:1185-1238).
    void encodeQuantizeRowsOutliers(void* stream, const float* source, int rowCount, int sourceRowStride, int destinationRowBase,
                                    int regularBits, int highPrecisionBits, int highPrecisionCount, bool preferQuantizationBenefitSelection,
                                    uint32_t* codes, uint32_t* residualSigns, uint32_t* outlierMask, float* metadata) const {
        check(er_turboquant_quantize_rows_outliers(source, static_cast<uint32_t>(rowCount), static_cast<uint32_t>(sourceRowStride),
                                                   static_cast<uint32_t>(destinationRowBase), static_cast<uint32_t>(regularBits),
                                                   static_cast<uint32_t>(highPrecisionBits), static_cast<uint32_t>(highPrecisionCount),
                                                   preferQuantizationBenefitSelection ? 1u : 0u, codes, residualSigns, outlierMask, metadata, stream));
    }
    // quantize_q8_0_rows (Shaders/Dequant_Q8_0.metal:19-49): 4 blocks of 34 bytes per 128-float row
    void encodeQuantizeQ8Rows(void* stream, const float* source, int rowCount, int sourceRowStride, int destinationRowBase,
                              uint8_t* destinationBlocks) const {
        check(er_quantize_q8_0_rows(source, static_cast<uint32_t>(rowCount), static_cast<uint32_t>(sourceRowStride),
                                    static_cast<uint32_t>(destinationRowBase), destinationBlocks, stream));
    }
};

// Free-list page allocator + per-sequence block tables for the paged layout.
class BlockTableAllocator {
public:
    BlockTableAllocator(int numPages, int pageSize, std::vector<int32_t> freeOrder = {}) : pageSize_(pageSize) {
        if (pageSize <= 0 || pageSize % 16 != 0) throw std::invalid_argument("pageSize must be a positive multiple of 16");
        if (freeOrder.empty()) {
            freeOrder.resize(static_cast<size_t>(numPages));
            for (int i = 0; i < numPages; ++i) freeOrder[static_cast<size_t>(i)] = i;
        }
        std::vector<int32_t> sorted = freeOrder;
        std::sort(sorted.begin(), sorted.end());
        for (int i = 0; i < numPages; ++i)
            if (static_cast<int>(sorted.size()) != numPages || sorted[static_cast<size_t>(i)] != i)
                throw std::invalid_argument("freeOrder must be a permutation of the page pool");
        free_.assign(freeOrder.rbegin(), freeOrder.rend());
    }
    int freePages() const { return static_cast<int>(free_.size()); }
    int pagesFor(int tokens) const { return (tokens + pageSize_ - 1) / pageSize_; }
    const std::vector<int32_t>& ensure(int seq, int tokens) {
        std::vector<int32_t>& table = tables_[seq];
        const int need = pagesFor(tokens) - static_cast<int>(table.size());
        if (need > static_cast<int>(free_.size())) throw KVCacheError(ER_ERR_OUT_OF_PAGES);
        for (int i = 0; i < need; ++i) { table.push_back(free_.back()); free_.pop_back(); }
        return table;
    }
    void release(int seq) {
        auto it = tables_.find(seq);
        if (it == tables_.end()) return;
        for (auto p = it->second.rbegin(); p != it->second.rend(); ++p) free_.push_back(*p);
        tables_.erase(it);
    }

private:
    int pageSize_;
    std::vector<int32_t> free_;
    std::unordered_map<int, std::vector<int32_t>> tables_;
};

}  // namespace edgerunner
