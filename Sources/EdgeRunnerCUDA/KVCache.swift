// EdgeRunnerCUDA.KVCache -- the CUDA counterpart of EdgeRunnerMetal.KVCache
// (Sources/EdgeRunnerMetal/KVCache.swift:12-1138): same public surface, storage on the GPU behind the C ABI of er_kv.h.
// Uncompiled in this repository (no Swift toolchain); the C++ mirror include/EdgeRunnerCUDA.hpp is the tested statement
// of the same layer.
import CEdgeRunnerCUDA

/// KVCacheError (KVCache.swift:1141-1148) plus the cases the CUDA backend adds.
public enum KVCacheError: Error, Sendable {
    case allocationFailed
    case invalidLayer(Int)
    case precisionMismatch
    case unsupportedStorage
    case compressedRetrieveRequiresDecodedAPI
    case compressedBufferAccessRequiresTurboQuantAPI
    case shape(String)
    case outOfPages(String)
    case deviceTimeout
    case backend(Int32, String)

    init(status: Int32, layer: Int = -1) {
        let detail = String(cString: er_last_error_string())
        switch status {
        case ER_ERR_ALLOCATION_FAILED: self = .allocationFailed
        case ER_ERR_INVALID_LAYER: self = .invalidLayer(layer)
        case ER_ERR_PRECISION_MISMATCH: self = .precisionMismatch
        case ER_ERR_UNSUPPORTED_STORAGE: self = .unsupportedStorage
        case ER_ERR_COMPRESSED_RETRIEVE_REQUIRES_DECODED_API: self = .compressedRetrieveRequiresDecodedAPI
        case ER_ERR_COMPRESSED_BUFFER_ACCESS_REQUIRES_TURBOQUANT_API: self = .compressedBufferAccessRequiresTurboQuantAPI
        case ER_ERR_SHAPE: self = .shape(detail)
        case ER_ERR_OUT_OF_PAGES: self = .outOfPages(detail)
        case ER_ERR_DEVICE_TIMEOUT: self = .deviceTimeout
        default: self = .backend(status, detail)
        }
    }
}

@inline(__always) func check(_ rc: Int32, layer: Int = -1) throws {
    guard rc >= 0 else { throw KVCacheError(status: rc, layer: layer) }
}

public final class KVCache: @unchecked Sendable {
    /// KVCache.Precision (KVCache.swift:39-49); raw values are the ER_KV_* constants.
    public enum Precision: UInt32, Sendable {
        case float32 = 0, float16, float8, q8_0, turboquantV2, turboQuantBalanced, turboQuantAggressive
    }
    /// Storage layouts of the CUDA backend; `.tokenMajor` is the reference's [slot][kvHead][dim] ring.
    public enum Layout: UInt32, Sendable { case tokenMajor = 0, headMajor, paged }

    public let maxSeqLen: Int
    public let numLayers: Int
    public let numKVHeads: Int
    public let headDim: Int
    public let precision: Precision
    public let maxBatch: Int
    let handle: OpaquePointer

    /// KVCache.init(device:maxSeqLen:numLayers:numKVHeads:headDim:precision:) (KVCache.swift:192-199); the device is the
    /// CUDA device current on the calling thread.
    public init(maxSeqLen: Int, numLayers: Int, numKVHeads: Int, headDim: Int, precision: Precision = .float16,
                keyType: UInt32 = 3, valueType: UInt32 = 3, compactNorms: Bool = false, maxBatch: Int = 1,
                layout: Layout = .headMajor, pageSize: Int = 0, numPages: Int = 0) throws {
        var cfg = er_kv_config()
        cfg.max_seq_len = UInt32(maxSeqLen); cfg.num_layers = UInt32(numLayers)
        cfg.num_kv_heads = UInt32(numKVHeads); cfg.head_dim = UInt32(headDim)
        cfg.precision = precision.rawValue; cfg.key_type = keyType; cfg.value_type = valueType
        cfg.norm_format = compactNorms ? 1 : 0
        cfg.max_batch = UInt32(maxBatch); cfg.layout = layout.rawValue
        cfg.page_size = UInt32(pageSize); cfg.num_pages = UInt32(numPages)
        var h: OpaquePointer?
        let rc = er_kv_create(&cfg, &h)
        guard rc == ER_OK, let h else { throw KVCacheError(status: rc) }
        handle = h
        self.maxSeqLen = maxSeqLen; self.numLayers = numLayers; self.numKVHeads = numKVHeads; self.headDim = headDim
        self.precision = precision; self.maxBatch = maxBatch
    }
    deinit { er_kv_destroy(handle) }

    // ---- getters (KVCache.swift:90-190) ----
    public var currentLength: Int { Int(er_kv_current_length(handle)) }
    public var elementsPerToken: Int { numKVHeads * headDim }
    public var denseBytesPerToken: Int? {
        switch precision { case .float32: return elementsPerToken * 4; case .float16: return elementsPerToken * 2; default: return nil }
    }
    public func totalWritten(layer: Int, sequence: Int = 0) -> Int { Int(er_kv_total_written(handle, UInt32(layer), UInt32(sequence))) }

    // ---- host append / retrieve (KVCache.swift:410-629) ----
    public func append(layer: Int, keys: [Float], values: [Float], sequence: Int = 0) throws {
        try check(er_kv_append_f32(handle, UInt32(layer), UInt32(sequence), keys, values, keys.count), layer: layer)
    }
    public func appendF16(layer: Int, keys: [UInt16], values: [UInt16], sequence: Int = 0) throws {
        try check(er_kv_append_f16(handle, UInt32(layer), UInt32(sequence), keys, values, keys.count), layer: layer)
    }
    public func retrieve(layer: Int, asType: Float.Type, sequence: Int = 0) throws -> (keys: [Float], values: [Float]) {
        let cap = maxSeqLen * elementsPerToken
        var k = [Float](repeating: 0, count: cap), v = k
        var tokens: UInt32 = 0
        try check(er_kv_retrieve(handle, UInt32(layer), UInt32(sequence), 4, &k, &v, cap, &tokens), layer: layer)
        let n = Int(tokens) * elementsPerToken
        return (Array(k[..<n]), Array(v[..<n]))
    }
    public func retrieveF16Bits(layer: Int, sequence: Int = 0) throws -> (keys: [UInt16], values: [UInt16]) {
        let cap = maxSeqLen * elementsPerToken
        var k = [UInt16](repeating: 0, count: cap), v = k
        var tokens: UInt32 = 0
        try check(er_kv_retrieve(handle, UInt32(layer), UInt32(sequence), 2, &k, &v, cap, &tokens), layer: layer)
        let n = Int(tokens) * elementsPerToken
        return (Array(k[..<n]), Array(v[..<n]))
    }
    public func retrieveDecodedTurboQuant(layer: Int, sequence: Int = 0) throws -> (keys: [Float], values: [Float]) {
        let cap = maxSeqLen * elementsPerToken
        var k = [Float](repeating: 0, count: cap), v = k
        var tokens: UInt32 = 0
        try check(er_kv_retrieve_decoded_turboquant(handle, UInt32(layer), UInt32(sequence), &k, &v, cap, &tokens), layer: layer)
        let n = Int(tokens) * elementsPerToken
        return (Array(k[..<n]), Array(v[..<n]))
    }
    public func retrieveDecodedQ8_0(layer: Int, sequence: Int = 0) throws -> (keys: [Float], values: [Float]) {
        let cap = maxSeqLen * elementsPerToken
        var k = [Float](repeating: 0, count: cap), v = k
        var tokens: UInt32 = 0
        try check(er_kv_retrieve_decoded_q8_0(handle, UInt32(layer), UInt32(sequence), &k, &v, cap, &tokens), layer: layer)
        let n = Int(tokens) * elementsPerToken
        return (Array(k[..<n]), Array(v[..<n]))
    }

    // ---- buffers / params / position control (KVCache.swift:631-729) ----
    /// Raw device pointers of one layer (replaces metalBuffers / turboQuantMetalBuffers).
    public func deviceBuffers(layer: Int) throws -> er_kv_buffers {
        var b = er_kv_buffers()
        try check(er_kv_device_buffers(handle, UInt32(layer), &b), layer: layer)
        return b
    }
    public func cacheParams(layer: Int, sequence: Int = 0) throws -> ERKVCacheParams {
        var p = ERKVCacheParams()
        try check(er_kv_cache_params(handle, UInt32(layer), UInt32(sequence), &p), layer: layer)
        return p
    }
    public func reset() throws { try check(er_kv_reset(handle)) }
    public func advanceWritePosition(layer: Int, by count: Int, sequence: Int? = nil) throws {
        try check(er_kv_advance_write_position(handle, UInt32(layer), sequence.map(UInt32.init) ?? UInt32.max, UInt32(count)), layer: layer)
    }
    public func setPosition(_ position: Int, sequence: Int? = nil) throws {
        try check(er_kv_set_position(handle, sequence.map(UInt32.init) ?? UInt32.max, UInt32(position)))
    }
    public func setBlockTable(sequence: Int, pages: [Int32]) throws {
        try check(er_kv_set_block_table(handle, UInt32(sequence), pages, UInt32(pages.count)))
    }

    // ---- device operators: what fusedDecodePass / fusedPrefillPass encode per layer (LlamaLanguageModel.swift:2940-2957, 3649-3941) ----
    public struct StepParameters {
        public var ropeTheta: Float = 10_000, ropeScaling: Float = 1, softmaxScale: Float = 0
        public var applyRoPE = true
        public var qNormWeight: UnsafePointer<Float>? = nil, kNormWeight: UnsafePointer<Float>? = nil
        public var rmsEps: Float = 1e-6
        public var normWeightLayerStride = 0, slidingWindow = 0
        public init() {}
        var c: er_step_params {
            var sp = er_step_params()
            sp.rope_theta = ropeTheta; sp.rope_scaling = ropeScaling; sp.softmax_scale = softmaxScale; sp.apply_rope = applyRoPE ? 1 : 0
            sp.q_norm_weight = qNormWeight; sp.k_norm_weight = kNormWeight; sp.rms_eps = rmsEps
            sp.norm_weight_layer_stride = UInt32(normWeightLayerStride); sp.sliding_window = UInt32(slidingWindow)
            return sp
        }
    }

    /// Append + attention + advance for `layers`: q [layers][batch][numHeads][headDim], k / v [layers][batch][numKVHeads][headDim]
    /// (device pointers).
    public func decodeStep(layers: Range<Int>, q: UnsafePointer<Float>, k: UnsafePointer<Float>, v: UnsafePointer<Float>,
                           out: UnsafeMutablePointer<Float>, numHeads: Int, parameters: StepParameters,
                           stream: UnsafeMutableRawPointer? = nil) throws {
        var sp = parameters.c
        try check(er_kv_decode_step(handle, UInt32(layers.lowerBound), UInt32(layers.upperBound), q, k, v, out, UInt32(numHeads), &sp, stream))
    }
    /// Same step with host buffers (pinned or pageable); waits for the result and reports a device-side failure of the step.
    public func decodeStepHost(layers: Range<Int>, q: UnsafePointer<Float>, k: UnsafePointer<Float>, v: UnsafePointer<Float>,
                               out: UnsafeMutablePointer<Float>, numHeads: Int, parameters: StepParameters,
                               stream: UnsafeMutableRawPointer? = nil) throws {
        var sp = parameters.c
        try check(er_kv_decode_step_host(handle, UInt32(layers.lowerBound), UInt32(layers.upperBound), q, k, v, out, UInt32(numHeads), &sp, stream))
    }
    public func writeRows(layer: Int, sequence: Int, start: Int, count: Int, k: UnsafePointer<Float>, v: UnsafePointer<Float>,
                          parameters: StepParameters, stream: UnsafeMutableRawPointer? = nil) throws {
        var sp = parameters.c
        try check(er_kv_write_rows(handle, UInt32(layer), UInt32(sequence), UInt32(start), UInt32(count), k, v, &sp, stream), layer: layer)
    }
    public func attentionPrefill(layer: Int, sequence: Int, q: UnsafePointer<Float>, out: UnsafeMutablePointer<Float>, numHeads: Int,
                                 seqLen: Int, qOffset: Int? = nil, parameters: StepParameters,
                                 stream: UnsafeMutableRawPointer? = nil) throws {
        var sp = parameters.c
        try check(er_kv_attention_prefill(handle, UInt32(layer), UInt32(sequence), q, out, UInt32(numHeads), UInt32(seqLen),
                                          qOffset.map(UInt32.init) ?? UInt32.max, &sp, stream), layer: layer)
    }
    /// Status word the kernels of this cache leave behind (a bounded wait that gave up, a row without a page).
    /// Layers whose keys and values use different row formats: attention with this cache's K rows and `values`' V rows.
    public func attentionDecode(withValuesOf values: KVCache, layers: Range<Int>, q: UnsafePointer<Float>, out: UnsafeMutablePointer<Float>,
                                numHeads: Int, pending: Int, params: inout er_step_params, stream: UnsafeMutableRawPointer? = nil) throws {
        try check(er_kv_attention_decode_pair(handle, values.handle, UInt32(layers.lowerBound), UInt32(layers.upperBound), q, out,
                                              UInt32(numHeads), UInt32(pending), &params, stream))
    }

    public func checkDeviceStatus() throws { try check(er_kv_device_status(handle)) }

    /// Pages as bytes (prefix reuse): `pageBytes` covers all layers; buffers may be device or (pinned) host memory.
    public var pageBytes: Int { Int(er_kv_page_bytes(handle)) }
    public func exportPages(_ pages: [Int32], into buffer: UnsafeMutableRawPointer, byteCount: Int, stream: UnsafeMutableRawPointer? = nil) throws {
        try check(er_kv_export_pages(handle, pages, UInt32(pages.count), buffer, byteCount, stream))
    }
    public func importPages(_ pages: [Int32], from buffer: UnsafeRawPointer, byteCount: Int, stream: UnsafeMutableRawPointer? = nil) throws {
        try check(er_kv_import_pages(handle, pages, UInt32(pages.count), buffer, byteCount, stream))
    }
}
