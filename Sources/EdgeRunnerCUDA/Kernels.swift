// Kernel holders of the CUDA backend, named after the Metal ones they replace:
//   GQAKernel            Sources/EdgeRunnerMetal/GQAKernel.swift:4-187
//   RoPEKernel           Sources/EdgeRunnerMetal/RoPEKernel.swift:4-307 (NeoX entry points)
//   TurboQuantKernel     Sources/EdgeRunnerMetal/TurboQuantKernel.swift:13-112
//   Gemma4DecodeKernels  Sources/EdgeRunnerMetal/Gemma4DecodeKernels.swift:537-660 (windowed decode attention only)
// `encode(commandBuffer:...)` becomes `encode(stream:...)`; MTLBuffers become device pointers.  Uncompiled here.
import CEdgeRunnerCUDA

public enum GQAError: Error, Sendable { case encodingFailed(Int32, String) }

@inline(__always) private func checkOp(_ rc: Int32) throws {
    guard rc >= 0 else { throw GQAError.encodingFailed(rc, String(cString: er_last_error_string())) }
}

public struct GQAKernel: Sendable {
    public static let blockSize = 16
    public static let maxOptimizedHeadDim = 128
    public static let maxSupportedHeadDim = 512
    public init() {}

    private func params(seqLen: Int, headDim: Int, numHeads: Int, numKVHeads: Int, causal: Bool, kvSeqLen: Int, qOffset: Int) -> ERGQAParams {
        precondition(numHeads % numKVHeads == 0, "numHeads must be divisible by numKVHeads")
        return ERGQAParams(seqLen: UInt32(seqLen), headDim: UInt32(headDim), numHeads: UInt32(numHeads), numKVHeads: UInt32(numKVHeads),
                           groupSize: UInt32(numHeads / numKVHeads), scale: 1.0 / Float(headDim).squareRoot(), causal: causal ? 1 : 0,
                           kvBlockSize: UInt32(Self.blockSize), qBlockSize: UInt32(Self.blockSize), kvSeqLen: UInt32(kvSeqLen),
                           qOffset: UInt32(qOffset))
    }

    /// GQAKernel.encode (GQAKernel.swift:113-172): float32 Q / K / V, optional additive mask [seqLen][kvSeqLen].
    public func encode(stream: UnsafeMutableRawPointer?, qBuffer: UnsafePointer<Float>, kBuffer: UnsafePointer<Float>,
                       vBuffer: UnsafePointer<Float>, outputBuffer: UnsafeMutablePointer<Float>, seqLen: Int, headDim: Int,
                       numHeads: Int, numKVHeads: Int, causal: Bool, kvSeqLen: Int = 0, qOffset: Int = 0,
                       additiveMaskBuffer: UnsafePointer<Float>? = nil) throws {
        var p = params(seqLen: seqLen, headDim: headDim, numHeads: numHeads, numKVHeads: numKVHeads, causal: causal, kvSeqLen: kvSeqLen, qOffset: qOffset)
        try checkOp(er_gqa_attention_f32(qBuffer, kBuffer, vBuffer, outputBuffer, additiveMaskBuffer, &p, stream))
    }
    /// The fp16-K/V pipeline (gqa_attention_f16kv, Shaders/GQA.metal:278-387).
    public func encodeF16KV(stream: UnsafeMutableRawPointer?, qBuffer: UnsafePointer<Float>, kBuffer: UnsafePointer<UInt16>,
                            vBuffer: UnsafePointer<UInt16>, outputBuffer: UnsafeMutablePointer<Float>, seqLen: Int, headDim: Int,
                            numHeads: Int, numKVHeads: Int, causal: Bool, kvSeqLen: Int = 0, qOffset: Int = 0) throws {
        var p = params(seqLen: seqLen, headDim: headDim, numHeads: numHeads, numKVHeads: numKVHeads, causal: causal, kvSeqLen: kvSeqLen, qOffset: qOffset)
        try checkOp(er_gqa_attention_f16kv(qBuffer, kBuffer, vBuffer, outputBuffer, &p, stream))
    }
    /// Same operator for hosts that must not allocate device memory (workspace built into the library).
    public func encodeF16KVStaticWorkspace(stream: UnsafeMutableRawPointer?, qBuffer: UnsafePointer<Float>, kBuffer: UnsafePointer<UInt16>,
                                           vBuffer: UnsafePointer<UInt16>, outputBuffer: UnsafeMutablePointer<Float>, seqLen: Int,
                                           headDim: Int, numHeads: Int, numKVHeads: Int, causal: Bool, kvSeqLen: Int = 0,
                                           qOffset: Int = 0) throws {
        var p = params(seqLen: seqLen, headDim: headDim, numHeads: numHeads, numKVHeads: numKVHeads, causal: causal, kvSeqLen: kvSeqLen, qOffset: qOffset)
        try checkOp(er_gqa_attention_f16kv_static(qBuffer, kBuffer, vBuffer, outputBuffer, &p, stream))
    }
}

public struct RoPEKernel: Sendable {
    public init() {}
    /// RoPEKernel.encodeNeoX (RoPEKernel.swift:240-260).
    public func encodeNeoX(stream: UnsafeMutableRawPointer?, inputBuffer: UnsafePointer<Float>, outputBuffer: UnsafeMutablePointer<Float>,
                           seqLen: Int, numHeads: Int, headDim: Int, startPos: Int, theta: Float = 10_000, scalingFactor: Float = 1,
                           partialRotaryFactor: Float = 1) throws {
        var p = ERRoPEParams(seqLen: UInt32(seqLen), numHeads: UInt32(numHeads), headDim: UInt32(headDim), startPos: UInt32(startPos),
                             theta: theta, scalingFactor: scalingFactor, partialRotaryFactor: partialRotaryFactor)
        try checkOp(er_rope_neox_f32(inputBuffer, outputBuffer, &p, stream))
    }
    /// rope_neox_f32_to_f16 (Shaders/RoPE.metal:498-531).
    public func encodeNeoXToF16(stream: UnsafeMutableRawPointer?, inputBuffer: UnsafePointer<Float>, outputBuffer: UnsafeMutablePointer<UInt16>,
                                seqLen: Int, numHeads: Int, headDim: Int, startPos: Int, theta: Float = 10_000, scalingFactor: Float = 1,
                                partialRotaryFactor: Float = 1) throws {
        var p = ERRoPEParams(seqLen: UInt32(seqLen), numHeads: UInt32(numHeads), headDim: UInt32(headDim), startPos: UInt32(startPos),
                             theta: theta, scalingFactor: scalingFactor, partialRotaryFactor: partialRotaryFactor)
        try checkOp(er_rope_neox_f32_to_f16(inputBuffer, outputBuffer, &p, stream))
    }
}

public struct TurboQuantKernel: Sendable {
    public init() {}
    /// turboquant_quantize_rows for the fixed presets (encodeTurboQuantRows, LlamaLanguageModel.swift:1754-1818).
    public func encodeQuantizeRows(stream: UnsafeMutableRawPointer?, source: UnsafePointer<Float>, rowCount: Int, sourceRowStride: Int,
                                   destinationRowBase: Int, bits: Int, codes: UnsafeMutablePointer<UInt32>,
                                   residualSigns: UnsafeMutablePointer<UInt32>?, outlierMask: UnsafeMutablePointer<UInt32>?,
                                   metadata: UnsafeMutablePointer<Float>) throws {
        try checkOp(er_turboquant_quantize_rows(source, UInt32(rowCount), UInt32(sourceRowStride), UInt32(destinationRowBase), UInt32(bits),
                                                codes, residualSigns, outlierMask, metadata, stream))
    }
    /// quantize_q8_0_rows (Shaders/Dequant_Q8_0.metal:19-49).
    public func encodeQuantizeQ8Rows(stream: UnsafeMutableRawPointer?, source: UnsafePointer<Float>, rowCount: Int, sourceRowStride: Int,
                                     destinationRowBase: Int, blocks: UnsafeMutablePointer<UInt8>) throws {
        try checkOp(er_quantize_q8_0_rows(source, UInt32(rowCount), UInt32(sourceRowStride), UInt32(destinationRowBase), blocks, stream))
    }
}

public struct Gemma4DecodeKernels: Sendable {
    public init() {}
    /// encodeDecodeGQAF16KVWindowedBestAvailable (Gemma4DecodeKernels.swift:537-660).
    public func encodeDecodeGQAF16KVWindowed(stream: UnsafeMutableRawPointer?, q: UnsafePointer<Float>, keyCache: UnsafePointer<UInt16>,
                                             valueCache: UnsafePointer<UInt16>, output: UnsafeMutablePointer<Float>, numHeads: Int,
                                             numKVHeads: Int, headDim: Int, kvStart: Int, kvCount: Int, kvCapacity: Int,
                                             attentionScale: Float? = nil) throws {
        var p = ERWindowedGQAParams(numHeads: UInt32(numHeads), numKVHeads: UInt32(numKVHeads), headDim: UInt32(headDim),
                                    kvStart: UInt32(kvStart), kvCount: UInt32(kvCount), kvCapacity: UInt32(kvCapacity),
                                    attentionScale: attentionScale ?? 0)
        try checkOp(er_gqa_attention_f16kv_windowed(q, keyCache, valueCache, output, &p, stream))
    }
}
