/*
 * er_kv.h -- C ABI of the B200 (sm_100a) backend for EdgeRunner's decode-time KV-cache path:
 * append of RoPE'd K / V rows, optional TurboQuant compression, GQA flash-decode attention.
 *
 * This is the surface an `EdgeRunnerCUDA` Swift target binds through a module map in place of
 * the EdgeRunnerMetal kernels.  Every entry point names the reference interface it replaces
 * (paths relative to the reference checkout).  Plain C: opaque handle, pointers, sizes, status
 * codes.  Unless stated otherwise `const float* ... /+device+/` arguments are device pointers and
 * work is enqueued on the given `cudaStream_t` (passed as `void*`, NULL = legacy default stream)
 * and returns without waiting; `host` arguments are ordinary host pointers and the call
 * synchronises before returning.
 *
 * There is no CPU fallback anywhere behind this header: every compute entry point launches
 * hand-written CUDA kernels and reports ER_ERR_CUDA if no device is usable.
 */
#ifndef ER_KV_H
#define ER_KV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library itself is built with -fvisibility=hidden */
#endif

/* ---- parameter structs shared verbatim with the reference (field names and order are the interface) ---- */

/* Sources/EdgeRunnerSharedTypes/include/KVCacheParams.h:12-19 */
typedef struct {
    uint32_t maxSeqLen;
    uint32_t currentLen;
    uint32_t writePos;
    uint32_t numKVHeads;
    uint32_t headDim;
    uint32_t precision;
} ERKVCacheParams;

/* Sources/EdgeRunnerSharedTypes/include/AttentionParams.h:15-27 */
typedef struct {
    uint32_t seqLen;
    uint32_t headDim;
    uint32_t numHeads;
    uint32_t numKVHeads;
    uint32_t groupSize;
    float scale;
    uint32_t causal;
    uint32_t kvBlockSize;
    uint32_t qBlockSize;
    uint32_t kvSeqLen; /* 0 = same as seqLen */
    uint32_t qOffset;  /* key k is visible to query row r iff k <= r + qOffset */
} ERGQAParams;

/* Sources/EdgeRunnerSharedTypes/include/RoPEParams.h:6-21 */
typedef struct {
    uint32_t seqLen;
    uint32_t numHeads;
    uint32_t headDim;
    uint32_t startPos;
    float theta;
    float scalingFactor;
    float partialRotaryFactor;
} ERRoPEParams;

/* ---- status codes: 0 ok, negatives 1:1 with KVCacheError (Sources/EdgeRunnerMetal/KVCache.swift:1141-1148);
 * shape preconditions that trap in the reference (KVCache.swift:413-414) are reported as ER_ERR_SHAPE. ---- */
enum {
    ER_OK = 0,
    ER_ERR_ALLOCATION_FAILED = -1,
    ER_ERR_INVALID_LAYER = -2,
    ER_ERR_PRECISION_MISMATCH = -3,
    ER_ERR_UNSUPPORTED_STORAGE = -4,
    ER_ERR_COMPRESSED_RETRIEVE_REQUIRES_DECODED_API = -5,
    ER_ERR_COMPRESSED_BUFFER_ACCESS_REQUIRES_TURBOQUANT_API = -6,
    ER_ERR_SHAPE = -7,
    ER_ERR_CUDA = -8,
    ER_ERR_INVALID_ARGUMENT = -9,
    ER_ERR_OUT_OF_PAGES = -10,
    ER_ERR_UNSUPPORTED = -11,
    ER_ERR_DEVICE_TIMEOUT = -12 /* a bounded device-side wait gave up; see er_kv_device_status */
};

/* KVCache.Precision raw values (KVCache.swift:39-49). float8 is accepted by er_kv_create only to report
 * ER_ERR_UNSUPPORTED_STORAGE.  BALANCED (3-bit codes, the 32 best channels 5-bit) and AGGRESSIVE (2-bit, 32 channels 3-bit)
 * keep every row as codes + outlier mask + QJL residual signs + (rowNorm, residualNorm); key_type / value_type then hold the
 * keys' / values' channel-selection rule (ER_TQ_SELECT_*), and key_residual_scale / value_residual_scale the weights of the
 * residual term in attention (TurboQuantV2Contract.keyResidualScale / valueResidualScale: 0 in the reference's contract). */
enum {
    ER_KV_FLOAT32 = 0,
    ER_KV_FLOAT16 = 1,
    ER_KV_FLOAT8 = 2,
    ER_KV_Q8_0 = 3,
    ER_KV_TURBOQUANT_V2 = 4,
    ER_KV_TURBOQUANT_BALANCED = 5,
    ER_KV_TURBOQUANT_AGGRESSIVE = 6
};

/* TurboQuantFixedType (TurboQuant.swift:172-190): the value is the bit width of the preset. */
enum { ER_TQ_TURBO2 = 2, ER_TQ_TURBO3 = 3, ER_TQ_TURBO4 = 4 };
/* TurboQuantOutlierSelection (TurboQuant.swift:1185-1238) for BALANCED / AGGRESSIVE caches.  DEFAULT is the reference's
 * contract: keys by magnitude, values by quantisation benefit (TurboQuantV2Contract.keyOutlierSelection / valueOutlierSelection). */
enum { ER_TQ_SELECT_DEFAULT = 0, ER_TQ_SELECT_MAGNITUDE = 1, ER_TQ_SELECT_QUANTIZATION_BENEFIT = 2 };

/* Storage layouts.  The reference has exactly one: a token-major ring per layer
 * ([slot][kvHead][dim], KVCache.swift:357-370).  HEAD_MAJOR keeps each kv head's tokens contiguous
 * ([seq][kvHead][slot][dim]) so a tile of tokens is one bulk copy; PAGED stores fixed-size pages
 * ([page][kvHead][slotInPage][dim]) addressed through a per-sequence block table. */
enum { ER_KV_LAYOUT_TOKEN_MAJOR = 0, ER_KV_LAYOUT_HEAD_MAJOR = 1, ER_KV_LAYOUT_PAGED = 2 };

/* Stored per-row TurboQuant norm: the reference keeps two floats (rowNorm, residualNorm;
 * KVCache.swift:1095-1096); the compact format keeps rowNorm as fp16 and drops the always-zero rest. */
enum { ER_TQ_NORM_FLOAT32 = 0, ER_TQ_NORM_FLOAT16 = 1 };

/* Chunked-prefill kernel choice (the counterpart of the reference's pipeline selection by shape in
 * GQAKernel.encode, GQAKernel.swift:136-160): AUTO runs the tcgen05 kernel when the chunk fills a 128-row CTA tile
 * and the mma.sync kernel otherwise; MMA_SYNC always runs the latter (A/B measurements). */
enum { ER_PREFILL_KERNEL_AUTO = 0, ER_PREFILL_KERNEL_MMA_SYNC = 1 };

/* Decode kernel choice for float16 caches.  The reference dispatches attention once per layer
 * (Sources/EdgeRunner/Models/LlamaLanguageModel.swift:3867-3881): a few MB of rows per call.  AUTO runs such small calls
 * (capacity of the addressed rows up to 128 MB, GQA group 1/2/4, no sliding window) on a kernel without a staging
 * pipeline, and everything else on the persistent stream-K kernel; PERSISTENT / SLIM force one of them where its shape
 * rules allow (parity tests run both).  SIMT: TurboQuant caches (fixed presets, balanced, aggressive) run their decode attention
 * on the plain SIMT kernel instead of the tensor-core policies of the persistent kernel (the same A/B use; other caches: as AUTO). */
enum { ER_DECODE_KERNEL_AUTO = 0, ER_DECODE_KERNEL_PERSISTENT = 1, ER_DECODE_KERNEL_SLIM = 2, ER_DECODE_KERNEL_SIMT = 3 };

typedef struct {
    uint32_t max_seq_len;   /* ring length per sequence (tokens) */
    uint32_t num_layers;
    uint32_t num_kv_heads;  /* heads held by THIS cache (a kv-head shard holds its slice only) */
    uint32_t head_dim;
    uint32_t precision;     /* ER_KV_* */
    uint32_t key_type;      /* ER_TQ_TURBO* when precision == ER_KV_TURBOQUANT_V2; ER_TQ_SELECT_* for BALANCED / AGGRESSIVE */
    uint32_t value_type;
    uint32_t norm_format;   /* ER_TQ_NORM_* */
    uint32_t max_batch;     /* sequences held (the reference's cache is the max_batch == 1 case) */
    uint32_t layout;        /* ER_KV_LAYOUT_* (TurboQuant storage ignores TOKEN_MAJOR and uses HEAD_MAJOR) */
    uint32_t page_size;     /* tokens per page, multiple of 16 (PAGED only) */
    uint32_t num_pages;     /* pages in the shared pool (PAGED only) */
    uint32_t prefill_kernel; /* ER_PREFILL_KERNEL_*: which chunked-prefill kernel er_kv_attention_prefill may use */
    uint32_t decode_kernel;  /* ER_DECODE_KERNEL_*: float16 caches; SIMT: TurboQuant caches */
    float key_residual_scale;   /* BALANCED / AGGRESSIVE: weight of the QJL residual term of the scores (0 = off, the contract) */
    float value_residual_scale; /* ... and of the outputs; also the residualWeight of decoded value rows */
} er_kv_config;

typedef struct er_kv er_kv;

/* Raw device buffers of one layer; replaces KVCache.metalBuffers / turboQuantMetalBuffers
 * (KVCache.swift:631-667).  Borrowed: valid until er_kv_destroy. */
typedef struct {
    void* keys;          /* dense: fp16/fp32 elements; TurboQuant: packed code words */
    void* values;
    void* key_norms;     /* TurboQuant only: one norm per row (format per config.norm_format) */
    void* value_norms;
    uint64_t key_bytes;
    uint64_t value_bytes;
    uint32_t key_row_bytes;   /* bytes of one (token, kv head) row */
    uint32_t value_row_bytes;
} er_kv_buffers;

/* Decode-step controls. */
typedef struct {
    float rope_theta;      /* ERRoPEParams.theta */
    float rope_scaling;    /* ERRoPEParams.scalingFactor (1.0 = none) */
    float softmax_scale;   /* 0 -> 1/sqrt(head_dim) (GQAKernel.encode, GQAKernel.swift:134) */
    uint32_t apply_rope;   /* 1: NeoX-rotate Q and K at the row's position inside the call */
    /* Per-head RMS norm of Q and K before RoPE -- the first half of fused_qk_norm_rope_neox (Shaders/RoPE.metal:119-173):
     * x * rsqrt(mean(x^2) + rms_eps) * weight[dim].  Device pointers to headDim floats per layer (layer l reads
     * weight + l * norm_weight_layer_stride; stride 0 = one vector for all layers); NULL = no norm for that tensor. */
    const float* q_norm_weight;
    const float* k_norm_weight;
    float rms_eps;
    uint32_t norm_weight_layer_stride;
    /* Sliding-window decode (Gemma4GPUKVCache.attentionRange, Sources/EdgeRunner/Models/Gemma4/Gemma4GPUKVCache.swift:206-216;
     * gemma4_decode_gqa_f16kv_windowed, Shaders/Gemma4Decode.metal:236-283): > 0 -> a decode call attends to the newest
     * min(sliding_window, rows in the ring) rows of each sequence, wherever they sit in the ring; 0 = every row held.
     * er_kv_attention_prefill applies the same rule per query row (row at position P sees keys P - sliding_window + 1 .. P).
     * Every cache format but float32; q8_0 / TurboQuant caches run windowed calls on the SIMT kernel, and their windowed prefill
     * chunks must end at the sequence's newest row. */
    uint32_t sliding_window;
    uint32_t reserved;
} er_step_params;

const char* er_status_string(int32_t status);
const char* er_last_error_string(void);              /* thread-local detail for the last failing call */
int32_t er_device_count(void);

/* ---- cache object: KVCache.init / deinit (KVCache.swift:192-275) ---- */
int32_t er_kv_create(const er_kv_config* config, er_kv** out);
void er_kv_destroy(er_kv* kv);
int32_t er_kv_get_config(const er_kv* kv, er_kv_config* out);

/* KVCache.currentLength (KVCache.swift:184-188): max over layers (and sequences) of min(totalWritten, maxSeqLen). */
int32_t er_kv_current_length(er_kv* kv);
/* Tokens written so far to (layer, seq), not clamped. */
int64_t er_kv_total_written(er_kv* kv, uint32_t layer, uint32_t seq);

/* KVCache.append(layer:keys:values:) (KVCache.swift:410-453): host float rows of numKVHeads*headDim elements,
 * stored as float32, or TurboQuant-encoded on the device; advances the ring.  ER_ERR_PRECISION_MISMATCH for a
 * float16 cache, exactly like the reference. */
int32_t er_kv_append_f32(er_kv* kv, uint32_t layer, uint32_t seq, const float* host_keys, const float* host_values,
                         size_t element_count);
/* KVCache.appendF16 (KVCache.swift:455-476): fp16 bit patterns. */
int32_t er_kv_append_f16(er_kv* kv, uint32_t layer, uint32_t seq, const uint16_t* host_keys,
                         const uint16_t* host_values, size_t element_count);

/* KVCache.retrieve(layer:asType:) (KVCache.swift:478-522): logical (oldest-first) order, [token][kvHead][dim].
 * element_bytes is the requested element size (4 = Float, 2 = Float16); capacity_elements bounds the copy.
 * *token_count receives the number of tokens returned. */
int32_t er_kv_retrieve(er_kv* kv, uint32_t layer, uint32_t seq, uint32_t element_bytes, void* host_keys,
                       void* host_values, size_t capacity_elements, uint32_t* token_count);
/* KVCache.retrieveDecodedTurboQuant (KVCache.swift:524-586): rows dequantised on the device. */
int32_t er_kv_retrieve_decoded_turboquant(er_kv* kv, uint32_t layer, uint32_t seq, float* host_keys,
                                          float* host_values, size_t capacity_elements, uint32_t* token_count);
/* KVCache.retrieveDecodedQ8_0 (KVCache.swift:882-908): rows of a q8_0 cache as scale * Float(q), logical order,
 * [token][kvHead][dim]. */
int32_t er_kv_retrieve_decoded_q8_0(er_kv* kv, uint32_t layer, uint32_t seq, float* host_keys, float* host_values,
                                    size_t capacity_elements, uint32_t* token_count);
/* The stored rows of a q8_0 cache in the reference's buffer format (KVCache.swift:175-184, 1007-1038): per row
 * headDim / 32 blocks of 34 bytes (fp16 scale, 32 int8), rows in logical order, row = token * numKVHeads + kvHead.
 * capacity_bytes bounds each copy. */
int32_t er_kv_retrieve_q8_0_rows(er_kv* kv, uint32_t layer, uint32_t seq, uint8_t* host_key_blocks, uint8_t* host_value_blocks,
                                 size_t capacity_bytes, uint32_t* token_count);
/* KVCache.retrieveTurboQuantRuntimeRows (KVCache.swift:588-629) in the reference's split-buffer row format:
 * codes [rows][words], residual signs [rows][4], outlier mask [rows][4], metadata [rows][2] = (rowNorm, residualNorm) --
 * signs, mask and residualNorm are zero for the fixed presets; BALANCED / AGGRESSIVE caches return what the encoder
 * stored (words = 14 / 9, split-plane codes).  rows = tokens*numKVHeads in logical order, row = token*numKVHeads + kvHead. */
int32_t er_kv_retrieve_turboquant_rows(er_kv* kv, uint32_t layer, uint32_t seq, int is_value, uint32_t* host_codes,
                                       uint32_t* host_residual_signs, uint32_t* host_outlier_mask,
                                       float* host_metadata, size_t capacity_rows, uint32_t* row_count);

/* KVCache.metalBuffers / turboQuantMetalBuffers (KVCache.swift:631-667). */
int32_t er_kv_device_buffers(er_kv* kv, uint32_t layer, er_kv_buffers* out);
/* KVCache.cacheParams (KVCache.swift:691-703). */
int32_t er_kv_cache_params(er_kv* kv, uint32_t layer, uint32_t seq, ERKVCacheParams* out);
/* KVCache.reset / advanceWritePosition / setPosition (KVCache.swift:705-729). seq == UINT32_MAX: all sequences. */
int32_t er_kv_reset(er_kv* kv);
int32_t er_kv_advance_write_position(er_kv* kv, uint32_t layer, uint32_t seq, uint32_t count);
int32_t er_kv_set_position(er_kv* kv, uint32_t seq, uint32_t position);

/* Paged layout: install the block table of one sequence (page ids into the shared pool, one per page_size
 * tokens).  The allocator that hands out page ids lives above this ABI (host side).  Entries beyond page_count hold no
 * page: a host-side write that would land there (er_kv_append_*, er_kv_write_rows) returns ER_ERR_OUT_OF_PAGES before
 * anything is launched; a device-side append (er_kv_append_rope_kv, er_kv_decode_step) drops the row and sets the
 * device status word to ER_ERR_OUT_OF_PAGES (see er_kv_device_status) -- no other sequence's page is touched. */
int32_t er_kv_set_block_table(er_kv* kv, uint32_t seq, const int32_t* host_page_ids, uint32_t page_count);
int32_t er_kv_get_block_table(er_kv* kv, uint32_t seq, int32_t* host_page_ids, uint32_t capacity, uint32_t* page_count);

/* ---- device-side operators ---- */

/* RoPEKernel.encodeNeoX -> rope_neox_f32 (RoPEKernel.swift:240-260, Shaders/RoPE.metal:57-93).
 * in/out: device [seqLen][numHeads][headDim] float; may alias. */
int32_t er_rope_neox_f32(const float* in, float* out, const ERRoPEParams* params, void* stream);
/* rope_neox_f32_to_f16 (Shaders/RoPE.metal:498-531): out is device fp16. */
int32_t er_rope_neox_f32_to_f16(const float* in, uint16_t* out, const ERRoPEParams* params, void* stream);

/* quantize_q8_0_rows (Shaders/Dequant_Q8_0.metal:19-49): source device [row_count][source_row_stride] float (the first
 * 128 of each row are used) -> device blocks, row destination_row_base + i, 4 blocks of 34 bytes per row. */
int32_t er_quantize_q8_0_rows(const float* source, uint32_t row_count, uint32_t source_row_stride, uint32_t destination_row_base,
                              uint8_t* destination_blocks, void* stream);

/* turboquant_quantize_rows for the fixed presets (Shaders/TurboQuant.metal:562-709; dispatched by
 * encodeTurboQuantRows, Sources/EdgeRunner/Models/LlamaLanguageModel.swift:1754-1818).  source: device
 * [row_count][source_row_stride] float (first 128 of each row are used); outputs are the reference's four
 * split device buffers written at rows destination_row_base + i. */
int32_t er_turboquant_quantize_rows(const float* source, uint32_t row_count, uint32_t source_row_stride,
                                    uint32_t destination_row_base, uint32_t bits, uint32_t* out_codes,
                                    uint32_t* out_residual_signs, uint32_t* out_outlier_mask, float* out_metadata,
                                    void* stream);

/* turboquant_quantize_rows for the presets with high-precision channels and a QJL residual (Shaders/TurboQuant.metal:562-709;
 * TurboQuantReferenceEncoder.encode, TurboQuant.swift:1003-1100): balanced = (3, 5, 32), aggressive = (2, 3, 32)
 * (TurboQuantPreset.descriptor, TurboQuant.swift:78-84, 117-124).  The `high_count` channels with the largest selection
 * score -- |rotated value| (keys, .magnitude), or the quantisation benefit (values, use_quantization_benefit != 0) --
 * get `high_bits` codes; the split device buffers are the reference's: codes [rows][base + side-band words] (split-plane
 * packing), residual signs [rows][4], outlier mask [rows][4], metadata [rows][2] = (rowNorm, residualNorm).  Bit-exact
 * against the CPU encoder on finite rows.  Storing such rows in an er_kv cache and attention over them are not built. */
int32_t er_turboquant_quantize_rows_outliers(const float* source, uint32_t row_count, uint32_t source_row_stride,
                                             uint32_t destination_row_base, uint32_t regular_bits, uint32_t high_bits,
                                             uint32_t high_count, uint32_t use_quantization_benefit, uint32_t* out_codes,
                                             uint32_t* out_residual_signs, uint32_t* out_outlier_mask, float* out_metadata,
                                             void* stream);

/* GQAKernel.encode / GQAKernel.execute (GQAKernel.swift:27-172) -> gqa_attention_f32, gqa_attention_f32_wide,
 * gqa_attention_f32_masked_wide (Shaders/GQA.metal:18-276): float32 K / V.  q/out: device [seqLen][numHeads][headDim]
 * float; k/v: device [kvSeqLen][numKVHeads][headDim] float; additive_mask: device [seqLen][kvSeqLen] float added to the
 * scaled scores (-inf entries hide a key), or NULL -- the additiveMaskBuffer argument.  headDim 1...512, divisible by 4
 * (the wrapper's preconditions); a query row with no visible finite score yields zeros. */
int32_t er_gqa_attention_f32(const float* q, const float* k, const float* v, float* out, const float* additive_mask,
                             const ERGQAParams* params, void* stream);

/* The fp16-K/V pipeline of the same holder -> gqa_attention_f16kv (GQAKernel.swift:113-172, Shaders/GQA.metal:278-387).
 * q/out: device [seqLen][numHeads][headDim] float; k/v: device [kvSeqLen][numKVHeads][headDim] fp16.
 * headDim 128 with 1/2/4/8 query heads per kv head and <= 16 kv heads: persistent flash-decode kernel (seqLen 1) or
 * tensor-core prefill kernel (seqLen > 1); other even headDim <= 512 / groups: a plain split kernel, one launch per row. */
int32_t er_gqa_attention_f16kv(const float* q, const uint16_t* k, const uint16_t* v, float* out,
                               const ERGQAParams* params, void* stream);

/* gemma4_decode_gqa_f16kv_windowed (Shaders/Gemma4Decode.metal:236-283; host wrapper runDecodeGQAF16KVWindowed,
 * Gemma4DecodeKernels.swift): one query token against ring rows (kvStart + i) % kvCapacity, i < kvCount, of a token-major
 * fp16 K/V pair.  q/out: device [numHeads][128] float; k/v: device [kvCapacity][numKVHeads][128] fp16.  kvCount == 0 or
 * kvCapacity == 0 writes zeros (the shader's rule); kvCount > kvCapacity is ER_ERR_SHAPE.  attentionScale 0 ->
 * 1/sqrt(headDim), the wrapper's default (Gemma 4 passes 1.0).  headDim 128 with 1/2/4/8 query heads per kv head runs the
 * persistent flash-decode kernel; any other even headDim <= 512 (the reference's Gemma shapes are 256 / 512) or group
 * runs a plain split kernel. */
typedef struct {
    uint32_t numHeads;
    uint32_t numKVHeads;
    uint32_t headDim;
    uint32_t kvStart;
    uint32_t kvCount;
    uint32_t kvCapacity;
    float attentionScale;
} ERWindowedGQAParams;
int32_t er_gqa_attention_f16kv_windowed(const float* q, const uint16_t* k, const uint16_t* v, float* out,
                                        const ERWindowedGQAParams* params, void* stream);

/* No counterpart in the reference.  Same operator and arguments as er_gqa_attention_f16kv, for hosts that cannot
 * let the library allocate: a server whose own pool already owns all free device memory, or a latency-critical
 * thread that must not take the driver's allocation path.  The split-K workspace is a ~1 MiB array compiled into
 * the library (every GPU that loads the library holds it until the process exits), so the call performs no
 * cudaMalloc / cudaFree of any kind.  Limits: numKVHeads <= 16, numHeads / numKVHeads in {1, 2, 4}, at most 256 SMs;
 * anything larger is rejected with ER_ERR_UNSUPPORTED.  The first call on a device looks up the array's device
 * address (make that call before starting a stream capture).  All calls share the one array: it keeps the last
 * call's contents (the counters are re-zeroed on the stream at every call; the status word stays until
 * er_gqa_attention_f16kv_static_status reads it) and two calls that overlap on the GPU race -- keep them on one stream
 * or order them yourself. */
int32_t er_gqa_attention_f16kv_static(const float* q, const uint16_t* k, const uint16_t* v, float* out,
                                      const ERGQAParams* params, void* stream);

/* Append one new token per sequence to layers [layer_begin, layer_end): the three per-layer dispatches of the
 * decode pass -- V row convert/quantise, K NeoX RoPE + convert/quantise -- at row position totalWritten
 * (LlamaLanguageModel.swift:3649-3684, 3757-3825).  k, v: device [layers][max_batch][numKVHeads][headDim] float.
 * Does not advance the write position. */
int32_t er_kv_append_rope_kv(er_kv* kv, uint32_t layer_begin, uint32_t layer_end, const float* k, const float* v,
                             const er_step_params* params, void* stream);

/* Decode attention of one query row per sequence over rows [0, min(totalWritten + pending, maxSeqLen)) of each
 * layer in [layer_begin, layer_end) -- gqa_attention_f16kv / gqa_attention_turboquant_decode with seqLen 1
 * (LlamaLanguageModel.swift:3867-3881, 3924-3938; Shaders/TurboQuant.metal:1794-2001).  `pending` is 1 when the
 * row just written by er_kv_append_rope_kv has not been committed by an advance yet, else 0.
 * q, out: device [layers][max_batch][num_heads][headDim] float.  With params->apply_rope, Q is rotated at
 * position totalWritten + pending - 1. */
int32_t er_kv_attention_decode(er_kv* kv, uint32_t layer_begin, uint32_t layer_end, const float* q, float* out,
                               uint32_t num_heads, uint32_t pending, const er_step_params* params, void* stream);

/* Chunked-prefill attention of `seq_len` query rows of (layer, seq) over the rows already in the cache -- the
 * seqLen > 1 dispatch of gqa_attention_f16kv / flash_attention_gqa_simd_qf32_kvf16 in fusedPrefillPass
 * (LlamaLanguageModel.swift:2940-2957; Shaders/GQA.metal:278-387, Shaders/FlashAttention.metal:194-264), on the tensor
 * cores.  Write the chunk's K/V rows first (er_kv_write_rows), then call this: query row r has absolute position
 * q_offset + r and sees keys 0 .. q_offset + r.  q_offset == UINT32_MAX means "the query rows are the newest seq_len
 * rows of the cache".  q, out: device [seq_len][num_heads][headDim] float.  float16 caches, and TurboQuant caches
 * (gqa_attention_turboquant, Shaders/TurboQuant.metal:1454-1649: the sequence's codes are expanded to fp16 rows in
 * a scratch buffer of the cache, so calls on one cache must not overlap). */
int32_t er_kv_attention_prefill(er_kv* kv, uint32_t layer, uint32_t seq, const float* q, float* out, uint32_t num_heads,
                                uint32_t seq_len, uint32_t q_offset, const er_step_params* params, void* stream);

/* Layers whose keys and values use DIFFERENT row formats (the reference's hybrid layers: q8_0 keys with TurboQuant values,
 * TurboQuant keys with float16 values, ...: gqa_attention_q8k_turboquant(_decode), gqa_attention_turboquant_decode_f16v,
 * Shaders/TurboQuant.metal:1651-2399; chosen per layer by TurboQuantV2Contract, TurboQuant.swift:432-488).  The two sides live
 * in two caches of the same geometry (max_seq_len, max_batch, num_kv_heads, num_layers): append the step's rows to both
 * (er_kv_append_rope_kv), run attention with the K rows of `key_cache` and the V rows of `value_cache`, advance both.  Any
 * pair of float16 (head-major / paged), q8_0 and TurboQuant caches (all presets) is accepted; positions are the key cache's.
 * Decode runs on the tensor cores for every pair of float16 (head-major / paged), q8_0 and fixed-preset TurboQuant caches (GQA
 * groups 1, 2, 4, 8; no sliding window); the prefill form expands both sides to fp16 rows and
 * runs the tensor-core prefill kernel for any pair; a plain SIMT kernel serves the other decode pairs and sliding windows (correct, not
 * tuned).  On the SIMT kernel (sliding windows, ER_DECODE_KERNEL_SIMT) the prefill form takes a chunk that ends at the newest row. */
int32_t er_kv_attention_decode_pair(er_kv* key_cache, er_kv* value_cache, uint32_t layer_begin, uint32_t layer_end, const float* q,
                                    float* out, uint32_t num_heads, uint32_t pending, const er_step_params* params, void* stream);
int32_t er_kv_attention_prefill_pair(er_kv* key_cache, er_kv* value_cache, uint32_t layer, uint32_t seq, const float* q, float* out,
                                     uint32_t num_heads, uint32_t seq_len, uint32_t q_offset, const er_step_params* params, void* stream);

/* Whole decode step for layers [layer_begin, layer_end): append + attention + advance of the write position by
 * one, enqueued back to back (the body of fusedDecodePass steps 2-5, LlamaLanguageModel.swift:3649-3941).
 * Positions live on the device, so a captured CUDA graph of this call can be replayed step after step. */
int32_t er_kv_decode_step(er_kv* kv, uint32_t layer_begin, uint32_t layer_end, const float* q, const float* k,
                          const float* v, float* out, uint32_t num_heads, const er_step_params* params, void* stream);

/* Same step with HOST buffers (pinned or pageable): q/k/v come from host memory, `out` goes back to it, and the call
 * returns when the rows are there (with the step's device status as its result).  This is the call a host-side model
 * loop makes when its activations live in host memory.  With every buffer pinned (cudaHostAlloc / er_host_alloc) a
 * float16 cache runs the step as ONE launch: the kernel pulls its q/k/v rows out of the mapped buffers while earlier
 * tiles stream, stores the output rows into host memory and reports to a host word the call polls -- no staging copy, no
 * stream synchronisation.  `host_out` may also be DEVICE memory (a kv-head shard writing into the gathered buffer of
 * er_kv_set_output_sharding): the call then only enqueues the step and returns; keep host_q/k/v untouched until `stream`
 * has passed it and read the status with er_kv_device_status.  One step in flight per cache. */
int32_t er_kv_decode_step_host(er_kv* kv, uint32_t layer_begin, uint32_t layer_end, const float* host_q,
                               const float* host_k, const float* host_v, float* host_out, uint32_t num_heads,
                               const er_step_params* params, void* stream);

/* Device advance of the write position of every sequence of layers [layer_begin, layer_end) by `count`. */
int32_t er_kv_advance(er_kv* kv, uint32_t layer_begin, uint32_t layer_end, uint32_t count, void* stream);

/* Bulk load of already-positioned rows (prefill / test set-up): rows [start, start+count) of (layer, seq) from
 * device float [count][numKVHeads][headDim]; K is NeoX-rotated at its row position when params->apply_rope.
 * Sets totalWritten of (layer, seq) to max(totalWritten, start + count). */
int32_t er_kv_write_rows(er_kv* kv, uint32_t layer, uint32_t seq, uint32_t start, uint32_t count, const float* k,
                         const float* v, const er_step_params* params, void* stream);

/* ---- pages as bytes (no counterpart in the reference, whose prefix reuse is setPosition on one ring) ----
 * A page of the paged layout (of the head-major layout: one sequence's whole ring, page id = sequence index) holds
 * page_size tokens of every kv head; er_kv_page_bytes is its size over ALL layers, side arrays (TurboQuant norms, q8_0
 * scales) included.  er_kv_export_pages packs pages page_ids[0..count) into `buffer` (device, or host memory -- pinned for
 * an asynchronous copy), er_kv_import_pages writes such bytes into pages of a cache of the same shape and format (this one or
 * another): a prompt prefix computed once can be parked on the host, handed to another cache, or attached to several
 * sequences (import into fresh pages, er_kv_set_block_table, er_kv_set_position).  Positions are not part of a page: RoPE'd
 * keys carry their absolute position, so a prefix keeps its meaning only at the same token offsets.  Copies are enqueued
 * on `stream` and ordered with the cache's kernels there. */
int64_t er_kv_page_bytes(er_kv* kv);
int32_t er_kv_export_pages(er_kv* kv, const int32_t* page_ids, uint32_t count, void* buffer, size_t buffer_bytes, void* stream);
int32_t er_kv_import_pages(er_kv* kv, const int32_t* page_ids, uint32_t count, const void* buffer, size_t buffer_bytes, void* stream);

/* ---- kv-head sharding across the GPUs of one node (no counterpart in the reference, which is single-device) ----
 * Rank r of G holds kv heads [r * Hkv / G, (r + 1) * Hkv / G) in its own er_kv cache and the query heads that attend to
 * them.  Attention needs no reduction across ranks, only the concatenation of the per-head outputs; two ways to get it:
 *
 * (1) Fused: er_kv_set_output_sharding makes every decode launch of the cache write its finished rows straight into a
 *     [layers][batch][heads_total][128] buffer at head offset `head_offset` -- the `out` argument of the call -- and into
 *     the same buffer at up to 8 more addresses (`peer_outputs`: the other GPUs' buffers obtained with er_peer_buffer_open -- and,
 *     when the call's `out` is pinned host memory, this GPU's own device buffer), with ordinary
 *     stores from the kernel's merge epilogue.  When every rank's launch has completed (order that with any barrier,
 *     e.g. a 4-byte all-reduce enqueued behind the step) each GPU holds all heads.  Nothing is read from a peer.
 *     heads_total == 0 turns it off.
 * (2) Library collective: each rank computes its [layers][batch][local_heads][128] slice, an all-gather (NCCL) yields
 *     [world][layers][batch][local_heads][128], and er_relayout_head_shards turns that into
 *     [layers][batch][world * local_heads][128] (pairs = layers * batch). */
int32_t er_kv_set_output_sharding(er_kv* kv, uint32_t heads_total, uint32_t head_offset, float* const* peer_outputs, uint32_t num_peers);
int32_t er_relayout_head_shards(const float* gathered, float* full, uint32_t world, uint32_t pairs, uint32_t local_heads, void* stream);
/* Device buffers another process of this node can map (CUDA IPC): create one here (zero-filled) and hand the 64-byte
 * handle to the peers (any channel); a peer maps it with er_peer_buffer_open (which also enables peer access between the
 * two GPUs) and unmaps it with er_peer_buffer_close before the owner calls er_peer_buffer_destroy. */
int32_t er_peer_buffer_create(size_t bytes, void** device_ptr, uint8_t* handle_out /* 64 bytes */);
int32_t er_peer_buffer_open(const uint8_t* handle /* 64 bytes */, void** device_ptr);
int32_t er_peer_buffer_close(void* opened_ptr);
int32_t er_peer_buffer_destroy(void* device_ptr);

/* Number of kernels this library has launched since load (all caches, this process). */
uint64_t er_kernel_launch_count(void);
/* Device status word of the cache (synchronises with the device): ER_OK, ER_ERR_DEVICE_TIMEOUT if a bounded wait inside a
 * kernel expired (the launch still ran to its end; its outputs are not valid), or ER_ERR_OUT_OF_PAGES if a device-side
 * append met a block-table entry without a page (that row was dropped, nothing else was touched).  The word is sticky
 * until er_kv_clear_device_status.  er_kv_decode_step_host returns the same codes by itself. */
int32_t er_kv_device_status(er_kv* kv);
int32_t er_kv_clear_device_status(er_kv* kv);
/* Test hook for that status path: decode launches of this cache that follow wait at most `wait_limit_us` microseconds
 * (0 = the normal 2 s) on each of their internal barriers, and with withhold_tiles != 0 their copy-issuing warp stays
 * idle, so the first wait runs out: the launch still runs to its end on its own (nothing traps or spins), its outputs
 * are undefined and the status word reads ER_ERR_DEVICE_TIMEOUT.  (0, 0) restores normal operation. */
int32_t er_kv_debug_wait_probe(er_kv* kv, uint32_t wait_limit_us, int withhold_tiles);
/* The same word for the raw-buffer operators (er_gqa_attention_f16kv, er_gqa_attention_f16kv_windowed) on the current
 * device; reading it clears it.  Those operators share one workspace per device: keep their calls on one stream (or
 * order them yourself), two that overlap on the GPU race on the split-K partials. */
int32_t er_workspace_status(void);
/* And for er_gqa_attention_f16kv_static's built-in workspace on the current device; reading it clears it. */
int32_t er_gqa_attention_f16kv_static_status(void);

/* Diagnostics (the counterpart of the reference's per-phase trace collectors,
 * Sources/EdgeRunner/Models/LlamaLanguageModel.swift:6322-6558): while a buffer is installed every CTA of a decode
 * launch writes 8 nanosecond timestamps (start, scheduled, first tile landed, streaming done, pre-exit barrier, ...)
 * to device_buffer[cta*8 ..].  Returns the number of CTAs a launch uses; a smaller capacity disables tracing.
 * NULL uninstalls. */
int32_t er_kv_set_trace(er_kv* kv, uint64_t* device_buffer, uint32_t capacity_ctas);

/* Pinned host memory helpers for callers without a CUDA runtime binding of their own. */
int32_t er_host_alloc(void** out, size_t bytes);
int32_t er_host_free(void* ptr);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* ER_KV_H */
