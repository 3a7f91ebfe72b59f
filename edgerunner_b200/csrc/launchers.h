// Launch entry points of the decode kernels, one translation unit per storage format so they compile in
// parallel.  Return value: cudaSuccess (0), a cudaError_t from configuration or launch, or -1 when the
// requested template combination is not built.
#pragma once

#include <cuda_runtime.h>

#include "flash_decode.cuh"

namespace er {

constexpr int kNotBuilt = -1;

int launch_decode_dense(int group, const DecodeParams& p, int grid, cudaStream_t stream);
// Slots per staged tile of the fp16 kernel built for `group` (the tensor maps' box height), 0 when not built.
int decode_dense_tile_tokens(int group);
// Fills p.k_map / p.v_map / p.use_tmap for token-major fp16 rows [layers][seqs][slots][kv_heads][128]; layer strides
// in bytes (0 with one layer).  Returns 0, or -1 when the driver entry point is missing or refuses the layout
// (p.use_tmap stays 0 and the kernel copies row by row).
int encode_token_major_maps(DecodeParams& p, int group, uint64_t layers, uint64_t seqs, uint64_t slots, uint64_t kv_heads);
// fp16 rows, small launches (decode_slim.cu): grid (splits, kv heads, (layer, sequence) pairs), no staging.  kNotBuilt when
// the launch uses something only the persistent kernel has (ring ranges, sliding windows, sharded outputs, groups > 4).
int decode_slim_splits(int group, int items, int max_units, int num_sms, size_t scratch_floats);
int launch_decode_slim(int group, const DecodeParams& p, int splits, cudaStream_t stream);
int launch_decode_turbo(int group, int kbits, int vbits, const DecodeParams& p, int grid, cudaStream_t stream);
int launch_decode_q8(int group, const DecodeParams& p, int grid, cudaStream_t stream);
// q8_0 keys (p.k_*, p.kn_*, p.addr) with TurboQuant values of a fixed preset (p.v_*, p.vn_*, p.addr_v): two caches (decode_hybrid.cu)
int launch_decode_q8k_turbov(int group, int vbits, const DecodeParams& p, int grid, cudaStream_t stream);
// float16 keys (head-major or paged rows) with TurboQuant values of a fixed preset; kNotBuilt for 4-bit values with eight heads per kv head
int launch_decode_densek_turbov(int group, int vbits, const DecodeParams& p, int grid, cudaStream_t stream);
// TurboQuant keys of a fixed preset with float16 values (head-major or paged rows); kNotBuilt for 4-bit keys with eight heads per kv head
int launch_decode_turbok_densev(int group, int kbits, const DecodeParams& p, int grid, cudaStream_t stream);
// q8_0 keys with float16 values (q8_keys != 0) or float16 keys with q8_0 values
int launch_decode_q8_dense_pair(int group, int q8_keys, const DecodeParams& p, int grid, cudaStream_t stream);
// TurboQuant keys of a fixed preset with q8_0 values (p.v_* rows, p.vn_* block scales)
int launch_decode_turbok_q8v(int group, int kbits, const DecodeParams& p, int grid, cudaStream_t stream);
// balanced (3 / 5 bits) and aggressive (2 / 3 bits) TurboQuant rows, groups 1, 2, 4 (decode_outlier.cu); kNotBuilt otherwise
int launch_decode_outlier(int group, int regular_bits, int high_bits, const DecodeParams& p, int grid, cudaStream_t stream);
struct PrefillParams;
int launch_prefill_f16(int group, const PrefillParams& p, int num_kv_heads, cudaStream_t stream);
// tcgen05 version of the same kernel.  outer_extent: pages in the pool (page-major rows) or sequences (token-major rows)
// behind p.k_layer; status: device word that receives kStatusTimeout if a bounded wait gives up.  kNotBuilt when the
// shape or the layout is not covered (the caller then uses launch_prefill_f16).
int launch_prefill_umma(int group, const PrefillParams& p, uint64_t outer_extent, int num_kv_heads, int* status, cudaStream_t stream);
// Floats of scratch (PrefillParams::split_partial) that let the tcgen05 kernel cut the tail of its grid along the keys.
size_t prefill_split_partial_floats(int num_sms);

// One query token against ring rows (start + i) % capacity, i < count, of token-major fp16 K/V [capacity][kv heads][head_dim];
// any even head_dim <= 512, any GQA group (decode_generic.cu).  scratch: nsplit x heads x (head_dim + 2) floats at most
// scratch_floats; counters: one zeroed int per head.  chunk / nsplit are filled by the launcher.
struct GenericDecodeParams {
    const float* q;      // [num_heads][head_dim]
    const __half* k;
    const __half* v;
    float* out;          // [num_heads][head_dim]
    int num_heads, num_kv_heads, head_dim;
    int start, count, capacity;
    float scale_log2;
    float* scratch;
    int* counters;
    int chunk, nsplit;
};
int launch_decode_generic(GenericDecodeParams p, int num_sms, size_t scratch_floats, size_t counter_ints, cudaStream_t stream);

// GQA attention over float32 K / V rows (attention_f32.cu): raw [kvSeqLen][kv heads][head_dim] buffers (lengths ==
// nullptr, one problem, seq_len query rows, optional additive mask [seq_len][mask_stride]) or a float32 cache (lengths
// set: one problem per (layer, sequence) of [layer_begin, ...), one query row each, kv length read on the device).
struct AttentionF32Params {
    const float* q;       // [problems][seq_len][num_heads][head_dim]
    float* out;
    const float* k;       // rows of layer 0
    const float* v;
    int64_t layer_stride_elems;
    const float* mask;    // additive, or nullptr
    int mask_stride;
    int seq_len, head_dim, num_heads, num_kv_heads;
    int causal, q_offset, kv_len;
    float scale;
    const int32_t* lengths;
    int layer_begin, batch, pending;
    int apply_rope;       // cache mode, head_dim 128: NeoX-rotate the query row at position kv_len - 1
    float rope_scaling;
    KVAddressing addr;
    InvFreqTable inv_freq;
};
int launch_attention_f32(const AttentionF32Params& p, int problems, cudaStream_t stream);

template <class POL, bool HOSTIO>
inline int launch_decode_variant(const DecodeParams& p, int grid, cudaStream_t stream) {
    constexpr int kSmem = DecodeSmem<POL>::kTotal;
    static_assert(kSmem <= 232448, "decode kernel exceeds the 227 KiB shared-memory limit of an sm_100 CTA");
    static int configured_device = -1;   // the attribute is per device and sticky: set it once
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (configured_device != device) {
        e = cudaFuncSetAttribute(flash_decode_kernel<POL, HOSTIO>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured_device = device;
    }
    // Programmatic dependent launch: the CTAs of this launch may be placed while the previous kernel of the stream drains
    // (one CTA per SM, so each starts when that SM's previous CTA has left); the kernel waits for the previous grid
    // (griddepcontrol.wait) before it touches global memory, so only launch latency and the CTA prologue overlap.
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3((POL::kUnitsPerTile * POL::kWarpGroups + 1) * 32);
    cfg.dynamicSmemBytes = kSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, flash_decode_kernel<POL, HOSTIO>, p));
}

// p.host_q set (host-buffer step on a policy with the fused append): the variant of the kernel that pulls the rows itself.
template <class POL>
inline int launch_decode_policy(const DecodeParams& p, int grid, cudaStream_t stream) {
    if constexpr (POL::kFusedAppend) {
        if (p.host_q != nullptr) return launch_decode_variant<POL, true>(p, grid, stream);
    }
    return launch_decode_variant<POL, false>(p, grid, stream);
}

}  // namespace er
