// TurboQuant quantise / dequantise kernels and their launchers (included by the host translation unit only).
// Device math and the bit-exactness notes live in tq_math.cuh.
#pragma once

#include "append.cuh"
#include "er_common.cuh"
#include "tq_math.cuh"

namespace er {

// ------------------------------------------------------------------------------------------ quantize kernels

constexpr int kQuantWarps = 4;
constexpr int kQuantRowsPerWarp = 16;
constexpr int kQuantRowStride = kHeadDim + 1;   // odd stride: one lane per row walks it without bank conflicts

// Shared body: quantises the `nrows` rows a warp holds in `tile` (float [16][129], already rotated by RoPE if
// wanted).  For row r it leaves the packed code words in pack[r][0..words) and returns, in lane r, the norm
// to store (rowNorm / ||centroids||, TurboQuant.swift:1056-1058) -- 0 for an all-zero row.
template <int BITS>
__device__ __forceinline__ float tq_quantize_tile(float* tile, uint32_t* pack, int nrows, int lane) {
    constexpr int kWords = tq_code_words(BITS);
    const float* cent = tq_centroids<BITS>();
    // (1) rowNorm = sqrt(sum x^2), accumulated left to right (TurboQuant.swift:1016).
    float norm = 0.f;
    if (lane < nrows) {
        const float* row = tile + lane * kQuantRowStride;
        float sum = 0.f;
#pragma unroll 8
        for (int d = 0; d < kHeadDim; ++d) sum = __fadd_rn(sum, __fmul_rn(row[d], row[d]));
        norm = __fsqrt_rn(sum);
    }
    // (2) per row: normalise, rotate, code, pack; centroid^2 overwrites the row for step (3).
    for (int r = 0; r < nrows; ++r) {
        const float rn = __shfl_sync(0xffffffffu, norm, r);
        float* row = tile + r * kQuantRowStride;
        uint32_t* words = pack + r * 16;
        if (lane < kWords) words[lane] = 0u;
        __syncwarp();
        if (rn > 0.f) {
            float a[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) a[c] = __fdiv_rn(row[4 * lane + c], rn);
            warp_tq_forward(a, lane);
            uint32_t piece = 0;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t code = tq_code_for<BITS>(a[c]);
                piece |= code << (BITS * c);
                const float cv = cent[code];
                row[4 * lane + c] = __fmul_rn(cv, cv);
            }
            // BitPacker.insert (TurboQuant.swift:1554-1573): code i at stream bits [i*BITS, i*BITS+BITS).
            const int off = 4 * BITS * lane, w0 = off >> 5, sh = off & 31;
            atomicOr(&words[w0], piece << sh);
            if (sh + 4 * BITS > 32) atomicOr(&words[w0 + 1], piece >> (32 - sh));
        }
        __syncwarp();
    }
    // (3) corrected norm: rowNorm / sqrt(sum centroid^2), the sum again left to right (TurboQuant.swift:1057).
    float stored = 0.f;
    if (lane < nrows && norm > 0.f) {
        const float* row = tile + lane * kQuantRowStride;
        float sum = 0.f;
#pragma unroll 8
        for (int d = 0; d < kHeadDim; ++d) sum = __fadd_rn(sum, row[d]);
        const float rec = __fsqrt_rn(sum);
        stored = rec > 0.f ? __fdiv_rn(norm, rec) : norm;
    }
    return stored;
}

// turboquant_quantize_rows for the fixed presets, writing the reference's four split buffers
// (codes, residual signs = 0, outlier mask = 0, metadata = (norm, 0)).
template <int BITS>
__global__ void __launch_bounds__(kQuantWarps * 32) tq_quantize_rows_kernel(const float* source, uint32_t row_count,
                                                                           uint32_t src_stride, uint32_t dst_row_base,
                                                                           uint32_t* out_codes, uint32_t* out_signs,
                                                                           uint32_t* out_mask, float* out_meta) {
    __shared__ float tile_all[kQuantWarps][kQuantRowsPerWarp * kQuantRowStride];
    __shared__ __align__(16) uint32_t pack_all[kQuantWarps][kQuantRowsPerWarp * 16];
    constexpr int kWords = tq_code_words(BITS);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* tile = tile_all[warp];
    uint32_t* pack = pack_all[warp];
    const uint32_t first = (blockIdx.x * kQuantWarps + warp) * kQuantRowsPerWarp;
    if (first >= row_count) return;
    const int nrows = static_cast<int>(min(static_cast<uint32_t>(kQuantRowsPerWarp), row_count - first));
    for (int r = 0; r < nrows; ++r) {
        const float4 x = *reinterpret_cast<const float4*>(source + static_cast<size_t>(first + r) * src_stride + 4 * lane);
        float* row = tile + r * kQuantRowStride + 4 * lane;
        row[0] = x.x; row[1] = x.y; row[2] = x.z; row[3] = x.w;
    }
    __syncwarp();
    const float stored = tq_quantize_tile<BITS>(tile, pack, nrows, lane);
    __syncwarp();
    for (int r = 0; r < nrows; ++r) {
        const size_t dst = static_cast<size_t>(dst_row_base) + first + r;
        if (lane < kWords) out_codes[dst * kWords + lane] = pack[r * 16 + lane];
        if (lane < 4) {
            if (out_signs) out_signs[dst * 4 + lane] = 0u;
            if (out_mask) out_mask[dst * 4 + lane] = 0u;
        }
    }
    if (lane < nrows) {
        const size_t dst = static_cast<size_t>(dst_row_base) + first + lane;
        out_meta[dst * 2] = stored;
        out_meta[dst * 2 + 1] = 0.f;
    }
}

struct TurboAppendParams {
    AppendParams base;           // k_base / v_base hold packed codes
    uint8_t* kn_base;
    uint8_t* vn_base;
    int64_t n_layer_stride_bytes;
    int norm_fp16;
};

// A source row of an append (kv head h of source row r) as a warp holds it -- lane L: coordinates 4L .. 4L + 3 -- with the
// NeoX rotation of K rows at the row's position applied (cos / sin exactly rounded: these values decide cache bits).
__device__ __forceinline__ float4 tq_append_load_row(const AppendParams& p, bool is_v, int r, int h, int lane) {
    const int hkv = p.addr.num_kv_heads;
    const float* src = (is_v ? p.v : p.k) + (static_cast<int64_t>(r) * hkv + h) * kHeadDim;
    float4 x = __ldg(reinterpret_cast<const float4*>(src + 4 * lane));
    if (!is_v && p.apply_rope) {
        int layer, seq;
        uint32_t pos;
        append_locate(p, r, layer, seq, pos);
        // lane holds dims 4*lane..+3; the NeoX partner (d +- 64) lives 16 lanes away.
        float xs[4] = {x.x, x.y, x.z, x.w}, ys[4];
        // Lanes l and l^16 need the same four (cos, sin) pairs: each computes two and they swap.
        const int base_pair = 4 * (lane & 15), mine = (lane >> 4) * 2;
        const float2 m0 = rope_cos_sin(pos, p.inv_freq.f[base_pair + mine], p.rope_scaling);
        const float2 m1 = rope_cos_sin(pos, p.inv_freq.f[base_pair + mine + 1], p.rope_scaling);
        float2 o0, o1;
        o0.x = __shfl_xor_sync(0xffffffffu, m0.x, 16); o0.y = __shfl_xor_sync(0xffffffffu, m0.y, 16);
        o1.x = __shfl_xor_sync(0xffffffffu, m1.x, 16); o1.y = __shfl_xor_sync(0xffffffffu, m1.y, 16);
        const float2 cs4[4] = {lane < 16 ? m0 : o0, lane < 16 ? m1 : o1, lane < 16 ? o0 : m0, lane < 16 ? o1 : m1};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float other = __shfl_xor_sync(0xffffffffu, xs[c], 16);
            float y0, y1;
            if (lane < 16) { rope_rotate(xs[c], other, cs4[c], y0, y1); ys[c] = y0; }
            else           { rope_rotate(other, xs[c], cs4[c], y0, y1); ys[c] = y1; }
        }
        x = make_float4(ys[0], ys[1], ys[2], ys[3]);
    }
    return x;
}

// Fused decode/prefill append for a TurboQuant cache: [NeoX RoPE on K] -> quantise -> packed row + norm
// into the cache slot.  Job j = (source row r, kv head h, K or V); a warp takes `jobs_per_warp`
// consecutive jobs.  Replaces RoPE(K) + 2 x turboquant_quantize_rows per layer
// (LlamaLanguageModel.swift:3659-3673, 3779-3811).
template <int KBITS, int VBITS>
__global__ void __launch_bounds__(kQuantWarps * 32) tq_append_kernel(const __grid_constant__ TurboAppendParams tp,
                                                                    int jobs_per_warp) {
    __shared__ float tile_all[kQuantWarps][kQuantRowsPerWarp * kQuantRowStride];
    __shared__ __align__(16) uint32_t pack_all[kQuantWarps][kQuantRowsPerWarp * 16];
    // the decode kernel behind this one is a programmatic dependent launch: its CTAs may be placed and build their tables now
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const AppendParams& p = tp.base;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* tile = tile_all[warp];
    uint32_t* pack = pack_all[warp];
    const int hkv = p.addr.num_kv_heads;
    const int64_t total_jobs = static_cast<int64_t>(p.rows) * hkv * 2;
    // K jobs first ([0, rows*hkv)), then V jobs, so a warp never mixes bit widths.
    const int64_t half_jobs = static_cast<int64_t>(p.rows) * hkv;
    const int64_t warps_k = (half_jobs + jobs_per_warp - 1) / jobs_per_warp;
    const int64_t gw = static_cast<int64_t>(blockIdx.x) * kQuantWarps + warp;
    if (gw >= 2 * warps_k) return;
    const bool is_v = gw >= warps_k;
    const int64_t first = (is_v ? gw - warps_k : gw) * jobs_per_warp;
    const int njobs = static_cast<int>(static_cast<int64_t>(jobs_per_warp) < half_jobs - first ? static_cast<int64_t>(jobs_per_warp) : half_jobs - first);
    (void)total_jobs;

    for (int jj = 0; jj < njobs; ++jj) {
        const int64_t job = first + jj;
        const int r = static_cast<int>(job / hkv), h = static_cast<int>(job % hkv);
        const float4 x = tq_append_load_row(p, is_v, r, h, lane);
        float* row = tile + jj * kQuantRowStride + 4 * lane;
        row[0] = x.x; row[1] = x.y; row[2] = x.z; row[3] = x.w;
    }
    __syncwarp();
    const float stored = is_v ? tq_quantize_tile<VBITS>(tile, pack, njobs, lane) : tq_quantize_tile<KBITS>(tile, pack, njobs, lane);
    __syncwarp();
    const int words = is_v ? tq_code_words(VBITS) : tq_code_words(KBITS);
    for (int jj = 0; jj < njobs; ++jj) {
        const int64_t job = first + jj;
        const int r = static_cast<int>(job / hkv), h = static_cast<int>(job % hkv);
        int layer, seq;
        uint32_t pos;
        append_locate(p, r, layer, seq, pos);
        const int slot = static_cast<int>(pos % static_cast<uint32_t>(p.addr.max_seq_len));
        const int64_t ridx = row_index_for_write(p.addr, seq, h, slot);
        if (ridx < 0) continue;   // no page behind the slot: dropped, the status word says so
        uint8_t* codes = (is_v ? p.v_base + layer * p.v_layer_stride_bytes : p.k_base + layer * p.k_layer_stride_bytes) +
                         ridx * (words * 4);
        // 16-byte vector stores: words*4 bytes = 32 / 48 / 64.
        if (lane < words / 4) reinterpret_cast<uint4*>(codes)[lane] = reinterpret_cast<const uint4*>(pack + jj * 16)[lane];
        const float nv = __shfl_sync(0xffffffffu, stored, jj);
        if (lane == 0) {
            uint8_t* nb = (is_v ? tp.vn_base : tp.kn_base) + layer * tp.n_layer_stride_bytes;
            if (tp.norm_fp16) reinterpret_cast<__half*>(nb)[ridx] = __float2half_rn(nv);
            else reinterpret_cast<float*>(nb)[ridx] = nv;
        }
    }
}

// ------------------------------------------------------------------------------------------ dequantise rows

struct TurboDecodeRowsParams {
    const uint8_t* codes;
    const uint8_t* norms;
    float* out;                 // [tokens][num_kv_heads][128] in logical order
    KVAddressing addr;
    int seq, first_slot, tokens, norm_fp16;
};

// approximateDecode (TurboQuant.swift:1117-1147): x_hat = inverse(centroids) * rowNorm.  One warp per row.
template <int BITS>
__global__ void tq_decode_rows_kernel(const __grid_constant__ TurboDecodeRowsParams p) {
    constexpr int kWords = tq_code_words(BITS);
    const float* cent = tq_centroids<BITS>();
    const int lane = threadIdx.x & 31;
    const int64_t total = static_cast<int64_t>(p.tokens) * p.addr.num_kv_heads;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < total;
         row += static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5)) {
        const int t = static_cast<int>(row / p.addr.num_kv_heads), h = static_cast<int>(row % p.addr.num_kv_heads);
        const int slot = (p.first_slot + t) % p.addr.max_seq_len;
        const int64_t ridx = row_index(p.addr, p.seq, h, slot);
        const uint32_t* words = reinterpret_cast<const uint32_t*>(p.codes + ridx * (kWords * 4));
        const float norm = p.norm_fp16 ? __half2float(reinterpret_cast<const __half*>(p.norms)[ridx])
                                       : reinterpret_cast<const float*>(p.norms)[ridx];
        const int off = 4 * BITS * lane, w0 = off >> 5, sh = off & 31;
        uint32_t bits = words[w0] >> sh;
        if (sh + 4 * BITS > 32) bits |= words[w0 + 1] << (32 - sh);
        float a[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) a[c] = cent[(bits >> (BITS * c)) & ((1u << BITS) - 1u)];
        warp_tq_inverse(a, lane);
        *reinterpret_cast<float4*>(p.out + row * kHeadDim + 4 * lane) =
            make_float4(__fmul_rn(a[0], norm), __fmul_rn(a[1], norm), __fmul_rn(a[2], norm), __fmul_rn(a[3], norm));
    }
}

// ---- pieces of the TurboQuant chunked-prefill path (gqa_attention_turboquant, Shaders/TurboQuant.metal:1454-1649) ----
// The contraction runs on the fp16 tensor-core prefill kernel in the *rotated* space:
//   score = <fwd(q), kNorm * centroids(K codes)> * scale ,  out = inverse( sum_t p_t * vNorm_t * centroids(V codes) ).

// Rows [0, *len) of (seq, every kv head): norm * centroid(code) as fp16, head-major [kv head][slot][128].
struct TurboExpandParams {
    const uint8_t* codes;
    const uint8_t* norms;
    __half* out;
    __half* out_lo;   // optional: fp16 of (value - fp16(value)), same shape
    KVAddressing addr;
    const int32_t* len_ptr;
    int seq, out_stride_rows, norm_fp16;
};

template <int BITS>
__global__ void tq_expand_rows_f16_kernel(const __grid_constant__ TurboExpandParams p) {
    constexpr int kWords = tq_code_words(BITS);
    // the codebook in shared memory: its entries lie in distinct banks, so a warp's 32 different codes cost one access
    // (the same reads from constant memory serialise, one pass per distinct code)
    __shared__ float cent[1 << BITS];
    if (threadIdx.x < (1 << BITS)) cent[threadIdx.x] = tq_centroids<BITS>()[threadIdx.x];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    int len = *p.len_ptr;
    len = len < p.addr.max_seq_len ? len : p.addr.max_seq_len;
    const int64_t total = static_cast<int64_t>(len) * p.addr.num_kv_heads;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < total;
         row += static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5)) {
        const int h = static_cast<int>(row / len), t = static_cast<int>(row % len);
        const int64_t ridx = row_index(p.addr, p.seq, h, t);
        const uint32_t* words = reinterpret_cast<const uint32_t*>(p.codes + ridx * (kWords * 4));
        const float norm = p.norm_fp16 ? __half2float(reinterpret_cast<const __half*>(p.norms)[ridx])
                                       : reinterpret_cast<const float*>(p.norms)[ridx];
        const int off = 4 * BITS * lane, w0 = off >> 5, sh = off & 31;
        uint32_t bits = words[w0] >> sh;
        if (sh + 4 * BITS > 32) bits |= words[w0 + 1] << (32 - sh);
        float a[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) a[c] = norm * cent[(bits >> (BITS * c)) & ((1u << BITS) - 1u)];
        uint2 o;
        const __half2 h01 = __floats2half2_rn(a[0], a[1]), h23 = __floats2half2_rn(a[2], a[3]);
        reinterpret_cast<__half2*>(&o)[0] = h01;
        reinterpret_cast<__half2*>(&o)[1] = h23;
        reinterpret_cast<uint2*>(p.out + (static_cast<int64_t>(h) * p.out_stride_rows + t) * kHeadDim)[lane] = o;
        if (p.out_lo != nullptr) {
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            reinterpret_cast<__half2*>(&o)[0] = __floats2half2_rn(a[0] - f01.x, a[1] - f01.y);
            reinterpret_cast<__half2*>(&o)[1] = __floats2half2_rn(a[2] - f23.x, a[3] - f23.y);
            reinterpret_cast<uint2*>(p.out_lo + (static_cast<int64_t>(h) * p.out_stride_rows + t) * kHeadDim)[lane] = o;
        }
    }
}

// rows [n][128] float: forward ([NeoX RoPE at position pos0 + row / heads ->] randomizedHadamard) or inverse transform,
// one warp per row; in == out allowed.
struct TurboRotateParams {
    const float* in;
    float* out;
    int rows, heads, inverse, apply_rope, pos_from_len, seq_len;
    uint32_t pos0;
    const int32_t* len_ptr;   // pos_from_len: pos0 = min(*len_ptr, max_len) - seq_len
    int max_len;
    float rope_scaling;
    InvFreqTable inv_freq;
};

__global__ void tq_rotate_rows_kernel(const __grid_constant__ TurboRotateParams p) {
    const int lane = threadIdx.x & 31;
    uint32_t pos0 = p.pos0;
    if (p.pos_from_len) {
        int len = *p.len_ptr;
        len = len < p.max_len ? len : p.max_len;
        pos0 = static_cast<uint32_t>(len - p.seq_len);
    }
    for (int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < p.rows; row += gridDim.x * (blockDim.x >> 5)) {
        const float4 x = *reinterpret_cast<const float4*>(p.in + static_cast<int64_t>(row) * kHeadDim + 4 * lane);
        float a[4] = {x.x, x.y, x.z, x.w};
        if (p.inverse) {
            warp_tq_inverse(a, lane);
        } else {
            if (p.apply_rope) {
                const uint32_t pos = pos0 + static_cast<uint32_t>(row / p.heads);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float other = __shfl_xor_sync(0xffffffffu, a[c], 16);
                    const float2 cs = rope_cos_sin_fast(pos, p.inv_freq.f[(4 * lane + c) & 63], p.rope_scaling);
                    float y0, y1;
                    if (lane < 16) { rope_rotate(a[c], other, cs, y0, y1); a[c] = y0; }
                    else           { rope_rotate(other, a[c], cs, y0, y1); a[c] = y1; }
                }
            }
            warp_tq_forward(a, lane);
        }
        *reinterpret_cast<float4*>(p.out + static_cast<int64_t>(row) * kHeadDim + 4 * lane) = make_float4(a[0], a[1], a[2], a[3]);
    }
}

// Stored norms -> the reference's metadata pairs (rowNorm, residualNorm = 0).
__global__ void widen_norms_kernel(const uint8_t* norms, float* meta, int rows, int norm_fp16) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    meta[2 * r] = norm_fp16 ? __half2float(reinterpret_cast<const __half*>(norms)[r]) : reinterpret_cast<const float*>(norms)[r];
    meta[2 * r + 1] = 0.f;
}

__global__ void set_min_length_kernel(int32_t* length, int value) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && *length < value) *length = value;
}

// ------------------------------------------------------------------------------------------ host launchers

typedef int32_t (*LaunchCheck)(const char*);

template <int BITS>
inline int32_t launch_quantize_rows_bits(const float* source, uint32_t row_count, uint32_t src_stride, uint32_t dst_row_base,
                                         uint32_t* codes, uint32_t* signs, uint32_t* mask, float* meta, cudaStream_t stream,
                                         LaunchCheck check) {
    const uint32_t per_block = kQuantWarps * kQuantRowsPerWarp;
    tq_quantize_rows_kernel<BITS><<<(row_count + per_block - 1) / per_block, kQuantWarps * 32, 0, stream>>>(
        source, row_count, src_stride, dst_row_base, codes, signs, mask, meta);
    return check("tq_quantize_rows_kernel");
}

inline int32_t launch_turbo_quantize_rows(const float* source, uint32_t row_count, uint32_t src_stride, uint32_t dst_row_base,
                                          int bits, uint32_t* codes, uint32_t* signs, uint32_t* mask, float* meta,
                                          cudaStream_t stream, LaunchCheck check) {
    switch (bits) {
        case 2: return launch_quantize_rows_bits<2>(source, row_count, src_stride, dst_row_base, codes, signs, mask, meta, stream, check);
        case 3: return launch_quantize_rows_bits<3>(source, row_count, src_stride, dst_row_base, codes, signs, mask, meta, stream, check);
        default: return launch_quantize_rows_bits<4>(source, row_count, src_stride, dst_row_base, codes, signs, mask, meta, stream, check);
    }
}

template <int KBITS, int VBITS>
inline int32_t launch_turbo_append_bits(const TurboAppendParams& tp, cudaStream_t stream, LaunchCheck check) {
    const int64_t half_jobs = static_cast<int64_t>(tp.base.rows) * tp.base.addr.num_kv_heads;
    // Few rows (a decode step): one row per warp keeps the serial norm walk off the critical path of other
    // rows; many rows (prefill): 16 rows per warp amortise it.
    const int jobs_per_warp = half_jobs >= 16384 ? kQuantRowsPerWarp : (half_jobs >= 2048 ? 4 : 1);
    const int64_t warps = 2 * ((half_jobs + jobs_per_warp - 1) / jobs_per_warp);
    const int blocks = static_cast<int>((warps + kQuantWarps - 1) / kQuantWarps);
    tq_append_kernel<KBITS, VBITS><<<blocks, kQuantWarps * 32, 0, stream>>>(tp, jobs_per_warp);
    return check("tq_append_kernel");
}

inline int32_t launch_turbo_append(const TurboAppendParams& tp, int kbits, int vbits, cudaStream_t stream, LaunchCheck check) {
#define ER_TQ_APPEND_CASE(KB, VB) \
    if (kbits == KB && vbits == VB) return launch_turbo_append_bits<KB, VB>(tp, stream, check);
    ER_TQ_APPEND_CASE(4, 4) ER_TQ_APPEND_CASE(4, 3) ER_TQ_APPEND_CASE(3, 3) ER_TQ_APPEND_CASE(3, 4)
    ER_TQ_APPEND_CASE(2, 2) ER_TQ_APPEND_CASE(4, 2) ER_TQ_APPEND_CASE(3, 2) ER_TQ_APPEND_CASE(2, 3) ER_TQ_APPEND_CASE(2, 4)
#undef ER_TQ_APPEND_CASE
    return -9;
}

inline int32_t launch_turbo_expand_rows(const TurboExpandParams& p, int bits, int max_rows, cudaStream_t stream, LaunchCheck check) {
    const int blocks = static_cast<int>((static_cast<int64_t>(max_rows) + 7) / 8 < 16384 ? (static_cast<int64_t>(max_rows) + 7) / 8 : 16384);
    switch (bits) {
        case 2: tq_expand_rows_f16_kernel<2><<<blocks, 256, 0, stream>>>(p); break;
        case 3: tq_expand_rows_f16_kernel<3><<<blocks, 256, 0, stream>>>(p); break;
        default: tq_expand_rows_f16_kernel<4><<<blocks, 256, 0, stream>>>(p); break;
    }
    return check("tq_expand_rows_f16_kernel");
}

inline int32_t launch_turbo_decode_rows(const TurboDecodeRowsParams& p, int bits, cudaStream_t stream, LaunchCheck check) {
    const int64_t rows = static_cast<int64_t>(p.tokens) * p.addr.num_kv_heads;
    const int blocks = static_cast<int>((rows + 7) / 8 < 8192 ? (rows + 7) / 8 : 8192);
    switch (bits) {
        case 2: tq_decode_rows_kernel<2><<<blocks, 256, 0, stream>>>(p); break;
        case 3: tq_decode_rows_kernel<3><<<blocks, 256, 0, stream>>>(p); break;
        default: tq_decode_rows_kernel<4><<<blocks, 256, 0, stream>>>(p); break;
    }
    return check("tq_decode_rows_kernel");
}

}  // namespace er
