// q8_0 KV rows: quantiser, cache append, export and expansion kernels.
//
// A q8_0 row of 128 elements is four blocks of 32: an fp16 scale and 32 int8 (34 bytes per block in the reference's
// buffers, KVCache.swift:175-184, 1007-1057; Shaders/Dequant_Q8_0.metal:19-49).  The cache keeps the two parts apart so
// that every access is aligned: 128 bytes of int8 per row in the K / V slabs and 4 fp16 scales (8 bytes) per row in the
// side slabs (the TurboQuant norm slabs' place); the reference's 34-byte blocks are produced on export.
// Inside a cached row the 32 words are permuted so that the decode kernel's lanes read contiguous bytes: the word that
// holds elements [4l, 4l + 4) (l = 0..31: block b = l / 8, 8-byte chunk c = (l % 8) / 2 of the block, half l % 2) is
// stored at word 8c + 2b + l % 2, i.e. the four chunks c of the four blocks are adjacent (q8_word_slot).
//   maxAbs = max |x| over the block (a NaN never becomes the maximum), scale = maxAbs > 0 ? maxAbs / 127 : 0 (fp32),
//   q = clamp(round-half-away(x / scale), -128, 127) with the unrounded scale, stored scale = fp16(scale).
#pragma once

#include "append.cuh"
#include "er_common.cuh"

namespace er {

constexpr int kQ8RowBytes = 128;      // int8 part of a row
constexpr int kQ8ScaleBytes = 8;      // four fp16 scales
constexpr int kQ8PackedRowBytes = 136;

// Position, inside a cached row, of the word that holds elements [4 lane, 4 lane + 4).
__host__ __device__ constexpr int q8_word_slot(int lane) { return 8 * ((lane & 7) >> 1) + 2 * (lane >> 3) + (lane & 1); }

// Lane holds elements [4 lane, 4 lane + 4) of a row; returns the four int8 as one word and the block's fp32 scale
// (identical in the 8 lanes of a block).
__device__ __forceinline__ uint32_t q8_quantize_lane(const float (&x)[4], float& scale_out) {
    float m = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const float a = fabsf(x[c]);
        m = a >= m ? a : m;
    }
#pragma unroll
    for (int off = 1; off < 8; off <<= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, m, off);
        m = o >= m ? o : m;
    }
    const float scale = m > 0.f ? __fdiv_rn(m, 127.f) : 0.f;
    uint32_t word = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        int q = 0;
        if (scale != 0.f) {
            float r = roundf(__fdiv_rn(x[c], scale));     // half away from zero
            if (!(r == r)) r = 0.f;
            r = fminf(fmaxf(r, -128.f), 127.f);
            q = static_cast<int>(r);
        }
        word |= (static_cast<uint32_t>(q) & 0xFFu) << (8 * c);
    }
    scale_out = scale;
    return word;
}

struct Q8AppendParams {
    AppendParams base;           // k_base / v_base hold the int8 rows
    uint8_t* ks_base;            // scales
    uint8_t* vs_base;
    int64_t s_layer_stride_bytes;
};

// [NeoX RoPE on K ->] quantise -> cache slot.  One warp per (source row, kv head, K | V) job.  Replaces rope_neox_f32 +
// 2 x quantize_q8_0_rows of the decode pass on a q8_0 layer.
__global__ void __launch_bounds__(256) q8_append_kernel(const __grid_constant__ Q8AppendParams qp) {
    // the decode kernel behind this one is a programmatic dependent launch: its CTAs may be placed and build their tables now
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const AppendParams& p = qp.base;
    const int lane = threadIdx.x & 31;
    const int hkv = p.addr.num_kv_heads;
    const int64_t half_jobs = static_cast<int64_t>(p.rows) * hkv;
    const int64_t job2 = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (job2 >= 2 * half_jobs) return;
    const bool is_v = job2 >= half_jobs;
    const int64_t job = is_v ? job2 - half_jobs : job2;
    const int r = static_cast<int>(job / hkv), h = static_cast<int>(job % hkv);
    int layer, seq;
    uint32_t pos;
    append_locate(p, r, layer, seq, pos);
    const float* src = (is_v ? p.v : p.k) + (static_cast<int64_t>(r) * hkv + h) * kHeadDim;
    const float4 x4 = __ldg(reinterpret_cast<const float4*>(src + 4 * lane));
    float x[4] = {x4.x, x4.y, x4.z, x4.w};
    if (!is_v && p.apply_rope) {
        // lane holds dims 4*lane..+3; the NeoX partner (d +- 64) lives 16 lanes away; lanes l and l^16 need the same four
        // (cos, sin) pairs: each computes two and they swap
        const int base_pair = 4 * (lane & 15), mine = (lane >> 4) * 2;
        const float2 m0 = rope_cos_sin(pos, p.inv_freq.f[base_pair + mine], p.rope_scaling);
        const float2 m1 = rope_cos_sin(pos, p.inv_freq.f[base_pair + mine + 1], p.rope_scaling);
        float2 o0, o1;
        o0.x = __shfl_xor_sync(0xffffffffu, m0.x, 16); o0.y = __shfl_xor_sync(0xffffffffu, m0.y, 16);
        o1.x = __shfl_xor_sync(0xffffffffu, m1.x, 16); o1.y = __shfl_xor_sync(0xffffffffu, m1.y, 16);
        const float2 cs4[4] = {lane < 16 ? m0 : o0, lane < 16 ? m1 : o1, lane < 16 ? o0 : m0, lane < 16 ? o1 : m1};
        float y[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float other = __shfl_xor_sync(0xffffffffu, x[c], 16);
            float y0, y1;
            if (lane < 16) { rope_rotate(x[c], other, cs4[c], y0, y1); y[c] = y0; }
            else           { rope_rotate(other, x[c], cs4[c], y0, y1); y[c] = y1; }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) x[c] = y[c];
    }
    float scale;
    const uint32_t word = q8_quantize_lane(x, scale);
    const int slot = static_cast<int>(pos % static_cast<uint32_t>(p.addr.max_seq_len));
    const int64_t ridx = row_index_for_write(p.addr, seq, h, slot);
    if (ridx < 0) return;   // no page behind the slot: dropped, the status word says so
    uint8_t* rows = is_v ? p.v_base + layer * p.v_layer_stride_bytes : p.k_base + layer * p.k_layer_stride_bytes;
    reinterpret_cast<uint32_t*>(rows + ridx * kQ8RowBytes)[q8_word_slot(lane)] = word;
    if ((lane & 7) == 0) {
        uint8_t* sc = (is_v ? qp.vs_base : qp.ks_base) + layer * qp.s_layer_stride_bytes;
        reinterpret_cast<__half*>(sc + ridx * kQ8ScaleBytes)[lane >> 3] = __float2half_rn(scale);
    }
}

// quantize_q8_0_rows (Shaders/Dequant_Q8_0.metal:19-49): float rows (stride in elements) -> 34-byte blocks, row
// `dst_row_base + r` of `blocks`; one warp per row of 128 elements.
__global__ void __launch_bounds__(256) q8_quantize_rows_packed_kernel(const float* __restrict__ src, uint32_t rows, uint32_t src_stride,
                                                                      uint32_t dst_row_base, uint8_t* __restrict__ blocks) {
    const int lane = threadIdx.x & 31;
    const uint32_t r = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= rows) return;
    const float* s = src + static_cast<int64_t>(r) * src_stride + 4 * lane;
    const float x[4] = {s[0], s[1], s[2], s[3]};
    float scale;
    const uint32_t word = q8_quantize_lane(x, scale);
    uint8_t* blk = blocks + (static_cast<int64_t>(dst_row_base) + r) * kQ8PackedRowBytes + (lane >> 3) * 34;
    // 34-byte blocks are only 2-byte aligned
    uint16_t* q16 = reinterpret_cast<uint16_t*>(blk + 2 + 4 * (lane & 7));
    q16[0] = static_cast<uint16_t>(word & 0xFFFFu);
    q16[1] = static_cast<uint16_t>(word >> 16);
    if ((lane & 7) == 0) *reinterpret_cast<__half*>(blk) = __float2half_rn(scale);
}

// Rows of (layer, seq) in ring order -> the reference's 34-byte blocks [token][kv head][136] and / or decoded floats
// [token][kv head][128] (KVCache.retrieveDecodedQ8_0, KVCache.swift:882-908; decodeQ8Row :1040-1057).
struct Q8ExportParams {
    const uint8_t* rows;      // layer base, int8 part
    const uint8_t* scales;    // layer base
    KVAddressing addr;
    int seq, tokens, first_slot;     // ring order: token i is slot (first_slot + i) % max_seq_len
    uint8_t* out_blocks;      // optional
    float* out_values;        // optional
};

__global__ void __launch_bounds__(256) q8_export_rows_kernel(const __grid_constant__ Q8ExportParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t total = static_cast<int64_t>(p.tokens) * p.addr.num_kv_heads;
    for (int64_t job = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); job < total; job += static_cast<int64_t>(gridDim.x) * 8) {
        const int t = static_cast<int>(job / p.addr.num_kv_heads), h = static_cast<int>(job % p.addr.num_kv_heads);
        const int slot = (p.first_slot + t) % p.addr.max_seq_len;
        const int64_t ridx = row_index(p.addr, p.seq, h, slot);
        const uint32_t word = reinterpret_cast<const uint32_t*>(p.rows + ridx * kQ8RowBytes)[q8_word_slot(lane)];
        const __half hs = reinterpret_cast<const __half*>(p.scales + ridx * kQ8ScaleBytes)[lane >> 3];
        if (p.out_blocks != nullptr) {
            uint8_t* blk = p.out_blocks + job * kQ8PackedRowBytes + (lane >> 3) * 34;
            uint16_t* q16 = reinterpret_cast<uint16_t*>(blk + 2 + 4 * (lane & 7));
            q16[0] = static_cast<uint16_t>(word & 0xFFFFu);
            q16[1] = static_cast<uint16_t>(word >> 16);
            if ((lane & 7) == 0) *reinterpret_cast<__half*>(blk) = hs;
        }
        if (p.out_values != nullptr) {
            const float sc = __half2float(hs);
            float4 o;
            o.x = __fmul_rn(sc, static_cast<float>(static_cast<int8_t>(word & 0xFF)));
            o.y = __fmul_rn(sc, static_cast<float>(static_cast<int8_t>((word >> 8) & 0xFF)));
            o.z = __fmul_rn(sc, static_cast<float>(static_cast<int8_t>((word >> 16) & 0xFF)));
            o.w = __fmul_rn(sc, static_cast<float>(static_cast<int8_t>(word >> 24)));
            reinterpret_cast<float4*>(p.out_values + job * kHeadDim)[lane] = o;
        }
    }
}

// Rows [0, *len) of (seq, every kv head): scale * q as fp16 (hi) and optionally the rounding residue (lo), head-major
// [kv head][slot][128]: the operands of the chunked-prefill kernels.
struct Q8ExpandParams {
    const uint8_t* rows;
    const uint8_t* scales;
    __half* out;
    __half* out_lo;
    KVAddressing addr;
    const int32_t* len_ptr;
    int seq, out_stride_rows;
};

__global__ void __launch_bounds__(256) q8_expand_rows_f16_kernel(const __grid_constant__ Q8ExpandParams p) {
    const int lane = threadIdx.x & 31;
    int len = *p.len_ptr;
    len = len < p.addr.max_seq_len ? len : p.addr.max_seq_len;
    const int64_t total = static_cast<int64_t>(len) * p.addr.num_kv_heads;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); row < total; row += static_cast<int64_t>(gridDim.x) * 8) {
        const int h = static_cast<int>(row / len), t = static_cast<int>(row % len);
        const int64_t ridx = row_index(p.addr, p.seq, h, t);
        const uint32_t word = reinterpret_cast<const uint32_t*>(p.rows + ridx * kQ8RowBytes)[q8_word_slot(lane)];
        const float sc = __half2float(reinterpret_cast<const __half*>(p.scales + ridx * kQ8ScaleBytes)[lane >> 3]);
        float a[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) a[c] = __fmul_rn(sc, static_cast<float>(static_cast<int8_t>((word >> (8 * c)) & 0xFF)));
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

}  // namespace er
