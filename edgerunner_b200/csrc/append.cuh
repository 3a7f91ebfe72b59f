// Row append / scatter / gather kernels for the dense (fp16 / fp32) KV cache.
//
// append_rope_dense_kernel fuses what the reference issues as separate dispatches per layer:
//   rope_neox_f32_to_f16   K row -> NeoX RoPE -> half() -> cache slot   (Shaders/RoPE.metal:498-531)
//   convert_f32_to_f16     V row -> half() -> cache slot                (LlamaLanguageModel.swift:3676-3684)
// for every (layer, sequence) of a decode step in one launch.  Each thread converts 2 x 8 contiguous
// elements (dims [8i,8i+8) and their RoPE partners [64+8i,64+8i+8)) and issues 16-byte stores.
#pragma once

#include "er_common.cuh"

namespace er {

struct AppendParams {
    const float* k;               // [rows][num_kv_heads][128]
    const float* v;
    uint8_t* k_base;
    uint8_t* v_base;
    int64_t k_layer_stride_bytes;
    int64_t v_layer_stride_bytes;
    const int32_t* lengths;       // decode mode: row position = lengths[layer][seq]
    int bulk;                     // 0: row r -> (layer_begin + r / batch, r % batch); 1: fixed (layer, seq), pos = start + r
    int layer_begin;
    int batch;
    int fixed_layer;
    int fixed_seq;
    int start_pos;
    int rows;
    float rope_scaling;
    int apply_rope;
    KVAddressing addr;
    InvFreqTable inv_freq;
};

// Per-head RMS norm, the first half of fused_qk_norm_rope_neox (Shaders/RoPE.metal:139-160):
//   out = (x * rsqrt(sum(x^2) / 128 + eps)) * weight[dim].
// The reference sums the 64 pair terms x[i]^2 + x[i+64]^2 with simd_sum per 32 pairs plus one add; the order inside
// simd_sum is not specified, so it is fixed here (and in the CPU restatement the tests compare with) as the xor
// butterfly 16, 8, 4, 2, 1 over the pair index, products and sums rounded separately, rsqrt correctly rounded.
// One warp per head row; rows are [groups][heads_per_group][128] with one weight vector per group (a layer).
struct HeadNormParams {
    const float* in;
    float* out;
    const float* weight;       // [groups][weight_stride] (stride 0: shared)
    int rows, rows_per_group, weight_stride;
    float eps;
};

__global__ void __launch_bounds__(256) head_rms_norm_kernel(const __grid_constant__ HeadNormParams p) {
    const int lane = threadIdx.x & 31;
    for (int row = blockIdx.x * 8 + (threadIdx.x >> 5); row < p.rows; row += gridDim.x * 8) {
        const float* x = p.in + static_cast<int64_t>(row) * kHeadDim;
        const float a = x[lane], b = x[lane + 64], c = x[lane + 32], d = x[lane + 96];
        float s0 = __fadd_rn(__fmul_rn(a, a), __fmul_rn(b, b));      // pair index lane
        float s1 = __fadd_rn(__fmul_rn(c, c), __fmul_rn(d, d));      // pair index lane + 32
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            s0 = __fadd_rn(s0, __shfl_xor_sync(0xffffffffu, s0, off));
            s1 = __fadd_rn(s1, __shfl_xor_sync(0xffffffffu, s1, off));
        }
        const float rs = __frsqrt_rn(__fadd_rn(__fdiv_rn(__fadd_rn(s0, s1), static_cast<float>(kHeadDim)), p.eps));
        const float* w = p.weight + static_cast<int64_t>(row / p.rows_per_group) * p.weight_stride;
        float* o = p.out + static_cast<int64_t>(row) * kHeadDim;
        o[lane] = __fmul_rn(__fmul_rn(a, rs), w[lane]);
        o[lane + 32] = __fmul_rn(__fmul_rn(c, rs), w[lane + 32]);
        o[lane + 64] = __fmul_rn(__fmul_rn(b, rs), w[lane + 64]);
        o[lane + 96] = __fmul_rn(__fmul_rn(d, rs), w[lane + 96]);
    }
}

__device__ __forceinline__ void append_locate(const AppendParams& p, int r, int& layer, int& seq, uint32_t& pos) {
    if (p.bulk) {
        layer = p.fixed_layer;
        seq = p.fixed_seq;
        pos = static_cast<uint32_t>(p.start_pos + r);
    } else {
        layer = p.layer_begin + r / p.batch;
        seq = r % p.batch;
        pos = static_cast<uint32_t>(p.lengths[layer * p.batch + seq]);
    }
}

template <typename ELEM>
__device__ __forceinline__ void store8(uint8_t* dst, const float* x);

template <>
__device__ __forceinline__ void store8<__half>(uint8_t* dst, const float* x) {
    uint4 u;
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __halves2half2(__float2half_rn(x[2 * i]), __float2half_rn(x[2 * i + 1]));
    *reinterpret_cast<uint4*>(dst) = u;
}

template <>
__device__ __forceinline__ void store8<float>(uint8_t* dst, const float* x) {
    reinterpret_cast<float4*>(dst)[0] = make_float4(x[0], x[1], x[2], x[3]);
    reinterpret_cast<float4*>(dst)[1] = make_float4(x[4], x[5], x[6], x[7]);
}

template <typename ELEM>
__global__ void __launch_bounds__(128) append_rope_dense_kernel(const __grid_constant__ AppendParams p) {
    __shared__ float2 cs[kHalfDim];
    const int r = blockIdx.x;
    int layer, seq;
    uint32_t pos;
    append_locate(p, r, layer, seq, pos);
    if (p.apply_rope && threadIdx.x < kHalfDim)
        cs[threadIdx.x] = rope_cos_sin(pos, p.inv_freq.f[threadIdx.x], p.rope_scaling);
    __syncthreads();
    const int slot = static_cast<int>(pos % static_cast<uint32_t>(p.addr.max_seq_len));
    constexpr int kRowBytes = kHeadDim * sizeof(ELEM);
    const int hkv = p.addr.num_kv_heads;
    for (int w = threadIdx.x; w < hkv * 16; w += blockDim.x) {
        const int h = w >> 4, part = w & 15, is_v = part >> 3, i = part & 7;
        const float* src = (is_v ? p.v : p.k) + (static_cast<int64_t>(r) * hkv + h) * kHeadDim;
        const float4 a0 = __ldg(reinterpret_cast<const float4*>(src + 8 * i));
        const float4 a1 = __ldg(reinterpret_cast<const float4*>(src + 8 * i + 4));
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(src + 64 + 8 * i));
        const float4 b1 = __ldg(reinterpret_cast<const float4*>(src + 64 + 8 * i + 4));
        float xa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        float xb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        if (!is_v && p.apply_rope) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                float y0, y1;
                rope_rotate(xa[c], xb[c], cs[8 * i + c], y0, y1);
                xa[c] = y0;
                xb[c] = y1;
            }
        }
        uint8_t* base = is_v ? p.v_base + layer * p.v_layer_stride_bytes : p.k_base + layer * p.k_layer_stride_bytes;
        const int64_t ridx = row_index_for_write(p.addr, seq, h, slot);
        if (ridx < 0) continue;   // no page behind the slot: dropped, the status word says so
        uint8_t* dst = base + ridx * kRowBytes;
        store8<ELEM>(dst + 8 * i * sizeof(ELEM), xa);
        store8<ELEM>(dst + (64 + 8 * i) * sizeof(ELEM), xb);
    }
}

// Generic element scatter (any head_dim, no rotation): one token row [num_kv_heads][head_dim] of raw
// elements into its cache slot.  Backs KVCache.append / appendF16 (KVCache.swift:410-476).
__global__ void scatter_row_kernel(const uint8_t* src, uint8_t* base, KVAddressing addr, int seq, int slot,
                                   int head_dim, int elem_bytes) {
    const int row_bytes = head_dim * elem_bytes;
    const int total = addr.num_kv_heads * row_bytes;
    for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < total; b += gridDim.x * blockDim.x) {
        const int h = b / row_bytes, off = b % row_bytes;
        const int64_t ridx = row_index_for_write(addr, seq, h, slot);
        if (ridx >= 0) base[ridx * row_bytes + off] = src[b];
    }
}

// Generic gather in logical (oldest-first) order for KVCache.retrieve (KVCache.swift:478-522):
// logical token i lives in slot (first_slot + i) % max_seq_len.
__global__ void gather_rows_kernel(const uint8_t* base, uint8_t* dst, KVAddressing addr, int seq, int first_slot,
                                   int tokens, int row_bytes) {
    const int64_t per_token = static_cast<int64_t>(addr.num_kv_heads) * row_bytes;
    const int64_t total = per_token * tokens;
    for (int64_t b = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; b < total;
         b += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int t = static_cast<int>(b / per_token);
        const int rem = static_cast<int>(b % per_token);
        const int h = rem / row_bytes, off = rem % row_bytes;
        const int slot = (first_slot + t) % addr.max_seq_len;
        dst[b] = base[row_index(addr, seq, h, slot) * row_bytes + off];
    }
}

// Rows [0, *len) of (seq, every kv head) of a float16 cache (head-major or paged) as head-major [kv head][slot][128] rows, and zeros
// as their second operand: the form the chunked-prefill kernels read expanded rows in (layers whose two sides use different formats).
struct F16ExpandParams {
    const uint8_t* rows;
    uint8_t* out;
    uint8_t* out_lo;
    KVAddressing addr;
    const int32_t* len_ptr;
    int seq, out_stride_rows;
};

__global__ void __launch_bounds__(256) f16_expand_rows_kernel(const __grid_constant__ F16ExpandParams p) {
    const int lane = threadIdx.x & 31;
    int len = *p.len_ptr;
    len = len < p.addr.max_seq_len ? len : p.addr.max_seq_len;
    const int64_t total = static_cast<int64_t>(len) * p.addr.num_kv_heads;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); row < total; row += static_cast<int64_t>(gridDim.x) * 8) {
        const int h = static_cast<int>(row / len), t = static_cast<int>(row % len);
        const int64_t ridx = row_index(p.addr, p.seq, h, t);
        const int64_t dst = (static_cast<int64_t>(h) * p.out_stride_rows + t) * 256;
        reinterpret_cast<uint2*>(p.out + dst)[lane] = reinterpret_cast<const uint2*>(p.rows + ridx * 256)[lane];
        reinterpret_cast<uint2*>(p.out_lo + dst)[lane] = make_uint2(0u, 0u);
    }
}

// rope_neox_f32 / rope_neox_f32_to_f16 as stand-alone operators (Shaders/RoPE.metal:57-93, 498-531),
// any even head_dim up to 512, partial rotary factor honoured.  inv_freq[pair] =
// 1.0f / powr(theta, float(2*pair)/float(headDim)) is tabulated by the host.
struct WideInvFreqTable {
    float f[256];
};

template <typename OUT>
__global__ void rope_neox_kernel(const float* in, OUT* out, uint32_t seq_len, uint32_t num_heads, uint32_t head_dim,
                                 uint32_t start_pos, float scaling, float partial,
                                 const __grid_constant__ WideInvFreqTable table) {
    const uint32_t half = head_dim / 2;
    const uint64_t total = static_cast<uint64_t>(seq_len) * num_heads * half;
    const uint32_t rotated = static_cast<uint32_t>(static_cast<float>(half) * partial);
    for (uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
         e += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint32_t pair = static_cast<uint32_t>(e % half);
        const uint64_t sh = e / half;
        const uint32_t seq = static_cast<uint32_t>(sh / num_heads);
        const uint64_t hb = sh * head_dim;
        float x0 = in[hb + pair], x1 = in[hb + pair + half];
        if (pair < rotated) {
            const float2 cs = rope_cos_sin(seq + start_pos, table.f[pair], scaling);
            float y0, y1;
            rope_rotate(x0, x1, cs, y0, y1);
            x0 = y0;
            x1 = y1;
        }
        out[hb + pair] = static_cast<OUT>(x0);
        out[hb + pair + half] = static_cast<OUT>(x1);
    }
}

// Host-buffer entry point: pulls this step's q / k / v rows out of pinned (device-mapped) host memory into the
// device staging area with plain 16-byte loads -- one launch instead of three copy-engine transfers.
__global__ void gather_host_inputs_kernel(const float4* q, const float4* k, const float4* v, float4* dq, float4* dk,
                                          float4* dv, int nq4, int nkv4) {
    // the decode kernel that follows is a programmatic dependent launch: let its CTAs be placed and run their
    // shared-memory prologue now (it waits for this grid before it reads the gathered rows)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int total = nq4 + 2 * nkv4;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        if (e < nq4) dq[e] = q[e];
        else if (e < nq4 + nkv4) dk[e - nq4] = k[e - nq4];
        else dv[e - nq4 - nkv4] = v[e - nq4 - nkv4];
    }
}

// After an all-gather of kv-head shards: gathered [world][pairs][local_heads][128] -> full [pairs][world * local_heads][128]
// (pair = (layer, sequence); rank r's heads land at head offset r * local_heads).  16-byte elements.
__global__ void relayout_head_shards_kernel(const float4* __restrict__ gathered, float4* __restrict__ full, uint32_t world,
                                            uint32_t pairs, uint32_t local_heads) {
    constexpr uint32_t kVec = kHeadDim / 4;
    const uint64_t per_rank = static_cast<uint64_t>(pairs) * local_heads * kVec;
    const uint64_t total = per_rank * world;
    for (uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint32_t r = static_cast<uint32_t>(e / per_rank);
        const uint64_t rem = e % per_rank;
        const uint64_t pair = rem / (local_heads * kVec);
        const uint32_t hv = static_cast<uint32_t>(rem % (local_heads * kVec));
        full[(pair * world + r) * local_heads * kVec + hv] = gathered[e];
    }
}

__global__ void add_lengths_kernel(int32_t* lengths, int begin, int count, int delta) {
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < count; e += gridDim.x * blockDim.x)
        lengths[begin + e] += delta;
}

}  // namespace er
