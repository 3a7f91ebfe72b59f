// Cache rows of the TurboQuant presets with high-precision channels and a QJL residual (balanced: 3-bit codes, 32 channels
// 5-bit; aggressive: 2-bit, 32 channels 3-bit) and everything that reads them: append, decode attention, the expansion the
// tensor-core prefill kernel runs on, approximateDecode and the export in the reference's split-buffer format.
//   rows                      TurboQuantEncodedRow, Sources/EdgeRunnerMetal/TurboQuant.swift:1003-1100
//   attention                 gqa_attention_turboquant_decode, Shaders/TurboQuant.metal:1794-2001 (the general form: per
//                             coordinate the mask bit chooses the codebook, the residual term enters when its scale != 0)
//   approximateDecode         TurboQuant.swift:1117-1170
// A cached row is one block of 32-bit words [codes: wpr][outlier mask: 4][residual signs: 4][rowNorm][residualNorm][pad to 16 B]:
// 96 bytes (balanced, wpr 14) or 80 bytes (aggressive, wpr 9) per token and kv head, in the head-major / paged slabs.
// Everything here works in the rotated space with a lane owning coordinates 4L .. 4L + 3 of a row:
//   e[d] = rowNorm * (centroid_{mask[d]}(code[d]) + coef * residualNorm * sign[d]),   coef = sqrt(pi/2) * residual scale
//   score = <fwd(q), eK> * scale ;  out = inverse( sum_t p_t * eV_t ) / sum_t p_t
// (the reference keeps the centroid part and the sign part in two accumulators and transforms both back with the same
// matrix -- its transforms ignore their seeds, TurboQuant.swift:891-921 -- so one accumulator holds their sum).
// Decode attention over these rows runs on the backend's SIMT kernel (simt_decode_kernel below: one token per warp step,
// any row format on either side): correct and bounded by instruction issue, not by HBM.
#pragma once

#include "q8.cuh"
#include "turboquant.cuh"
#include "turboquant_outlier.cuh"

namespace er {

constexpr float kQjlScale = 1.2533141373155001f;   // sqrt(pi / 2), TurboQuantTransform.qjlScale

struct OutlierFormat {
    int rb, hb, high_count;   // regular bits, high-precision bits, number of high-precision channels
    int wpr;                  // code words per row, ceil((128 * rb + high_count * (hb - rb)) / 32)
    int row_words;            // words of a cached row: wpr + 10, rounded up to a multiple of 4
};

__host__ __device__ inline OutlierFormat outlier_format(int rb, int hb, int high_count) {
    OutlierFormat f;
    f.rb = rb; f.hb = hb; f.high_count = high_count;
    f.wpr = (kHeadDim * rb + high_count * (hb - rb) + 31) / 32;
    f.row_words = (f.wpr + 10 + 3) & ~3;
    return f;
}

__device__ __forceinline__ uint32_t tq_extract_bits(const uint32_t* words, int bit_offset, int width) {
    const int w0 = bit_offset >> 5, sh = bit_offset & 31;
    uint32_t v = words[w0] >> sh;
    if (sh + width > 32) v |= words[w0 + 1] << (32 - sh);
    return v & ((1u << width) - 1u);
}

// The lane's four effective coordinates of a cached row (see the header): res_coef = sqrt(pi/2) * residual scale, 0 = centroids only.
__device__ __forceinline__ void tq_outlier_lane_values(const uint32_t* row, const OutlierFormat& f, int lane, float res_coef,
                                                       bool scale_by_norm, float e[4]) {
    const uint32_t* mask = row + f.wpr;
    const uint32_t* signs = mask + 4;
    const int mw = lane >> 3, msh = 4 * (lane & 7);
    uint32_t m[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) m[i] = mask[i];
    int before = 0;   // selected channels below coordinate 4L: the rank of this lane's first high-precision code
#pragma unroll
    for (int i = 0; i < 4; ++i) before += i < mw ? __popc(m[i]) : 0;
    const uint32_t mine = m[mw];
    before += __popc(mine & ((1u << msh) - 1u));
    const uint32_t nib = (mine >> msh) & 15u;
    const uint32_t piece = tq_extract_bits(row, 4 * f.rb * lane, 4 * f.rb);
    const uint32_t sgn = (signs[mw] >> msh) & 15u;
    const float row_norm = reinterpret_cast<const float*>(signs + 4)[0];
    const float res = res_coef != 0.f ? res_coef * reinterpret_cast<const float*>(signs + 4)[1] : 0.f;
    const int side_w = f.hb - f.rb;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint32_t code = (piece >> (f.rb * c)) & ((1u << f.rb) - 1u);
        const bool high = (nib >> c) & 1u;
        if (high) {
            code |= tq_extract_bits(row, kHeadDim * f.rb + before * side_w, side_w) << f.rb;
            ++before;
        }
        float v = tq_centroids_rt(high ? f.hb : f.rb)[code];
        v = fmaf(res, ((sgn >> c) & 1u) ? 1.f : -1.f, v);
        e[c] = scale_by_norm ? v * row_norm : v;
    }
}

// ------------------------------------------------------------------------------------------ append

struct OutlierAppendParams {
    AppendParams base;     // k_base / v_base: the row slabs
    OutlierFormat fmt;
    int k_use_benefit;     // outlier selection rule of the keys / values: 0 = magnitude, 1 = quantisation benefit
    int v_use_benefit;
};

// [NeoX RoPE on K] -> encode -> cached row.  One warp per (source row, kv head, K or V).
__global__ void __launch_bounds__(kOutlierWarps * 32) tq_outlier_append_kernel(const __grid_constant__ OutlierAppendParams op) {
    __shared__ OutlierScratch s_scratch[kOutlierWarps];
    __shared__ __align__(16) uint32_t s_row[kOutlierWarps][32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const AppendParams& p = op.base;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hkv = p.addr.num_kv_heads;
    const int64_t half_jobs = static_cast<int64_t>(p.rows) * hkv;
    for (int64_t job = static_cast<int64_t>(blockIdx.x) * kOutlierWarps + warp; job < 2 * half_jobs;
         job += static_cast<int64_t>(gridDim.x) * kOutlierWarps) {
        const bool is_v = job >= half_jobs;
        const int64_t j = is_v ? job - half_jobs : job;
        const int r = static_cast<int>(j / hkv), h = static_cast<int>(j % hkv);
        const float4 x4 = tq_append_load_row(p, is_v, r, h, lane);
        const float x[4] = {x4.x, x4.y, x4.z, x4.w};
        uint32_t* out = s_row[warp];
        if (lane < op.fmt.row_words) out[lane] = 0u;
        tq_encode_outlier_row(x, lane, s_scratch[warp], op.fmt.rb, op.fmt.hb, op.fmt.high_count, is_v ? op.v_use_benefit : op.k_use_benefit,
                              op.fmt.wpr, out, out + op.fmt.wpr + 4, out + op.fmt.wpr, reinterpret_cast<float*>(out + op.fmt.wpr + 8));
        __syncwarp();
        int layer, seq;
        uint32_t pos;
        append_locate(p, r, layer, seq, pos);
        const int slot = static_cast<int>(pos % static_cast<uint32_t>(p.addr.max_seq_len));
        const int64_t ridx = row_index_for_write(p.addr, seq, h, slot);
        if (ridx >= 0) {   // a slot without a page keeps the row out of the cache (status word set)
            uint8_t* dst = (is_v ? p.v_base + layer * p.v_layer_stride_bytes : p.k_base + layer * p.k_layer_stride_bytes) +
                           ridx * (op.fmt.row_words * 4);
            if (lane < op.fmt.row_words / 4) reinterpret_cast<uint4*>(dst)[lane] = reinterpret_cast<const uint4*>(out)[lane];
        }
        __syncwarp();
    }
}

// ------------------------------------------------------------------------------------------ decode attention (SIMT, any row format)

// Where the K rows or the V rows of an attention call come from: any row format of the backend, read with a lane owning
// coordinates 4L .. 4L + 3.  The two sides of a call are independent -- they may differ in format and even lie in
// different caches (layers whose keys and values use different cache types: gqa_attention_q8k_turboquant(_decode),
// gqa_attention_turboquant_decode_f16v, Shaders/TurboQuant.metal:1651-2399).
enum RowFormat : int { kRowsF16 = 0, kRowsQ8 = 1, kRowsTurbo = 2, kRowsOutlier = 3 };

struct RowSource {
    int format;                 // RowFormat
    const uint8_t* rows;        // first row of layer 0
    const uint8_t* side;        // q8_0: four fp16 scales per row; TurboQuant fixed presets: one norm per row
    int64_t layer_stride_bytes, side_layer_stride_bytes;
    int bits;                   // kRowsTurbo: code width
    int norm_fp16;              // kRowsTurbo: the stored norm is fp16
    OutlierFormat ofmt;         // kRowsOutlier
    float res_coef;             // kRowsOutlier: sqrt(pi/2) * residual scale
    KVAddressing addr;
};

// A row on its way through a warp: the raw words a lane fetched (issued early, used one token later).
struct RowRegs {
    uint32_t w0, w1;   // fp16: the lane's 8 bytes; q8_0: its int8 word; TurboQuant: word `lane` of the row (coalesced), shared by shuffles
    float side;        // q8_0: the block's scale; TurboQuant fixed presets: the row's norm
};

// Issues the loads of row `slot` of (layer, seq, kv head); nothing here depends on loaded data except the block-table entry.
__device__ __forceinline__ RowRegs load_row(const RowSource& s, int layer, int seq, int head, int slot, int lane) {
    RowRegs r;
    r.w0 = r.w1 = 0u;
    r.side = 0.f;
    const int64_t ridx = row_index(s.addr, seq, head, slot);
    const uint8_t* rows = s.rows + static_cast<int64_t>(layer) * s.layer_stride_bytes;
    if (s.format == kRowsF16) {
        const uint2 w = *reinterpret_cast<const uint2*>(rows + ridx * kRowBytesF16 + 8 * lane);
        r.w0 = w.x; r.w1 = w.y;
    } else if (s.format == kRowsQ8) {
        r.w0 = reinterpret_cast<const uint32_t*>(rows + ridx * kQ8RowBytes)[q8_word_slot(lane)];
        const uint8_t* side = s.side + static_cast<int64_t>(layer) * s.side_layer_stride_bytes;
        r.side = __half2float(reinterpret_cast<const __half*>(side + ridx * kQ8ScaleBytes)[lane >> 3]);
    } else if (s.format == kRowsTurbo) {
        const int words = (kHeadDim * s.bits + 31) / 32;
        if (lane < words) r.w0 = reinterpret_cast<const uint32_t*>(rows + ridx * (words * 4))[lane];
        const uint8_t* side = s.side + static_cast<int64_t>(layer) * s.side_layer_stride_bytes;
        r.side = s.norm_fp16 ? __half2float(reinterpret_cast<const __half*>(side)[ridx]) : reinterpret_cast<const float*>(side)[ridx];
    } else {
        if (lane < s.ofmt.row_words) r.w0 = reinterpret_cast<const uint32_t*>(rows + ridx * (s.ofmt.row_words * 4))[lane];
    }
    return r;
}

// `width` bits at bit `offset` of a row whose word i sits in lane i's `w` (all lanes call; offset may differ per lane).
__device__ __forceinline__ uint32_t warp_row_bits(uint32_t w, int offset, int width) {
    const int w0 = offset >> 5, sh = offset & 31;
    const uint32_t lo = __shfl_sync(0xffffffffu, w, w0), hi = __shfl_sync(0xffffffffu, w, (w0 + 1) & 31);
    const uint32_t v = sh == 0 ? lo : ((lo >> sh) | (hi << (32 - sh)));
    return v & ((1u << width) - 1u);
}

// The lane's four coordinates of the row, scaled by the row's norm / block scale.  All 32 lanes call (shuffles inside).
// `tables`: the four codebooks in shared memory, [bits - 2][code] (divergent indices serialise on the constant cache).
__device__ __forceinline__ void decode_row_lane4(const RowSource& s, const RowRegs& r, int lane, const float (*tables)[32], float e[4]) {
    if (s.format == kRowsF16) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.w0)), b = __half22float2(*reinterpret_cast<const __half2*>(&r.w1));
        e[0] = a.x; e[1] = a.y; e[2] = b.x; e[3] = b.y;
    } else if (s.format == kRowsQ8) {
#pragma unroll
        for (int c = 0; c < 4; ++c) e[c] = r.side * static_cast<float>(static_cast<int8_t>((r.w0 >> (8 * c)) & 0xFF));
    } else if (s.format == kRowsTurbo) {
        const uint32_t piece = warp_row_bits(r.w0, 4 * s.bits * lane, 4 * s.bits);
        const float* cent = tables[s.bits - 2];
#pragma unroll
        for (int c = 0; c < 4; ++c) e[c] = r.side * cent[(piece >> (s.bits * c)) & ((1u << s.bits) - 1u)];
    } else {
        // [codes: wpr][mask 4][signs 4][rowNorm][residualNorm]: the same arithmetic as tq_outlier_lane_values on shuffled words
        const OutlierFormat& f = s.ofmt;
        const int mw = lane >> 3, msh = 4 * (lane & 7);
        int before = 0;
        uint32_t mine = 0u;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t mi = __shfl_sync(0xffffffffu, r.w0, f.wpr + i);
            before += i < mw ? __popc(mi) : 0;
            mine = i == mw ? mi : mine;
        }
        before += __popc(mine & ((1u << msh) - 1u));
        const uint32_t nib = (mine >> msh) & 15u;
        const uint32_t sgn = (__shfl_sync(0xffffffffu, r.w0, f.wpr + 4 + mw) >> msh) & 15u;
        const float row_norm = __uint_as_float(__shfl_sync(0xffffffffu, r.w0, f.wpr + 8));
        const float res_norm = __uint_as_float(__shfl_sync(0xffffffffu, r.w0, f.wpr + 9));
        const float res = s.res_coef != 0.f ? s.res_coef * res_norm : 0.f;
        const uint32_t piece = warp_row_bits(r.w0, 4 * f.rb * lane, 4 * f.rb);
        const int side_w = f.hb - f.rb;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const bool high = (nib >> c) & 1u;
            // every lane takes part in the shuffles; a lane without a high-precision code here reads (and drops) the bits at its rank
            const uint32_t hi_bits = warp_row_bits(r.w0, kHeadDim * f.rb + (before < f.high_count ? before : 0) * side_w, side_w);
            uint32_t code = (piece >> (f.rb * c)) & ((1u << f.rb) - 1u);
            if (high) { code |= hi_bits << f.rb; ++before; }
            float v = tables[(high ? f.hb : f.rb) - 2][code];
            v = fmaf(res, ((sgn >> c) & 1u) ? 1.f : -1.f, v);
            e[c] = v * row_norm;
        }
    }
}

__host__ __device__ inline bool rows_are_rotated(int format) { return format == kRowsTurbo || format == kRowsOutlier; }

struct SimtDecodeParams {
    const float* q;               // [pairs][rows_per_pair][num_q_heads][128]
    RowSource k, v;
    const int32_t* lengths;       // tokens written, [layers][batch] of the KEY side's cache
    int layer_begin, batch, num_q_heads, pending, splits;
    int fixed_seq;                // >= 0: every problem is this sequence and pair = layer offset (chunks of one sequence)
    // rows_per_pair > 1: a chunk of query rows per (layer, sequence); row r sees keys [0, kv_len - (rows_per_pair - 1 - r))
    // and sits at position q_pos0 + r (q_pos0 < 0: the chunk's last row is the newest token)
    int rows_per_pair, q_pos0;
    int window;                   // > 0: a query row sees only the newest `window` of its visible rows (sliding-window layers)
    float scale_log2, rope_scaling;
    int apply_rope;
    InvFreqTable inv_freq;
    float* partial;               // [pairs * rows * kv heads][splits][group][132]: max (log2 domain), sum, pad, pad, acc[128]
    float* out;                   // [pairs][rows][out_heads][128]
    int out_heads_total, out_head_offset;
};

constexpr int kSimtDecodeWarps = 8;
constexpr int kSimtPartialStride = 132;

// grid (splits, kv heads, (layer, sequence) pairs x query rows); every warp walks tokens split_begin + warp, + 8, ...
// Scores live in the keys' space (rotated for TurboQuant keys: the query is transformed once), outputs in the values' space
// (one inverse transform at the end for TurboQuant values).
// the per-token chain of shuffles and lookups is latency-bound: resident warps are what hides it
template <int GROUP>
__global__ void __launch_bounds__(kSimtDecodeWarps * 32, GROUP <= 2 ? 4 : (GROUP == 4 ? 2 : 1)) simt_decode_kernel(const __grid_constant__ SimtDecodeParams p) {
    __shared__ __align__(16) float s_q[GROUP][kHeadDim];
    __shared__ float s_ml[kSimtDecodeWarps][GROUP][2];
    __shared__ __align__(16) float s_acc[kSimtDecodeWarps][GROUP][kHeadDim];
    __shared__ float s_cent[4][32];
    if (threadIdx.x < 128) {
        const int bits = 2 + (threadIdx.x >> 5), code = threadIdx.x & 31;
        s_cent[bits - 2][code] = code < (1 << bits) ? tq_centroids_rt(bits)[code] : 0.f;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x, head = blockIdx.y;
    const int problem = blockIdx.z, pair = problem / p.rows_per_pair, qrow = problem % p.rows_per_pair;
    const int hkv = p.k.addr.num_kv_heads;
    const int layer = p.fixed_seq >= 0 ? p.layer_begin + pair : p.layer_begin + pair / p.batch;
    const int seq = p.fixed_seq >= 0 ? p.fixed_seq : pair % p.batch;
    const int written = p.lengths[layer * p.batch + seq] + p.pending;
    const int cap = p.k.addr.max_seq_len;
    const int visible = written - (p.rows_per_pair - 1 - qrow);
    const int kv_len = visible < 0 ? 0 : (visible < cap ? visible : cap);
    const uint32_t q_pos = static_cast<uint32_t>(p.q_pos0 >= 0 ? p.q_pos0 + qrow : (visible > 0 ? visible - 1 : 0));
    // ---- the group's query rows: [NeoX RoPE ->] [randomizedHadamard ->] scaled for exp2 ----
    for (int g = warp; g < GROUP; g += kSimtDecodeWarps) {
        const float4 x = *reinterpret_cast<const float4*>(p.q + (static_cast<int64_t>(problem) * p.num_q_heads + head * GROUP + g) * kHeadDim + 4 * lane);
        float a[4] = {x.x, x.y, x.z, x.w};
        if (p.apply_rope) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float other = __shfl_xor_sync(0xffffffffu, a[c], 16);
                const float2 cs = rope_cos_sin_fast(q_pos, p.inv_freq.f[(4 * lane + c) & 63], p.rope_scaling);
                float y0, y1;
                if (lane < 16) { rope_rotate(a[c], other, cs, y0, y1); a[c] = y0; }
                else           { rope_rotate(other, a[c], cs, y0, y1); a[c] = y1; }
            }
        }
        if (rows_are_rotated(p.k.format)) warp_tq_forward(a, lane);
        *reinterpret_cast<float4*>(&s_q[g][4 * lane]) = make_float4(a[0] * p.scale_log2, a[1] * p.scale_log2, a[2] * p.scale_log2, a[3] * p.scale_log2);
    }
    __syncthreads();
    float qr[GROUP][4];
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
        const float4 t = *reinterpret_cast<const float4*>(&s_q[g][4 * lane]);
        qr[g][0] = t.x; qr[g][1] = t.y; qr[g][2] = t.z; qr[g][3] = t.w;
    }
    // the rows visited: logical positions [visible - count, visible), i.e. ring slots position % capacity
    const int count = p.window > 0 && p.window < kv_len ? p.window : kv_len;
    const int first_pos = (visible > 0 ? visible : 0) - count;
    const int per = (count + p.splits - 1) / p.splits;
    const int t_begin = split * per, t_end = min(count, t_begin + per);
    float m[GROUP], l[GROUP], acc[GROUP][4];
#pragma unroll
    for (int g = 0; g < GROUP; ++g) { m[g] = -INFINITY; l[g] = 0.f; acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f; }
    // the next token's words are on their way while this token is decoded and used
    RowRegs nk{}, nv{};
    if (t_begin + warp < t_end) {
        const int t = (first_pos + t_begin + warp) % cap;
        nk = load_row(p.k, layer, seq, head, t, lane);
        nv = load_row(p.v, layer, seq, head, t, lane);
    }
    for (int i = t_begin + warp; i < t_end; i += kSimtDecodeWarps) {
        const RowRegs ck = nk, cv = nv;
        if (i + kSimtDecodeWarps < t_end) {
            const int t = (first_pos + i + kSimtDecodeWarps) % cap;
            nk = load_row(p.k, layer, seq, head, t, lane);
            nv = load_row(p.v, layer, seq, head, t, lane);
        }
        float ek[4], ev[4];
        decode_row_lane4(p.k, ck, lane, s_cent, ek);
        decode_row_lane4(p.v, cv, lane, s_cent, ev);
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
            float s = fmaf(qr[g][3], ek[3], fmaf(qr[g][2], ek[2], fmaf(qr[g][1], ek[1], qr[g][0] * ek[0])));
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            const float mn = fmaxf(m[g], s);
            const float corr = fast_exp2(m[g] - mn), pr = fast_exp2(s - mn);   // ex2(-inf) = 0 on the first token
            l[g] = fmaf(l[g], corr, pr);
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[g][c] = fmaf(acc[g][c], corr, pr * ev[c]);
            m[g] = mn;
        }
    }
    // ---- merge the warps of this CTA, write the split's partial ----
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
        if (lane == 0) { s_ml[warp][g][0] = m[g]; s_ml[warp][g][1] = l[g]; }
        *reinterpret_cast<float4*>(&s_acc[warp][g][4 * lane]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
    }
    __syncthreads();
    const int item = problem * hkv + head;
    for (int idx = threadIdx.x; idx < GROUP * kHeadDim; idx += kSimtDecodeWarps * 32) {
        const int g = idx >> 7, d = idx & 127;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kSimtDecodeWarps; ++w) M = fmaxf(M, s_ml[w][g][0]);
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < kSimtDecodeWarps; ++w) {
            const float wgt = s_ml[w][g][0] == -INFINITY ? 0.f : exp2f(s_ml[w][g][0] - M);
            L = fmaf(s_ml[w][g][1], wgt, L);
            A = fmaf(s_acc[w][g][d], wgt, A);
        }
        float* dst = p.partial + ((static_cast<int64_t>(item) * p.splits + split) * GROUP + g) * kSimtPartialStride;
        if (d == 0) { dst[0] = M; dst[1] = L; }
        dst[4 + d] = A;
    }
}

// One warp per (item, head of the group): combine the splits, transform back, normalise, store.
template <int GROUP>
__global__ void simt_decode_merge_kernel(const __grid_constant__ SimtDecodeParams p, int items) {
    const int lane = threadIdx.x & 31;
    const int64_t job = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (job >= static_cast<int64_t>(items) * GROUP) return;
    const int item = static_cast<int>(job / GROUP), g = static_cast<int>(job % GROUP);
    const int hkv = p.k.addr.num_kv_heads;
    const int problem = item / hkv, head = item % hkv;
    const float* base = p.partial + (static_cast<int64_t>(item) * p.splits * GROUP + g) * kSimtPartialStride;
    float M = -INFINITY;
    for (int s = 0; s < p.splits; ++s) M = fmaxf(M, base[static_cast<int64_t>(s) * GROUP * kSimtPartialStride]);
    float L = 0.f, a[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < p.splits; ++s) {
        const float* ps = base + static_cast<int64_t>(s) * GROUP * kSimtPartialStride;
        const float wgt = ps[0] == -INFINITY ? 0.f : exp2f(ps[0] - M);
        L = fmaf(ps[1], wgt, L);
        const float4 v = *reinterpret_cast<const float4*>(ps + 4 + 4 * lane);
        a[0] = fmaf(v.x, wgt, a[0]); a[1] = fmaf(v.y, wgt, a[1]); a[2] = fmaf(v.z, wgt, a[2]); a[3] = fmaf(v.w, wgt, a[3]);
    }
    if (rows_are_rotated(p.v.format)) warp_tq_inverse(a, lane);
    const float inv = L > 0.f ? 1.f / L : 0.f;   // a sequence without rows: zeros (invSum = 0 rule)
    const int out_heads = p.out_heads_total > 0 ? p.out_heads_total : p.num_q_heads;
    float* dst = p.out + (static_cast<int64_t>(problem) * out_heads + p.out_head_offset + head * GROUP + g) * kHeadDim;
    *reinterpret_cast<float4*>(dst + 4 * lane) = make_float4(a[0] * inv, a[1] * inv, a[2] * inv, a[3] * inv);
}

inline int launch_simt_decode(int group, const SimtDecodeParams& p, int pairs, cudaStream_t stream) {
    const int problems = pairs * p.rows_per_pair;
    const dim3 grid(static_cast<unsigned>(p.splits), static_cast<unsigned>(p.k.addr.num_kv_heads), static_cast<unsigned>(problems));
    const int items = problems * p.k.addr.num_kv_heads;
    const int merge_blocks = (items * group + 7) / 8;
    switch (group) {
#define ER_SIMT_CASE(G)                                                                   \
    case G:                                                                               \
        simt_decode_kernel<G><<<grid, kSimtDecodeWarps * 32, 0, stream>>>(p);          \
        simt_decode_merge_kernel<G><<<merge_blocks, 256, 0, stream>>>(p, items);          \
        break;
        ER_SIMT_CASE(1) ER_SIMT_CASE(2) ER_SIMT_CASE(4) ER_SIMT_CASE(8)
#undef ER_SIMT_CASE
        default: return kNotBuilt;
    }
    return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------ expansion, decode, export

// Rows [0, *len) of (seq, every kv head) as fp16 hi + lo of the effective coordinates, head-major [kv head][slot][128]: what
// the tensor-core prefill kernel reads (gqa_attention_turboquant, Shaders/TurboQuant.metal:1454-1649, in the rotated space).
struct OutlierExpandParams {
    const uint8_t* rows;
    __half* out;
    __half* out_lo;
    OutlierFormat fmt;
    KVAddressing addr;
    const int32_t* len_ptr;
    int seq, out_stride_rows;
    float res_coef;
};

__global__ void tq_outlier_expand_rows_kernel(const __grid_constant__ OutlierExpandParams p) {
    const int lane = threadIdx.x & 31;
    int len = *p.len_ptr;
    len = len < p.addr.max_seq_len ? len : p.addr.max_seq_len;
    const int64_t total = static_cast<int64_t>(len) * p.addr.num_kv_heads;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < total;
         row += static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5)) {
        const int h = static_cast<int>(row / len), t = static_cast<int>(row % len);
        const int64_t ridx = row_index(p.addr, p.seq, h, t);
        float a[4];
        tq_outlier_lane_values(reinterpret_cast<const uint32_t*>(p.rows + ridx * (p.fmt.row_words * 4)), p.fmt, lane, p.res_coef, true, a);
        uint2 o;
        const __half2 h01 = __floats2half2_rn(a[0], a[1]), h23 = __floats2half2_rn(a[2], a[3]);
        reinterpret_cast<__half2*>(&o)[0] = h01;
        reinterpret_cast<__half2*>(&o)[1] = h23;
        reinterpret_cast<uint2*>(p.out + (static_cast<int64_t>(h) * p.out_stride_rows + t) * kHeadDim)[lane] = o;
        const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
        reinterpret_cast<__half2*>(&o)[0] = __floats2half2_rn(a[0] - f01.x, a[1] - f01.y);
        reinterpret_cast<__half2*>(&o)[1] = __floats2half2_rn(a[2] - f23.x, a[3] - f23.y);
        reinterpret_cast<uint2*>(p.out_lo + (static_cast<int64_t>(h) * p.out_stride_rows + t) * kHeadDim)[lane] = o;
    }
}

// approximateDecode (TurboQuant.swift:1117-1170), rows in logical order [tokens][kv heads][128]:
//   x = (inverse(centroids) + inverse(+-1 signs) * (sqrt(pi/2) / 128 * residualNorm * residualWeight)) * rowNorm
struct OutlierDecodeRowsParams {
    const uint8_t* rows;
    float* out;
    OutlierFormat fmt;
    KVAddressing addr;
    int seq, first_slot, tokens;
    float residual_weight;
};

__global__ void tq_outlier_decode_rows_kernel(const __grid_constant__ OutlierDecodeRowsParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t total = static_cast<int64_t>(p.tokens) * p.addr.num_kv_heads;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < total;
         row += static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5)) {
        const int t = static_cast<int>(row / p.addr.num_kv_heads), h = static_cast<int>(row % p.addr.num_kv_heads);
        const int slot = (p.first_slot + t) % p.addr.max_seq_len;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(p.rows + row_index(p.addr, p.seq, h, slot) * (p.fmt.row_words * 4));
        float a[4], s[4];
        tq_outlier_lane_values(src, p.fmt, lane, 0.f, false, a);
        const uint32_t sgn = (src[p.fmt.wpr + 4 + (lane >> 3)] >> (4 * (lane & 7))) & 15u;
#pragma unroll
        for (int c = 0; c < 4; ++c) s[c] = ((sgn >> c) & 1u) ? 1.f : -1.f;
        warp_tq_inverse(a, lane);
        warp_tq_inverse(s, lane);
        const float row_norm = reinterpret_cast<const float*>(src + p.fmt.wpr + 8)[0];
        const float res_norm = reinterpret_cast<const float*>(src + p.fmt.wpr + 8)[1];
        // qjl * qjlScale * (1 / 128) * residualNorm * residualWeight, multiplied left to right as the reference writes it
        float o[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float qj = __fmul_rn(__fmul_rn(__fmul_rn(__fmul_rn(s[c], kQjlScale), 1.0f / 128.0f), res_norm), p.residual_weight);
            o[c] = __fmul_rn(__fadd_rn(a[c], qj), row_norm);
        }
        *reinterpret_cast<float4*>(p.out + row * kHeadDim + 4 * lane) = make_float4(o[0], o[1], o[2], o[3]);
    }
}

// The reference's four split buffers (retrieveTurboQuantRuntimeRows, KVCache.swift:588-629), rows in logical order.
struct OutlierExportParams {
    const uint8_t* rows;
    uint32_t* codes;     // [tokens * kv heads][wpr]
    uint32_t* signs;     // [..][4]
    uint32_t* mask;      // [..][4]
    float* meta;         // [..][2]
    OutlierFormat fmt;
    KVAddressing addr;
    int seq, first_slot, tokens;
};

__global__ void tq_outlier_export_rows_kernel(const __grid_constant__ OutlierExportParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t total = static_cast<int64_t>(p.tokens) * p.addr.num_kv_heads;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < total;
         row += static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5)) {
        const int t = static_cast<int>(row / p.addr.num_kv_heads), h = static_cast<int>(row % p.addr.num_kv_heads);
        const int slot = (p.first_slot + t) % p.addr.max_seq_len;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(p.rows + row_index(p.addr, p.seq, h, slot) * (p.fmt.row_words * 4));
        if (lane < p.fmt.wpr) p.codes[row * p.fmt.wpr + lane] = src[lane];
        if (lane < 4) { p.mask[row * 4 + lane] = src[p.fmt.wpr + lane]; p.signs[row * 4 + lane] = src[p.fmt.wpr + 4 + lane]; }
        if (lane < 2) p.meta[row * 2 + lane] = reinterpret_cast<const float*>(src + p.fmt.wpr + 8)[lane];
    }
}

}  // namespace er
