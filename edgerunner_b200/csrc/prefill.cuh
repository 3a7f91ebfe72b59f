// Chunked-prefill GQA attention over an fp16 KV cache on the tensor cores.
//
// Replaces the seqLen > 1 uses of gqa_attention_f16kv (Shaders/GQA.metal:278-387) and
// flash_attention_gqa_simd_qf32_kvf16 (Shaders/FlashAttention.metal:194-264): query row r (absolute position
// r + qOffset) attends to keys 0 .. r + qOffset (causal rule of GQA.metal:345), online softmax, fp32 accumulation.
// The reference runs this as scalar FMAs (no matrix units); here the two contractions run on mma.sync m16n8k16
// (fp16 operands, fp32 accumulators):
//   * a CTA owns 64 "M rows" of one kv head: (64 / GROUP) consecutive query rows x the GROUP query heads that share
//     the kv head, so every K/V tile fetched from HBM feeds all of them; warp w owns M rows [16w, 16w+16);
//   * Q (fp32) is pre-multiplied by scale*log2(e) and split into fp16 hi + lo parts, so the QK^T product keeps
//     ~22 mantissa bits of Q at the price of a second MMA per tile (K is fp16 in the cache, i.e. exact);
//   * K/V tiles of 64 tokens are staged with 16-byte cp.async into XOR-swizzled shared memory (double buffered) and
//     read back with ldmatrix (K) / ldmatrix.trans (V);
//   * P is split into fp16 hi + lo parts as well (V is fp16 in the cache), so both products are exact to ~2^-22.
#pragma once

#include "er_common.cuh"

namespace er {

constexpr int kPfTileTokens = 64;
constexpr int kPfRows = 64;                      // M rows per CTA
constexpr int kPfThreads = 128;
constexpr int kPfTileBytes = kPfTileTokens * kHeadDim * 2;   // 16 KiB per K or V tile
constexpr int kPfSmemBytes = 4 * kPfTileBytes;               // K,V x 2 stages
constexpr int kPfSmemBytesSplit = 8 * kPfTileBytes;          // K hi, V hi, K lo, V lo x 2 stages

struct PrefillParams {
    const float* q;          // [seq_len][num_q_heads][128]
    float* out;              // same shape
    const uint8_t* k_layer;  // first row of the layer
    const uint8_t* v_layer;
    const uint8_t* k_lo_layer;   // KSPLIT kernels: second fp16 operand of K (rows = k - fp16(k) of an fp32 source), same addressing
    const uint8_t* v_lo_layer;   // ... and of V (set together with k_lo_layer)
    KVAddressing addr;
    int seq;                 // sequence index inside the cache
    int seq_len;             // query rows
    int kv_len;              // rows present in the cache (used when kv_len_ptr is null)
    const int32_t* kv_len_ptr;   // device: tokens written to (layer, seq); clamped to addr.max_seq_len
    int q_offset_from_end;   // 1: q_offset = kv_len - seq_len (the query rows are the newest rows of the cache)
    int q_offset;            // absolute position of query row 0
    int causal;
    int window;              // > 0: query row at position P also ignores keys before P - window + 1 (sliding-window layers;
                             // Gemma4GPUKVCache.attentionRange)
    int num_q_heads;
    float scale_log2;
    float rope_scaling;
    int apply_rope;          // NeoX-rotate Q at position q_offset + row
    InvFreqTable inv_freq;
    // tcgen05 kernel only: CTA tiles (query tile x kv head) with linear index >= split_from are each run by split_parts CTAs
    // that share the tile's key range and leave (max, sum, unnormalised row) partials in split_partial
    // [tile - split_from][part][128 rows][132]; a merge launch combines them.  The launcher fills these in (the tail of the grid
    // that would occupy only part of the SMs is cut along the keys); split_partial == nullptr turns it off.
    float* split_partial;
    size_t split_partial_floats;
    int split_from, split_parts;
};

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}

__device__ __forceinline__ void cp_async_16(uint32_t smem_addr, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;   // zero-fill rows past the cache length
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Byte offset of 16-byte chunk `chunk` (0..15) of row `row` inside a swizzled [64][256 B] tile.
__device__ __forceinline__ uint32_t pf_swizzle(int row, int chunk) {
    return static_cast<uint32_t>(row * 256 + (((chunk & 8) | ((chunk ^ row) & 7)) << 4));
}

// KSPLIT: K and V are each the sum of two fp16 tensors (k_layer + k_lo_layer, v_layer + v_lo_layer), as produced from
// fp32 rows that must not lose their low mantissa bits (TurboQuant norm * centroid, q8_0 scale * code); one more mma per
// fragment on either side (qh.kh + ql.kh + qh.kl;  ph.vh + pl.vh + ph.vl).
template <int GROUP, bool KSPLIT = false>
__global__ void __launch_bounds__(kPfThreads) prefill_f16_kernel(const __grid_constant__ PrefillParams p) {
    constexpr int kStageTiles = KSPLIT ? 4 : 2;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = lane >> 2, qlane = lane & 3;
    constexpr int kQRowsPerCta = kPfRows / GROUP;
    const int kv_head = blockIdx.y;
    const int q0 = blockIdx.x * kQRowsPerCta;            // first query row of this CTA
    const uint32_t smem_base = smem_u32(smem);
    PrefillParams pp = p;   // resolve device-side lengths
    if (p.kv_len_ptr != nullptr) {
        const int n = *p.kv_len_ptr;
        pp.kv_len = n < p.addr.max_seq_len ? n : p.addr.max_seq_len;
    }
    if (p.q_offset_from_end) pp.q_offset = pp.kv_len - p.seq_len;

    // M row m (0..63) -> query row q0 + m / GROUP, query head kv_head*GROUP + m % GROUP
    const int m_lo = warp * 16 + quad, m_hi = m_lo + 8;
    const int qi_lo = q0 + m_lo / GROUP, qi_hi = q0 + m_hi / GROUP;
    const int head_lo = kv_head * GROUP + m_lo % GROUP, head_hi = kv_head * GROUP + m_hi % GROUP;
    const bool row_lo_ok = qi_lo < p.seq_len, row_hi_ok = qi_hi < p.seq_len;

    // ---- Q fragments: fp32 -> [RoPE] -> * scale*log2e -> fp16 hi + lo ----
    uint32_t qh[8][4], ql[8][4];
    {
        const float* row_lo = p.q + (static_cast<int64_t>(row_lo_ok ? qi_lo : 0) * p.num_q_heads + head_lo) * kHeadDim;
        const float* row_hi = p.q + (static_cast<int64_t>(row_hi_ok ? qi_hi : 0) * p.num_q_heads + head_hi) * kHeadDim;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {          // k-steps kk and kk+4 hold the RoPE partners (d, d+64)
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const float* src = hrow ? row_hi : row_lo;
                const bool ok = hrow ? row_hi_ok : row_lo_ok;
                const uint32_t pos = static_cast<uint32_t>(pp.q_offset + (hrow ? qi_hi : qi_lo));
#pragma unroll
                for (int part = 0; part < 2; ++part) {   // cols 2*qlane (+8)
                    const int d = 16 * kk + 8 * part + 2 * qlane;
                    float2 a = ok ? *reinterpret_cast<const float2*>(src + d) : make_float2(0.f, 0.f);
                    float2 b = ok ? *reinterpret_cast<const float2*>(src + d + 64) : make_float2(0.f, 0.f);
                    if (p.apply_rope) {
                        const float2 c0 = rope_cos_sin_fast(pos, p.inv_freq.f[d], p.rope_scaling);
                        const float2 c1 = rope_cos_sin_fast(pos, p.inv_freq.f[d + 1], p.rope_scaling);
                        float y0, y1;
                        rope_rotate(a.x, b.x, c0, y0, y1); a.x = y0; b.x = y1;
                        rope_rotate(a.y, b.y, c1, y0, y1); a.y = y0; b.y = y1;
                    }
                    a.x *= p.scale_log2; a.y *= p.scale_log2; b.x *= p.scale_log2; b.y *= p.scale_log2;
                    const uint32_t ah = pack_half2(a.x, a.y), bh = pack_half2(b.x, b.y);
                    const float2 ahf = __half22float2(*reinterpret_cast<const __half2*>(&ah));
                    const float2 bhf = __half22float2(*reinterpret_cast<const __half2*>(&bh));
                    const int reg = hrow + 2 * part;    // a0: (row, cols) a1: (row+8, cols) a2: (row, cols+8) a3: (row+8, cols+8)
                    qh[kk][reg] = ah;
                    ql[kk][reg] = pack_half2(a.x - ahf.x, a.y - ahf.y);
                    qh[kk + 4][reg] = bh;
                    ql[kk + 4][reg] = pack_half2(b.x - bhf.x, b.y - bhf.y);
                }
            }
        }
    }

    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[j][c] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    // keys visible to this CTA: up to its last query row
    const int q_last = min(q0 + kQRowsPerCta, p.seq_len) - 1;
    const int kv_hi = p.causal ? min(pp.kv_len, q_last + pp.q_offset + 1) : pp.kv_len;
    const int num_tiles = (kv_hi + kPfTileTokens - 1) / kPfTileTokens;
    // a sliding window hides every tile that ends before the first query row's window begins
    const int tile_lo = p.window > 0 ? max(0, q0 + pp.q_offset - p.window + 1) / kPfTileTokens : 0;

    auto load_tile = [&](int tile, int stage) {
        const int t0 = tile * kPfTileTokens;
        const uint32_t ks = smem_base + stage * kStageTiles * kPfTileBytes, vs = ks + kPfTileBytes, kls = vs + kPfTileBytes, vls = kls + kPfTileBytes;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = tid + i * kPfThreads;       // 1024 chunks of 16 bytes per tensor
            const int row = c >> 4, chunk = c & 15;
            const int t = t0 + row;
            const bool ok = t < pp.kv_len;
            const int64_t ridx = row_index(p.addr, p.seq, kv_head, ok ? t : 0);
            cp_async_16(ks + pf_swizzle(row, chunk), p.k_layer + ridx * 256 + chunk * 16, ok);
            cp_async_16(vs + pf_swizzle(row, chunk), p.v_layer + ridx * 256 + chunk * 16, ok);
            if (KSPLIT) {
                cp_async_16(kls + pf_swizzle(row, chunk), p.k_lo_layer + ridx * 256 + chunk * 16, ok);
                cp_async_16(vls + pf_swizzle(row, chunk), p.v_lo_layer + ridx * 256 + chunk * 16, ok);
            }
        }
        cp_async_commit();
    };

    if (num_tiles > tile_lo) load_tile(tile_lo, 0);
    for (int tile = tile_lo; tile < num_tiles; ++tile) {
        const int stage = (tile - tile_lo) & 1;
        if (tile + 1 < num_tiles) { load_tile(tile + 1, stage ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
        const uint32_t ks = smem_base + stage * kStageTiles * kPfTileBytes, vs = ks + kPfTileBytes, kls = vs + kPfTileBytes, vls = kls + kPfTileBytes;
        const int t0 = tile * kPfTileTokens;

        // ---- S = Q K^T (log2 domain) ----
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int c = 0; c < 4; ++c) s[j][c] = 0.f;
#pragma unroll
            for (int kk2 = 0; kk2 < 4; ++kk2) {       // two k-steps per ldmatrix.x4
                uint32_t b[4];
                const int row = 8 * j + (lane & 7), chunk = 4 * kk2 + (lane >> 3);
                ldmatrix_x4(b, ks + pf_swizzle(row, chunk));
                mma_16816(s[j], qh[2 * kk2], b[0], b[1]);
                mma_16816(s[j], ql[2 * kk2], b[0], b[1]);
                mma_16816(s[j], qh[2 * kk2 + 1], b[2], b[3]);
                mma_16816(s[j], ql[2 * kk2 + 1], b[2], b[3]);
                if (KSPLIT) {
                    ldmatrix_x4(b, kls + pf_swizzle(row, chunk));
                    mma_16816(s[j], qh[2 * kk2], b[0], b[1]);
                    mma_16816(s[j], qh[2 * kk2 + 1], b[2], b[3]);
                }
            }
        }
        // ---- mask + online softmax ----
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int t = t0 + 8 * j + 2 * qlane + (c & 1);
                const int hrow = c >> 1;
                const int qi = hrow ? qi_hi : qi_lo;
                const bool vis = t < pp.kv_len && (!p.causal || t <= qi + pp.q_offset) &&
                                 (p.window <= 0 || t > qi + pp.q_offset - p.window);
                s[j][c] = vis ? s[j][c] : -INFINITY;
                mx[hrow] = fmaxf(mx[hrow], s[j][c]);
            }
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            corr[h] = (m_new == -INFINITY) ? 1.f : fast_exp2(m_run[h] - m_new);
            m_run[h] = m_new;
        }
        float psum[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int h = c >> 1;
                s[j][c] = (m_run[h] == -INFINITY) ? 0.f : fast_exp2(s[j][c] - m_run[h]);   // s now holds P
                psum[h] += s[j][c];
            }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 1);
            psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 2);
            l_run[h] = fmaf(l_run[h], corr[h], psum[h]);
        }
        // The tensor cores add into their fp32 accumulators with truncation, which biases a long accumulation chain by about
        // half an ulp of the accumulator per instruction (measured: error growing linearly with the context, 6e-5 of the
        // row's largest output at 20000 keys).  So each tile's P V product starts from zero (a chain of 8 to 12
        // instructions) and is added to the running output with ordinary round-to-nearest fp32 arithmetic.
        float ot[16][4];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            ot[j][0] = ot[j][1] = ot[j][2] = ot[j][3] = 0.f;
        }
        // ---- O_tile = P V, P as fp16 hi + lo A fragments (k-step t16 = tokens 16*t16 .. +15 = score tiles 2*t16, 2*t16+1) ----
#pragma unroll
        for (int t16 = 0; t16 < 4; ++t16) {
            uint32_t ph[4], pl[4];
#pragma unroll
            for (int half = 0; half < 2; ++half)
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const float x0 = s[2 * t16 + half][2 * hrow], x1 = s[2 * t16 + half][2 * hrow + 1];
                    const uint32_t hi = pack_half2(x0, x1);
                    const float2 hf = __half22float2(*reinterpret_cast<const __half2*>(&hi));
                    ph[2 * half + hrow] = hi;
                    pl[2 * half + hrow] = pack_half2(x0 - hf.x, x1 - hf.y);
                }
#pragma unroll
            for (int jd2 = 0; jd2 < 8; ++jd2) {        // two 8-dim tiles per ldmatrix.x4.trans
                uint32_t b[4];
                const int row = 16 * t16 + (lane & 7) + ((lane >> 3) & 1) * 8, chunk = 2 * jd2 + (lane >> 4);
                ldmatrix_x4_trans(b, vs + pf_swizzle(row, chunk));
                mma_16816(ot[2 * jd2], ph, b[0], b[1]);
                mma_16816(ot[2 * jd2], pl, b[0], b[1]);
                mma_16816(ot[2 * jd2 + 1], ph, b[2], b[3]);
                mma_16816(ot[2 * jd2 + 1], pl, b[2], b[3]);
                if (KSPLIT) {
                    ldmatrix_x4_trans(b, vls + pf_swizzle(row, chunk));
                    mma_16816(ot[2 * jd2], ph, b[0], b[1]);
                    mma_16816(ot[2 * jd2 + 1], ph, b[2], b[3]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            o[j][0] = fmaf(o[j][0], corr[0], ot[j][0]); o[j][1] = fmaf(o[j][1], corr[0], ot[j][1]);
            o[j][2] = fmaf(o[j][2], corr[1], ot[j][2]); o[j][3] = fmaf(o[j][3], corr[1], ot[j][3]);
        }
        __syncthreads();
    }

    // ---- normalise and store ----
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const bool ok = h ? row_hi_ok : row_lo_ok;
        if (!ok) continue;
        const int qi = h ? qi_hi : qi_lo, head = h ? head_hi : head_lo;
        const float inv = l_run[h] > 0.f ? 1.0f / l_run[h] : 0.f;
        float* dst = p.out + (static_cast<int64_t>(qi) * p.num_q_heads + head) * kHeadDim;
#pragma unroll
        for (int j = 0; j < 16; ++j)
            *reinterpret_cast<float2*>(dst + 8 * j + 2 * qlane) = make_float2(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
    }
}

}  // namespace er
