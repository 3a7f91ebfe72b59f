// TurboQuant storage policy of the persistent flash-decode kernel (see flash_decode.cuh).
//
// Follows gqa_attention_turboquant_decode (Shaders/TurboQuant.metal:1794-2001) for the fixed presets:
//   qR = randomizedHadamard(q)                          once per q head and item
//   score_t = kNorm_t * sum_d qR[d] * centroidK(code_t[d]) * scale
//   acc[d] += p_t * vNorm_t * centroidV(code_t[d])      accumulated in the rotated space
//   out = inverseRandomizedHadamard(acc) / sum p        one inverse transform after the split merge
//                                                        (the transform is linear, so it commutes with it)
// Rows are `words` packed 32-bit words (BitPacker layout, Sources/EdgeRunnerMetal/TurboQuant.swift:1554-1573)
// plus one stored norm (fp32, or fp16 in the compact format); pages keep each kv head's rows contiguous,
// so a tile is four bulk copies per touched page: K codes, V codes, K norms, V norms.
#pragma once

#include "flash_decode.cuh"
#include "tq_math.cuh"

namespace er {

template <int GROUP, int KBITS, int VBITS, int UNITS_PER_TILE = 8, int WARP_GROUPS = 1, int STAGES = 4>
struct TurboPolicy {
    static constexpr int kGroup = GROUP;
    static constexpr int kUnitsPerTile = UNITS_PER_TILE;
    static constexpr int kWarpGroups = WARP_GROUPS;
    static constexpr int kStages = STAGES;
    static constexpr int kTileTokens = UNITS_PER_TILE * kUnitTokens;
    static constexpr int kThreads = (UNITS_PER_TILE * WARP_GROUPS + 1) * 32;
    static constexpr int kKW = tq_code_words(KBITS);
    static constexpr int kVW = tq_code_words(VBITS);
    static constexpr int kKcBytes = kTileTokens * kKW * 4;
    static constexpr int kVcBytes = kTileTokens * kVW * 4;
    static constexpr int kOffKn = kKcBytes + kVcBytes;
    static constexpr int kOffVn = kOffKn + kTileTokens * 4;
    static constexpr int kStageBytes = kOffVn + kTileTokens * 4;
    // Pair tables: entry (code of dim d) | (code of dim d+1) << bits -> (centroid, centroid), one column per lane so
    // that 32 lanes looking up 32 different pairs never collide on a bank.
    static constexpr int kKPairs = 1 << (2 * KBITS), kVPairs = 1 << (2 * VBITS);
    static constexpr int kOffLutK = 0;                       // float2 [kKPairs][32]
    static constexpr int kOffLutV = kKPairs * 32 * 8;        // float2 [kVPairs][32]
    static constexpr int kOffQrot = kOffLutV + kVPairs * 32 * 8;   // [GROUP][128] rotated queries
    static constexpr int kOffFin = kOffQrot + GROUP * kHeadDim * 4;
    static constexpr int kExtraBytes = kOffFin + GROUP * kHeadDim * 4;
    static constexpr bool kRotated = true;
    static constexpr bool kFusedAppend = false;   // rows are quantised by the separate append kernel
    static_assert(STAGES % WARP_GROUPS == 0, "STAGES must be a multiple of WARP_GROUPS");
    __device__ static void patch_new_row(const DecodeParams&, uint8_t*, int, int, int, int, int, int, const float*, const float*,
                                         const float2*, int) {}
    static constexpr int kQRegs = 16;                        // per head: rotated dims [16i, 16i+16), i = lane % 8

    __device__ static void init_extra(uint8_t* extra, int tid) {
        float2* lk = reinterpret_cast<float2*>(extra + kOffLutK);
        float2* lv = reinterpret_cast<float2*>(extra + kOffLutV);
        for (int e = tid; e < kKPairs * 32; e += kThreads) {
            const int pv = e >> 5;
            lk[e] = make_float2(tq_centroids<KBITS>()[pv & ((1 << KBITS) - 1)], tq_centroids<KBITS>()[pv >> KBITS]);
        }
        for (int e = tid; e < kVPairs * 32; e += kThreads) {
            const int pv = e >> 5;
            lv[e] = make_float2(tq_centroids<VBITS>()[pv & ((1 << VBITS) - 1)], tq_centroids<VBITS>()[pv >> VBITS]);
        }
    }

    __device__ static void issue_tile(const DecodeParams& p, uint8_t* stage, uint64_t* bar, int layer, int seq, int head,
                                      int t0, int ntok, int lane) {
        const int nb = p.norm_fp16 ? 2 : 4;
        const uint8_t* kc = p.k_base + static_cast<int64_t>(layer) * p.k_layer_stride_bytes;
        const uint8_t* vc = p.v_base + static_cast<int64_t>(layer) * p.v_layer_stride_bytes;
        const uint8_t* kn = p.kn_base + static_cast<int64_t>(layer) * p.n_layer_stride_bytes;
        const uint8_t* vn = p.vn_base + static_cast<int64_t>(layer) * p.n_layer_stride_bytes;
        if (lane == 0)
            mbar_arrive_expect_tx(bar, static_cast<uint32_t>(ntok) * (kKW + kVW) * 4 + 2u * ((static_cast<uint32_t>(ntok) * nb + 15u) & ~15u));
        __syncwarp();
        const int ps = p.addr.page_size;
        const int first_page = t0 / ps;
        const int nseg = (t0 + ntok - 1) / ps - first_page + 1;
        for (int c = lane; c < 4 * nseg; c += 32) {
            const int kind = c & 3, sgi = c >> 2;
            const int tb = max(t0, (first_page + sgi) * ps);
            const int te = min(t0 + ntok, (first_page + sgi + 1) * ps);
            const int64_t row = row_index(p.addr, seq, head, tb);
            const uint32_t rows = static_cast<uint32_t>(te - tb);
            if (kind == 0) bulk_g2s(stage + (tb - t0) * kKW * 4, kc + row * (kKW * 4), rows * kKW * 4, bar);
            else if (kind == 1) bulk_g2s(stage + kKcBytes + (tb - t0) * kVW * 4, vc + row * (kVW * 4), rows * kVW * 4, bar);
            else if (kind == 2) bulk_g2s(stage + kOffKn + (tb - t0) * nb, kn + row * nb, (rows * nb + 15u) & ~15u, bar);
            else bulk_g2s(stage + kOffVn + (tb - t0) * nb, vn + row * nb, (rows * nb + 15u) & ~15u, bar);
        }
    }

    // Warps 0..GROUP-1 each rotate one q head ([RoPE ->] randomizedHadamard) and publish it; every lane then
    // reads the 16 rotated coordinates it multiplies against.
    __device__ static void load_q(const DecodeParams& p, float (&q)[GROUP][kQRegs], const float* qrow, const float2* cs,
                                  uint8_t* extra, int warp, int lane) {
        float* qrot = reinterpret_cast<float*>(extra + kOffQrot);
        if (warp < GROUP) {
            const float4 x = __ldg(reinterpret_cast<const float4*>(qrow + warp * kHeadDim + 4 * lane));
            float a[4] = {x.x, x.y, x.z, x.w};
            if (p.apply_rope) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float other = __shfl_xor_sync(0xffffffffu, a[c], 16);
                    const float2 t = cs[(4 * lane + c) & 63];
                    float y0, y1;
                    if (lane < 16) { rope_rotate(a[c], other, t, y0, y1); a[c] = y0; }
                    else           { rope_rotate(other, a[c], t, y0, y1); a[c] = y1; }
                }
            }
            warp_tq_forward(a, lane);
            *reinterpret_cast<float4*>(qrot + warp * kHeadDim + 4 * lane) = make_float4(a[0], a[1], a[2], a[3]);
        }
        consumer_sync<UNITS_PER_TILE * WARP_GROUPS * 32>();
        const int i = lane & 7;
#pragma unroll
        for (int g = 0; g < GROUP; ++g)
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                const float4 t = *reinterpret_cast<const float4*>(qrot + g * kHeadDim + 16 * i + 4 * c4);
                q[g][4 * c4] = t.x; q[g][4 * c4 + 1] = t.y; q[g][4 * c4 + 2] = t.z; q[g][4 * c4 + 3] = t.w;
            }
    }

    __device__ static float load_norm(const uint8_t* base, int idx, int fp16) {
        return fp16 ? __half2float(reinterpret_cast<const __half*>(base)[idx]) : reinterpret_cast<const float*>(base)[idx];
    }

    __device__ static void process_unit(const DecodeParams& p, const uint8_t* stage, int unit, int nvalid,
                                        const float (&q)[GROUP][kQRegs], float (&m)[GROUP], float (&l)[GROUP],
                                        float (&acc)[GROUP][4], float* prob, const uint8_t* extra, int lane) {
        const float2* lutk = reinterpret_cast<const float2*>(extra + kOffLutK) + lane;
        const float2* lutv = reinterpret_cast<const float2*>(extra + kOffLutV) + lane;
        const uint32_t* kc = reinterpret_cast<const uint32_t*>(stage) + unit * kUnitTokens * kKW;
        const uint32_t* vc = reinterpret_cast<const uint32_t*>(stage + kKcBytes) + unit * kUnitTokens * kVW;
        const uint8_t* kn = stage + kOffKn;
        const uint8_t* vn = stage + kOffVn;
        const int j = lane >> 3, i = lane & 7;
        float s[4][GROUP];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int row = 4 * r + j;
            const uint32_t* words = kc + row * kKW;
            uint64_t bits;
            if (KBITS == 2) {
                bits = words[i];
            } else {
                const int off = 16 * KBITS * i, w0 = off >> 5, sh = off & 31;
                bits = ((static_cast<uint64_t>(words[w0 + 1]) << 32) | words[w0]) >> sh;
            }
            float cv[16];
#pragma unroll
            for (int c2 = 0; c2 < 8; ++c2) {
                uint32_t pv;
                if (KBITS == 4) {      // byte c2 of the two words
                    const uint32_t w = c2 < 4 ? static_cast<uint32_t>(bits) : static_cast<uint32_t>(bits >> 32);
                    pv = (w >> (8 * (c2 & 3))) & 0xFFu;
                } else {
                    pv = static_cast<uint32_t>(bits >> (2 * KBITS * c2)) & (kKPairs - 1);
                }
                const float2 t = lutk[pv * 32];
                cv[2 * c2] = t.x;
                cv[2 * c2 + 1] = t.y;
            }
#pragma unroll
            for (int g = 0; g < GROUP; ++g) {
                float d0 = 0.f, d1 = 0.f;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    d0 = fmaf(q[g][c], cv[c], d0);
                    d1 = fmaf(q[g][8 + c], cv[8 + c], d1);
                }
                s[r][g] = d0 + d1;
            }
        }
        float vnorm[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int row = 4 * r + j;
            const bool ok = row < nvalid;
            const float knorm = ok ? load_norm(kn, unit * kUnitTokens + row, p.norm_fp16) : 0.f;
            vnorm[r] = ok ? load_norm(vn, unit * kUnitTokens + row, p.norm_fp16) : 0.f;
#pragma unroll
            for (int g = 0; g < GROUP; ++g) {
                float v = s[r][g];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                s[r][g] = ok ? (knorm * v) * p.scale_log2 : -INFINITY;
            }
        }
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
            float mx = fmaxf(fmaxf(s[0][g], s[1][g]), fmaxf(s[2][g], s[3][g]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(m[g], mx);
            const float corr = fast_exp2(m[g] - m_new);
            float psum = 0.f;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float pr = fast_exp2(s[r][g] - m_new);
                psum += pr;
                if (i == 0) prob[g * kUnitTokens + 4 * r + j] = pr * vnorm[r];   // p_t * vNorm_t
            }
            psum += __shfl_xor_sync(0xffffffffu, psum, 8);
            psum += __shfl_xor_sync(0xffffffffu, psum, 16);
            l[g] = fmaf(l[g], corr, psum);
            m[g] = m_new;
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[g][c] *= corr;
        }
        __syncwarp();
        // P.V in the rotated space: lane owns rotated dims [4*lane, 4*lane+4) = stream bits [4*VBITS*lane, +4*VBITS).
        const int voff = 4 * VBITS * lane, vw0 = voff >> 5, vsh = voff & 31;
        for (int t = 0; t < nvalid; ++t) {
            const uint32_t* words = vc + t * kVW;
            uint32_t bits = words[vw0] >> vsh;
            if (VBITS == 3 && vsh > 20) bits |= words[vw0 + 1] << (32 - vsh);
            const float2 v01 = lutv[(bits & (kVPairs - 1)) * 32];
            const float2 v23 = lutv[((bits >> (2 * VBITS)) & (kVPairs - 1)) * 32];
            const float cv[4] = {v01.x, v01.y, v23.x, v23.y};
#pragma unroll
            for (int g = 0; g < GROUP; ++g) {
                const float w = prob[g * kUnitTokens + t];
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[g][c] = fmaf(w, cv[c], acc[g][c]);
            }
        }
        __syncwarp();
    }

    __device__ static void store_out(float* out_item, const float* fin, int warp, int lane) {
        if (warp < GROUP) {
            const float4 t = *reinterpret_cast<const float4*>(fin + warp * kHeadDim + 4 * lane);
            float a[4] = {t.x, t.y, t.z, t.w};
            warp_tq_inverse(a, lane);
            *reinterpret_cast<float4*>(out_item + warp * kHeadDim + 4 * lane) = make_float4(a[0], a[1], a[2], a[3]);
        }
    }
};

}  // namespace er
