// TurboQuant rows in the persistent flash-decode kernel (see flash_decode.cuh): the stage layout, the producer's
// copies and the query rotation.  The per-unit compute is TurboMmaPolicy (flash_decode_turbo_mma.cuh).
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
struct TurboStaging {
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
    static constexpr bool kRotated = true;
    static constexpr bool kFusedAppend = false;   // rows are quantised by the separate append kernel
    static_assert(STAGES % WARP_GROUPS == 0, "STAGES must be a multiple of WARP_GROUPS");
    static_assert(UNITS_PER_TILE * WARP_GROUPS >= GROUP, "one consumer warp per query head rotates it and transforms its output back");
    __device__ static void patch_new_row(const DecodeParams&, uint8_t*, int, int, int, int, int, int, const float*, const float*,
                                         const float2*, int) {}
    template <class WAIT>
    __device__ static void issue_tile(const DecodeParams& p, uint8_t* stage, uint64_t* bar, int layer, int seq, int head,
                                      int t0, int ntok, int lane, int /*ring start: fp16 rows only*/, WAIT&& wait_free) {
        const int nb = p.norm_fp16 ? 2 : 4;
        const uint8_t* kc = p.k_base + static_cast<int64_t>(layer) * p.k_layer_stride_bytes;
        const uint8_t* vc = p.v_base + static_cast<int64_t>(layer) * p.v_layer_stride_bytes;
        const uint8_t* kn = p.kn_base + static_cast<int64_t>(layer) * p.n_layer_stride_bytes;
        const uint8_t* vn = p.vn_base + static_cast<int64_t>(layer) * p.n_layer_stride_bytes;
        const int ps = p.addr.page_size;
        const int first_page = t0 / ps;
        const int nseg = (t0 + ntok - 1) / ps - first_page + 1;
        // the lane's first copy: its page is looked up in the block table while the stage is still busy
        const int64_t row0 = lane < 4 * nseg ? row_index(p.addr, seq, head, max(t0, (first_page + (lane >> 2)) * ps)) : 0;
        wait_free();
        if (lane == 0)
            mbar_arrive_expect_tx(bar, static_cast<uint32_t>(ntok) * (kKW + kVW) * 4 + 2u * ((static_cast<uint32_t>(ntok) * nb + 15u) & ~15u));
        __syncwarp();
        for (int c = lane; c < 4 * nseg; c += 32) {
            const int kind = c & 3, sgi = c >> 2;
            const int tb = max(t0, (first_page + sgi) * ps);
            const int te = min(t0 + ntok, (first_page + sgi + 1) * ps);
            const int64_t row = c == lane ? row0 : row_index(p.addr, seq, head, tb);
            const uint32_t rows = static_cast<uint32_t>(te - tb);
            if (kind == 0) bulk_g2s(stage + (tb - t0) * kKW * 4, kc + row * (kKW * 4), rows * kKW * 4, bar);
            else if (kind == 1) bulk_g2s(stage + kKcBytes + (tb - t0) * kVW * 4, vc + row * (kVW * 4), rows * kVW * 4, bar);
            else if (kind == 2) bulk_g2s(stage + kOffKn + (tb - t0) * nb, kn + row * nb, (rows * nb + 15u) & ~15u, bar);
            else bulk_g2s(stage + kOffVn + (tb - t0) * nb, vn + row * nb, (rows * nb + 15u) & ~15u, bar);
        }
    }

    // Warps 0..GROUP-1 each rotate one q head ([RoPE ->] randomizedHadamard) and publish it; every lane then
    // reads the 16 rotated coordinates it multiplies against.
    __device__ static void rotate_queries(const DecodeParams& p, float* qrot, const float* qrow, const float2* cs, int warp, int lane) {
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
    }

    __device__ static float load_norm(const uint8_t* base, int idx, int fp16) {
        return fp16 ? __half2float(reinterpret_cast<const __half*>(base)[idx]) : reinterpret_cast<const float*>(base)[idx];
    }

    __device__ static void store_out(const DecodeParams& p, int64_t out_off, const float* fin, int warp, int lane) {
        if (warp < GROUP) {
            const float4 t = *reinterpret_cast<const float4*>(fin + warp * kHeadDim + 4 * lane);
            float a[4] = {t.x, t.y, t.z, t.w};
            warp_tq_inverse(a, lane);
            const float4 o = make_float4(a[0], a[1], a[2], a[3]);
            const int64_t e = out_off + warp * kHeadDim + 4 * lane;
            *reinterpret_cast<float4*>(p.out + e) = o;
            for (int r = 0; r < p.num_peers; ++r) *reinterpret_cast<float4*>(p.peer_out[r] + e) = o;   // kv-head sharding
        }
    }
};

}  // namespace er
