// Layers whose keys and values use different row formats (chosen per layer by TurboQuantV2Contract, TurboQuant.swift:432-488) in
// the persistent flash-decode kernel.  The two sides live in two caches of the same geometry, so DecodeParams names two
// addressings: k_* / kn_* / addr / lengths describe the key cache, v_* / vn_* / addr_v the value cache.  Each policy here joins
// the score half of one single-format policy to the output half of another; the halves meet in the score fragment
// (token g | g + 8) x (head 2c | 2c + 1), which all of them use.
//
// TurboValuesPolicy: TurboQuant values of a fixed preset with q8_0 keys (gqa_attention_q8k_turboquant_decode,
// Shaders/TurboQuant.metal:1651-1792: earlyQ8KeyLayers, a q8_0 key cache type) or float16 keys (a dense key cache type).
//
// Scores are Q8MmaPolicy's (queries in their own space, int8 exact in fp16, one accumulator per 32-element block) or
// DenseMmaPolicy's (the float16 rows as they lie), outputs
// are TurboMmaPolicy's (value centroids looked up as fp16 hi + lo pairs, accumulated in the rotated space, one inverse
// transform after the merge); the fragment layouts of the two policies meet in the score fragment (token g | g + 8) x
// (head 2c | 2c + 1), which both use.  Stage = K rows [| K block scales] | V codes | V norms.
#pragma once

#include <type_traits>

#include "flash_decode_dense_mma.cuh"   // includes the q8_0 and TurboQuant policies

namespace er {

// DenseMmaPolicy's score block for any state with its query fragments: the float16 key rows at `krows` (256 bytes each) are the A
// operands as they lie (16-byte chunks 4j + c of tokens g and g + 8).  s = (token g | g + 8) x (head 2c | 2c + 1), log2 domain.
template <bool PACKED, class ST>
__device__ __forceinline__ void dense_unit_scores(const DecodeParams& p, uint32_t krows, int unit, int nvalid, const ST& st, int lane, float (&s)[4]) {
    const int g = lane >> 2, c = lane & 3;
    const bool ok0 = g < nvalid, ok1 = g + 8 < nvalid;
    const uint32_t krow = krows + (unit * kUnitTokens + g) * kRowBytesF16 + 16 * c;
    s[0] = s[1] = s[2] = s[3] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t k0[4], k1[4];
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(k0[0]), "=r"(k0[1]), "=r"(k0[2]), "=r"(k0[3]) : "r"(krow + 64 * j) : "memory");
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(k1[0]), "=r"(k1[1]), "=r"(k1[2]), "=r"(k1[3]) : "r"(krow + 64 * j + 8 * kRowBytesF16) : "memory");
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            mma_m16n8k16(s, k0[2 * u], k1[2 * u], k0[2 * u + 1], k1[2 * u + 1], st.qh[2 * j + u][0], st.qh[2 * j + u][1]);
            if constexpr (!PACKED) mma_m16n8k16(s, k0[2 * u], k1[2 * u], k0[2 * u + 1], k1[2 * u + 1], st.ql[2 * j + u][0], st.ql[2 * j + u][1]);
        }
    }
    if constexpr (PACKED) {
#pragma unroll
        for (int i = 0; i < 4; ++i) s[i] += __shfl_xor_sync(0xffffffffu, s[i], 2);
    }
    // rows at or past nvalid were never copied (stale shared memory, possibly NaN patterns): the select discards them
    s[0] = ok0 ? s[0] * p.scale_log2 : -INFINITY;
    s[1] = ok0 ? s[1] * p.scale_log2 : -INFINITY;
    s[2] = ok1 ? s[2] * p.scale_log2 : -INFINITY;
    s[3] = ok1 ? s[3] * p.scale_log2 : -INFINITY;
}

// DenseMmaPolicy's output block for any state with its accumulator order: B = 4096 p as fp16 hi + lo, A = transposed value blocks
// of the 256-byte rows at `vrows`.
template <bool PACKED, class ST>
__device__ __forceinline__ void dense_unit_values(ST& st, uint32_t vrows, int unit, int nvalid, const float (&pr)[4], int lane) {
    constexpr float kProbScale = 4096.f;   // DenseMmaPolicy::kProbScale: State::publish divides it out
    const int g = lane >> 2, c = lane & 3;
    const bool ok0 = g < nvalid, ok1 = g + 8 < nvalid;
    const float w0 = pr[0] * kProbScale, w1 = pr[1] * kProbScale, w2 = pr[2] * kProbScale, w3 = pr[3] * kProbScale;
    const __half2 h01 = __floats2half2_rn(w0, w1), h23 = __floats2half2_rn(w2, w3);
    const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
    const uint32_t hi01 = *reinterpret_cast<const uint32_t*>(&h01), hi23 = *reinterpret_cast<const uint32_t*>(&h23);
    const uint32_t lo01 = pack_half2(w0 - f01.x, w1 - f01.y), lo23 = pack_half2(w2 - f23.x, w3 - f23.y);
    const uint32_t b0 = movmatrix_trans(PACKED && c >= 2 ? lo01 : hi01);
    const uint32_t b1 = movmatrix_trans(PACKED && c >= 2 ? lo23 : hi23);
    uint32_t b0l = 0, b1l = 0;
    if constexpr (!PACKED) {
        b0l = movmatrix_trans(lo01);
        b1l = movmatrix_trans(lo23);
    }
    const uint32_t vrow = vrows + (unit * kUnitTokens + g) * kRowBytesF16 + 16 * c;
    const bool partial = nvalid < kUnitTokens;   // warp-uniform
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t v0[4], v1[4];
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v0[0]), "=r"(v0[1]), "=r"(v0[2]), "=r"(v0[3]) : "r"(vrow + 64 * j) : "memory");
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v1[0]), "=r"(v1[1]), "=r"(v1[2]), "=r"(v1[3]) : "r"(vrow + 64 * j + 8 * kRowBytesF16) : "memory");
        if (partial) {   // 0 x NaN would poison the accumulators: stale rows become zeros
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                v0[e] = ok0 ? v0[e] : 0u;
                v1[e] = ok1 ? v1[e] : 0u;
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const uint32_t a0 = movmatrix_trans(v0[2 * u]);
            const uint32_t a1 = movmatrix_trans(v0[2 * u + 1]);
            const uint32_t a2 = movmatrix_trans(v1[2 * u]);
            const uint32_t a3 = movmatrix_trans(v1[2 * u + 1]);
            mma_m16n8k16(st.acc[2 * j + u], a0, a1, a2, a3, b0, b1);
            if constexpr (!PACKED) mma_m16n8k16(st.acc[2 * j + u], a0, a1, a2, a3, b0l, b1l);
        }
    }
}

template <int GROUP, int VBITS, bool Q8_KEYS, int UNITS_PER_TILE = 11, int WARP_GROUPS = 1, int STAGES = 3>
struct TurboValuesPolicy : TurboMmaPolicy<GROUP, VBITS, VBITS, UNITS_PER_TILE, WARP_GROUPS, STAGES> {
    using TM = TurboMmaPolicy<GROUP, VBITS, VBITS, UNITS_PER_TILE, WARP_GROUPS, STAGES>;   // tables, value lookups, state, output transform
    using Q8 = Q8MmaPolicy<GROUP, UNITS_PER_TILE, WARP_GROUPS, STAGES>;                    // query fragments, scores
    using State = typename TM::State;
    static constexpr int kTileTokens = UNITS_PER_TILE * kUnitTokens;
    static constexpr int kVW = tq_code_words(VBITS);
    static constexpr int kKRowBytes = Q8_KEYS ? 128 : kRowBytesF16;
    static constexpr int kOffKs = kTileTokens * kKRowBytes;                           // q8_0 keys: the rows' block scales
    static constexpr int kOffVc = kOffKs + (Q8_KEYS ? kTileTokens * 8 : 0);
    static constexpr int kOffVn = kOffVc + kTileTokens * kVW * 4;
    static constexpr int kStageBytes = kOffVn + kTileTokens * 4;
    static_assert(TM::kPacked == Q8::kPacked, "both sides pack the hi and lo parts of their B operands the same way");

    template <class WAIT>
    __device__ static void issue_tile(const DecodeParams& p, uint8_t* stage, uint64_t* bar, int layer, int seq, int head,
                                      int t0, int ntok, int lane, int /*ring start: fp16 rows only*/, WAIT&& wait_free) {
        const int nb = p.norm_fp16 ? 2 : 4;
        const uint8_t* kc = p.k_base + static_cast<int64_t>(layer) * p.k_layer_stride_bytes;
        const uint8_t* ks = Q8_KEYS ? p.kn_base + static_cast<int64_t>(layer) * p.n_layer_stride_bytes : nullptr;
        const uint8_t* vc = p.v_base + static_cast<int64_t>(layer) * p.v_layer_stride_bytes;
        const uint8_t* vn = p.vn_base + static_cast<int64_t>(layer) * p.vn_layer_stride_bytes;
        // page segments of the tile in each cache (a head-major cache is one page per sequence)
        const int kps = p.addr.page_size, vps = p.addr_v.page_size;
        const int kfirst = t0 / kps, kseg = (t0 + ntok - 1) / kps - kfirst + 1;
        const int vfirst = t0 / vps, vseg = (t0 + ntok - 1) / vps - vfirst + 1;
        wait_free();
        if (lane == 0) {   // side copies are rounded up to 16 bytes per page segment
            uint32_t bytes = static_cast<uint32_t>(ntok) * (kKRowBytes + kVW * 4u);
            if constexpr (Q8_KEYS) {
                for (int i = 0; i < kseg; ++i) {
                    const int tb = max(t0, (kfirst + i) * kps), te = min(t0 + ntok, (kfirst + i + 1) * kps);
                    bytes += (static_cast<uint32_t>(te - tb) * 8u + 15u) & ~15u;
                }
            }
            for (int i = 0; i < vseg; ++i) {
                const int tb = max(t0, (vfirst + i) * vps), te = min(t0 + ntok, (vfirst + i + 1) * vps);
                bytes += (static_cast<uint32_t>(te - tb) * nb + 15u) & ~15u;
            }
            mbar_arrive_expect_tx(bar, bytes);
        }
        __syncwarp();
        for (int c = lane; c < 2 * (kseg + vseg); c += 32) {
            const bool value_side = c >= 2 * kseg;
            const int i = value_side ? c - 2 * kseg : c, kind = i & 1, sgi = i >> 1;
            const int ps = value_side ? vps : kps, first = value_side ? vfirst : kfirst;
            const int tb = max(t0, (first + sgi) * ps), te = min(t0 + ntok, (first + sgi + 1) * ps);
            const uint32_t rows = static_cast<uint32_t>(te - tb);
            const int64_t row = row_index(value_side ? p.addr_v : p.addr, seq, head, tb);
            if (!value_side) {
                if (kind == 0) bulk_g2s(stage + (tb - t0) * kKRowBytes, kc + row * kKRowBytes, rows * kKRowBytes, bar);
                else if constexpr (Q8_KEYS) bulk_g2s(stage + kOffKs + (tb - t0) * 8, ks + row * 8, (rows * 8 + 15u) & ~15u, bar);
            } else {
                if (kind == 0) bulk_g2s(stage + kOffVc + (tb - t0) * kVW * 4, vc + row * (kVW * 4), rows * kVW * 4, bar);
                else bulk_g2s(stage + kOffVn + (tb - t0) * nb, vn + row * nb, (rows * nb + 15u) & ~15u, bar);
            }
        }
    }

    // queries stay in their own space (q8_0 and float16 keys are not rotated; both key policies use the same fragment order); the
    // tables are the value side's
    __device__ static void load_q(const DecodeParams& p, State& st, const float* qrow, const float2* cs, uint8_t* extra, int, int lane, int) {
        const TurboSmemPlan pl = TM::plan(extra);
        st.lut_k = pl.lut_k | (lane << 3);
        st.lut_v = pl.lut_v | (lane << 3);
        Q8::load_q_fragments(p, st, qrow, cs, lane);
    }

    __device__ static void process_unit(const DecodeParams& p, const uint8_t* stage, int unit, int nvalid, State& st, float*,
                                        const uint8_t*, int lane) {
        const int g = lane >> 2, c = lane & 3;
        const uint32_t sbase = smem_u32(stage);
        const bool ok0 = g < nvalid, ok1 = g + 8 < nvalid;
        // value codes: dims [16g, 16g + 16) of tokens 2c, 2c + 1, 2c + 8, 2c + 9 (TurboMmaPolicy's value layout), read ahead of the scores
        uint32_t vlo[4], vhi[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t row = sbase + kOffVc + (unit * kUnitTokens + 2 * c + (j & 1) + 8 * (j >> 1)) * kVW * 4;
            if constexpr (VBITS == 4) {
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(vlo[j]), "=r"(vhi[j]) : "r"(row + 8 * g) : "memory");
            } else if constexpr (VBITS == 3) {
                const uint32_t w = row + ((3 * g) >> 1) * 4;
                const uint32_t wa = lds_u32_stage(w), wb = lds_u32_stage(w + 4);
                const uint32_t sh = (g & 1) * 16;
                vlo[j] = __funnelshift_r(wa, wb, sh);
                vhi[j] = wb >> sh;
            } else {
                vlo[j] = lds_u32_stage(row + 4 * g);
                vhi[j] = 0;
            }
        }
        const int r0 = unit * kUnitTokens + g;
        constexpr float inv_sv = 1.f / tq_fp16_scale<VBITS>();
        const float vn0 = ok0 ? TM::load_norm(stage + kOffVn, r0, p.norm_fp16) * inv_sv : 0.f;
        const float vn1 = ok1 ? TM::load_norm(stage + kOffVn, r0 + 8, p.norm_fp16) * inv_sv : 0.f;

        float s[4], pr[4];
        if constexpr (Q8_KEYS) {
            Q8::unit_scores(p, sbase, sbase + kOffKs, unit, nvalid, st, lane, s);
        } else {
            dense_unit_scores<TM::kPacked>(p, sbase, unit, nvalid, st, lane, s);
        }
        mma_softmax_step(st, s, pr);

        // (p_t * vNorm_t)[token][head] as fp16 hi + lo parts, transposed and duplicated on the (hi, lo) labels of a centroid
        const float w0 = pr[0] * vn0, w1 = pr[1] * vn0, w2 = pr[2] * vn1, w3 = pr[3] * vn1;
        const __half2 h01 = __floats2half2_rn(w0, w1), h23 = __floats2half2_rn(w2, w3);
        const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
        const uint32_t hi01 = *reinterpret_cast<const uint32_t*>(&h01), hi23 = *reinterpret_cast<const uint32_t*>(&h23);
        const uint32_t lo01 = pack_half2(w0 - f01.x, w1 - f01.y), lo23 = pack_half2(w2 - f23.x, w3 - f23.y);
        if constexpr (TM::kPacked) {
            const uint32_t x0 = movmatrix_trans(c < 2 ? hi01 : lo01), x1 = movmatrix_trans(c < 2 ? hi23 : lo23);
            const uint32_t bh[4] = {__byte_perm(x0, x0, 0x1010), __byte_perm(x0, x0, 0x3232), __byte_perm(x1, x1, 0x1010), __byte_perm(x1, x1, 0x3232)};
            TM::template value_tiles<0>(st, vlo, vhi, bh, bh);
        } else {
            const uint32_t x0 = movmatrix_trans(hi01), x1 = movmatrix_trans(hi23);
            const uint32_t y0 = movmatrix_trans(lo01), y1 = movmatrix_trans(lo23);
            const uint32_t bh[4] = {__byte_perm(x0, x0, 0x1010), __byte_perm(x0, x0, 0x3232), __byte_perm(x1, x1, 0x1010), __byte_perm(x1, x1, 0x3232)};
            const uint32_t bl[4] = {__byte_perm(y0, y0, 0x1010), __byte_perm(y0, y0, 0x3232), __byte_perm(y1, y1, 0x1010), __byte_perm(y1, y1, 0x3232)};
            TM::template value_tiles<0>(st, vlo, vhi, bh, bl);
        }
    }
};

template <int GROUP, int VBITS, int UNITS_PER_TILE = 11, int WARP_GROUPS = 1, int STAGES = 3>
using Q8KTurboVPolicy = TurboValuesPolicy<GROUP, VBITS, true, UNITS_PER_TILE, WARP_GROUPS, STAGES>;
template <int GROUP, int VBITS, int UNITS_PER_TILE = 11, int WARP_GROUPS = 1, int STAGES = 2>
using DenseKTurboVPolicy = TurboValuesPolicy<GROUP, VBITS, false, UNITS_PER_TILE, WARP_GROUPS, STAGES>;

// TurboKeysPolicy: TurboQuant keys of a fixed preset with float16 values (gqa_attention_turboquant_decode_f16v,
// Shaders/TurboQuant.metal:2003-2239) or q8_0 values (the boundary layers of TurboQuantAdaptiveMode.boundaryQ8).  Scores are
// TurboMmaPolicy's (rotated queries, key centroids looked up as fp16 hi + lo pairs); outputs are DenseMmaPolicy's (value rows as
// they lie, through movmatrix, probabilities carried times 4096) or Q8MmaPolicy's (int8 pairs, probabilities times the block
// scales), in the values' own space: no output transform.  Stage = K codes | K norms | V rows [| V block scales].
template <int GROUP, int KBITS, bool Q8_VALUES, int UNITS_PER_TILE = 11, int WARP_GROUPS = 1, int STAGES = 2>
struct TurboKeysPolicy {
    using TM = TurboMmaPolicy<GROUP, KBITS, KBITS, UNITS_PER_TILE, WARP_GROUPS, STAGES>;   // key table, score fragments, query rotation
    using DM = DenseMmaPolicy<GROUP, UNITS_PER_TILE, WARP_GROUPS, STAGES>;
    using Q8 = Q8MmaPolicy<GROUP, UNITS_PER_TILE, WARP_GROUPS, STAGES>;
    using VState = std::conditional_t<Q8_VALUES, typename Q8::State, typename DM::State>;   // the value side's accumulator order
    struct State : VState {
        uint32_t lut_k;   // this lane's column of the key table
    };
    static constexpr int kGroup = GROUP;
    static constexpr int kUnitsPerTile = UNITS_PER_TILE;
    static constexpr int kWarpGroups = WARP_GROUPS;
    static constexpr int kStages = STAGES;
    static constexpr int kTileTokens = UNITS_PER_TILE * kUnitTokens;
    static constexpr int kThreads = (UNITS_PER_TILE * WARP_GROUPS + 1) * 32;
    static constexpr int kKW = tq_code_words(KBITS);
    static constexpr int kVRowBytes = Q8_VALUES ? 128 : kRowBytesF16;
    static constexpr int kOffKn = kTileTokens * kKW * 4;
    static constexpr int kOffV = kOffKn + kTileTokens * 4;
    static constexpr int kOffVs = kOffV + kTileTokens * kVRowBytes;
    static constexpr int kStageBytes = kOffVs + (Q8_VALUES ? kTileTokens * 8 : 0);
    static constexpr int kExtraBytes = -1;          // the key table sits on a 64 KB boundary of the shared window (TurboSmemPlan)
    static constexpr bool kRotated = false;         // outputs are in the values' space
    static constexpr bool kFusedAppend = false;
    static constexpr int kFoldUnits = 32;
    static constexpr bool kPacked = TM::kPacked;
    static_assert(STAGES % WARP_GROUPS == 0, "STAGES must be a multiple of WARP_GROUPS");

    __device__ static float* fin_ptr(uint8_t*) { return nullptr; }
    __device__ static bool init_extra(uint8_t* extra, int tid, int smem_bytes_after_extra) { return TM::init_extra(extra, tid, smem_bytes_after_extra); }
    __device__ static void patch_new_row(const DecodeParams&, uint8_t*, int, int, int, int, int, int, const float*, const float*,
                                         const float2*, int) {}
    __device__ static void store_out(const DecodeParams&, int64_t, const float*, int, int) {}

    template <class WAIT>
    __device__ static void issue_tile(const DecodeParams& p, uint8_t* stage, uint64_t* bar, int layer, int seq, int head,
                                      int t0, int ntok, int lane, int /*ring start: fp16 caches only*/, WAIT&& wait_free) {
        const int nb = p.norm_fp16 ? 2 : 4;
        const uint8_t* kc = p.k_base + static_cast<int64_t>(layer) * p.k_layer_stride_bytes;
        const uint8_t* kn = p.kn_base + static_cast<int64_t>(layer) * p.n_layer_stride_bytes;
        const uint8_t* vr = p.v_base + static_cast<int64_t>(layer) * p.v_layer_stride_bytes;
        const uint8_t* vs = Q8_VALUES ? p.vn_base + static_cast<int64_t>(layer) * p.vn_layer_stride_bytes : nullptr;
        const int kps = p.addr.page_size, vps = p.addr_v.page_size;
        const int kfirst = t0 / kps, kseg = (t0 + ntok - 1) / kps - kfirst + 1;
        const int vfirst = t0 / vps, vseg = (t0 + ntok - 1) / vps - vfirst + 1;
        wait_free();
        if (lane == 0) {   // side copies are rounded up to 16 bytes per page segment
            uint32_t bytes = static_cast<uint32_t>(ntok) * (kKW * 4u + kVRowBytes);
            for (int i = 0; i < kseg; ++i) {
                const int tb = max(t0, (kfirst + i) * kps), te = min(t0 + ntok, (kfirst + i + 1) * kps);
                bytes += (static_cast<uint32_t>(te - tb) * nb + 15u) & ~15u;
            }
            if constexpr (Q8_VALUES) {
                for (int i = 0; i < vseg; ++i) {
                    const int tb = max(t0, (vfirst + i) * vps), te = min(t0 + ntok, (vfirst + i + 1) * vps);
                    bytes += (static_cast<uint32_t>(te - tb) * 8u + 15u) & ~15u;
                }
            }
            mbar_arrive_expect_tx(bar, bytes);
        }
        __syncwarp();
        for (int c = lane; c < 2 * (kseg + vseg); c += 32) {
            const bool value_side = c >= 2 * kseg;
            const int i = value_side ? c - 2 * kseg : c, kind = i & 1, sgi = i >> 1;
            const int ps = value_side ? vps : kps, first = value_side ? vfirst : kfirst;
            const int tb = max(t0, (first + sgi) * ps), te = min(t0 + ntok, (first + sgi + 1) * ps);
            const uint32_t rows = static_cast<uint32_t>(te - tb);
            const int64_t row = row_index(value_side ? p.addr_v : p.addr, seq, head, tb);
            if (!value_side) {
                if (kind == 0) bulk_g2s(stage + (tb - t0) * kKW * 4, kc + row * (kKW * 4), rows * kKW * 4, bar);
                else bulk_g2s(stage + kOffKn + (tb - t0) * nb, kn + row * nb, (rows * nb + 15u) & ~15u, bar);
            } else {
                if (kind == 0) bulk_g2s(stage + kOffV + (tb - t0) * kVRowBytes, vr + row * kVRowBytes, rows * kVRowBytes, bar);
                else if constexpr (Q8_VALUES) bulk_g2s(stage + kOffVs + (tb - t0) * 8, vs + row * 8, (rows * 8 + 15u) & ~15u, bar);
            }
        }
    }

    // Rotated queries -> B fragments in TurboMmaPolicy's order (k-step s: label 2c + e -> dim 32c + 4s + e, 2c + 8 + e -> + 2)
    __device__ static void load_q(const DecodeParams& p, State& st, const float* qrow, const float2* cs, uint8_t* extra, int warp, int lane, int) {
        const TurboSmemPlan pl = TM::plan(extra);
        float* qrot = TM::window_ptr(extra, pl.rows);
        TM::rotate_queries(p, qrot, qrow, cs, warp, lane);
        st.lut_k = pl.lut_k | (lane << 3);
        const int g = lane >> 2, c = lane & 3;
        const int head = kPacked ? (g & 3) : g;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            if (head < GROUP) t = *reinterpret_cast<const float4*>(qrot + head * kHeadDim + 32 * c + 4 * s);
            const __half2 h01 = __floats2half2_rn(t.x, t.y), h23 = __floats2half2_rn(t.z, t.w);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            const uint32_t hi0 = *reinterpret_cast<const uint32_t*>(&h01), hi1 = *reinterpret_cast<const uint32_t*>(&h23);
            const uint32_t lo0 = pack_half2(t.x - f01.x, t.y - f01.y), lo1 = pack_half2(t.z - f23.x, t.w - f23.y);
            if constexpr (kPacked) {
                st.qh[s][0] = g < 4 ? hi0 : lo0;
                st.qh[s][1] = g < 4 ? hi1 : lo1;
            } else {
                st.qh[s][0] = hi0; st.qh[s][1] = hi1;
                st.ql[s][0] = lo0; st.ql[s][1] = lo1;
            }
        }
        st.reset();
    }

    __device__ static void process_unit(const DecodeParams& p, const uint8_t* stage, int unit, int nvalid, State& st, float*,
                                        const uint8_t*, int lane) {
        const int g = lane >> 2, c = lane & 3;
        const uint32_t sbase = smem_u32(stage);
        const bool ok0 = g < nvalid, ok1 = g + 8 < nvalid;
        const int r0 = unit * kUnitTokens + g;
        // ---- scores (TurboMmaPolicy): the thread's 32 codes of tokens g and g + 8 ----
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const uint32_t kc = sbase + (r0 * kKW + c * KBITS) * 4;
            uint32_t k0[KBITS], k1[KBITS];
            load_code_chunk<KBITS>(kc, k0);
            load_code_chunk<KBITS>(kc + 32 * kKW, k1);
            typename TM::State ts;   // the score steps read the query fragments and the table column only
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                ts.qh[i][0] = st.qh[i][0]; ts.qh[i][1] = st.qh[i][1];
                if constexpr (!kPacked) { ts.ql[i][0] = st.ql[i][0]; ts.ql[i][1] = st.ql[i][1]; }
            }
            ts.lut_k = st.lut_k;
            if constexpr (kPacked) {
                float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
                TM::template score_steps_packed<0>(sa, sb, k0, k1, ts);
                s[0] = sa[0] + sa[2]; s[1] = sa[1] + sa[3]; s[2] = sb[0] + sb[2]; s[3] = sb[1] + sb[3];
#pragma unroll
                for (int i = 0; i < 4; ++i) s[i] += __shfl_xor_sync(0xffffffffu, s[i], 2);
            } else {
                TM::template score_steps<0>(s, k0, k1, ts);
            }
            const float kn0 = ok0 ? TM::load_norm(stage + kOffKn, r0, p.norm_fp16) : 0.f;
            const float kn1 = ok1 ? TM::load_norm(stage + kOffKn, r0 + 8, p.norm_fp16) : 0.f;
            const float sc = p.scale_log2 * (1.f / tq_fp16_scale<KBITS>());
            s[0] = ok0 ? (kn0 * s[0]) * sc : -INFINITY;
            s[1] = ok0 ? (kn0 * s[1]) * sc : -INFINITY;
            s[2] = ok1 ? (kn1 * s[2]) * sc : -INFINITY;
            s[3] = ok1 ? (kn1 * s[3]) * sc : -INFINITY;
        }
        float pr[4];
        mma_softmax_step(st, s, pr);
        if constexpr (Q8_VALUES) Q8::unit_values(st, sbase + kOffV, sbase + kOffVs, unit, nvalid, pr, lane);
        else dense_unit_values<kPacked>(st, sbase + kOffV, unit, nvalid, pr, lane);
    }
};

template <int GROUP, int KBITS, int UNITS_PER_TILE = 11, int WARP_GROUPS = 1, int STAGES = 2>
using TurboKDenseVPolicy = TurboKeysPolicy<GROUP, KBITS, false, UNITS_PER_TILE, WARP_GROUPS, STAGES>;
template <int GROUP, int KBITS, int UNITS_PER_TILE = 11, int WARP_GROUPS = 1, int STAGES = 3>
using TurboKQ8VPolicy = TurboKeysPolicy<GROUP, KBITS, true, UNITS_PER_TILE, WARP_GROUPS, STAGES>;

// PlainPairPolicy: q8_0 keys with float16 values or float16 keys with q8_0 values -- neither side is rotated and neither needs a
// table; Q8MmaPolicy and DenseMmaPolicy share one query fragment order and one accumulator order.
// Stage = K rows [| K block scales] | V rows [| V block scales].
template <int GROUP, bool Q8_KEYS, int UNITS_PER_TILE = 11, int WARP_GROUPS = 1, int STAGES = 2>
struct PlainPairPolicy {
    static constexpr bool Q8_VALUES = !Q8_KEYS;
    using DM = DenseMmaPolicy<GROUP, UNITS_PER_TILE, WARP_GROUPS, STAGES>;
    using Q8 = Q8MmaPolicy<GROUP, UNITS_PER_TILE, WARP_GROUPS, STAGES>;
    using State = std::conditional_t<Q8_VALUES, typename Q8::State, typename DM::State>;   // the value side's probability scale
    static constexpr int kGroup = GROUP;
    static constexpr int kUnitsPerTile = UNITS_PER_TILE;
    static constexpr int kWarpGroups = WARP_GROUPS;
    static constexpr int kStages = STAGES;
    static constexpr int kTileTokens = UNITS_PER_TILE * kUnitTokens;
    static constexpr int kThreads = (UNITS_PER_TILE * WARP_GROUPS + 1) * 32;
    static constexpr int kKRowBytes = Q8_KEYS ? 128 : kRowBytesF16, kVRowBytes = Q8_VALUES ? 128 : kRowBytesF16;
    static constexpr int kOffKs = kTileTokens * kKRowBytes;
    static constexpr int kOffV = kOffKs + (Q8_KEYS ? kTileTokens * 8 : 0);
    static constexpr int kOffVs = kOffV + kTileTokens * kVRowBytes;
    static constexpr int kStageBytes = kOffVs + (Q8_VALUES ? kTileTokens * 8 : 0);
    static constexpr int kExtraBytes = 0;
    static constexpr bool kRotated = false;
    static constexpr bool kFusedAppend = false;
    static constexpr int kFoldUnits = 32;
    static constexpr bool kPacked = Q8::kPacked;
    static_assert(STAGES % WARP_GROUPS == 0, "STAGES must be a multiple of WARP_GROUPS");

    __device__ static float* fin_ptr(uint8_t*) { return nullptr; }
    __device__ static bool init_extra(uint8_t*, int, int) { return true; }
    __device__ static void patch_new_row(const DecodeParams&, uint8_t*, int, int, int, int, int, int, const float*, const float*,
                                         const float2*, int) {}
    __device__ static void store_out(const DecodeParams&, int64_t, const float*, int, int) {}

    template <class WAIT>
    __device__ static void issue_tile(const DecodeParams& p, uint8_t* stage, uint64_t* bar, int layer, int seq, int head,
                                      int t0, int ntok, int lane, int /*ring start: fp16 caches only*/, WAIT&& wait_free) {
        const uint8_t* kr = p.k_base + static_cast<int64_t>(layer) * p.k_layer_stride_bytes;
        const uint8_t* ks = Q8_KEYS ? p.kn_base + static_cast<int64_t>(layer) * p.n_layer_stride_bytes : nullptr;
        const uint8_t* vr = p.v_base + static_cast<int64_t>(layer) * p.v_layer_stride_bytes;
        const uint8_t* vs = Q8_VALUES ? p.vn_base + static_cast<int64_t>(layer) * p.vn_layer_stride_bytes : nullptr;
        const int kps = p.addr.page_size, vps = p.addr_v.page_size;
        const int kfirst = t0 / kps, kseg = (t0 + ntok - 1) / kps - kfirst + 1;
        const int vfirst = t0 / vps, vseg = (t0 + ntok - 1) / vps - vfirst + 1;
        wait_free();
        if (lane == 0) {   // scale copies are rounded up to 16 bytes per page segment of the q8_0 side
            uint32_t bytes = static_cast<uint32_t>(ntok) * (kKRowBytes + kVRowBytes);
            const int ps = Q8_KEYS ? kps : vps, first = Q8_KEYS ? kfirst : vfirst, nseg = Q8_KEYS ? kseg : vseg;
            for (int i = 0; i < nseg; ++i) {
                const int tb = max(t0, (first + i) * ps), te = min(t0 + ntok, (first + i + 1) * ps);
                bytes += (static_cast<uint32_t>(te - tb) * 8u + 15u) & ~15u;
            }
            mbar_arrive_expect_tx(bar, bytes);
        }
        __syncwarp();
        for (int c = lane; c < 2 * (kseg + vseg); c += 32) {
            const bool value_side = c >= 2 * kseg;
            const int i = value_side ? c - 2 * kseg : c, kind = i & 1, sgi = i >> 1;
            const int ps = value_side ? vps : kps, first = value_side ? vfirst : kfirst;
            const int tb = max(t0, (first + sgi) * ps), te = min(t0 + ntok, (first + sgi + 1) * ps);
            const uint32_t rows = static_cast<uint32_t>(te - tb);
            const int64_t row = row_index(value_side ? p.addr_v : p.addr, seq, head, tb);
            if (!value_side) {
                if (kind == 0) bulk_g2s(stage + (tb - t0) * kKRowBytes, kr + row * kKRowBytes, rows * kKRowBytes, bar);
                else if constexpr (Q8_KEYS) bulk_g2s(stage + kOffKs + (tb - t0) * 8, ks + row * 8, (rows * 8 + 15u) & ~15u, bar);
            } else {
                if (kind == 0) bulk_g2s(stage + kOffV + (tb - t0) * kVRowBytes, vr + row * kVRowBytes, rows * kVRowBytes, bar);
                else if constexpr (Q8_VALUES) bulk_g2s(stage + kOffVs + (tb - t0) * 8, vs + row * 8, (rows * 8 + 15u) & ~15u, bar);
            }
        }
    }

    __device__ static void load_q(const DecodeParams& p, State& st, const float* qrow, const float2* cs, uint8_t*, int, int lane, int) {
        Q8::load_q_fragments(p, st, qrow, cs, lane);
    }

    __device__ static void process_unit(const DecodeParams& p, const uint8_t* stage, int unit, int nvalid, State& st, float*,
                                        const uint8_t*, int lane) {
        const uint32_t sbase = smem_u32(stage);
        float s[4], pr[4];
        if constexpr (Q8_KEYS) Q8::unit_scores(p, sbase, sbase + kOffKs, unit, nvalid, st, lane, s);
        else dense_unit_scores<kPacked>(p, sbase, unit, nvalid, st, lane, s);
        mma_softmax_step(st, s, pr);
        if constexpr (Q8_VALUES) Q8::unit_values(st, sbase + kOffV, sbase + kOffVs, unit, nvalid, pr, lane);
        else dense_unit_values<kPacked>(st, sbase + kOffV, unit, nvalid, pr, lane);
    }
};

}  // namespace er
