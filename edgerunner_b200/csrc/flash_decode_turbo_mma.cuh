// TurboQuant storage policy of the persistent flash-decode kernel with both contractions on the tensor cores
// (mma.sync m16n8k16, fp16 operands, fp32 accumulate); staging by TurboStaging.  The math of
// gqa_attention_turboquant_decode (Shaders/TurboQuant.metal:1794-2001) as two small GEMMs per 16-token unit:
//   S[token][head]  = K~[token][dim] . qR[head][dim]      A = centroid pairs looked up from the code stream, B = qR
//   O^T[dim][head] += V~^T[dim][token] . P^T[token][head]  A = transposed centroid pairs, B = transposed (p_t * vNorm_t)
// A code stream yields two adjacent *dims* of one token per lookup (one half2 register).  That is an A fragment when
// the contraction runs over dims (scores); for the P.V product the contraction runs over tokens, so every looked-up
// 8x8 block passes through movmatrix.trans first.
//
// Thread (g = lane / 4, c = lane % 4) reads tokens g and g + 8 of the warp's 16-token unit, and of each row the 32
// consecutive codes [32c, 32c + 32) (4 * bits bytes).  The contraction index of an mma is only a label, so the labels
// are assigned to make that chunk contiguous:
//   scores, k-step s:   label 2c + e -> dim 32c + 4s + e,     label 2c + 8 + e -> dim 32c + 4s + 2 + e      (e = 0, 1)
//   outputs, m-tile mt: row n        -> dim 32(n/2) + 4mt + n%2,   row n + 8   -> dim 32(n/2) + 4mt + 2 + n%2
// Queries, probabilities and the keys' centroids enter as fp16 hi + lo pairs (scores: qh.ch + ql.ch + qh.cl); the values'
// centroids as one fp16.  All tables hold sigma * centroid with a per-codebook sigma chosen so that every centroid
// rounds to fp16 with < 6e-5 relative error (tq_fp16_scales.h); 1 / sigma is folded into the softmax scale and the
// value norms.
#pragma once

#include "flash_decode_turbo.cuh"
#include "tq_fp16_scales.h"

namespace er {

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 8x8 matrix of 16-bit elements held one row per four lanes (lane holds row lane/4, columns 2(lane%4), +1) -> its transpose
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Shared-memory reads by 32-bit window address (the generic-pointer form costs 64-bit address arithmetic per read).
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void lds_u32x2(uint32_t addr, uint32_t& x, uint32_t& y) {
    asm("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(x), "=r"(y) : "r"(addr));
}
// fresh data of the stage ring: volatile so that a read is never hoisted above the wait on the stage's barrier
__device__ __forceinline__ uint32_t lds_u32_stage(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

// 32 codes of BITS bits = BITS words
template <int BITS>
__device__ __forceinline__ void load_code_chunk(uint32_t addr, uint32_t (&w)[BITS]) {
    if constexpr (BITS == 4) {
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr) : "memory");
    } else if constexpr (BITS == 2) {
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "r"(addr) : "memory");
    } else {
#pragma unroll
        for (int i = 0; i < BITS; ++i) w[i] = lds_u32_stage(addr + 4 * i);
    }
}

// Byte offset of pair `PI` (codes 2 PI, 2 PI + 1) of the chunk in a table of (1 << LOG2_ENTRY)-byte entries.
template <int BITS, int PI, int LOG2_ENTRY>
__device__ __forceinline__ uint32_t pair_offset(const uint32_t (&w)[BITS]) {
    constexpr int bit = PI * 2 * BITS, word = bit >> 5, sh = bit & 31;
    constexpr uint32_t mask = ((1u << (2 * BITS)) - 1u) << LOG2_ENTRY;
    uint32_t v;
    if constexpr (sh + 2 * BITS > 32) v = __funnelshift_r(w[word], w[word + 1], sh - LOG2_ENTRY);
    else if constexpr (sh >= LOG2_ENTRY) v = w[word] >> (sh - LOG2_ENTRY);
    else v = w[word] << (LOG2_ENTRY - sh);
    return v & mask;
}

template <int BITS>
__host__ __device__ constexpr float tq_fp16_scale() {
    return BITS == 2 ? ER_TQ_FP16_SCALE_2BIT : BITS == 3 ? ER_TQ_FP16_SCALE_3BIT : ER_TQ_FP16_SCALE_4BIT;
}

template <int GROUP, int KBITS, int VBITS, int UNITS_PER_TILE = 6, int WARP_GROUPS = 2, int STAGES = 4>
struct TurboMmaPolicy : TurboStaging<GROUP, KBITS, VBITS, UNITS_PER_TILE, WARP_GROUPS, STAGES> {
    using Base = TurboStaging<GROUP, KBITS, VBITS, UNITS_PER_TILE, WARP_GROUPS, STAGES>;
    static_assert(GROUP <= 8, "one n-tile of heads");
    static constexpr int kKPairs = 1 << (2 * KBITS), kVPairs = 1 << (2 * VBITS);
    // Lookup tables indexed by a pair of codes, one column per lane (no bank conflicts):
    //   keys    [pairs][32 lanes] x 8 bytes: half2 (hi parts of the two centroids), half2 (lo parts); scores pass through
    //           exp2, so the keys' centroids keep their fp16 rounding residue as a second operand
    //   values  [pairs][32 lanes] x 4 bytes: half2 of the two centroids
    static constexpr int kOffQrot = 0;
    static constexpr int kOffFin = GROUP * kHeadDim * 4;
    static constexpr int kOffLutK = 2 * GROUP * kHeadDim * 4;
    static constexpr int kOffLutV = kOffLutK + kKPairs * 256;
    static constexpr int kExtraBytes = kOffLutV + kVPairs * 128;

    struct State {
        uint32_t qh[8][2], ql[8][2];   // B fragments of the rotated queries per k-step: fp16 hi and lo parts
        float m[2], l[2];              // heads 2c, 2c + 1
        float acc[8][4];               // O^T fragments: [m-tile][(row g | row g + 8) x (head 2c | 2c + 1)]
        __device__ __forceinline__ void reset() {
            m[0] = m[1] = -INFINITY;
            l[0] = l[1] = 0.f;
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;
        }
        __device__ __forceinline__ void publish(float* ml, float* accs, int lane) const {
            const int g = lane >> 2, c = lane & 3;
            const int d0 = 32 * (g >> 1) + (g & 1);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int h = 2 * c + e;
                if (h < GROUP) {
                    if (g == 0) {
                        ml[h * 2] = m[e];
                        ml[h * 2 + 1] = l[e];
                    }
#pragma unroll
                    for (int t = 0; t < 8; ++t) {
                        accs[h * kHeadDim + d0 + 4 * t] = acc[t][e];
                        accs[h * kHeadDim + d0 + 4 * t + 2] = acc[t][2 + e];
                    }
                }
            }
        }
    };

    __device__ static void init_extra(uint8_t* extra, int tid) {
        const uint32_t lk = smem_u32(extra) + kOffLutK, lv = smem_u32(extra) + kOffLutV;
        for (int e = tid; e < kKPairs * 32; e += Base::kThreads) {
            const int pv = e >> 5;
            const float c0 = __fmul_rn(tq_centroids<KBITS>()[pv & ((1 << KBITS) - 1)], tq_fp16_scale<KBITS>());
            const float c1 = __fmul_rn(tq_centroids<KBITS>()[pv >> KBITS], tq_fp16_scale<KBITS>());
            const __half2 hi = __floats2half2_rn(c0, c1);
            const float2 hf = __half22float2(hi);
            asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(lk + 8 * e), "r"(*reinterpret_cast<const uint32_t*>(&hi)),
                         "r"(pack_half2(c0 - hf.x, c1 - hf.y))
                         : "memory");
        }
        for (int e = tid; e < kVPairs * 32; e += Base::kThreads) {
            const int pv = e >> 5;
            const uint32_t v = pack_half2(__fmul_rn(tq_centroids<VBITS>()[pv & ((1 << VBITS) - 1)], tq_fp16_scale<VBITS>()),
                                          __fmul_rn(tq_centroids<VBITS>()[pv >> VBITS], tq_fp16_scale<VBITS>()));
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(lv + 4 * e), "r"(v) : "memory");
        }
    }

    __device__ static void load_q(const DecodeParams& p, State& st, const float* qrow, const float2* cs, uint8_t* extra,
                                  int warp, int lane, int) {
        float* qrot = reinterpret_cast<float*>(extra + kOffQrot);
        Base::rotate_queries(p, qrot, qrow, cs, warp, lane);
        const int g = lane >> 2, c = lane & 3;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            if (g < GROUP) t = *reinterpret_cast<const float4*>(qrot + g * kHeadDim + 32 * c + 4 * s);
            const __half2 h01 = __floats2half2_rn(t.x, t.y), h23 = __floats2half2_rn(t.z, t.w);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            st.qh[s][0] = *reinterpret_cast<const uint32_t*>(&h01);
            st.qh[s][1] = *reinterpret_cast<const uint32_t*>(&h23);
            st.ql[s][0] = pack_half2(t.x - f01.x, t.y - f01.y);
            st.ql[s][1] = pack_half2(t.z - f23.x, t.w - f23.y);
        }
        st.reset();
    }

    template <int S>
    __device__ __forceinline__ static void score_steps(float (&s)[4], uint32_t lutk, const uint32_t (&k0)[KBITS],
                                                       const uint32_t (&k1)[KBITS], const State& st) {
        if constexpr (S < 8) {
            uint32_t a0, a1, a2, a3, e0, e1, e2, e3;
            lds_u32x2(lutk + pair_offset<KBITS, 2 * S, 8>(k0), a0, e0);
            lds_u32x2(lutk + pair_offset<KBITS, 2 * S, 8>(k1), a1, e1);
            lds_u32x2(lutk + pair_offset<KBITS, 2 * S + 1, 8>(k0), a2, e2);
            lds_u32x2(lutk + pair_offset<KBITS, 2 * S + 1, 8>(k1), a3, e3);
            mma_m16n8k16(s, a0, a1, a2, a3, st.qh[S][0], st.qh[S][1]);
            mma_m16n8k16(s, a0, a1, a2, a3, st.ql[S][0], st.ql[S][1]);
            mma_m16n8k16(s, e0, e1, e2, e3, st.qh[S][0], st.qh[S][1]);
            score_steps<S + 1>(s, lutk, k0, k1, st);
        }
    }

    template <int T>
    __device__ __forceinline__ static void value_tiles(State& st, uint32_t lutv, const uint32_t (&v0)[VBITS],
                                                       const uint32_t (&v1)[VBITS], uint32_t b0, uint32_t b1, uint32_t b0l, uint32_t b1l) {
        if constexpr (T < 8) {
            const uint32_t a0 = movmatrix_trans(lds_u32(lutv + pair_offset<VBITS, 2 * T, 7>(v0)));
            const uint32_t a1 = movmatrix_trans(lds_u32(lutv + pair_offset<VBITS, 2 * T + 1, 7>(v0)));
            const uint32_t a2 = movmatrix_trans(lds_u32(lutv + pair_offset<VBITS, 2 * T, 7>(v1)));
            const uint32_t a3 = movmatrix_trans(lds_u32(lutv + pair_offset<VBITS, 2 * T + 1, 7>(v1)));
            mma_m16n8k16(st.acc[T], a0, a1, a2, a3, b0, b1);
            mma_m16n8k16(st.acc[T], a0, a1, a2, a3, b0l, b1l);
            value_tiles<T + 1>(st, lutv, v0, v1, b0, b1, b0l, b1l);
        }
    }

    __device__ static void process_unit(const DecodeParams& p, const uint8_t* stage, int unit, int nvalid, State& st, float*,
                                        const uint8_t* extra, int lane) {
        const uint32_t lutk = smem_u32(extra) + kOffLutK + 8 * lane, lutv = smem_u32(extra) + kOffLutV + 4 * lane;
        const int g = lane >> 2, c = lane & 3;
        const uint32_t sbase = smem_u32(stage);
        const uint32_t kc = sbase + ((unit * kUnitTokens + g) * Base::kKW + c * KBITS) * 4;
        const uint32_t vc = sbase + Base::kKcBytes + ((unit * kUnitTokens + g) * Base::kVW + c * VBITS) * 4;
        uint32_t k0[KBITS], k1[KBITS], v0[VBITS], v1[VBITS];
        load_code_chunk<KBITS>(kc, k0);
        load_code_chunk<KBITS>(kc + 32 * Base::kKW, k1);
        load_code_chunk<VBITS>(vc, v0);
        load_code_chunk<VBITS>(vc + 32 * Base::kVW, v1);
        const bool ok0 = g < nvalid, ok1 = g + 8 < nvalid;
        const int r0 = unit * kUnitTokens + g;
        const float kn0 = ok0 ? Base::load_norm(stage + Base::kOffKn, r0, p.norm_fp16) : 0.f;
        const float kn1 = ok1 ? Base::load_norm(stage + Base::kOffKn, r0 + 8, p.norm_fp16) : 0.f;
        constexpr float inv_sk = 1.f / tq_fp16_scale<KBITS>(), inv_sv = 1.f / tq_fp16_scale<VBITS>();
        const float vn0 = ok0 ? Base::load_norm(stage + Base::kOffVn, r0, p.norm_fp16) * inv_sv : 0.f;
        const float vn1 = ok1 ? Base::load_norm(stage + Base::kOffVn, r0 + 8, p.norm_fp16) * inv_sv : 0.f;
        const float sc = p.scale_log2 * inv_sk;

        float s[4] = {0.f, 0.f, 0.f, 0.f};   // (token g | g + 8) x (head 2c | 2c + 1)
        score_steps<0>(s, lutk, k0, k1, st);
        s[0] = ok0 ? (kn0 * s[0]) * sc : -INFINITY;
        s[1] = ok0 ? (kn0 * s[1]) * sc : -INFINITY;
        s[2] = ok1 ? (kn1 * s[2]) * sc : -INFINITY;
        s[3] = ok1 ? (kn1 * s[3]) * sc : -INFINITY;

        float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        const float m0 = fmaxf(st.m[0], mx0), m1 = fmaxf(st.m[1], mx1);   // finite: token 0 of the unit is valid
        const float corr0 = fast_exp2(st.m[0] - m0), corr1 = fast_exp2(st.m[1] - m1);
        const float p0 = fast_exp2(s[0] - m0), p1 = fast_exp2(s[1] - m1), p2 = fast_exp2(s[2] - m0), p3 = fast_exp2(s[3] - m1);
        float sum0 = p0 + p2, sum1 = p1 + p3;
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            sum0 += __shfl_xor_sync(0xffffffffu, sum0, off);
            sum1 += __shfl_xor_sync(0xffffffffu, sum1, off);
        }
        st.l[0] = fmaf(st.l[0], corr0, sum0);
        st.l[1] = fmaf(st.l[1], corr1, sum1);
        st.m[0] = m0;
        st.m[1] = m1;
        if (__any_sync(0xffffffffu, corr0 != 1.f || corr1 != 1.f)) {
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                st.acc[t][0] *= corr0; st.acc[t][1] *= corr1; st.acc[t][2] *= corr0; st.acc[t][3] *= corr1;
            }
        }
        // (p_t * vNorm_t)[token][head] blocks, as fp16 hi + lo parts -> B fragments [token pair][head]
        const float w0 = p0 * vn0, w1 = p1 * vn0, w2 = p2 * vn1, w3 = p3 * vn1;
        const __half2 h01 = __floats2half2_rn(w0, w1), h23 = __floats2half2_rn(w2, w3);
        const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
        const uint32_t b0 = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&h01));
        const uint32_t b1 = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&h23));
        const uint32_t b0l = movmatrix_trans(pack_half2(w0 - f01.x, w1 - f01.y));
        const uint32_t b1l = movmatrix_trans(pack_half2(w2 - f23.x, w3 - f23.y));
        value_tiles<0>(st, lutv, v0, v1, b0, b1, b0l, b1l);
    }
};

}  // namespace er
