// TurboQuant storage policy of the persistent flash-decode kernel with both contractions on the tensor cores
// (mma.sync m16n8k16, fp16 operands, fp32 accumulate); staging by TurboStaging.  The math of
// gqa_attention_turboquant_decode (Shaders/TurboQuant.metal:1794-2001) as two small GEMMs per 16-token unit:
//   S[token][head]  = K~[token][dim] . qR[head][dim]      A = centroid pairs looked up from the code stream, B = qR
//   O^T[dim][head] += V~^T[dim][token] . P^T[token][head]  A = transposed centroid pairs, B = transposed (p_t * vNorm_t)
// Row, column and contraction indices of an mma are only labels, so they are assigned to suit the code stream:
//
// Scores.  Thread (g = lane / 4, c = lane % 4) reads, of the two tokens behind S rows g and g + 8, the 32 consecutive codes
// [32c, 32c + 32) (4 * bits bytes).  A lookup of a code PAIR (two adjacent dims of one token) returns the A-fragment
// registers directly (hi parts, lo parts); k-step s: label 2c + e -> dim 32c + 4s + e, label 2c + 8 + e -> dim
// 32c + 4s + 2 + e (e = 0, 1).  Queries enter as fp16 hi + lo B fragments: S = Kh.qh + Kh.ql + Kl.qh (8 heads per kv head).
// Up to 4 heads per kv head (kPacked) the hi parts of the queries take columns 0..3 of the n-tile and the lo parts columns
// 4..7, and rows g + 8 of the A fragment carry the lo parts of the token in row g: the two registers a table read returns
// are adjacent A registers as they come, an mma covers 8 tokens x 16 dims x (hi, lo) of both operands, and
// S = (Kh + Kl).(qh + ql) is the sum of an accumulator's rows g and g + 8 and of columns n and n + 4 (lanes c and c ^ 2).
//
// Outputs.  The contraction runs over tokens, and a code stream never yields two tokens of one dim.  So the value table is
// indexed by a SINGLE code and returns half2(hi, lo) of its centroid: the two halves sit on adjacent contraction labels
// (2c, 2c + 1) and the probability of that token is duplicated on both, which makes one mma.k16 cover 8 tokens with
// fp32-accurate values: O^T += [Vh | Vl] . [p ; p].  Thread (g, c) owns dims [16g, 16g + 16) (m-tile mt: row g -> dim
// 16g + 2mt, row g + 8 -> dim 16g + 2mt + 1) of tokens 2c, 2c + 1, 2c + 8, 2c + 9, a contiguous 2 * bits bytes per token: the
// tokens movmatrix.trans of the S fragment (rows g, g + 8) hands thread (g', c') -- rows 2c', 2c' + 1 and 2c' + 8, 2c' + 9.
// The probabilities enter as hi + lo too: two B fragments (8 heads), or one with the hi parts in columns 0..3 and the lo
// parts in columns 4..7 (kPacked; the two column halves of O^T are added when the state is folded or published).
//
// Queries, probabilities and all centroids therefore carry ~22 significant bits (fp16 hi + lo), which keeps the outputs
// within the element-wise 2e-3 bound of the fp32 CPU statement.  Tables hold sigma * centroid with a per-codebook sigma
// (tq_fp16_scales.h) that minimises the hi parts' rounding; 1 / sigma is folded into the softmax scale and the value norms.
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

// Shared-memory plan of the TurboQuant policy.  The CTA takes the whole 227 KB.  The key table sits on a 64 KB boundary of the
// shared window so that the address of an entry is ONE instruction away from the code word: for 4-bit keys the index of
// a code pair is a byte of the word, and prmt drops it into byte 1 of (table | lane << 3); 3-bit pairs need a shift and one
// logic op.  Everything the kernel itself lays out (stages, merge buffers, ...) lies below that boundary, the value table
// and the query / output staging rows above the table.
struct TurboSmemPlan {
    uint32_t lut_k;    // window address of the key table, 64 KB aligned
    uint32_t lut_v;    // window address of the value table (16 KB aligned), right behind the key table
    uint32_t rows;     // window address of the rotated-query and output staging rows
};

template <int GROUP, int KBITS, int VBITS, int UNITS_PER_TILE = 6, int WARP_GROUPS = 2, int STAGES = 4>
struct TurboMmaPolicy : TurboStaging<GROUP, KBITS, VBITS, UNITS_PER_TILE, WARP_GROUPS, STAGES> {
    using Base = TurboStaging<GROUP, KBITS, VBITS, UNITS_PER_TILE, WARP_GROUPS, STAGES>;
    static_assert(GROUP <= 8, "one n-tile of heads");
    static constexpr int kKPairs = 1 << (2 * KBITS);
    // Up to four heads leave half of the n-tile's eight columns free: the hi parts of the queries (and of the probabilities)
    // take columns 0..3 and the lo parts columns 4..7, so ONE mma multiplies an A fragment by both; the two column halves
    // are added across lanes c and c ^ 2 (scores: per unit; outputs: when the accumulators are folded or published).
    static constexpr bool kPacked = GROUP <= 4;
    // Lookup tables, one column per lane (no bank conflicts), 8-byte entries:
    //   keys    [code pairs (dims d, d + 1 of a token)][32 lanes]: half2 (hi parts of the two centroids), half2 (lo parts)
    //   values  3-bit: [code pairs][32 lanes]: half2 (hi, lo) of dim d, half2 (hi, lo) of dim d + 1 -- the two A registers of an
    //           output m-tile.  4-bit values with 4-bit keys read the key table (same codebook) and re-pair the halves with two
    //           prmt; 4-bit values with 3-bit keys keep a table of their own.
    static constexpr bool kVSharesK = (VBITS == KBITS);
    static constexpr int kVPairs = 1 << (2 * VBITS);
    static constexpr int kLutKBytes = kKPairs * 256;                       // 64 KB for 4-bit keys, 16 KB for 3-bit
    static constexpr int kLutVBytes = kVSharesK ? 0 : kVPairs * 256;
    static constexpr bool kValuesFirst = kLutVBytes > kLutKBytes;          // the 64 KB table takes the 64 KB boundary
    static constexpr int kExtraBytes = -1;                                 // DecodeSmem: the kernel takes the CTA maximum

    __device__ __forceinline__ static TurboSmemPlan plan(const uint8_t* extra) {
        TurboSmemPlan pl;
        const uint32_t first = (smem_u32(extra) + 65535u) & ~65535u;
        pl.lut_k = kValuesFirst ? first + kLutVBytes : first;
        pl.lut_v = kVSharesK ? pl.lut_k : (kValuesFirst ? first : first + kLutKBytes);
        pl.rows = first + kLutKBytes + kLutVBytes;
        return pl;
    }
    // generic pointer to a window address at or above `extra`
    __device__ __forceinline__ static float* window_ptr(uint8_t* extra, uint32_t addr) {
        return reinterpret_cast<float*>(extra + (addr - smem_u32(extra)));
    }
    __device__ __forceinline__ static float* fin_ptr(uint8_t* extra) { return window_ptr(extra, plan(extra).rows + GROUP * kHeadDim * 4); }

    struct State {
        uint32_t qh[8][2], ql[8][2];   // B fragments of the rotated queries per k-step: fp16 hi and lo parts (packed: qh holds both)
        float m[2], l[2];              // heads 2c, 2c + 1
        float acc[8][4];               // O^T fragments: [m-tile][(row g | row g + 8) x (head 2c | 2c + 1)]
        uint32_t lut_k, lut_v;         // this lane's column of the tables: table address | lane << 3
        __device__ __forceinline__ void reset() {
            m[0] = m[1] = -INFINITY;
            l[0] = l[1] = 0.f;
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;
        }
        // packed columns: V . P_hi (lanes c < 2) + V . P_lo (lanes c >= 2) of the same heads
        __device__ __forceinline__ void gather() {
            if constexpr (kPacked) {
#pragma unroll
                for (int t = 0; t < 8; ++t)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[t][e] += __shfl_xor_sync(0xffffffffu, acc[t][e], 2);
            }
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {   // denominators: per-lane partial sums over the lane's tokens
                l[0] += __shfl_xor_sync(0xffffffffu, l[0], off);
                l[1] += __shfl_xor_sync(0xffffffffu, l[1], off);
            }
        }
        __device__ __forceinline__ void publish(float* ml, float* accs, int lane) {
            const int g = lane >> 2, c = lane & 3;
            gather();
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int h = 2 * c + e;
                if (h < GROUP) {
                    if (g == 0) {
                        ml[h * 2] = m[e];
                        ml[h * 2 + 1] = l[e];
                    }
#pragma unroll
                    for (int t = 0; t < 8; ++t)   // m-tile t: row g -> dim 16g + 2t, row g + 8 -> dim 16g + 2t + 1
                        *reinterpret_cast<float2*>(accs + h * kHeadDim + 16 * g + 2 * t) = make_float2(acc[t][e], acc[t][2 + e]);
                }
            }
        }
        __device__ __forceinline__ void fold(float* ml, float* accs, int lane, bool first) {
            gather();
            mma_state_fold<GROUP>(m, l, acc, ml, accs, lane, first, 1.f, 1.f, [](int t, int g, int second) { return 16 * g + 2 * t + second; });
        }
    };
    static constexpr int kFoldUnits = 32;   // chains of about 128 accumulating mma per output fragment

    // false when the plan does not fit the CTA's shared memory (the window base is not where this layout expects it)
    __device__ static bool init_extra(uint8_t* extra, int tid, int smem_bytes_after_extra) {
        const TurboSmemPlan pl = plan(extra);
        if (pl.rows + 2u * GROUP * kHeadDim * 4u > smem_u32(extra) + static_cast<uint32_t>(smem_bytes_after_extra)) return false;
        for (int e = tid; e < kKPairs * 32; e += Base::kThreads) {
            const int pv = e >> 5;
            const float c0 = __fmul_rn(tq_centroids<KBITS>()[pv & ((1 << KBITS) - 1)], tq_fp16_scale<KBITS>());
            const float c1 = __fmul_rn(tq_centroids<KBITS>()[pv >> KBITS], tq_fp16_scale<KBITS>());
            const __half2 hi = __floats2half2_rn(c0, c1);
            const float2 hf = __half22float2(hi);
            asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(pl.lut_k + 8 * e), "r"(*reinterpret_cast<const uint32_t*>(&hi)),
                         "r"(pack_half2(c0 - hf.x, c1 - hf.y))
                         : "memory");
        }
        if constexpr (!kVSharesK) {
            for (int e = tid; e < kVPairs * 32; e += Base::kThreads) {
                const int pv = e >> 5;
                const float c0 = __fmul_rn(tq_centroids<VBITS>()[pv & ((1 << VBITS) - 1)], tq_fp16_scale<VBITS>());
                const float c1 = __fmul_rn(tq_centroids<VBITS>()[pv >> VBITS], tq_fp16_scale<VBITS>());
                const float h0 = __half2float(__float2half_rn(c0)), h1 = __half2float(__float2half_rn(c1));
                asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(pl.lut_v + 8 * e), "r"(pack_half2(h0, c0 - h0)), "r"(pack_half2(h1, c1 - h1))
                             : "memory");
            }
        }
        return true;
    }

    __device__ static void load_q(const DecodeParams& p, State& st, const float* qrow, const float2* cs, uint8_t* extra,
                                  int warp, int lane, int) {
        const TurboSmemPlan pl = plan(extra);
        float* qrot = window_ptr(extra, pl.rows);
        Base::rotate_queries(p, qrot, qrow, cs, warp, lane);
        st.lut_k = pl.lut_k | (lane << 3);
        st.lut_v = pl.lut_v | (lane << 3);
        const int g = lane >> 2, c = lane & 3;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            const int head = kPacked ? (g & 3) : g;   // packed: column g carries head g % 4, hi part below column 4
            if (head < GROUP) t = *reinterpret_cast<const float4*>(qrot + head * kHeadDim + 32 * c + 4 * s);
            const __half2 h01 = __floats2half2_rn(t.x, t.y), h23 = __floats2half2_rn(t.z, t.w);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            const uint32_t hi0 = *reinterpret_cast<const uint32_t*>(&h01), hi1 = *reinterpret_cast<const uint32_t*>(&h23);
            const uint32_t lo0 = pack_half2(t.x - f01.x, t.y - f01.y), lo1 = pack_half2(t.z - f23.x, t.w - f23.y);
            if constexpr (kPacked) {
                st.qh[s][0] = g < 4 ? hi0 : lo0;
                st.qh[s][1] = g < 4 ? hi1 : lo1;
            } else {
                st.qh[s][0] = hi0;
                st.qh[s][1] = hi1;
                st.ql[s][0] = lo0;
                st.ql[s][1] = lo1;
            }
        }
        st.reset();
    }

    // Address of the key-table entry of code pair PI (dims 2 PI, 2 PI + 1 of the lane's 32-code chunk).
    template <int PI>
    __device__ __forceinline__ static uint32_t key_entry(const uint32_t (&w)[KBITS], uint32_t lut) {
        if constexpr (KBITS == 4) {
            return __byte_perm(w[PI >> 2], lut, 0x7604 | ((PI & 3) << 4));   // byte PI of the chunk -> byte 1 of the address
        } else {
            constexpr int bit = PI * 2 * KBITS, word = bit >> 5, sh = bit & 31;
            constexpr uint32_t mask = static_cast<uint32_t>(kKPairs - 1) << 8;
            uint32_t v;
            if constexpr (sh + 2 * KBITS > 32) v = __funnelshift_r(w[word], w[word + 1], sh - 8);
            else if constexpr (sh >= 8) v = w[word] >> (sh - 8);
            else v = w[word] << (8 - sh);
            return (v & mask) | lut;
        }
    }

    template <int S>
    __device__ __forceinline__ static void score_steps(float (&s)[4], const uint32_t (&k0)[KBITS], const uint32_t (&k1)[KBITS],
                                                       const State& st) {
        if constexpr (S < 8) {
            uint32_t a0, a1, a2, a3, e0, e1, e2, e3;
            lds_u32x2(key_entry<2 * S>(k0, st.lut_k), a0, e0);
            lds_u32x2(key_entry<2 * S>(k1, st.lut_k), a1, e1);
            lds_u32x2(key_entry<2 * S + 1>(k0, st.lut_k), a2, e2);
            lds_u32x2(key_entry<2 * S + 1>(k1, st.lut_k), a3, e3);
            mma_m16n8k16(s, a0, a1, a2, a3, st.qh[S][0], st.qh[S][1]);
            mma_m16n8k16(s, a0, a1, a2, a3, st.ql[S][0], st.ql[S][1]);
            mma_m16n8k16(s, e0, e1, e2, e3, st.qh[S][0], st.qh[S][1]);
            score_steps<S + 1>(s, k0, k1, st);
        }
    }

    // Packed form (kPacked).  Rows g + 8 of the A fragment carry the LO parts of the token whose hi parts sit in row g, so the
    // two registers a table read returns (hi pair, lo pair) are two adjacent A registers as they come, and an mma covers 8
    // tokens: sa takes tokens 0..7 of the unit, sb tokens 8..15; row g of an accumulator holds Kh . q, row g + 8 Kl . q.
    template <int S>
    __device__ __forceinline__ static void score_steps_packed(float (&sa)[4], float (&sb)[4], const uint32_t (&k0)[KBITS],
                                                              const uint32_t (&k1)[KBITS], const State& st) {
        if constexpr (S < 8) {
            uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
            lds_u32x2(key_entry<2 * S>(k0, st.lut_k), a0, a1);
            lds_u32x2(key_entry<2 * S + 1>(k0, st.lut_k), a2, a3);
            lds_u32x2(key_entry<2 * S>(k1, st.lut_k), b0, b1);
            lds_u32x2(key_entry<2 * S + 1>(k1, st.lut_k), b2, b3);
            mma_m16n8k16(sa, a0, a1, a2, a3, st.qh[S][0], st.qh[S][1]);
            mma_m16n8k16(sb, b0, b1, b2, b3, st.qh[S][0], st.qh[S][1]);
            score_steps_packed<S + 1>(sa, sb, k0, k1, st);
        }
    }

    // The two A registers of output m-tile T for one token: half2 (hi, lo) of dims 16g + 2T and 16g + 2T + 1, looked up by the
    // code pair T of the token's 16-code chunk (lo: bits 0..31, hi: the rest).
    template <int T>
    __device__ __forceinline__ static void value_pair(uint32_t lut, uint32_t lo, uint32_t hi, uint32_t& a_even, uint32_t& a_odd) {
        uint32_t addr;
        if constexpr (VBITS == 4) {
            addr = __byte_perm(T < 4 ? lo : hi, lut, 0x7604 | ((T & 3) << 4));
        } else {
            constexpr int bit = T * 2 * VBITS;
            constexpr uint32_t mask = static_cast<uint32_t>(kVPairs - 1) << 8;
            uint32_t v;
            if constexpr (bit < 32 && bit + 2 * VBITS > 32) v = __funnelshift_r(lo, hi, bit - 8);
            else if constexpr (bit >= 32) { if constexpr (bit - 32 >= 8) v = hi >> (bit - 32 - 8); else v = hi << (8 - (bit - 32)); }
            else if constexpr (bit >= 8) v = lo >> (bit - 8);
            else v = lo << (8 - bit);
            addr = (v & mask) | lut;
        }
        uint32_t x, y;
        lds_u32x2(addr, x, y);
        if constexpr (kVSharesK) {   // key-table layout (hi, hi), (lo, lo) -> (hi, lo) per dim
            a_even = __byte_perm(x, y, 0x5410);
            a_odd = __byte_perm(x, y, 0x7632);
        } else {
            a_even = x;
            a_odd = y;
        }
    }

    // m-tile T of O^T: dims 16g + 2T (row g) and 16g + 2T + 1 (row g + 8), both k-steps (tokens 2c, 2c + 1 | 2c + 8, 2c + 9).
    template <int T>
    __device__ __forceinline__ static void value_tiles(State& st, const uint32_t (&vlo)[4], const uint32_t (&vhi)[4],
                                                       const uint32_t (&bh)[4], const uint32_t (&bl)[4]) {
        if constexpr (T < 8) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t a0, a1, a2, a3;
                value_pair<T>(st.lut_v, vlo[2 * j], vhi[2 * j], a0, a1);
                value_pair<T>(st.lut_v, vlo[2 * j + 1], vhi[2 * j + 1], a2, a3);
                mma_m16n8k16(st.acc[T], a0, a1, a2, a3, bh[2 * j], bh[2 * j + 1]);
                if constexpr (!kPacked) mma_m16n8k16(st.acc[T], a0, a1, a2, a3, bl[2 * j], bl[2 * j + 1]);
            }
            value_tiles<T + 1>(st, vlo, vhi, bh, bl);
        }
    }

    __device__ static void process_unit(const DecodeParams& p, const uint8_t* stage, int unit, int nvalid, State& st, float*,
                                        const uint8_t* extra, int lane) {
        const int g = lane >> 2, c = lane & 3;
        const int tk0 = g;                          // token behind S row g (row g + 8: g + 8)
        const uint32_t sbase = smem_u32(stage);
        const uint32_t kc = sbase + ((unit * kUnitTokens + tk0) * Base::kKW + c * KBITS) * 4;
        uint32_t k0[KBITS], k1[KBITS], vlo[4], vhi[4];
        load_code_chunk<KBITS>(kc, k0);
        load_code_chunk<KBITS>(kc + 32 * Base::kKW, k1);
        // value codes: dims [16g, 16g + 16) of tokens 2c, 2c + 1, 2c + 8, 2c + 9 -- 2 * VBITS bytes at byte 2 * VBITS * g of the row
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t row = sbase + Base::kKcBytes + (unit * kUnitTokens + 2 * c + (j & 1) + 8 * (j >> 1)) * Base::kVW * 4;
            if constexpr (VBITS == 4) {
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(vlo[j]), "=r"(vhi[j]) : "r"(row + 8 * g) : "memory");
            } else if constexpr (VBITS == 3) {
                // 6 bytes at offset 6g: the two aligned words around them, shifted by 16 bits for odd g
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
        const bool ok0 = tk0 < nvalid, ok1 = tk0 + 8 < nvalid;
        const int r0 = unit * kUnitTokens + tk0;
        const float kn0 = ok0 ? Base::load_norm(stage + Base::kOffKn, r0, p.norm_fp16) : 0.f;
        const float kn1 = ok1 ? Base::load_norm(stage + Base::kOffKn, r0 + 8, p.norm_fp16) : 0.f;
        constexpr float inv_sk = 1.f / tq_fp16_scale<KBITS>(), inv_sv = 1.f / tq_fp16_scale<VBITS>();
        const float vn0 = ok0 ? Base::load_norm(stage + Base::kOffVn, r0, p.norm_fp16) * inv_sv : 0.f;
        const float vn1 = ok1 ? Base::load_norm(stage + Base::kOffVn, r0 + 8, p.norm_fp16) * inv_sv : 0.f;
        const float sc = p.scale_log2 * inv_sk;

        float s[4] = {0.f, 0.f, 0.f, 0.f};   // (token tk0 | tk0 + 8) x (head 2c | 2c + 1)
        if constexpr (kPacked) {
            float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
            score_steps_packed<0>(sa, sb, k0, k1, st);
            s[0] = sa[0] + sa[2];   // Kh . q + Kl . q of token g
            s[1] = sa[1] + sa[3];
            s[2] = sb[0] + sb[2];   // of token g + 8
            s[3] = sb[1] + sb[3];
#pragma unroll
            for (int i = 0; i < 4; ++i) s[i] += __shfl_xor_sync(0xffffffffu, s[i], 2);   // columns 2c, 2c + 1 (q hi) + their partners four on (q lo)
        } else {
            score_steps<0>(s, k0, k1, st);
        }
        s[0] = ok0 ? (kn0 * s[0]) * sc : -INFINITY;
        s[1] = ok0 ? (kn0 * s[1]) * sc : -INFINITY;
        s[2] = ok1 ? (kn1 * s[2]) * sc : -INFINITY;
        s[3] = ok1 ? (kn1 * s[3]) * sc : -INFINITY;

        // The running maxima change only when some token of the unit exceeds them (always in a fresh state: token 0 of a unit
        // is valid, its score finite): the cross-lane maximum and the rescale run only then.  The denominators stay per-lane
        // partial sums (every lane applies the same corrections); State::gather adds them up when the state is read.
        float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
        float m0 = st.m[0], m1 = st.m[1];
        if (__any_sync(0xffffffffu, mx0 > m0 || mx1 > m1)) {
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
            }
            m0 = fmaxf(m0, mx0);
            m1 = fmaxf(m1, mx1);
            const float corr0 = fast_exp2(st.m[0] - m0), corr1 = fast_exp2(st.m[1] - m1);
            st.l[0] *= corr0;
            st.l[1] *= corr1;
            st.m[0] = m0;
            st.m[1] = m1;
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                st.acc[t][0] *= corr0; st.acc[t][1] *= corr1; st.acc[t][2] *= corr0; st.acc[t][3] *= corr1;
            }
        }
        const float p0 = fast_exp2(s[0] - m0), p1 = fast_exp2(s[1] - m1), p2 = fast_exp2(s[2] - m0), p3 = fast_exp2(s[3] - m1);
        st.l[0] += p0 + p2;
        st.l[1] += p1 + p3;
        // (p_t * vNorm_t)[token][head] as fp16 hi + lo parts, transposed: thread (g', c') receives head g' of tokens 2c', 2c' + 1
        // and, from the rows g + 8, of 2c' + 8, 2c' + 9; each value is duplicated on the two
        // contraction labels that carry the hi and the lo half of a centroid
        const float w0 = p0 * vn0, w1 = p1 * vn0, w2 = p2 * vn1, w3 = p3 * vn1;
        const __half2 h01 = __floats2half2_rn(w0, w1), h23 = __floats2half2_rn(w2, w3);
        const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
        const uint32_t hi01 = *reinterpret_cast<const uint32_t*>(&h01), hi23 = *reinterpret_cast<const uint32_t*>(&h23);
        const uint32_t lo01 = pack_half2(w0 - f01.x, w1 - f01.y), lo23 = pack_half2(w2 - f23.x, w3 - f23.y);
        if constexpr (kPacked) {
            // lanes c and c ^ 2 hold the same probabilities: the first pair supplies the hi parts (columns 0..3), the second the lo parts
            const uint32_t x0 = movmatrix_trans(c < 2 ? hi01 : lo01);
            const uint32_t x1 = movmatrix_trans(c < 2 ? hi23 : lo23);
            const uint32_t bh[4] = {__byte_perm(x0, x0, 0x1010), __byte_perm(x0, x0, 0x3232), __byte_perm(x1, x1, 0x1010), __byte_perm(x1, x1, 0x3232)};
            value_tiles<0>(st, vlo, vhi, bh, bh);
        } else {
            const uint32_t x0 = movmatrix_trans(hi01), x1 = movmatrix_trans(hi23);
            const uint32_t y0 = movmatrix_trans(lo01), y1 = movmatrix_trans(lo23);
            const uint32_t bh[4] = {__byte_perm(x0, x0, 0x1010), __byte_perm(x0, x0, 0x3232), __byte_perm(x1, x1, 0x1010), __byte_perm(x1, x1, 0x3232)};
            const uint32_t bl[4] = {__byte_perm(y0, y0, 0x1010), __byte_perm(y0, y0, 0x3232), __byte_perm(y1, y1, 0x1010), __byte_perm(y1, y1, 0x3232)};
            value_tiles<0>(st, vlo, vhi, bh, bl);
        }
    }
};

}  // namespace er
