// fp16 rows in the persistent flash-decode kernel with both contractions on the tensor cores (mma.sync m16n8k16, fp16
// operands, fp32 accumulate) -- the policy for large GQA groups, where the lane-owns-dims form of DensePolicy runs out of
// FMA issue slots (4 heads: 512 FMAs per lane and 16-token unit) and of registers (8 heads: 128 query registers).
// Same math as DensePolicy (gqa_attention_f16kv, Shaders/GQA.metal:278-387, one query row per sequence):
//   S[token][head]  = K[token][dim] . q[head][dim]           A = cached fp16 rows as they lie, B = q as fp16 hi + lo
//   O^T[dim][head] += V^T[dim][token] . P^T[token][head]      A = cached rows through movmatrix.trans, B = p as fp16 hi + lo
// K and V are exact in fp16; q and p enter as hi + lo pairs, so the products keep fp32 accuracy.  p (<= 1) is carried times
// 4096 so that the lo part of a small probability stays a normal fp16 number; the outputs are divided by 4096 when
// published.
//
// Staging, copies, the fused append and the ring / window handling are DensePolicy's (rows lie in shared memory as in the
// cache, 256 bytes each).  Thread (g = lane / 4, c = lane % 4) reads tokens g and g + 8 of the warp's 16-token unit and of
// each row the four 16-byte chunks 4j + c (dims [32j + 8c, 32j + 8c + 8)): a quarter warp reads two rows x 64 contiguous
// bytes per load.  The contraction index of an mma is only a label, so k-step 2j + u takes label 2c + e -> dim
// 32j + 8c + 4u + e and label 2c + 8 + e -> dim 32j + 8c + 4u + 2 + e (the mapping of Q8MmaPolicy, whose query
// preparation and output order are reused).
#pragma once

#include "flash_decode_q8.cuh"

namespace er {

template <int GROUP, int UNITS_PER_TILE, int WARP_GROUPS, int STAGES>
struct DenseMmaPolicy : DensePolicy<GROUP, UNITS_PER_TILE, WARP_GROUPS, STAGES> {
    using Base = DensePolicy<GROUP, UNITS_PER_TILE, WARP_GROUPS, STAGES>;
    static_assert(GROUP <= 8, "one n-tile of heads");
    static constexpr float kProbScale = 4096.f, kInvProbScale = 1.f / 4096.f;
    static constexpr bool kPacked = GROUP <= 4;   // hi parts in columns 0..3 of the n-tile, lo parts in 4..7 (see Q8MmaPolicy)

    struct State {
        uint32_t qh[8][2], ql[8][2];   // B fragments of the queries per k-step: fp16 hi and lo parts (packed: qh holds both)
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
        __device__ __forceinline__ void gather() {   // packed columns: V . p_hi (lanes c < 2) + V . p_lo (lanes c >= 2)
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
        // m-tile t = 2j + u: row n -> dim 32j + 8(n/2) + 4u + n%2, row n + 8 -> that + 2
        __device__ __forceinline__ void publish(float* ml, float* accs, int lane) {
            const int g = lane >> 2, c = lane & 3;
            gather();
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int h = 2 * c + e;
                if (h < GROUP) {
                    if (g == 0) {
                        ml[h * 2] = m[e];
                        ml[h * 2 + 1] = l[e] * kProbScale;   // acc carries the factor too: it cancels in acc / l
                    }
#pragma unroll
                    for (int t = 0; t < 8; ++t) {
                        const int d0 = 32 * (t >> 1) + 8 * (g >> 1) + 4 * (t & 1) + (g & 1);
                        accs[h * kHeadDim + d0] = acc[t][e];
                        accs[h * kHeadDim + d0 + 2] = acc[t][2 + e];
                    }
                }
            }
        }
        __device__ __forceinline__ void fold(float* ml, float* accs, int lane, bool first) {
            gather();
            mma_state_fold<GROUP>(m, l, acc, ml, accs, lane, first, 1.f, kProbScale,
                                  [](int t, int g, int second) { return 32 * (t >> 1) + 8 * (g >> 1) + 4 * (t & 1) + (g & 1) + 2 * second; });
        }
    };
    static constexpr int kFoldUnits = 32;   // chains of about 128 accumulating mma per output fragment

    // Q rows (per-head RMS norm, then NeoX rotation, when asked) -> B fragments; thread (g, c) holds head g.
    template <bool COHERENT = false>
    __device__ static void load_q(const DecodeParams& p, State& st, const float* qrow, const float2* cs, uint8_t*, int, int lane,
                                  int layer) {
        const int g = lane >> 2, c = lane & 3;
        const int head = kPacked ? (g & 3) : g;   // packed: column g carries head g % 4, its hi part below column 4
        const float* qw = p.q_norm_w ? p.q_norm_w + static_cast<int64_t>(layer) * p.norm_stride : nullptr;
        float rs = 1.f;
        if (qw != nullptr) {
#pragma unroll
            for (int h = 0; h < GROUP; ++h) {
                const float r = head_rms_scale<COHERENT>(qrow + h * kHeadDim, p.rms_eps, lane);
                if (h == head) rs = r;
            }
        }
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            float x[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] = 0.f;
            if (head < GROUP) {
                const int d0 = 32 * b + 8 * c;
                auto load8 = [&](int d, float (&out)[8]) {
                    const float4 lo4 = ld_step_row<COHERENT>(reinterpret_cast<const float4*>(qrow + head * kHeadDim + d));
                    const float4 hi4 = ld_step_row<COHERENT>(reinterpret_cast<const float4*>(qrow + head * kHeadDim + d + 4));
                    out[0] = lo4.x; out[1] = lo4.y; out[2] = lo4.z; out[3] = lo4.w;
                    out[4] = hi4.x; out[5] = hi4.y; out[6] = hi4.z; out[7] = hi4.w;
                    if (qw != nullptr) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) out[e] = __fmul_rn(__fmul_rn(out[e], rs), __ldg(qw + d + e));
                    }
                };
                load8(d0, x);
                if (p.apply_rope) {
                    // partner of dim d is d +- 64: blocks b and b ^ 2, same offset inside the block
                    float y[8];
                    load8(d0 ^ 64, y);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float2 t = cs[(d0 + e) & 63];
                        float y0, y1;
                        if (d0 < 64) { rope_rotate(x[e], y[e], t, y0, y1); x[e] = y0; }
                        else         { rope_rotate(y[e], x[e], t, y0, y1); x[e] = y1; }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const float a0 = x[4 * u + 2 * half], a1 = x[4 * u + 2 * half + 1];
                    const __half2 hh = __floats2half2_rn(a0, a1);
                    const float2 hf = __half22float2(hh);
                    const uint32_t hi = *reinterpret_cast<const uint32_t*>(&hh), lo = pack_half2(a0 - hf.x, a1 - hf.y);
                    if constexpr (kPacked) {
                        st.qh[2 * b + u][half] = g < 4 ? hi : lo;
                    } else {
                        st.qh[2 * b + u][half] = hi;
                        st.ql[2 * b + u][half] = lo;
                    }
                }
        }
        st.reset();
    }

    __device__ static void process_unit(const DecodeParams& p, const uint8_t* stage, int unit, int nvalid, State& st, float*,
                                        const uint8_t*, int lane) {
        const int g = lane >> 2, c = lane & 3;
        const uint32_t sbase = smem_u32(stage);
        const int r0 = unit * kUnitTokens + g;
        const uint32_t krow = sbase + r0 * kRowBytesF16 + 16 * c;
        const uint32_t vrow = krow + Base::kTileBytesF16;
        const bool ok0 = g < nvalid, ok1 = g + 8 < nvalid;
        auto load_chunk = [](uint32_t addr, uint32_t (&w)[4]) {   // halves (0,1) (2,3) (4,5) (6,7) of one 16-byte chunk
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr) : "memory");
        };

        float s[4] = {0.f, 0.f, 0.f, 0.f};   // (token g | g + 8) x (head 2c | 2c + 1)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t k0[4], k1[4];
            load_chunk(krow + 64 * j, k0);
            load_chunk(krow + 64 * j + 8 * kRowBytesF16, k1);
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                mma_m16n8k16(s, k0[2 * u], k1[2 * u], k0[2 * u + 1], k1[2 * u + 1], st.qh[2 * j + u][0], st.qh[2 * j + u][1]);
                if constexpr (!kPacked) mma_m16n8k16(s, k0[2 * u], k1[2 * u], k0[2 * u + 1], k1[2 * u + 1], st.ql[2 * j + u][0], st.ql[2 * j + u][1]);
            }
        }
        if constexpr (kPacked) {   // columns 2c, 2c + 1 (K . q_hi) and their partners four columns on (K . q_lo)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[i] += __shfl_xor_sync(0xffffffffu, s[i], 2);
        }
        // rows at or past nvalid were never copied (stale shared memory, possibly NaN patterns): the select discards them
        s[0] = ok0 ? s[0] * p.scale_log2 : -INFINITY;
        s[1] = ok0 ? s[1] * p.scale_log2 : -INFINITY;
        s[2] = ok1 ? s[2] * p.scale_log2 : -INFINITY;
        s[3] = ok1 ? s[3] * p.scale_log2 : -INFINITY;

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
        // ---- outputs: B = 4096 p as fp16 hi + lo (transposed to [token pair][head]), A = transposed value blocks ----
        const float w0 = p0 * kProbScale, w1 = p1 * kProbScale, w2 = p2 * kProbScale, w3 = p3 * kProbScale;
        const __half2 h01 = __floats2half2_rn(w0, w1), h23 = __floats2half2_rn(w2, w3);
        const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
        const uint32_t hi01 = *reinterpret_cast<const uint32_t*>(&h01), hi23 = *reinterpret_cast<const uint32_t*>(&h23);
        const uint32_t lo01 = pack_half2(w0 - f01.x, w1 - f01.y), lo23 = pack_half2(w2 - f23.x, w3 - f23.y);
        // packed: lanes c and c ^ 2 hold the same probabilities; the first pair supplies the hi columns, the second the lo columns
        const uint32_t b0 = movmatrix_trans(kPacked && c >= 2 ? lo01 : hi01);
        const uint32_t b1 = movmatrix_trans(kPacked && c >= 2 ? lo23 : hi23);
        uint32_t b0l = 0, b1l = 0;
        if constexpr (!kPacked) {
            b0l = movmatrix_trans(lo01);
            b1l = movmatrix_trans(lo23);
        }
        const bool partial = nvalid < kUnitTokens;   // warp-uniform
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t v0[4], v1[4];
            load_chunk(vrow + 64 * j, v0);
            load_chunk(vrow + 64 * j + 8 * kRowBytesF16, v1);
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
                if constexpr (!kPacked) mma_m16n8k16(st.acc[2 * j + u], a0, a1, a2, a3, b0l, b1l);
            }
        }
    }
};

}  // namespace er
