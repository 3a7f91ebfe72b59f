// q8_0 rows in the persistent flash-decode kernel (see flash_decode.cuh): gqa_attention_q8kv (Shaders/GQA.metal:389-522)
// for one query row per sequence.
//
// Stage = K int8 rows | V int8 rows | K scales | V scales (128 B + 8 B per row and tensor, see q8.cuh).  Both contractions
// run on mma.sync m16n8k16 with fp16 operands: an int8 is exact in fp16, so
//   S[token][head] = sum_b kScale[token][b] * ( K8[token][block b] . q[head][block b] )     one accumulator per block b
//   O^T[dim][head] += V8^T[dim][token] . ( p[token][head] * vScale[token][block(dim)] )^T    one B operand per block
// keep fp32 accuracy with the queries and the scaled probabilities entering as fp16 hi + lo pairs.  p * vScale is small
// (vScale = maxAbs / 127, p ~ 1 / context): it is carried times 64 so that its lo part stays a normal fp16 number
// (64 * vScale <= 65504 for every scale an fp16-sourced row can have), and the outputs are divided by 64 when published.
// With up to four heads per kv head (kPacked) the hi parts sit in columns 0..3 of the n-tile and the lo parts in columns
// 4..7, so one mma multiplies an A fragment by both; scores add the two column halves across lanes c and c ^ 2, outputs
// when the state is folded or published.
// Thread (g = lane / 4, c = lane % 4) reads tokens g and g + 8 of the warp's 16-token unit and, of every 32-element
// block, the 8 bytes [8c, 8c + 8) -- adjacent in the cached row (q8_word_slot: 32 bytes at 32c, two 16-byte reads
// that the warp's lanes spread over all banks; the plain element order made eight rows collide on the same banks and cost
// 128 of the kernel's 198 shared-memory wavefronts per unit): byte pairs (0,1) and (2,3) feed the block's first k-step, (4,5) and (6,7) the second
// (scores); for the outputs the same four pairs are the column pairs of the block's two 16-dim m-tiles, transposed with
// movmatrix because there the contraction runs over tokens.  Pair conversion: the two bytes (sign bit flipped) become the
// low mantissa bytes of two halves 0x64xx = 1024 + x + 128, minus 1152.
#pragma once

#include "flash_decode.cuh"
#include "flash_decode_turbo_mma.cuh"   // mma_m16n8k16, movmatrix_trans, pack_half2

namespace er {

// bytes 2i, 2i+1 of `w` (already xor 0x80808080) -> half2 of the two signed values
template <int PAIR>
__device__ __forceinline__ uint32_t q8_pair_to_half2(uint32_t w_flipped) {
    const uint32_t sel = PAIR == 0 ? 0x7170u : 0x7372u;     // result bytes: [w.b(2P), 0x64, w.b(2P+1), 0x64]
    uint32_t h;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(h) : "r"(w_flipped), "r"(0x64646464u), "r"(sel));
    const __half2 bias = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));   // 1152
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&h), bias);
    return *reinterpret_cast<const uint32_t*>(&r);
}

template <int GROUP, int UNITS_PER_TILE = 7, int WARP_GROUPS = 2, int STAGES = 4>
struct Q8MmaPolicy {
    static_assert(GROUP <= 8, "one n-tile of heads");
    static constexpr int kGroup = GROUP;
    static constexpr int kUnitsPerTile = UNITS_PER_TILE;
    static constexpr int kWarpGroups = WARP_GROUPS;
    static constexpr int kStages = STAGES;
    static constexpr int kTileTokens = UNITS_PER_TILE * kUnitTokens;
    static constexpr int kThreads = (UNITS_PER_TILE * WARP_GROUPS + 1) * 32;
    static constexpr int kOffV = kTileTokens * 128;
    static constexpr int kOffKs = 2 * kTileTokens * 128;
    static constexpr int kOffVs = kOffKs + kTileTokens * 8;
    static constexpr int kStageBytes = kOffVs + kTileTokens * 8;
    static constexpr int kExtraBytes = 0;
    __device__ static float* fin_ptr(uint8_t*) { return nullptr; }
    static constexpr bool kRotated = false;
    static constexpr bool kFusedAppend = false;   // rows are quantised by q8_append_kernel
    static_assert(STAGES % WARP_GROUPS == 0, "STAGES must be a multiple of WARP_GROUPS");

    static constexpr float kProbScale = 64.f, kInvProbScale = 1.f / 64.f;
    // Up to four heads: the hi parts of queries and probabilities take columns 0..3 of the n-tile and the lo parts columns
    // 4..7, so one mma multiplies an A fragment by both; the column halves are added across lanes c and c ^ 2.
    static constexpr bool kPacked = GROUP <= 4;

    struct State {
        uint32_t qh[8][2], ql[8][2];   // B fragments of the (rotated) queries per k-step: fp16 hi and lo parts (packed: qh holds both)
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
        // m-tile t = 2b + u of block b: row n -> dim 32b + 8(n/2) + 4u + n%2, row n + 8 -> that + 2
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
                    for (int t = 0; t < 8; ++t) {
                        const int d0 = 32 * (t >> 1) + 8 * (g >> 1) + 4 * (t & 1) + (g & 1);
                        accs[h * kHeadDim + d0] = acc[t][e] * kInvProbScale;
                        accs[h * kHeadDim + d0 + 2] = acc[t][2 + e] * kInvProbScale;
                    }
                }
            }
        }
        __device__ __forceinline__ void fold(float* ml, float* accs, int lane, bool first) {
            gather();
            mma_state_fold<GROUP>(m, l, acc, ml, accs, lane, first, kInvProbScale, 1.f,
                                  [](int t, int g, int second) { return 32 * (t >> 1) + 8 * (g >> 1) + 4 * (t & 1) + (g & 1) + 2 * second; });
        }
    };
    static constexpr int kFoldUnits = 32;   // chains of about 128 accumulating mma per output fragment

    __device__ static bool init_extra(uint8_t*, int, int) { return true; }
    __device__ static void patch_new_row(const DecodeParams&, uint8_t*, int, int, int, int, int, int, const float*, const float*,
                                         const float2*, int) {}
    __device__ static void store_out(const DecodeParams&, int64_t, const float*, int, int) {}

    template <class WAIT>
    __device__ static void issue_tile(const DecodeParams& p, uint8_t* stage, uint64_t* bar, int layer, int seq, int head,
                                      int t0, int ntok, int lane, int /*ring start: fp16 rows only*/, WAIT&& wait_free) {
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
        if (lane == 0) {   // scale copies are rounded up to 16 bytes per page segment
            uint32_t bytes = static_cast<uint32_t>(ntok) * 256u;
            for (int sgi = 0; sgi < nseg; ++sgi) {
                const int tb = max(t0, (first_page + sgi) * ps), te = min(t0 + ntok, (first_page + sgi + 1) * ps);
                bytes += 2u * ((static_cast<uint32_t>(te - tb) * 8u + 15u) & ~15u);
            }
            mbar_arrive_expect_tx(bar, bytes);
        }
        __syncwarp();
        for (int c = lane; c < 4 * nseg; c += 32) {
            const int kind = c & 3, sgi = c >> 2;
            const int tb = max(t0, (first_page + sgi) * ps);
            const int te = min(t0 + ntok, (first_page + sgi + 1) * ps);
            const int64_t row = c == lane ? row0 : row_index(p.addr, seq, head, tb);
            const uint32_t rows = static_cast<uint32_t>(te - tb);
            if (kind == 0) bulk_g2s(stage + (tb - t0) * 128, kc + row * 128, rows * 128, bar);
            else if (kind == 1) bulk_g2s(stage + kOffV + (tb - t0) * 128, vc + row * 128, rows * 128, bar);
            else if (kind == 2) bulk_g2s(stage + kOffKs + (tb - t0) * 8, kn + row * 8, (rows * 8 + 15u) & ~15u, bar);
            else bulk_g2s(stage + kOffVs + (tb - t0) * 8, vn + row * 8, (rows * 8 + 15u) & ~15u, bar);
        }
    }

    // Q row (NeoX-rotated when asked) -> B fragments.  k-step 2b + u of block b: label 2c + e -> dim 32b + 8c + 4u + e,
    // label 2c + 8 + e -> dim 32b + 8c + 4u + 2 + e; thread (g, c) holds head g.
    __device__ static void load_q(const DecodeParams& p, State& st, const float* qrow, const float2* cs, uint8_t*, int, int lane, int) {
        load_q_fragments(p, st, qrow, cs, lane);
    }
    // ST: any state with qh / ql fragments and reset() (the policies of layers with q8_0 keys and other values share this)
    template <class ST>
    __device__ static void load_q_fragments(const DecodeParams& p, ST& st, const float* qrow, const float2* cs, int lane) {
        const int g = lane >> 2, c = lane & 3;
        const int head = kPacked ? (g & 3) : g;   // packed: column g carries head g % 4, its hi part below column 4
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            float x[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] = 0.f;
            if (head < GROUP) {
                const int d0 = 32 * b + 8 * c;
                const float4 lo4 = __ldg(reinterpret_cast<const float4*>(qrow + head * kHeadDim + d0));
                const float4 hi4 = __ldg(reinterpret_cast<const float4*>(qrow + head * kHeadDim + d0 + 4));
                x[0] = lo4.x; x[1] = lo4.y; x[2] = lo4.z; x[3] = lo4.w; x[4] = hi4.x; x[5] = hi4.y; x[6] = hi4.z; x[7] = hi4.w;
                if (p.apply_rope) {
                    // partner of dim d is d +- 64: blocks b and b ^ 2, same offset inside the block
                    const int dp = d0 ^ 64;
                    const float4 plo = __ldg(reinterpret_cast<const float4*>(qrow + head * kHeadDim + dp));
                    const float4 phi = __ldg(reinterpret_cast<const float4*>(qrow + head * kHeadDim + dp + 4));
                    const float y[8] = {plo.x, plo.y, plo.z, plo.w, phi.x, phi.y, phi.z, phi.w};
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

    // words 2b, 2b + 1 = the thread's 8 bytes of block b of a cached row
    __device__ __forceinline__ static void load_row_words(uint32_t addr, uint32_t (&w)[8]) {
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr) : "memory");
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "r"(addr + 16) : "memory");
    }
    // a row's four block scales (fp16), zeros for a row that was never copied
    __device__ __forceinline__ static void load_scales4(uint32_t addr, float (&out)[4], bool ok) {
        uint32_t w[2];
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "r"(addr) : "memory");
        const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&w[0]));
        const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&w[1]));
        out[0] = ok ? f01.x : 0.f; out[1] = ok ? f01.y : 0.f; out[2] = ok ? f23.x : 0.f; out[3] = ok ? f23.y : 0.f;
    }

    // Scores of one unit, s = (token g | g + 8) x (head 2c | 2c + 1) in the log2 domain, -inf for rows at or past nvalid.
    // krows / kscales: shared-window addresses of the tile's int8 rows (128 B per row) and block scales (8 B per row).
    // ST: any state with the query fragments load_q_fragments wrote.
    template <class ST>
    __device__ __forceinline__ static void unit_scores(const DecodeParams& p, uint32_t krows, uint32_t kscales, int unit, int nvalid,
                                                       const ST& st, int lane, float (&s)[4]) {
        const int g = lane >> 2, c = lane & 3;
        const int r0 = unit * kUnitTokens + g;
        const uint32_t krow = krows + r0 * 128 + 32 * c;
        const bool ok0 = g < nvalid, ok1 = g + 8 < nvalid;
        float sb[4][4];   // one accumulator per 32-element block
        {
            uint32_t k0[8], k1[8];
            load_row_words(krow, k0);
            load_row_words(krow + 8 * 128, k1);
#pragma unroll
            for (int b = 0; b < 4; ++b) {
#pragma unroll
                for (int e = 0; e < 4; ++e) sb[b][e] = 0.f;
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const uint32_t w0 = k0[2 * b + u] ^ 0x80808080u, w1 = k1[2 * b + u] ^ 0x80808080u;
                    const uint32_t a0 = q8_pair_to_half2<0>(w0), a1 = q8_pair_to_half2<0>(w1);
                    const uint32_t a2 = q8_pair_to_half2<1>(w0), a3 = q8_pair_to_half2<1>(w1);
                    mma_m16n8k16(sb[b], a0, a1, a2, a3, st.qh[2 * b + u][0], st.qh[2 * b + u][1]);
                    if constexpr (!kPacked) mma_m16n8k16(sb[b], a0, a1, a2, a3, st.ql[2 * b + u][0], st.ql[2 * b + u][1]);
                }
            }
        }
        float ks0[4], ks1[4];
        load_scales4(kscales + r0 * 8, ks0, ok0);
        load_scales4(kscales + (r0 + 8) * 8, ks1, ok1);
        s[0] = ks0[0] * sb[0][0] + ks0[1] * sb[1][0] + ks0[2] * sb[2][0] + ks0[3] * sb[3][0];
        s[1] = ks0[0] * sb[0][1] + ks0[1] * sb[1][1] + ks0[2] * sb[2][1] + ks0[3] * sb[3][1];
        s[2] = ks1[0] * sb[0][2] + ks1[1] * sb[1][2] + ks1[2] * sb[2][2] + ks1[3] * sb[3][2];
        s[3] = ks1[0] * sb[0][3] + ks1[1] * sb[1][3] + ks1[2] * sb[2][3] + ks1[3] * sb[3][3];
        if constexpr (kPacked) {   // columns 2c, 2c + 1 (K . q_hi) and their partners four columns on (K . q_lo)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[i] += __shfl_xor_sync(0xffffffffu, s[i], 2);
        }
        s[0] = ok0 ? s[0] * p.scale_log2 : -INFINITY;
        s[1] = ok0 ? s[1] * p.scale_log2 : -INFINITY;
        s[2] = ok1 ? s[2] * p.scale_log2 : -INFINITY;
        s[3] = ok1 ? s[3] * p.scale_log2 : -INFINITY;
    }

    // Outputs of one unit: O^T += V8^T . (p * vScale[block])^T block by block, B = (p * vScale) as fp16 hi + lo, A = transposed int8
    // pairs.  vrows / vscales: shared-window addresses of the tile's int8 value rows and block scales; pr = the probabilities of
    // (token g | g + 8) x (head 2c | 2c + 1).  ST: any state with this policy's accumulator order (State::publish).
    template <class ST>
    __device__ __forceinline__ static void unit_values(ST& st, uint32_t vrows, uint32_t vscales, int unit, int nvalid, const float (&pr)[4], int lane) {
        const int g = lane >> 2, c = lane & 3;
        const int r0 = unit * kUnitTokens + g;
        const uint32_t vrow = vrows + r0 * 128 + 32 * c;
        const bool ok0 = g < nvalid, ok1 = g + 8 < nvalid;
        float vs0[4], vs1[4];
        load_scales4(vscales + r0 * 8, vs0, ok0);
        load_scales4(vscales + (r0 + 8) * 8, vs1, ok1);
#pragma unroll
        for (int b = 0; b < 4; ++b) { vs0[b] *= kProbScale; vs1[b] *= kProbScale; }
        uint32_t v0[8], v1[8];
        load_row_words(vrow, v0);
        load_row_words(vrow + 8 * 128, v1);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const float w0 = pr[0] * vs0[b], w1 = pr[1] * vs0[b], w2 = pr[2] * vs1[b], w3 = pr[3] * vs1[b];
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
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                // rows at or past nvalid were never copied: their bytes are stale but finite after conversion, and p = 0
                const uint32_t x0 = v0[2 * b + u] ^ 0x80808080u, x1 = v1[2 * b + u] ^ 0x80808080u;
                const uint32_t a0 = movmatrix_trans(q8_pair_to_half2<0>(x0));
                const uint32_t a1 = movmatrix_trans(q8_pair_to_half2<1>(x0));
                const uint32_t a2 = movmatrix_trans(q8_pair_to_half2<0>(x1));
                const uint32_t a3 = movmatrix_trans(q8_pair_to_half2<1>(x1));
                mma_m16n8k16(st.acc[2 * b + u], a0, a1, a2, a3, b0, b1);
                if constexpr (!kPacked) mma_m16n8k16(st.acc[2 * b + u], a0, a1, a2, a3, b0l, b1l);
            }
        }
    }

    __device__ static void process_unit(const DecodeParams& p, const uint8_t* stage, int unit, int nvalid, State& st, float*,
                                        const uint8_t*, int lane) {
        const uint32_t sbase = smem_u32(stage);
        float s[4], pr[4];
        unit_scores(p, sbase, sbase + kOffKs, unit, nvalid, st, lane, s);
        mma_softmax_step(st, s, pr);
        unit_values(st, sbase + kOffV, sbase + kOffVs, unit, nvalid, pr, lane);
    }
};

}  // namespace er
