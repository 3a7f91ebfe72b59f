// Balanced / aggressive TurboQuant rows (regular channels at RB bits, 32 high-precision channels at HB bits, a QJL sign per
// channel, row norm and residual norm: the general form of gqa_attention_turboquant_decode, Shaders/TurboQuant.metal:1794-2001,
// rows as TurboQuantReferenceEncoder.encode writes them, TurboQuant.swift:1003-1100) in the persistent flash-decode kernel,
// both contractions on the tensor cores.  The effective coordinate of a cached row is
//     e[d] = rowNorm * ( centroid[d] + sqrt(pi / 2) * residualScale * residualNorm * sign[d] )
// with centroid[d] from the RB-bit codebook, or from the HB-bit one where the row's mask marks channel d (its code is the RB
// regular bits plus HB - RB bits of the side stream, in channel order).  So per 16-token unit, in the rotated space:
//     S[token][head]   = kNorm * ( C_k . q  +  rho_k * ( SIGN_k . q ) )                 rho = sqrt(pi/2) * scale * residualNorm
//     O^T[dim][head]  += C_v^T . (p * vNorm)  +  SIGN_v^T . (p * vNorm * rho_v)
// The centroid products use TurboMmaPolicy's packed layouts (hi parts of q and p in columns 0..3 of the n-tile, lo parts in
// 4..7; lo parts of a key centroid in rows g + 8), so queries, probabilities and centroids enter with ~22 significant bits.
// What differs is the lookup: a row has its own mask, so a code's table index is built per CHANNEL -- regular bits, the mask
// bit, and the side bits at the channel's rank, kept in a running shift of the side stream -- and one 4-byte read of the
// unified table [mask bit][code] returns half2 (hi, lo) of the centroid; two reads are re-paired with two prmt for a score
// fragment, and are output fragments as they come.  Signs are exact in fp16, so SIGN . q and SIGN^T . p are plain 16-token
// mma whose +-1 fragments come from two 16-entry tables indexed by four sign bits; a side whose residual scale is 0 (the
// reference's contract) leaves its sign products out.
//
// Thread (g = lane / 4, c = lane % 4): scores -- tokens g and g + 8, channels [32c, 32c + 32) = mask word c, sign word c and
// RB code words; outputs -- tokens 2c, 2c + 1, 2c + 8, 2c + 9, channels [16g, 16g + 16) = one half of mask word g / 2.
// Built for up to four query heads per kv head; eight heads, sliding windows and layers whose two sides use different formats
// run on the SIMT kernel (simt_decode_kernel).
#pragma once

#include "flash_decode_turbo_mma.cuh"

namespace er {

template <int GROUP, int RB, int HB, int UNITS_PER_TILE = 11, int WARP_GROUPS = 1, int STAGES = 3>
struct OutlierMmaPolicy {
    static_assert(GROUP <= 4, "packed columns: hi and lo parts share the n-tile");
    static_assert(HB > RB && HB - RB <= 2, "side stream of 32 or 64 bits");
    using TS = TurboStaging<GROUP, 4, 4, UNITS_PER_TILE, WARP_GROUPS, STAGES>;        // query rotation, output transform
    using State = typename TurboMmaPolicy<GROUP, 4, 4, UNITS_PER_TILE, WARP_GROUPS, STAGES>::State;
    static constexpr int kGroup = GROUP;
    static constexpr int kUnitsPerTile = UNITS_PER_TILE;
    static constexpr int kWarpGroups = WARP_GROUPS;
    static constexpr int kStages = STAGES;
    static constexpr int kTileTokens = UNITS_PER_TILE * kUnitTokens;
    static constexpr int kThreads = (UNITS_PER_TILE * WARP_GROUPS + 1) * 32;
    // a cached row: [codes 4 RB words][side stream][mask 4][signs 4][rowNorm][residualNorm][pad] (OutlierFormat)
    static constexpr int kSideW = HB - RB;                 // side bits per high-precision channel = words of the side stream
    static constexpr int kOffSide = 4 * RB;
    static constexpr int kOffMask = kOffSide + kSideW;
    static constexpr int kOffSigns = kOffMask + 4;
    static constexpr int kOffNorms = kOffMask + 8;
    static constexpr int kRowWords = (kOffMask + 10 + 3) & ~3;
    static constexpr int kRowBytes = kRowWords * 4;
    static constexpr int kSideBytes = kTileTokens * kRowBytes;     // K rows, then V rows
    static constexpr int kStageBytes = 2 * kSideBytes;
    static constexpr int kTableBytes = (2 << HB) * 128;            // [mask bit][code][32 lanes] half2 (hi, lo)
    // sign fragments: [4 sign bits][32 lanes] two registers of +-1 halves, one table per contraction (their bit orders differ)
    static constexpr int kSignTableBytes = 16 * 256;
    static constexpr int kExtraBytes = 2 * kTableBytes + 2 * kSignTableBytes + 2 * GROUP * kHeadDim * 4;
    static constexpr bool kRotated = true;
    static constexpr bool kFusedAppend = false;                    // rows are written by tq_outlier_append_kernel
    static constexpr int kFoldUnits = 32;
    static_assert(STAGES % WARP_GROUPS == 0, "STAGES must be a multiple of WARP_GROUPS");

    __device__ __forceinline__ static uint32_t table_addr(const uint8_t* extra) {
        return (smem_u32(extra) + kTableBytes - 1) & ~static_cast<uint32_t>(kTableBytes - 1);
    }
    // the two sign tables follow the centroid table (whose size is a multiple of theirs, so they are aligned to their size)
    __device__ __forceinline__ static uint32_t sign_table_addr(const uint8_t* extra) { return table_addr(extra) + kTableBytes; }
    __device__ __forceinline__ static float* rows_ptr(uint8_t* extra) {
        return reinterpret_cast<float*>(extra + (sign_table_addr(extra) + 2 * kSignTableBytes - smem_u32(extra)));
    }
    __device__ __forceinline__ static float* fin_ptr(uint8_t* extra) { return rows_ptr(extra) + GROUP * kHeadDim; }

    // bits 0 and 1 of `bits` -> half2 (+-1, +-1): a set bit is +1 (TurboQuant.swift:1158: sign bit ? 1 : -1)
    __device__ __forceinline__ static uint32_t sign_pair(uint32_t bits) {
        return 0xBC00BC00u ^ ((bits & 1u) << 15) ^ ((bits & 2u) << 30);
    }

    __device__ static bool init_extra(uint8_t* extra, int tid, int) {
        const uint32_t table = table_addr(extra);
        for (int e = tid; e < (2 << HB) * 32; e += kThreads) {
            const int idx = e >> 5, high = idx >> HB, code = idx & ((1 << HB) - 1);
            const float cv = high ? tq_centroids_rt(HB)[code] : (code < (1 << RB) ? tq_centroids_rt(RB)[code] : 0.f);
            const float hi = __half2float(__float2half_rn(cv));
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(table + 4 * e), "r"(pack_half2(hi, cv - hi)) : "memory");
        }
        // index i = x | y << 2 (two sign bits of each of two tokens).  Scores: registers (pair of x, pair of y) -- two adjacent
        // channels of token x, of token y.  Outputs: (bit 0 of x and y, bit 1 of x and y) -- one channel of both tokens each.
        const uint32_t signs = sign_table_addr(extra);
        for (int e = tid; e < 16 * 32; e += kThreads) {
            const uint32_t i = e >> 5, x = i & 3u, y = i >> 2;
            asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(signs + 8 * e), "r"(sign_pair(x)), "r"(sign_pair(y)) : "memory");
            asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(signs + kSignTableBytes + 8 * e), "r"(sign_pair((x & 1u) | ((y & 1u) << 1))),
                         "r"(sign_pair((x >> 1) | (y & 2u)))
                         : "memory");
        }
        return true;
    }
    __device__ static void patch_new_row(const DecodeParams&, uint8_t*, int, int, int, int, int, int, const float*, const float*,
                                         const float2*, int) {}
    __device__ static void store_out(const DecodeParams& p, int64_t out_off, const float* fin, int warp, int lane) {
        TS::store_out(p, out_off, fin, warp, lane);
    }

    // One or two bulk copies per page segment: the K rows and the V rows of the tile (whole cached rows).
    template <class WAIT>
    __device__ static void issue_tile(const DecodeParams& p, uint8_t* stage, uint64_t* bar, int layer, int seq, int head,
                                      int t0, int ntok, int lane, int /*ring start: fp16 rows only*/, WAIT&& wait_free) {
        const uint8_t* kc = p.k_base + static_cast<int64_t>(layer) * p.k_layer_stride_bytes;
        const uint8_t* vc = p.v_base + static_cast<int64_t>(layer) * p.v_layer_stride_bytes;
        const int ps = p.addr.page_size;
        const int first_page = t0 / ps;
        const int nseg = (t0 + ntok - 1) / ps - first_page + 1;
        const int64_t row0 = lane < 2 * nseg ? row_index(p.addr, seq, head, max(t0, (first_page + (lane >> 1)) * ps)) : 0;
        wait_free();
        if (lane == 0) mbar_arrive_expect_tx(bar, 2u * static_cast<uint32_t>(ntok) * kRowBytes);
        __syncwarp();
        for (int c = lane; c < 2 * nseg; c += 32) {
            const int kind = c & 1, sgi = c >> 1;
            const int tb = max(t0, (first_page + sgi) * ps);
            const int te = min(t0 + ntok, (first_page + sgi + 1) * ps);
            const int64_t row = c == lane ? row0 : row_index(p.addr, seq, head, tb);
            const uint32_t bytes = static_cast<uint32_t>(te - tb) * kRowBytes;
            if (kind == 0) bulk_g2s(stage + (tb - t0) * kRowBytes, kc + row * kRowBytes, bytes, bar);
            else bulk_g2s(stage + kSideBytes + (tb - t0) * kRowBytes, vc + row * kRowBytes, bytes, bar);
        }
    }

    // Rotated queries -> packed B fragments (column g: head g % 4, hi part below column 4, lo part from it on).
    __device__ static void load_q(const DecodeParams& p, State& st, const float* qrow, const float2* cs, uint8_t* extra,
                                  int warp, int lane, int) {
        float* qrot = rows_ptr(extra);
        TS::rotate_queries(p, qrot, qrow, cs, warp, lane);
        st.lut_k = table_addr(extra) | (lane << 2);           // centroid table, 4-byte entries
        st.lut_v = sign_table_addr(extra) | (lane << 3);      // sign tables, 8-byte entries: scores, then outputs
        const int g = lane >> 2, c = lane & 3;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            if ((g & 3) < GROUP) t = *reinterpret_cast<const float4*>(qrot + (g & 3) * kHeadDim + 32 * c + 4 * s);
            const __half2 h01 = __floats2half2_rn(t.x, t.y), h23 = __floats2half2_rn(t.z, t.w);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            st.qh[s][0] = g < 4 ? *reinterpret_cast<const uint32_t*>(&h01) : pack_half2(t.x - f01.x, t.y - f01.y);
            st.qh[s][1] = g < 4 ? *reinterpret_cast<const uint32_t*>(&h23) : pack_half2(t.z - f23.x, t.w - f23.y);
        }
        st.reset();
    }

    // ---- per-channel lookups ----
    // Running view of a row's side stream over at most 16 channels (32 side bits): bit 0 of `lo` is the first side bit of the
    // next high-precision channel.  `rank` = high-precision channels of the row before the view's first channel.
    struct SideBits {
        uint32_t lo;
        __device__ __forceinline__ void start(uint32_t s0, uint32_t s1, int rank) {
            const int sh = rank * kSideW;   // 0 .. 32 kSideW
            if constexpr (kSideW == 1) {
                lo = sh >= 32 ? 0u : s0 >> sh;
            } else {
                lo = sh >= 64 ? 0u : (sh >= 32 ? s1 >> (sh - 32) : __funnelshift_r(s0, s1, sh));
            }
        }
    };
    // What a 32-channel span needs to restart its view at channel 16.
    struct SideSource {
        uint32_t s0, s1;
        int rank;
    };

    // Shared-window address of the table entry of channel J of a span whose regular codes start at bit 0 of w[]; channels
    // must be visited in ascending order (a marked channel consumes its side bits).
    template <int J, int NW>
    __device__ __forceinline__ static uint32_t entry_addr(const uint32_t (&w)[NW], uint32_t mask_bits, SideBits& side, uint32_t lut) {
        constexpr int bit = J * RB, word = bit >> 5, sh = bit & 31;
        constexpr uint32_t cm = ((1u << RB) - 1u) << 7;
        uint32_t v;
        if constexpr (sh + RB > 32) v = __funnelshift_r(w[word], w[word + 1], sh - 7);
        else if constexpr (sh >= 7) v = w[word] >> (sh - 7);
        else v = w[word] << (7 - sh);
        uint32_t addr = (v & cm) | lut;
        if ((mask_bits >> J) & 1u) {
            // mask bit at index bit HB = RB + kSideW, side bits below it: one and-or, one shift-add
            addr += ((side.lo & ((1u << kSideW) - 1u)) | (1u << kSideW)) << (RB + 7);
            side.lo >>= kSideW;
        }
        return addr;
    }

    // Two registers of +-1 halves for sign bits [B, B + 2) of x and of y (see init_extra for the two register orders).
    template <int B>
    __device__ __forceinline__ static void sign_regs(uint32_t lut, uint32_t x, uint32_t y, uint32_t& r0, uint32_t& r1) {
        uint32_t ix, iy;   // (bits of x) << 8 | (bits of y) << 10
        if constexpr (B >= 8) ix = x >> (B - 8); else ix = x << (8 - B);
        if constexpr (B >= 10) iy = y >> (B - 10); else iy = y << (10 - B);
        lds_u32x2(lut + ((ix & 0x300u) | (iy & 0xC00u)), r0, r1);   // the table is aligned to 2 KB at least, not to its 4 KB: add
    }
    __device__ __forceinline__ static float lds_f32(uint32_t addr) {
        float v;
        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
        return v;
    }

    // The span's bookkeeping words of one cached row: mask bits of the span, the side stream positioned at the span's first
    // high-precision channel, sign bits of the span.  HALF = false: the 32 channels of mask word `w`; true: its half `h`.
    template <bool HALF>
    __device__ __forceinline__ static void span_words(uint32_t row, int w, int h, uint32_t& mask_bits, SideBits& side, uint32_t& signs,
                                                      SideSource* src = nullptr) {
        int rank = 0;
        uint32_t mine = 0u;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t m = lds_u32_stage(row + (kOffMask + i) * 4);
            rank += i < w ? __popc(m) : 0;
            mine = i == w ? m : mine;
        }
        uint32_t sg = lds_u32_stage(row + (kOffSigns + w) * 4);
        if constexpr (HALF) {
            rank += h ? __popc(mine & 0xFFFFu) : 0;
            mine = h ? mine >> 16 : mine & 0xFFFFu;
            sg = h ? sg >> 16 : sg & 0xFFFFu;
        }
        mask_bits = mine;
        signs = sg;
        const uint32_t s0 = lds_u32_stage(row + kOffSide * 4);
        const uint32_t s1 = kSideW == 2 ? lds_u32_stage(row + (kOffSide + 1) * 4) : 0u;
        side.start(s0, s1, rank);
        if (src != nullptr) { src->s0 = s0; src->s1 = s1; src->rank = rank; }
    }

    // Score k-step S for tokens g (sa) and g + 8 (sb): channels 4S .. 4S + 3 of the thread's 32; ss = SIGN . q of both tokens
    // (SIGNS = false: the residual scale of the keys is 0, the reference's contract, and the sign products are left out).
    template <int S, bool SIGNS>
    __device__ __forceinline__ static void score_steps(float (&sa)[4], float (&sb)[4], float (&ss)[4], const uint32_t (&ka)[RB],
                                                       const uint32_t (&kb)[RB], uint32_t ma, uint32_t mb, SideBits& da, SideBits& db,
                                                       const SideSource& ra, const SideSource& rb, uint32_t ga, uint32_t gb, const State& st) {
        if constexpr (S < 8) {
            if constexpr (S == 4) {   // channel 16: a view holds the side bits of 16 channels
                da.start(ra.s0, ra.s1, ra.rank + __popc(ma & 0xFFFFu));
                db.start(rb.s0, rb.s1, rb.rank + __popc(mb & 0xFFFFu));
            }
            const uint32_t ea0 = lds_u32(entry_addr<4 * S>(ka, ma, da, st.lut_k)), ea1 = lds_u32(entry_addr<4 * S + 1>(ka, ma, da, st.lut_k));
            const uint32_t ea2 = lds_u32(entry_addr<4 * S + 2>(ka, ma, da, st.lut_k)), ea3 = lds_u32(entry_addr<4 * S + 3>(ka, ma, da, st.lut_k));
            const uint32_t eb0 = lds_u32(entry_addr<4 * S>(kb, mb, db, st.lut_k)), eb1 = lds_u32(entry_addr<4 * S + 1>(kb, mb, db, st.lut_k));
            const uint32_t eb2 = lds_u32(entry_addr<4 * S + 2>(kb, mb, db, st.lut_k)), eb3 = lds_u32(entry_addr<4 * S + 3>(kb, mb, db, st.lut_k));
            // entries are half2 (hi, lo) per channel; a score fragment wants (hi, hi) in row g and (lo, lo) in row g + 8
            mma_m16n8k16(sa, __byte_perm(ea0, ea1, 0x5410), __byte_perm(ea0, ea1, 0x7632), __byte_perm(ea2, ea3, 0x5410),
                         __byte_perm(ea2, ea3, 0x7632), st.qh[S][0], st.qh[S][1]);
            mma_m16n8k16(sb, __byte_perm(eb0, eb1, 0x5410), __byte_perm(eb0, eb1, 0x7632), __byte_perm(eb2, eb3, 0x5410),
                         __byte_perm(eb2, eb3, 0x7632), st.qh[S][0], st.qh[S][1]);
            if constexpr (SIGNS) {
                uint32_t g0, g1, g2, g3;   // (token g, token g + 8) x channels (4S, 4S + 1 | 4S + 2, 4S + 3)
                sign_regs<4 * S>(st.lut_v, ga, gb, g0, g1);
                sign_regs<4 * S + 2>(st.lut_v, ga, gb, g2, g3);
                mma_m16n8k16(ss, g0, g1, g2, g3, st.qh[S][0], st.qh[S][1]);
            }
            score_steps<S + 1, SIGNS>(sa, sb, ss, ka, kb, ma, mb, da, db, ra, rb, ga, gb, st);
        }
    }

    static constexpr int kVWords = RB == 2 ? 1 : 2;   // 16 channels of RB bits
    // Output m-tile T (dims 16g + 2T in row g, 16g + 2T + 1 in row g + 8): centroids of the thread's four tokens against the
    // duplicated probabilities, signs of all four against the (token pair) sign weights.
    template <int T, bool SIGNS>
    __device__ __forceinline__ static void value_tiles(State& st, const uint32_t (&vw)[4][kVWords], const uint32_t (&vm)[4], SideBits (&vd)[4],
                                                       const uint32_t (&vg)[4], const uint32_t (&bh)[4], uint32_t bs0, uint32_t bs1) {
        if constexpr (T < 8) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t a0 = lds_u32(entry_addr<2 * T>(vw[2 * j], vm[2 * j], vd[2 * j], st.lut_k));
                const uint32_t a1 = lds_u32(entry_addr<2 * T + 1>(vw[2 * j], vm[2 * j], vd[2 * j], st.lut_k));
                const uint32_t a2 = lds_u32(entry_addr<2 * T>(vw[2 * j + 1], vm[2 * j + 1], vd[2 * j + 1], st.lut_k));
                const uint32_t a3 = lds_u32(entry_addr<2 * T + 1>(vw[2 * j + 1], vm[2 * j + 1], vd[2 * j + 1], st.lut_k));
                mma_m16n8k16(st.acc[T], a0, a1, a2, a3, bh[2 * j], bh[2 * j + 1]);
            }
            if constexpr (SIGNS) {
                uint32_t g0, g1, g2, g3;   // (channel 2T, channel 2T + 1) x tokens (2c, 2c + 1 | 2c + 8, 2c + 9)
                sign_regs<2 * T>(st.lut_v + kSignTableBytes, vg[0], vg[1], g0, g1);
                sign_regs<2 * T>(st.lut_v + kSignTableBytes, vg[2], vg[3], g2, g3);
                mma_m16n8k16(st.acc[T], g0, g1, g2, g3, bs0, bs1);
            }
            value_tiles<T + 1, SIGNS>(st, vw, vm, vd, vg, bh, bs0, bs1);
        }
    }

    __device__ static void process_unit(const DecodeParams& p, const uint8_t* stage, int unit, int nvalid, State& st, float*,
                                        const uint8_t*, int lane) {
        const int g = lane >> 2, c = lane & 3;
        const uint32_t sbase = smem_u32(stage);
        const uint32_t krow_a = sbase + (unit * kUnitTokens + g) * kRowBytes, krow_b = krow_a + 8 * kRowBytes;
        const uint32_t vrow_a = krow_a + kSideBytes, vrow_b = krow_b + kSideBytes;     // the V rows of tokens g and g + 8 (norms)
        const bool ok0 = g < nvalid, ok1 = g + 8 < nvalid;
        // rows at or past nvalid were never copied: their words are stale (any table index they form stays inside the table),
        // their norms are replaced by zeros and their scores by -inf
        const float kn0 = ok0 ? lds_f32(krow_a + kOffNorms * 4) : 0.f, kn1 = ok1 ? lds_f32(krow_b + kOffNorms * 4) : 0.f;
        const float kr0 = ok0 ? p.k_res_coef * lds_f32(krow_a + (kOffNorms + 1) * 4) : 0.f;
        const float kr1 = ok1 ? p.k_res_coef * lds_f32(krow_b + (kOffNorms + 1) * 4) : 0.f;
        const float vn0 = ok0 ? lds_f32(vrow_a + kOffNorms * 4) : 0.f, vn1 = ok1 ? lds_f32(vrow_b + kOffNorms * 4) : 0.f;
        const float vr0 = ok0 ? p.v_res_coef * lds_f32(vrow_a + (kOffNorms + 1) * 4) : 0.f;
        const float vr1 = ok1 ? p.v_res_coef * lds_f32(vrow_b + (kOffNorms + 1) * 4) : 0.f;

        float s[4];   // (token g | g + 8) x (head 2c | 2c + 1)
        {
            uint32_t ka[RB], kb[RB], ma, mb, ga, gb;
            SideBits da, db;
            SideSource ra, rb;
#pragma unroll
            for (int i = 0; i < RB; ++i) {
                ka[i] = lds_u32_stage(krow_a + (c * RB + i) * 4);
                kb[i] = lds_u32_stage(krow_b + (c * RB + i) * 4);
            }
            span_words<false>(krow_a, c, 0, ma, da, ga, &ra);
            span_words<false>(krow_b, c, 0, mb, db, gb, &rb);
            float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f}, ss[4] = {0.f, 0.f, 0.f, 0.f};
            if (p.k_res_coef != 0.f) score_steps<0, true>(sa, sb, ss, ka, kb, ma, mb, da, db, ra, rb, ga, gb, st);   // launch-uniform
            else score_steps<0, false>(sa, sb, ss, ka, kb, ma, mb, da, db, ra, rb, ga, gb, st);
            s[0] = fmaf(kr0, ss[0], sa[0] + sa[2]);   // (Ch + Cl) . q + rho * SIGN . q of token g
            s[1] = fmaf(kr0, ss[1], sa[1] + sa[3]);
            s[2] = fmaf(kr1, ss[2], sb[0] + sb[2]);   // of token g + 8
            s[3] = fmaf(kr1, ss[3], sb[1] + sb[3]);
#pragma unroll
            for (int i = 0; i < 4; ++i) s[i] += __shfl_xor_sync(0xffffffffu, s[i], 2);   // columns 2c, 2c + 1 (q hi) + their partners four on (q lo)
        }
        s[0] = ok0 ? (kn0 * s[0]) * p.scale_log2 : -INFINITY;
        s[1] = ok0 ? (kn0 * s[1]) * p.scale_log2 : -INFINITY;
        s[2] = ok1 ? (kn1 * s[2]) * p.scale_log2 : -INFINITY;
        s[3] = ok1 ? (kn1 * s[3]) * p.scale_log2 : -INFINITY;

        // running maxima and per-lane denominators as in TurboMmaPolicy::process_unit
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

        // B operands, transposed to [token][head] with the hi parts in columns 0..3 and the lo parts in 4..7 (lanes c and c ^ 2 hold
        // the same values): w = p * vNorm, duplicated on the (hi, lo) labels of a centroid; ws = w * rho_v, one token per label
        auto packed_trans = [&](float a, float b) {
            const __half2 h = __floats2half2_rn(a, b);
            const float2 f = __half22float2(h);
            return movmatrix_trans(c < 2 ? *reinterpret_cast<const uint32_t*>(&h) : pack_half2(a - f.x, b - f.y));
        };
        const float w0 = p0 * vn0, w1 = p1 * vn0, w2 = p2 * vn1, w3 = p3 * vn1;
        const uint32_t x0 = packed_trans(w0, w1), x1 = packed_trans(w2, w3);
        const uint32_t bs0 = packed_trans(w0 * vr0, w1 * vr0), bs1 = packed_trans(w2 * vr1, w3 * vr1);
        const uint32_t bh[4] = {__byte_perm(x0, x0, 0x1010), __byte_perm(x0, x0, 0x3232), __byte_perm(x1, x1, 0x1010), __byte_perm(x1, x1, 0x3232)};

        // value rows: channels [16g, 16g + 16) of tokens 2c, 2c + 1, 2c + 8, 2c + 9
        uint32_t vw[4][kVWords], vm[4], vg[4];
        SideBits vd[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t row = sbase + kSideBytes + (unit * kUnitTokens + 2 * c + (j & 1) + 8 * (j >> 1)) * kRowBytes;
            if constexpr (RB == 2) {
                vw[j][0] = lds_u32_stage(row + 4 * g);
            } else {
                // 48 bits at bit 48g: the two aligned words around them, shifted by 16 bits for odd g
                const uint32_t w = row + ((3 * g) >> 1) * 4;
                const uint32_t wa = lds_u32_stage(w), wb = lds_u32_stage(w + 4);
                const uint32_t sh = (g & 1) * 16;
                vw[j][0] = __funnelshift_r(wa, wb, sh);
                vw[j][1] = wb >> sh;
            }
            span_words<true>(row, g >> 1, g & 1, vm[j], vd[j], vg[j]);
        }
        if (p.v_res_coef != 0.f) value_tiles<0, true>(st, vw, vm, vd, vg, bh, bs0, bs1);   // launch-uniform
        else value_tiles<0, false>(st, vw, vm, vd, vg, bh, bs0, bs1);
    }
};

}  // namespace er
