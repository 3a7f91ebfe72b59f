// Persistent split-K GQA flash-decode over the KV cache (fp16 rows or TurboQuant codes).
//
// Replaces the decode use (seqLen == 1) of gqa_attention_f16kv (Shaders/GQA.metal:278-387), the attention
// phase of fused_qk_norm_rope_gqa (Shaders/RoPE.metal:395-494) and gqa_attention_turboquant_decode
// (Shaders/TurboQuant.metal:1794-2001); the split/merge arithmetic is the log-sum-exp merge of
// gqa_decode_attention_packed_f16kv_reduce (Shaders/GQA.metal:753-776).
//
// Work decomposition.  An *item* is one (layer, sequence, kv head); its rows are cut into *units* of 16
// tokens.  All units of the launch form one flat list that is divided evenly among the CTAs (one CTA per
// SM), so every SM streams the same number of bytes however the sequence lengths are distributed.  A CTA
// walks its contiguous unit range; when the range covers an item only partly the CTA writes an
// un-normalised partial (max, sum, acc[128]) per q head to global scratch and the last CTA to arrive at
// the item (an atomic counter, nobody waits) merges the partials and writes the output.
//
// Inside a CTA one producer warp stages tiles of up to 128 tokens (the rows of one kv head) into a
// shared-memory ring with bulk asynchronous copies completing on mbarriers; 8 consumer warps each take one
// 16-token unit of the tile, keep their own online-softmax state and are merged once per item.  All q
// heads of the kv head (GROUP of them) share every staged byte, so each cache byte is read once.
//
// The storage format is a policy (DensePolicy below, TurboMmaPolicy in flash_decode_turbo_mma.cuh) providing the
// stage layout, the copy issue, the Q register preparation and the per-unit arithmetic.
#pragma once

#include "er_common.cuh"

namespace er {

constexpr int kRowBytesF16 = kHeadDim * 2;                  // 256

struct DecodeParams {
    // Token-major fp16 rows only (use_tmap): tensor maps over [layer][seq][slot][kv head][128 halves] of K and V with a
    // box of one kv head x the policy's tile of slots, so a tile is one TMA load per tensor instead of a copy per row.
    CUtensorMap k_map, v_map;
    int use_tmap;
    const float* q;               // [layers][batch][num_q_heads][128]
    float* out;                   // same shape
    const uint8_t* k_base;        // first row of layer 0 (fp16 rows or packed codes)
    const uint8_t* v_base;
    int64_t k_layer_stride_bytes;
    int64_t v_layer_stride_bytes;
    const uint8_t* kn_base;       // TurboQuant: stored norms
    const uint8_t* vn_base;
    int64_t n_layer_stride_bytes;
    int norm_fp16;
    int32_t* lengths;             // device [total_layers][batch] tokens written; nullptr -> fixed_* below
    int fixed_kv_len;
    int fixed_q_pos;
    int layer_begin;
    int num_layers;               // layers covered by this launch
    int batch;
    int num_q_heads;
    const float* k_new;           // fused append: this step's K / V rows, [layers][batch][kv_heads][128] float
    const float* v_new;
    int fused_append;             // 1: the warp that owns the new row's unit converts it, uses it and stores it
    unsigned long long* trace;    // optional [gridDim.x][8] globaltimer stamps (diagnostics), else nullptr
    int pending;                  // rows appended but not yet committed to `lengths`
    // Sliding-window / ring-range attention over fp16 rows (gemma4_decode_gqa_f16kv_windowed, Shaders/Gemma4Decode.metal:236-283):
    // the rows visited are ring slots (start + i) % max_seq_len, i < count.  With `lengths`: window > 0 keeps the newest
    // min(window, rows written) rows; window == 0 visits slots [0, count) as before.  Without: start = fixed_start.
    int window;
    int fixed_start;
    int advance;                  // added to lengths[...] by the last CTA to finish
    // Diagnostics of the bounded waits: wait_limit_us > 0 replaces the 2 s patience of every mbarrier wait of the launch;
    // withhold_tiles = 1 makes the producer warp issue no copy at all, so the consumers' first wait runs out, the launch
    // walks its whole control flow with the abort flag set and the status word reads kStatusTimeout (outputs undefined).
    uint32_t wait_limit_us;
    int withhold_tiles;
    // kv-head sharding across GPUs: this launch computes num_q_heads of out_heads_total query heads (0 = not sharded) and
    // writes its rows at head offset out_head_offset of a [pair][out_heads_total][128] buffer -- its own (`out`) and the
    // same buffer at up to 8 more addresses (peer_out: the other GPUs' mapped buffers; a host-buffer step adds this GPU's own device buffer while `out` is host memory), so that every GPU ends the step holding all
    // heads without a separate all-gather.  Plain stores to peer memory; nothing is ever read from a peer.
    int out_heads_total;
    int out_head_offset;
    int num_peers;
    float* peer_out[8];
    float scale_log2;             // softmax scale * log2(e)
    float k_res_coef, v_res_coef; // balanced / aggressive TurboQuant rows: sqrt(pi / 2) * residual scale of each side
    float rope_scaling;
    int apply_rope;
    // fp16 policy only: per-head RMS norm of Q and of the fused-append K row before RoPE (fused_qk_norm_rope_neox,
    // Shaders/RoPE.metal:119-173); weights [layer][norm_stride], null = none
    const float* q_norm_w;
    const float* k_norm_w;
    int norm_stride;
    float rms_eps;
    KVAddressing addr;
    // Layers whose keys and values live in two caches (different row formats): the value cache's addressing and the layer
    // stride of its side array; k_* / kn_* / addr / lengths then describe the key cache, v_* / vn_* the value cache.
    KVAddressing addr_v;
    int64_t vn_layer_stride_bytes;
    float* scratch;               // [gridDim.x][2][GROUP][130]
    int* item_counters;           // [pairs * kv heads], zero between launches
    int* done_counter;            // zero between launches
    int* status;
    // Host-buffer steps (fp16 policies with the fused append): the step's q / k / v rows still lie in pinned, device-mapped
    // host memory at host_q / host_k / host_v (same shapes as q / k_new / v_new, which then name device staging buffers).
    // The producer warp of every CTA pulls the rows of the CTA's own item visits over the bus one visit ahead of the
    // consumers and stores them at q / k_new / v_new; the consumers wait on a counter in shared memory.  host_done (mapped
    // host memory, two ints) receives {host_epoch, status word} from the last CTA after every output row: the host waits
    // on it instead of on the stream.
    const float* host_q;
    const float* host_k;
    const float* host_v;
    int* host_done;
    int host_epoch;
    InvFreqTable inv_freq;
};

// 16-byte load that is never served from a stale cache line (mapped host memory changes between launches).
__device__ __forceinline__ float4 ld_volatile_f4(const float4* ptr) {
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(ptr) : "memory");
    return v;
}

template <class POL>
struct DecodeSmem {
    static constexpr int G = POL::kGroup;
    static constexpr int NW = POL::kUnitsPerTile * POL::kWarpGroups;   // consumer warps
    static constexpr int kOffPrefix = POL::kStages * POL::kStageBytes;
    static constexpr int kOffMergeAcc = kOffPrefix + (kMaxPairs + 4) * 4;
    static constexpr int kOffMergeML = kOffMergeAcc + NW * G * kHeadDim * 4;
    static constexpr int kOffProb = kOffMergeML + NW * G * 2 * 4;
    static constexpr int kOffCosSin = kOffProb + NW * G * kUnitTokens * 4;
    static constexpr int kOffBars = kOffCosSin + 2 * kHalfDim * 8;
    static constexpr int kOffFlags = kOffBars + 2 * POL::kStages * 8;
    static constexpr int kOffExtra = (kOffFlags + 32 + 127) & ~127;
    // kExtraBytes < 0: the policy lays its own tables out over everything up to the CTA maximum of 227 KB
    static constexpr int kTotal = POL::kExtraBytes < 0 ? 232448 : kOffExtra + POL::kExtraBytes;
};

__device__ __forceinline__ int64_t cta_range_start(int cta, int64_t total_units, int active) {
    return static_cast<int64_t>(cta) * total_units / active;
}
__device__ __forceinline__ int cta_of_unit(int64_t unit, int64_t total_units, int active) {
    return static_cast<int>(((unit + 1) * active - 1) / total_units);
}

// One (possibly partial) item visit of a CTA: units [u0, u1) of an item that has `units` units.
struct Segment {
    int pair, head, u0, u1, units;
    int64_t item_unit0;   // global index of the item's first unit
};

__device__ __forceinline__ Segment locate_segment(const int* prefix, int num_pairs, int hkv, int64_t cur,
                                                  int64_t range_end) {
    int lo = 0, hi = num_pairs;   // find the pair j with prefix[j]*hkv <= cur < prefix[j+1]*hkv
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (static_cast<int64_t>(prefix[mid]) * hkv <= cur) lo = mid; else hi = mid;
    }
    Segment s;
    s.pair = lo;
    s.units = prefix[lo + 1] - prefix[lo];
    const int64_t rel = cur - static_cast<int64_t>(prefix[lo]) * hkv;
    s.head = static_cast<int>(rel / s.units);
    s.u0 = static_cast<int>(rel % s.units);
    s.item_unit0 = cur - s.u0;
    const int64_t left = range_end - cur;
    s.u1 = (s.units - s.u0 <= left) ? s.units : s.u0 + static_cast<int>(left);
    return s;
}

__device__ __forceinline__ int kv_length(const DecodeParams& p, int pair) {
    if (p.lengths == nullptr) return p.fixed_kv_len;
    const int layer = p.layer_begin + pair / p.batch, seq = pair % p.batch;
    int n = p.lengths[layer * p.batch + seq] + p.pending;
    n = n < p.addr.max_seq_len ? n : p.addr.max_seq_len;
    return (p.window > 0 && p.window < n) ? p.window : n;
}

// First ring slot of the rows an item visits (count = kv_length of the pair).
__device__ __forceinline__ int kv_start(const DecodeParams& p, int pair, int count) {
    if (p.lengths == nullptr) return p.fixed_start;
    if (p.window <= 0) return 0;
    const int layer = p.layer_begin + pair / p.batch, seq = pair % p.batch;
    return (p.lengths[layer * p.batch + seq] + p.pending - count) % p.addr.max_seq_len;
}

// ------------------------------------------------------------------------------------------ dense fp16 policy

// Per-warp running state of one item in the lane-owns-dims form: lane holds output dims [4*lane, 4*lane+4) of every
// q head of the group, the running maximum / denominator (replicated over lanes) and its slice of the queries.
template <int GROUP, int QREGS>
struct LaneState {
    float q[GROUP][QREGS], m[GROUP], l[GROUP], acc[GROUP][4];
    __device__ __forceinline__ void reset() {
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
            m[g] = -INFINITY;
            l[g] = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[g][c] = 0.f;
        }
    }
    // ml: [GROUP][2] (max, denominator); accs: [GROUP][128] un-normalised outputs of this warp
    __device__ __forceinline__ void publish(float* ml, float* accs, int lane) const {
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
            if (lane == 0) {
                ml[g * 2] = m[g];
                ml[g * 2 + 1] = l[g];
            }
            *reinterpret_cast<float4*>(accs + g * kHeadDim + 4 * lane) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
        }
    }
};

// Tensor-core policies: fold a warp's running (max, denominator, O^T fragments) into the warp's merge buffer and restart
// the accumulators from zero.  The tensor cores add into their fp32 accumulators with truncation, so a long chain of
// accumulating mma instructions drifts by about half an ulp of the accumulator per instruction (measured on the prefill
// kernels: an error growing linearly with the context); folding every few units keeps each chain short and does the long
// sum in round-to-nearest fp32.  The buffer holds the same (max, denominator) / [head][128] layout State::publish writes,
// so the CTA-level merge is unchanged.  dim_of(t, g, second) maps fragment (m-tile t, row g or g + 8) to its output dim.
template <int GROUP, class DIM>
__device__ __forceinline__ void mma_state_fold(float (&m)[2], float (&l)[2], float (&acc)[8][4], float* ml, float* accs, int lane,
                                               bool first, float acc_scale, float l_scale, DIM dim_of) {
    const int g = lane >> 2, c = lane & 3;
    float wb[2], ws[2], mn[2], lb[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int h = 2 * c + e;
        const float mb = (first || h >= GROUP) ? -INFINITY : ml[h * 2];
        lb[e] = (first || h >= GROUP) ? 0.f : ml[h * 2 + 1];
        mn[e] = fmaxf(mb, m[e]);
        wb[e] = mb == -INFINITY ? 0.f : fast_exp2(mb - mn[e]);
        ws[e] = m[e] == -INFINITY ? 0.f : fast_exp2(m[e] - mn[e]);
    }
    __syncwarp();   // every lane has read the buffer's (max, denominator) before the g == 0 lanes replace them
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int h = 2 * c + e;
        if (h < GROUP) {
            if (g == 0) {
                ml[h * 2] = mn[e];
                ml[h * 2 + 1] = fmaf(lb[e], wb[e], l[e] * l_scale * ws[e]);
            }
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                float* a0 = accs + h * kHeadDim + dim_of(t, g, 0);
                float* a1 = accs + h * kHeadDim + dim_of(t, g, 1);
                *a0 = fmaf(first ? 0.f : *a0, wb[e], acc[t][e] * acc_scale * ws[e]);
                *a1 = fmaf(first ? 0.f : *a1, wb[e], acc[t][2 + e] * acc_scale * ws[e]);
            }
        }
        l[e] = 0.f;
    }
#pragma unroll
    for (int t = 0; t < 8; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;
    __syncwarp();
}

// One unit's step of the online softmax of the tensor-core policies: s = the thread's four scores (token g | g + 8) x (head 2c |
// 2c + 1) in the log2 domain (-inf where masked; token 0 of a unit is always valid), pr = their probabilities against the
// (possibly grown) running maxima.  The cross-lane maximum and the rescale of the accumulators run only when some score exceeds
// a running maximum; the denominators stay per-lane partial sums until the state is read (State::gather).
template <class ST>
__device__ __forceinline__ void mma_softmax_step(ST& st, const float (&s)[4], float (&pr)[4]) {
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
    pr[0] = fast_exp2(s[0] - m0); pr[1] = fast_exp2(s[1] - m1); pr[2] = fast_exp2(s[2] - m0); pr[3] = fast_exp2(s[3] - m1);
    st.l[0] += pr[0] + pr[2];
    st.l[1] += pr[1] + pr[3];
}

template <int GROUP, int UNITS_PER_TILE = 8, int WARP_GROUPS = 1, int STAGES = 3>
struct DensePolicy {
    static constexpr int kGroup = GROUP;
    static constexpr int kUnitsPerTile = UNITS_PER_TILE;   // 16-token units staged per tile, one consumer warp each
    static constexpr int kWarpGroups = WARP_GROUPS;        // consumer warp groups taking tiles round-robin
    static constexpr int kStages = STAGES;
    static constexpr int kTileBytesF16 = UNITS_PER_TILE * kUnitTokens * kRowBytesF16;   // per K or V tile
    static constexpr int kStageBytes = 2 * kTileBytesF16;
    static constexpr int kExtraBytes = 0;
    static constexpr bool kRotated = false;
    static constexpr int kFoldUnits = 0;   // scalar fp32 FMAs round to nearest: no accumulator folding
    __device__ static float* fin_ptr(uint8_t*) { return nullptr; }
    static constexpr bool kFusedAppend = true;
    // A warp group must meet consecutive phases of the stages it visits: tiles go to groups round-robin.
    static_assert(STAGES % WARP_GROUPS == 0, "STAGES must be a multiple of WARP_GROUPS");
    static constexpr int kQRegs = 16;   // per head: dims [8i,8i+8) then [64+8i,64+8i+8), i = lane % 8
    using State = LaneState<GROUP, kQRegs>;

    __device__ static bool init_extra(uint8_t*, int, int) { return true; }
    template <bool COHERENT = false>
    __device__ __forceinline__ static void load_q(const DecodeParams& p, State& st, const float* qrow, const float2* cs,
                                                  uint8_t* extra, int warp, int lane, int layer) {
        load_q<COHERENT>(p, st.q, qrow, cs, extra, warp, lane, p.q_norm_w ? p.q_norm_w + static_cast<int64_t>(layer) * p.norm_stride : nullptr);
        st.reset();
    }
    __device__ __forceinline__ static void process_unit(const DecodeParams& p, const uint8_t* stage, int unit, int nvalid,
                                                        State& st, float* prob, const uint8_t* extra, int lane) {
        process_unit(p, stage, unit, nvalid, st.q, st.m, st.l, st.acc, prob, extra, lane);
    }

    // Producer: K and V rows [t0, t0+ntok) of (layer, seq, head) -> stage.  Token-major storage needs one
    // 256-byte copy per row; page-major storage one copy per touched page.
    template <class WAIT>
    __device__ static void issue_tile(const DecodeParams& p, uint8_t* stage, uint64_t* bar, int layer, int seq,
                                      int head, int t0, int ntok, int lane, int start, WAIT&& wait_free) {
        const uint8_t* kl = p.k_base + static_cast<int64_t>(layer) * p.k_layer_stride_bytes;
        const uint8_t* vl = p.v_base + static_cast<int64_t>(layer) * p.v_layer_stride_bytes;
        if (start == 0 && !p.use_tmap && !p.addr.token_major && p.addr.pages_per_seq != 0) {
            // Paged rows: each lane looks its page up in the block table BEFORE waiting for the stage, so that the
            // dependent global read overlaps the time the consumers still need (it sat on the refill path otherwise).
            const int ps = p.addr.page_size;
            const int first_page = t0 / ps;
            const int ncopy = 2 * ((t0 + ntok - 1) / ps - first_page + 1);
            const int tb = max(t0, (first_page + (lane >> 1)) * ps);
            const int te = min(t0 + ntok, (first_page + (lane >> 1) + 1) * ps);
            const int64_t row = lane < ncopy ? row_index(p.addr, seq, head, tb) : 0;
            wait_free();
            if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(ntok) * kRowBytesF16 * 2);
            __syncwarp();
            if (lane < ncopy)
                bulk_g2s(stage + (lane & 1) * kTileBytesF16 + (tb - t0) * kRowBytesF16, ((lane & 1) ? vl : kl) + row * kRowBytesF16,
                         static_cast<uint32_t>(te - tb) * kRowBytesF16, bar);
            for (int c = lane + 32; c < ncopy; c += 32) {
                const int is_v = c & 1, sgi = c >> 1;
                const int b = max(t0, (first_page + sgi) * ps);
                const int e = min(t0 + ntok, (first_page + sgi + 1) * ps);
                bulk_g2s(stage + is_v * kTileBytesF16 + (b - t0) * kRowBytesF16,
                         (is_v ? vl : kl) + row_index(p.addr, seq, head, b) * kRowBytesF16, static_cast<uint32_t>(e - b) * kRowBytesF16, bar);
            }
            return;
        }
        wait_free();
        if (start != 0) {
            // Ring range: row t of the item sits in slot (start + t) % max_seq_len, so a tile is one or two slot runs.
            if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(ntok) * kRowBytesF16 * 2);
            __syncwarp();
            const int cap = p.addr.max_seq_len;
            const int s0 = (start + t0) % cap;
            const int n0 = min(ntok, cap - s0);
            issue_rows(p, stage, bar, kl, vl, seq, head, s0, n0, lane);
            if (n0 < ntok) issue_rows(p, stage + n0 * kRowBytesF16, bar, kl, vl, seq, head, 0, ntok - n0, lane);
            return;
        }
        if (p.use_tmap) {
            if (lane == 0) {
                mbar_arrive_expect_tx(bar, 2u * kTileBytesF16);
                tma_load_5d(stage, &p.k_map, 0, head, t0, seq, layer, bar);
                tma_load_5d(stage + kTileBytesF16, &p.v_map, 0, head, t0, seq, layer, bar);
            }
            __syncwarp();
            return;
        }
        if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(ntok) * kRowBytesF16 * 2);
        __syncwarp();
        issue_rows(p, stage, bar, kl, vl, seq, head, t0, ntok, lane);
    }

    // K and V rows of slots [t0, t0+ntok) -> stage (K tile) and stage + kTileBytesF16 (V tile); the caller has armed `bar`.
    __device__ __forceinline__ static void issue_rows(const DecodeParams& p, uint8_t* stage, uint64_t* bar, const uint8_t* kl,
                                                      const uint8_t* vl, int seq, int head, int t0, int ntok, int lane) {
        if (p.addr.token_major) {
            for (int c = lane; c < 2 * ntok; c += 32) {
                const int is_v = c >= ntok;
                const int r = is_v ? c - ntok : c;
                const int64_t row = row_index(p.addr, seq, head, t0 + r);
                bulk_g2s(stage + is_v * kTileBytesF16 + r * kRowBytesF16, (is_v ? vl : kl) + row * kRowBytesF16,
                         kRowBytesF16, bar);
            }
        } else {
            const int ps = p.addr.page_size;
            const int first_page = t0 / ps;
            const int nseg = (t0 + ntok - 1) / ps - first_page + 1;
            for (int c = lane; c < 2 * nseg; c += 32) {
                const int is_v = c & 1, sgi = c >> 1;
                const int tb = max(t0, (first_page + sgi) * ps);
                const int te = min(t0 + ntok, (first_page + sgi + 1) * ps);
                const int64_t row = row_index(p.addr, seq, head, tb);
                bulk_g2s(stage + is_v * kTileBytesF16 + (tb - t0) * kRowBytesF16, (is_v ? vl : kl) + row * kRowBytesF16,
                         static_cast<uint32_t>(te - tb) * kRowBytesF16, bar);
            }
        }
    }

    // Consumers: per-lane Q registers, NeoX-rotated in registers when asked.
    template <bool COHERENT = false>
    __device__ static void load_q(const DecodeParams& p, float (&q)[GROUP][kQRegs], const float* qrow, const float2* cs,
                                  uint8_t*, int, int lane, const float* qw) {
        const int i = lane & 7;
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
            const float4* src = reinterpret_cast<const float4*>(qrow + g * kHeadDim + 8 * i);
            const float4 a0 = ld_step_row<COHERENT>(src), a1 = ld_step_row<COHERENT>(src + 1), b0 = ld_step_row<COHERENT>(src + 16), b1 = ld_step_row<COHERENT>(src + 17);
            float xa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            float xb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            if (qw != nullptr) {
                const float rs = head_rms_scale<COHERENT>(qrow + g * kHeadDim, p.rms_eps, lane);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    xa[c] = __fmul_rn(__fmul_rn(xa[c], rs), __ldg(qw + 8 * i + c));
                    xb[c] = __fmul_rn(__fmul_rn(xb[c], rs), __ldg(qw + 64 + 8 * i + c));
                }
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                if (p.apply_rope) {
                    rope_rotate(xa[c], xb[c], cs[8 * i + c], q[g][c], q[g][8 + c]);
                } else {
                    q[g][c] = xa[c];
                    q[g][8 + c] = xb[c];
                }
            }
        }
    }

    // Scores, online softmax and P.V of one 16-token unit held in shared memory.
    //   QK: lane (j = lane/8, i = lane%8) visits rows 4r+j, r = 0..3 -> two conflict-free 16-byte reads per
    //       row; an 8-lane butterfly finishes the dot product.
    //   PV: lane owns output dims [4*lane, 4*lane+4) and walks the 16 rows (one 8-byte read each).
    __device__ static void process_unit(const DecodeParams& p, const uint8_t* stage, int unit, int nvalid,
                                        const float (&q)[GROUP][kQRegs], float (&m)[GROUP], float (&l)[GROUP],
                                        float (&acc)[GROUP][4], float* prob, const uint8_t*, int lane) {
        const uint8_t* ks = stage + unit * kUnitTokens * kRowBytesF16;
        const uint8_t* vs = stage + kTileBytesF16 + unit * kUnitTokens * kRowBytesF16;
        const int j = lane >> 3, i = lane & 7;
        float s[4][GROUP];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int row = 4 * r + j;
            const uint4 ka = *reinterpret_cast<const uint4*>(ks + row * kRowBytesF16 + i * 16);
            const uint4 kb = *reinterpret_cast<const uint4*>(ks + row * kRowBytesF16 + 128 + i * 16);
            float fa[8], fb[8];
            unpack8(ka, fa);
            unpack8(kb, fb);
#pragma unroll
            for (int g = 0; g < GROUP; ++g) {
                float d0 = 0.f, d1 = 0.f;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    d0 = fmaf(q[g][c], fa[c], d0);
                    d1 = fmaf(q[g][8 + c], fb[c], d1);
                }
                s[r][g] = d0 + d1;
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int g = 0; g < GROUP; ++g) {
                float v = s[r][g];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                s[r][g] = (4 * r + j < nvalid) ? v * p.scale_log2 : -INFINITY;
            }
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
            float mx = fmaxf(fmaxf(s[0][g], s[1][g]), fmaxf(s[2][g], s[3][g]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(m[g], mx);               // finite: the unit has at least one valid row
            const float corr = fast_exp2(m[g] - m_new);        // m == -inf -> 0
            float psum = 0.f;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float pr = fast_exp2(s[r][g] - m_new);   // masked rows -> 0
                psum += pr;
                if (i == 0) prob[g * kUnitTokens + 4 * r + j] = pr;
            }
            psum += __shfl_xor_sync(0xffffffffu, psum, 8);
            psum += __shfl_xor_sync(0xffffffffu, psum, 16);
            l[g] = fmaf(l[g], corr, psum);
            m[g] = m_new;
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[g][c] *= corr;
        }
        __syncwarp();
        const uint8_t* vrow = vs + lane * 8;
        if (nvalid == kUnitTokens) {
#pragma unroll
            for (int t4 = 0; t4 < kUnitTokens; t4 += 4) {
                float4 pg[GROUP];
#pragma unroll
                for (int g = 0; g < GROUP; ++g) pg[g] = *reinterpret_cast<const float4*>(prob + g * kUnitTokens + t4);
#pragma unroll
                for (int tt = 0; tt < 4; ++tt) {
                    float vf[4];
                    unpack4(*reinterpret_cast<const uint2*>(vrow + (t4 + tt) * kRowBytesF16), vf);
#pragma unroll
                    for (int g = 0; g < GROUP; ++g) {
                        const float w = tt == 0 ? pg[g].x : tt == 1 ? pg[g].y : tt == 2 ? pg[g].z : pg[g].w;
#pragma unroll
                        for (int c = 0; c < 4; ++c) acc[g][c] = fmaf(w, vf[c], acc[g][c]);
                    }
                }
            }
        } else {
            for (int t = 0; t < nvalid; ++t) {   // rows past nvalid were never copied: do not touch them
                float vf[4];
                unpack4(*reinterpret_cast<const uint2*>(vrow + t * kRowBytesF16), vf);
#pragma unroll
                for (int g = 0; g < GROUP; ++g) {
                    const float w = prob[g * kUnitTokens + t];
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[g][c] = fmaf(w, vf[c], acc[g][c]);
                }
            }
        }
        __syncwarp();
    }

    // Fused append (rope_neox_f32_to_f16 + convert_f32_to_f16 of the decode pass, Shaders/RoPE.metal:498-531,
    // LlamaLanguageModel.swift:3676-3684): the warp whose unit holds the new token's slot converts the new K/V
    // row into the staged tile (so attention sees it) and stores both rows to the cache with 16-byte stores.
    template <bool COHERENT = false>
    __device__ static void patch_new_row(const DecodeParams& p, uint8_t* stage, int unit, int r, int layer, int seq,
                                         int head, int slot, const float* k_src, const float* v_src, const float2* cs,
                                         int lane) {
        uint8_t* krow = stage + (unit * kUnitTokens + r) * kRowBytesF16;
        uint8_t* vrow = stage + kTileBytesF16 + (unit * kUnitTokens + r) * kRowBytesF16;
        __half* kh = reinterpret_cast<__half*>(krow);
        const float* kw = p.k_norm_w ? p.k_norm_w + static_cast<int64_t>(layer) * p.norm_stride : nullptr;
        const float rs = kw ? head_rms_scale<COHERENT>(k_src, p.rms_eps, lane) : 1.f;
#pragma unroll
        for (int part = 0; part < 2; ++part) {
            const int d = lane + 32 * part;
            float x0 = ld_step_row<COHERENT>(k_src + d), x1 = ld_step_row<COHERENT>(k_src + d + kHalfDim);
            if (kw != nullptr) {
                x0 = __fmul_rn(__fmul_rn(x0, rs), __ldg(kw + d));
                x1 = __fmul_rn(__fmul_rn(x1, rs), __ldg(kw + d + kHalfDim));
            }
            if (p.apply_rope) {
                float y0, y1;
                rope_rotate(x0, x1, cs[d], y0, y1);
                x0 = y0;
                x1 = y1;
            }
            kh[d] = __float2half_rn(x0);
            kh[d + kHalfDim] = __float2half_rn(x1);
        }
        const float4 v4 = ld_step_row<COHERENT>(reinterpret_cast<const float4*>(v_src) + lane);
        uint2 vv;
        reinterpret_cast<__half2*>(&vv)[0] = __halves2half2(__float2half_rn(v4.x), __float2half_rn(v4.y));
        reinterpret_cast<__half2*>(&vv)[1] = __halves2half2(__float2half_rn(v4.z), __float2half_rn(v4.w));
        reinterpret_cast<uint2*>(vrow)[lane] = vv;
        __syncwarp();
        const int64_t row = row_index_for_write(p.addr, seq, head, slot);
        const bool is_v = lane >= 16;
        const uint4 val = *reinterpret_cast<const uint4*>((is_v ? vrow : krow) + (lane & 15) * 16);
        uint8_t* dst = const_cast<uint8_t*>(is_v ? p.v_base + static_cast<int64_t>(layer) * p.v_layer_stride_bytes
                                                 : p.k_base + static_cast<int64_t>(layer) * p.k_layer_stride_bytes);
        if (row >= 0)   // a slot without a page keeps the row out of the cache (status word set)
            *reinterpret_cast<uint4*>(dst + row * kRowBytesF16 + (lane & 15) * 16) = val;
        // generic-proxy writes to the stage precede its next refill by the async proxy
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }

    __device__ static void store_out(const DecodeParams&, int64_t, const float*, int, int) {}
};

// ------------------------------------------------------------------------------------------ the kernel

// HOSTIO: the variant that pulls the step's rows out of mapped host memory and reports to a host word (host-buffer steps on
// fused-append policies); a separate instantiation, so that the ordinary launch carries none of its code.
template <class POL, bool HOSTIO = false>
__global__ void __launch_bounds__((POL::kUnitsPerTile * POL::kWarpGroups + 1) * 32, 1)
flash_decode_kernel(const __grid_constant__ DecodeParams p) {
    static_assert(!HOSTIO || POL::kFusedAppend, "host rows are pulled by the policies that append the new row themselves");
    using L = DecodeSmem<POL>;
    constexpr int GROUP = POL::kGroup;
    constexpr int kStages = POL::kStages;
    constexpr int UPT = POL::kUnitsPerTile;          // units (= consumer warps of one group) per tile
    constexpr int NG = POL::kWarpGroups;
    constexpr int NW = UPT * NG;                     // consumer warps; warp NW is the producer
    extern __shared__ __align__(128) uint8_t smem[];
    int* prefix = reinterpret_cast<int*>(smem + L::kOffPrefix);
    float* merge_acc = reinterpret_cast<float*>(smem + L::kOffMergeAcc);
    float* merge_ml = reinterpret_cast<float*>(smem + L::kOffMergeML);
    float* prob_all = reinterpret_cast<float*>(smem + L::kOffProb);
    float2* cos_sin = reinterpret_cast<float2*>(smem + L::kOffCosSin);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kOffBars);
    uint64_t* empty_bar = full_bar + kStages;
    volatile int* flags = reinterpret_cast<volatile int*>(smem + L::kOffFlags);   // [0] abort [1] item-last [2] grid-last [3] item visits whose host rows have landed
    uint8_t* extra = smem + L::kOffExtra;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hkv = p.addr.num_kv_heads;
    auto stamp = [&](int slot) {   // diagnostics: per-CTA phase times
        if (p.trace != nullptr) p.trace[blockIdx.x * 8 + slot] = global_timer_ns();
    };
    const int num_pairs = p.num_layers * p.batch;

    // let the next kernel of the stream be placed as this one's CTAs leave (it waits below before reading anything)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        flags[0] = 0; flags[1] = 0; flags[2] = 0; flags[3] = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], UPT);
        }
        mbar_init_fence();
    }
    if (!POL::init_extra(extra, tid, L::kTotal - L::kOffExtra)) {   // CTA-uniform: the policy's shared-memory plan does not fit
        if (tid == 0) atomicExch(p.status, kStatusBadLayout);
        return;
    }
    // everything above touches shared memory only; global memory (lengths, cache rows, scratch, counters, trace) belongs to
    // the previous kernel of the stream until it has completed
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) stamp(0);
    // ---- unit prefix over (layer, sequence) pairs: all threads fetch the lengths (one round of global reads), warp 0
    // turns the unit counts into an exclusive scan in place ----
    {
        int len[8];   // eight independent reads in flight per thread, then the (never needed at >= 256 threads) remainder
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int j = tid + i * static_cast<int>(blockDim.x);
            len[i] = j < num_pairs ? kv_length(p, j) : 0;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int j = tid + i * static_cast<int>(blockDim.x);
            if (j < num_pairs) prefix[j] = (len[i] + kUnitTokens - 1) / kUnitTokens;
        }
        for (int j = tid + 8 * static_cast<int>(blockDim.x); j < num_pairs; j += blockDim.x)
            prefix[j] = (kv_length(p, j) + kUnitTokens - 1) / kUnitTokens;
    }
    __syncthreads();
    if (warp == 0) {   // 32 consecutive entries per pass (conflict-free), running total carried in registers
        int carry = 0;
        for (int base = 0; base < num_pairs; base += 32) {
            const int j = base + lane;
            const int units = j < num_pairs ? prefix[j] : 0;
            int incl = units;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            if (j < num_pairs) prefix[j] = carry + incl - units;
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) prefix[num_pairs] = carry;
    }
    __syncthreads();
    if (tid == 0) stamp(1);

    const int64_t total_units = static_cast<int64_t>(prefix[num_pairs]) * hkv;
    int active = static_cast<int>(min(static_cast<int64_t>(gridDim.x), (total_units + UPT - 1) / UPT));
    const int cta = blockIdx.x;

    const int out_heads = p.out_heads_total > 0 ? p.out_heads_total : p.num_q_heads;   // heads per row of the output buffer
    // Sequences without any row produce a zero output row (invSum = 0 rule, Shaders/GQA.metal:379).
    for (int j = cta; j < num_pairs; j += gridDim.x) {
        if (prefix[j + 1] == prefix[j]) {
            const int64_t off = (static_cast<int64_t>(j) * out_heads + p.out_head_offset) * kHeadDim;
            for (int e = tid; e < p.num_q_heads * kHeadDim; e += blockDim.x) {
                p.out[off + e] = 0.f;
                for (int r = 0; r < p.num_peers; ++r) p.peer_out[r][off + e] = 0.f;
            }
        }
    }

    if (cta < active && total_units > 0) {
        const int64_t range_begin = cta_range_start(cta, total_units, active);
        const int64_t range_end = cta_range_start(cta + 1, total_units, active);

        const uint64_t wait_ns = p.wait_limit_us > 0 ? static_cast<uint64_t>(p.wait_limit_us) * 1000ull : 2000000000ull;
        if (warp == NW) {
            // ================= producer warp =================
            int k = 0;
            int64_t cur = p.withhold_tiles ? range_end : range_begin;
            // host-buffer step: rows of the next item visit, in flight over the bus while this visit's tiles are issued
            constexpr bool hostio = HOSTIO;
            float4 hq_r[GROUP], hk_r = make_float4(0.f, 0.f, 0.f, 0.f), hv_r = hk_r;
            int64_t hq_off = 0, hkv_off = 0;
            int landed = 0;
            auto host_load = [&](const Segment& s2) {
                hq_off = (static_cast<int64_t>(s2.pair) * p.num_q_heads + s2.head * GROUP) * kHeadDim;
                hkv_off = (static_cast<int64_t>(s2.pair) * hkv + s2.head) * kHeadDim;
#pragma unroll
                for (int g = 0; g < GROUP; ++g) hq_r[g] = ld_volatile_f4(reinterpret_cast<const float4*>(p.host_q + hq_off) + g * 32 + lane);
                hk_r = ld_volatile_f4(reinterpret_cast<const float4*>(p.host_k + hkv_off) + lane);
                hv_r = ld_volatile_f4(reinterpret_cast<const float4*>(p.host_v + hkv_off) + lane);
            };
            auto host_store = [&]() {   // the loaded rows become the staged rows of their visit; then the consumers may start it
#pragma unroll
                for (int g = 0; g < GROUP; ++g) reinterpret_cast<float4*>(const_cast<float*>(p.q) + hq_off)[g * 32 + lane] = hq_r[g];
                reinterpret_cast<float4*>(const_cast<float*>(p.k_new) + hkv_off)[lane] = hk_r;
                reinterpret_cast<float4*>(const_cast<float*>(p.v_new) + hkv_off)[lane] = hv_r;
                __threadfence();
                __syncwarp();
                if (lane == 0) flags[3] = ++landed;
            };
            if constexpr (hostio) { if (cur < range_end) host_load(locate_segment(prefix, num_pairs, hkv, cur, range_end)); }
            while (cur < range_end) {
                const Segment sg = locate_segment(prefix, num_pairs, hkv, cur, range_end);
                const int layer = p.layer_begin + sg.pair / p.batch, seq = sg.pair % p.batch;
                const int kv_len = kv_length(p, sg.pair);
                const int start = kv_start(p, sg.pair, kv_len);
                [[maybe_unused]] bool rows_pending = hostio;   // staged right after the visit's first tile is on its way
                if (!hostio) {
                    // The consumers read this item's query rows (and the new K/V row) only when they get here, several tiles
                    // later: pull the lines into L2 now so that the item switch does not wait on DRAM.
                    if (lane < GROUP * 4)
                        prefetch_l2(reinterpret_cast<const uint8_t*>(p.q + (static_cast<int64_t>(sg.pair) * p.num_q_heads + sg.head * GROUP) * kHeadDim) + lane * 128);
                    if (POL::kFusedAppend && p.fused_append && lane >= 24) {
                        const int64_t off = (static_cast<int64_t>(sg.pair) * hkv + sg.head) * kHeadDim * 4 + (lane & 3) * 128;
                        prefetch_l2(reinterpret_cast<const uint8_t*>((lane & 4) ? p.v_new : p.k_new) + off);
                    }
                }
                for (int tu = sg.u0; tu < sg.u1; tu += UPT, ++k) {
                    const int nun = min(UPT, sg.u1 - tu);
                    const int t0 = tu * kUnitTokens;
                    const int ntok = min(kv_len, (tu + nun) * kUnitTokens) - t0;
                    const int s = k % kStages;
                    // the policy calls this once, after any address lookups that can run while the stage is still busy
                    auto wait_free = [&]() {
                        if (k >= kStages) mbar_wait(&empty_bar[s], ((k / kStages) - 1) & 1, &flags[0], p.status, wait_ns);
                    };
                    POL::issue_tile(p, smem + s * POL::kStageBytes, &full_bar[s], layer, seq, sg.head, t0, ntok, lane, start, wait_free);
                    if constexpr (hostio) {
                        if (rows_pending) {
                            rows_pending = false;
                            host_store();
                            const int64_t nxt = cur + (sg.u1 - sg.u0);
                            if (nxt < range_end) host_load(locate_segment(prefix, num_pairs, hkv, nxt, range_end));
                        }
                    }
                }
                cur += sg.u1 - sg.u0;
            }
        } else {
            // ================= consumer warps =================
            float* prob = prob_all + warp * GROUP * kUnitTokens;
            const int wgroup = warp / UPT, wunit = warp % UPT;   // tiles k with k % NG == wgroup are this warp's
            int k = 0, cs_buf = 0, cs_pos = -1, visit = 0;
            int64_t cur = range_begin;
            while (cur < range_end) {
                const Segment sg = locate_segment(prefix, num_pairs, hkv, cur, range_end);
                const int layer = p.layer_begin + sg.pair / p.batch, seq = sg.pair % p.batch;
                const int kv_len = kv_length(p, sg.pair);
                const int q_pos = (p.lengths == nullptr) ? p.fixed_q_pos : p.lengths[layer * p.batch + seq] + p.pending - 1;
                // The (cos, sin) table depends on the position only: the kv heads of a sequence and all layers of a sequence
                // share it, so it is rebuilt (double-precision sincos) only when the position changes.  Two buffers: a
                // rebuild never touches the one the previous visit's stragglers may still be reading.
                if (p.apply_rope && q_pos != cs_pos) {
                    cs_buf ^= 1;
                    cs_pos = q_pos;
                    if (tid < kHalfDim)
                        cos_sin[cs_buf * kHalfDim + tid] = rope_cos_sin(static_cast<uint32_t>(q_pos), p.inv_freq.f[tid], p.rope_scaling);
                }
                float2* cs = cos_sin + cs_buf * kHalfDim;
                consumer_sync<NW * 32>();
                if constexpr (HOSTIO) {   // the producer warp has this visit's host rows staged?
                    if (flags[3] <= visit && !flags[0]) {
                        const uint64_t t_start = global_timer_ns();
                        uint32_t spins = 0;
                        while (flags[3] <= visit && !flags[0]) {
                            if ((++spins & 0xFFu) == 0u && global_timer_ns() - t_start > wait_ns) {
                                flags[0] = 1;
                                atomicExch(p.status, kStatusTimeout);
                            }
                        }
                    }
                    __threadfence();
                    ++visit;
                }

                typename POL::State st;
                const float* qrow = p.q + (static_cast<int64_t>(sg.pair) * p.num_q_heads + sg.head * GROUP) * kHeadDim;
                if constexpr (HOSTIO) POL::template load_q<true>(p, st, qrow, cs, extra, warp, lane, layer);
                else POL::load_q(p, st, qrow, cs, extra, warp, lane, layer);

                float* my_ml = merge_ml + warp * GROUP * 2;
                float* my_acc = merge_acc + warp * GROUP * kHeadDim;
                int since_fold = 0;
                bool folded = false;
                for (int tu = sg.u0; tu < sg.u1; tu += UPT, ++k) {
                    if (NG > 1 && k % NG != wgroup) continue;
                    const int nun = min(UPT, sg.u1 - tu);
                    const int t0 = tu * kUnitTokens;
                    const int ntok = min(kv_len, (tu + nun) * kUnitTokens) - t0;
                    const int s = k % kStages;
                    mbar_wait(&full_bar[s], (k / kStages) & 1, &flags[0], p.status, wait_ns);
                    if (k == 0 && tid == 0) stamp(2);
                    if (POL::kFusedAppend && p.fused_append && !flags[0]) {
                        const int slot_new = q_pos % p.addr.max_seq_len;
                        const int row_new = p.window > 0 ? kv_len - 1 : slot_new;   // the newest row closes a window
                        if (wunit < nun && tu + wunit == (row_new >> 4)) {
                            if constexpr (HOSTIO) POL::template patch_new_row<true>(p, smem + s * POL::kStageBytes, wunit, row_new & 15, layer, seq, sg.head, slot_new,
                                               p.k_new + (static_cast<int64_t>(sg.pair) * hkv + sg.head) * kHeadDim,
                                               p.v_new + (static_cast<int64_t>(sg.pair) * hkv + sg.head) * kHeadDim, cs, lane);
                            else POL::patch_new_row(p, smem + s * POL::kStageBytes, wunit, row_new & 15, layer, seq, sg.head, slot_new,
                                               p.k_new + (static_cast<int64_t>(sg.pair) * hkv + sg.head) * kHeadDim,
                                               p.v_new + (static_cast<int64_t>(sg.pair) * hkv + sg.head) * kHeadDim, cs, lane);
                        }
                    }
                    if (wunit < nun && !flags[0]) {
                        const int nvalid = min(kUnitTokens, ntok - wunit * kUnitTokens);
                        POL::process_unit(p, smem + s * POL::kStageBytes, wunit, nvalid, st, prob, extra, lane);
                        if constexpr (POL::kFoldUnits > 0) {
                            if (++since_fold == POL::kFoldUnits) {   // keep the tensor cores' accumulation chains short
                                st.fold(my_ml, my_acc, lane, !folded);
                                folded = true;
                                since_fold = 0;
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty_bar[s]);
                }

                if (tid == 0) stamp(3);   // last write wins: end of this CTA's streaming
                // ---- merge the consumer warps of this CTA ----
                if constexpr (POL::kFoldUnits > 0) {
                    if (folded) st.fold(my_ml, my_acc, lane, false); else st.publish(my_ml, my_acc, lane);
                } else {
                    st.publish(my_ml, my_acc, lane);
                }
                consumer_sync<NW * 32>();
                const bool sole = (sg.u0 == 0 && sg.u1 == sg.units);
                const int item = sg.pair * hkv + sg.head;
                const int64_t out_off = (static_cast<int64_t>(sg.pair) * out_heads + p.out_head_offset + sg.head * GROUP) * kHeadDim;
                float* out_item = p.out + out_off;
                // Outputs of the rotated (TurboQuant) space pass through shared memory for the inverse transform.
                float* fin = POL::kRotated ? POL::fin_ptr(extra) : out_item;
                auto emit = [&](int idx, float val) {   // a finished output element: local buffer (or staging) + the peers' copies
                    fin[idx] = val;
                    if (!POL::kRotated)
                        for (int r = 0; r < p.num_peers; ++r) p.peer_out[r][out_off + idx] = val;
                };
                const int slot = (range_begin > sg.item_unit0) ? 0 : 1;
                float* my_scratch = p.scratch + (static_cast<int64_t>(cta) * 2 + slot) * GROUP * 130;
                for (int idx = tid; idx < GROUP * kHeadDim; idx += NW * 32) {
                    const int g = idx >> 7, d = idx & 127;
                    float M = -INFINITY;
#pragma unroll
                    for (int w = 0; w < NW; ++w) M = fmaxf(M, merge_ml[(w * GROUP + g) * 2]);
                    float Lsum = 0.f, A = 0.f;
#pragma unroll
                    for (int w = 0; w < NW; ++w) {
                        const float wgt = fast_exp2(merge_ml[(w * GROUP + g) * 2] - M);
                        Lsum = fmaf(merge_ml[(w * GROUP + g) * 2 + 1], wgt, Lsum);
                        A = fmaf(merge_acc[(w * GROUP + g) * kHeadDim + d], wgt, A);
                    }
                    if (sole) {
                        emit(idx, Lsum > 0.f ? A / Lsum : 0.f);
                    } else {
                        if (d == 0) {
                            my_scratch[g * 130] = M;
                            my_scratch[g * 130 + 1] = Lsum;
                        }
                        my_scratch[g * 130 + 2 + d] = A;
                    }
                }
                bool wrote = sole;
                if (!sole) {
                    const int64_t item_end = sg.item_unit0 + sg.units;
                    const int c_first = cta_of_unit(sg.item_unit0, total_units, active);
                    const int c_last = cta_of_unit(item_end - 1, total_units, active);
                    __threadfence();
                    consumer_sync<NW * 32>();
                    if (tid == 0) {
                        const int prev = atomicAdd(p.item_counters + item, 1);
                        flags[1] = (prev == c_last - c_first) ? 1 : 0;
                    }
                    consumer_sync<NW * 32>();
                    if (flags[1]) {
                        wrote = true;
                        __threadfence();
                        // Only the first contributor can have started at or before the item: every later one
                        // begins inside it and therefore used slot 0.
                        const int first_slot = (cta_range_start(c_first, total_units, active) > sg.item_unit0) ? 0 : 1;
                        const float* first_partial = p.scratch + (static_cast<int64_t>(c_first) * 2 + first_slot) * GROUP * 130;
                        const int ncontrib = c_last - c_first + 1;
                        for (int idx = tid; idx < GROUP * kHeadDim; idx += NW * 32) {
                            const int g = idx >> 7, d = idx & 127;
                            float M = __ldcg(first_partial + g * 130);
#pragma unroll 4
                            for (int c = 1; c < ncontrib; ++c)
                                M = fmaxf(M, __ldcg(p.scratch + static_cast<int64_t>(c_first + c) * 2 * GROUP * 130 + g * 130));
                            float wgt = fast_exp2(__ldcg(first_partial + g * 130) - M);
                            float Lsum = __ldcg(first_partial + g * 130 + 1) * wgt;
                            float A = __ldcg(first_partial + g * 130 + 2 + d) * wgt;
#pragma unroll 4
                            for (int c = 1; c < ncontrib; ++c) {
                                const float* sc = p.scratch + static_cast<int64_t>(c_first + c) * 2 * GROUP * 130 + g * 130;
                                wgt = fast_exp2(__ldcg(sc) - M);
                                Lsum = fmaf(__ldcg(sc + 1), wgt, Lsum);
                                A = fmaf(__ldcg(sc + 2 + d), wgt, A);
                            }
                            emit(idx, Lsum > 0.f ? A / Lsum : 0.f);
                        }
                        if (tid == 0) p.item_counters[item] = 0;
                    }
                }
                if (POL::kRotated && wrote) {   // CTA-uniform condition
                    consumer_sync<NW * 32>();
                    POL::store_out(p, out_off, fin, warp, lane);
                }
                cur += sg.u1 - sg.u0;
            }
        }
    }

    // ---- the last CTA to finish commits the new row: lengths += advance ----
    if (tid == 0) stamp(4);
    __syncthreads();
    if (tid == 0) stamp(5);
    if (tid == 0) {
        if constexpr (HOSTIO) __threadfence_system(); else __threadfence();   // HOSTIO: output rows may lie in host memory
        const int prev = atomicAdd(p.done_counter, 1);
        flags[2] = (prev == static_cast<int>(gridDim.x) - 1) ? 1 : 0;
    }
    __syncthreads();
    if (flags[2]) {
        if (p.advance != 0 && p.lengths != nullptr)
            for (int e = tid; e < num_pairs; e += blockDim.x) p.lengths[p.layer_begin * p.batch + e] += p.advance;
        if (tid == 0) {
            *p.done_counter = 0;
            if (HOSTIO && p.host_done != nullptr) {   // every CTA's rows are out (their fences precede the counter): tell the host
                __threadfence_system();
                const int st = *reinterpret_cast<volatile int*>(p.status);
                reinterpret_cast<volatile int*>(p.host_done)[1] = st;
                __threadfence_system();
                reinterpret_cast<volatile int*>(p.host_done)[0] = p.host_epoch;
            }
        }
    }
    if (tid == 0) stamp(6);
}

}  // namespace er
