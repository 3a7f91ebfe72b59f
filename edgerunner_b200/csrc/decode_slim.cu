// Decode attention over fp16 rows for SMALL launches: one layer of a small batch (a few MB to a few tens of MB of K / V),
// the shape of the reference's per-layer dispatch (fusedDecodePass issues gqa_attention_f16kv once per layer,
// Sources/EdgeRunner/Models/LlamaLanguageModel.swift:3867-3881).  The persistent kernel (flash_decode.cuh) is built for
// launches that keep every SM streaming for tens of microseconds: its 220 KB shared-memory prologue, work-list scan and
// mbarrier ring cost ~15 us before they pay off.  Here there is no ring and no producer warp: the grid is (split, kv head,
// (layer, sequence)), a CTA's token range holds at most one 16-token unit per warp, and every warp fetches its own unit
// with one bulk asynchronous copy per tensor (completion on the warp's own mbarrier, bounded wait) -- all of a CTA's
// rows are in flight at once, which plain loads into registers cannot do (an SM tracks too few outstanding loads:
// 2.6 TB/s measured that way).  The arithmetic is DensePolicy's (process_unit, load_q, patch_new_row: the new token's K / V
// row is converted with the exactly rounded RoPE table and stored by the warp whose unit holds its slot).  Warps are merged
// through static shared memory, splits through global scratch by the last CTA to arrive (an atomic counter, nobody waits).
// Launched with programmatic stream serialisation.
//
// Same math as gqa_attention_f16kv (Shaders/GQA.metal:278-387) / fused_qk_norm_rope_gqa (Shaders/RoPE.metal:324-494);
// log-sum-exp merge as gqa_decode_attention_packed_f16kv_reduce (Shaders/GQA.metal:753-776).
#include <cuda_runtime.h>

#include "launchers.h"

namespace er {

namespace {

template <int GROUP>
struct SlimShape {
    static constexpr int kWarps = GROUP <= 2 ? 16 : 8;            // one 16-token unit per warp; registers bound the warp count
    static constexpr int kStageBytes = kWarps * 2 * kUnitTokens * kRowBytesF16;   // K rows + V rows of every warp's unit
};

template <int GROUP>
__global__ void __launch_bounds__(SlimShape<GROUP>::kWarps * 32, 1) decode_slim_kernel(const __grid_constant__ DecodeParams p) {
    using POL = DensePolicy<GROUP, 1, 1, 1>;   // its per-unit arithmetic, query preparation and new-row conversion, one unit per "tile"
    constexpr int NW = SlimShape<GROUP>::kWarps;
    constexpr int kUnitBytes = 2 * kUnitTokens * kRowBytesF16;   // 8 KB: K tile then V tile, the layout POL::process_unit reads
    extern __shared__ __align__(128) uint8_t slim_stage[];
    __shared__ __align__(16) float s_acc[NW][GROUP][kHeadDim];
    __shared__ float s_ml[NW][GROUP][2];
    __shared__ float s_prob[NW][GROUP][kUnitTokens];
    __shared__ float s_pm[64][GROUP], s_pl[64][GROUP];   // split merge: maxima and denominators of up to 64 partials
    __shared__ float2 s_cs[kHalfDim];
    __shared__ uint64_t s_bar[NW];
    __shared__ int s_flag[3];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, nsplit = gridDim.x, head = blockIdx.y, hkv = p.addr.num_kv_heads, pair = blockIdx.z;
    const int layer = p.layer_begin + pair / p.batch, seq = pair % p.batch;

    const int cta_linear = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    auto stamp = [&](int slot) {   // diagnostics: per-CTA phase times (er_kv_set_trace)
        if (p.trace != nullptr && tid == 0) p.trace[cta_linear * 8 + slot] = global_timer_ns();
    };
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (lane == 0) mbar_init(&s_bar[warp], 1);
    if (tid == 0) s_flag[2] = 0;   // abort flag of the bounded waits
    mbar_init_fence();
    __syncthreads();
    asm volatile("griddepcontrol.wait;" ::: "memory");   // lengths, rows, scratch and counters belong to the previous kernel until here
    stamp(0);

    const int kv_len = kv_length(p, pair);
    const int q_pos = p.lengths[layer * p.batch + seq] + p.pending - 1;
    const int units = (kv_len + kUnitTokens - 1) / kUnitTokens;
    const int per = (units + nsplit - 1) / nsplit;                     // units per split: at most NW by the host's choice of splits
    const int active = per > 0 ? (units + per - 1) / per : 0;          // splits that have rows
    const int u0 = split * per, u1 = min(units, u0 + per);
    const int64_t out_off = (static_cast<int64_t>(pair) * p.num_q_heads + head * GROUP) * kHeadDim;
    if (per > NW) {   // cannot happen with a split count from decode_slim_splits; never touch rows that were not staged
        if (tid == 0) atomicExch(p.status, kStatusBadLayout);
        return;
    }

    // ---- this warp's unit: bulk copies of its K and V rows into the warp's 8 KB of the stage, completion on the warp's barrier ----
    const int u = u0 + warp;
    const bool has = u < u1;
    uint8_t* stage = slim_stage + warp * kUnitBytes;
    const int nvalid = has ? min(kUnitTokens, kv_len - u * kUnitTokens) : 0;
    if (has) {
        const uint8_t* kl = p.k_base + static_cast<int64_t>(layer) * p.k_layer_stride_bytes;
        const uint8_t* vl = p.v_base + static_cast<int64_t>(layer) * p.v_layer_stride_bytes;
        if (lane == 0) mbar_arrive_expect_tx(&s_bar[warp], static_cast<uint32_t>(nvalid) * kRowBytesF16 * 2);
        __syncwarp();
        if (p.addr.token_major) {      // a copy per row: lanes 0..15 the K rows, 16..31 the V rows
            const int r = lane & 15, is_v = lane >> 4;
            if (r < nvalid)
                bulk_g2s(stage + is_v * (kUnitTokens * kRowBytesF16) + r * kRowBytesF16,
                         (is_v ? vl : kl) + row_index(p.addr, seq, head, u * kUnitTokens + r) * kRowBytesF16, kRowBytesF16, &s_bar[warp]);
        } else if (lane < 2) {         // a unit never straddles a page (pages are multiples of 16 tokens): one copy per tensor
            const int64_t row = row_index(p.addr, seq, head, u * kUnitTokens);
            bulk_g2s(stage + lane * (kUnitTokens * kRowBytesF16), (lane ? vl : kl) + row * kRowBytesF16,
                     static_cast<uint32_t>(nvalid) * kRowBytesF16, &s_bar[warp]);
        }
    }
    // (cos, sin) of the position, exactly rounded (the new K row goes into the cache), while the copies are in flight
    if (p.apply_rope && tid < kHalfDim) s_cs[tid] = rope_cos_sin(static_cast<uint32_t>(q_pos), p.inv_freq.f[tid], p.rope_scaling);
    __syncthreads();
    stamp(1);

    typename POL::State st;
    st.reset();
    if (has) {
        POL::load_q(p, st, p.q + out_off, s_cs, nullptr, warp, lane, layer);
        mbar_wait(&s_bar[warp], 0, &s_flag[2], p.status);
        if (!s_flag[2]) {
            const int slot_new = q_pos % p.addr.max_seq_len;
            if (p.fused_append && (slot_new >> 4) == u)   // this unit holds the new token's slot: convert, use and store the step's row
                POL::patch_new_row(p, stage, 0, slot_new & 15, layer, seq, head, slot_new,
                                   p.k_new + (static_cast<int64_t>(pair) * hkv + head) * kHeadDim,
                                   p.v_new + (static_cast<int64_t>(pair) * hkv + head) * kHeadDim, s_cs, lane);
            POL::process_unit(p, stage, 0, nvalid, st, &s_prob[warp][0][0], nullptr, lane);
        }
    }

    // ---- merge the warps of this CTA ----
    if (warp == 0) stamp(2);
    st.publish(&s_ml[warp][0][0], &s_acc[warp][0][0], lane);
    __syncthreads();
    stamp(3);
    const int item = pair * hkv + head;
    float* part = p.scratch + (static_cast<int64_t>(item) * nsplit + split) * GROUP * 130;
    const bool sole = active <= 1;
    if (u0 < u1 || (sole && split == 0)) {
        for (int idx = tid; idx < GROUP * kHeadDim; idx += NW * 32) {
            const int g = idx >> 7, d = idx & 127;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < NW; ++w) M = fmaxf(M, s_ml[w][g][0]);
            float Lsum = 0.f, A = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) {
                const float wgt = M == -INFINITY ? 0.f : fast_exp2(s_ml[w][g][0] - M);   // a warp without rows: exp2(-inf) = 0
                Lsum = fmaf(s_ml[w][g][1], wgt, Lsum);
                A = fmaf(s_acc[w][g][d], wgt, A);
            }
            if (sole) {
                p.out[out_off + idx] = Lsum > 0.f ? A / Lsum : 0.f;   // no rows -> zeros (invSum = 0 rule, Shaders/GQA.metal:379)
            } else {
                if (d == 0) { part[g * 130] = M; part[g * 130 + 1] = Lsum; }
                part[g * 130 + 2 + d] = A;
            }
        }
    }
    if (!sole && u0 < u1) {
        __threadfence();
        __syncthreads();
        if (tid == 0) s_flag[0] = (atomicAdd(p.item_counters + item, 1) == active - 1) ? 1 : 0;
        __syncthreads();
        if (s_flag[0]) {   // the last split to arrive merges all of them
            __threadfence();
            const float* first = p.scratch + static_cast<int64_t>(item) * nsplit * GROUP * 130;
            for (int e = tid; e < active * GROUP; e += NW * 32) {      // every partial's (max, denominator), one coalesced pass
                const int c = e / GROUP, g = e % GROUP;
                s_pm[c][g] = __ldcg(first + (c * GROUP + g) * 130);
                s_pl[c][g] = __ldcg(first + (c * GROUP + g) * 130 + 1);
            }
            __syncthreads();
            for (int idx = tid; idx < GROUP * kHeadDim; idx += NW * 32) {
                const int g = idx >> 7, d = idx & 127;
                float M = -INFINITY;
                for (int c = 0; c < active; ++c) M = fmaxf(M, s_pm[c][g]);
                float Lsum = 0.f, A = 0.f;
                int c = 0;
                for (; c + 8 <= active; c += 8) {                       // eight independent loads in flight per thread
                    float a[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) a[k] = __ldcg(first + ((c + k) * GROUP + g) * 130 + 2 + d);
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const float wgt = fast_exp2(s_pm[c + k][g] - M);
                        Lsum = fmaf(s_pl[c + k][g], wgt, Lsum);
                        A = fmaf(a[k], wgt, A);
                    }
                }
                for (; c < active; ++c) {
                    const float wgt = fast_exp2(s_pm[c][g] - M);
                    Lsum = fmaf(s_pl[c][g], wgt, Lsum);
                    A = fmaf(__ldcg(first + (c * GROUP + g) * 130 + 2 + d), wgt, A);
                }
                p.out[out_off + idx] = Lsum > 0.f ? A / Lsum : 0.f;
            }
            if (tid == 0) p.item_counters[item] = 0;
        }
    }

    // ---- the last CTA of the launch commits the step: lengths += advance ----
    stamp(4);
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const int total = static_cast<int>(gridDim.x * gridDim.y * gridDim.z);
        s_flag[1] = (atomicAdd(p.done_counter, 1) == total - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_flag[1]) {
        const int num_pairs = p.num_layers * p.batch;
        if (p.advance != 0)
            for (int e = tid; e < num_pairs; e += NW * 32) p.lengths[p.layer_begin * p.batch + e] += p.advance;
        if (tid == 0) *p.done_counter = 0;
    }
    stamp(5);
}

template <int GROUP>
int launch_slim(const DecodeParams& p, int splits, cudaStream_t stream) {
    constexpr int kSmem = SlimShape<GROUP>::kStageBytes;
    static int configured_device = -1;   // the attribute is per device and sticky: set it once
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (configured_device != device) {
        e = cudaFuncSetAttribute(decode_slim_kernel<GROUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured_device = device;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(splits), static_cast<unsigned>(p.addr.num_kv_heads), static_cast<unsigned>(p.num_layers * p.batch));
    cfg.blockDim = dim3(SlimShape<GROUP>::kWarps * 32);
    cfg.dynamicSmemBytes = kSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, decode_slim_kernel<GROUP>, p));
}

}  // namespace

// Split count for a launch of `items` (layer, sequence, kv head) items whose rings hold up to `max_units` 16-token units, on
// `num_sms` SMs, with room for `scratch_floats` of partials: about one CTA per SM, and enough splits that a split's units
// fit the CTA's warps (one unit each); at most 64 splits (the merge's tables).  0 = the launch is not one for this kernel.
int decode_slim_splits(int group, int items, int max_units, int num_sms, size_t scratch_floats) {
    if (items <= 0 || max_units <= 0 || (group != 1 && group != 2 && group != 4)) return 0;
    const int warps = group <= 2 ? 16 : 8;
    int splits = num_sms / items;
    const int need = (max_units + warps - 1) / warps;
    if (splits < need) splits = need;
    if (splits < 1) splits = 1;
    if (splits > 64) return 0;
    if (static_cast<size_t>(items) * splits * group * 130 > scratch_floats) return 0;
    return splits;
}

int launch_decode_slim(int group, const DecodeParams& p, int splits, cudaStream_t stream) {
    if (p.lengths == nullptr || p.window > 0 || p.out_heads_total > 0 || splits <= 0 || p.num_layers * p.batch > 65535) return kNotBuilt;
    switch (group) {
        case 1: return launch_slim<1>(p, splits, stream);
        case 2: return launch_slim<2>(p, splits, stream);
        case 4: return launch_slim<4>(p, splits, stream);
        default: return kNotBuilt;
    }
}

}  // namespace er
