// Decode attention over fp16 rows for SMALL launches: one layer of a small batch (a few MB to a few tens of MB of K / V),
// the shape of the reference's per-layer dispatch (fusedDecodePass issues gqa_attention_f16kv once per layer,
// Sources/EdgeRunner/Models/LlamaLanguageModel.swift:3867-3881).  The persistent kernel (flash_decode.cuh) is built for
// launches that keep every SM streaming for tens of microseconds: its 220 KB shared-memory prologue, work-list scan and
// mbarrier ring cost ~15 us before they pay off.  Here nothing is staged: the grid is (split, kv head, (layer, sequence)),
// a warp takes 16-token units of its CTA's token range, loads the rows of a unit straight into registers (all of a
// CTA's loads are in flight at once: 8 KB per warp), and runs the same lane-owns-dims arithmetic as DensePolicy::process_unit.
// Warps are merged through a few KB of static shared memory, splits through global scratch by the last CTA to arrive
// (an atomic counter, nobody waits).  The new token's K / V row is converted (NeoX RoPE, exactly rounded table) and
// stored by the warp whose unit holds its slot, as in DensePolicy::patch_new_row.  Launched with programmatic stream
// serialisation: consecutive layer launches overlap their launch latency and prologue with the previous tail.
//
// Same math as gqa_attention_f16kv (Shaders/GQA.metal:278-387) / fused_qk_norm_rope_gqa (Shaders/RoPE.metal:324-494);
// log-sum-exp merge as gqa_decode_attention_packed_f16kv_reduce (Shaders/GQA.metal:753-776).
#include <cuda_runtime.h>

#include "launchers.h"

namespace er {

namespace {

template <int GROUP>
struct SlimShape {
    static constexpr int kWarps = GROUP <= 2 ? 16 : 8;   // registers: 64 staging + 16 * GROUP query + accumulators per lane
};

template <int GROUP>
__global__ void __launch_bounds__(SlimShape<GROUP>::kWarps * 32, 1) decode_slim_kernel(const __grid_constant__ DecodeParams p) {
    constexpr int NW = SlimShape<GROUP>::kWarps;
    __shared__ __align__(16) float s_acc[NW][GROUP][kHeadDim];
    __shared__ float s_ml[NW][GROUP][2];
    __shared__ float s_prob[NW][GROUP][kUnitTokens];
    __shared__ float2 s_cs[kHalfDim];
    __shared__ int s_flag[2];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, nsplit = gridDim.x, head = blockIdx.y, hkv = p.addr.num_kv_heads, pair = blockIdx.z;
    const int layer = p.layer_begin + pair / p.batch, seq = pair % p.batch;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");   // lengths, rows, scratch and counters belong to the previous kernel until here

    const int kv_len = kv_length(p, pair);
    const int q_pos = p.lengths[layer * p.batch + seq] + p.pending - 1;
    const int units = (kv_len + kUnitTokens - 1) / kUnitTokens;
    const int per = (units + nsplit - 1) / nsplit;                     // units per split
    const int active = per > 0 ? (units + per - 1) / per : 0;          // splits that have rows
    const int u0 = split * per, u1 = min(units, u0 + per);
    const int64_t out_off = (static_cast<int64_t>(pair) * p.num_q_heads + head * GROUP) * kHeadDim;

    // (cos, sin) of the query position: float sincos (the query is consumed, never stored)
    if (p.apply_rope && tid < kHalfDim) s_cs[tid] = rope_cos_sin_fast(static_cast<uint32_t>(q_pos), p.inv_freq.f[tid], p.rope_scaling);
    __syncthreads();

    const int j = lane >> 3, i = lane & 7;
    const uint8_t* kl = p.k_base + static_cast<int64_t>(layer) * p.k_layer_stride_bytes;
    const uint8_t* vl = p.v_base + static_cast<int64_t>(layer) * p.v_layer_stride_bytes;
    const int64_t row_stride = p.addr.token_major ? static_cast<int64_t>(hkv) * kRowBytesF16 : kRowBytesF16;
    const int slot_new = q_pos % p.addr.max_seq_len;

    float q[GROUP][16], m[GROUP], l[GROUP], acc[GROUP][4];
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[g][c] = 0.f;
    }
    bool have_q = false;
    float* prob = &s_prob[warp][0][0];

    for (int u = u0 + warp; u < u1; u += NW) {
        const int t0 = u * kUnitTokens;
        const int nvalid = min(kUnitTokens, kv_len - t0);
        // ---- the unit's rows: K 4 rows x 2 x 16 bytes and V 16 rows x 8 bytes per lane, all issued before anything is used ----
        const int64_t base = row_index(p.addr, seq, head, t0) * kRowBytesF16;   // a unit never straddles a page (pages are multiples of 16)
        uint4 ka[4], kb[4];
        uint2 vv[kUnitTokens];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int row = 4 * r + j;
            if (row < nvalid) {
                const uint8_t* src = kl + base + row * row_stride + i * 16;
                ka[r] = __ldg(reinterpret_cast<const uint4*>(src));
                kb[r] = __ldg(reinterpret_cast<const uint4*>(src + 128));
            } else {
                ka[r] = make_uint4(0, 0, 0, 0);
                kb[r] = make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int t = 0; t < kUnitTokens; ++t)
            vv[t] = t < nvalid ? __ldg(reinterpret_cast<const uint2*>(vl + base + t * row_stride + lane * 8)) : make_uint2(0, 0);

        if (!have_q) {   // the query rows, once per warp, while the loads above are in flight
            have_q = true;
            const float* qrow = p.q + out_off;
            const float* qw = p.q_norm_w ? p.q_norm_w + static_cast<int64_t>(layer) * p.norm_stride : nullptr;
#pragma unroll
            for (int g = 0; g < GROUP; ++g) {
                const float4* src = reinterpret_cast<const float4*>(qrow + g * kHeadDim + 8 * i);
                const float4 a0 = __ldg(src), a1 = __ldg(src + 1), b0 = __ldg(src + 16), b1 = __ldg(src + 17);
                float xa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                float xb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                if (qw != nullptr) {
                    const float rs = head_rms_scale(qrow + g * kHeadDim, p.rms_eps, lane);
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        xa[c] = __fmul_rn(__fmul_rn(xa[c], rs), __ldg(qw + 8 * i + c));
                        xb[c] = __fmul_rn(__fmul_rn(xb[c], rs), __ldg(qw + 64 + 8 * i + c));
                    }
                }
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    if (p.apply_rope) {
                        rope_rotate(xa[c], xb[c], s_cs[8 * i + c], q[g][c], q[g][8 + c]);
                    } else {
                        q[g][c] = xa[c];
                        q[g][8 + c] = xb[c];
                    }
                }
            }
        }

        // ---- fused append: this unit holds the new token's slot -> convert the step's K / V row, use it, store it ----
        if (p.fused_append && (slot_new >> 4) == u) {
            const int r_in = slot_new & 15;
            const float* k_src = p.k_new + (static_cast<int64_t>(pair) * hkv + head) * kHeadDim;
            const float* v_src = p.v_new + (static_cast<int64_t>(pair) * hkv + head) * kHeadDim;
            const float* kw = p.k_norm_w ? p.k_norm_w + static_cast<int64_t>(layer) * p.norm_stride : nullptr;
            const float rs = kw ? head_rms_scale(k_src, p.rms_eps, lane) : 1.f;
            const int64_t dst_row = row_index_for_write(p.addr, seq, head, slot_new);
            if (j == (r_in & 3)) {   // the eight lanes that hold this K row: dims [8i, 8i + 8) and their partners + 64
                uint4 na, nb;
                __half2* ha = reinterpret_cast<__half2*>(&na);
                __half2* hb = reinterpret_cast<__half2*>(&nb);
#pragma unroll
                for (int c2 = 0; c2 < 4; ++c2) {
                    float y[4];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int d = 8 * i + 2 * c2 + e;
                        float x0 = __ldg(k_src + d), x1 = __ldg(k_src + d + kHalfDim);
                        if (kw != nullptr) {
                            x0 = __fmul_rn(__fmul_rn(x0, rs), __ldg(kw + d));
                            x1 = __fmul_rn(__fmul_rn(x1, rs), __ldg(kw + d + kHalfDim));
                        }
                        if (p.apply_rope) {
                            // rows that go into the cache use the exactly rounded table (double sincos), as every append path does
                            const float2 cs = rope_cos_sin(static_cast<uint32_t>(q_pos), p.inv_freq.f[d], p.rope_scaling);
                            rope_rotate(x0, x1, cs, y[e], y[2 + e]);
                        } else {
                            y[e] = x0;
                            y[2 + e] = x1;
                        }
                    }
                    ha[c2] = __halves2half2(__float2half_rn(y[0]), __float2half_rn(y[1]));
                    hb[c2] = __halves2half2(__float2half_rn(y[2]), __float2half_rn(y[3]));
                }
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    if (r == (r_in >> 2)) { ka[r] = na; kb[r] = nb; }
                if (dst_row >= 0) {
                    uint8_t* dst = const_cast<uint8_t*>(kl) + dst_row * kRowBytesF16 + i * 16;
                    *reinterpret_cast<uint4*>(dst) = na;
                    *reinterpret_cast<uint4*>(dst + 128) = nb;
                }
            }
            {
                const float4 v4 = __ldg(reinterpret_cast<const float4*>(v_src) + lane);
                uint2 nv;
                reinterpret_cast<__half2*>(&nv)[0] = __halves2half2(__float2half_rn(v4.x), __float2half_rn(v4.y));
                reinterpret_cast<__half2*>(&nv)[1] = __halves2half2(__float2half_rn(v4.z), __float2half_rn(v4.w));
#pragma unroll
                for (int t = 0; t < kUnitTokens; ++t)
                    if (t == r_in) vv[t] = nv;
                if (dst_row >= 0) *reinterpret_cast<uint2*>(const_cast<uint8_t*>(vl) + dst_row * kRowBytesF16 + lane * 8) = nv;
            }
        }

        // ---- scores: lane (j, i) holds rows 4r + j; an 8-lane butterfly finishes each dot product ----
        float s[4][GROUP];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            float fa[8], fb[8];
            unpack8(ka[r], fa);
            unpack8(kb[r], fb);
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
            const float corr = fast_exp2(m[g] - m_new);
            float psum = 0.f;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float pr = fast_exp2(s[r][g] - m_new);
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
        // ---- P.V: lane owns output dims [4 lane, 4 lane + 4) ----
#pragma unroll
        for (int t4 = 0; t4 < kUnitTokens; t4 += 4) {
            float4 pg[GROUP];
#pragma unroll
            for (int g = 0; g < GROUP; ++g) pg[g] = *reinterpret_cast<const float4*>(prob + g * kUnitTokens + t4);
#pragma unroll
            for (int tt = 0; tt < 4; ++tt) {
                float vf[4];
                unpack4(vv[t4 + tt], vf);
#pragma unroll
                for (int g = 0; g < GROUP; ++g) {
                    const float w = tt == 0 ? pg[g].x : tt == 1 ? pg[g].y : tt == 2 ? pg[g].z : pg[g].w;   // rows past nvalid: 0 * 0
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[g][c] = fmaf(w, vf[c], acc[g][c]);
                }
            }
        }
        __syncwarp();
    }

    // ---- merge the warps of this CTA ----
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
        if (lane == 0) { s_ml[warp][g][0] = m[g]; s_ml[warp][g][1] = l[g]; }
        *reinterpret_cast<float4*>(&s_acc[warp][g][4 * lane]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
    }
    __syncthreads();
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
                const float wgt = fast_exp2(s_ml[w][g][0] - M);      // a warp without rows: exp2(-inf) = 0 (M finite) ...
                Lsum = fmaf(s_ml[w][g][1], M == -INFINITY ? 0.f : wgt, Lsum);   // ... and no rows at all: everything stays 0
                A = fmaf(s_acc[w][g][d], M == -INFINITY ? 0.f : wgt, A);
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
            for (int idx = tid; idx < GROUP * kHeadDim; idx += NW * 32) {
                const int g = idx >> 7, d = idx & 127;
                float M = -INFINITY;
                for (int c = 0; c < active; ++c) M = fmaxf(M, __ldcg(first + (c * GROUP + g) * 130));
                float Lsum = 0.f, A = 0.f;
                for (int c = 0; c < active; ++c) {
                    const float* sc = first + (c * GROUP + g) * 130;
                    const float wgt = fast_exp2(__ldcg(sc) - M);
                    Lsum = fmaf(__ldcg(sc + 1), wgt, Lsum);
                    A = fmaf(__ldcg(sc + 2 + d), wgt, A);
                }
                p.out[out_off + idx] = Lsum > 0.f ? A / Lsum : 0.f;
            }
            if (tid == 0) p.item_counters[item] = 0;
        }
    }

    // ---- the last CTA of the launch commits the step: lengths += advance ----
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
}

template <int GROUP>
int launch_slim(const DecodeParams& p, int splits, cudaStream_t stream) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(splits), static_cast<unsigned>(p.addr.num_kv_heads), static_cast<unsigned>(p.num_layers * p.batch));
    cfg.blockDim = dim3(SlimShape<GROUP>::kWarps * 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, decode_slim_kernel<GROUP>, p));
}

}  // namespace

// Split count for a launch of `items` (layer, sequence, kv head) items on `num_sms` SMs with room for `scratch_floats` of
// partials: about one CTA per SM, at most 64 splits, never more than the scratch can hold.  0 = the launch is not one
// for this kernel.
int decode_slim_splits(int group, int items, int num_sms, size_t scratch_floats) {
    if (items <= 0 || (group != 1 && group != 2 && group != 4)) return 0;
    int splits = num_sms / items;
    if (splits < 1) splits = 1;
    if (splits > 64) splits = 64;
    while (splits > 1 && static_cast<size_t>(items) * splits * group * 130 > scratch_floats) --splits;
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
