// GQA attention over float32 K / V rows, with the optional additive mask: what GQAKernel.encode / execute dispatch
// (Sources/EdgeRunnerMetal/GQAKernel.swift:27-172) -- gqa_attention_f32, gqa_attention_f32_wide and
// gqa_attention_f32_masked_wide (Sources/EdgeRunnerMetal/Shaders/GQA.metal:18-276):
//   score[k] = scale * <Q[r][h], K[k][h / group]> (+ mask[r * kvSeqLen + k]);  key k visible iff !causal or k <= r + qOffset;
//   O[r][h] = sum_k softmax(score)[k] * V[k][h / group];  no visible finite score -> 0.
// The same kernel serves attention over a float32 er_kv cache (rows addressed through the cache's layout, lengths read
// on the device).  One CTA per (query row, q head): four warps walk the keys round-robin with an online softmax each
// (lane owns dims lane, lane + 32, ...), and are merged through shared memory.  Any head size <= 512 that is a multiple
// of 4.  This is the API-parity path of the fp32 operator, not the bandwidth path (fp16 / q8_0 / TurboQuant rows are).
#include <cuda_runtime.h>

#include <cmath>

#include "er_common.cuh"
#include "launchers.h"

namespace er {

namespace {

constexpr int kF32Warps = 4;
constexpr int kF32MaxPerLane = 16;   // head_dim <= 512

__global__ void __launch_bounds__(kF32Warps * 32) attention_f32_kernel(const __grid_constant__ AttentionF32Params p) {
    __shared__ float s_acc[kF32Warps][512];
    __shared__ float s_ml[kF32Warps][2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x, head = blockIdx.y, prob = blockIdx.z;
    const int D = p.head_dim, per_lane = (D + 31) / 32;
    const int kv_head = head / (p.num_heads / p.num_kv_heads);
    int layer = 0, seq = 0, kv_len = p.kv_len;
    if (p.lengths != nullptr) {   // cache mode: problem = (layer, sequence), one query row each
        layer = p.layer_begin + prob / p.batch;
        seq = prob % p.batch;
        const int n = p.lengths[layer * p.batch + seq] + p.pending;
        kv_len = n < p.addr.max_seq_len ? n : p.addr.max_seq_len;
    }
    const float* q = p.q + ((static_cast<int64_t>(prob) * p.seq_len + row) * p.num_heads + head) * D;
    float* out = p.out + ((static_cast<int64_t>(prob) * p.seq_len + row) * p.num_heads + head) * D;
    const float* kl = p.k + static_cast<int64_t>(layer) * p.layer_stride_elems;
    const float* vl = p.v + static_cast<int64_t>(layer) * p.layer_stride_elems;
    const int64_t limit = p.causal ? static_cast<int64_t>(row) + p.q_offset : static_cast<int64_t>(kv_len) - 1;
    const int visible = static_cast<int>(limit + 1 < kv_len ? limit + 1 : kv_len);

    float qr[kF32MaxPerLane], acc[kF32MaxPerLane];
#pragma unroll
    for (int i = 0; i < kF32MaxPerLane; ++i) {
        const int d = lane + 32 * i;
        qr[i] = (i < per_lane && d < D) ? q[d] : 0.f;
        acc[i] = 0.f;
    }
    if (p.apply_rope && D == kHeadDim && p.lengths != nullptr) {
        // lane holds dims lane, lane + 32 (first halves) and their NeoX partners lane + 64, lane + 96
        const uint32_t pos = static_cast<uint32_t>(p.lengths[layer * p.batch + seq] + p.pending - 1);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float2 cs = rope_cos_sin_fast(pos, p.inv_freq.f[lane + 32 * i], p.rope_scaling);
            float y0, y1;
            rope_rotate(qr[i], qr[i + 2], cs, y0, y1);
            qr[i] = y0;
            qr[i + 2] = y1;
        }
    }
    float m = -INFINITY, l = 0.f;
    for (int t = warp; t < visible; t += kF32Warps) {
        const int64_t ridx = row_index(p.addr, seq, kv_head, t);
        const float* kr = kl + ridx * D;
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < kF32MaxPerLane; ++i) {
            const int d = lane + 32 * i;
            if (i < per_lane && d < D) dot = fmaf(qr[i], kr[d], dot);
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        float score = dot * p.scale;
        if (p.mask != nullptr) score += p.mask[static_cast<int64_t>(row) * p.mask_stride + t];
        if (score == -INFINITY) continue;   // warp-uniform: the reduced dot and the mask entry are the same in every lane
        const float m_new = fmaxf(m, score);
        const float corr = expf(m - m_new), w = expf(score - m_new);
        l = fmaf(l, corr, w);
        m = m_new;
        const float* vr = vl + ridx * D;
#pragma unroll
        for (int i = 0; i < kF32MaxPerLane; ++i) {
            const int d = lane + 32 * i;
            if (i < per_lane && d < D) acc[i] = fmaf(w, vr[d], acc[i] * corr);
        }
    }
    if (lane == 0) { s_ml[warp][0] = m; s_ml[warp][1] = l; }
#pragma unroll
    for (int i = 0; i < kF32MaxPerLane; ++i) {
        const int d = lane + 32 * i;
        if (i < per_lane && d < D) s_acc[warp][d] = acc[i];
    }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kF32Warps; ++w) M = fmaxf(M, s_ml[w][0]);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float L = 0.f, A = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < kF32Warps; ++w) {
                const float wgt = s_ml[w][0] == -INFINITY ? 0.f : expf(s_ml[w][0] - M);
                L = fmaf(s_ml[w][1], wgt, L);
                A = fmaf(s_acc[w][d], wgt, A);
            }
        }
        out[d] = L > 0.f ? A / L : 0.f;
    }
}

}  // namespace

int launch_attention_f32(const AttentionF32Params& p, int problems, cudaStream_t stream) {
    if (p.head_dim <= 0 || p.head_dim > 512 || p.num_kv_heads <= 0 || p.num_heads % p.num_kv_heads != 0) return kNotBuilt;
    if (p.seq_len <= 0 || problems <= 0) return 0;
    if (p.num_heads > 65535 || problems > 65535) return kNotBuilt;
    attention_f32_kernel<<<dim3(static_cast<unsigned>(p.seq_len), static_cast<unsigned>(p.num_heads), static_cast<unsigned>(problems)),
                           kF32Warps * 32, 0, stream>>>(p);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace er
