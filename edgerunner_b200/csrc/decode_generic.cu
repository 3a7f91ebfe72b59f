// Decode attention for shapes the persistent flash-decode kernels are not built for: head sizes other than 128 (the
// reference's Gemma 4 layers use 256 and 512; gemma4_decode_gqa_f16kv_windowed, Shaders/Gemma4Decode.metal:222-342), GQA
// groups other than 1/2/4/8, more than 16 kv heads.  Same arithmetic (fp32 dot products of the float query with the fp16 rows,
// online softmax, log-sum-exp merge of partials as in Shaders/GQA.metal:753-776), plain structure: CTA (head, split) walks a
// contiguous part of the ring range with one token per warp at a time (lanes over dims, 4-byte loads), the 8 warps merge
// through shared memory, and with more than one split the last CTA to arrive at a head merges the splits from global
// scratch (an atomic counter; nobody waits).  Meant for the short windows and small head counts of those layers, not for
// the bandwidth-bound configurations.
#include <algorithm>

#include "launchers.h"

namespace er {

namespace {

constexpr int kGenericWarps = 8;
constexpr int kGenericMaxDim = 512;
constexpr int kGenericRegs = kGenericMaxDim / 64;   // half2 pairs per lane

__global__ void __launch_bounds__(kGenericWarps * 32)
generic_decode_kernel(const GenericDecodeParams p) {
    __shared__ float sm_ml[kGenericWarps][2];
    __shared__ float sm_acc[kGenericWarps][kGenericMaxDim];
    __shared__ int sm_last;
    const int head = blockIdx.x, split = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = p.head_dim;
    const int kv_head = head / (p.num_heads / p.num_kv_heads);
    const int i0 = split * p.chunk, i1 = min(p.count, i0 + p.chunk);

    float2 qr[kGenericRegs];
#pragma unroll
    for (int r = 0; r < kGenericRegs; ++r) {
        const int d = 2 * lane + 64 * r;
        qr[r] = d < D ? *reinterpret_cast<const float2*>(p.q + static_cast<size_t>(head) * D + d) : make_float2(0.f, 0.f);
        qr[r].x *= p.scale_log2;
        qr[r].y *= p.scale_log2;
    }
    float m = -INFINITY, l = 0.f;
    float2 acc[kGenericRegs];
#pragma unroll
    for (int r = 0; r < kGenericRegs; ++r) acc[r] = make_float2(0.f, 0.f);

    for (int i = i0 + warp; i < i1; i += kGenericWarps) {
        const size_t row = (static_cast<size_t>((p.start + i) % p.capacity) * p.num_kv_heads + kv_head) * D;
        const __half2* kr = reinterpret_cast<const __half2*>(p.k + row);
        const __half2* vr = reinterpret_cast<const __half2*>(p.v + row);
        float dot = 0.f;
        float2 vv[kGenericRegs];
#pragma unroll
        for (int r = 0; r < kGenericRegs; ++r) {
            const int d = 2 * lane + 64 * r;
            if (d < D) {
                const float2 kf = __half22float2(kr[lane + 32 * r]);
                vv[r] = __half22float2(vr[lane + 32 * r]);
                dot = fmaf(qr[r].x, kf.x, dot);
                dot = fmaf(qr[r].y, kf.y, dot);
            } else {
                vv[r] = make_float2(0.f, 0.f);
            }
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        const float m_new = fmaxf(m, dot);
        const float corr = fast_exp2(m - m_new), pw = fast_exp2(dot - m_new);
        l = fmaf(l, corr, pw);
#pragma unroll
        for (int r = 0; r < kGenericRegs; ++r) {
            acc[r].x = fmaf(acc[r].x, corr, pw * vv[r].x);
            acc[r].y = fmaf(acc[r].y, corr, pw * vv[r].y);
        }
        m = m_new;
    }
    if (lane == 0) { sm_ml[warp][0] = m; sm_ml[warp][1] = l; }
#pragma unroll
    for (int r = 0; r < kGenericRegs; ++r) {
        const int d = 2 * lane + 64 * r;
        if (d < D) *reinterpret_cast<float2*>(&sm_acc[warp][d]) = acc[r];
    }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kGenericWarps; ++w) M = fmaxf(M, sm_ml[w][0]);   // finite: the split holds at least one row
    float L = 0.f;
#pragma unroll
    for (int w = 0; w < kGenericWarps; ++w) L = fmaf(sm_ml[w][1], fast_exp2(sm_ml[w][0] - M), L);
    float* out = p.out + static_cast<size_t>(head) * D;
    float* part = p.scratch + (static_cast<size_t>(head) * p.nsplit + split) * (D + 2);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float A = 0.f;
#pragma unroll
        for (int w = 0; w < kGenericWarps; ++w) A = fmaf(sm_acc[w][d], fast_exp2(sm_ml[w][0] - M), A);
        if (p.nsplit == 1) out[d] = L > 0.f ? A / L : 0.f;
        else part[2 + d] = A;
    }
    if (p.nsplit == 1) return;
    if (threadIdx.x == 0) { part[0] = M; part[1] = L; }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) sm_last = (atomicAdd(p.counters + head, 1) == p.nsplit - 1) ? 1 : 0;
    __syncthreads();
    if (!sm_last) return;
    __threadfence();
    const float* parts = p.scratch + static_cast<size_t>(head) * p.nsplit * (D + 2);
    float GM = -INFINITY;
    for (int s = 0; s < p.nsplit; ++s) GM = fmaxf(GM, __ldcg(parts + static_cast<size_t>(s) * (D + 2)));
    float GL = 0.f;
    for (int s = 0; s < p.nsplit; ++s) {
        const float* ps = parts + static_cast<size_t>(s) * (D + 2);
        GL = fmaf(__ldcg(ps + 1), fast_exp2(__ldcg(ps) - GM), GL);
    }
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float A = 0.f;
        for (int s = 0; s < p.nsplit; ++s) {
            const float* ps = parts + static_cast<size_t>(s) * (D + 2);
            A = fmaf(__ldcg(ps + 2 + d), fast_exp2(__ldcg(ps) - GM), A);
        }
        out[d] = GL > 0.f ? A / GL : 0.f;
    }
    if (threadIdx.x == 0) p.counters[head] = 0;
}

}  // namespace

int launch_decode_generic(GenericDecodeParams p, int num_sms, size_t scratch_floats, size_t counter_ints, cudaStream_t stream) {
    if (p.head_dim <= 0 || p.head_dim > kGenericMaxDim || p.head_dim % 2 != 0 || p.count <= 0 || p.capacity <= 0 ||
        p.num_kv_heads <= 0 || p.num_heads % p.num_kv_heads != 0 || static_cast<size_t>(p.num_heads) > counter_ints)
        return kNotBuilt;
    // enough CTAs to cover the GPU twice, at least 64 rows per split, and the partials must fit the scratch
    int nsplit = std::max(1, std::min((2 * num_sms + p.num_heads - 1) / p.num_heads, (p.count + 63) / 64));
    const size_t per_head = static_cast<size_t>(p.head_dim) + 2;
    nsplit = static_cast<int>(std::min<size_t>(nsplit, std::max<size_t>(1, scratch_floats / (per_head * p.num_heads))));
    p.chunk = (p.count + nsplit - 1) / nsplit;
    p.nsplit = (p.count + p.chunk - 1) / p.chunk;   // no empty split
    generic_decode_kernel<<<dim3(p.num_heads, p.nsplit), kGenericWarps * 32, 0, stream>>>(p);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace er
