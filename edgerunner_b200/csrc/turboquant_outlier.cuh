// TurboQuant encoder for the presets with high-precision channels and a QJL residual -- balanced (3-bit codes, the 32
// largest channels 5-bit) and aggressive (2-bit, 32 channels 3-bit): the residual path of
//   TurboQuantReferenceEncoder.encode   Sources/EdgeRunnerMetal/TurboQuant.swift:1003-1100
//   turboquant_quantize_rows            Sources/EdgeRunnerMetal/Shaders/TurboQuant.metal:562-709 (one thread per row there)
// One warp per row here; lane L holds coordinates 4L .. 4L + 3.  Everything that decides a bit is issued in the
// reference's order with round-to-nearest intrinsics: the two sums of squares run left to right (lane 0 walks the row
// in shared memory), x / norm is a true division, the transforms are warp_tq_forward / warp_tq_inverse.
// Channel selection: the `count` largest scores, equal scores in channel order (TurboQuant.swift:1185-1208 and the
// selection loop of the shader, :637-652) -- every element counts the elements that beat it (score greater, or equal with
// a lower index) and is selected when fewer than `count` do: 128 x 128 comparisons per row, 512 per lane.
// Codes are packed split-plane (BitPacker.packCodes with a mask, TurboQuant.swift:1463-1488): the low regularBits of every
// code at bit d * regularBits, the remaining high bits of the selected channels appended from bit 128 * regularBits on,
// in channel order.  Rows with a norm that is not > 0 (zero, NaN) come out as all-zero rows, as in the Swift encoder.
#pragma once

#include "tq_math.cuh"

namespace er {

static __constant__ float c_tq_thr2[3] = ER_TQ_THRESHOLDS_2BIT;
static __constant__ float c_tq_thr3[7] = ER_TQ_THRESHOLDS_3BIT;
static __constant__ float c_tq_thr4[15] = ER_TQ_THRESHOLDS_4BIT;
static __constant__ float c_tq_thr5[31] = ER_TQ_THRESHOLDS_5BIT;

// TurboQuantCodebook.code(for:) with a run-time bit width: number of thresholds t with !(value < t).
__device__ __forceinline__ uint32_t tq_code_for_rt(float v, int bits) {
    const float* thr = bits == 2 ? c_tq_thr2 : bits == 3 ? c_tq_thr3 : bits == 4 ? c_tq_thr4 : c_tq_thr5;
    const int n = (1 << bits) - 1;
    uint32_t code = 0;
    for (int i = 0; i < n; ++i) code += !(v < thr[i]);
    return code;
}

struct TurboOutlierParams {
    const float* source;        // [rows][stride], the first 128 of each row are used
    uint32_t rows, stride, dst_row_base;
    int regular_bits, high_bits, high_count, use_benefit, words_per_row;
    uint32_t* out_codes;        // [..][words_per_row]
    uint32_t* out_signs;        // [..][4]
    uint32_t* out_mask;         // [..][4]
    float* out_meta;            // [..][2] = (rowNorm, residualNorm)
};

constexpr int kOutlierWarps = 4;

// Per-warp shared scratch of the encoder.
struct OutlierScratch {
    float row[kHeadDim];     // a row's values for the sequential sums, then its scores
    uint32_t words[32];      // packed code words (at most 128 * 5 / 32 = 20)
    uint32_t bits[8];        // [0..3] outlier mask words, [4..7] residual sign words
};

// Encodes one row held by a warp (lane L: coordinates 4L .. 4L + 3 in x) and stores it: `words_per_row` code words at
// out_codes, 4 + 4 words at out_mask / out_signs, (rowNorm, residualNorm) at out_meta.  All lanes must call.
__device__ __forceinline__ void tq_encode_outlier_row(const float x[4], int lane, OutlierScratch& sc, int rb, int hb, int high_count,
                                                      int use_benefit, int words_per_row, uint32_t* out_codes, uint32_t* out_signs,
                                                      uint32_t* out_mask, float* out_meta) {
    float* row = sc.row;
    uint32_t* words = sc.words;
    uint32_t* bits = sc.bits;
    const int side_w = hb - rb;
    __syncwarp();
#pragma unroll
    for (int c = 0; c < 4; ++c) row[4 * lane + c] = x[c];
    words[lane] = 0u;
    if (lane < 8) bits[lane] = 0u;
    __syncwarp();
    float norm = 0.f;
    if (lane == 0) {   // rowNorm = sqrt(sum x^2), left to right (TurboQuant.swift:1016)
        float sum = 0.f;
        for (int d = 0; d < kHeadDim; ++d) sum = __fadd_rn(sum, __fmul_rn(row[d], row[d]));
        norm = __fsqrt_rn(sum);
    }
    norm = __shfl_sync(0xffffffffu, norm, 0);
    if (!(norm > 0.f)) {   // all-zero row
        for (int w = lane; w < words_per_row; w += 32) out_codes[w] = 0u;
        if (lane < 4) { out_signs[lane] = 0u; out_mask[lane] = 0u; }
        if (lane < 2) out_meta[lane] = 0.f;
        __syncwarp();
        return;
    }
    float nrm[4], rot[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) { nrm[c] = __fdiv_rn(x[c], norm); rot[c] = nrm[c]; }
    warp_tq_forward(rot, lane);
    // ---- selection scores ----
    float score[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        if (use_benefit) {   // (value - regularCentroid)^2 - (value - highCentroid)^2, each product rounded (TurboQuant.swift:1228-1238)
            const float re = __fsub_rn(rot[c], tq_centroids_rt(rb)[tq_code_for_rt(rot[c], rb)]);
            const float he = __fsub_rn(rot[c], tq_centroids_rt(hb)[tq_code_for_rt(rot[c], hb)]);
            score[c] = __fsub_rn(__fmul_rn(re, re), __fmul_rn(he, he));
        } else {
            score[c] = fabsf(rot[c]);
        }
    }
    __syncwarp();
#pragma unroll
    for (int c = 0; c < 4; ++c) row[4 * lane + c] = score[c];
    __syncwarp();
    bool sel[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const int i = 4 * lane + c;
        int beaten = 0;
        for (int j = 0; j < kHeadDim; ++j) {
            const float sj = row[j];
            beaten += (sj > score[c] || (sj == score[c] && j < i)) ? 1 : 0;
        }
        sel[c] = beaten < high_count;
    }
    // ---- codes, centroids, outlier mask, split-plane packing ----
    float recon[4];
    uint32_t code[4], piece = 0, nib = 0;
    int mine = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const int bw = sel[c] ? hb : rb;
        code[c] = tq_code_for_rt(rot[c], bw);
        recon[c] = tq_centroids_rt(bw)[code[c]];
        piece |= (code[c] & ((1u << rb) - 1u)) << (rb * c);
        nib |= (sel[c] ? 1u : 0u) << c;
        mine += sel[c] ? 1 : 0;
    }
    atomicOr(&bits[lane >> 3], nib << (4 * (lane & 7)));
    {
        const int off = 4 * rb * lane, w0 = off >> 5, sh = off & 31;
        atomicOr(&words[w0], piece << sh);
        if (sh + 4 * rb > 32) atomicOr(&words[w0 + 1], piece >> (32 - sh));
    }
    int before = mine;   // selected channels in lower lanes: exclusive prefix over the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, before, o);
        if (lane >= o) before += t;
    }
    before -= mine;
    if (side_w > 0) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (sel[c]) {
                const int off = kHeadDim * rb + before * side_w, w0 = off >> 5, sh = off & 31;
                const uint32_t hi = code[c] >> rb;
                atomicOr(&words[w0], hi << sh);
                if (sh + side_w > 32) atomicOr(&words[w0 + 1], hi >> (32 - sh));
                ++before;
            }
        }
    }
    // ---- residual: normalized - inverse(centroids); its norm left to right; signs of its forward transform ----
    warp_tq_inverse(recon, lane);
    float res[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) res[c] = __fsub_rn(nrm[c], recon[c]);
    __syncwarp();
#pragma unroll
    for (int c = 0; c < 4; ++c) row[4 * lane + c] = res[c];
    __syncwarp();
    float res_norm = 0.f;
    if (lane == 0) {
        float sum = 0.f;
        for (int d = 0; d < kHeadDim; ++d) sum = __fadd_rn(sum, __fmul_rn(row[d], row[d]));
        res_norm = __fsqrt_rn(sum);
    }
    warp_tq_forward(res, lane);
    uint32_t sgn = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) sgn |= (res[c] >= 0.f ? 1u : 0u) << c;
    atomicOr(&bits[4 + (lane >> 3)], sgn << (4 * (lane & 7)));
    __syncwarp();
    for (int w = lane; w < words_per_row; w += 32) out_codes[w] = words[w];
    if (lane < 4) { out_mask[lane] = bits[lane]; out_signs[lane] = bits[4 + lane]; }
    if (lane == 0) { out_meta[0] = norm; out_meta[1] = res_norm; }
    __syncwarp();
}

__global__ void __launch_bounds__(kOutlierWarps * 32) tq_quantize_rows_outlier_kernel(const __grid_constant__ TurboOutlierParams p) {
    __shared__ OutlierScratch s_scratch[kOutlierWarps];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t r = blockIdx.x * kOutlierWarps + warp; r < p.rows; r += gridDim.x * kOutlierWarps) {
        const float4 x4 = *reinterpret_cast<const float4*>(p.source + static_cast<size_t>(r) * p.stride + 4 * lane);
        const float x[4] = {x4.x, x4.y, x4.z, x4.w};
        const size_t dst = static_cast<size_t>(p.dst_row_base) + r;
        tq_encode_outlier_row(x, lane, s_scratch[warp], p.regular_bits, p.high_bits, p.high_count, p.use_benefit, p.words_per_row,
                              p.out_codes + dst * p.words_per_row, p.out_signs + dst * 4, p.out_mask + dst * 4, p.out_meta + dst * 2);
    }
}

}  // namespace er
