// TurboQuant device math (tables, code lookup, warp-level transforms) shared by the quantise kernels and the
// decode policy.  TurboQuant row codec on the device: randomized Hadamard rotation with the reference's fixed sign tables (the reference ignores its seed, TurboQuant.swift:918-921), Lloyd-Max scalar codes,
// corrected per-row norm.  Restates, warp-cooperatively, what the reference does with one thread per row:
//   turboquant_quantize_rows           Shaders/TurboQuant.metal:562-709
//   TurboQuantReferenceEncoder.encode  Sources/EdgeRunnerMetal/TurboQuant.swift:1003-1074 (fixed presets)
//   TurboQuantTransform                Sources/EdgeRunnerMetal/TurboQuant.swift:875-916, 985-999
//   BitPacker                          Sources/EdgeRunnerMetal/TurboQuant.swift:1441-1594
//
// Bit-exactness.  The packed codes depend on last-ulp values, so every float operation that feeds a
// threshold compare is issued in the reference's order with IEEE round-to-nearest intrinsics (no FMA
// contraction): the sum of squares runs left to right over the 128 coordinates (one lane walks one row),
// x/norm is a true division, the butterfly computes (lower + upper, lower - upper) per stage, and the
// final scale multiplies by +-(1/sqrt(128)) (float 0x3DB504F3).
#pragma once

#include "er_common.cuh"
#include "tq_tables.h"

namespace er {

__host__ __device__ constexpr int tq_code_words(int bits) { return (kHeadDim * bits + 31) / 32; }

static __constant__ float c_tq_cent2[4] = ER_TQ_CENTROIDS_2BIT;
static __constant__ float c_tq_cent3[8] = ER_TQ_CENTROIDS_3BIT;
static __constant__ float c_tq_cent4[16] = ER_TQ_CENTROIDS_4BIT;
static __constant__ float c_tq_cent5[32] = ER_TQ_CENTROIDS_5BIT;
static __constant__ uint32_t c_tq_signs1[4] = ER_TQ_SIGNS1_NEGMASK;
static __constant__ uint32_t c_tq_signs2[4] = ER_TQ_SIGNS2_NEGMASK;

constexpr float kTqForwardScale = 0.08838834764831845f;   // 1/sqrt(Float(128)), TurboQuant.swift:877

template <int BITS>
__device__ __forceinline__ const float* tq_centroids() {
    return BITS == 2 ? c_tq_cent2 : BITS == 3 ? c_tq_cent3 : c_tq_cent4;
}

// the codebook of a run-time bit width (2 .. 5)
__device__ __forceinline__ const float* tq_centroids_rt(int bits) {
    return bits == 2 ? c_tq_cent2 : bits == 3 ? c_tq_cent3 : bits == 4 ? c_tq_cent4 : c_tq_cent5;
}

// TurboQuantCodebook.code(for:) (TurboQuant.swift:692-697): index of the first threshold strictly greater
// than the value, else the last code.  With sorted thresholds that is the number of thresholds t with
// !(value < t), which also sends NaN to the last code.
template <int BITS>
__device__ __forceinline__ uint32_t tq_code_for(float v) {
    uint32_t code = 0;
    if (BITS == 2) {
        constexpr float thr[3] = ER_TQ_THRESHOLDS_2BIT;
#pragma unroll
        for (int i = 0; i < 3; ++i) code += !(v < thr[i]);
    } else if (BITS == 3) {
        constexpr float thr[7] = ER_TQ_THRESHOLDS_3BIT;
#pragma unroll
        for (int i = 0; i < 7; ++i) code += !(v < thr[i]);
    } else {
        constexpr float thr[15] = ER_TQ_THRESHOLDS_4BIT;
#pragma unroll
        for (int i = 0; i < 15; ++i) code += !(v < thr[i]);
    }
    return code;
}

__device__ __forceinline__ float tq_sign(const uint32_t* negmask, int i) {
    return (negmask[i >> 5] >> (i & 31)) & 1u ? -1.0f : 1.0f;
}

// Unnormalised 128-point FWHT across a warp; lane holds coordinates 4*lane .. 4*lane+3.
// hadamardInPlace (TurboQuant.swift:985-999): widths 1, 2 in registers, 4 .. 64 by lane exchange;
// the lower index keeps lhs + rhs, the upper index gets lhs - rhs.
__device__ __forceinline__ void warp_fwht128(float (&a)[4], int lane) {
    float t0 = __fadd_rn(a[0], a[1]), t1 = __fsub_rn(a[0], a[1]);
    float t2 = __fadd_rn(a[2], a[3]), t3 = __fsub_rn(a[2], a[3]);
    a[0] = __fadd_rn(t0, t2);
    a[2] = __fsub_rn(t0, t2);
    a[1] = __fadd_rn(t1, t3);
    a[3] = __fsub_rn(t1, t3);
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const bool upper = (lane & o) != 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float other = __shfl_xor_sync(0xffffffffu, a[c], o);
            a[c] = upper ? __fsub_rn(other, a[c]) : __fadd_rn(a[c], other);
        }
    }
}

// randomizedHadamard (TurboQuant.swift:891-906): (H (x . s1)) . (s2 * forwardScale)
__device__ __forceinline__ void warp_tq_forward(float (&a)[4], int lane) {
#pragma unroll
    for (int c = 0; c < 4; ++c) a[c] = __fmul_rn(a[c], tq_sign(c_tq_signs1, 4 * lane + c));
    warp_fwht128(a, lane);
#pragma unroll
    for (int c = 0; c < 4; ++c) a[c] = __fmul_rn(a[c], __fmul_rn(tq_sign(c_tq_signs2, 4 * lane + c), kTqForwardScale));
}

// inverseRandomizedHadamard (TurboQuant.swift:908-916): ((H (y . s2)) . s1) * forwardScale
__device__ __forceinline__ void warp_tq_inverse(float (&a)[4], int lane) {
#pragma unroll
    for (int c = 0; c < 4; ++c) a[c] = __fmul_rn(a[c], tq_sign(c_tq_signs2, 4 * lane + c));
    warp_fwht128(a, lane);
#pragma unroll
    for (int c = 0; c < 4; ++c) a[c] = __fmul_rn(__fmul_rn(a[c], tq_sign(c_tq_signs1, 4 * lane + c)), kTqForwardScale);
}

}  // namespace er
