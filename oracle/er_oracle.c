/*
 * er_oracle.c -- CPU restatement of the EdgeRunner decode-time KV-cache path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped CUDA library calls, links or
 * loads this file; it exists so that tests (and the CPU-baseline leg of the
 * benchmark) have an independent statement of what the reference computes.
 *
 * Parity status: the reference is Swift + Metal and cannot be compiled or run in
 * this environment.  This restatement is pinned against every literal the
 * reference's own tests hold for the path (append/retrieve rows and ring-wrap
 * order, KVCacheTests.swift:43-99; TurboQuant layout word counts,
 * TurboQuantReferenceTests.swift:121-143; FWHT round trip, :7-18; RoPE known
 * value, RoPETests.swift:189-210) and against analytically derived known answers.
 * The reference holds NO literal golden code words or attention outputs (it pins
 * those by GPU==CPU equality at run time), so for packed codes and attention
 * outputs this oracle is "parity unpinned": it follows the cited Swift line by
 * line but has not been compared with output of the reference itself.
 *
 * Every function cites the reference file:line it follows (paths relative to the
 * reference checkout).  Build with -ffp-contract=off: the Swift code never fuses
 * a multiply into an add, and the packed codes depend on last-ulp values.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "er_tq_tables.h"

#define ERO_API __attribute__((visibility("default")))
#define ERO_DIM 128

/* ------------------------------------------------------------------ half <-> float */

/* Float16(Float) in Swift and half(float) in MSL round to nearest even
 * (KVCache.swift:1059-1064, RoPE.metal:529-530). */
ERO_API uint16_t ero_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t abs = x & 0x7FFFFFFFu;
    if (abs >= 0x7F800000u) {                       /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((abs > 0x7F800000u) ? 0x0200u : 0u));
    }
    if (abs >= 0x477FF000u) {                       /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (abs < 0x38800000u) {                        /* subnormal half or zero */
        if (abs < 0x33000000u) return (uint16_t)sign;   /* < 2^-25 -> 0 */
        uint32_t exp = abs >> 23;                   /* 102..112 */
        uint32_t man = (abs & 0x007FFFFFu) | 0x00800000u;
        uint32_t shift = 126u - exp;                /* 14..24 */
        uint32_t half = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1u);
        if (rem > halfway || (rem == halfway && (half & 1u))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((abs - 0x38000000u) >> 13);
    uint32_t rem = abs & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;
    return (uint16_t)(sign | half);
}

ERO_API float ero_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t x;
    if (exp == 0) {
        if (man == 0) {
            x = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            x = sign | ((uint32_t)(112 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        x = sign | 0x7F800000u | (man << 13);
    } else {
        x = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

static float *g_half_lut = NULL;
static const float *half_lut(void) {
    if (!g_half_lut) {
        float *t = (float *)malloc(65536 * sizeof(float));
        for (uint32_t i = 0; i < 65536; ++i) t[i] = ero_f16_to_f32((uint16_t)i);
        g_half_lut = t;
    }
    return g_half_lut;
}

/* ------------------------------------------------------------------ RoPE */

/* The shaders evaluate powr/cos/sin in float with Metal's (unspecified-ulp) math
 * library.  The oracle evaluates the same expressions through double and rounds
 * once to float, i.e. the correctly rounded value of each float expression:
 *   exponent  = float(2*pair)/float(headDim)
 *   frequency = 1.0f / powr(theta, exponent)
 *   angle     = float(seq+startPos) * (frequency / scalingFactor)
 * (RoPE.metal:40-44, 83-87, 521-525). */
static void rope_cos_sin(uint32_t pair, uint32_t head_dim, uint32_t position, float theta,
                         float scaling, float *c, float *s) {
    float exponent = (float)(2u * pair) / (float)head_dim;
    float p = (float)pow((double)theta, (double)exponent);
    float frequency = 1.0f / p;
    float angle = (float)position * (frequency / scaling);
    *c = (float)cos((double)angle);
    *s = (float)sin((double)angle);
}

/* rope_f32 (interleaved pairs (2d, 2d+1)), RoPE.metal:16-53. */
ERO_API void ero_rope_interleaved_f32(const float *in, float *out, uint32_t seq_len, uint32_t num_heads,
                                      uint32_t head_dim, uint32_t start_pos, float theta, float scaling,
                                      float partial) {
    uint32_t half = head_dim / 2;
    uint32_t rotated = (uint32_t)((float)half * partial);
    for (uint32_t s = 0; s < seq_len; ++s)
        for (uint32_t h = 0; h < num_heads; ++h)
            for (uint32_t d = 0; d < half; ++d) {
                size_t base = ((size_t)s * num_heads + h) * head_dim + 2u * d;
                if (d >= rotated) { out[base] = in[base]; out[base + 1] = in[base + 1]; continue; }
                float c, sn;
                rope_cos_sin(d, head_dim, s + start_pos, theta, scaling, &c, &sn);
                float x0 = in[base], x1 = in[base + 1];
                out[base] = x0 * c - x1 * sn;
                out[base + 1] = x0 * sn + x1 * c;
            }
}

/* rope_neox_f32 (pairs (d, d+headDim/2)), RoPE.metal:57-93.  `positions` may be NULL
 * (position = seq + start_pos, the shader's rule) or give one absolute position per row. */
ERO_API void ero_rope_neox_f32(const float *in, float *out, uint32_t seq_len, uint32_t num_heads,
                               uint32_t head_dim, uint32_t start_pos, float theta, float scaling,
                               float partial) {
    uint32_t half = head_dim / 2;
    uint32_t rotated = (uint32_t)((float)half * partial);
    for (uint32_t s = 0; s < seq_len; ++s)
        for (uint32_t h = 0; h < num_heads; ++h) {
            size_t hb = ((size_t)s * num_heads + h) * head_dim;
            for (uint32_t d = 0; d < half; ++d) {
                if (d >= rotated) { out[hb + d] = in[hb + d]; out[hb + d + half] = in[hb + d + half]; continue; }
                float c, sn;
                rope_cos_sin(d, head_dim, s + start_pos, theta, scaling, &c, &sn);
                float x0 = in[hb + d], x1 = in[hb + d + half];
                out[hb + d] = x0 * c - x1 * sn;
                out[hb + d + half] = x0 * sn + x1 * c;
            }
        }
}

/* rope_neox_f32_to_f16: same rotation, half() store (RoPE.metal:498-531). */
ERO_API void ero_rope_neox_f32_to_f16(const float *in, uint16_t *out, uint32_t seq_len, uint32_t num_heads,
                                      uint32_t head_dim, uint32_t start_pos, float theta, float scaling,
                                      float partial) {
    size_t n = (size_t)seq_len * num_heads * head_dim;
    float *tmp = (float *)malloc(n * sizeof(float));
    ero_rope_neox_f32(in, tmp, seq_len, num_heads, head_dim, start_pos, theta, scaling, partial);
    for (size_t i = 0; i < n; ++i) out[i] = ero_f32_to_f16(tmp[i]);
    free(tmp);
}

/* convert_f32_to_f16: the V-row append of the dense decode path
 * (LlamaLanguageModel.swift:3676-3684). */
ERO_API void ero_convert_f32_to_f16(const float *in, uint16_t *out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = ero_f32_to_f16(in[i]);
}

ERO_API void ero_convert_f16_to_f32(const uint16_t *in, float *out, size_t n) {
    const float *lut = half_lut();
    for (size_t i = 0; i < n; ++i) out[i] = lut[in[i]];
}

/* ------------------------------------------------------------------ dense GQA attention */

/* cpuGQA, GQATests.swift:9-67: two-pass softmax, [S,H,D] layouts, causal rule
 * "key k visible to query row r iff k <= r + qOffset".  Masked scores are
 * -greatestFiniteMagnitude (their exp underflows to 0).  additive_mask (or NULL) is
 * [seq_len][kv_seq_len], added to the scaled score (GQATests.swift:46). */
static void gqa_one_head(const float *q, const float *k, const float *v, float *out, int seq_len,
                         int head_dim, int num_heads, int num_kv_heads, int causal, int kv_seq_len,
                         int q_offset, int head, float *scores, const float *additive_mask) {
    float scale = 1.0f / sqrtf((float)head_dim);
    int group = num_heads / num_kv_heads;
    int q_stride = num_heads * head_dim;
    int kv_stride = num_kv_heads * head_dim;
    int kv_head = head / group;
    for (int q_row = 0; q_row < seq_len; ++q_row) {
        const float *qv = q + (size_t)q_row * q_stride + (size_t)head * head_dim;
        for (int k_row = 0; k_row < kv_seq_len; ++k_row) {
            if (causal && k_row > q_row + q_offset) { scores[k_row] = -3.402823466e+38f; continue; }
            const float *kv = k + (size_t)k_row * kv_stride + (size_t)kv_head * head_dim;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; ++d) dot += qv[d] * kv[d];
            scores[k_row] = dot * scale + (additive_mask ? additive_mask[(size_t)q_row * kv_seq_len + k_row] : 0.0f);
        }
        float max_val = 0.0f;
        if (kv_seq_len > 0) {
            max_val = scores[0];
            for (int i = 1; i < kv_seq_len; ++i) if (scores[i] > max_val) max_val = scores[i];
        }
        float sum = 0.0f;
        for (int i = 0; i < kv_seq_len; ++i) { scores[i] = expf(scores[i] - max_val); sum += scores[i]; }
        for (int i = 0; i < kv_seq_len; ++i) scores[i] = scores[i] / sum;
        float *ov = out + (size_t)q_row * q_stride + (size_t)head * head_dim;
        for (int d = 0; d < head_dim; ++d) {
            float value = 0.0f;
            for (int k_row = 0; k_row < kv_seq_len; ++k_row)
                value += scores[k_row] * v[(size_t)k_row * kv_stride + (size_t)kv_head * head_dim + d];
            ov[d] = value;
        }
    }
}

ERO_API void ero_gqa_f32_masked(const float *q, const float *k, const float *v, float *out, int seq_len,
                                int head_dim, int num_heads, int num_kv_heads, int causal, int kv_seq_len,
                                int q_offset, int threads, const float *additive_mask);

ERO_API void ero_gqa_f32(const float *q, const float *k, const float *v, float *out, int seq_len,
                         int head_dim, int num_heads, int num_kv_heads, int causal, int kv_seq_len,
                         int q_offset, int threads) {
    ero_gqa_f32_masked(q, k, v, out, seq_len, head_dim, num_heads, num_kv_heads, causal, kv_seq_len, q_offset, threads, NULL);
}

ERO_API void ero_gqa_f32_masked(const float *q, const float *k, const float *v, float *out, int seq_len,
                                int head_dim, int num_heads, int num_kv_heads, int causal, int kv_seq_len,
                                int q_offset, int threads, const float *additive_mask) {
    if (kv_seq_len <= 0) kv_seq_len = seq_len;
    (void)threads;
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
    {
        float *scores = (float *)malloc(sizeof(float) * (size_t)(kv_seq_len > 0 ? kv_seq_len : 1));
#pragma omp for schedule(dynamic, 1)
        for (int head = 0; head < num_heads; ++head)
            gqa_one_head(q, k, v, out, seq_len, head_dim, num_heads, num_kv_heads, causal, kv_seq_len,
                         q_offset, head, scores, additive_mask);
        free(scores);
    }
}

/* What gqa_attention_f16kv computes (GQA.metal:278-387): the same attention with
 * K/V read from fp16 storage and widened to float before the fp32 dot products.
 * k16/v16 have an explicit row stride (elements between consecutive tokens) so a
 * cache slab can be read in place. */
ERO_API void ero_gqa_f16kv(const float *q, const uint16_t *k16, const uint16_t *v16, float *out, int seq_len,
                           int head_dim, int num_heads, int num_kv_heads, int causal, int kv_seq_len,
                           int q_offset, int threads) {
    if (kv_seq_len <= 0) kv_seq_len = seq_len;
    size_t n = (size_t)kv_seq_len * num_kv_heads * head_dim;
    float *k = (float *)malloc(n * sizeof(float));
    float *v = (float *)malloc(n * sizeof(float));
    const float *lut = half_lut();
#pragma omp parallel for num_threads(threads > 0 ? threads : 1)
    for (long i = 0; i < (long)n; ++i) { k[i] = lut[k16[i]]; v[i] = lut[v16[i]]; }
    ero_gqa_f32(q, k, v, out, seq_len, head_dim, num_heads, num_kv_heads, causal, kv_seq_len, q_offset, threads);
    free(k);
    free(v);
}

/* gemma4_decode_gqa_f16kv_windowed (Shaders/Gemma4Decode.metal:222-283): one query token against the ring rows
 * physical = (kvStart + i) % kvCapacity, i < kvCount of a token-major fp16 cache.  Per output element: a pass for the
 * largest score, then value += exp(score - max) * V and sum += exp(score - max) in row order, output value / sum
 * (0 when sum is not positive or there are no rows).  The score is a sequential fp32 dot product times the scale.
 * Parity unpinned: the reference's tests for this kernel (Gemma4DecodeKernelTests.swift:335-474) compare against a CPU
 * routine on generated inputs and hold no literal outputs. */
ERO_API void ero_gqa_f16kv_windowed(const float *q, const uint16_t *k16, const uint16_t *v16, float *out, int num_heads,
                                    int num_kv_heads, int head_dim, int kv_start, int kv_count, int kv_capacity,
                                    float scale) {
    const float *lut = half_lut();
    int group = num_heads / num_kv_heads;
    if (kv_count <= 0 || kv_capacity <= 0) {
        for (int i = 0; i < num_heads * head_dim; ++i) out[i] = 0.0f;
        return;
    }
    float *scores = (float *)malloc(sizeof(float) * (size_t)kv_count);
    for (int head = 0; head < num_heads; ++head) {
        int kv_head = head / group;
        float max_score = -INFINITY;
        for (int i = 0; i < kv_count; ++i) {
            size_t base = ((size_t)((kv_start + i) % kv_capacity) * num_kv_heads + kv_head) * head_dim;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; ++d) dot += q[(size_t)head * head_dim + d] * lut[k16[base + d]];
            scores[i] = dot * scale;
            if (scores[i] > max_score) max_score = scores[i];
        }
        for (int d = 0; d < head_dim; ++d) {
            float sum = 0.0f, value = 0.0f;
            for (int i = 0; i < kv_count; ++i) {
                size_t base = ((size_t)((kv_start + i) % kv_capacity) * num_kv_heads + kv_head) * head_dim;
                float w = expf(scores[i] - max_score);
                value += w * lut[v16[base + d]];
                sum += w;
            }
            out[(size_t)head * head_dim + d] = sum > 0.0f ? value / sum : 0.0f;
        }
    }
    free(scores);
}

/* Split-K merge of per-block (max, sum, unnormalised acc) partials as in
 * gqa_decode_attention_packed_f16kv_reduce, GQA.metal:753-776. */
ERO_API void ero_splitk_merge(const float *part_max, const float *part_sum, const float *part_acc,
                              int num_parts, int head_dim, float *out) {
    float gmax = -INFINITY;
    for (int p = 0; p < num_parts; ++p) if (part_sum[p] > 0.0f && part_max[p] > gmax) gmax = part_max[p];
    float gsum = 0.0f;
    for (int d = 0; d < head_dim; ++d) out[d] = 0.0f;
    for (int p = 0; p < num_parts; ++p) {
        if (!(part_sum[p] > 0.0f)) continue;
        float w = expf(part_max[p] - gmax);
        gsum += part_sum[p] * w;
        for (int d = 0; d < head_dim; ++d) out[d] += part_acc[(size_t)p * head_dim + d] * w;
    }
    float inv = gsum > 0.0f ? 1.0f / gsum : 0.0f;
    for (int d = 0; d < head_dim; ++d) out[d] *= inv;
}

/* ------------------------------------------------------------------ TurboQuant */

static const float kCent2[4] = ER_TQ_CENTROIDS_2BIT;
static const float kThr2[3] = ER_TQ_THRESHOLDS_2BIT;
static const float kCent3[8] = ER_TQ_CENTROIDS_3BIT;
static const float kThr3[7] = ER_TQ_THRESHOLDS_3BIT;
static const float kCent4[16] = ER_TQ_CENTROIDS_4BIT;
static const float kThr4[15] = ER_TQ_THRESHOLDS_4BIT;
static const float kCent5[32] = ER_TQ_CENTROIDS_5BIT;
static const float kThr5[31] = ER_TQ_THRESHOLDS_5BIT;
static const uint32_t kSigns1Neg[4] = ER_TQ_SIGNS1_NEGMASK;
static const uint32_t kSigns2Neg[4] = ER_TQ_SIGNS2_NEGMASK;

static const float *centroids_for(int bits) { return bits == 2 ? kCent2 : bits == 3 ? kCent3 : bits == 4 ? kCent4 : bits == 5 ? kCent5 : NULL; }
static const float *thresholds_for(int bits) { return bits == 2 ? kThr2 : bits == 3 ? kThr3 : bits == 4 ? kThr4 : bits == 5 ? kThr5 : NULL; }

static float sign1(int i) { return (kSigns1Neg[i >> 5] >> (i & 31)) & 1u ? -1.0f : 1.0f; }
static float sign2(int i) { return (kSigns2Neg[i >> 5] >> (i & 31)) & 1u ? -1.0f : 1.0f; }

ERO_API float ero_tq_sign(int which, int i) { return which == 1 ? sign1(i) : sign2(i); }
ERO_API float ero_tq_centroid(int bits, int code) { return centroids_for(bits)[code]; }
ERO_API float ero_tq_threshold(int bits, int i) { return thresholds_for(bits)[i]; }

/* TurboQuantLayout.init, TurboQuant.swift:275-319 restricted to the fixed presets
 * (highPrecisionChannelCount == 0): words = ceil(128*bits/32); bytesPerRow adds
 * 4 residual-sign words, 4 outlier-mask words and two float scalars (:321-326). */
ERO_API int ero_tq_code_words_per_row(int bits) { return (ERO_DIM * bits + 31) / 32; }
ERO_API int ero_tq_bytes_per_row(int bits) { return (ero_tq_code_words_per_row(bits) + 4 + 4) * 4 + 2 * 4; }

/* Generic layout arithmetic of the same initialiser for presets with a
 * high-precision side band, so every word count asserted by
 * TurboQuantReferenceTests.swift:121-143 can be reproduced. */
ERO_API void ero_tq_layout_words(int regular_bits, int high_bits, int high_count, int *code_words,
                                 int *base_words, int *sideband_words) {
    int code_bits = (ERO_DIM - high_count) * regular_bits + high_count * high_bits;
    int base_bits = ERO_DIM * regular_bits;
    int side_bits = high_count * (high_bits - regular_bits);
    /* codeBitsPerRow == runtimeBaseBits + runtimeSidebandBits for every preset. */
    *code_words = (code_bits + 31) / 32;
    *base_words = (base_bits + 31) / 32;
    *sideband_words = (side_bits + 31) / 32;
}

/* hadamardInPlace, TurboQuant.swift:985-999: unnormalised FWHT, butterfly widths
 * 1,2,...,64, lower index is lhs: (lhs+rhs, lhs-rhs). */
ERO_API void ero_tq_fwht(float *v) {
    for (int width = 1; width < ERO_DIM; width <<= 1) {
        int step = width << 1;
        for (int base = 0; base < ERO_DIM; base += step)
            for (int i = 0; i < width; ++i) {
                float lhs = v[base + i], rhs = v[base + i + width];
                v[base + i] = lhs + rhs;
                v[base + i + width] = lhs - rhs;
            }
    }
}

/* forwardScale = 1 / sqrt(Float(128)) evaluated in Float (TurboQuant.swift:877). */
static float forward_scale(void) { return 1.0f / sqrtf(128.0f); }
ERO_API float ero_tq_forward_scale(void) { return forward_scale(); }

/* randomizedHadamard, TurboQuant.swift:891-906: zero-pad to 128, multiply by signs1,
 * FWHT, multiply by (signs2 * forwardScale).  The seed argument is ignored by the
 * reference and therefore absent here. */
ERO_API void ero_tq_forward(const float *in, int count, float *out) {
    float scale = forward_scale();
    for (int i = 0; i < ERO_DIM; ++i) out[i] = (i < count ? in[i] : 0.0f) * sign1(i);
    ero_tq_fwht(out);
    for (int i = 0; i < ERO_DIM; ++i) out[i] *= sign2(i) * scale;
}

/* inverseRandomizedHadamard, TurboQuant.swift:908-916. */
ERO_API void ero_tq_inverse(const float *in, float *out) {
    float scale = forward_scale();
    for (int i = 0; i < ERO_DIM; ++i) out[i] = in[i] * sign2(i);
    ero_tq_fwht(out);
    for (int i = 0; i < ERO_DIM; ++i) out[i] = (out[i] * sign1(i)) * scale;
}

/* TurboQuantCodebook.code(for:), TurboQuant.swift:692-697: index of the first threshold
 * strictly greater than the value, else the last code (NaN falls through to the last). */
ERO_API int ero_tq_code_for(float value, int bits) {
    const float *thr = thresholds_for(bits);
    int n = (1 << bits) - 1;
    for (int i = 0; i < n; ++i) if (value < thr[i]) return i;
    return n;
}

/* BitPacker.insert / packCodes for outlier-free rows, TurboQuant.swift:1463-1488,1554-1573:
 * code i occupies bits [i*b, i*b+b) of a little-endian stream of 32-bit words. */
ERO_API void ero_tq_pack_codes(const uint8_t *codes, int count, int bits, uint32_t *words) {
    int nwords = (count * bits + 31) / 32;
    for (int w = 0; w < nwords; ++w) words[w] = 0;
    uint32_t mask = (1u << bits) - 1u;
    for (int i = 0; i < count; ++i) {
        int off = i * bits, wi = off / 32, shift = off % 32;
        uint32_t code = codes[i] & mask;
        words[wi] |= code << shift;
        int spill = shift + bits - 32;
        if (spill > 0) words[wi + 1] |= code >> (bits - spill);
    }
}

/* BitPacker.extract / unpackCodes, TurboQuant.swift:1490-1511,1575-1594. */
ERO_API void ero_tq_unpack_codes(const uint32_t *words, int count, int bits, uint8_t *codes) {
    int nwords = (count * bits + 31) / 32;
    uint32_t mask = (1u << bits) - 1u;
    for (int i = 0; i < count; ++i) {
        int off = i * bits, wi = off / 32, shift = off % 32;
        uint32_t value = (words[wi] >> shift) & mask;
        int spill = shift + bits - 32;
        if (spill > 0 && wi + 1 < nwords) {
            uint32_t high = words[wi + 1] & ((1u << spill) - 1u);
            value |= high << (bits - spill);
        }
        codes[i] = (uint8_t)value;
    }
}

/* BitPacker.packCodes with an outlier side band (TurboQuant.swift:1463-1488): the
 * low regularBits of every code go in the base plane; the extra high bits of masked
 * channels are appended after bit 128*regularBits in channel order.  Needed only to
 * reproduce the split-plane round trip of TurboQuantReferenceTests.swift:166-194. */
static void insert_bits(uint32_t *words, uint32_t code, int width, int off) {
    int wi = off / 32, shift = off % 32;
    uint32_t mask = (1u << width) - 1u;
    words[wi] |= (code & mask) << shift;
    int spill = shift + width - 32;
    if (spill > 0) words[wi + 1] |= (code & mask) >> (width - spill);
}
static uint32_t extract_bits(const uint32_t *words, int nwords, int width, int off) {
    int wi = off / 32, shift = off % 32;
    uint32_t mask = (1u << width) - 1u;
    uint32_t value = (words[wi] >> shift) & mask;
    int spill = shift + width - 32;
    if (spill > 0 && wi + 1 < nwords) value |= (words[wi + 1] & ((1u << spill) - 1u)) << (width - spill);
    return value;
}
ERO_API int ero_tq_pack_codes_split(const uint8_t *codes, const uint8_t *mask, int count, int regular_bits,
                                    int high_bits, uint32_t *words) {
    int side_w = high_bits - regular_bits, side_bits = 0;
    for (int i = 0; i < count; ++i) if (mask[i]) side_bits += side_w;
    int base_bits = count * regular_bits;
    int nwords = (base_bits + side_bits + 31) / 32;
    for (int w = 0; w < nwords; ++w) words[w] = 0;
    int side_off = base_bits;
    for (int i = 0; i < count; ++i) {
        insert_bits(words, codes[i] & ((1u << regular_bits) - 1u), regular_bits, i * regular_bits);
        if (mask[i] && side_w > 0) { insert_bits(words, (uint32_t)codes[i] >> regular_bits, side_w, side_off); side_off += side_w; }
    }
    return nwords;
}
ERO_API void ero_tq_unpack_codes_split(const uint32_t *words, int nwords, const uint8_t *mask, int count,
                                       int regular_bits, int high_bits, uint8_t *codes) {
    int side_w = high_bits - regular_bits, side_off = count * regular_bits;
    for (int i = 0; i < count; ++i) {
        uint32_t raw = extract_bits(words, nwords, regular_bits, i * regular_bits);
        if (mask[i] && side_w > 0) { raw |= extract_bits(words, nwords, side_w, side_off) << regular_bits; side_off += side_w; }
        codes[i] = (uint8_t)raw;
    }
}

/* TurboQuantReferenceEncoder.encode for the fixed presets turbo2/3/4
 * (TurboQuant.swift:1003-1074; usesResidualPath == false, :1420-1426):
 *   rowNorm = sqrt(sum of squares, accumulated left to right in Float)
 *   zero row  -> all-zero row, norms 0
 *   normalized = x / rowNorm ; rotated = randomizedHadamard(normalized)
 *   code[d] = codebook.code(for: rotated[d]) ; recon[d] = centroid(code[d])
 *   stored norm = rowNorm / sqrt(sum recon^2)   (rowNorm itself if that sum is 0)
 *   residualSigns = 0, outlierMask = 0, residualNorm = 0.
 * `rotated_out` (optional) receives the rotated coordinates for diagnostics. */
ERO_API void ero_tq_encode(const float *x, int count, int bits, uint32_t *code_words, uint32_t *residual_signs,
                           uint32_t *outlier_mask, float *row_norm, float *residual_norm, float *rotated_out) {
    int nwords = ero_tq_code_words_per_row(bits);
    float sum = 0.0f;
    for (int i = 0; i < count; ++i) sum = sum + (x[i] * x[i]);
    float norm = sqrtf(sum);
    for (int i = 0; i < 4; ++i) { residual_signs[i] = 0; outlier_mask[i] = 0; }
    *residual_norm = 0.0f;
    if (!(norm > 0.0f)) {
        for (int w = 0; w < nwords; ++w) code_words[w] = 0;
        *row_norm = 0.0f;
        if (rotated_out) for (int i = 0; i < ERO_DIM; ++i) rotated_out[i] = 0.0f;
        return;
    }
    float normalized[ERO_DIM], rotated[ERO_DIM];
    for (int i = 0; i < count; ++i) normalized[i] = x[i] / norm;
    ero_tq_forward(normalized, count, rotated);
    const float *cent = centroids_for(bits);
    uint8_t codes[ERO_DIM];
    float recon_sq = 0.0f;
    for (int i = 0; i < ERO_DIM; ++i) {
        int code = ero_tq_code_for(rotated[i], bits);
        codes[i] = (uint8_t)code;
        float c = cent[code];
        recon_sq = recon_sq + (c * c);
    }
    float recon_norm = sqrtf(recon_sq);
    *row_norm = recon_norm > 0.0f ? (norm / recon_norm) : norm;
    ero_tq_pack_codes(codes, ERO_DIM, bits, code_words);
    if (rotated_out) memcpy(rotated_out, rotated, sizeof(rotated));
}

/* ---- presets with high-precision channels and a QJL residual: balanced (3 + 5 bits, 32 channels) and aggressive
 * (2 + 3 bits, 32 channels), TurboQuantPreset.descriptor, TurboQuant.swift:78-84, 117-124 ---- */

/* TurboQuantReferenceEncoder.topKMask (TurboQuant.swift:1185-1238): the `count` channels with the largest selection score,
 *   .magnitude            |value|
 *   .quantizationBenefit  (value - regularCentroid)^2 - (value - highCentroid)^2   (products and difference rounded separately)
 * Equal scores keep channel order (the sort is applied to an index-ordered sequence and the GPU twin, the selection loop of
 * turboquant_quantize_rows, Shaders/TurboQuant.metal:637-652, takes the first maximum): score descending, index ascending. */
static float selection_score(float value, int regular_bits, int high_bits, int use_benefit) {
    if (!use_benefit) return fabsf(value);
    float rc = centroids_for(regular_bits)[ero_tq_code_for(value, regular_bits)];
    float hc = centroids_for(high_bits)[ero_tq_code_for(value, high_bits)];
    float re = value - rc, he = value - hc;
    float re2 = re * re, he2 = he * he;
    return re2 - he2;
}
ERO_API void ero_tq_topk_mask(const float *values, int count, int regular_bits, int high_bits, int use_benefit, uint8_t *mask) {
    float score[ERO_DIM];
    for (int i = 0; i < ERO_DIM; ++i) { score[i] = selection_score(values[i], regular_bits, high_bits, use_benefit); mask[i] = 0; }
    for (int pick = 0; pick < count && pick < ERO_DIM; ++pick) {
        int best = -1;
        for (int i = 0; i < ERO_DIM; ++i) {
            if (mask[i]) continue;
            if (best < 0 || score[i] > score[best]) best = i;
        }
        mask[best] = 1;
    }
}

/* TurboQuantLayout code words of such a preset (TurboQuant.swift:275-319): base plane 128 * regularBits bits, side band
 * highCount * (highBits - regularBits) bits, each rounded up to words: aggressive 8 + 1, balanced 12 + 2. */
ERO_API int ero_tq_preset_code_words(int regular_bits, int high_bits, int high_count) {
    return (ERO_DIM * regular_bits + 31) / 32 + (high_count * (high_bits - regular_bits) + 31) / 32;
}

/* TurboQuantReferenceEncoder.encode, the residual path (TurboQuant.swift:1003-1100; usesResidualPath, :1420-1426):
 *   rowNorm (left-to-right Float sum); !(rowNorm > 0) -> all-zero row
 *   normalized = x / rowNorm; rotated = randomizedHadamard(normalized); mask = topKMask(rotated)
 *   code[d] = (mask[d] ? highBook : regularBook).code(for: rotated[d]); recon[d] = that book's centroid
 *   residual = normalized - inverseRandomizedHadamard(recon); residualNorm = sqrt(sum residual^2)
 *   residualSigns bit d = randomizedHadamard(residual)[d] >= 0          (the seeds are ignored by the transform, :891-921)
 *   codes packed split-plane (BitPacker.packCodes with a mask, :1463-1488); stored rowNorm is the plain row norm. */
ERO_API void ero_tq_encode_preset(const float *x, int count, int regular_bits, int high_bits, int high_count, int use_benefit,
                                  uint32_t *code_words, uint32_t *residual_signs, uint32_t *outlier_mask, float *row_norm,
                                  float *residual_norm) {
    int nwords = ero_tq_preset_code_words(regular_bits, high_bits, high_count);
    float sum = 0.0f;
    for (int i = 0; i < count; ++i) sum = sum + (x[i] * x[i]);
    float norm = sqrtf(sum);
    for (int w = 0; w < nwords; ++w) code_words[w] = 0;
    for (int i = 0; i < 4; ++i) { residual_signs[i] = 0; outlier_mask[i] = 0; }
    *row_norm = 0.0f;
    *residual_norm = 0.0f;
    if (!(norm > 0.0f)) return;
    float normalized[ERO_DIM], rotated[ERO_DIM], recon[ERO_DIM], approx[ERO_DIM], residual[ERO_DIM], projected[ERO_DIM];
    for (int i = 0; i < ERO_DIM; ++i) normalized[i] = i < count ? x[i] / norm : 0.0f;
    ero_tq_forward(normalized, ERO_DIM, rotated);
    uint8_t mask[ERO_DIM], codes[ERO_DIM];
    ero_tq_topk_mask(rotated, high_count, regular_bits, high_bits, use_benefit, mask);
    for (int i = 0; i < ERO_DIM; ++i) {
        int bits = mask[i] ? high_bits : regular_bits;
        codes[i] = (uint8_t)ero_tq_code_for(rotated[i], bits);
        recon[i] = centroids_for(bits)[codes[i]];
        if (mask[i]) outlier_mask[i >> 5] |= 1u << (i & 31);
    }
    ero_tq_inverse(recon, approx);
    float rsum = 0.0f;
    for (int i = 0; i < ERO_DIM; ++i) { residual[i] = normalized[i] - approx[i]; rsum = rsum + (residual[i] * residual[i]); }
    ero_tq_forward(residual, ERO_DIM, projected);
    for (int i = 0; i < ERO_DIM; ++i) if (projected[i] >= 0.0f) residual_signs[i >> 5] |= 1u << (i & 31);
    uint32_t packed[32];
    int n = ero_tq_pack_codes_split(codes, mask, ERO_DIM, regular_bits, high_bits, packed);
    for (int w = 0; w < n && w < nwords; ++w) code_words[w] = packed[w];
    *row_norm = norm;
    *residual_norm = sqrtf(rsum);
}

/* approximateDecode of such a row (TurboQuant.swift:1117-1170):
 *   x_hat = (inverse(centroids) + inverse(+-1 signs) * qjlScale / 128 * residualNorm * residualWeight) * rowNorm,
 * qjlScale = sqrt(pi / 2) (TurboQuantTransform.qjlScale, :876). */
ERO_API void ero_tq_decode_preset(const uint32_t *code_words, const uint32_t *residual_signs, const uint32_t *outlier_mask,
                                  int regular_bits, int high_bits, int high_count, float row_norm, float residual_norm,
                                  float residual_weight, int count, float *out) {
    uint8_t mask[ERO_DIM], codes[ERO_DIM];
    float recon[ERO_DIM], approx[ERO_DIM], dir[ERO_DIM], qjl[ERO_DIM];
    for (int i = 0; i < ERO_DIM; ++i) mask[i] = (outlier_mask[i >> 5] >> (i & 31)) & 1u;
    int nwords = ero_tq_preset_code_words(regular_bits, high_bits, high_count);
    ero_tq_unpack_codes_split(code_words, nwords, mask, ERO_DIM, regular_bits, high_bits, codes);
    for (int i = 0; i < ERO_DIM; ++i) recon[i] = centroids_for(mask[i] ? high_bits : regular_bits)[codes[i]];
    ero_tq_inverse(recon, approx);
    for (int i = 0; i < ERO_DIM; ++i) dir[i] = (residual_signs[i >> 5] >> (i & 31)) & 1u ? 1.0f : -1.0f;
    ero_tq_inverse(dir, qjl);
    const float qjl_scale = sqrtf(3.14159265358979323846f / 2.0f);
    for (int i = 0; i < count; ++i) {
        float q = qjl[i] * qjl_scale * (1.0f / (float)ERO_DIM) * residual_norm * residual_weight;
        out[i] = (approx[i] + q) * row_norm;
    }
}

/* approximateDecode for fixed presets, TurboQuant.swift:1117-1147:
 * x_hat = inverseRandomizedHadamard(centroids) * rowNorm, truncated to `count`. */
ERO_API void ero_tq_decode(const uint32_t *code_words, int bits, float row_norm, int count, float *out) {
    uint8_t codes[ERO_DIM];
    float recon[ERO_DIM], inv[ERO_DIM];
    const float *cent = centroids_for(bits);
    ero_tq_unpack_codes(code_words, ERO_DIM, bits, codes);
    for (int i = 0; i < ERO_DIM; ++i) recon[i] = cent[codes[i]];
    ero_tq_inverse(recon, inv);
    for (int i = 0; i < count; ++i) out[i] = inv[i] * row_norm;
}

/* approximateScoreTerms for fixed presets, TurboQuant.swift:1314-1374:
 * mseDot = sum_d fwd(q)[d] * centroid(code[d]) ; score = rowNorm * mseDot * scale. */
ERO_API float ero_tq_score(const float *q, int count, const uint32_t *code_words, int bits, float row_norm,
                           float scale, float *mse_dot_out) {
    float q_rot[ERO_DIM];
    uint8_t codes[ERO_DIM];
    const float *cent = centroids_for(bits);
    ero_tq_forward(q, count, q_rot);
    ero_tq_unpack_codes(code_words, ERO_DIM, bits, codes);
    float mse = 0.0f;
    for (int d = 0; d < ERO_DIM; ++d) mse += q_rot[d] * cent[codes[d]];
    if (mse_dot_out) *mse_dot_out = mse;
    return row_norm * (mse + 0.0f) * scale;
}

/* Compressed-cache attention for one decode query row, restating
 *   cpuTurboQuantAttention      TurboQuantAttentionTests.swift:1207-1260  (scores, two-pass softmax)
 *   cpuGroupedTurboQuantAttention                      :1262-1288        (kvHead = head / groupSize)
 *   decodeTurboValueOutput                             :1394-1440        (V accumulated in rotated space,
 *                                                                         one inverse transform at the end)
 * and the kernel's visibility rule kvLimit = causal ? min(kvSeqLen, qOffset+1) : kvSeqLen
 * (TurboQuant.metal:1824).  Rows are indexed row = token*numKVHeads + kvHead
 * (KVCache.swift:922, TurboQuant.metal:1874); score = kNorm * mseDot * scale.
 *
 * k_codes/v_codes: [tokens*numKVHeads][words]; k_norm/v_norm: one float per row (the caller
 * passes whatever the cache stores: float, or fp16 widened to float, for the compact format). */
ERO_API void ero_tq_attention_decode(const float *q, const uint32_t *k_codes, const float *k_norm, int k_bits,
                                     const uint32_t *v_codes, const float *v_norm, int v_bits, float *out,
                                     int num_heads, int num_kv_heads, int kv_len, float scale, int threads) {
    int group = num_heads / num_kv_heads;
    int kw = ero_tq_code_words_per_row(k_bits), vw = ero_tq_code_words_per_row(v_bits);
    const float *kc = centroids_for(k_bits), *vc = centroids_for(v_bits);
    (void)threads;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : 1)
    for (int head = 0; head < num_heads; ++head) {
        int kv_head = head / group;
        float q_rot[ERO_DIM];
        ero_tq_forward(q + (size_t)head * ERO_DIM, ERO_DIM, q_rot);
        float *scores = (float *)malloc(sizeof(float) * (size_t)(kv_len > 0 ? kv_len : 1));
        uint8_t codes[ERO_DIM];
        for (int t = 0; t < kv_len; ++t) {
            size_t row = (size_t)t * num_kv_heads + kv_head;
            ero_tq_unpack_codes(k_codes + row * kw, ERO_DIM, k_bits, codes);
            float mse = 0.0f;
            for (int d = 0; d < ERO_DIM; ++d) mse += q_rot[d] * kc[codes[d]];
            scores[t] = k_norm[row] * mse * scale;
        }
        float acc[ERO_DIM];
        for (int d = 0; d < ERO_DIM; ++d) acc[d] = 0.0f;
        if (kv_len > 0) {
            float max_score = scores[0];
            for (int t = 1; t < kv_len; ++t) if (scores[t] > max_score) max_score = scores[t];
            float sum = 0.0f;
            for (int t = 0; t < kv_len; ++t) { scores[t] = expf(scores[t] - max_score); sum += scores[t]; }
            for (int t = 0; t < kv_len; ++t) {
                size_t row = (size_t)t * num_kv_heads + kv_head;
                float weight = scores[t] / sum;
                ero_tq_unpack_codes(v_codes + row * vw, ERO_DIM, v_bits, codes);
                for (int d = 0; d < ERO_DIM; ++d) acc[d] += weight * v_norm[row] * vc[codes[d]];
            }
        }
        ero_tq_inverse(acc, out + (size_t)head * ERO_DIM);
        free(scores);
    }
}

/* The same attention over rows of a preset with high-precision channels and a QJL residual (balanced, aggressive), restating
 *   cpuTurboQuantAttention          TurboQuantAttentionTests.swift:1207-1260 (score = rowNorm * (mseDot + qjlScale * residualNorm *
 *                                   keyResidualScale * residualDot) * scale, two-pass softmax)
 *   decodeTurboValueOutput          :1394-1440 (rotated MSE part + rotated residual part, one inverse transform each, output =
 *                                   mse + residual * qjlScale * valueResidualScale)
 * and gqa_attention_turboquant_decode (Shaders/TurboQuant.metal:1794-2001), whose residual path is off when keyResidualScale == 0
 * (:1818).  The transforms ignore their seeds (TurboQuant.swift:891-921), so qResidual == qRot.  Rows as the encoder writes them:
 * codes [rows][words] split-plane, signs / mask [rows][4], meta [rows][2] = (rowNorm, residualNorm); row = token*numKVHeads + kvHead. */
ERO_API void ero_tq_attention_decode_preset(const float *q, const uint32_t *k_codes, const uint32_t *k_signs, const uint32_t *k_mask,
                                            const float *k_meta, const uint32_t *v_codes, const uint32_t *v_signs,
                                            const uint32_t *v_mask, const float *v_meta, int regular_bits, int high_bits,
                                            int high_count, float key_residual_scale, float value_residual_scale, float *out,
                                            int num_heads, int num_kv_heads, int kv_len, float scale, int threads) {
    int group = num_heads / num_kv_heads;
    int words = ero_tq_preset_code_words(regular_bits, high_bits, high_count);
    const float qjl = sqrtf(3.14159265358979323846f / 2.0f);
    (void)threads;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : 1)
    for (int head = 0; head < num_heads; ++head) {
        int kv_head = head / group;
        float q_rot[ERO_DIM];
        ero_tq_forward(q + (size_t)head * ERO_DIM, ERO_DIM, q_rot);
        float *scores = (float *)malloc(sizeof(float) * (size_t)(kv_len > 0 ? kv_len : 1));
        uint8_t codes[ERO_DIM], mask[ERO_DIM];
        for (int t = 0; t < kv_len; ++t) {
            size_t row = (size_t)t * num_kv_heads + kv_head;
            for (int d = 0; d < ERO_DIM; ++d) mask[d] = (k_mask[row * 4 + (d >> 5)] >> (d & 31)) & 1u;
            ero_tq_unpack_codes_split(k_codes + row * words, words, mask, ERO_DIM, regular_bits, high_bits, codes);
            float mse = 0.0f, res = 0.0f;
            for (int d = 0; d < ERO_DIM; ++d) {
                mse += q_rot[d] * centroids_for(mask[d] ? high_bits : regular_bits)[codes[d]];
                res += q_rot[d] * (((k_signs[row * 4 + (d >> 5)] >> (d & 31)) & 1u) ? 1.0f : -1.0f);
            }
            scores[t] = k_meta[row * 2] * (mse + (qjl * k_meta[row * 2 + 1] * key_residual_scale * res)) * scale;
        }
        float acc[ERO_DIM], acc_res[ERO_DIM], o_mse[ERO_DIM], o_res[ERO_DIM];
        for (int d = 0; d < ERO_DIM; ++d) { acc[d] = 0.0f; acc_res[d] = 0.0f; }
        if (kv_len > 0) {
            float max_score = scores[0];
            for (int t = 1; t < kv_len; ++t) if (scores[t] > max_score) max_score = scores[t];
            float sum = 0.0f;
            for (int t = 0; t < kv_len; ++t) { scores[t] = expf(scores[t] - max_score); sum += scores[t]; }
            for (int t = 0; t < kv_len; ++t) {
                size_t row = (size_t)t * num_kv_heads + kv_head;
                float weight = scores[t] / sum;
                for (int d = 0; d < ERO_DIM; ++d) mask[d] = (v_mask[row * 4 + (d >> 5)] >> (d & 31)) & 1u;
                ero_tq_unpack_codes_split(v_codes + row * words, words, mask, ERO_DIM, regular_bits, high_bits, codes);
                for (int d = 0; d < ERO_DIM; ++d)
                    acc[d] += weight * v_meta[row * 2] * centroids_for(mask[d] ? high_bits : regular_bits)[codes[d]];
                if (value_residual_scale != 0.0f && v_meta[row * 2 + 1] != 0.0f) {
                    float mag = weight * v_meta[row * 2] * v_meta[row * 2 + 1];
                    for (int d = 0; d < ERO_DIM; ++d)
                        acc_res[d] += mag * (((v_signs[row * 4 + (d >> 5)] >> (d & 31)) & 1u) ? 1.0f : -1.0f);
                }
            }
        }
        ero_tq_inverse(acc, o_mse);
        ero_tq_inverse(acc_res, o_res);
        for (int d = 0; d < ERO_DIM; ++d) out[(size_t)head * ERO_DIM + d] = o_mse[d] + (o_res[d] * qjl * value_residual_scale);
        free(scores);
    }
}

/* ------------------------------------------------------------------ KV ring cache (host logic) */

/* KVCache, KVCache.swift:12-1138, reduced to what the hot path uses: float32 / float16
 * dense storage and turboquantV2 with fixed key/value types.  Layout per layer is the
 * reference's [slot][kvHead][dim] ring (byte offset = writePos * bytesPerToken, :417-431);
 * turbo rows are indexed writePos*numKVHeads + kvHead (:922) in four split buffers
 * (codes, residual signs, outlier mask, metadata; :1072-1097). */
enum { ERO_PREC_F32 = 0, ERO_PREC_F16 = 1, ERO_PREC_TURBO_V2 = 4 };

typedef struct {
    int max_seq_len, num_layers, num_kv_heads, head_dim, precision, key_bits, value_bits;
    int *write_pos, *total_written;
    void **key_dense, **value_dense;                        /* float or uint16_t slabs */
    uint32_t **k_codes, **k_signs, **k_mask, **v_codes, **v_signs, **v_mask;
    float **k_meta, **v_meta;
} ero_kv;

enum { ERO_OK = 0, ERO_ERR_ALLOC = -1, ERO_ERR_INVALID_LAYER = -2, ERO_ERR_PRECISION_MISMATCH = -3,
       ERO_ERR_UNSUPPORTED_STORAGE = -4, ERO_ERR_COMPRESSED_RETRIEVE = -5, ERO_ERR_COMPRESSED_BUFFER = -6,
       ERO_ERR_SHAPE = -7 };

ERO_API ero_kv *ero_kv_create(int max_seq_len, int num_layers, int num_kv_heads, int head_dim, int precision,
                              int key_bits, int value_bits) {
    ero_kv *c = (ero_kv *)calloc(1, sizeof(ero_kv));
    c->max_seq_len = max_seq_len; c->num_layers = num_layers; c->num_kv_heads = num_kv_heads;
    c->head_dim = head_dim; c->precision = precision; c->key_bits = key_bits; c->value_bits = value_bits;
    c->write_pos = (int *)calloc((size_t)num_layers, sizeof(int));
    c->total_written = (int *)calloc((size_t)num_layers, sizeof(int));
    size_t n = (size_t)num_layers;
    c->key_dense = (void **)calloc(n, sizeof(void *)); c->value_dense = (void **)calloc(n, sizeof(void *));
    c->k_codes = (uint32_t **)calloc(n, sizeof(void *)); c->k_signs = (uint32_t **)calloc(n, sizeof(void *));
    c->k_mask = (uint32_t **)calloc(n, sizeof(void *)); c->v_codes = (uint32_t **)calloc(n, sizeof(void *));
    c->v_signs = (uint32_t **)calloc(n, sizeof(void *)); c->v_mask = (uint32_t **)calloc(n, sizeof(void *));
    c->k_meta = (float **)calloc(n, sizeof(void *)); c->v_meta = (float **)calloc(n, sizeof(void *));
    size_t elems = (size_t)max_seq_len * num_kv_heads * head_dim;
    size_t rows = (size_t)max_seq_len * num_kv_heads;
    for (int l = 0; l < num_layers; ++l) {
        if (precision == ERO_PREC_F32 || precision == ERO_PREC_F16) {
            size_t bpe = precision == ERO_PREC_F32 ? 4 : 2;
            c->key_dense[l] = calloc(elems, bpe); c->value_dense[l] = calloc(elems, bpe);
        } else {
            c->k_codes[l] = (uint32_t *)calloc(rows * (size_t)ero_tq_code_words_per_row(key_bits), 4);
            c->v_codes[l] = (uint32_t *)calloc(rows * (size_t)ero_tq_code_words_per_row(value_bits), 4);
            c->k_signs[l] = (uint32_t *)calloc(rows * 4, 4); c->v_signs[l] = (uint32_t *)calloc(rows * 4, 4);
            c->k_mask[l] = (uint32_t *)calloc(rows * 4, 4); c->v_mask[l] = (uint32_t *)calloc(rows * 4, 4);
            c->k_meta[l] = (float *)calloc(rows * 2, 4); c->v_meta[l] = (float *)calloc(rows * 2, 4);
        }
    }
    return c;
}

ERO_API void ero_kv_destroy(ero_kv *c) {
    if (!c) return;
    for (int l = 0; l < c->num_layers; ++l) {
        free(c->key_dense[l]); free(c->value_dense[l]);
        free(c->k_codes[l]); free(c->k_signs[l]); free(c->k_mask[l]); free(c->k_meta[l]);
        free(c->v_codes[l]); free(c->v_signs[l]); free(c->v_mask[l]); free(c->v_meta[l]);
    }
    free(c->key_dense); free(c->value_dense); free(c->k_codes); free(c->k_signs); free(c->k_mask); free(c->k_meta);
    free(c->v_codes); free(c->v_signs); free(c->v_mask); free(c->v_meta);
    free(c->write_pos); free(c->total_written); free(c);
}

/* nextWritePosition, KVCache.swift:823-830. */
static int next_write_position(ero_kv *c, int layer) {
    int wp = c->write_pos[layer];
    c->write_pos[layer] = (wp + 1) % c->max_seq_len;
    c->total_written[layer] += 1;
    return wp;
}

/* currentLength, KVCache.swift:184-188: max over layers of min(totalWritten, maxSeqLen). */
ERO_API int ero_kv_current_length(const ero_kv *c) {
    int best = 0;
    for (int l = 0; l < c->num_layers; ++l) {
        int n = c->total_written[l] < c->max_seq_len ? c->total_written[l] : c->max_seq_len;
        if (n > best) best = n;
    }
    return best;
}

/* append(layer:keys:values:), KVCache.swift:410-453 (+ appendTurboQuant :909-975). */
ERO_API int ero_kv_append_f32(ero_kv *c, int layer, const float *keys, const float *values) {
    if (layer < 0 || layer >= c->num_layers) return ERO_ERR_INVALID_LAYER;
    size_t per_token = (size_t)c->num_kv_heads * c->head_dim;
    if (c->precision == ERO_PREC_F32) {
        int wp = next_write_position(c, layer);
        memcpy((float *)c->key_dense[layer] + (size_t)wp * per_token, keys, per_token * 4);
        memcpy((float *)c->value_dense[layer] + (size_t)wp * per_token, values, per_token * 4);
        return ERO_OK;
    }
    if (c->precision == ERO_PREC_TURBO_V2) {
        int wp = next_write_position(c, layer);
        int kw = ero_tq_code_words_per_row(c->key_bits), vw = ero_tq_code_words_per_row(c->value_bits);
        for (int h = 0; h < c->num_kv_heads; ++h) {
            size_t row = (size_t)wp * c->num_kv_heads + h;
            ero_tq_encode(keys + (size_t)h * c->head_dim, c->head_dim, c->key_bits, c->k_codes[layer] + row * kw,
                          c->k_signs[layer] + row * 4, c->k_mask[layer] + row * 4, c->k_meta[layer] + row * 2,
                          c->k_meta[layer] + row * 2 + 1, NULL);
            ero_tq_encode(values + (size_t)h * c->head_dim, c->head_dim, c->value_bits, c->v_codes[layer] + row * vw,
                          c->v_signs[layer] + row * 4, c->v_mask[layer] + row * 4, c->v_meta[layer] + row * 2,
                          c->v_meta[layer] + row * 2 + 1, NULL);
        }
        return ERO_OK;
    }
    return ERO_ERR_PRECISION_MISMATCH;       /* "default: throw precisionMismatch", :450-452 */
}

/* appendF16, KVCache.swift:455-476. */
ERO_API int ero_kv_append_f16(ero_kv *c, int layer, const uint16_t *keys, const uint16_t *values) {
    if (layer < 0 || layer >= c->num_layers) return ERO_ERR_INVALID_LAYER;
    if (c->precision != ERO_PREC_F16) return ERO_ERR_PRECISION_MISMATCH;
    size_t per_token = (size_t)c->num_kv_heads * c->head_dim;
    int wp = next_write_position(c, layer);
    memcpy((uint16_t *)c->key_dense[layer] + (size_t)wp * per_token, keys, per_token * 2);
    memcpy((uint16_t *)c->value_dense[layer] + (size_t)wp * per_token, values, per_token * 2);
    return ERO_OK;
}

/* orderedRowIndices, KVCache.swift:1130-1138: identity until the ring wraps, then
 * [writePos..<max] + [0..<writePos]. */
ERO_API int ero_kv_ordered_slots(const ero_kv *c, int layer, int *slots) {
    int total = c->total_written[layer], maxn = c->max_seq_len;
    int len = total < maxn ? total : maxn, n = 0;
    if (total <= maxn) { for (int i = 0; i < len; ++i) slots[n++] = i; return n; }
    for (int i = c->write_pos[layer]; i < maxn; ++i) slots[n++] = i;
    for (int i = 0; i < c->write_pos[layer]; ++i) slots[n++] = i;
    return n;
}

/* retrieve(layer:asType:), KVCache.swift:478-522.  elem_bytes is the requested element
 * size (4 = Float, 2 = Float16); a mismatch with the storage precision is
 * precisionMismatch (validateRequestedType, :866-883).  Returns the token count. */
ERO_API int ero_kv_retrieve(const ero_kv *c, int layer, int elem_bytes, void *keys, void *values) {
    if (layer < 0 || layer >= c->num_layers) return ERO_ERR_INVALID_LAYER;
    if (c->precision == ERO_PREC_TURBO_V2) return ERO_ERR_COMPRESSED_RETRIEVE;
    if ((c->precision == ERO_PREC_F32 && elem_bytes != 4) || (c->precision == ERO_PREC_F16 && elem_bytes != 2))
        return ERO_ERR_PRECISION_MISMATCH;
    int *slots = (int *)malloc(sizeof(int) * (size_t)c->max_seq_len);
    int n = ero_kv_ordered_slots(c, layer, slots);
    size_t row_bytes = (size_t)c->num_kv_heads * c->head_dim * (size_t)elem_bytes;
    for (int i = 0; i < n; ++i) {
        memcpy((char *)keys + (size_t)i * row_bytes, (char *)c->key_dense[layer] + (size_t)slots[i] * row_bytes, row_bytes);
        memcpy((char *)values + (size_t)i * row_bytes, (char *)c->value_dense[layer] + (size_t)slots[i] * row_bytes, row_bytes);
    }
    free(slots);
    return n;
}

/* retrieveDecodedTurboQuant, KVCache.swift:524-586. */
ERO_API int ero_kv_retrieve_decoded_turboquant(const ero_kv *c, int layer, float *keys, float *values) {
    if (layer < 0 || layer >= c->num_layers) return ERO_ERR_INVALID_LAYER;
    if (c->precision != ERO_PREC_TURBO_V2) return ERO_ERR_PRECISION_MISMATCH;
    int *slots = (int *)malloc(sizeof(int) * (size_t)c->max_seq_len);
    int n = ero_kv_ordered_slots(c, layer, slots);
    int kw = ero_tq_code_words_per_row(c->key_bits), vw = ero_tq_code_words_per_row(c->value_bits);
    size_t o = 0;
    for (int i = 0; i < n; ++i)
        for (int h = 0; h < c->num_kv_heads; ++h, o += (size_t)c->head_dim) {
            size_t row = (size_t)slots[i] * c->num_kv_heads + h;
            ero_tq_decode(c->k_codes[layer] + row * kw, c->key_bits, c->k_meta[layer][row * 2], c->head_dim, keys + o);
            ero_tq_decode(c->v_codes[layer] + row * vw, c->value_bits, c->v_meta[layer][row * 2], c->head_dim, values + o);
        }
    free(slots);
    return n;
}

/* Raw split-buffer access (turboQuantMetalBuffers, KVCache.swift:647-667). which: 0 codes,
 * 1 residual signs, 2 outlier mask, 3 metadata; is_value selects V. */
ERO_API const void *ero_kv_turbo_buffer(const ero_kv *c, int layer, int is_value, int which) {
    if (layer < 0 || layer >= c->num_layers || c->precision != ERO_PREC_TURBO_V2) return NULL;
    switch (which) {
        case 0: return is_value ? c->v_codes[layer] : c->k_codes[layer];
        case 1: return is_value ? c->v_signs[layer] : c->k_signs[layer];
        case 2: return is_value ? c->v_mask[layer] : c->k_mask[layer];
        default: return is_value ? (void *)c->v_meta[layer] : (void *)c->k_meta[layer];
    }
}
ERO_API const void *ero_kv_dense_buffer(const ero_kv *c, int layer, int is_value) {
    if (layer < 0 || layer >= c->num_layers) return NULL;
    return is_value ? c->value_dense[layer] : c->key_dense[layer];
}

/* cacheParams, KVCache.swift:691-703: {maxSeqLen, currentLen, writePos, numKVHeads, headDim, precision}. */
ERO_API int ero_kv_params(const ero_kv *c, int layer, uint32_t *out6) {
    if (layer < 0 || layer >= c->num_layers) return ERO_ERR_INVALID_LAYER;
    int total = c->total_written[layer];
    out6[0] = (uint32_t)c->max_seq_len;
    out6[1] = (uint32_t)(total < c->max_seq_len ? total : c->max_seq_len);
    out6[2] = (uint32_t)c->write_pos[layer];
    out6[3] = (uint32_t)c->num_kv_heads;
    out6[4] = (uint32_t)c->head_dim;
    out6[5] = (uint32_t)c->precision;
    return ERO_OK;
}

/* reset / advanceWritePosition / setPosition, KVCache.swift:705-729. */
ERO_API void ero_kv_reset(ero_kv *c) {
    for (int l = 0; l < c->num_layers; ++l) { c->write_pos[l] = 0; c->total_written[l] = 0; }
}
ERO_API void ero_kv_advance_write_position(ero_kv *c, int layer, int count) {
    for (int i = 0; i < count; ++i) {
        c->write_pos[layer] = (c->write_pos[layer] + 1) % c->max_seq_len;
        c->total_written[layer] += 1;
    }
}
ERO_API void ero_kv_set_position(ero_kv *c, int position) {
    for (int l = 0; l < c->num_layers; ++l) { c->write_pos[l] = position % c->max_seq_len; c->total_written[l] = position; }
}

/* ------------------------------------------------------------------ whole decode step (baseline timing + parity) */

/* One decode step of one layer over a dense fp16 [slot][kvHead][dim] cache, following the
 * fallback path of fusedDecodePass (LlamaLanguageModel.swift:3649-3938):
 *   V row -> fp16 slot `pos` (convert_f32_to_f16), Q -> NeoX RoPE at `pos` (f32),
 *   K -> NeoX RoPE at `pos` -> fp16 slot `pos`, then gqa_attention_f16kv with
 *   seqLen 1, kvSeqLen pos+1, qOffset pos.
 * q is overwritten with its rotated value when q_rot_out is NULL-safe copy target. */
ERO_API void ero_decode_step_f16(const float *q, const float *k, const float *v, uint16_t *k_cache,
                                 uint16_t *v_cache, float *out, float *q_rot_out, int pos, int num_heads,
                                 int num_kv_heads, int head_dim, float theta, float scaling, int threads) {
    size_t per_token = (size_t)num_kv_heads * head_dim;
    float *q_rot = (float *)malloc(sizeof(float) * (size_t)num_heads * head_dim);
    ero_convert_f32_to_f16(v, v_cache + (size_t)pos * per_token, per_token);
    ero_rope_neox_f32(q, q_rot, 1, (uint32_t)num_heads, (uint32_t)head_dim, (uint32_t)pos, theta, scaling, 1.0f);
    ero_rope_neox_f32_to_f16(k, k_cache + (size_t)pos * per_token, 1, (uint32_t)num_kv_heads, (uint32_t)head_dim,
                             (uint32_t)pos, theta, scaling, 1.0f);
    ero_gqa_f16kv(q_rot, k_cache, v_cache, out, 1, head_dim, num_heads, num_kv_heads, 1, pos + 1, pos, threads);
    if (q_rot_out) memcpy(q_rot_out, q_rot, sizeof(float) * (size_t)num_heads * head_dim);
    free(q_rot);
}

/* Same step over a TurboQuant cache (pure-turbo path, LlamaLanguageModel.swift:3659-3673,
 * 3779-3811, 3867-3881): V row and RoPE'd K row are encoded per kv head into row
 * pos*numKVHeads + kvHead; attention over rows 0..pos.  Norm arrays hold one float per row;
 * when norm_fp16 != 0 the stored norm is rounded to fp16 first (compact format). */
ERO_API void ero_decode_step_turboquant(const float *q, const float *k, const float *v, uint32_t *k_codes,
                                        float *k_norm, int k_bits, uint32_t *v_codes, float *v_norm, int v_bits,
                                        float *out, int pos, int num_heads, int num_kv_heads, float theta,
                                        float scaling, int norm_fp16, int threads) {
    int kw = ero_tq_code_words_per_row(k_bits), vw = ero_tq_code_words_per_row(v_bits);
    float *q_rot = (float *)malloc(sizeof(float) * (size_t)num_heads * ERO_DIM);
    float *k_rot = (float *)malloc(sizeof(float) * (size_t)num_kv_heads * ERO_DIM);
    ero_rope_neox_f32(q, q_rot, 1, (uint32_t)num_heads, ERO_DIM, (uint32_t)pos, theta, scaling, 1.0f);
    ero_rope_neox_f32(k, k_rot, 1, (uint32_t)num_kv_heads, ERO_DIM, (uint32_t)pos, theta, scaling, 1.0f);
    for (int h = 0; h < num_kv_heads; ++h) {
        size_t row = (size_t)pos * num_kv_heads + h;
        uint32_t signs[4], mask[4];
        float rn, resn;
        ero_tq_encode(k_rot + (size_t)h * ERO_DIM, ERO_DIM, k_bits, k_codes + row * kw, signs, mask, &rn, &resn, NULL);
        k_norm[row] = norm_fp16 ? ero_f16_to_f32(ero_f32_to_f16(rn)) : rn;
        ero_tq_encode(v + (size_t)h * ERO_DIM, ERO_DIM, v_bits, v_codes + row * vw, signs, mask, &rn, &resn, NULL);
        v_norm[row] = norm_fp16 ? ero_f16_to_f32(ero_f32_to_f16(rn)) : rn;
    }
    ero_tq_attention_decode(q_rot, k_codes, k_norm, k_bits, v_codes, v_norm, v_bits, out, num_heads, num_kv_heads,
                            pos + 1, 1.0f / sqrtf((float)ERO_DIM), threads);
    free(q_rot);
    free(k_rot);
}

/* ------------------------------------------------------------------ q8_0 KV rows
 * KVCache.encodeQ8Row / decodeQ8Row (KVCache.swift:1007-1057; the GPU twin is quantize_q8_0_rows,
 * Shaders/Dequant_Q8_0.metal:19-49): blocks of 32 elements, 34 bytes each = fp16 scale + 32 int8.
 *   maxAbs  = running max(maxAbs, |x|) with Swift's max (a NaN operand never replaces maxAbs)
 *   scale   = maxAbs > 0 ? maxAbs / 127 : 0           (fp32; the *unrounded* scale divides the values)
 *   q       = Int8(clamping: (x / scale).rounded())   (round half away from zero; the Metal kernel uses rint and
 *             clamps to [-127, 127] -- the two differ only on exact .5 ties and on -128, which |x| <= maxAbs excludes
 *             up to rounding)
 *   stored scale = Float16(scale)
 * Decoding multiplies Float(Float16 scale) by Float(q). */
ERO_API void ero_q8_encode_row(const float *x, int count, uint8_t *blocks) {
    for (int b = 0; b < count / 32; ++b) {
        const float *src = x + 32 * b;
        uint8_t *dst = blocks + 34 * b;
        float max_abs = 0.0f;
        for (int i = 0; i < 32; ++i) {
            float a = fabsf(src[i]);
            if (a >= max_abs) max_abs = a;      /* Swift max(x, y) = y >= x ? y : x */
        }
        float scale = max_abs > 0.0f ? max_abs / 127.0f : 0.0f;
        uint16_t hs = ero_f32_to_f16(scale);
        dst[0] = (uint8_t)(hs & 0xFF);
        dst[1] = (uint8_t)(hs >> 8);
        for (int i = 0; i < 32; ++i) {
            int q = 0;
            if (scale != 0.0f) {
                float r = roundf(src[i] / scale);          /* half away from zero */
                if (!(r == r)) r = 0.0f;                    /* NaN ratio (inf / inf): the reference would trap */
                if (r > 127.0f) r = 127.0f;
                if (r < -128.0f) r = -128.0f;
                q = (int)r;
            }
            dst[2 + i] = (uint8_t)(int8_t)q;
        }
    }
}

ERO_API void ero_q8_decode_row(const uint8_t *blocks, int count, float *out) {
    for (int b = 0; b < count / 32; ++b) {
        const uint8_t *src = blocks + 34 * b;
        float scale = ero_f16_to_f32((uint16_t)(src[0] | (src[1] << 8)));
        for (int i = 0; i < 32; ++i) out[32 * b + i] = scale * (float)(int8_t)src[2 + i];
    }
}

/* gqa_attention_q8kv (Shaders/GQA.metal:389-522): rows are decoded to float (scale * float(q)), then the same
 * attention as cpuGQA.  k/v: [kv_seq_len][num_kv_heads] rows of (head_dim / 32) * 34 bytes. */
ERO_API void ero_gqa_q8kv(const float *q, const uint8_t *k8, const uint8_t *v8, float *out, int seq_len, int head_dim,
                          int num_heads, int num_kv_heads, int causal, int kv_seq_len, int q_offset, int threads) {
    if (kv_seq_len <= 0) kv_seq_len = seq_len;
    size_t rows = (size_t)kv_seq_len * num_kv_heads, row_bytes = (size_t)(head_dim / 32) * 34;
    float *k = (float *)malloc(rows * head_dim * sizeof(float));
    float *v = (float *)malloc(rows * head_dim * sizeof(float));
#pragma omp parallel for num_threads(threads > 0 ? threads : 1)
    for (long r = 0; r < (long)rows; ++r) {
        ero_q8_decode_row(k8 + r * row_bytes, head_dim, k + r * head_dim);
        ero_q8_decode_row(v8 + r * row_bytes, head_dim, v + r * head_dim);
    }
    ero_gqa_f32(q, k, v, out, seq_len, head_dim, num_heads, num_kv_heads, causal, kv_seq_len, q_offset, threads);
    free(k);
    free(v);
}

/* One decode step of a q8_0 cache (fusedDecodePass on a q8_0 layer: NeoX RoPE of Q and K in fp32, quantize_q8_0_rows
 * of the K and V rows into row pos*numKVHeads + kvHead, gqa_attention_q8kv over rows 0..pos). */
ERO_API void ero_decode_step_q8(const float *q, const float *k, const float *v, uint8_t *k_cache, uint8_t *v_cache, float *out,
                                int pos, int num_heads, int num_kv_heads, float theta, float scaling, int threads) {
    float *q_rot = (float *)malloc(sizeof(float) * (size_t)num_heads * ERO_DIM);
    float *k_rot = (float *)malloc(sizeof(float) * (size_t)num_kv_heads * ERO_DIM);
    const size_t row_bytes = (ERO_DIM / 32) * 34;
    ero_rope_neox_f32(q, q_rot, 1, (uint32_t)num_heads, ERO_DIM, (uint32_t)pos, theta, scaling, 1.0f);
    ero_rope_neox_f32(k, k_rot, 1, (uint32_t)num_kv_heads, ERO_DIM, (uint32_t)pos, theta, scaling, 1.0f);
    for (int h = 0; h < num_kv_heads; ++h) {
        size_t row = (size_t)pos * num_kv_heads + h;
        ero_q8_encode_row(k_rot + (size_t)h * ERO_DIM, ERO_DIM, k_cache + row * row_bytes);
        ero_q8_encode_row(v + (size_t)h * ERO_DIM, ERO_DIM, v_cache + row * row_bytes);
    }
    ero_gqa_q8kv(q_rot, k_cache, v_cache, out, 1, ERO_DIM, num_heads, num_kv_heads, 1, pos + 1, pos, threads);
    free(q_rot);
    free(k_rot);
}

/* Per-head RMS norm, the first half of fused_qk_norm_rope_neox (Shaders/RoPE.metal:139-160):
 *   rs = rsqrt(sumSq / headDim + eps), out = raw * rs * weight[dim].
 * sumSq is the simd_sum of the pair terms raw0^2 + raw1^2 (dims i and i + 64) over each 32 pairs plus one add; the order
 * inside simd_sum is not specified by the reference, so it is fixed as the xor butterfly 16, 8, 4, 2, 1 over the pair
 * index (the GPU kernel uses the same order).  rsqrt is evaluated in double and rounded once. */
ERO_API void ero_head_rms_norm(const float *in, const float *weight, float eps, int rows, float *out) {
    for (int r = 0; r < rows; ++r) {
        const float *x = in + (size_t)r * ERO_DIM;
        float s[2][32], t[32];
        for (int half = 0; half < 2; ++half) {
            for (int i = 0; i < 32; ++i) {
                float a = x[32 * half + i], b = x[32 * half + i + 64];
                float aa = a * a, bb = b * b;
                s[half][i] = aa + bb;
            }
            for (int off = 16; off >= 1; off >>= 1) {
                for (int i = 0; i < 32; ++i) t[i] = s[half][i] + s[half][i ^ off];
                memcpy(s[half], t, sizeof(t));
            }
        }
        float sum = s[0][0] + s[1][0];
        float mean = sum / (float)ERO_DIM;
        float arg = mean + eps;
        float rs = (float)(1.0 / sqrt((double)arg));
        for (int d = 0; d < ERO_DIM; ++d) {
            float y = x[d] * rs;
            out[(size_t)r * ERO_DIM + d] = y * weight[d];
        }
    }
}

ERO_API int ero_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
