// Shared device helpers: mbarrier / bulk-async-copy PTX wrappers (sm_90+ instructions, compiled for
// sm_100a), bounded waits, fp16 unpacking and the exactly-rounded RoPE angle arithmetic.
#pragma once

#include <cuda_fp16.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace er {

constexpr int kHeadDim = 128;          // the attention / TurboQuant kernels are specialised for head_dim 128
constexpr int kHalfDim = 64;
constexpr int kUnitTokens = 16;        // scheduling quantum: 16 tokens of one kv head
constexpr int kMaxPairs = 2048;        // (layer, sequence) pairs one launch can schedule

// Device status codes mirrored to the host as ER_ERR_DEVICE_TIMEOUT.
constexpr int kStatusTimeout = -12;
// A row of a paged cache fell into a block-table entry that holds no page (mirrored as ER_ERR_OUT_OF_PAGES).
constexpr int kStatusOutOfPages = -10;
// A kernel found its shared-memory window somewhere its table layout cannot use (mirrored as ER_ERR_UNSUPPORTED).
constexpr int kStatusBadLayout = -11;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait on an mbarrier phase.  `abort_flag` lives in shared memory: once any thread of the CTA has
// given up, every later wait returns at once, so the CTA still walks its whole control flow (all named
// barriers and arrivals are reached) and exits; the host sees the status word, never a hung kernel.
// `limit_ns` is the patience of this wait (2 s unless the launch carries a shorter one for a test of this very path).
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          uint64_t limit_ns = 2000000000ull) {
    if (*abort_flag) return;
    if (mbar_try_wait(bar, parity)) return;
    const uint64_t start = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0x3FFu) == 0u) {
            if (*abort_flag) return;
            if (global_timer_ns() - start > limit_ns) {
                *abort_flag = 1;
                atomicExch(status, kStatusTimeout);
                return;
            }
        }
    }
}

// Bulk asynchronous copy global -> shared, completion counted in bytes on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Tiled TMA load of a 5-D box (coordinates innermost first) global -> shared, completion on an mbarrier.  The
// innermost coordinate times the element size must be a multiple of 16 bytes (always 0 here); destination 128-byte
// aligned.  Out-of-range rows are filled with zeros and still count towards the box's bytes.
__device__ __forceinline__ void tma_load_5d(void* dst_smem, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(
            smem_u32(dst_smem)),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void prefetch_l2(const void* ptr) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
}

// Per-head RMS-norm factor rsqrt(sum(x^2) / 128 + eps) of a 128-float row, summed in the order head_rms_norm_kernel uses
// (pair terms x[i]^2 + x[i+64]^2, xor butterfly 16..1 over each 32 pairs, one add).  All 32 lanes take part.
// A load of a step's q / k / v row.  COHERENT = false: the rows are inputs of the launch (read-only path, L1).  true: the
// launch itself staged them (host-buffer steps), so they are read at L2, the point its own stores are visible at.
template <bool COHERENT, typename T>
__device__ __forceinline__ T ld_step_row(const T* ptr) {
    if constexpr (COHERENT) return __ldcg(ptr); else return __ldg(ptr);
}

template <bool COHERENT = false>
__device__ __forceinline__ float head_rms_scale(const float* row, float eps, int lane) {
    const float a = ld_step_row<COHERENT>(row + lane), b = ld_step_row<COHERENT>(row + lane + 64), c = ld_step_row<COHERENT>(row + lane + 32),
                d = ld_step_row<COHERENT>(row + lane + 96);
    float s0 = __fadd_rn(__fmul_rn(a, a), __fmul_rn(b, b));
    float s1 = __fadd_rn(__fmul_rn(c, c), __fmul_rn(d, d));
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        s0 = __fadd_rn(s0, __shfl_xor_sync(0xffffffffu, s0, off));
        s1 = __fadd_rn(s1, __shfl_xor_sync(0xffffffffu, s1, off));
    }
    return __frsqrt_rn(__fadd_rn(__fdiv_rn(__fadd_rn(s0, s1), static_cast<float>(kHeadDim)), eps));
}

// Named barrier among the consumer warps only (the producer warp never joins it).
template <int THREADS>
__device__ __forceinline__ void consumer_sync() {
    asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

__device__ __forceinline__ void unpack4(const uint2& v, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    const float2 a = __half22float2(h[0]);
    const float2 b = __half22float2(h[1]);
    f[0] = a.x;
    f[1] = a.y;
    f[2] = b.x;
    f[3] = b.y;
}

// RoPE angle -> (cos, sin), each the correctly rounded float of the float-typed expression
//   angle = float(position) * (frequency / scaling)          (Shaders/RoPE.metal:83-87)
// `inv_freq` = 1.0f / powr(theta, float(2*pair)/float(headDim)) is tabulated on the host.
// cos/sin go through double so the result does not depend on the ulp error of a float libm.
__device__ __forceinline__ float2 rope_cos_sin(uint32_t position, float inv_freq, float scaling) {
    const float angle = __fmul_rn(__uint2float_rn(position), __fdiv_rn(inv_freq, scaling));
    double s, c;
    sincos(static_cast<double>(angle), &s, &c);
    return make_float2(static_cast<float>(c), static_cast<float>(s));
}

// Same table in float arithmetic, for rows that are consumed and never stored (prefill queries): accurate to float
// rounding of sincosf, a few hundred times cheaper than the double path.
__device__ __forceinline__ float2 rope_cos_sin_fast(uint32_t position, float inv_freq, float scaling) {
    const float angle = __fmul_rn(__uint2float_rn(position), __fdiv_rn(inv_freq, scaling));
    float s, c;
    sincosf(angle, &s, &c);
    return make_float2(c, s);
}

// (x0, x1) -> (x0*c - x1*s, x0*s + x1*c) with separately rounded products (no FMA contraction), as the
// Swift/Metal source spells it.
__device__ __forceinline__ void rope_rotate(float x0, float x1, float2 cs, float& y0, float& y1) {
    y0 = __fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y));
    y1 = __fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x));
}

struct InvFreqTable {
    float f[kHalfDim];
};

// Where the rows of one layer live.  HEAD_MAJOR storage is the PAGED addressing with one page per
// sequence (page id = sequence index, page_size = ring length), so only two address rules exist.
struct KVAddressing {
    int token_major;        // 1: [seq][slot][kvHead][row]; 0: [page][kvHead][slotInPage][row]
    int num_kv_heads;
    int max_seq_len;        // ring length
    int page_size;          // tokens per page (== padded ring length for HEAD_MAJOR)
    int pages_per_seq;      // block-table stride; 0 = identity (page id = sequence index)
    const int32_t* block_table;   // [seq][pages_per_seq] page ids, -1 = no page assigned
    int* status;            // device status word of the owning cache (paged layout only), else nullptr
};

__device__ __forceinline__ int64_t row_index(const KVAddressing& a, int seq, int head, int slot) {
    if (a.token_major) {
        return (static_cast<int64_t>(seq) * a.max_seq_len + slot) * a.num_kv_heads + head;
    }
    int page, in_page;
    if (a.pages_per_seq == 0) {
        page = seq;
        in_page = slot;
    } else {
        page = __ldg(a.block_table + static_cast<int64_t>(seq) * a.pages_per_seq + slot / a.page_size);
        in_page = slot % a.page_size;
        if (page < 0) {   // no page behind this slot: readers get page 0 (in bounds, flagged), never a wild address
            if (a.status != nullptr) atomicExch(a.status, kStatusOutOfPages);
            page = 0;
        }
    }
    return (static_cast<int64_t>(page) * a.num_kv_heads + head) * a.page_size + in_page;
}

// Row index for a WRITE: -1 (and the status word set) when the slot's block-table entry holds no page, so that a row
// beyond the pages a sequence was given is dropped instead of landing in another sequence's page.
__device__ __forceinline__ int64_t row_index_for_write(const KVAddressing& a, int seq, int head, int slot) {
    if (!a.token_major && a.pages_per_seq != 0 &&
        __ldg(a.block_table + static_cast<int64_t>(seq) * a.pages_per_seq + slot / a.page_size) < 0) {
        if (a.status != nullptr) atomicExch(a.status, kStatusOutOfPages);
        return -1;
    }
    return row_index(a, seq, head, slot);
}

}  // namespace er
