// Chunked-prefill GQA attention on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory,
// operands staged by TMA).  Same contract as prefill_f16_kernel (prefill.cuh): query row r at absolute position
// r + qOffset attends to keys 0 .. r + qOffset (Shaders/GQA.metal:278-387, Shaders/FlashAttention.metal:194-264).
//
// One CTA owns 128 "M rows" of one kv head: 128 / GROUP consecutive query rows x the GROUP query heads that share it.
//   warps 0-7 (256 threads)  two threads per M row: thread (h, r) reads columns [32h, 32h+32) of row r of S straight out of
//                            tensor memory, the two halves agree on the row maximum through shared memory (one named
//                            barrier per tile), each writes its half of the P row back over S, and rescales its 64 columns
//                            of the O row when the maximum moved.  Half a row per thread keeps the softmax of a tile
//                            shorter than the tile's matrix products, which run meanwhile on the other S buffer.
//   warp 8, one lane         issues the score products S_b = Q.K^T, as far ahead as the three S buffers allow
//   warp 10, one lane        issues the products O += P_b.V as the P rows arrive; two issuing threads, because the waits
//                            of a single one (about 450 clocks per tile) left the tensor pipe idle between batches.  Products of
//                            different threads are not ordered by issue: S_b of tile j+3 waits for a commit after P.V of tile j
//   warp 9, one lane         issues the TMA loads of the K / V tiles (64 tokens, ring of 6 or 4 stages); a thread of its own,
//                            because issuing a tile's loads costs about as many clocks as issuing its products
// Per 64-token tile j, b = j % 3:  S_b[128x64] = Qhi.K^T + Qlo.K^T [+ Qhi.Klo^T]   8 k-steps of 16 dims, N = 64
//                                  O[128x128] += Phi_b.V + Plo_b.V                   4 k-steps of 16 tokens, N = 128
// (measured issue intervals of tcgen05.mma with M = 128, K = 16: 48 clocks at N = 64, 64 at N = 128, 127 at N = 256,
// the same for an A operand in shared or tensor memory).
// The A operands (Q, P) live in tensor memory: row r is lane r, column c holds elements 2c and 2c+1 as fp16, a
// 16-element k-step is 8 columns.  Tensor memory (512 columns allocated): S_0, S_1, S_2 at 0, 64, 128 (P_b overwrites S_b
// in place: hi parts in its first 32 columns, lo parts in the other 32; the products execute in issue order and S_b of
// tile j+3 is issued after the P.V product of tile j), O at 192, Q hi at 320, Q lo at 384.  Issue order: S(j+2), then
// O += P(j).V(j): the softmax of tile j has two tiles' worth of products to hide behind.
// Q (pre-multiplied by scale*log2 e) and P enter as fp16 hi + lo pairs so that, with K and V exact in fp16, the result
// keeps fp32 accuracy; the optional second K operand serves caches whose rows are expanded from fp32 (TurboQuant).
// Shared-memory operand tiles use the 128-byte swizzle (what TMA writes with SWIZZLE_128B and what the matrix descriptors
// name): rows of 64 halves at a 128-byte pitch, 16-byte chunk c of row r stored at chunk c ^ (r & 7); K and Q/P are
// K-major operands (8-row group stride 1024 B), V is an MN-major B operand (the contraction runs over its rows): leading
// offset = distance between its two 64-dim column blocks, stride offset = 1024 B between 8-token groups.
// Every wait is bounded (2 s); on a timeout the CTA raises its abort flag and the status word, skips the remaining
// waits, frees its tensor memory and returns.
#pragma once

#include "prefill.cuh"

namespace er {

constexpr int kUmRows = 128;          // M rows per CTA
constexpr int kUmPartialStride = 132; // floats per row of a split tile's partial: max, sum, pad, pad, 128 columns
__host__ __device__ constexpr int um_tile(bool ksplit) { return ksplit ? 64 : 128; }   // tokens per K/V tile
constexpr int kUmThreads = 352;
__host__ __device__ constexpr int um_kv_region(bool ksplit) { return um_tile(ksplit) * 128; }   // tile tokens x 64 halves
constexpr int kUmColS = 0, kUmColO = 256, kUmColQhi = 384, kUmColQlo = 448;   // tensor-memory columns
// S / P buffers: two of 128 columns, or three of 64 with the second key operand (whose stages are half again as large)
__host__ __device__ constexpr int um_sbufs(bool ksplit) { return ksplit ? 3 : 2; }
__host__ __device__ constexpr int um_stage_bytes(bool ksplit) { return (ksplit ? 8 : 4) * um_kv_region(ksplit); }   // K [Klo] V [Vlo]
__host__ __device__ constexpr int um_stages(bool) { return 3; }
__host__ __device__ constexpr int um_smem_bytes(bool ksplit) {
    return um_stages(ksplit) * um_stage_bytes(ksplit) + 256 + 3072 + 1024;   // + barriers, (max, denominator) exchange, alignment slack
}

struct UmmaPrefillParams {
    CUtensorMap k_map, v_map, klo_map, vlo_map;   // 5-D, box {64 dims, ...}: see encode_prefill_maps
    PrefillParams base;
    int box_rows;                        // tokens per TMA box (64 / box_rows boxes per region and tile)
    int layer;                           // coordinate of the maps' outermost dimension
    int* status;
};

__device__ __forceinline__ void tma_load_5d_sw(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
        : "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.  The issuing thread keeps the
// constant high word in a register and forms the low word (start address >> 4 | leading offset >> 4 << 16) with one add
// per instruction: the scalar code between two tcgen05.mma is what bounds their issue rate.
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
    return ((smem_addr & 0x3FFFFu) >> 4) | ((lbo_bytes >> 4) << 16);
}
__host__ __device__ constexpr uint32_t umma_desc_hi(uint32_t sbo_bytes) { return (sbo_bytes >> 4) | (1u << 14) | (2u << 29); }
__device__ __forceinline__ uint64_t umma_desc_pack(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}
// Instruction descriptor of kind::f16: fp32 accumulate, fp16 A and B, A K-major.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, bool b_mn_major) {
    return (1u << 4) | (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d_tmem), "l"(adesc),
                 "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// A operand in tensor memory
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }" ::"r"(d_tmem), "r"(a_tmem),
                 "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 consecutive columns of this thread's lane; the caller issues tmem_ld_wait() before using them
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
        "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
        "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32_words(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,"
        "%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]),
        "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]),
        "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16_words(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
                 "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
                 "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,"
        "%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 16-byte chunk `chunk` (0..7) of row `row` in a 128-byte-swizzled region
__device__ __forceinline__ uint32_t um_swz(int row, int chunk) { return static_cast<uint32_t>(row * 128 + ((chunk ^ (row & 7)) << 4)); }

template <int GROUP, bool KSPLIT>
__global__ void __launch_bounds__(kUmThreads, 1) prefill_umma_kernel(const __grid_constant__ UmmaPrefillParams up) {
    constexpr int kStages = um_stages(KSPLIT);
    constexpr int kStageBytes = um_stage_bytes(KSPLIT);
    constexpr int kUmTile = um_tile(KSPLIT), kUmKvRegion = um_kv_region(KSPLIT), kUmSBufs = um_sbufs(KSPLIT);
    constexpr int kHalfCols = kUmTile / 2;     // S columns per softmax thread = P words per row and part
    constexpr int kOffV = (KSPLIT ? 4 : 2) * kUmKvRegion;     // inside a stage: K (2 regions) [Klo (2)] V (2) [Vlo (2)]
    constexpr int kOffKlo = 2 * kUmKvRegion, kOffVlo = 6 * kUmKvRegion;
    constexpr int kBarKvFull = 0, kBarKvEmpty = kStages, kBarSFull = 2 * kStages, kBarPFull = kBarSFull + kUmSBufs,
                  kBarSFree = kBarPFull + kUmSBufs, kBarOFull = kBarSFree + kUmSBufs, kBarQFull = kBarOFull + 1, kNumBars = kBarQFull + 1;
    static_assert(kNumBars * 8 + 16 <= 256, "barrier block");
    extern __shared__ uint8_t um_smem_raw[];
    const PrefillParams& p = up.base;
    const uint32_t sbase = (smem_u32(um_smem_raw) + 1023u) & ~1023u;   // operand tiles need 1024-byte alignment
    uint8_t* sgen = um_smem_raw + (sbase - smem_u32(um_smem_raw));
    uint64_t* bar_gen = reinterpret_cast<uint64_t*>(sgen + kStages * kStageBytes);
    const uint32_t bars = smem_u32(bar_gen);
    auto bar = [&](int i) { return bars + 8u * i; };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_gen + kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + kNumBars) + 1;
    float* xchg = reinterpret_cast<float*>(sgen + kStages * kStageBytes + 256);   // maxima [2 tile parities][2 halves][128 rows], then denominators [2][128]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int kQRowsPerCta = kUmRows / GROUP;
    // linear CTA index -> (tile = query tile x kv head, part of the tile's key range)
    int tile_id = static_cast<int>(blockIdx.x), part = 0, nparts = 1;
    if (p.split_partial != nullptr && tile_id >= p.split_from) {
        const int r = tile_id - p.split_from;
        tile_id = p.split_from + r / p.split_parts;
        part = r % p.split_parts;
        nparts = p.split_parts;
    }
    const int q_tiles = (p.seq_len + kQRowsPerCta - 1) / kQRowsPerCta;
    const int kv_head = tile_id / q_tiles;
    const int q0 = (tile_id % q_tiles) * kQRowsPerCta;

    int kv_len = p.kv_len;
    if (p.kv_len_ptr != nullptr) {
        const int n = *p.kv_len_ptr;
        kv_len = n < p.addr.max_seq_len ? n : p.addr.max_seq_len;
    }
    const int q_offset = p.q_offset_from_end ? kv_len - p.seq_len : p.q_offset;
    const int q_last = min(q0 + kQRowsPerCta, p.seq_len) - 1;
    const int kv_hi = p.causal ? min(kv_len, q_last + q_offset + 1) : kv_len;
    const int total_tiles = (kv_hi + kUmTile - 1) / kUmTile;
    // sliding window: the CTA's first query row is the one that looks furthest back; tiles before its window are skipped
    const int first_tile = p.window > 0 ? max(0, q_offset + q0 - p.window + 1) / kUmTile : 0;
    int tile_begin = min(first_tile, total_tiles), num_tiles = total_tiles - tile_begin;     // this CTA's key tiles: [tile_begin, tile_begin + num_tiles)
    if (nparts > 1) {
        const int per = (num_tiles + nparts - 1) / nparts;
        const int b0 = min(num_tiles, part * per);
        num_tiles = min(num_tiles, b0 + per) - b0;
        tile_begin += b0;
    }

    if (tid == 0) {
        for (int i = 0; i < kNumBars; ++i)
            mbar_init(bar_gen + i, ((i >= kBarPFull && i < kBarPFull + kUmSBufs) || i == kBarQFull) ? 256u : 1u);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 9) {
        // ================= loader: TMA (one lane) =================
        if (lane == 0 && num_tiles > 0) {
            const int boxes = kUmTile / up.box_rows;
            for (int tile = 0; tile < num_tiles; ++tile) {
                const int st = tile % kStages;
                if (tile >= kStages) mbar_wait(bar_gen + kBarKvEmpty + st, ((tile / kStages) - 1) & 1, abort_flag, up.status);
                if (*abort_flag) break;
                const int t0 = (tile_begin + tile) * kUmTile;
                const uint32_t stage = sbase + st * kStageBytes;
                // rows past the cache length are not fetched (their pages may not exist); the consumers clear V there
                int nbox = 0;
                for (int b = 0; b < boxes; ++b) nbox += (t0 + b * up.box_rows < kv_len) ? 1 : 0;
                const uint32_t box_bytes = static_cast<uint32_t>(up.box_rows) * 128u;
                mbar_arrive_expect_tx(bar_gen + kBarKvFull + st, nbox * box_bytes * (KSPLIT ? 8u : 4u));
                for (int b = 0; b < nbox; ++b) {
                    const int slot = t0 + b * up.box_rows;
                    int c1, c2, c3;
                    if (p.addr.token_major) {
                        c1 = kv_head; c2 = slot; c3 = p.seq;
                    } else {
                        const int page_local = slot / p.addr.page_size;
                        c1 = slot - page_local * p.addr.page_size;
                        c2 = kv_head;
                        c3 = p.addr.pages_per_seq > 0 ? p.addr.block_table[p.seq * p.addr.pages_per_seq + page_local] : p.seq;
                    }
                    const uint32_t off = static_cast<uint32_t>(b) * box_bytes;
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        tma_load_5d_sw(stage + r * kUmKvRegion + off, &up.k_map, 64 * r, c1, c2, c3, up.layer, bar(kBarKvFull + st));
                        tma_load_5d_sw(stage + kOffV + r * kUmKvRegion + off, &up.v_map, 64 * r, c1, c2, c3, up.layer, bar(kBarKvFull + st));
                        if (KSPLIT) {
                            tma_load_5d_sw(stage + kOffKlo + r * kUmKvRegion + off, &up.klo_map, 64 * r, c1, c2, c3, up.layer, bar(kBarKvFull + st));
                            tma_load_5d_sw(stage + kOffVlo + r * kUmKvRegion + off, &up.vlo_map, 64 * r, c1, c2, c3, up.layer, bar(kBarKvFull + st));
                        }
                    }
                }
            }
        }
    } else if (warp == 8) {
        // ================= MMA issue (one lane) =================
        if (lane == 0 && num_tiles > 0) {
            constexpr uint32_t idesc_qk = umma_idesc(kUmRows, kUmTile, false);
            constexpr uint32_t idesc_pv = umma_idesc(kUmRows, kHeadDim, true);
            // descriptor low words of the B operands at k-step 0 of stage 0; every other one is a constant away
            constexpr uint32_t kHi = umma_desc_hi(1024);
            const uint32_t k_lo = umma_desc_lo(sbase, 16), klo_lo = umma_desc_lo(sbase + kOffKlo, 16);
            const uint32_t v_lo = umma_desc_lo(sbase + kOffV, kUmKvRegion);
            auto issue_qk = [&](int tile) {   // waits for the tile's K, then S_b = Q K^T
                const int st = tile % kStages, b = tile % kUmSBufs;
                mbar_wait(bar_gen + kBarKvFull + st, (tile / kStages) & 1, abort_flag, up.status);
                tc_fence_after();
                if (*abort_flag) return;
                const uint32_t st_off = static_cast<uint32_t>(st) * (kStageBytes >> 4);
                const uint32_t d = tmem + kUmColS + static_cast<uint32_t>(kUmTile) * b;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t koff = ((kk >> 2) * kUmKvRegion + (kk & 3) * 32) >> 4;
                    const uint64_t kd = umma_desc_pack(k_lo + st_off + koff, kHi);
                    umma_f16_ts(d, tmem + kUmColQhi + 8u * kk, kd, idesc_qk, kk > 0);
                    umma_f16_ts(d, tmem + kUmColQlo + 8u * kk, kd, idesc_qk, 1);
                    if (KSPLIT) umma_f16_ts(d, tmem + kUmColQhi + 8u * kk, umma_desc_pack(klo_lo + st_off + koff, kHi), idesc_qk, 1);
                }
                umma_commit(bar(kBarSFull + b));
            };
            mbar_wait(bar_gen + kBarQFull, 0, abort_flag, up.status);   // Q rows are in tensor memory
            tc_fence_after();
            for (int t = 0; t < num_tiles; ++t) {
                // S_b still holds the P rows of tile t - 3 until their product has been executed
                if (t >= kUmSBufs) mbar_wait(bar_gen + kBarSFree + t % kUmSBufs, ((t / kUmSBufs) - 1) & 1, abort_flag, up.status);
                issue_qk(t);
            }
        }
    } else if (warp == 10) {
        // ================= O += P.V issue (one lane) =================
        if (lane == 0 && num_tiles > 0) {
            constexpr uint32_t idesc_pv = umma_idesc(kUmRows, kHeadDim, true);
            constexpr uint32_t kHi = umma_desc_hi(1024);
            const uint32_t v_lo = umma_desc_lo(sbase + kOffV, kUmKvRegion), vlo_lo = umma_desc_lo(sbase + kOffVlo, kUmKvRegion);
            for (int j = 0; j < num_tiles; ++j) {
                const int st = j % kStages, b = j % kUmSBufs;
                mbar_wait(bar_gen + kBarPFull + b, (j / kUmSBufs) & 1, abort_flag, up.status);   // P of tile j written over S_b
                tc_fence_after();
                if (*abort_flag) break;
                const uint32_t st_off = static_cast<uint32_t>(st) * (kStageBytes >> 4);
                const uint32_t d = tmem + kUmColO, pa = tmem + kUmColS + static_cast<uint32_t>(kUmTile) * b;
#pragma unroll
                for (int kt = 0; kt < kUmTile / 16; ++kt) {
                    const uint64_t vd = umma_desc_pack(v_lo + st_off + ((kt * 2048) >> 4), kHi);
                    umma_f16_ts(d, pa + 8u * kt, vd, idesc_pv, kt > 0 ? 1u : 0u);   // every tile's product starts from zero (see the softmax warps)
                    umma_f16_ts(d, pa + kHalfCols + 8u * kt, vd, idesc_pv, 1u);
                    if (KSPLIT) umma_f16_ts(d, pa + 8u * kt, umma_desc_pack(vlo_lo + st_off + ((kt * 2048) >> 4), kHi), idesc_pv, 1u);
                }
                umma_commit(bar(kBarOFull));           // O includes tile j
                umma_commit(bar(kBarKvEmpty + st));    // stage free
                umma_commit(bar(kBarSFree + b));       // S_b free
            }
        }
    } else {
        // ================= softmax: thread (h, m) = columns [32h, 32h+32) of M row m =================
        const int h = warp >> 2, m = tid & 127;
        const int qi = q0 + m / GROUP, head = kv_head * GROUP + m % GROUP;
        const bool row_ok = qi < p.seq_len;
        const int qpos = q_offset + qi;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        // ---- Q row: fp32 -> [RoPE] -> * scale*log2e -> fp16 hi + lo words; half 0 stores the hi parts, half 1 the lo parts ----
        {
            const float* src = p.q + (static_cast<int64_t>(row_ok ? qi : 0) * p.num_q_heads + head) * kHeadDim;
            uint32_t w[64];   // word c = dims 2c, 2c+1
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {          // dims [8 c8, 8 c8 + 8) and their rotation partners + 64
                float a[8], b[8];
#pragma unroll
                for (int h4 = 0; h4 < 2; ++h4) {
                    const float4 x = row_ok ? *reinterpret_cast<const float4*>(src + 8 * c8 + 4 * h4) : make_float4(0.f, 0.f, 0.f, 0.f);
                    const float4 y = row_ok ? *reinterpret_cast<const float4*>(src + 64 + 8 * c8 + 4 * h4) : make_float4(0.f, 0.f, 0.f, 0.f);
                    a[4 * h4] = x.x; a[4 * h4 + 1] = x.y; a[4 * h4 + 2] = x.z; a[4 * h4 + 3] = x.w;
                    b[4 * h4] = y.x; b[4 * h4 + 1] = y.y; b[4 * h4 + 2] = y.z; b[4 * h4 + 3] = y.w;
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    if (p.apply_rope) {
                        const float2 cs = rope_cos_sin_fast(static_cast<uint32_t>(qpos), p.inv_freq.f[8 * c8 + e], p.rope_scaling);
                        float y0, y1;
                        rope_rotate(a[e], b[e], cs, y0, y1);
                        a[e] = y0; b[e] = y1;
                    }
                    a[e] *= p.scale_log2;
                    b[e] *= p.scale_log2;
                }
#pragma unroll
                for (int e2 = 0; e2 < 4; ++e2) {
                    const uint32_t ah = pack_half2(a[2 * e2], a[2 * e2 + 1]), bh = pack_half2(b[2 * e2], b[2 * e2 + 1]);
                    if (h == 0) {
                        w[4 * c8 + e2] = ah;
                        w[32 + 4 * c8 + e2] = bh;
                    } else {
                        const float2 af = __half22float2(*reinterpret_cast<const __half2*>(&ah));
                        const float2 bf = __half22float2(*reinterpret_cast<const __half2*>(&bh));
                        w[4 * c8 + e2] = pack_half2(a[2 * e2] - af.x, a[2 * e2 + 1] - af.y);
                        w[32 + 4 * c8 + e2] = pack_half2(b[2 * e2] - bf.x, b[2 * e2 + 1] - bf.y);
                    }
                }
            }
            const uint32_t qcol = tmem + (h == 0 ? kUmColQhi : kUmColQlo) + lane_base;
            uint32_t half_words[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) half_words[c] = w[c];
            tmem_st32_words(qcol, half_words);
#pragma unroll
            for (int c = 0; c < 32; ++c) half_words[c] = w[32 + c];
            tmem_st32_words(qcol + 32u, half_words);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(bar_gen + kBarQFull);
        }

        float m_run = -INFINITY, l_run = 0.f;   // m_run: maximum of the whole row; l_run: denominator of this thread's columns
        // The running output lives in registers: the tensor cores add into their fp32 accumulators with truncation, which
        // biases a long accumulation chain (measured: an error growing linearly with the context, 6e-5 of the row's largest
        // output at 20000 keys when O accumulated in tensor memory over the whole context).  Each tile's P.V product
        // therefore starts from zero in tensor memory and is folded into these registers with round-to-nearest arithmetic.
        float o_run[64];
#pragma unroll
        for (int c = 0; c < 64; ++c) o_run[c] = 0.f;
        const uint32_t tmem_o = tmem + kUmColO + 64u * h + lane_base;   // this thread's 64 columns of the O row
        const int limit = min(kv_len - 1, p.causal ? qpos : kv_len - 1);   // last visible token of this row
        const int lower = p.window > 0 ? qpos - p.window + 1 : 0;          // first one (sliding-window layers)
        for (int j = 0; j < num_tiles; ++j) {
            const int t0 = (tile_begin + j) * kUmTile + kHalfCols * h, b = j % kUmSBufs, xb = j & 1;
            const uint32_t tmem_s = tmem + kUmColS + static_cast<uint32_t>(kUmTile) * b + lane_base;
            mbar_wait(bar_gen + kBarSFull + b, (j / kUmSBufs) & 1, abort_flag, up.status);
            tc_fence_after();
            float s[kHalfCols];
            {
                uint32_t r0[32], r1[32];
                tmem_ld32_nowait(tmem_s + kHalfCols * h, r0);
                if (kHalfCols == 64) tmem_ld32_nowait(tmem_s + kHalfCols * h + 32u, r1);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    s[c] = __uint_as_float(r0[c]);
                    if (kHalfCols == 64) s[(32 + c) % kHalfCols] = __uint_as_float(r1[c]);
                }
            }
            if (t0 + kHalfCols - 1 > limit || t0 < lower) {
#pragma unroll
                for (int c = 0; c < kHalfCols; ++c) s[c] = (t0 + c <= limit && t0 + c >= lower) ? s[c] : -INFINITY;
            }
            float mx4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
            for (int c = 4; c < kHalfCols; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], s[c]);
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            xchg[(xb * 2 + h) * 128 + m] = mx;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const float m_new = fmaxf(m_run, fmaxf(mx, xchg[(xb * 2 + (h ^ 1)) * 128 + m]));
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = fast_exp2(m_run - m_use);
            m_run = m_new;
            float ps4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < kHalfCols; ++c) {
                s[c] = fast_exp2(s[c] - m_use);
                ps4[c & 3] += s[c];
            }
            l_run = fmaf(l_run, corr, (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]));
            // fold the previous tile's product (relative to the previous maximum, like o_run) and move both to the new maximum;
            // the read is complete before this thread arrives on the P barrier below, which is what lets the next product
            // overwrite the tile accumulator
            if (j > 0) {
                mbar_wait(bar_gen + kBarOFull, (j - 1) & 1, abort_flag, up.status);
                tc_fence_after();
                if (!*abort_flag) {
#pragma unroll
                    for (int c0 = 0; c0 < 64; c0 += 32) {
                        float o[32];
                        tmem_ld32(tmem_o + c0, o);
#pragma unroll
                        for (int c = 0; c < 32; ++c) o_run[c0 + c] = (o_run[c0 + c] + o[c]) * corr;
                    }
                }
            }
            // the last tile: V rows past the cache length were not fetched; clear them (0 * stale bits must not be NaN)
            if ((tile_begin + j) * kUmTile + kUmTile > kv_len) {
                mbar_wait(bar_gen + kBarKvFull + j % kStages, (j / kStages) & 1, abort_flag, up.status);
                uint8_t* vst = sgen + (j % kStages) * kStageBytes + kOffV;
                const int first = kv_len - (tile_begin + j) * kUmTile;
                for (int idx = tid; idx < (kUmTile - first) * 16; idx += 256) {
                    const int row = first + idx / 16, part = idx % 16;    // 2 regions x 8 chunks
                    *reinterpret_cast<uint4*>(vst + (part >> 3) * kUmKvRegion + row * 128 + (part & 7) * 16) = make_uint4(0, 0, 0, 0);
                    if (KSPLIT)
                        *reinterpret_cast<uint4*>(vst + (kOffVlo - kOffV) + (part >> 3) * kUmKvRegion + row * 128 + (part & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_async_smem();
            }
            // this thread's half of the P row over the S row: hi words in columns [W h, W h + W), lo words W columns further,
            // W = kHalfCols / 2 words per thread and part; hi parts of the whole row fill the buffer's first half
            // (the other half-row thread has read its half of S_b: it published its maximum before the barrier above)
            {
                constexpr int W = kHalfCols / 2;
                uint32_t ph[W], pl[W];
#pragma unroll
                for (int c = 0; c < W; ++c) {
                    const float x0 = s[2 * c], x1 = s[2 * c + 1];
                    ph[c] = pack_half2(x0, x1);
                    const float2 hf = __half22float2(*reinterpret_cast<const __half2*>(&ph[c]));
                    pl[c] = pack_half2(x0 - hf.x, x1 - hf.y);
                }
                if constexpr (W == 32) {
                    tmem_st32_words(tmem_s + W * h, ph);
                    tmem_st32_words(tmem_s + kHalfCols + W * h, pl);
                } else {
                    tmem_st16_words(tmem_s + W * h, ph);
                    tmem_st16_words(tmem_s + kHalfCols + W * h, pl);
                }
                tmem_st_wait();
            }
            tc_fence_before();
            mbar_arrive(bar_gen + kBarPFull + b);
        }
        // ---- O / l: thread (h, m) writes dims [64h, 64h+64) of its row ----
        if (num_tiles > 0) {
            mbar_wait(bar_gen + kBarOFull, (num_tiles - 1) & 1, abort_flag, up.status);
            tc_fence_after();
        }
        xchg[512 + h * 128 + m] = l_run;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const float lsum = l_run + xchg[512 + (h ^ 1) * 128 + m];
        // a part of a split tile leaves (max, sum, unnormalised row) for the merge launch instead of the finished row
        const bool partial = nparts > 1;
        const float inv = partial ? 1.f : (lsum > 0.f ? 1.0f / lsum : 0.f);
        float* prow = partial ? p.split_partial + (static_cast<int64_t>(static_cast<int>(blockIdx.x) - p.split_from) * kUmRows + m) * kUmPartialStride : nullptr;
        if (partial && h == 0) { prow[0] = m_run; prow[1] = lsum; }
        float* dst = partial ? prow + 4 + 64 * h : p.out + (static_cast<int64_t>(row_ok ? qi : 0) * p.num_q_heads + head) * kHeadDim + 64 * h;
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 32) {
            if (num_tiles > 0 && !*abort_flag) {   // the last tile's product
                float o[32];
                tmem_ld32(tmem_o + c0, o);
#pragma unroll
                for (int c = 0; c < 32; ++c) o_run[c0 + c] += o[c];
            }
            if (row_ok || partial) {
#pragma unroll
                for (int c = 0; c < 32; c += 4)
                    *reinterpret_cast<float4*>(dst + c0 + c) =
                        make_float4(o_run[c0 + c] * inv, o_run[c0 + c + 1] * inv, o_run[c0 + c + 2] * inv, o_run[c0 + c + 3] * inv);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
}

// Combines the parts of the split tiles: one warp per (split tile, M row), a lane per 4 dims.
template <int GROUP>
__global__ void prefill_umma_merge_kernel(const __grid_constant__ PrefillParams p, int tiles) {
    const int lane = threadIdx.x & 31;
    const int64_t job = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (job >= static_cast<int64_t>(tiles) * kUmRows) return;
    const int t = static_cast<int>(job / kUmRows), m = static_cast<int>(job % kUmRows);
    constexpr int kQRowsPerCta = kUmRows / GROUP;
    const int tile_id = p.split_from + t;
    const int q_tiles = (p.seq_len + kQRowsPerCta - 1) / kQRowsPerCta;
    const int kv_head = tile_id / q_tiles, qi = (tile_id % q_tiles) * kQRowsPerCta + m / GROUP, head = kv_head * GROUP + m % GROUP;
    if (qi >= p.seq_len) return;
    const float* base = p.split_partial + (static_cast<int64_t>(t) * p.split_parts * kUmRows + m) * kUmPartialStride;
    float M = -INFINITY;
    for (int s = 0; s < p.split_parts; ++s) M = fmaxf(M, base[static_cast<int64_t>(s) * kUmRows * kUmPartialStride]);
    float L = 0.f, a[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < p.split_parts; ++s) {
        const float* ps = base + static_cast<int64_t>(s) * kUmRows * kUmPartialStride;
        const float wgt = ps[0] == -INFINITY ? 0.f : exp2f(ps[0] - M);
        L = fmaf(ps[1], wgt, L);
        const float4 v = *reinterpret_cast<const float4*>(ps + 4 + 4 * lane);
        a[0] = fmaf(v.x, wgt, a[0]); a[1] = fmaf(v.y, wgt, a[1]); a[2] = fmaf(v.z, wgt, a[2]); a[3] = fmaf(v.w, wgt, a[3]);
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    *reinterpret_cast<float4*>(p.out + (static_cast<int64_t>(qi) * p.num_q_heads + head) * kHeadDim + 4 * lane) =
        make_float4(a[0] * inv, a[1] * inv, a[2] * inv, a[3] * inv);
}

}  // namespace er
