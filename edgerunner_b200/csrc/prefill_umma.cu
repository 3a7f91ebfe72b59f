// Launcher of the tcgen05 chunked-prefill attention kernel: encodes the K / V tensor maps of the call and launches
// prefill_umma_kernel (GQA groups 1, 2, 4, 8; optional second K operand).
#include "prefill_umma.cuh"

#include <algorithm>

#include "launchers.h"
#include "tmap.h"

namespace er {

namespace {
// fp16 rows [outer][...][128]; box = 64 dims x box_rows tokens, 128-byte swizzle.
//   token-major: dims {128, kv heads, slots, seqs, 1}        box {64, 1, box_rows, 1, 1}
//   page-major : dims {128, page tokens, kv heads, pages, 1}  box {64, box_rows, 1, 1, 1}
bool um_encode(CUtensorMap* map, const uint8_t* base, const KVAddressing& a, uint64_t outer_extent, int box_rows) {
    EncodeTiledFn fn = tensor_map_encode_entry();
    if (fn == nullptr || base == nullptr || (reinterpret_cast<uintptr_t>(base) & 15u) != 0) return false;
    const cuuint64_t row = 256, hkv = static_cast<cuuint64_t>(a.num_kv_heads);
    cuuint64_t dims[5], strides[4];
    cuuint32_t box[5];
    if (a.token_major) {
        const cuuint64_t slots = static_cast<cuuint64_t>(a.max_seq_len);
        dims[0] = 128; dims[1] = hkv; dims[2] = slots; dims[3] = outer_extent; dims[4] = 1;
        strides[0] = row; strides[1] = hkv * row; strides[2] = slots * hkv * row; strides[3] = outer_extent * slots * hkv * row;
        box[0] = 64; box[1] = 1; box[2] = static_cast<cuuint32_t>(box_rows); box[3] = 1; box[4] = 1;
    } else {
        const cuuint64_t pt = static_cast<cuuint64_t>(a.page_size);
        dims[0] = 128; dims[1] = pt; dims[2] = hkv; dims[3] = outer_extent; dims[4] = 1;
        strides[0] = row; strides[1] = pt * row; strides[2] = hkv * pt * row; strides[3] = outer_extent * hkv * pt * row;
        box[0] = 64; box[1] = static_cast<cuuint32_t>(box_rows); box[2] = 1; box[3] = 1; box[4] = 1;
    }
    const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<uint8_t*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int GROUP, bool KSPLIT>
int um_launch(const UmmaPrefillParams& up, int num_kv_heads, cudaStream_t stream) {
    constexpr int kSmem = um_smem_bytes(KSPLIT);
    static_assert(kSmem <= 232448, "prefill kernel exceeds the shared memory of an sm_100 CTA");
    static int configured_device = -1;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (configured_device != device) {
        e = cudaFuncSetAttribute(prefill_umma_kernel<GROUP, KSPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured_device = device;
    }
    constexpr int rows_per_cta = kUmRows / GROUP;
    const int tiles = ((up.base.seq_len + rows_per_cta - 1) / rows_per_cta) * num_kv_heads;
    // One CTA per SM at a time: a grid of `tiles` equal CTAs runs in ceil(tiles / SMs) rounds, the last one on `rest` SMs only.
    // Those last tiles are cut along the keys into `parts` CTAs each (their partial rows merged by a second launch), so the
    // tail round takes 1 / parts of a tile's time: 512 tiles on 148 SMs = 3 rounds + 68 tiles x 2 halves instead of 4 rounds.
    UmmaPrefillParams launch = up;
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    int rest = sms > 0 ? tiles % sms : 0, parts = 1;
    if (launch.base.split_partial != nullptr && rest > 0) {
        parts = std::min(4, sms / rest);
        while (parts > 1 && static_cast<size_t>(rest) * parts * kUmRows * kUmPartialStride > launch.base.split_partial_floats) --parts;
    }
    if (parts > 1) {
        launch.base.split_from = tiles - rest;
        launch.base.split_parts = parts;
    } else {
        launch.base.split_partial = nullptr;
        rest = 0;
    }
    const int ctas = tiles - rest + rest * parts;
    prefill_umma_kernel<GROUP, KSPLIT><<<ctas, kUmThreads, kSmem, stream>>>(launch);
    if (parts > 1) prefill_umma_merge_kernel<GROUP><<<(rest * kUmRows + 7) / 8, 256, 0, stream>>>(launch.base, rest);
    return static_cast<int>(cudaGetLastError());
}

template <int GROUP>
int um_launch_group(const UmmaPrefillParams& up, int num_kv_heads, cudaStream_t stream) {
    return up.base.k_lo_layer != nullptr ? um_launch<GROUP, true>(up, num_kv_heads, stream) : um_launch<GROUP, false>(up, num_kv_heads, stream);
}
}  // namespace

size_t prefill_split_partial_floats(int num_sms) {
    // at most (SMs - 1) tail tiles x parts <= SMs CTAs of partial rows
    return static_cast<size_t>(std::max(num_sms, 1)) * kUmRows * kUmPartialStride;
}

int launch_prefill_umma(int group, const PrefillParams& p, uint64_t outer_extent, int num_kv_heads, int* status, cudaStream_t stream) {
    if (status == nullptr) return kNotBuilt;
    int box_rows = 64;
    if (!p.addr.token_major && p.addr.pages_per_seq > 0) {
        box_rows = p.addr.page_size % 64 == 0 ? 64 : p.addr.page_size % 32 == 0 ? 32 : 16;
        if (p.addr.page_size % 16 != 0) return kNotBuilt;
    }
    UmmaPrefillParams up{};
    up.base = p;
    up.box_rows = box_rows;
    up.layer = 0;
    up.status = status;
    if (!um_encode(&up.k_map, p.k_layer, p.addr, outer_extent, box_rows) || !um_encode(&up.v_map, p.v_layer, p.addr, outer_extent, box_rows))
        return kNotBuilt;
    if (p.k_lo_layer != nullptr && (p.v_lo_layer == nullptr || !um_encode(&up.klo_map, p.k_lo_layer, p.addr, outer_extent, box_rows) ||
                                    !um_encode(&up.vlo_map, p.v_lo_layer, p.addr, outer_extent, box_rows)))
        return kNotBuilt;
    switch (group) {
        case 1: return um_launch_group<1>(up, num_kv_heads, stream);
        case 2: return um_launch_group<2>(up, num_kv_heads, stream);
        case 4: return um_launch_group<4>(up, num_kv_heads, stream);
        case 8: return um_launch_group<8>(up, num_kv_heads, stream);
        default: return kNotBuilt;
    }
}

}  // namespace er
