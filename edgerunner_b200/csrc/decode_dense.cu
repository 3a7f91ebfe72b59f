// Instantiations of the persistent flash-decode kernel for fp16 rows (GQA group sizes 1, 2, 4, 8).
#include "launchers.h"
#include "flash_decode_dense_mma.cuh"
#include "tmap.h"

namespace er {

using Dense4 = DenseMmaPolicy<4, 11, 1, 2>;
using Dense8 = DenseMmaPolicy<8, 10, 1, 2>;
constexpr int kDenseMmaMinSlots = 16384;   // group 2: rings at least this long take the tensor-core policy

int launch_decode_dense(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    switch (group) {
        case 1: return launch_decode_policy<DensePolicy<1, 6, 2, 4>>(p, grid, stream);
        // Group 2: 12 consumer warps in two groups over 96-token tiles, 4 stages (best of the measured shapes on B200).
        // The scalar policy is ahead on short rings (cfg1 shape, 4352 slots: 82.5 against 83.3 us per step) because its state
        // is cheaper to set up and publish per visit; on long rings the tensor-core policy needs fewer instructions per byte
        // and keeps a higher clock under the power cap (context 32768: 6.9 against 6.4 TB/s).  The ring capacity decides.
        case 2:
            if (p.addr.max_seq_len >= kDenseMmaMinSlots) return launch_decode_policy<DenseMmaPolicy<2, 6, 2, 4>>(p, grid, stream);
            return launch_decode_policy<DensePolicy<2, 6, 2, 4>>(p, grid, stream);
        // groups 4 and 8 run both contractions on the tensor cores (the lane-owns-dims form needs 512 FMAs per lane and unit
        // for 4 heads and 128 query registers for 8): 11 consumer warps + producer keep the 168-register budget (warps
        // are allocated in fours); one group over 176-token tiles, 2 stages
        case 4: return launch_decode_policy<Dense4>(p, grid, stream);
        case 8: return launch_decode_policy<Dense8>(p, grid, stream);
        default: return kNotBuilt;
    }
}

int decode_dense_tile_tokens(int group) {
    switch (group) {
        case 1: return DensePolicy<1, 6, 2, 4>::kUnitsPerTile * kUnitTokens;
        case 2: return DensePolicy<2, 6, 2, 4>::kUnitsPerTile * kUnitTokens;   // both policies of this group
        case 4: return Dense4::kUnitsPerTile * kUnitTokens;
        case 8: return Dense8::kUnitsPerTile * kUnitTokens;
        default: return 0;
    }
}

namespace {
bool encode_one(CUtensorMap* map, const uint8_t* base, int64_t layer_stride, int tile, uint64_t layers, uint64_t seqs, uint64_t slots,
                uint64_t kv_heads) {
    EncodeTiledFn fn = tensor_map_encode_entry();
    if (fn == nullptr || (reinterpret_cast<uintptr_t>(base) & 15u) != 0) return false;
    const cuuint64_t row = kRowBytesF16;
    const cuuint64_t dims[5] = {kHeadDim, kv_heads, slots, seqs, layers};
    const cuuint64_t seq_stride = slots * kv_heads * row;
    // a stride of a dimension of extent 1 is never used to form an address but must still be a valid multiple of 16
    const cuuint64_t strides[4] = {row, kv_heads * row, seq_stride, layers > 1 ? static_cast<cuuint64_t>(layer_stride) : seqs * seq_stride};
    const cuuint32_t box[5] = {kHeadDim, 1, static_cast<cuuint32_t>(tile), 1, 1};
    const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<uint8_t*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace

int encode_token_major_maps(DecodeParams& p, int group, uint64_t layers, uint64_t seqs, uint64_t slots, uint64_t kv_heads) {
    p.use_tmap = 0;
    const int tile = decode_dense_tile_tokens(group);
    if (tile == 0 || !p.addr.token_major) return -1;
    if (!encode_one(&p.k_map, p.k_base, p.k_layer_stride_bytes, tile, layers, seqs, slots, kv_heads) ||
        !encode_one(&p.v_map, p.v_base, p.v_layer_stride_bytes, tile, layers, seqs, slots, kv_heads))
        return -1;
    p.use_tmap = 1;
    return 0;
}

}  // namespace er
