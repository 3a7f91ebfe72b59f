// Instantiations of the persistent flash-decode kernel for layers whose keys and values use different row formats (two caches).
#include "flash_decode_hybrid.cuh"
#include "launchers.h"

namespace er {

// Q8MmaPolicy's shape, one group of 11 consumer warps over 176-token tiles, where the value table leaves room: the table sits on
// a 64 KB boundary of the shared window behind the stages and merge buffers (TurboSmemPlan), so 4-bit values (a 64 KB table)
// keep those below 128 KB with 2 stages, and with 8 warps for eight heads per kv head (one warp per head transforms the outputs back).
template <int VB>
static int launch_group(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    constexpr int kStages = VB == 4 ? 2 : 3;
    switch (group) {
        case 1: return launch_decode_policy<Q8KTurboVPolicy<1, VB, 11, 1, kStages>>(p, grid, stream);
        case 2: return launch_decode_policy<Q8KTurboVPolicy<2, VB, 11, 1, kStages>>(p, grid, stream);
        case 4: return launch_decode_policy<Q8KTurboVPolicy<4, VB, 11, 1, kStages>>(p, grid, stream);
        case 8: return launch_decode_policy<Q8KTurboVPolicy<8, VB, VB == 4 ? 8 : 11, 1, 2>>(p, grid, stream);
        default: return kNotBuilt;
    }
}

int launch_decode_q8k_turbov(int group, int vbits, const DecodeParams& p, int grid, cudaStream_t stream) {
    if (vbits == 4) return launch_group<4>(group, p, grid, stream);
    if (vbits == 3) return launch_group<3>(group, p, grid, stream);
    if (vbits == 2) return launch_group<2>(group, p, grid, stream);
    return kNotBuilt;
}

// float16 keys with TurboQuant values: the bytes per token of TurboQuant keys with float16 values below, so those shapes.
template <int VB>
static int launch_dense_keys(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    constexpr int kUnits = VB == 4 ? 8 : 11;
    switch (group) {
        case 1: return launch_decode_policy<DenseKTurboVPolicy<1, VB, kUnits, 1, 2>>(p, grid, stream);
        case 2: return launch_decode_policy<DenseKTurboVPolicy<2, VB, kUnits, 1, 2>>(p, grid, stream);
        case 4: return launch_decode_policy<DenseKTurboVPolicy<4, VB, kUnits, 1, 2>>(p, grid, stream);
        case 8:
            if constexpr (VB == 4) return kNotBuilt;
            else return launch_decode_policy<DenseKTurboVPolicy<8, VB, kUnits, 1, 2>>(p, grid, stream);
        default: return kNotBuilt;
    }
}

int launch_decode_densek_turbov(int group, int vbits, const DecodeParams& p, int grid, cudaStream_t stream) {
    if (vbits == 4) return launch_dense_keys<4>(group, p, grid, stream);
    if (vbits == 3) return launch_dense_keys<3>(group, p, grid, stream);
    if (vbits == 2) return launch_dense_keys<2>(group, p, grid, stream);
    return kNotBuilt;
}

// TurboQuant keys with float16 values: a 256-byte value row per token leaves room for two stages; with 4-bit keys (64 KB table on
// a 64 KB boundary) the tiles shrink to 128 tokens, and eight heads per kv head do not fit beside that table (kNotBuilt: the caller
// keeps such layers on the SIMT kernel).
template <int KB>
static int launch_dense_values(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    constexpr int kUnits = KB == 4 ? 8 : 11;
    switch (group) {
        case 1: return launch_decode_policy<TurboKDenseVPolicy<1, KB, kUnits, 1, 2>>(p, grid, stream);
        case 2: return launch_decode_policy<TurboKDenseVPolicy<2, KB, kUnits, 1, 2>>(p, grid, stream);
        case 4: return launch_decode_policy<TurboKDenseVPolicy<4, KB, kUnits, 1, 2>>(p, grid, stream);
        case 8:
            if constexpr (KB == 4) return kNotBuilt;
            else return launch_decode_policy<TurboKDenseVPolicy<8, KB, kUnits, 1, 2>>(p, grid, stream);
        default: return kNotBuilt;
    }
}

// TurboQuant keys with q8_0 values: the bytes per token of Q8KTurboVPolicy, so its shapes.
template <int KB>
static int launch_q8_values(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    constexpr int kStages = KB == 4 ? 2 : 3;
    switch (group) {
        case 1: return launch_decode_policy<TurboKQ8VPolicy<1, KB, 11, 1, kStages>>(p, grid, stream);
        case 2: return launch_decode_policy<TurboKQ8VPolicy<2, KB, 11, 1, kStages>>(p, grid, stream);
        case 4: return launch_decode_policy<TurboKQ8VPolicy<4, KB, 11, 1, kStages>>(p, grid, stream);
        case 8: return launch_decode_policy<TurboKQ8VPolicy<8, KB, KB == 4 ? 8 : 11, 1, 2>>(p, grid, stream);
        default: return kNotBuilt;
    }
}

int launch_decode_turbok_q8v(int group, int kbits, const DecodeParams& p, int grid, cudaStream_t stream) {
    if (kbits == 4) return launch_q8_values<4>(group, p, grid, stream);
    if (kbits == 3) return launch_q8_values<3>(group, p, grid, stream);
    if (kbits == 2) return launch_q8_values<2>(group, p, grid, stream);
    return kNotBuilt;
}

int launch_decode_turbok_densev(int group, int kbits, const DecodeParams& p, int grid, cudaStream_t stream) {
    if (kbits == 4) return launch_dense_values<4>(group, p, grid, stream);
    if (kbits == 3) return launch_dense_values<3>(group, p, grid, stream);
    if (kbits == 2) return launch_dense_values<2>(group, p, grid, stream);
    return kNotBuilt;
}

// q8_0 with float16 rows (either way round): no table, two stages of 176 tokens.
template <bool Q8_KEYS>
static int launch_plain(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    switch (group) {
        case 1: return launch_decode_policy<PlainPairPolicy<1, Q8_KEYS, 11, 1, 2>>(p, grid, stream);
        case 2: return launch_decode_policy<PlainPairPolicy<2, Q8_KEYS, 11, 1, 2>>(p, grid, stream);
        case 4: return launch_decode_policy<PlainPairPolicy<4, Q8_KEYS, 11, 1, 2>>(p, grid, stream);
        case 8: return launch_decode_policy<PlainPairPolicy<8, Q8_KEYS, 11, 1, 2>>(p, grid, stream);
        default: return kNotBuilt;
    }
}

int launch_decode_q8_dense_pair(int group, int q8_keys, const DecodeParams& p, int grid, cudaStream_t stream) {
    return q8_keys ? launch_plain<true>(group, p, grid, stream) : launch_plain<false>(group, p, grid, stream);
}

}  // namespace er
