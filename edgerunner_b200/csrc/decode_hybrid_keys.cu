// Instantiations of the persistent flash-decode kernel for layers with TurboQuant keys and float16 or q8_0 values (two caches).
#include "flash_decode_hybrid.cuh"
#include "launchers.h"

namespace er {

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

}  // namespace er
