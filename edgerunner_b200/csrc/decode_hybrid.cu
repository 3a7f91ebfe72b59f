// Instantiations of the persistent flash-decode kernel for layers with TurboQuant values and q8_0 or float16 keys (two caches).
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

}  // namespace er
