// Instantiations of the persistent flash-decode kernel for TurboQuant rows: key/value presets turbo3 and
// turbo4 in every combination, GQA group sizes 1, 2, 4.
#include "flash_decode_turbo_mma.cuh"
#include "launchers.h"

namespace er {

template <int KB, int VB>
static int launch_group(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    // 14 consumer warps in two groups (112-token tiles, 4 stages, 136 registers): the fastest of the measured shapes; 16
    // and 20 warps spill, 12 warps and thinner tiles hide less of the table-lookup latency.
    switch (group) {
        case 1: return launch_decode_policy<TurboMmaPolicy<1, KB, VB, 7, 2, 4>>(p, grid, stream);
        case 2: return launch_decode_policy<TurboMmaPolicy<2, KB, VB, 7, 2, 4>>(p, grid, stream);
        case 4: return launch_decode_policy<TurboMmaPolicy<4, KB, VB, 7, 2, 4>>(p, grid, stream);
        default: return kNotBuilt;
    }
}

int launch_decode_turbo(int group, int kbits, int vbits, const DecodeParams& p, int grid, cudaStream_t stream) {
    if (kbits == 4 && vbits == 4) return launch_group<4, 4>(group, p, grid, stream);
    if (kbits == 4 && vbits == 3) return launch_group<4, 3>(group, p, grid, stream);
    if (kbits == 3 && vbits == 3) return launch_group<3, 3>(group, p, grid, stream);
    if (kbits == 3 && vbits == 4) return launch_group<3, 4>(group, p, grid, stream);
    return kNotBuilt;
}

}  // namespace er
