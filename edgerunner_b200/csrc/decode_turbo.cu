// Instantiations of the persistent flash-decode kernel for TurboQuant rows: key/value presets turbo3 and
// turbo4 in every combination, GQA group sizes 1, 2, 4, 8.
#include "flash_decode_turbo_mma.cuh"
#include "launchers.h"

namespace er {

template <int KB, int VB>
static int launch_group(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    // one group of 15 consumer warps over 240-token tiles, 3 stages: the fastest of the measured shapes for group 2 (3.55 ms
    // per cfg2 step; two alternating groups of 7 warps 3.90, one group of 11 warps 3.98).  Group 4 keeps its merge buffers
    // within shared memory with 11 warps, group 8 with 11 warps and 2 stages.
    switch (group) {
        case 1: return launch_decode_policy<TurboMmaPolicy<1, KB, VB, 15, 1, 3>>(p, grid, stream);
        case 2: return launch_decode_policy<TurboMmaPolicy<2, KB, VB, 15, 1, 3>>(p, grid, stream);
        case 4: return launch_decode_policy<TurboMmaPolicy<4, KB, VB, 11, 1, 3>>(p, grid, stream);
        case 8: return launch_decode_policy<TurboMmaPolicy<8, KB, VB, 11, 1, 2>>(p, grid, stream);
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
