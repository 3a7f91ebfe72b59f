// Instantiations of the persistent flash-decode kernel for TurboQuant rows with a 2-bit side (turbo2 keys and / or values:
// the value type of the reference's boundary modes, TurboQuantV2Contract, TurboQuant.swift:432-488).  Same shapes as decode_turbo.cu.
#include "flash_decode_turbo_mma.cuh"
#include "launchers.h"

namespace er {

template <int KB, int VB>
static int launch_group(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    switch (group) {
        case 1: return launch_decode_policy<TurboMmaPolicy<1, KB, VB, 15, 1, 3>>(p, grid, stream);
        case 2: return launch_decode_policy<TurboMmaPolicy<2, KB, VB, 15, 1, 3>>(p, grid, stream);
        case 4: return launch_decode_policy<TurboMmaPolicy<4, KB, VB, 15, 1, 2>>(p, grid, stream);
        case 8: return launch_decode_policy<TurboMmaPolicy<8, KB, VB, 11, 1, 2>>(p, grid, stream);
        default: return kNotBuilt;
    }
}

int launch_decode_turbo_2bit(int group, int kbits, int vbits, const DecodeParams& p, int grid, cudaStream_t stream) {
    if (kbits == 4 && vbits == 2) return launch_group<4, 2>(group, p, grid, stream);
    if (kbits == 3 && vbits == 2) return launch_group<3, 2>(group, p, grid, stream);
    if (kbits == 2 && vbits == 2) return launch_group<2, 2>(group, p, grid, stream);
    if (kbits == 2 && vbits == 3) return launch_group<2, 3>(group, p, grid, stream);
    if (kbits == 2 && vbits == 4) return launch_group<2, 4>(group, p, grid, stream);
    return kNotBuilt;
}

}  // namespace er
