// Instantiations of the persistent flash-decode kernel for TurboQuant rows: key/value presets turbo3 and
// turbo4 in every combination, GQA group sizes 1, 2, 4, 8.
#include "flash_decode_turbo_mma.cuh"
#include "launchers.h"

namespace er {

template <int KB, int VB>
static int launch_group(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    // one group of 15 consumer warps over 240-token tiles: the fastest of the measured shapes (group 2, cfg2: two alternating
    // groups of 7 warps +7 %, one group of 11 warps +9 %).  Groups 1 and 2 run 3 stages; group 4 keeps its merge buffers and
    // the 64 KB-aligned table within shared memory with 2 stages (cfg4 decode: 4.43 ms per step against 4.68 ms with 11 warps
    // and 3 stages: the kernel is bound by shared-memory reads, and resident warps are what keeps that pipe busy); group 8
    // (unpacked query fragments: 168 registers) stays at 11 warps and 2 stages.
    switch (group) {
        case 1: return launch_decode_policy<TurboMmaPolicy<1, KB, VB, 15, 1, 3>>(p, grid, stream);
        case 2: return launch_decode_policy<TurboMmaPolicy<2, KB, VB, 15, 1, 3>>(p, grid, stream);
        case 4: return launch_decode_policy<TurboMmaPolicy<4, KB, VB, 15, 1, 2>>(p, grid, stream);
        case 8: return launch_decode_policy<TurboMmaPolicy<8, KB, VB, 11, 1, 2>>(p, grid, stream);
        default: return kNotBuilt;
    }
}

int launch_decode_turbo_2bit(int group, int kbits, int vbits, const DecodeParams& p, int grid, cudaStream_t stream);   // decode_turbo2.cu

int launch_decode_turbo(int group, int kbits, int vbits, const DecodeParams& p, int grid, cudaStream_t stream) {
    if (kbits == 4 && vbits == 4) return launch_group<4, 4>(group, p, grid, stream);
    if (kbits == 4 && vbits == 3) return launch_group<4, 3>(group, p, grid, stream);
    if (kbits == 3 && vbits == 3) return launch_group<3, 3>(group, p, grid, stream);
    if (kbits == 3 && vbits == 4) return launch_group<3, 4>(group, p, grid, stream);
    if (kbits == 2 || vbits == 2) return launch_decode_turbo_2bit(group, kbits, vbits, p, grid, stream);
    return kNotBuilt;
}

}  // namespace er
