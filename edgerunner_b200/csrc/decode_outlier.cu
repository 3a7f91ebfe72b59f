// Instantiations of the persistent flash-decode kernel for balanced (3 / 5 bits) and aggressive (2 / 3 bits) TurboQuant rows.
#include "flash_decode_outlier_mma.cuh"
#include "launchers.h"

namespace er {

// One group of 15 consumer warps over 240-token tiles, 2 stages (128 registers, no spills): the kernel is bound by its integer
// instructions, and 16 resident warps keep that pipe busier than 12 with 168 registers (balanced rows, 4-layer cfg2 shape:
// 1.36 against 1.49 ms).
template <int RB, int HB>
static int launch_group(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    switch (group) {
        case 1: return launch_decode_policy<OutlierMmaPolicy<1, RB, HB, 15, 1, 2>>(p, grid, stream);
        case 2: return launch_decode_policy<OutlierMmaPolicy<2, RB, HB, 15, 1, 2>>(p, grid, stream);
        case 4: return launch_decode_policy<OutlierMmaPolicy<4, RB, HB, 15, 1, 2>>(p, grid, stream);
        default: return kNotBuilt;
    }
}

int launch_decode_outlier(int group, int regular_bits, int high_bits, const DecodeParams& p, int grid, cudaStream_t stream) {
    if (regular_bits == 3 && high_bits == 5) return launch_group<3, 5>(group, p, grid, stream);
    if (regular_bits == 2 && high_bits == 3) return launch_group<2, 3>(group, p, grid, stream);
    return kNotBuilt;
}

}  // namespace er
