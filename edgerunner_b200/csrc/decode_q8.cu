// Instantiations of the persistent flash-decode kernel for q8_0 rows (GQA group sizes 1, 2, 4, 8).
#include "flash_decode_q8.cuh"
#include "launchers.h"

namespace er {

int launch_decode_q8(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    // one group of 11 consumer warps over 176-token tiles, 3 stages: 12 warps leave each thread 168 registers (warps are
    // allocated in fours); the same warps in two alternating groups, or 14-16 warps, measured 25-40 % slower
    switch (group) {
        case 1: return launch_decode_policy<Q8MmaPolicy<1, 11, 1, 3>>(p, grid, stream);
        case 2: return launch_decode_policy<Q8MmaPolicy<2, 11, 1, 3>>(p, grid, stream);
        case 4: return launch_decode_policy<Q8MmaPolicy<4, 11, 1, 3>>(p, grid, stream);
        case 8: return launch_decode_policy<Q8MmaPolicy<8, 11, 1, 3>>(p, grid, stream);
        default: return kNotBuilt;
    }
}

}  // namespace er
