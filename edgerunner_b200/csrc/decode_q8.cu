// Instantiations of the persistent flash-decode kernel for q8_0 rows (GQA group sizes 1, 2, 4, 8).
#include "flash_decode_q8.cuh"
#include "launchers.h"

namespace er {

int launch_decode_q8(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    switch (group) {
        case 1: return launch_decode_policy<Q8MmaPolicy<1>>(p, grid, stream);
        case 2: return launch_decode_policy<Q8MmaPolicy<2>>(p, grid, stream);
        case 4: return launch_decode_policy<Q8MmaPolicy<4>>(p, grid, stream);
        case 8: return launch_decode_policy<Q8MmaPolicy<8>>(p, grid, stream);
        default: return kNotBuilt;
    }
}

}  // namespace er
