// Instantiations of the persistent flash-decode kernel for fp16 rows (GQA group sizes 1, 2, 4).
#include "launchers.h"

namespace er {

int launch_decode_dense(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    switch (group) {
        case 1: return launch_decode_policy<DensePolicy<1, 6, 2, 4>>(p, grid, stream);
        // 12 consumer warps in two groups over 96-token tiles, 4 stages: best of the measured shapes on B200
        case 2: return launch_decode_policy<DensePolicy<2, 6, 2, 4>>(p, grid, stream);
        case 4: return launch_decode_policy<DensePolicy<4>>(p, grid, stream);
        default: return kNotBuilt;
    }
}

}  // namespace er
