// Instantiations of the persistent flash-decode kernel for fp16 rows (GQA group sizes 1, 2, 4).
#include "launchers.h"

namespace er {

int launch_decode_dense(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    switch (group) {
        case 1: return launch_decode_policy<DensePolicy<1>>(p, grid, stream);
        case 2: return launch_decode_policy<DensePolicy<2>>(p, grid, stream);
        case 4: return launch_decode_policy<DensePolicy<4>>(p, grid, stream);
        default: return kNotBuilt;
    }
}

}  // namespace er
