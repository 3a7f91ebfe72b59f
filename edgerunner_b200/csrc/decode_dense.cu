// Instantiations of the persistent flash-decode kernel for fp16 rows (GQA group sizes 1, 2, 4).
#include <cstdlib>

#include "launchers.h"

namespace er {

int launch_decode_dense(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    static const int variant = [] { const char* e = std::getenv("ER_DENSE_VARIANT"); return e ? std::atoi(e) : 0; }();
    switch (group) {
        case 1: return launch_decode_policy<DensePolicy<1>>(p, grid, stream);
        case 2:
            switch (variant) {
                case 1: return launch_decode_policy<DensePolicy<2, 6, 2, 4>>(p, grid, stream);
                case 2: return launch_decode_policy<DensePolicy<2, 8, 2, 2>>(p, grid, stream);
                case 3: return launch_decode_policy<DensePolicy<2, 4, 3, 6>>(p, grid, stream);
                case 4: return launch_decode_policy<DensePolicy<2, 4, 4, 4>>(p, grid, stream);
                case 5: return launch_decode_policy<DensePolicy<2, 6, 2, 2>>(p, grid, stream);
                case 6: return launch_decode_policy<DensePolicy<2, 8, 1, 2>>(p, grid, stream);
                default: return launch_decode_policy<DensePolicy<2>>(p, grid, stream);
            }
        case 4: return launch_decode_policy<DensePolicy<4>>(p, grid, stream);
        default: return kNotBuilt;
    }
}

}  // namespace er
