// Instantiations of the persistent flash-decode kernel for layers with q8_0 keys and float16 values or the reverse (two caches).
#include "flash_decode_hybrid.cuh"
#include "launchers.h"

namespace er {

// q8_0 with float16 rows (either way round): no table, two stages of 176 tokens.
template <bool Q8_KEYS>
static int launch_plain(int group, const DecodeParams& p, int grid, cudaStream_t stream) {
    switch (group) {
        case 1: return launch_decode_policy<PlainPairPolicy<1, Q8_KEYS, 11, 1, 2>>(p, grid, stream);
        case 2: return launch_decode_policy<PlainPairPolicy<2, Q8_KEYS, 11, 1, 2>>(p, grid, stream);
        case 4: return launch_decode_policy<PlainPairPolicy<4, Q8_KEYS, 11, 1, 2>>(p, grid, stream);
        case 8: return launch_decode_policy<PlainPairPolicy<8, Q8_KEYS, 11, 1, 2>>(p, grid, stream);
        default: return kNotBuilt;
    }
}

int launch_decode_q8_dense_pair(int group, int q8_keys, const DecodeParams& p, int grid, cudaStream_t stream) {
    return q8_keys ? launch_plain<true>(group, p, grid, stream) : launch_plain<false>(group, p, grid, stream);
}

}  // namespace er
