// Instantiations and launcher of the tensor-core chunked-prefill attention kernel (GQA groups 1, 2, 4, 8).
#include "prefill.cuh"

namespace er {

template <int GROUP, bool KSPLIT>
static int launch_variant(const PrefillParams& p, int num_kv_heads, cudaStream_t stream) {
    constexpr int kSmem = KSPLIT ? kPfSmemBytesSplit : kPfSmemBytes;
    static int configured_device = -1;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (configured_device != device) {
        e = cudaFuncSetAttribute(prefill_f16_kernel<GROUP, KSPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured_device = device;
    }
    constexpr int rows_per_cta = kPfRows / GROUP;
    dim3 grid((p.seq_len + rows_per_cta - 1) / rows_per_cta, num_kv_heads);
    prefill_f16_kernel<GROUP, KSPLIT><<<grid, kPfThreads, kSmem, stream>>>(p);
    return static_cast<int>(cudaGetLastError());
}

template <int GROUP>
static int launch_group(const PrefillParams& p, int num_kv_heads, cudaStream_t stream) {
    return p.k_lo_layer != nullptr ? launch_variant<GROUP, true>(p, num_kv_heads, stream) : launch_variant<GROUP, false>(p, num_kv_heads, stream);
}

int launch_prefill_f16(int group, const PrefillParams& p, int num_kv_heads, cudaStream_t stream) {
    switch (group) {
        case 1: return launch_group<1>(p, num_kv_heads, stream);
        case 2: return launch_group<2>(p, num_kv_heads, stream);
        case 4: return launch_group<4>(p, num_kv_heads, stream);
        case 8: return launch_group<8>(p, num_kv_heads, stream);
        default: return -1;
    }
}

}  // namespace er
