// Grouped decode GEMV instances (several weight matrices, one activation row, one launch); templates in gemv_impl.cuh.
#include "gemv_impl.cuh"

namespace b200q {
int gemv_group(int elem, int nmat, const int* types, const void* const* ws, void* const* dsts, const int* Ns, int K, const void* x,
               cudaStream_t s, const PeerExchange* px) {
    if (elem == ELEM_BF16) return launch_gemv_group<__nv_bfloat16>(nmat, types, ws, dsts, Ns, K, x, s, px);
    if (elem == ELEM_F16) return launch_gemv_group<__half>(nmat, types, ws, dsts, Ns, K, x, s, px);
    if (elem == ELEM_F32) return launch_gemv_group<float>(nmat, types, ws, dsts, Ns, K, x, s, px);
    return B200Q_ERR_UNSUPPORTED;
}
}  // namespace b200q
