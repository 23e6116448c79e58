// Grouped decode GEMV instances (several weight matrices, one activation row, one launch); templates in gemv_impl.cuh.
#include "gemv_impl.cuh"

namespace b200q {
template <typename T>
static int gemv_group_t(int nmat, const int* types, const void* const* ws, void* const* dsts, const int* Ns, int K, const void* x,
                        cudaStream_t s, const PeerExchange* px, int act_mode) {
    if (act_mode == ACT_RAW_CPU) return launch_gemv_group<T, ACT_RAW_CPU>(nmat, types, ws, dsts, Ns, K, x, s, px);
    if (act_mode == ACT_RAW_Q8_1) return launch_gemv_group<T, ACT_RAW_Q8_1>(nmat, types, ws, dsts, Ns, K, x, s, px);
    return B200Q_ERR_UNSUPPORTED;
}

// act_mode: ACT_RAW_Q8_1 (the decode quantizer's arithmetic) or ACT_RAW_CPU (the reference CPU path's activation format)
int gemv_group(int elem, int nmat, const int* types, const void* const* ws, void* const* dsts, const int* Ns, int K, const void* x,
               cudaStream_t s, const PeerExchange* px, int act_mode) {
    if (elem == ELEM_BF16) return gemv_group_t<__nv_bfloat16>(nmat, types, ws, dsts, Ns, K, x, s, px, act_mode);
    if (elem == ELEM_F16) return gemv_group_t<__half>(nmat, types, ws, dsts, Ns, K, x, s, px, act_mode);
    if (elem == ELEM_F32) return gemv_group_t<float>(nmat, types, ws, dsts, Ns, K, x, s, px, act_mode);
    return B200Q_ERR_UNSUPPORTED;
}
}  // namespace b200q
