// Decode GEMV instances for Q4_K weights (templates in gemv_impl.cuh).
#include "gemv_impl.cuh"

B200Q_DEFINE_GEMV_TYPE(q4_k, b200q::TYPE_Q4_K)
