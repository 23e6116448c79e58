// Decode GEMV instances for Q6_K weights (templates in gemv_impl.cuh).
#include "gemv_impl.cuh"

B200Q_DEFINE_GEMV_TYPE(q6_k, b200q::TYPE_Q6_K)
