// Decode GEMV instances for Q8_0 weights (templates in gemv_impl.cuh).
#include "gemv_impl.cuh"

B200Q_DEFINE_GEMV_TYPE(q8_0, b200q::TYPE_Q8_0)
