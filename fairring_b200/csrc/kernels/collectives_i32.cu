// Kernel instantiations for tensors of int32_t carried as int32_t.
#include "collectives_impl.cuh"

FR_INSTANTIATE_COMBO(i32, int32_t, int32_t)
