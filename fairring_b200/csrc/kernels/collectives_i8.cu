// Kernel instantiations for tensors of int8_t carried as int8_t.
#include "collectives_impl.cuh"

FR_INSTANTIATE_COMBO(i8, int8_t, int8_t)
