// Kernel instantiations for tensors of float carried as __half.
#include "collectives_impl.cuh"

FR_INSTANTIATE_COMBO(f32_f16, float, __half)
