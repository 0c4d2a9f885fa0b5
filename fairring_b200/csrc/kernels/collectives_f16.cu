// Kernel instantiations for tensors of __half carried as __half.
#include "collectives_impl.cuh"

FR_INSTANTIATE_COMBO(f16, __half, __half)
