// Kernel instantiations for tensors of float carried as float.
#include "collectives_impl.cuh"

FR_INSTANTIATE_COMBO(f32, float, float)
