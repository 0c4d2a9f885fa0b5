// Kernel instantiations for tensors of uint8_t carried as uint8_t.
#include "collectives_impl.cuh"

FR_INSTANTIATE_COMBO(u8, uint8_t, uint8_t)
