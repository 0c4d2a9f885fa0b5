// Kernel instantiations for tensors of float carried as __nv_bfloat16.
#include "collectives_impl.cuh"

FR_INSTANTIATE_COMBO(f32_bf16, float, __nv_bfloat16)
