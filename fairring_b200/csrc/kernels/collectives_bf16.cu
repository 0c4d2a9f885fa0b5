// Kernel instantiations for tensors of __nv_bfloat16 carried as __nv_bfloat16.
#include "collectives_impl.cuh"

FR_INSTANTIATE_COMBO(bf16, __nv_bfloat16, __nv_bfloat16)
