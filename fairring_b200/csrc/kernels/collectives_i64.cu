// Kernel instantiations for tensors of int64_t carried as int64_t.
#include "collectives_impl.cuh"

FR_INSTANTIATE_COMBO(i64, int64_t, int64_t)
