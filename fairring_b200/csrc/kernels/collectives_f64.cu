// Kernel instantiations for tensors of double carried as double.
#include "collectives_impl.cuh"

FR_INSTANTIATE_COMBO(f64, double, double)
