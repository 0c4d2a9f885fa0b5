// Host interface of the single-GPU fused kernels (no torch dependency).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace fairring {

struct AdamWArgs {
  float lr;
  float beta1;
  float beta2;
  float eps;
  float weight_decay;
  float step_size;       // lr / (1 - beta1^t)
  float inv_sqrt_bias2;  // 1 / sqrt(1 - beta2^t)
  float grad_scale;      // multiplied into the gradient first (clipping, loss scale)
};

// p, g, m, v: fp32, 16-byte aligned, n elements each.  Decoupled weight decay,
// same update as torch.optim.AdamW.
// shadow_bf16 (may be null): receives a bf16 copy of the updated parameters.
cudaError_t launchAdamWFlat(float* p, const float* g, float* m, float* v, void* shadow_bf16,
                            int64_t n, const AdamWArgs& a, int sm_count, cudaStream_t stream);
// dst (fp32, 16-byte aligned) = or += src (bf16, 16-byte aligned), n elements.
cudaError_t launchBf16GradToF32(float* dst, const void* src_bf16, int64_t n, bool accumulate,
                                int sm_count, cudaStream_t stream);
// *out += sum(x^2); the caller zeroes *out.
cudaError_t launchSumSq(const float* x, int64_t n, float* out, int sm_count, cudaStream_t stream);

// Device-to-device copy by a kernel of at most `blocks` blocks (falls back to
// cudaMemcpyAsync when a pointer is not 16-byte aligned).
cudaError_t launchCopy(void* dst, const void* src, size_t bytes, int blocks, cudaStream_t stream);

uint64_t localLaunchCountImpl();

}  // namespace fairring
