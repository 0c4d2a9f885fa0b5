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

// LayerNorm over the last dimension (`cols`, a multiple of 8, at most 8192) of a
// [rows, cols] tensor; x / dx are fp32 or bf16, y / dy are fp32 or bf16, the
// affine parameters and the saved per-row mean and 1/std are fp32.
cudaError_t launchLayerNormForward(const void* x, bool x_bf16, const float* gamma, const float* beta,
                                   void* y, bool y_bf16, float* mean, float* rstd, int64_t rows,
                                   int cols, float eps, int sm_count, cudaStream_t stream);
// `partial`: scratch of layerNormBackwardBlocks(rows, sm_count) x 2 x cols floats.
int layerNormBackwardBlocks(int64_t rows, int sm_count);
cudaError_t launchLayerNormBackward(const void* dy, bool y_bf16, const void* x, bool x_bf16,
                                    const float* gamma, const float* mean, const float* rstd, void* dx,
                                    float* partial, float* dgamma, float* dbeta, int64_t rows, int cols,
                                    int sm_count, cudaStream_t stream);

// xnew = x + branch (x fp32, branch fp32 or bf16), y = LayerNorm(xnew); the
// backward adds `gres` (gradient arriving at xnew along the residual path, may
// be null) to the LayerNorm gradient and can also write the sum in bf16
// (`dbranch_bf16`, may be null).
cudaError_t launchAddLayerNormForward(const float* x, const void* branch, bool branch_bf16,
                                      const float* gamma, const float* beta, float* xnew, void* y,
                                      bool y_bf16, float* mean, float* rstd, int64_t rows, int cols,
                                      float eps, int sm_count, cudaStream_t stream);
cudaError_t launchAddLayerNormBackward(const void* dy, bool y_bf16, const float* xnew, const float* gres,
                                       const float* gamma, const float* mean, const float* rstd,
                                       float* dx, void* dbranch_bf16, float* partial, float* dgamma,
                                       float* dbeta, int64_t rows, int cols, int sm_count,
                                       cudaStream_t stream);

// Softmax cross-entropy over [rows, vocab] logits (fp32 or bf16, vocab a
// multiple of 8): per-row loss and log-sum-exp; the backward overwrites the
// logits with their gradient, scaled by *upstream (a device scalar) * scale.
cudaError_t launchCrossEntropyForward(const void* logits, bool bf16, const int64_t* targets, float* loss,
                                      float* lse, int64_t rows, int vocab, int sm_count,
                                      cudaStream_t stream);
cudaError_t launchCrossEntropyBackward(void* logits, bool bf16, const int64_t* targets, const float* lse,
                                       const float* upstream, float scale, int64_t rows, int vocab,
                                       int sm_count, cudaStream_t stream);

uint64_t localLaunchCountImpl();
void noteLocalLaunch();

}  // namespace fairring
