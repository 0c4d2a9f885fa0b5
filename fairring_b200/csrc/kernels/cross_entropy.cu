// Softmax cross-entropy over a [rows, vocab] logits matrix (sm_100a) for the
// language-model workloads.  torch's path under bf16 autocast widens the bf16
// logits to fp32 (a pass), runs log_softmax (a pass each way), nll_loss, and
// narrows the fp32 gradient back to bf16 (another pass): more than ten bytes of
// HBM traffic per logit.  Here the forward reads every logit once from HBM (the
// second sweep over the 100 KB row hits L2) and keeps one float per row; the
// backward recomputes the softmax from the logits and that float and writes the
// gradient over the logits, in their own dtype: five bytes per bf16 logit in all.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "local_kernels.h"

namespace fairring {
namespace {

constexpr int kCeThreads = 512;

__device__ __forceinline__ float toFloat(float v) { return v; }
__device__ __forceinline__ float toFloat(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> struct Vec8;
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

__device__ __forceinline__ float blockReduce(float v, bool is_max, float* scratch) {
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, other) : v + other;
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = scratch[0];
#pragma unroll
  for (int i = 1; i < kCeThreads / 32; ++i) r = is_max ? fmaxf(r, scratch[i]) : r + scratch[i];
  return r;
}

// loss[r] = logsumexp(row r) - row r[target]; lse[r] kept for the backward.
// A negative target marks a row that does not count: loss 0.
template <typename T>
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_fwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ targets,
                         float* __restrict__ loss, float* __restrict__ lse, int64_t rows, int vocab) {
  __shared__ float scratch[kCeThreads / 32];
  const int nvec = vocab / 8;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* row = logits + r * vocab;
    float m = -INFINITY;
    for (int i = threadIdx.x; i < nvec; i += kCeThreads) {
      float v[8];
      Vec8<T>::load(row + i * 8, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) m = fmaxf(m, v[k]);
    }
    m = blockReduce(m, true, scratch);
    float s = 0.f;
    for (int i = threadIdx.x; i < nvec; i += kCeThreads) {
      float v[8];
      Vec8<T>::load(row + i * 8, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) s += __expf(v[k] - m);
    }
    s = blockReduce(s, false, scratch);
    if (threadIdx.x == 0) {
      const float l = m + logf(s);
      lse[r] = l;
      const int64_t t = targets[r];
      loss[r] = t >= 0 && t < vocab ? l - toFloat(row[t]) : 0.f;
    }
  }
}

// logits[r][j] <- (softmax(row r)[j] - [j == target]) * (*upstream) * scale, in place.
template <typename T>
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_bwd_kernel(T* __restrict__ logits, const int64_t* __restrict__ targets,
                         const float* __restrict__ lse, const float* __restrict__ upstream, float scale,
                         int64_t rows, int vocab) {
  const int nvec = vocab / 8;
  const float g = (*upstream) * scale;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    T* row = logits + r * vocab;
    const int64_t t = targets[r];
    const bool counts = t >= 0 && t < vocab;
    const float l = lse[r];
    for (int i = threadIdx.x; i < nvec; i += kCeThreads) {
      float v[8];
      Vec8<T>::load(row + i * 8, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float p = __expf(v[k] - l);
        v[k] = counts ? (p - ((int64_t)i * 8 + k == t ? 1.f : 0.f)) * g : 0.f;
      }
      Vec8<T>::store(row + i * 8, v);
    }
  }
}

}  // namespace

cudaError_t launchCrossEntropyForward(const void* logits, bool bf16, const int64_t* targets, float* loss,
                                      float* lse, int64_t rows, int vocab, int sm_count,
                                      cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  if (vocab % 8 != 0) return cudaErrorInvalidValue;
  int64_t blocks = (int64_t)sm_count * 4;
  if (blocks > rows) blocks = rows;
  if (bf16)
    cross_entropy_fwd_kernel<__nv_bfloat16><<<(unsigned)blocks, kCeThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(logits), targets, loss, lse, rows, vocab);
  else
    cross_entropy_fwd_kernel<float><<<(unsigned)blocks, kCeThreads, 0, stream>>>(
        static_cast<const float*>(logits), targets, loss, lse, rows, vocab);
  noteLocalLaunch();
  return cudaGetLastError();
}

cudaError_t launchCrossEntropyBackward(void* logits, bool bf16, const int64_t* targets, const float* lse,
                                       const float* upstream, float scale, int64_t rows, int vocab,
                                       int sm_count, cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  if (vocab % 8 != 0) return cudaErrorInvalidValue;
  int64_t blocks = (int64_t)sm_count * 4;
  if (blocks > rows) blocks = rows;
  if (bf16)
    cross_entropy_bwd_kernel<__nv_bfloat16><<<(unsigned)blocks, kCeThreads, 0, stream>>>(
        static_cast<__nv_bfloat16*>(logits), targets, lse, upstream, scale, rows, vocab);
  else
    cross_entropy_bwd_kernel<float><<<(unsigned)blocks, kCeThreads, 0, stream>>>(
        static_cast<float*>(logits), targets, lse, upstream, scale, rows, vocab);
  noteLocalLaunch();
  return cudaGetLastError();
}

}  // namespace fairring
