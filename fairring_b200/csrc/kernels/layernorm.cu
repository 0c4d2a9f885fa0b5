// Fused LayerNorm for the training workloads (sm_100a): one pass over the row
// in each direction, the output written directly in the dtype the next GEMM
// wants.  Under bf16 autocast torch runs layer_norm in fp32 and the following
// linear layer casts its output to bf16 in a pass of its own; backward is two
// more kernels.  Here: forward reads x once and writes y (bf16 or fp32) plus
// two floats per row; backward reads dy and x once, writes dx, and accumulates
// the weight and bias gradients in registers over the rows of a block, followed
// by one small column reduction over the blocks.
//
// A thread owns 8 consecutive columns of up to four 8-column groups
// (row length <= 8192, a multiple of 8); a block of 256 threads owns one row
// at a time.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "local_kernels.h"

namespace fairring {
namespace {

constexpr int kLnThreads = 256;

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// Sum of two values over the block; every thread gets the result.
__device__ __forceinline__ float2 blockSum2(float a, float b, float2* scratch) {
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
  const int w = threadIdx.x >> 5;
  __syncthreads();  // scratch may still be read from the previous row
  if ((threadIdx.x & 31) == 0) scratch[w] = make_float2(a, b);
  __syncthreads();
  float2 s = scratch[0];
#pragma unroll
  for (int i = 1; i < kLnThreads / 32; ++i) {
    s.x += scratch[i].x;
    s.y += scratch[i].y;
  }
  return s;
}

template <typename TX, typename TY, int ITER>
__global__ void __launch_bounds__(kLnThreads, ITER == 1 ? 8 : 1)
layer_norm_fwd_kernel(const TX* __restrict__ x, const float* __restrict__ gamma,
                      const float* __restrict__ beta, TY* __restrict__ y, float* __restrict__ mean_out,
                      float* __restrict__ rstd_out, int64_t rows, int cols, float eps) {
  __shared__ float2 scratch[kLnThreads / 32];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    float v[ITER][8];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = (it * kLnThreads + threadIdx.x) * 8;
      if (c < cols) {
        load8<TX>(x + r * cols + c, v[it]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          s += v[it][i];
          ss += v[it][i] * v[it][i];
        }
      }
    }
    const float2 t = blockSum2(s, ss, scratch);
    const float mean = t.x / cols;
    const float var = fmaxf(t.y / cols - mean * mean, 0.f);
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
      mean_out[r] = mean;
      rstd_out[r] = rstd;
    }
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = (it * kLnThreads + threadIdx.x) * 8;
      if (c < cols) {
        float g[8], b[8], o[8];
        load8<float>(gamma + c, g);
        load8<float>(beta + c, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (v[it][i] - mean) * rstd * g[i] + b[i];
        store8<TY>(y + r * cols + c, o);
      }
    }
  }
}

// dx for the rows of this block, plus this block's partial sums of the weight
// and bias gradients: partial[block][0][col] = sum dy * xhat, [block][1][col] = sum dy.
template <typename TX, typename TY, int ITER>
__global__ void __launch_bounds__(kLnThreads, ITER == 1 ? 4 : 1)
layer_norm_bwd_kernel(const TY* __restrict__ dy, const TX* __restrict__ x,
                      const float* __restrict__ gamma, const float* __restrict__ mean_in,
                      const float* __restrict__ rstd_in, TX* __restrict__ dx,
                      float* __restrict__ partial, int64_t rows, int cols) {
  __shared__ float2 scratch[kLnThreads / 32];
  float dg[ITER][8], db[ITER][8];
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
#pragma unroll
    for (int i = 0; i < 8; ++i) dg[it][i] = db[it][i] = 0.f;
  }
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float mean = mean_in[r], rstd = rstd_in[r];
    float xh[ITER][8], w[ITER][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = (it * kLnThreads + threadIdx.x) * 8;
      if (c < cols) {
        float xv[8], dv[8], gv[8];
        load8<TX>(x + r * cols + c, xv);
        load8<TY>(dy + r * cols + c, dv);
        load8<float>(gamma + c, gv);  // stays in L1: keeping it in registers costs a block of occupancy
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[it][i] = (xv[i] - mean) * rstd;
          w[it][i] = dv[i] * gv[i];
          s1 += w[it][i];
          s2 += w[it][i] * xh[it][i];
          dg[it][i] += dv[i] * xh[it][i];
          db[it][i] += dv[i];
        }
      }
    }
    const float2 t = blockSum2(s1, s2, scratch);
    const float m1 = t.x / cols, m2 = t.y / cols;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = (it * kLnThreads + threadIdx.x) * 8;
      if (c < cols) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (w[it][i] - m1 - xh[it][i] * m2);
        store8<TX>(dx + r * cols + c, o);
      }
    }
  }
  float* p = partial + (size_t)blockIdx.x * 2 * cols;
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int c = (it * kLnThreads + threadIdx.x) * 8;
    if (c < cols) {
      store8<float>(p + c, dg[it]);
      store8<float>(p + cols + c, db[it]);
    }
  }
}

// dgamma[c] = sum over blocks of partial[b][0][c]; dbeta likewise.  A block of
// 8 warps owns 32 of the 2 x cols columns: warp w sums partial rows w, w+8, ...
// (one 128-byte line per load, four loads in flight), then the warps' sums
// are added through shared memory.
__global__ void __launch_bounds__(256)
layer_norm_param_grad_kernel(const float* __restrict__ partial, int nblocks, int cols,
                             float* __restrict__ dgamma, float* __restrict__ dbeta) {
  __shared__ float acc[8][33];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  const size_t stride = (size_t)2 * cols;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (c < 2 * cols) {
    int b = w;
    for (; b + 24 < nblocks; b += 32) {
      s0 += partial[(size_t)b * stride + c];
      s1 += partial[(size_t)(b + 8) * stride + c];
      s2 += partial[(size_t)(b + 16) * stride + c];
      s3 += partial[(size_t)(b + 24) * stride + c];
    }
    for (; b < nblocks; b += 8) s0 += partial[(size_t)b * stride + c];
  }
  acc[w][lane] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (w == 0 && c < 2 * cols) {
    float s = acc[0][lane];
#pragma unroll
    for (int i = 1; i < 8; ++i) s += acc[i][lane];
    if (c < cols)
      dgamma[c] = s;
    else
      dbeta[c - cols] = s;
  }
}

// ---- residual add + LayerNorm ---------------------------------------------------
// xnew = x + branch (the fp32 residual stream plus a block's output, bf16 under
// autocast), y = LayerNorm(xnew).  A separate add reads and writes the stream
// once more per LayerNorm; here the sum is formed in the registers that the
// statistics are computed from.
template <typename TB, typename TY, int ITER>
__global__ void __launch_bounds__(kLnThreads, ITER == 1 ? 6 : 1)
add_layer_norm_fwd_kernel(const float* __restrict__ x, const TB* __restrict__ branch,
                          const float* __restrict__ gamma, const float* __restrict__ beta,
                          float* __restrict__ xnew, TY* __restrict__ y, float* __restrict__ mean_out,
                          float* __restrict__ rstd_out, int64_t rows, int cols, float eps) {
  __shared__ float2 scratch[kLnThreads / 32];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    float v[ITER][8];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = (it * kLnThreads + threadIdx.x) * 8;
      if (c < cols) {
        float b[8];
        load8<float>(x + r * cols + c, v[it]);
        load8<TB>(branch + r * cols + c, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          v[it][i] += b[i];
          s += v[it][i];
          ss += v[it][i] * v[it][i];
        }
        store8<float>(xnew + r * cols + c, v[it]);
      }
    }
    const float2 t = blockSum2(s, ss, scratch);
    const float mean = t.x / cols;
    const float var = fmaxf(t.y / cols - mean * mean, 0.f);
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
      mean_out[r] = mean;
      rstd_out[r] = rstd;
    }
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = (it * kLnThreads + threadIdx.x) * 8;
      if (c < cols) {
        float g[8], b[8], o[8];
        load8<float>(gamma + c, g);
        load8<float>(beta + c, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (v[it][i] - mean) * rstd * g[i] + b[i];
        store8<TY>(y + r * cols + c, o);
      }
    }
  }
}

// dx = LayerNorm backward of dy at xnew, plus `gres`, the gradient that reaches
// xnew along the residual path (null: none).  dx is the gradient of both
// addends; `dbranch` (null: not wanted) receives it in bf16 for a bf16 branch.
template <typename TY, int ITER>
__global__ void __launch_bounds__(kLnThreads, ITER == 1 ? 4 : 1)
add_layer_norm_bwd_kernel(const TY* __restrict__ dy, const float* __restrict__ xnew,
                          const float* __restrict__ gres, const float* __restrict__ gamma,
                          const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                          float* __restrict__ dx, __nv_bfloat16* __restrict__ dbranch,
                          float* __restrict__ partial, int64_t rows, int cols) {
  __shared__ float2 scratch[kLnThreads / 32];
  float dg[ITER][8], db[ITER][8];
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
#pragma unroll
    for (int i = 0; i < 8; ++i) dg[it][i] = db[it][i] = 0.f;
  }
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float mean = mean_in[r], rstd = rstd_in[r];
    float xh[ITER][8], w[ITER][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = (it * kLnThreads + threadIdx.x) * 8;
      if (c < cols) {
        float xv[8], dv[8], gv[8];
        load8<float>(xnew + r * cols + c, xv);
        load8<TY>(dy + r * cols + c, dv);
        load8<float>(gamma + c, gv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[it][i] = (xv[i] - mean) * rstd;
          w[it][i] = dv[i] * gv[i];
          s1 += w[it][i];
          s2 += w[it][i] * xh[it][i];
          dg[it][i] += dv[i] * xh[it][i];
          db[it][i] += dv[i];
        }
      }
    }
    const float2 t = blockSum2(s1, s2, scratch);
    const float m1 = t.x / cols, m2 = t.y / cols;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = (it * kLnThreads + threadIdx.x) * 8;
      if (c < cols) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (w[it][i] - m1 - xh[it][i] * m2);
        if (gres != nullptr) {
          float gr[8];
          load8<float>(gres + r * cols + c, gr);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += gr[i];
        }
        store8<float>(dx + r * cols + c, o);
        if (dbranch != nullptr) store8<__nv_bfloat16>(dbranch + r * cols + c, o);
      }
    }
  }
  float* p = partial + (size_t)blockIdx.x * 2 * cols;
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int c = (it * kLnThreads + threadIdx.x) * 8;
    if (c < cols) {
      store8<float>(p + c, dg[it]);
      store8<float>(p + cols + c, db[it]);
    }
  }
}

template <typename TB, typename TY>
cudaError_t addFwdDispatch(const float* x, const void* branch, const float* gamma, const float* beta,
                           float* xnew, void* y, float* mean, float* rstd, int64_t rows, int cols,
                           float eps, int blocks, cudaStream_t s) {
  const int iter = (cols / 8 + kLnThreads - 1) / kLnThreads;
#define FR_ALN_FWD(I)                                                                         \
  add_layer_norm_fwd_kernel<TB, TY, I><<<blocks, kLnThreads, 0, s>>>(                          \
      x, static_cast<const TB*>(branch), gamma, beta, xnew, static_cast<TY*>(y), mean, rstd, rows, cols, eps)
  switch (iter) {
    case 1: FR_ALN_FWD(1); break;
    case 2: FR_ALN_FWD(2); break;
    case 3: FR_ALN_FWD(3); break;
    case 4: FR_ALN_FWD(4); break;
    default: return cudaErrorInvalidValue;
  }
#undef FR_ALN_FWD
  return cudaGetLastError();
}

template <typename TY>
cudaError_t addBwdDispatch(const void* dy, const float* xnew, const float* gres, const float* gamma,
                           const float* mean, const float* rstd, float* dx, void* dbranch,
                           float* partial, int64_t rows, int cols, int blocks, cudaStream_t s) {
  const int iter = (cols / 8 + kLnThreads - 1) / kLnThreads;
#define FR_ALN_BWD(I)                                                                         \
  add_layer_norm_bwd_kernel<TY, I><<<blocks, kLnThreads, 0, s>>>(                              \
      static_cast<const TY*>(dy), xnew, gres, gamma, mean, rstd, dx,                           \
      static_cast<__nv_bfloat16*>(dbranch), partial, rows, cols)
  switch (iter) {
    case 1: FR_ALN_BWD(1); break;
    case 2: FR_ALN_BWD(2); break;
    case 3: FR_ALN_BWD(3); break;
    case 4: FR_ALN_BWD(4); break;
    default: return cudaErrorInvalidValue;
  }
#undef FR_ALN_BWD
  return cudaGetLastError();
}

template <typename TX, typename TY>
cudaError_t fwdDispatch(const void* x, const float* gamma, const float* beta, void* y, float* mean,
                        float* rstd, int64_t rows, int cols, float eps, int blocks, cudaStream_t s) {
  const int iter = (cols / 8 + kLnThreads - 1) / kLnThreads;
#define FR_LN_FWD(I)                                                                            \
  layer_norm_fwd_kernel<TX, TY, I><<<blocks, kLnThreads, 0, s>>>(                               \
      static_cast<const TX*>(x), gamma, beta, static_cast<TY*>(y), mean, rstd, rows, cols, eps)
  switch (iter) {
    case 1: FR_LN_FWD(1); break;
    case 2: FR_LN_FWD(2); break;
    case 3: FR_LN_FWD(3); break;
    case 4: FR_LN_FWD(4); break;
    default: return cudaErrorInvalidValue;
  }
#undef FR_LN_FWD
  return cudaGetLastError();
}

template <typename TX, typename TY>
cudaError_t bwdDispatch(const void* dy, const void* x, const float* gamma, const float* mean,
                        const float* rstd, void* dx, float* partial, int64_t rows, int cols,
                        int blocks, cudaStream_t s) {
  const int iter = (cols / 8 + kLnThreads - 1) / kLnThreads;
#define FR_LN_BWD(I)                                                                            \
  layer_norm_bwd_kernel<TX, TY, I><<<blocks, kLnThreads, 0, s>>>(                               \
      static_cast<const TY*>(dy), static_cast<const TX*>(x), gamma, mean, rstd,                 \
      static_cast<TX*>(dx), partial, rows, cols)
  switch (iter) {
    case 1: FR_LN_BWD(1); break;
    case 2: FR_LN_BWD(2); break;
    case 3: FR_LN_BWD(3); break;
    case 4: FR_LN_BWD(4); break;
    default: return cudaErrorInvalidValue;
  }
#undef FR_LN_BWD
  return cudaGetLastError();
}

}  // namespace

int layerNormBackwardBlocks(int64_t rows, int sm_count) {
  int64_t b = (int64_t)sm_count * 4;
  if (b > rows) b = rows;
  return (int)(b < 1 ? 1 : b);
}

cudaError_t launchLayerNormForward(const void* x, bool x_bf16, const float* gamma, const float* beta,
                                   void* y, bool y_bf16, float* mean, float* rstd, int64_t rows,
                                   int cols, float eps, int sm_count, cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  if (cols % 8 != 0 || cols > 8192) return cudaErrorInvalidValue;
  int64_t blocks = (int64_t)sm_count * 8;
  if (blocks > rows) blocks = rows;
  cudaError_t e;
  if (x_bf16)
    e = y_bf16 ? fwdDispatch<__nv_bfloat16, __nv_bfloat16>(x, gamma, beta, y, mean, rstd, rows, cols, eps, (int)blocks, stream)
               : fwdDispatch<__nv_bfloat16, float>(x, gamma, beta, y, mean, rstd, rows, cols, eps, (int)blocks, stream);
  else
    e = y_bf16 ? fwdDispatch<float, __nv_bfloat16>(x, gamma, beta, y, mean, rstd, rows, cols, eps, (int)blocks, stream)
               : fwdDispatch<float, float>(x, gamma, beta, y, mean, rstd, rows, cols, eps, (int)blocks, stream);
  noteLocalLaunch();
  return e;
}

cudaError_t launchLayerNormBackward(const void* dy, bool y_bf16, const void* x, bool x_bf16,
                                    const float* gamma, const float* mean, const float* rstd, void* dx,
                                    float* partial, float* dgamma, float* dbeta, int64_t rows, int cols,
                                    int sm_count, cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  if (cols % 8 != 0 || cols > 8192) return cudaErrorInvalidValue;
  const int blocks = layerNormBackwardBlocks(rows, sm_count);
  cudaError_t e;
  if (x_bf16)
    e = y_bf16 ? bwdDispatch<__nv_bfloat16, __nv_bfloat16>(dy, x, gamma, mean, rstd, dx, partial, rows, cols, blocks, stream)
               : bwdDispatch<__nv_bfloat16, float>(dy, x, gamma, mean, rstd, dx, partial, rows, cols, blocks, stream);
  else
    e = y_bf16 ? bwdDispatch<float, __nv_bfloat16>(dy, x, gamma, mean, rstd, dx, partial, rows, cols, blocks, stream)
               : bwdDispatch<float, float>(dy, x, gamma, mean, rstd, dx, partial, rows, cols, blocks, stream);
  if (e != cudaSuccess) return e;
  layer_norm_param_grad_kernel<<<(2 * cols + 31) / 32, 256, 0, stream>>>(partial, blocks, cols, dgamma, dbeta);
  noteLocalLaunch();
  noteLocalLaunch();
  return cudaGetLastError();
}

cudaError_t launchAddLayerNormForward(const float* x, const void* branch, bool branch_bf16,
                                      const float* gamma, const float* beta, float* xnew, void* y,
                                      bool y_bf16, float* mean, float* rstd, int64_t rows, int cols,
                                      float eps, int sm_count, cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  if (cols % 8 != 0 || cols > 8192) return cudaErrorInvalidValue;
  int64_t blocks = (int64_t)sm_count * 6;
  if (blocks > rows) blocks = rows;
  cudaError_t e;
  if (branch_bf16)
    e = y_bf16 ? addFwdDispatch<__nv_bfloat16, __nv_bfloat16>(x, branch, gamma, beta, xnew, y, mean, rstd, rows, cols, eps, (int)blocks, stream)
               : addFwdDispatch<__nv_bfloat16, float>(x, branch, gamma, beta, xnew, y, mean, rstd, rows, cols, eps, (int)blocks, stream);
  else
    e = y_bf16 ? addFwdDispatch<float, __nv_bfloat16>(x, branch, gamma, beta, xnew, y, mean, rstd, rows, cols, eps, (int)blocks, stream)
               : addFwdDispatch<float, float>(x, branch, gamma, beta, xnew, y, mean, rstd, rows, cols, eps, (int)blocks, stream);
  noteLocalLaunch();
  return e;
}

cudaError_t launchAddLayerNormBackward(const void* dy, bool y_bf16, const float* xnew, const float* gres,
                                       const float* gamma, const float* mean, const float* rstd,
                                       float* dx, void* dbranch_bf16, float* partial, float* dgamma,
                                       float* dbeta, int64_t rows, int cols, int sm_count,
                                       cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  if (cols % 8 != 0 || cols > 8192) return cudaErrorInvalidValue;
  const int blocks = layerNormBackwardBlocks(rows, sm_count);
  cudaError_t e = y_bf16 ? addBwdDispatch<__nv_bfloat16>(dy, xnew, gres, gamma, mean, rstd, dx, dbranch_bf16, partial, rows, cols, blocks, stream)
                         : addBwdDispatch<float>(dy, xnew, gres, gamma, mean, rstd, dx, dbranch_bf16, partial, rows, cols, blocks, stream);
  if (e != cudaSuccess) return e;
  layer_norm_param_grad_kernel<<<(2 * cols + 31) / 32, 256, 0, stream>>>(partial, blocks, cols, dgamma, dbeta);
  noteLocalLaunch();
  noteLocalLaunch();
  return cudaGetLastError();
}

}  // namespace fairring
