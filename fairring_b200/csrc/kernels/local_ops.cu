// Single-GPU fused ops used by the training drivers around the collectives:
// a flat AdamW step over one contiguous fp32 parameter buffer (one launch for
// the whole model instead of one per tensor) and a sum of squares for gradient
// clipping.  Both are bandwidth-bound streaming kernels: 16-byte accesses,
// grid-stride, one pass over the data.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "local_kernels.h"

namespace fairring {
namespace {

std::atomic<uint64_t> g_local_launches{0};

template <bool kShadow>
__global__ void __launch_bounds__(512)
adamw_flat_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                  float* __restrict__ v, __nv_bfloat16* __restrict__ shadow, int64_t n,
                  AdamWArgs a) {
  const int64_t n4 = n / 4;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  float4* p4 = reinterpret_cast<float4*>(p);
  float4* m4 = reinterpret_cast<float4*>(m);
  float4* v4 = reinterpret_cast<float4*>(v);
  const float decay = 1.0f - a.lr * a.weight_decay;
  auto upd = [&](float& pp, float gg, float& mm, float& vv) {
    gg *= a.grad_scale;
    mm = a.beta1 * mm + (1.0f - a.beta1) * gg;
    vv = a.beta2 * vv + (1.0f - a.beta2) * gg * gg;
    const float denom = sqrtf(vv) * a.inv_sqrt_bias2 + a.eps;
    pp = pp * decay - a.step_size * (mm / denom);
  };
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4;
       i += (int64_t)gridDim.x * blockDim.x) {
    float4 pp = p4[i], gg = g4[i], mm = m4[i], vv = v4[i];
    upd(pp.x, gg.x, mm.x, vv.x);
    upd(pp.y, gg.y, mm.y, vv.y);
    upd(pp.z, gg.z, mm.z, vv.z);
    upd(pp.w, gg.w, mm.w, vv.w);
    p4[i] = pp;
    m4[i] = mm;
    v4[i] = vv;
    if constexpr (kShadow) {
      // bf16 copy of the new weights, for the layers that compute in bf16
      __nv_bfloat162 lo = __floats2bfloat162_rn(pp.x, pp.y), hi = __floats2bfloat162_rn(pp.z, pp.w);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(shadow)[i] = packed;
    }
  }
  // ragged tail (n not a multiple of 4)
  const int64_t tail = n4 * 4 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (tail < n) {
    upd(p[tail], g[tail], m[tail], v[tail]);
    if constexpr (kShadow) shadow[tail] = __float2bfloat16_rn(p[tail]);
  }
}

// dst (fp32) = or += src (bf16): how bf16 weight gradients enter the flat fp32
// gradient buffer.  8 elements per thread and step: one 16-byte load, two
// 16-byte stores.
__global__ void __launch_bounds__(512)
bf16_grad_to_f32_kernel(float* __restrict__ dst, const __nv_bfloat16* __restrict__ src, int64_t n,
                        int accumulate) {
  const int64_t n8 = n / 8;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n8;
       i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 raw = reinterpret_cast<const uint4*>(src)[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float4 a, b;
    float2 f0 = __bfloat1622float2(h[0]), f1 = __bfloat1622float2(h[1]);
    float2 f2 = __bfloat1622float2(h[2]), f3 = __bfloat1622float2(h[3]);
    a = make_float4(f0.x, f0.y, f1.x, f1.y);
    b = make_float4(f2.x, f2.y, f3.x, f3.y);
    float4* d = reinterpret_cast<float4*>(dst) + 2 * i;
    if (accumulate) {
      const float4 o0 = d[0], o1 = d[1];
      a.x += o0.x; a.y += o0.y; a.z += o0.z; a.w += o0.w;
      b.x += o1.x; b.y += o1.y; b.z += o1.z; b.w += o1.w;
    }
    d[0] = a;
    d[1] = b;
  }
  const int64_t tail = n8 * 8 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (tail < n) {
    const float x = __bfloat162float(src[tail]);
    dst[tail] = accumulate ? dst[tail] + x : x;
  }
}

// Plain device-to-device copy, 4 x 16 bytes in flight per thread.  Used to move
// a big ordinary tensor into and out of a symmetric bounce buffer on the
// collective's own stream (a cudaMemcpyAsync costs ~7 us of host time per call
// and measured 0.9 TB/s here).
__global__ void __launch_bounds__(512)
copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, int64_t n16,
            unsigned char* __restrict__ dst_tail, const unsigned char* __restrict__ src_tail,
            int tail_bytes) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n16; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    dst[i] = a;
    dst[i + stride] = b;
    dst[i + 2 * stride] = c;
    dst[i + 3 * stride] = d;
  }
  for (; i < n16; i += stride) dst[i] = src[i];
  if (blockIdx.x == 0 && (int)threadIdx.x < tail_bytes) dst_tail[threadIdx.x] = src_tail[threadIdx.x];
}

__global__ void __launch_bounds__(512)
sumsq_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ out) {
  const int64_t n4 = n / 4;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  float acc = 0.f;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4;
       i += (int64_t)gridDim.x * blockDim.x) {
    float4 t = x4[i];
    acc += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
  }
  const int64_t tail = n4 * 4 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (tail < n) acc += x[tail] * x[tail];
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float warp_sums[16];
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float s = threadIdx.x < (blockDim.x >> 5) ? warp_sums[threadIdx.x] : 0.f;
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) atomicAdd(out, s);
  }
}

}  // namespace

cudaError_t launchAdamWFlat(float* p, const float* g, float* m, float* v, void* shadow_bf16,
                            int64_t n, const AdamWArgs& a, int sm_count, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  if (((uintptr_t)p | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15u) return cudaErrorMisalignedAddress;
  if (((uintptr_t)shadow_bf16) & 7u) return cudaErrorMisalignedAddress;
  int64_t blocks = (n / 4 + 511) / 512;
  const int64_t cap = (int64_t)sm_count * 4;  // 4 resident CTAs of 512 threads per SM
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (shadow_bf16 != nullptr)
    adamw_flat_kernel<true><<<(unsigned)blocks, 512, 0, stream>>>(
        p, g, m, v, static_cast<__nv_bfloat16*>(shadow_bf16), n, a);
  else
    adamw_flat_kernel<false><<<(unsigned)blocks, 512, 0, stream>>>(p, g, m, v, nullptr, n, a);
  g_local_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

cudaError_t launchSumSq(const float* x, int64_t n, float* out, int sm_count, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  if (((uintptr_t)x) & 15u) return cudaErrorMisalignedAddress;
  int64_t blocks = (n / 4 + 511) / 512;
  const int64_t cap = (int64_t)sm_count * 4;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  sumsq_kernel<<<(unsigned)blocks, 512, 0, stream>>>(x, n, out);
  g_local_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

cudaError_t launchBf16GradToF32(float* dst, const void* src_bf16, int64_t n, bool accumulate,
                                int sm_count, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  if ((((uintptr_t)dst) & 15u) || (((uintptr_t)src_bf16) & 15u)) return cudaErrorMisalignedAddress;
  int64_t blocks = (n / 8 + 511) / 512;
  const int64_t cap = (int64_t)sm_count * 4;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  bf16_grad_to_f32_kernel<<<(unsigned)blocks, 512, 0, stream>>>(
      dst, static_cast<const __nv_bfloat16*>(src_bf16), n, accumulate ? 1 : 0);
  g_local_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

cudaError_t launchCopy(void* dst, const void* src, size_t bytes, int blocks, cudaStream_t stream) {
  if (bytes == 0) return cudaSuccess;
  if ((((uintptr_t)dst) | ((uintptr_t)src)) & 15u)
    return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream);
  const int64_t n16 = (int64_t)(bytes / 16);
  const int tail = (int)(bytes % 16);
  int64_t want = (n16 + 4 * 512 - 1) / (4 * 512);
  if (want < 1) want = 1;
  if (want < blocks) blocks = (int)want;
  copy_kernel<<<(unsigned)blocks, 512, 0, stream>>>(
      static_cast<uint4*>(dst), static_cast<const uint4*>(src), n16,
      static_cast<unsigned char*>(dst) + n16 * 16, static_cast<const unsigned char*>(src) + n16 * 16,
      tail);
  g_local_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError();
}

uint64_t localLaunchCountImpl() { return g_local_launches.load(std::memory_order_relaxed); }
void noteLocalLaunch() { g_local_launches.fetch_add(1, std::memory_order_relaxed); }

}  // namespace fairring
