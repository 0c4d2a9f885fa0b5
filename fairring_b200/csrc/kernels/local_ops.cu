// Single-GPU fused ops used by the training drivers around the collectives:
// a flat AdamW step over one contiguous fp32 parameter buffer (one launch for
// the whole model instead of one per tensor) and a sum of squares for gradient
// clipping.  Both are bandwidth-bound streaming kernels: 16-byte accesses,
// grid-stride, one pass over the data.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "local_kernels.h"

namespace fairring {
namespace {

std::atomic<uint64_t> g_local_launches{0};

__global__ void __launch_bounds__(512)
adamw_flat_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                  float* __restrict__ v, int64_t n, AdamWArgs a) {
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
  }
  // ragged tail (n not a multiple of 4)
  const int64_t tail = n4 * 4 + blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (tail < n) upd(p[tail], g[tail], m[tail], v[tail]);
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

cudaError_t launchAdamWFlat(float* p, const float* g, float* m, float* v, int64_t n,
                            const AdamWArgs& a, int sm_count, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  if (((uintptr_t)p | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15u) return cudaErrorMisalignedAddress;
  int64_t blocks = (n / 4 + 511) / 512;
  const int64_t cap = (int64_t)sm_count * 4;  // 4 resident CTAs of 512 threads per SM
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  adamw_flat_kernel<<<(unsigned)blocks, 512, 0, stream>>>(p, g, m, v, n, a);
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

uint64_t localLaunchCountImpl() { return g_local_launches.load(std::memory_order_relaxed); }

}  // namespace fairring
