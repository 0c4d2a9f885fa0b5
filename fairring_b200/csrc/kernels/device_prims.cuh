// Device-side building blocks: 16-byte accesses with explicit memory
// semantics, flag signalling between GPUs with a bounded wait, element-type
// traits, and the NVLS multimem instructions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <type_traits>

#include "kernels.h"

namespace fairring {
namespace dev {

// ---- memory accesses -------------------------------------------------------
// Staging memory is written by other GPUs while a kernel runs, so it is read
// with relaxed system-scope loads (never through the non-coherent path).
__device__ __forceinline__ uint4 ldStage(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void stStage(void* p, const uint4& v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint32_t ldAcquireSys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void stReleaseSys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void stRelaxedSys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ldVolatile(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t globalTimerNs() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- bounded wait ------------------------------------------------------------
// Spins until *flag has reached `epoch` (wrap-safe).  Gives up after
// timeout_ns, after an iteration cap derived from it, or when the host raises
// the abort flag; the caller then records a status and leaves the kernel.
// Returns kStatusOk, kStatusTimeout or kStatusAborted.
__device__ __forceinline__ uint32_t waitFlag(const uint32_t* flag, uint32_t epoch,
                                             uint64_t timeout_ns,
                                             const uint32_t* abort_flag) {
  uint64_t t0 = 0;
  const uint64_t iter_cap = timeout_ns / 32 + (1ull << 20);
  for (uint64_t n = 1;; ++n) {
    uint32_t v = ldAcquireSys(flag);
    if ((int32_t)(v - epoch) >= 0) return kStatusOk;
    if ((n & 63) == 0) {
      uint64_t now = globalTimerNs();
      if (t0 == 0) t0 = now;
      if (now - t0 > timeout_ns || n > iter_cap) return kStatusTimeout;
      if ((n & 1023) == 0 && abort_flag != nullptr && ldVolatile(abort_flag) != 0)
        return kStatusAborted;
    }
  }
}

// ---- element types -------------------------------------------------------------
template <typename T> struct Tr;
template <> struct Tr<uint8_t> {
  using Acc = int32_t;
  static __device__ __forceinline__ Acc up(uint8_t x) { return x; }
  static __device__ __forceinline__ uint8_t down(Acc a) { return (uint8_t)a; }
};
template <> struct Tr<int8_t> {
  using Acc = int32_t;
  static __device__ __forceinline__ Acc up(int8_t x) { return x; }
  static __device__ __forceinline__ int8_t down(Acc a) { return (int8_t)a; }
};
template <> struct Tr<int32_t> {
  using Acc = int32_t;
  static __device__ __forceinline__ Acc up(int32_t x) { return x; }
  static __device__ __forceinline__ int32_t down(Acc a) { return a; }
};
template <> struct Tr<int64_t> {
  using Acc = int64_t;
  static __device__ __forceinline__ Acc up(int64_t x) { return x; }
  static __device__ __forceinline__ int64_t down(Acc a) { return a; }
};
template <> struct Tr<__half> {
  using Acc = float;
  static __device__ __forceinline__ Acc up(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half down(Acc a) { return __float2half_rn(a); }
};
template <> struct Tr<__nv_bfloat16> {
  using Acc = float;
  static __device__ __forceinline__ Acc up(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 down(Acc a) { return __float2bfloat16_rn(a); }
};
template <> struct Tr<float> {
  using Acc = float;
  static __device__ __forceinline__ Acc up(float x) { return x; }
  static __device__ __forceinline__ float down(Acc a) { return a; }
};
template <> struct Tr<double> {
  using Acc = double;
  static __device__ __forceinline__ Acc up(double x) { return x; }
  static __device__ __forceinline__ double down(Acc a) { return a; }
};

template <typename A>
__device__ __forceinline__ A combine(A a, A b, int op) {
  if (op == (int)RedOp::SUM) return a + b;
  if (op == (int)RedOp::MAX) return a > b ? a : b;
  return a < b ? a : b;
}

template <typename T, int V>
__device__ __forceinline__ void unpack(const uint4& u, typename Tr<T>::Acc (&a)[V]) {
  static_assert(V * sizeof(T) == 16, "one vector is 16 bytes");
  const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
  for (int i = 0; i < V; ++i) a[i] = Tr<T>::up(e[i]);
}
template <typename T, int V>
__device__ __forceinline__ uint4 pack(const typename Tr<T>::Acc (&a)[V]) {
  static_assert(V * sizeof(T) == 16, "one vector is 16 bytes");
  uint4 u;
  T* e = reinterpret_cast<T*>(&u);
#pragma unroll
  for (int i = 0; i < V; ++i) e[i] = Tr<T>::down(a[i]);
  return u;
}

// V elements of the user's tensor starting at p -> accumulator type.
// `aligned`: p is 16-byte aligned; `nvalid` (0..V): how many of them exist.
template <typename IO, int V>
__device__ __forceinline__ void loadUser(const IO* p, int nvalid, bool aligned,
                                         typename Tr<IO>::Acc (&a)[V]) {
  constexpr int NV = V * sizeof(IO) / 16;
  if (aligned && nvalid == V) {
    uint4 raw[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) raw[k] = reinterpret_cast<const uint4*>(p)[k];
    const IO* e = reinterpret_cast<const IO*>(raw);
#pragma unroll
    for (int i = 0; i < V; ++i) a[i] = Tr<IO>::up(e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) a[i] = i < nvalid ? Tr<IO>::up(p[i]) : typename Tr<IO>::Acc(0);
  }
}
template <typename IO, int V>
__device__ __forceinline__ void storeUser(IO* p, int nvalid, bool aligned,
                                          const typename Tr<IO>::Acc (&a)[V]) {
  constexpr int NV = V * sizeof(IO) / 16;
  if (aligned && nvalid == V) {
    uint4 raw[NV];
    IO* e = reinterpret_cast<IO*>(raw);
#pragma unroll
    for (int i = 0; i < V; ++i) e[i] = Tr<IO>::down(a[i]);
#pragma unroll
    for (int k = 0; k < NV; ++k) reinterpret_cast<uint4*>(p)[k] = raw[k];
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i)
      if (i < nvalid) p[i] = Tr<IO>::down(a[i]);
  }
}

// ---- NVLS (NVSwitch multicast address) -------------------------------------------
// ld_reduce: the switch fetches the word from every GPU bound to the multicast
// object and returns the reduction.  st: the switch writes to every GPU.
template <typename WIRE>
__device__ __forceinline__ uint4 multimemLdReduce(const void* mc, int op) {
  uint4 v = make_uint4(0, 0, 0, 0);
  if constexpr (sizeof(WIRE) == 4) {  // float, SUM only
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
  } else if constexpr (sizeof(WIRE) == 2) {
    constexpr bool kBf16 = std::is_same<WIRE, __nv_bfloat16>::value;
    if (op == (int)RedOp::SUM) {
      if constexpr (kBf16)
        asm volatile(
            "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
            : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
            : "l"(mc)
            : "memory");
      else
        asm volatile(
            "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
            : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
            : "l"(mc)
            : "memory");
    } else if (op == (int)RedOp::MAX) {
      if constexpr (kBf16)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.max.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "l"(mc)
                     : "memory");
      else
        asm volatile("multimem.ld_reduce.relaxed.sys.global.max.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "l"(mc)
                     : "memory");
    } else {
      if constexpr (kBf16)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.min.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "l"(mc)
                     : "memory");
      else
        asm volatile("multimem.ld_reduce.relaxed.sys.global.min.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "l"(mc)
                     : "memory");
    }
  }
  return v;
}
__device__ __forceinline__ void multimemSt(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc),
               "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

}  // namespace dev
}  // namespace fairring
