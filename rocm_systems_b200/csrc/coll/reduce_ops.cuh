// Element types and reduction operators of the collective kernels.
//
// Twelve element types (rccl.h:416-455) and Sum/Prod/Max/Min with two scale modes: Avg is Sum
// followed by a division by the rank count, PreMulSum (rccl.h:489-516) multiplies every input
// by a scalar before the sum. 16- and 8-bit floats accumulate in fp32 across all ranks and are
// rounded once.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "device.h"

namespace b200 {

template <typename T> struct ElemTraits {
  using Acc = T;
  static __device__ __forceinline__ Acc up(T v) { return v; }
  static __device__ __forceinline__ T down(Acc v) { return v; }
  static constexpr bool isFloat = false;
};
template <> struct ElemTraits<float> {
  using Acc = float;
  static __device__ __forceinline__ Acc up(float v) { return v; }
  static __device__ __forceinline__ float down(Acc v) { return v; }
  static constexpr bool isFloat = true;
};
template <> struct ElemTraits<double> {
  using Acc = double;
  static __device__ __forceinline__ Acc up(double v) { return v; }
  static __device__ __forceinline__ double down(Acc v) { return v; }
  static constexpr bool isFloat = true;
};
template <> struct ElemTraits<__half> {
  using Acc = float;
  static __device__ __forceinline__ Acc up(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half down(Acc v) { return __float2half_rn(v); }
  static constexpr bool isFloat = true;
};
template <> struct ElemTraits<__nv_bfloat16> {
  using Acc = float;
  static __device__ __forceinline__ Acc up(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 down(Acc v) { return __float2bfloat16_rn(v); }
  static constexpr bool isFloat = true;
};
template <> struct ElemTraits<__nv_fp8_e4m3> {
  using Acc = float;
  static __device__ __forceinline__ Acc up(__nv_fp8_e4m3 v) { return float(v); }
  static __device__ __forceinline__ __nv_fp8_e4m3 down(Acc v) { return __nv_fp8_e4m3(v); }
  static constexpr bool isFloat = true;
};
template <> struct ElemTraits<__nv_fp8_e5m2> {
  using Acc = float;
  static __device__ __forceinline__ Acc up(__nv_fp8_e5m2 v) { return float(v); }
  static __device__ __forceinline__ __nv_fp8_e5m2 down(Acc v) { return __nv_fp8_e5m2(v); }
  static constexpr bool isFloat = true;
};

struct OpSum  { template <typename A> static __device__ __forceinline__ A apply(A a, A b) { return a + b; } };
struct OpProd { template <typename A> static __device__ __forceinline__ A apply(A a, A b) { return a * b; } };
struct OpMax  { template <typename A> static __device__ __forceinline__ A apply(A a, A b) { return a > b ? a : b; } };
struct OpMin  { template <typename A> static __device__ __forceinline__ A apply(A a, A b) { return a < b ? a : b; } };

// 16 bytes of elements viewed as accumulators.
template <typename T> struct Pack {
  static constexpr int N = 16 / sizeof(T);
  using Acc = typename ElemTraits<T>::Acc;
  union U { uint4 v; T e[N]; __device__ U() {} };
  static __device__ __forceinline__ void up(const uint4& v, Acc (&a)[N]) {
    U u; u.v = v;
#pragma unroll
    for (int i = 0; i < N; i++) a[i] = ElemTraits<T>::up(u.e[i]);
  }
  static __device__ __forceinline__ uint4 down(const Acc (&a)[N]) {
    U u;
#pragma unroll
    for (int i = 0; i < N; i++) u.e[i] = ElemTraits<T>::down(a[i]);
    return u.v;
  }
};

template <typename T>
__device__ __forceinline__ typename ElemTraits<T>::Acc scalarFromBits(unsigned long long bits) {
  union { unsigned long long b; T t; } u;
  u.b = bits;
  return ElemTraits<T>::up(u.t);
}

// The PreMulSum scalar of a call: an immediate captured when the operator was made, or a device word read now, by the
// kernel, so that the host neither waits for the stream nor reads the value earlier than stream order says.
template <typename T>
__device__ __forceinline__ typename ElemTraits<T>::Acc scalarOf(unsigned long long bits, const void* devPtr) {
  if (devPtr != nullptr) return ElemTraits<T>::up(*(const volatile T*)devPtr);
  return scalarFromBits<T>(bits);
}

template <typename T>
__device__ __forceinline__ typename ElemTraits<T>::Acc postDiv(typename ElemTraits<T>::Acc a, int n) {
  using Acc = typename ElemTraits<T>::Acc;
  if constexpr (ElemTraits<T>::isFloat) return a * (Acc(1) / Acc(n));
  else return (Acc)(a / (Acc)n);
}

}  // namespace b200
