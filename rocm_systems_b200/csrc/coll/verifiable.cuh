// Verifiable data for collectives: inputs whose reduction is exactly predictable, the matching
// expected outputs, and a bitwise checker — for every element type and reduction operator.
//
// The idea is that of the rccl-tests oracle (rccl-tests/verifiable/verifiable.h:16-34,
// verifiable.cpp:665-1019): every value is a pure function of (seed, element index, rank), and
// floating-point inputs are built so that the reduction has no rounding in any order, so results
// can be compared bit for bit without running a reference reduction. The construction here is this
// project's own: per element one shared power-of-two scale and small integer mantissas whose sum
// over all ranks stays inside the type's significand; products use powers of two; Min/Max use
// arbitrary finite values; Avg is checked with a ULP tolerance because 1/n is not exact.
// All generators are __host__ __device__, so the CPU oracle and the GPU kernels are the same code.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace b200 {
namespace ver {

enum Op : int { OP_SUM = 0, OP_PROD = 1, OP_MAX = 2, OP_MIN = 3, OP_AVG = 4, OP_MULSUM = 5, OP_NONE = 6 };

__host__ __device__ inline uint64_t mix(uint64_t x) {
  x ^= x >> 31;
  x *= 0x9fb21c651e98df25ull;
  x ^= x >> 29;
  x *= 0xd6e8feb86659fd93ull;
  x ^= x >> 32;
  return x;
}
__host__ __device__ inline uint64_t hash3(uint64_t seed, uint64_t index, uint64_t rank) {
  return mix(mix(seed * 0x2545f4914f6cdd1dull + index) ^ (rank + 1) * 0x9e3779b97f4a7c15ull);
}

// Significand bits usable for exact integer sums, and a safe exponent window, per float type.
template <typename T> struct FloatInfo;
template <> struct FloatInfo<float> { static constexpr int sig = 24, emin = -20, emax = 20; };
template <> struct FloatInfo<double> { static constexpr int sig = 53, emin = -40, emax = 40; };
template <> struct FloatInfo<__half> { static constexpr int sig = 11, emin = -6, emax = 4; };
template <> struct FloatInfo<__nv_bfloat16> { static constexpr int sig = 8, emin = -20, emax = 20; };
template <> struct FloatInfo<__nv_fp8_e4m3> { static constexpr int sig = 4, emin = -3, emax = 3; };
template <> struct FloatInfo<__nv_fp8_e5m2> { static constexpr int sig = 3, emin = -6, emax = 6; };

template <typename T> struct IsFloat { static constexpr bool v = false; };
template <> struct IsFloat<float> { static constexpr bool v = true; };
template <> struct IsFloat<double> { static constexpr bool v = true; };
template <> struct IsFloat<__half> { static constexpr bool v = true; };
template <> struct IsFloat<__nv_bfloat16> { static constexpr bool v = true; };
template <> struct IsFloat<__nv_fp8_e4m3> { static constexpr bool v = true; };
template <> struct IsFloat<__nv_fp8_e5m2> { static constexpr bool v = true; };

template <typename T> __host__ __device__ inline T fromDouble(double v) { return (T)v; }
template <> __host__ __device__ inline __half fromDouble<__half>(double v) { return __float2half_rn((float)v); }
template <> __host__ __device__ inline __nv_bfloat16 fromDouble<__nv_bfloat16>(double v) { return __float2bfloat16_rn((float)v); }
template <> __host__ __device__ inline __nv_fp8_e4m3 fromDouble<__nv_fp8_e4m3>(double v) { return __nv_fp8_e4m3((float)v); }
template <> __host__ __device__ inline __nv_fp8_e5m2 fromDouble<__nv_fp8_e5m2>(double v) { return __nv_fp8_e5m2((float)v); }
template <typename T> __host__ __device__ inline double toDouble(T v) { return (double)v; }
template <> __host__ __device__ inline double toDouble<__half>(__half v) { return (double)__half2float(v); }
template <> __host__ __device__ inline double toDouble<__nv_bfloat16>(__nv_bfloat16 v) { return (double)__bfloat162float(v); }
template <> __host__ __device__ inline double toDouble<__nv_fp8_e4m3>(__nv_fp8_e4m3 v) { return (double)float(v); }
template <> __host__ __device__ inline double toDouble<__nv_fp8_e5m2>(__nv_fp8_e5m2 v) { return (double)float(v); }

__host__ __device__ inline double pow2i(int e) { return ldexp(1.0, e); }

// The PreMulSum scalar of a rank: 1 on even ranks, 2 on odd ranks (rccl-tests/verifiable/verifiable.h:38-43).
__host__ __device__ inline double mulsumScalar(int rank) { return (rank & 1) ? 2.0 : 1.0; }

// ---- one input element as a double that is exactly representable in T -------------------------------
template <typename T>
__host__ __device__ inline double genInputF(int op, uint64_t seed, uint64_t index, int rank, int nranks) {
  using I = FloatInfo<T>;
  const uint64_t hIdx = mix(seed ^ (index * 0x9e3779b97f4a7c15ull));  // shared by all ranks of this element
  const uint64_t h = hash3(seed, index, (uint64_t)rank);
  if (op == OP_NONE) {  // non-reducing collectives: any exactly representable value
    const int e = I::emin + (int)(hIdx % (uint64_t)(I::emax - I::emin + 1));
    const int64_t m = (int64_t)(h % (1ull << (I::sig - 1))) + 1;
    return ((h >> 40) & 1 ? -1.0 : 1.0) * (double)m * pow2i(e - (I::sig - 1));
  }
  if (op == OP_PROD) {
    // Powers of two whose exponents sum to something representable; rank 0 carries a mantissa.
    const int span = (I::emax - I::emin) / (2 * (nranks > 1 ? nranks : 1));
    const int e = span > 0 ? (int)(h % (uint64_t)(2 * span + 1)) - span : 0;
    double v = pow2i(e);
    if (rank == 0) v *= 1.0 + (double)(hIdx % (1ull << (I::sig - 1))) / (double)(1ull << (I::sig - 1));
    return (h >> 50) & 1 ? -v : v;
  }
  if (op == OP_MAX || op == OP_MIN) {
    const int e = I::emin + (int)(h % (uint64_t)(I::emax - I::emin + 1));
    const int64_t m = (int64_t)((h >> 8) % (1ull << (I::sig - 1))) + (1ll << (I::sig - 1));
    return ((h >> 44) & 1 ? -1.0 : 1.0) * (double)m * pow2i(e - (I::sig - 1));
  }
  // Sum / Avg / MulSum: integer mantissas on a shared scale. Budget: |sum| < 2^(sig-1), with the
  // MulSum scalar (at most 2) taken into account.
  // Every integer up to 2^sig is representable, so partial sums stay exact while the total of
  // |scalar * mantissa| over the ranks stays within that. Types too narrow to give every rank a
  // non-zero mantissa (fp8 with 8 ranks) let only some ranks contribute, rotating with the index.
  const int64_t cap = 1ll << I::sig;
  const int64_t scal = op == OP_MULSUM ? 2 : 1;
  const int nr = nranks > 0 ? nranks : 1;
  int64_t maxAbs = cap / (nr * scal);
  int active = nr;
  if (maxAbs < 1) {
    maxAbs = 1;
    active = (int)(cap / scal);
    if (active < 1) active = 1;
  }
  int64_t m = (int64_t)(h % (uint64_t)(2 * maxAbs + 1)) - maxAbs;
  if ((int)(((uint64_t)rank + hIdx) % (uint64_t)nr) >= active) m = 0;
  if (op == OP_AVG) m = m < 0 ? -m : m;  // same sign keeps the average away from cancellation
  const int e = I::emin / 2 + (int)(hIdx % (uint64_t)(I::emax / 2 - I::emin / 2 + 1));
  return (double)m * pow2i(e);
}

template <typename T>
__host__ __device__ inline T genInput(int op, uint64_t seed, uint64_t index, int rank, int nranks) {
  if constexpr (IsFloat<T>::v) {
    return fromDouble<T>(genInputF<T>(op, seed, index, rank, nranks));
  } else {
    uint64_t h = hash3(seed, index, (uint64_t)rank);
    if (op == OP_PROD) h |= 1;  // never zero, so a product keeps information
    return (T)h;                 // integer arithmetic wraps, which is exact
  }
}

// ---- expected output element -------------------------------------------------------------------------------
template <typename T>
__host__ __device__ inline T genExpected(int op, uint64_t seed, uint64_t index, int nranks) {
  if constexpr (IsFloat<T>::v) {
    double acc = 0;
    for (int r = 0; r < nranks; r++) {
      double v = genInputF<T>(op, seed, index, r, nranks);
      if (op == OP_MULSUM) v *= mulsumScalar(r);
      if (r == 0) acc = v;
      else if (op == OP_PROD) acc *= v;
      else if (op == OP_MAX) acc = v > acc ? v : acc;
      else if (op == OP_MIN) acc = v < acc ? v : acc;
      else acc += v;
    }
    if (op == OP_AVG) acc = acc / (double)nranks;
    return fromDouble<T>(acc);
  } else {
    T acc = 0;
    for (int r = 0; r < nranks; r++) {
      T v = genInput<T>(op, seed, index, r, nranks);
      if (op == OP_MULSUM) v = (T)(v * (T)mulsumScalar(r));
      if (r == 0) acc = v;
      else if (op == OP_PROD) acc = (T)(acc * v);
      else if (op == OP_MAX) acc = v > acc ? v : acc;
      else if (op == OP_MIN) acc = v < acc ? v : acc;
      else acc = (T)(acc + v);
    }
    if (op == OP_AVG) acc = (T)(acc / (T)nranks);
    return acc;
  }
}

// ---- kernels (launch shape of the reference: at most 32 blocks of 512 threads, verifiable.cpp:1055-1086) ----
template <typename T>
__global__ void kPrepareInput(T* buf, size_t count, size_t index0, int op, uint64_t seed, int rank, int nranks) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
    buf[i] = genInput<T>(op, seed, index0 + i, rank, nranks);
}
template <typename T>
__global__ void kPrepareExpected(T* buf, size_t count, size_t index0, int op, uint64_t seed, int nranks) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
    buf[i] = genExpected<T>(op, seed, index0 + i, nranks);
}
// Bit patterns compared as unsigned integers of the element width; `tolUlp` > 0 only for float Avg.
template <typename T, typename U>
__global__ void kVerify(const T* got, const T* want, size_t count, unsigned tolUlp, unsigned long long* mismatches) {
  unsigned long long bad = 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
    const U a = reinterpret_cast<const U*>(got)[i], b = reinterpret_cast<const U*>(want)[i];
    if (a == b) continue;
    if (tolUlp) {
      const U d = a > b ? a - b : b - a;
      if (d <= (U)tolUlp) continue;
    }
    bad++;
  }
  if (bad) atomicAdd(mismatches, bad);
}

inline int blocksFor(size_t count) {
  size_t b = (count + 2047) / 2048;
  return (int)(b < 1 ? 1 : (b > 32 ? 32 : b));
}

// ULP allowance for Avg, growing slowly with the rank count like the reference's
// calcSumFloatTolerance (verifiable.cpp:1249-1283).
inline unsigned avgToleranceUlp(int elemBytes, int nranks) {
  const double n = nranks;
  if (elemBytes >= 4) return (unsigned)(1 + 1.25 * pow(n, 0.51));
  if (elemBytes == 2) return (unsigned)(1 + 0.75 * pow(n, 0.91));
  return (unsigned)(1 + 0.66 * pow(n, 0.91));
}

// Dispatch on the NCCL datatype code (0 int8 … 11 fp8 e5m2). Returns false for an unknown type.
template <typename F> inline bool dispatchType(int dt, F&& f) {
  switch (dt) {
    case 0: f((int8_t)0, (uint8_t)0); return true;
    case 1: f((uint8_t)0, (uint8_t)0); return true;
    case 2: f((int32_t)0, (uint32_t)0); return true;
    case 3: f((uint32_t)0, (uint32_t)0); return true;
    case 4: f((int64_t)0, (uint64_t)0); return true;
    case 5: f((uint64_t)0, (uint64_t)0); return true;
    case 6: f(__half(), (uint16_t)0); return true;
    case 7: f((float)0, (uint32_t)0); return true;
    case 8: f((double)0, (uint64_t)0); return true;
    case 9: f(__nv_bfloat16(), (uint16_t)0); return true;
    case 10: f(__nv_fp8_e4m3(), (uint8_t)0); return true;
    case 11: f(__nv_fp8_e5m2(), (uint8_t)0); return true;
    default: return false;
  }
}

inline cudaError_t prepareInput(void* buf, size_t count, size_t index0, int dt, int op, uint64_t seed, int rank, int nranks, cudaStream_t s) {
  if (count == 0) return cudaSuccess;
  bool ok = dispatchType(dt, [&](auto t, auto) {
    using T = decltype(t);
    kPrepareInput<T><<<blocksFor(count), 512, 0, s>>>((T*)buf, count, index0, op, seed, rank, nranks);
  });
  return ok ? cudaGetLastError() : cudaErrorInvalidValue;
}
inline cudaError_t prepareExpected(void* buf, size_t count, size_t index0, int dt, int op, uint64_t seed, int nranks, cudaStream_t s) {
  if (count == 0) return cudaSuccess;
  bool ok = dispatchType(dt, [&](auto t, auto) {
    using T = decltype(t);
    kPrepareExpected<T><<<blocksFor(count), 512, 0, s>>>((T*)buf, count, index0, op, seed, nranks);
  });
  return ok ? cudaGetLastError() : cudaErrorInvalidValue;
}
// `mismatches` must be device-accessible (device or mapped host memory) and is added to.
inline cudaError_t verify(const void* got, const void* want, size_t count, int dt, int op, int nranks, unsigned long long* mismatches, cudaStream_t s) {
  if (count == 0) return cudaSuccess;
  bool ok = dispatchType(dt, [&](auto t, auto u) {
    using T = decltype(t);
    using U = decltype(u);
    const unsigned tol = (IsFloat<T>::v && op == OP_AVG) ? avgToleranceUlp((int)sizeof(T), nranks) : 0u;
    kVerify<T, U><<<blocksFor(count), 512, 0, s>>>((const T*)got, (const T*)want, count, tol, mismatches);
  });
  return ok ? cudaGetLastError() : cudaErrorInvalidValue;
}

}  // namespace ver
}  // namespace b200
