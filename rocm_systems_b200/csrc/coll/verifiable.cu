// Library face of the verifiable oracle: device generators/checker for tools that link the
// library, and a host-only self-check of the "exact in any order" property.
#include "verifiable.cuh"

#include <vector>

using namespace b200::ver;

extern "C" {

int b200verPrepareInput(void* buf, size_t count, size_t index0, int dtype, int op, unsigned long long seed, int rank, int nranks, cudaStream_t s) {
  return (int)prepareInput(buf, count, index0, dtype, op, seed, rank, nranks, s);
}
int b200verPrepareExpected(void* buf, size_t count, size_t index0, int dtype, int op, unsigned long long seed, int nranks, cudaStream_t s) {
  return (int)prepareExpected(buf, count, index0, dtype, op, seed, nranks, s);
}
int b200verVerify(const void* got, const void* want, size_t count, int dtype, int op, int nranks, unsigned long long* mismatchesDev, cudaStream_t s) {
  return (int)verify(got, want, count, dtype, op, nranks, mismatchesDev, s);
}

// CPU only: generate every rank's inputs for `count` elements, reduce them IN THE ELEMENT TYPE
// (rounding after every step) in forward and in reverse rank order, and compare both with the
// closed-form expected value. Returns the number of elements where any of the three differ
// (Avg: beyond its ULP allowance). 0 means the construction is order-independent and exact.
long long b200verHostSelfCheck(int dtype, int op, int nranks, size_t count, unsigned long long seed) {
  long long bad = 0;
  bool ok = dispatchType(dtype, [&](auto t, auto u) {
    using T = decltype(t);
    using U = decltype(u);
    const unsigned tol = (IsFloat<T>::v && op == OP_AVG) ? avgToleranceUlp((int)sizeof(T), nranks) : 0u;
    for (size_t i = 0; i < count; i++) {
      T want = genExpected<T>(op, seed, i, nranks);
      T res[2];
      for (int dir = 0; dir < 2; dir++) {
        T acc{};
        for (int k = 0; k < nranks; k++) {
          const int r = dir ? nranks - 1 - k : k;
          T v = genInput<T>(op, seed, i, r, nranks);
          if constexpr (IsFloat<T>::v) {
            double x = toDouble(v);
            if (op == OP_MULSUM) x = toDouble(fromDouble<T>(x * mulsumScalar(r)));
            double a = toDouble(acc);
            if (k == 0) a = x;
            else if (op == OP_PROD) a = a * x;
            else if (op == OP_MAX) a = x > a ? x : a;
            else if (op == OP_MIN) a = x < a ? x : a;
            else a = a + x;
            acc = fromDouble<T>(a);
          } else {
            if (op == OP_MULSUM) v = (T)(v * (T)mulsumScalar(r));
            if (k == 0) acc = v;
            else if (op == OP_PROD) acc = (T)(acc * v);
            else if (op == OP_MAX) acc = v > acc ? v : acc;
            else if (op == OP_MIN) acc = v < acc ? v : acc;
            else acc = (T)(acc + v);
          }
        }
        if (op == OP_AVG) {
          if constexpr (IsFloat<T>::v) acc = fromDouble<T>(toDouble(acc) / (double)nranks);
          else acc = (T)(acc / (T)nranks);
        }
        res[dir] = acc;
      }
      for (int dir = 0; dir < 2; dir++) {
        U a, b;
        memcpy(&a, &res[dir], sizeof(U));
        memcpy(&b, &want, sizeof(U));
        const U d = a > b ? a - b : b - a;
        if (d > (U)tol) { bad++; break; }
      }
    }
  });
  return ok ? bad : -1;
}

}  // extern "C"
