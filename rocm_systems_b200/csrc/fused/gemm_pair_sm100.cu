// Host side of the CTA-pair bf16 GEMM (gemm_pair_sm100.cuh): tensor maps for either operand major, cluster launch.
#include "gemm_pair_sm100.cuh"

#include "gemm_host.h"

namespace b200 {
namespace gemm2 {

// CTA pairs the device can hold at once (a GPC with an odd number of SMs leaves one SM out), asked once per device.
int pairsOnDevice() {
  static int pairs[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return gemm::smCount() / 2;
  if (!pairs[dev]) {
    auto kernel = gemmPairKernel<256, false, false>;
    int n = 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<256>::kSmemBytes) == cudaSuccess) {
      cudaLaunchConfig_t q{};
      q.gridDim = dim3(2 * gemm::smCount());
      q.blockDim = dim3(kThreads);
      q.dynamicSmemBytes = Cfg<256>::kSmemBytes;
      cudaLaunchAttribute at{};
      at.id = cudaLaunchAttributeClusterDimension;
      at.val.clusterDim.x = 2;
      at.val.clusterDim.y = 1;
      at.val.clusterDim.z = 1;
      q.attrs = &at;
      q.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&n, kernel, &q) != cudaSuccess) n = 0;
    }
    (void)cudaGetLastError();
    pairs[dev] = n > 0 ? n : gemm::smCount() / 2;
  }
  return pairs[dev];
}

namespace {

template <int BN, bool A_MN, bool B_MN>
cudaError_t launchPair(const Params& p, int maxCtas, cudaStream_t s) {
  auto kernel = gemmPairKernel<BN, A_MN, B_MN>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<BN>::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  int pairs = pairsOnDevice();
  if (maxCtas > 0 && maxCtas / 2 < pairs) pairs = maxCtas / 2 > 0 ? maxCtas / 2 : 1;
  const int tiles = p.tilesM * p.tilesN;
  if (tiles < pairs) pairs = tiles;
  kernel<<<2 * pairs, kThreads, Cfg<BN>::kSmemBytes, s>>>(p);  // cluster shape (2, 1, 1) is part of the kernel
  return cudaGetLastError();
}

template <int BN>
cudaError_t dispatchMajor(const Params& p, bool aMn, bool bMn, int maxCtas, cudaStream_t s) {
  if (aMn) return bMn ? launchPair<BN, true, true>(p, maxCtas, s) : launchPair<BN, true, false>(p, maxCtas, s);
  return bMn ? launchPair<BN, false, true>(p, maxCtas, s) : launchPair<BN, false, false>(p, maxCtas, s);
}

}  // namespace

// A: logical [M, K]; aMn = false: stored [M, K] with row stride lda; aMn = true: stored [K, M] with row stride lda.
// B: logical [N, K]; likewise with ldb. C [M, N] bf16 with row stride ldc.
cudaError_t gemmPairBf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, bool aMn, bool bMn, int bn, int maxCtas,
                         cudaStream_t s) {
  if (M <= 0 || N <= 0 || K <= 0) return cudaSuccess;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || (ldc & 7)) return cudaErrorInvalidValue;  // rows of C are written in 16-byte pieces
  // 256-wide tiles unless the caller says otherwise: on 128-wide ones the issuing thread's per-stage work (barrier wait,
  // descriptors, commit) is no longer hidden behind the MMAs, and the kernel ran 1.6x slower on the same problem.
  if (bn != 128 && bn != 256) bn = N > 128 ? 256 : 128;
  Params p{};
  const bool okA = aMn ? gemm::makeTileMap(&p.mapA, A, K, M, lda, 64, 2) : gemm::makeTileMap(&p.mapA, A, M, K, lda, BM, 2);
  const bool okB = bMn ? gemm::makeTileMap(&p.mapB, B, K, N, ldb, 64, 2) : gemm::makeTileMap(&p.mapB, B, N, K, ldb, bn / 2, 2);
  if (!okA || !okB) return cudaErrorInvalidValue;
  p.C = (__nv_bfloat16*)C;
  p.ldc = ldc;
  p.M = M;
  p.N = N;
  p.K = K;
  p.tilesM = (M + 2 * BM - 1) / (2 * BM);
  p.tilesN = (N + bn - 1) / bn;
  p.err = gemm::errWord();
  if (!p.err) return cudaErrorMemoryAllocation;
  return bn == 256 ? dispatchMajor<256>(p, aMn, bMn, maxCtas, s) : dispatchMajor<128>(p, aMn, bMn, maxCtas, s);
}

}  // namespace gemm2
}  // namespace b200

extern "C" {

// CTA pairs the current device runs at once (what the tile-width choice divides the tiles by).
int b200ops_gemm_pairs_on_device(void) { return b200::gemm2::pairsOnDevice(); }

// C[M, N] (bf16, ldc) = A * B^T on CTA pairs. A is logical [M, K], B logical [N, K]; aMn / bMn != 0 says the operand is
// stored with its row index contiguous ([K, M] resp. [K, N] row-major, leading dimension = the row stride of that
// storage). bn: 0 auto, 128 or 256. Errors of bounded waits are read with b200ops_gemm_take_error.
int b200ops_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int aMn, int bMn, int bn, int maxCtas,
                           cudaStream_t s) {
  return (int)b200::gemm2::gemmPairBf16(A, B, C, M, N, K, lda, ldb, ldc, aMn != 0, bMn != 0, bn, maxCtas, s);
}
}
