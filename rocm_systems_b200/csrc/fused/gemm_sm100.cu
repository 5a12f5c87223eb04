// Host side of the tcgen05 GEMM: tensor-map encoding, launch, error read-back.
#include "gemm_sm100.cuh"

#include <mutex>

#include "../core/cudrv.h"
#include "gemm_host.h"

namespace b200 {
namespace gemm {

// [rows, cols] bf16 row-major with leading dimension `ld` (elements): box of `boxRows` rows by
// 64 columns, 128-byte swizzle, out-of-range reads return zeros.
bool makeTileMap(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t boxRows, uint32_t elemBytes) {
  const CuDrv& d = CuDrv::get();
  if (!d.cuTensorMapEncodeTiled) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * elemBytes) & 15)) return false;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * elemBytes};
  cuuint32_t box[2] = {128u / elemBytes, boxRows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elemBytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = d.cuTensorMapEncodeTiled(map, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

static std::mutex gErrMu;
static int* gErrWord[64] = {};

int* errWord() {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(gErrMu);
  if (dev < 0 || dev >= 64) return nullptr;
  if (!gErrWord[dev]) {
    if (cudaMalloc(&gErrWord[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(gErrWord[dev], 0, sizeof(int));
  }
  return gErrWord[dev];
}

int smCount() {
  static int n[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!n[dev]) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev] ? n[dev] : 148;
}

template <int BN>
cudaError_t launch(const Params& p, const PlainPolicy<BN>& pol, int ctas, cudaStream_t s) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemmKernel<BN, PlainPolicy<BN>>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<BN>::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  gemmKernel<BN, PlainPolicy<BN>><<<ctas, kThreads, Cfg<BN>::kSmemBytes, s>>>(p, pol);
  return cudaGetLastError();
}

cudaError_t gemmBf16TN(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int bn, int maxCtas, cudaStream_t s) {
  if (M <= 0 || N <= 0 || K <= 0) return cudaSuccess;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || (ldc & 7)) return cudaErrorInvalidValue;  // rows of C are written in 16-byte pieces
  if (bn != 128 && bn != 256) bn = N >= 256 ? 256 : 128;
  Params p{};
  if (!makeTileMap(&p.mapA, A, M, K, lda, BM, 2) || !makeTileMap(&p.mapB, B, N, K, ldb, bn, 2)) return cudaErrorInvalidValue;
  p.M = M;
  p.N = N;
  p.K = K;
  p.tilesM = (M + BM - 1) / BM;
  p.tilesN = (N + bn - 1) / bn;
  p.err = errWord();
  if (!p.err) return cudaErrorMemoryAllocation;
  int ctas = smCount();
  if (maxCtas > 0 && maxCtas < ctas) ctas = maxCtas;
  const int tiles = p.tilesM * p.tilesN;
  if (tiles < ctas) ctas = tiles;
  if (bn == 256) return launch<256>(p, PlainPolicy<256>{(__nv_bfloat16*)C, ldc, N, M}, ctas, s);
  return launch<128>(p, PlainPolicy<128>{(__nv_bfloat16*)C, ldc, N, M}, ctas, s);
}

}  // namespace gemm
}  // namespace b200

extern "C" {

// C[M,N] (bf16, row-major, ldc) = A[M,K] (bf16, lda) * B[N,K]^T (bf16, ldb). bn: 0 auto, 128 or 256.
int b200ops_gemm_bf16_tn(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int bn, int maxCtas, cudaStream_t s) {
  return (int)b200::gemm::gemmBf16TN(A, B, C, M, N, K, lda, ldb, ldc, bn, maxCtas, s);
}

// Synchronises the device and returns (and clears) the code of the first bounded wait that gave
// up inside a tcgen05 kernel on this device; 0 when none did.
int b200ops_gemm_take_error(void) {
  int* w = b200::gemm::errWord();
  if (!w) return -1;
  int v = 0;
  if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (v) cudaMemset(w, 0, sizeof(int));
  return v;
}
}
