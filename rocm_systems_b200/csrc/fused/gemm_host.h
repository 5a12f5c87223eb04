// Host-side helpers shared by the tcgen05 GEMM and the fused GEMM+collective launchers.
#pragma once

#include <cuda.h>
#include <cuda_runtime_api.h>
#include <stdint.h>

namespace b200 {
namespace gemm {

bool makeTileMap(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t boxRows, uint32_t elemBytes);
int* errWord();   // per-device error word of the tcgen05 kernels (device memory)
int smCount();
cudaError_t gemmBf16TN(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int bn, int maxCtas, cudaStream_t s);

}  // namespace gemm
}  // namespace b200
