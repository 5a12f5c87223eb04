/* The smallest complete program on the C API: one process drives every GPU of the box with
 * ncclCommInitAll, sums a buffer across them and checks the result. Plain C on purpose: nccl.h has
 * to be usable from C.
 *
 *   gcc examples/allreduce.c -I rocm_systems_b200/csrc/include -I /usr/local/cuda/include \
 *       -L rocm_systems_b200/lib -lb200coll -L /usr/local/cuda/lib64 -lcudart -o allreduce
 */
#include <cuda_runtime_api.h>
#include <stdio.h>
#include <stdlib.h>

#include "b200coll/nccl.h"

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_)); return 1; } } while (0)
#define NK(x) do { ncclResult_t r_ = (x); if (r_ != ncclSuccess) { fprintf(stderr, "%s: %s (%s)\n", #x, ncclGetErrorString(r_), ncclGetLastError(NULL)); return 1; } } while (0)

int main(void) {
  int n = 0;
  CK(cudaGetDeviceCount(&n));
  if (n > 8) n = 8;
  if (n < 1) { fprintf(stderr, "no GPU\n"); return 1; }
  const size_t count = 1u << 20;
  ncclComm_t comms[8];
  float* buf[8];
  cudaStream_t streams[8];
  NK(ncclCommInitAll(comms, n, NULL));
  float* host = (float*)malloc(count * sizeof(float));
  for (int d = 0; d < n; d++) {
    CK(cudaSetDevice(d));
    CK(cudaMalloc((void**)&buf[d], count * sizeof(float)));
    CK(cudaStreamCreate(&streams[d]));
    for (size_t i = 0; i < count; i++) host[i] = (float)(d + 1);
    CK(cudaMemcpy(buf[d], host, count * sizeof(float), cudaMemcpyHostToDevice));
  }
  NK(ncclGroupStart());  /* one thread, several communicators: the calls must be grouped */
  for (int d = 0; d < n; d++) NK(ncclAllReduce(buf[d], buf[d], count, ncclFloat32, ncclSum, comms[d], streams[d]));
  NK(ncclGroupEnd());
  int wrong = 0;
  for (int d = 0; d < n; d++) {
    CK(cudaSetDevice(d));
    CK(cudaStreamSynchronize(streams[d]));
    ncclResult_t async;
    NK(ncclCommGetAsyncError(comms[d], &async));
    if (async != ncclSuccess) { fprintf(stderr, "GPU %d: %s\n", d, ncclGetLastError(comms[d])); return 1; }
    CK(cudaMemcpy(host, buf[d], count * sizeof(float), cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < count; i++) wrong += host[i] != (float)(n * (n + 1) / 2);
  }
  printf("all-reduce over %d GPUs: %d wrong\n", n, wrong);
  for (int d = 0; d < n; d++) {
    CK(cudaSetDevice(d));
    CK(cudaFree(buf[d]));
    CK(cudaStreamDestroy(streams[d]));
    NK(ncclCommDestroy(comms[d]));
  }
  free(host);
  return wrong != 0;
}
