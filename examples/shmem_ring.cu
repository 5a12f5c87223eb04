// Device-initiated communication from a user kernel: every PE's kernel puts a block of data into
// its right neighbour's symmetric buffer together with a signal, waits (bounded) for the signal
// of its left neighbour, and checks what arrived. The host side only sets things up.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a examples/shmem_ring.cu -I rocm_systems_b200/csrc/include \
//       -L rocm_systems_b200/lib -lb200coll -o shmem_ring      # one process per GPU, e.g. under torchrun or mpirun
#include <cstdio>
#include <cstdlib>

#include "b200coll/nccl.h"
#include "b200coll/shmem.h"
#include "b200coll/shmem_device.cuh"

__global__ void ringStep(b200shmem_dev_t dev, int* inbox, const int* outbox, unsigned long long* sig, int count, unsigned long long round,
                         int* errors) {
  const int right = (dev.pe + 1) % dev.npes, left = (dev.pe + dev.npes - 1) % dev.npes;
  // data first, then the signal, as the receiver will see them
  b200shmem::putmem_signal_block(dev, inbox, outbox, (size_t)count * sizeof(int), sig, round, B200SHMEM_SIGNAL_SET, right);
  __shared__ int status;
  if (threadIdx.x == 0) status = b200shmem::signal_wait_until(dev, sig, B200SHMEM_CMP_GE, round);  // gives up after the context's budget
  __syncthreads();
  if (status != B200SHMEM_OK) {
    if (threadIdx.x == 0) atomicAdd(errors, 1 << 20);
    return;
  }
  int bad = 0;
  for (int i = threadIdx.x; i < count; i += blockDim.x) bad += inbox[i] != left * 1000 + i + (int)round;
  if (bad) atomicAdd(errors, bad);
}

__global__ void fill(int* outbox, int count, int pe, int round) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) outbox[i] = pe * 1000 + i + round;
}

#define NK(x) do { ncclResult_t r_ = (x); if (r_ != ncclSuccess) { fprintf(stderr, "%s: %s (%s)\n", #x, ncclGetErrorString(r_), ncclGetLastError(nullptr)); return 1; } } while (0)

int main() {
  // Rank and size come from the launcher; the id travels through NCCL_COMM_ID / B200COLL_COMM_ID ("ip:port").
  const char* r = getenv("RANK");
  const char* w = getenv("WORLD_SIZE");
  const int rank = r ? atoi(r) : 0, world = w ? atoi(w) : 1;
  const char* lr = getenv("LOCAL_RANK");
  cudaSetDevice(lr ? atoi(lr) : rank);
  ncclUniqueId id;
  NK(ncclGetUniqueId(&id));  // with COMM_ID set every rank derives the same id
  ncclComm_t comm;
  NK(ncclCommInitRank(&comm, world, id, rank));
  b200shmem_ctx_t ctx;
  NK(b200shmem_init(comm, 16u << 20, &ctx));
  const int count = 1 << 16;
  int* inbox = (int*)b200shmem_malloc(ctx, count * sizeof(int));
  auto* sig = (unsigned long long*)b200shmem_malloc(ctx, 256);
  int *outbox, *errors;
  cudaMalloc(&outbox, count * sizeof(int));
  cudaMalloc(&errors, sizeof(int));
  cudaMemset(errors, 0, sizeof(int));
  cudaMemset(sig, 0, 256);
  b200shmem_dev_t dev;
  NK(b200shmem_device_ctx(ctx, &dev));
  NK(b200shmem_barrier_all_on_stream(ctx, 0));
  for (int round = 1; round <= 4; round++) {
    fill<<<64, 256>>>(outbox, count, rank, round);
    ringStep<<<1, 512>>>(dev, inbox, outbox, sig, count, (unsigned long long)round, errors);
    NK(b200shmem_barrier_all_on_stream(ctx, 0));  // nobody overwrites an inbox that is still being checked
  }
  int host = -1;
  cudaMemcpy(&host, errors, sizeof(int), cudaMemcpyDeviceToHost);
  printf("PE %d of %d: %d errors, status %d\n", rank, world, host, b200shmem_take_status(ctx));
  b200shmem_free(ctx, sig);
  b200shmem_free(ctx, inbox);
  NK(b200shmem_finalize(ctx));
  NK(ncclCommDestroy(comm));
  return host != 0;
}
