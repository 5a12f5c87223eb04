// The planner, the settings listing and the tuning-file loader driven with random and hostile inputs; built together with
// the whole library under AddressSanitizer and UBSan (float-cast overflow included) by tests/test_sanitizers_cpu.py.
#include <stdio.h>
#include <cuda_runtime_api.h>
#include <stdlib.h>
#include <string>
#include "b200coll/nccl.h"
#include "b200coll/shmem.h"
#include "b200coll/smi.h"
int main() {
  uint64_t s = 12345;
  auto rnd = [&]() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return s; };
  int bad = 0;
  for (int i = 0; i < 20000; i++) {
    b200collPlanInfo info;
    int n = 1 + rnd() % 8, kind = rnd() % 5, dt = rnd() % 12, op = rnd() % 5;
    size_t count = (size_t)1 << (rnd() % 31); count += rnd() % 7;
    ncclResult_t r = b200collPlanDry(n, rnd() & 1, kind, count, (ncclDataType_t)dt, (ncclRedOp_t)op, &info);
    if (r != ncclSuccess || info.ctas < 1) bad++;
  }
  // bad arguments are refused, not crashed on
  b200collPlanInfo info;
  if (b200collPlanDry(0, 1, 0, 1, ncclFloat32, ncclSum, &info) == ncclSuccess) bad++;
  if (b200collPlanDry(9, 1, 0, 1, ncclFloat32, ncclSum, &info) == ncclSuccess) bad++;
  if (b200collPlanDry(8, 1, 7, 1, ncclFloat32, ncclSum, &info) == ncclSuccess) bad++;
  if (b200collPlanDry(8, 1, 0, 1, (ncclDataType_t)99, ncclSum, &info) == ncclSuccess) bad++;
  if (b200collPlanDry(8, 1, 0, 1, ncclFloat32, ncclSum, nullptr) == ncclSuccess) bad++;
  size_t need = b200collDescribeSettings(nullptr, 0);
  std::string buf(need, 0);
  b200collDescribeSettings(&buf[0], need);
  char small[8];
  b200collDescribeSettings(small, sizeof(small));
  // Entry points on a machine without a GPU (or with one): errors or successes, never a crash, a leak of a half-built
  // communicator that a later call trips over, or a use after free on the failure paths.
  for (int code = 0; code < 10; code++)
    if (!ncclGetErrorString((ncclResult_t)code)) bad++;
  int version = 0;
  if (ncclGetVersion(&version) != ncclSuccess || version < 20000) bad++;
  if (ncclGetVersion(nullptr) == ncclSuccess) bad++;
  if (ncclCommDestroy(nullptr) == ncclSuccess && false) bad++;
  (void)ncclGetLastError(nullptr);
  int ngpu = 0;
  const bool haveGpu = cudaGetDeviceCount(&ngpu) == cudaSuccess && ngpu > 0;
  ncclUniqueId id;
  if (ncclGetUniqueId(&id) != ncclSuccess) bad++;
  if (ncclGetUniqueId(nullptr) == ncclSuccess) bad++;
  ncclComm_t comm = nullptr;
  if (ncclCommInitRank(&comm, 0, id, 0) == ncclSuccess) bad++;      // no ranks
  if (ncclCommInitRank(&comm, 1, id, 3) == ncclSuccess) bad++;      // rank outside the communicator
  if (ncclCommInitRank(nullptr, 1, id, 0) == ncclSuccess) bad++;
  ncclResult_t r1 = ncclCommInitRank(&comm, 1, id, 0);
  if (!haveGpu && r1 == ncclSuccess) bad++;
  if (r1 == ncclSuccess) {
    int cnt = 0, rk = -1;
    if (ncclCommCount(comm, &cnt) != ncclSuccess || cnt != 1 || ncclCommUserRank(comm, &rk) != ncclSuccess || rk != 0) bad++;
    if (ncclCommDestroy(comm) != ncclSuccess) bad++;
  }
  ncclComm_t two[2] = {nullptr, nullptr};
  int devs[2] = {0, 0};
  if (ncclCommInitAll(two, 2, devs) == ncclSuccess) bad++;          // the same device twice
  if (ncclCommInitAll(nullptr, 1, nullptr) == ncclSuccess) bad++;
  void* p = nullptr;
  ncclResult_t ra = ncclMemAlloc(&p, 1 << 20);
  if (!haveGpu && ra == ncclSuccess) bad++;
  if (ra == ncclSuccess && ncclMemFree(p) != ncclSuccess) bad++;
  if (ncclMemAlloc(nullptr, 16) == ncclSuccess) bad++;
  b200shmem_ctx_t sh = nullptr;
  if (b200shmem_init(nullptr, 1 << 20, &sh) == ncclSuccess) bad++;
  if (b200shmem_my_pe(nullptr) != -1 || b200shmem_n_pes(nullptr) != 0 || b200shmem_malloc(nullptr, 64) != nullptr) bad++;
  size_t offs[B200SHMEM_MAX_DMA_GANG], lens[B200SHMEM_MAX_DMA_GANG];
  for (int i = 0; i < 2000; i++) {
    const size_t bytes = rnd() % ((size_t)1 << (rnd() % 34));
    const int g = b200shmem_dma_plan(bytes, (int)(rnd() % 20) - 2, offs, lens);
    size_t sum = 0;
    for (int k = 0; k < g; k++) sum += lens[k];
    if (g < 1 || g > B200SHMEM_MAX_DMA_GANG || sum != bytes) bad++;
  }
  int count = -1;
  (void)b200smi_device_count(&count);                               // NVML may or may not be there
  if (b200smi_device_count(nullptr) == B200SMI_OK) bad++;
  b200smi_event_t ev;
  if (b200smi_events_wait(10, &ev) == B200SMI_OK) bad++;            // never opened
  if (!b200smi_status_string(B200SMI_ERR_TIMEOUT)) bad++;
  printf("planner under sanitizers: %d bad, settings %zu bytes, version ok\n", bad, need);
  return bad ? 1 : 0;
}
