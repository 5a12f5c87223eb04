// Host side of a collective call: validation, algorithm choice, launch.
#pragma once

#include <vector>

#include "../core/comm.h"

namespace b200 {

struct CollReq {
  int apiId;            // b200collApiId, for the tracer
  int kind;             // CollKind
  const void* send;
  void* recv;
  size_t count;
  ncclDataType_t dt;
  int op;               // raw ncclRedOp_t value (built-in or PreMulSum handle)
  int root;
  Comm* comm;
  cudaStream_t stream;
  int forceAlgo = ALGO_AUTO;  // schedule-file override
  int forceCtas = 0;
  bool allowDirect = true;    // false: stage even when the buffers lie in symmetric windows
};
ncclResult_t enqueueColl(const CollReq& r);

struct P2pReq {
  bool isSend;
  void* buf;
  size_t bytes;
  int peer;
  cudaStream_t stream;
  int apiId;
};
// All sends and receives one group made on one communicator.
ncclResult_t enqueueP2pGroup(Comm* c, std::vector<P2pReq>& ops);
// All-to-all of chunks small enough for the flag-in-data buffers (llAllToAllFits), as one kernel.
bool llAllToAllFits(Comm* c, size_t bytesPerPeer);
int llCtaCap(size_t bytes, int nranks);
// All-to-all of large chunks through the staging halves (peer stores, one barrier per step), as one kernel.
void stagedAllToAllArgs(Comm* c, const void* send, void* recv, size_t count, ncclDataType_t dt, int forceCtas, CollArgs* args, DevComm* dc, int* ctas);
ncclResult_t enqueueStagedAllToAll(Comm* c, int apiId, const void* send, void* recv, size_t count, ncclDataType_t dt, cudaStream_t stream);
ncclResult_t enqueueLLAllToAll(Comm* c, int apiId, const void* send, void* recv, size_t count, ncclDataType_t dt, cudaStream_t stream);

// What the chooser would pick (exposed for tests and the tuner).
struct Plan {
  int algo; int ctas; bool direct; size_t chunks;
  // What the zero-copy decision rests on, for the cross-rank check: ids and offsets of the windows the buffers lie in (0: none).
  uint64_t sendWin = 0, recvWin = 0;
  size_t sendOff = 0, recvOff = 0;
};
ncclResult_t planColl(const CollReq& r, Plan* plan);
// One rank's share of a collective for the single-kernel emulation of several ranks on one GPU: everything enqueueColl
// does up to the launch (validation, plan, kernel arguments, sequence numbers, staging parity), nothing launched.
// plan->algo == ALGO_LL: `ll` is filled, otherwise `args`.
ncclResult_t emuPrepare(const CollReq& r, Plan* plan, CollArgs* args, LLArgs* ll, DevComm* dc);

}  // namespace b200
