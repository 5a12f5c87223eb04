// Structures shared by the host launcher and the collective kernels.
#pragma once

#include <stdint.h>

#include "../core/common.h"

namespace b200 {

// Status word a kernel fills when one of its bounded waits gives up. It lives in mapped host
// memory so the host can read it while the stream is still busy (the role of the queue error /
// system-event callbacks in rocr-runtime/runtime/hsa-runtime/core/runtime/runtime.cpp:1774-1944;
// here the kernel returns normally and the GPU context stays usable).
struct DevStatus {
  uint32_t code;      // 0 ok, 1 wait timed out, 2 aborted by the host
  uint32_t what;      // which wait: see WaitKind
  uint32_t peer;      // rank that did not answer
  uint32_t cta;       // block index of the waiter
  uint32_t expected;  // flag value waited for
  uint32_t seen;      // flag value last read
  uint64_t opSeq;     // sequence number of the collective on this communicator
};
enum WaitKind : uint32_t { WAIT_BARRIER = 1, WAIT_LL = 2, WAIT_P2P_DATA = 3, WAIT_P2P_CREDIT = 4, WAIT_SHMEM = 5, WAIT_FUSED = 6, WAIT_BULK = 7 };

// One record per traced collective, filled by the kernel with %globaltimer stamps.
struct TraceStamp {
  unsigned long long begin;  // min over CTAs of the entry time (ns)
  unsigned long long end;    // max over CTAs of the exit time (ns)
};

// Per-communicator state in this rank's own device memory (not mapped by peers).
struct LocalState {
  uint32_t barEpoch[kMaxCtas];                 // barriers completed, per CTA slot
  uint32_t failed;                             // set once a wait gave up: later waits return at once
  uint32_t pad[3];
  unsigned long long p2pSent[kMaxRanks][kMaxP2pSubs];    // chunks pushed to (peer, sub-channel) so far
  unsigned long long p2pRecvd[kMaxRanks][kMaxP2pSubs];   // chunks consumed from (peer, sub-channel) so far
};

// Byte offsets inside the symmetric workspace of every rank.
constexpr size_t kWsBarOff = 0;          // uint32 bar[kMaxCtas][kMaxRanks]
constexpr size_t kWsP2pCtrlOff = 8192;   // uint64 tail[kMaxRanks][kMaxP2pSubs], then head[kMaxRanks][kMaxP2pSubs]
constexpr size_t kWsUserFlagsOff = 16384;  // 48 KiB of flags for the shmem layer (barrier_all, …)
constexpr size_t kWsLLOff = 65536;

struct DevComm {
  int rank, nranks;
  char* ws[kMaxRanks];     // this rank's mapping of every rank's workspace
  char* wsMc;              // multicast alias of the workspace, or null
  size_t llSlotBytes;      // bytes of one source-rank slot of the flag-in-data buffer
  size_t stageOff;         // workspace offset of staging half 0
  size_t stageBytes;       // bytes per staging half
  size_t p2pOff;           // workspace offset of the send/recv FIFOs
  size_t p2pChunkBytes;    // bytes per FIFO slot
  int p2pSubs;             // sub-channels (CTAs) per peer and direction
  int p2pSlots;            // FIFO depth
  LocalState* local;
  DevStatus* status;               // mapped host memory
  volatile uint32_t* abortFlag;    // mapped host memory; non-zero ends every wait
  unsigned long long timeoutNs;
  unsigned long long opSeq;
  TraceStamp* stamp;       // null when tracing is off
};

enum CollKind : int { COLL_ALLREDUCE = 0, COLL_REDUCESCATTER = 1, COLL_REDUCE = 2, COLL_ALLGATHER = 3, COLL_BROADCAST = 4,
                      COLL_ALLTOALL = 5 /* flag-in-data kernel only; larger ones are grouped send/recv */ };

// How a reducing collective post-processes: Avg divides, PreMulSum scales the inputs.
enum ScaleMode : int { SCALE_NONE = 0, SCALE_POST_DIV_N = 1, SCALE_PRE_MUL = 2 };

struct CollArgs {
  const void* send;
  void* recv;
  size_t count;          // AllReduce/Reduce/Broadcast: elements; ReduceScatter: recvcount; AllGather: sendcount
  int kind;              // CollKind
  int root;
  int scaleMode;
  int stageHalf;         // staging half of the first chunk; alternates per chunk
  unsigned long long scalarBits;  // PreMulSum scalar, in the element type, zero-extended
  const void* scalarPtr;          // PreMulSum scalar in device memory (read by the kernel when it runs); null: scalarBits
  // Zero-copy windows: when both are set the buffers are symmetric and staging is skipped.
  char* sendPeer[kMaxRanks];
  char* recvPeer[kMaxRanks];
  char* sendMc;
  char* recvMc;
  int direct;            // 1: use the windows above
  size_t chunkBytes;     // staged reduce: bytes per pipeline chunk (per slice for ReduceScatter); 0 = a whole staging half
};

struct LLArgs {
  const void* send;
  void* recv;
  size_t count;          // elements per rank (all-reduce: the message; reduce-scatter / all-gather: one rank's slice); all-gather: bytes
  int kind;              // COLL_ALLREDUCE, COLL_REDUCESCATTER, COLL_ALLGATHER or COLL_ALLTOALL (count: bytes per peer)
  int scaleMode;
  unsigned long long scalarBits;
  const void* scalarPtr;  // see CollArgs
  uint32_t seq;          // flag value of this operation (never 0)
};

// All-to-all between receive buffers that lie in a symmetric window: every rank stores its chunk for peer p straight into
// p's buffer, at the place of the sending rank.
struct A2aDirectArgs {
  const char* send;              // n chunks of chunkBytes, chunk p goes to rank p
  char* recvPeer[kMaxRanks];     // every rank's receive buffer as mapped here
  size_t chunkBytes;             // a multiple of 16
};

struct P2pWork {
  int peer;
  int isSend;
  const char* src;       // send: user buffer
  char* dst;             // recv: user buffer
  size_t bytes;
};
constexpr int kMaxP2pWork = 2 * kMaxRanks;  // one send and one recv per peer and launch
struct P2pArgs {
  int nwork;
  P2pWork work[kMaxP2pWork];
};

}  // namespace b200
