// <collective>_perf — benchmark and correctness harness in the style of rccl-tests
// (rccl-tests/src/common.cpp: flags :1340-1562, timing loop :756-850, table :1844-1875, busbw
// factors in the per-collective files). One source, compiled once per collective
// (-DPERF_COLL_ALL_REDUCE=1 …) and once more against stock NCCL (-DPERF_STOCK_NCCL=1) so the same
// harness produces the baseline.
//
// Ranks: `-g N` runs N GPUs as N threads of one process (ncclCommInitAll); under a launcher that
// sets RANK / WORLD_SIZE / LOCAL_RANK (torchrun) every process is one rank and the unique id
// travels through a file next to MASTER_PORT. Each size is timed two ways: host wall clock over
// the enqueue loop, averaged over ranks (the reference's default, `-a 1`), and CUDA events on the
// stream, maximum over ranks (the number this project reports). Then a correctness pass runs
// against the verifiable oracle and counts wrong elements.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <string>
#include <thread>
#include <vector>

#ifdef PERF_STOCK_NCCL
#include <nccl.h>
#define PERF_IMPL "nccl"
#else
#include "b200coll/nccl.h"
#define PERF_IMPL "b200coll"
#endif
#include "../coll/verifiable.cuh"

#ifndef PERF_NAME
#define PERF_NAME "all_reduce"
#endif

using b200::ver::Op;

#define CK(cmd)                                                                                   \
  do {                                                                                            \
    cudaError_t e__ = (cmd);                                                                      \
    if (e__ != cudaSuccess) { fprintf(stderr, "%s:%d CUDA error %s\n", __FILE__, __LINE__, cudaGetErrorString(e__)); exit(2); } \
  } while (0)
#define NK(cmd)                                                                                   \
  do {                                                                                            \
    ncclResult_t r__ = (cmd);                                                                     \
    if (r__ != ncclSuccess) { fprintf(stderr, "%s:%d NCCL error %s\n", __FILE__, __LINE__, ncclGetErrorString(r__)); exit(3); } \
  } while (0)

struct Args {
  int nGpus = 1;
  size_t minBytes = 32u << 20, maxBytes = 32u << 20, stepBytes = 1u << 20;
  double stepFactor = 1;
  int iters = 20, warmup = 5, agg = 1, cycles = 1, check = 1;
  std::string op = "sum", dtype = "float";
  int root = 0, blocking = 0, average = 1, reg = 0, outOfPlace = -1, graph = 0, cputime = 0, timeoutSec = 0;
  int parallelInit = 0, streamNull = 0, delayUs = 0, rotating = 0;
  std::string memType = "coarse";
  std::string outFile, outFormat = "csv";
};

// -E: consecutive iterations use buffers this far apart (rccl-tests common.cpp:32, 631-634).
static const size_t kRotateBytes = 192u << 20;

struct TypeInfo { const char* name; ncclDataType_t dt; int bytes; };
static const TypeInfo kTypes[] = {{"int8", ncclInt8, 1}, {"uint8", ncclUint8, 1}, {"int32", ncclInt32, 4}, {"uint32", ncclUint32, 4},
                                  {"int64", ncclInt64, 8}, {"uint64", ncclUint64, 8}, {"half", ncclFloat16, 2}, {"float", ncclFloat32, 4},
                                  {"double", ncclFloat64, 8}, {"bfloat16", ncclBfloat16, 2}
#ifndef PERF_STOCK_NCCL
                                  , {"fp8_e4m3", ncclFp8E4M3, 1}, {"fp8_e5m2", ncclFp8E5M2, 1}
#endif
};
static const char* kOps[] = {"sum", "prod", "max", "min", "avg", "mulsum"};

static size_t parseSize(const char* s) {
  char* end;
  double v = strtod(s, &end);
  switch (*end) {
    case 'G': case 'g': v *= 1024;  // fall through
    case 'M': case 'm': v *= 1024;  // fall through
    case 'K': case 'k': v *= 1024;
    default: break;
  }
  return (size_t)v;
}

// ---- what each collective moves ---------------------------------------------------------------------------------
struct Sizes { size_t sendCount, recvCount, paramCount; size_t sendInplaceOff, recvInplaceOff; };

static bool reducing() {
#if defined(PERF_COLL_ALL_REDUCE) || defined(PERF_COLL_REDUCE_SCATTER) || defined(PERF_COLL_REDUCE)
  return true;
#else
  return false;
#endif
}
static bool rooted() {
#if defined(PERF_COLL_BROADCAST) || defined(PERF_COLL_REDUCE) || defined(PERF_COLL_GATHER) || defined(PERF_COLL_SCATTER)
  return true;
#else
  return false;
#endif
}

// `count` = elements derived from the byte size; mirrors getCollByteCount of each rccl-tests file.
static Sizes sizesFor(size_t count, int n, int rank, int eltBytes) {
  Sizes s{};
#if defined(PERF_COLL_ALL_REDUCE) || defined(PERF_COLL_BROADCAST) || defined(PERF_COLL_REDUCE) || defined(PERF_COLL_SENDRECV) || defined(PERF_COLL_HYPERCUBE)
  s.sendCount = s.recvCount = s.paramCount = count;
#if defined(PERF_COLL_HYPERCUBE)
  s.paramCount = count / n;
  s.sendCount = s.paramCount;
  s.recvCount = s.paramCount * n;
  s.sendInplaceOff = (size_t)rank * s.paramCount;
#endif
#elif defined(PERF_COLL_ALL_GATHER)
  s.paramCount = count / n;
  s.sendCount = s.paramCount;
  s.recvCount = s.paramCount * n;
  s.sendInplaceOff = (size_t)rank * s.paramCount;
#elif defined(PERF_COLL_REDUCE_SCATTER)
  s.paramCount = count / n;
  s.sendCount = s.paramCount * n;
  s.recvCount = s.paramCount;
  s.recvInplaceOff = (size_t)rank * s.paramCount;
#else  // alltoall, alltoallv, gather, scatter: 16-byte aligned chunks (rccl-tests/src/alltoall.cpp:16-18)
  size_t per = (count / n) & ~(size_t)(16 / eltBytes - 1);
  if (eltBytes >= 16) per = count / n;
  s.paramCount = per;
  s.sendCount = s.recvCount = per * n;
#if defined(PERF_COLL_GATHER)
  s.sendCount = per;
#elif defined(PERF_COLL_SCATTER)
  s.recvCount = per;
#endif
#endif
  (void)rank;
  return s;
}

static double busFactor(int n) {
#if defined(PERF_COLL_ALL_REDUCE)
  return 2.0 * (n - 1) / n;
#elif defined(PERF_COLL_ALL_GATHER) || defined(PERF_COLL_REDUCE_SCATTER) || defined(PERF_COLL_ALLTOALL) || defined(PERF_COLL_ALLTOALLV) || \
    defined(PERF_COLL_GATHER) || defined(PERF_COLL_SCATTER)
  return (double)(n - 1) / n;
#else
  return 1.0;
#endif
}

// Bytes the "size" column and algbw refer to.
static size_t algBytes(const Sizes& s, int n, int eltBytes) {
#if defined(PERF_COLL_ALL_GATHER) || defined(PERF_COLL_HYPERCUBE)
  return s.recvCount * eltBytes;
#elif defined(PERF_COLL_REDUCE_SCATTER)
  return s.sendCount * eltBytes;
#elif defined(PERF_COLL_GATHER)
  return s.recvCount * eltBytes;
#elif defined(PERF_COLL_SCATTER)
  return s.sendCount * eltBytes;
#else
  (void)n;
  return s.sendCount * eltBytes;
#endif
}

static ncclResult_t runColl(const void* send, void* recv, const Sizes& s, ncclDataType_t dt, ncclRedOp_t op, int root, int rank, int n, int eltBytes,
                            ncclComm_t comm, cudaStream_t st) {
  (void)op; (void)root; (void)rank; (void)n; (void)eltBytes;
#if defined(PERF_COLL_ALL_REDUCE)
  return ncclAllReduce(send, recv, s.paramCount, dt, op, comm, st);
#elif defined(PERF_COLL_ALL_GATHER)
  return ncclAllGather(send, recv, s.paramCount, dt, comm, st);
#elif defined(PERF_COLL_REDUCE_SCATTER)
  return ncclReduceScatter(send, recv, s.paramCount, dt, op, comm, st);
#elif defined(PERF_COLL_BROADCAST)
  return ncclBroadcast(send, recv, s.paramCount, dt, root, comm, st);
#elif defined(PERF_COLL_REDUCE)
  return ncclReduce(send, recv, s.paramCount, dt, op, root, comm, st);
#elif defined(PERF_COLL_SENDRECV)
  ncclGroupStart();
  ncclSend(send, s.paramCount, dt, (rank + 1) % n, comm, st);
  ncclRecv(recv, s.paramCount, dt, (rank + n - 1) % n, comm, st);
  return ncclGroupEnd();
#elif defined(PERF_COLL_HYPERCUBE)
  // log2(n) exchange steps with rank ^ mask, doubling the block each time (rccl-tests/src/hypercube.cpp:81-88).
  char* r = (char*)recv;
  const size_t blk = s.paramCount * eltBytes;
  if ((const char*)send != r + (size_t)rank * blk) cudaMemcpyAsync(r + (size_t)rank * blk, send, blk, cudaMemcpyDeviceToDevice, st);
  for (int mask = 1; mask < n; mask <<= 1) {
    const int peer = rank ^ mask;
    const int myBase = rank & ~(mask - 1), peerBase = peer & ~(mask - 1);
    ncclGroupStart();
    ncclSend(r + (size_t)myBase * blk, s.paramCount * mask, dt, peer, comm, st);
    ncclRecv(r + (size_t)peerBase * blk, s.paramCount * mask, dt, peer, comm, st);
    ncclResult_t e = ncclGroupEnd();
    if (e != ncclSuccess) return e;
  }
  return ncclSuccess;
#elif defined(PERF_COLL_ALLTOALL) && !defined(PERF_STOCK_NCCL)
  return ncclAllToAll(send, recv, s.paramCount, dt, comm, st);
#elif defined(PERF_COLL_ALLTOALLV) && !defined(PERF_STOCK_NCCL)
  {
    std::vector<size_t> c(n, s.paramCount), d(n);
    for (int i = 0; i < n; i++) d[i] = (size_t)i * s.paramCount;
    return ncclAllToAllv(send, c.data(), d.data(), recv, c.data(), d.data(), dt, comm, st);
  }
#elif defined(PERF_COLL_GATHER) && !defined(PERF_STOCK_NCCL)
  return ncclGather(send, recv, s.paramCount, dt, root, comm, st);
#elif defined(PERF_COLL_SCATTER) && !defined(PERF_STOCK_NCCL)
  return ncclScatter(send, recv, s.paramCount, dt, root, comm, st);
#else
  // Stock NCCL has no all-to-all / gather / scatter entry points: grouped send/recv.
  const size_t blk = s.paramCount * eltBytes;
  ncclGroupStart();
#if defined(PERF_COLL_GATHER)
  ncclSend(send, s.paramCount, dt, root, comm, st);
  if (rank == root) for (int p = 0; p < n; p++) ncclRecv((char*)recv + (size_t)p * blk, s.paramCount, dt, p, comm, st);
#elif defined(PERF_COLL_SCATTER)
  if (rank == root) for (int p = 0; p < n; p++) ncclSend((const char*)send + (size_t)p * blk, s.paramCount, dt, p, comm, st);
  ncclRecv(recv, s.paramCount, dt, root, comm, st);
#else
  for (int p = 0; p < n; p++) {
    ncclSend((const char*)send + (size_t)p * blk, s.paramCount, dt, p, comm, st);
    ncclRecv((char*)recv + (size_t)p * blk, s.paramCount, dt, p, comm, st);
  }
#endif
  return ncclGroupEnd();
#endif
}

// ---- data -------------------------------------------------------------------------------------------------------
static int opCode(const std::string& op) {
  for (int i = 0; i < 6; i++) if (op == kOps[i]) return i;
  return -1;
}

static void initSend(void* send, const Sizes& s, int dtIdx, int op, uint64_t seed, int rank, int n, int root, cudaStream_t st) {
  const int dt = (int)kTypes[dtIdx].dt;
  if (reducing()) {
    CK(b200::ver::prepareInput(send, s.sendCount, 0, dt, op, seed, rank, n, st));
    return;
  }
  (void)root;
  // Non-reducing: the stream of values belongs to the source rank (seed * 33 + source).
  CK(b200::ver::prepareInput(send, s.sendCount, 0, dt, b200::ver::OP_NONE, seed * 33 + rank, 0, 1, st));
}

static void initExpected(void* exp, const Sizes& s, int dtIdx, int op, uint64_t seed, int rank, int n, int root, cudaStream_t st) {
  const int dt = (int)kTypes[dtIdx].dt;
  const int eb = kTypes[dtIdx].bytes;
  const size_t p = s.paramCount;
#if defined(PERF_COLL_ALL_REDUCE) || defined(PERF_COLL_REDUCE)
  CK(b200::ver::prepareExpected(exp, s.recvCount, 0, dt, op, seed, n, st));
#elif defined(PERF_COLL_REDUCE_SCATTER)
  CK(b200::ver::prepareExpected(exp, p, (size_t)rank * p, dt, op, seed, n, st));
#elif defined(PERF_COLL_ALL_GATHER) || defined(PERF_COLL_HYPERCUBE) || defined(PERF_COLL_GATHER)
  for (int src = 0; src < n; src++) CK(b200::ver::prepareInput((char*)exp + (size_t)src * p * eb, p, 0, dt, b200::ver::OP_NONE, seed * 33 + src, 0, 1, st));
#elif defined(PERF_COLL_BROADCAST)
  CK(b200::ver::prepareInput(exp, s.recvCount, 0, dt, b200::ver::OP_NONE, seed * 33 + root, 0, 1, st));
#elif defined(PERF_COLL_SENDRECV)
  CK(b200::ver::prepareInput(exp, s.recvCount, 0, dt, b200::ver::OP_NONE, seed * 33 + (rank + n - 1) % n, 0, 1, st));
#elif defined(PERF_COLL_SCATTER)
  CK(b200::ver::prepareInput(exp, p, (size_t)rank * p, dt, b200::ver::OP_NONE, seed * 33 + root, 0, 1, st));
#else  // alltoall(v): block from source `src` is that rank's block number `rank`
  for (int src = 0; src < n; src++)
    CK(b200::ver::prepareInput((char*)exp + (size_t)src * p * eb, p, (size_t)rank * p, dt, b200::ver::OP_NONE, seed * 33 + src, 0, 1, st));
#endif
  (void)op; (void)root; (void)eb; (void)p;
}

static bool checksOnThisRank(int rank, int root) {
#if defined(PERF_COLL_REDUCE) || defined(PERF_COLL_GATHER)
  return rank == root;
#else
  (void)rank; (void)root;
  return true;
#endif
}

static bool hasInPlace() {
#if defined(PERF_COLL_ALLTOALL) || defined(PERF_COLL_ALLTOALLV) || defined(PERF_COLL_SENDRECV) || defined(PERF_COLL_GATHER) || defined(PERF_COLL_SCATTER) || \
    defined(PERF_COLL_HYPERCUBE)
  return false;
#else
  return true;
#endif
}

static void scalarBytes(double v, int dtIdx, void* out) {
  switch (kTypes[dtIdx].dt) {
    case ncclFloat32: { float f = (float)v; memcpy(out, &f, 4); break; }
    case ncclFloat64: memcpy(out, &v, 8); break;
    case ncclFloat16: { __half h = __float2half((float)v); memcpy(out, &h, 2); break; }
    case ncclBfloat16: { __nv_bfloat16 h = __float2bfloat16((float)v); memcpy(out, &h, 2); break; }
    case ncclInt8: case ncclUint8: { uint8_t i = (uint8_t)v; memcpy(out, &i, 1); break; }
    case ncclInt32: case ncclUint32: { uint32_t i = (uint32_t)v; memcpy(out, &i, 4); break; }
    case ncclInt64: case ncclUint64: { uint64_t i = (uint64_t)v; memcpy(out, &i, 8); break; }
    default: { __nv_fp8_e4m3 q((float)v); memcpy(out, &q, 1); break; }
  }
}

// ---- one rank ---------------------------------------------------------------------------------------------------------
struct RankCtx {
  int rank, n, dev;
  ncclComm_t comm;
  const Args* a;
  FILE* out;          // result file (the reporting rank only)
  bool report;        // prints the table: rank 0 of the whole job, as in the reference harness
  double bwSum = 0;
  int bwCount = 0;
  long long wrongTotal = 0;
};

// Aggregates over the ranks with the communicator under test: v[0], v[1] are summed, v[2] is maximised; v[3] and v[4]
// come back as the maximum and the minimum of v[0] (for -a 3 and -a 2).
static void crossRank(RankCtx& c, double* dbuf, double v[5], cudaStream_t st) {
  double in[5] = {v[0], v[1], v[2], v[0], -v[0]};
  CK(cudaMemcpyAsync(dbuf, in, sizeof(in), cudaMemcpyHostToDevice, st));
  NK(ncclAllReduce(dbuf, dbuf, 2, ncclFloat64, ncclSum, c.comm, st));
  NK(ncclAllReduce(dbuf + 2, dbuf + 2, 3, ncclFloat64, ncclMax, c.comm, st));
  CK(cudaMemcpyAsync(v, dbuf, sizeof(in), cudaMemcpyDeviceToHost, st));
  CK(cudaStreamSynchronize(st));
  v[4] = -v[4];
}

static void runRank(RankCtx& c) {
  const Args& a = *c.a;
  CK(cudaSetDevice(c.dev));
  cudaStream_t st = nullptr;  // -y 1: the NULL stream
  if (!a.streamNull) CK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  const int n = c.n, rank = c.rank;
  std::vector<int> typeIdx, opIdx;
  const int nTypes = (int)(sizeof(kTypes) / sizeof(kTypes[0]));
  for (int i = 0; i < nTypes; i++) if (a.dtype == "all" || a.dtype == kTypes[i].name) typeIdx.push_back(i);
  if (reducing()) { for (int i = 0; i < 6; i++) if (a.op == "all" || a.op == kOps[i]) opIdx.push_back(i); }
  else opIdx.push_back(0);
  if (typeIdx.empty() || opIdx.empty()) { if (c.report) fprintf(stderr, "unknown -d %s or -o %s\n", a.dtype.c_str(), a.op.c_str()); exit(1); }

  // Buffers sized for the largest message; with -R they come from ncclMemAlloc and are registered.
  // -E adds the rotation distance; -Y picks where unregistered buffers live (coarse and fine are both plain device
  // memory here: CUDA has no uncached device allocation).
  const size_t maxBytes = a.maxBytes + 4096 + (a.rotating ? kRotateBytes : 0);
  void *send = nullptr, *recv = nullptr, *expect = nullptr;
  void *hs = nullptr, *hr = nullptr;
  if (a.reg) {
    NK(ncclMemAlloc(&send, maxBytes));
    NK(ncclMemAlloc(&recv, maxBytes));
    NK(ncclCommRegister(c.comm, send, maxBytes, &hs));
    NK(ncclCommRegister(c.comm, recv, maxBytes, &hr));
  } else if (a.memType == "host") {
    CK(cudaHostAlloc(&send, maxBytes, cudaHostAllocPortable));
    CK(cudaHostAlloc(&recv, maxBytes, cudaHostAllocPortable));
  } else if (a.memType == "managed") {
    CK(cudaMallocManaged(&send, maxBytes));
    CK(cudaMallocManaged(&recv, maxBytes));
  } else {
    CK(cudaMalloc(&send, maxBytes));
    CK(cudaMalloc(&recv, maxBytes));
  }
  CK(cudaMemset(send, 1, maxBytes));  // places that only the timed loop visits hold finite values too
  CK(cudaMemset(recv, 1, maxBytes));
  CK(cudaMalloc(&expect, maxBytes));
  double* dbuf;
  CK(cudaMalloc(&dbuf, 64));
  unsigned long long* wrongDev;
  CK(cudaMalloc(&wrongDev, 8));
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));

  for (int cyc = 0; cyc < a.cycles; cyc++)
  for (int ti : typeIdx) for (int oi : opIdx) {
    const int eb = kTypes[ti].bytes;
    const ncclDataType_t dt = kTypes[ti].dt;
    if (oi == 1 && eb == 1 && (int)dt >= 10) continue;  // fp8 x prod is skipped, as in rccl-tests (all_reduce.cpp:114-118)
    ncclRedOp_t op = (ncclRedOp_t)(oi < 5 ? oi : 0);
    bool customOp = false;
    if (reducing() && oi == 5) {
      char sc[8] = {};
      scalarBytes(b200::ver::mulsumScalar(rank), ti, sc);
      NK(ncclRedOpCreatePreMulSum(&op, sc, dt, ncclScalarHostImmediate, c.comm));
      customOp = true;
    }
    for (size_t bytes = a.minBytes; bytes <= a.maxBytes; bytes = (a.stepFactor > 1 ? (size_t)(bytes * a.stepFactor) : bytes + a.stepBytes)) {
      const size_t count = bytes / eb;
      const Sizes s = sizesFor(count, n, rank, eb);
      const size_t ab = algBytes(s, n, eb);
      double timeUs[2] = {-1, -1}, devUs[2] = {-1, -1}, wrong[2] = {-1, -1};
      for (int inplace = 0; inplace < 2; inplace++) {
        if (inplace && !hasInPlace()) continue;
        if (a.outOfPlace == 1 && inplace) continue;
        if (a.outOfPlace == 0 && !inplace) continue;
        if (s.paramCount == 0) { timeUs[inplace] = devUs[inplace] = 0; wrong[inplace] = 0; continue; }
        // In-place pointers follow the API's rules: the buffer under test is `recv` for gather-like
        // collectives (send lives inside it) and `send` for scatter-like ones.
        char* sp = (char*)send;
        char* rp = (char*)recv;
        if (inplace) {
#if defined(PERF_COLL_REDUCE_SCATTER)
          rp = sp + s.recvInplaceOff * eb;
#else
          sp = rp + s.sendInplaceOff * eb;
#endif
        }
        const uint64_t seed = 1 + (uint64_t)cyc;
        auto initData = [&](uint64_t sd) {
          if (inplace) {
#if defined(PERF_COLL_REDUCE_SCATTER)
            initSend(sp, s, ti, oi, sd, rank, n, a.root, st);
#else
            CK(cudaMemsetAsync(rp, 0, s.recvCount * eb, st));
            initSend(sp, s, ti, oi, sd, rank, n, a.root, st);
#endif
          } else {
            CK(cudaMemsetAsync(rp, 0, s.recvCount * eb, st));
            initSend(sp, s, ti, oi, sd, rank, n, a.root, st);
          }
        };
        initData(seed);
        // Every iteration works at a different offset so that a message is not served from cache and buffer
        // exchange is exercised: with -E two places 192 MiB apart, otherwise as many places as the largest
        // message leaves room for (common.cpp:625-640). Offsets are multiples of 512 bytes.
        const size_t span = (std::max(s.sendCount, s.recvCount) * eb + 511) & ~(size_t)511;
        const size_t places = a.rotating ? 2 : std::max<size_t>(1, a.maxBytes / std::max<size_t>(span, 1));
        auto shiftOf = [&](int it) -> size_t { return a.rotating ? kRotateBytes * (it & 1) : span * ((size_t)it % places); };
        auto timedColl = [&](int it) { const size_t sh = shiftOf(it); return runColl(sp + sh, rp + sh, s, dt, op, a.root, rank, n, eb, c.comm, st); };
        for (int w = 0; w < a.warmup; w++) NK(timedColl(w));
        CK(cudaStreamSynchronize(st));
        double agg[5] = {0, 0, 0, 0, 0};
        crossRank(c, dbuf, agg, st);  // barrier
        cudaGraph_t graph = nullptr;
        cudaGraphExec_t gexec = nullptr;
        const bool useGraph = a.graph && !a.streamNull;  // the NULL stream cannot be captured
        if (useGraph) {
          CK(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
          for (int it = 0; it < a.iters; it++) for (int m = 0; m < a.agg; m++) NK(timedColl(it));
          CK(cudaStreamEndCapture(st, &graph));
          CK(cudaGraphInstantiate(&gexec, graph, 0));
        }
        auto t0 = std::chrono::steady_clock::now();
        CK(cudaEventRecord(e0, st));
        if (useGraph) {
          CK(cudaGraphLaunch(gexec, st));
        } else {
          for (int it = 0; it < a.iters; it++) {
            for (int m = 0; m < a.agg; m++) NK(timedColl(it));
            if (a.blocking) CK(cudaStreamSynchronize(st));
          }
        }
        auto tEnq = std::chrono::steady_clock::now();
        CK(cudaEventRecord(e1, st));
        // Completion: poll the stream and the communicator, abort on error or -T timeout (common.cpp:559-620).
        while (true) {
          cudaError_t q = cudaStreamQuery(st);
          if (q == cudaSuccess) break;
          if (q != cudaErrorNotReady) CK(q);
          ncclResult_t ae = ncclSuccess;
          ncclCommGetAsyncError(c.comm, &ae);
          double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
          if (ae != ncclSuccess || (a.timeoutSec > 0 && el > a.timeoutSec)) {
            fprintf(stderr, "rank %d: %s; aborting the communicator\n", rank, ae != ncclSuccess ? ncclGetErrorString(ae) : "test timeout");
            ncclCommAbort(c.comm);
            exit(4);
          }
          sched_yield();
        }
        auto t1 = std::chrono::steady_clock::now();
        float ms = 0;
        CK(cudaEventElapsedTime(&ms, e0, e1));
        const double calls = (double)a.iters * a.agg;
        double wallUs = std::chrono::duration<double, std::micro>((a.cputime ? tEnq : t1) - t0).count() / calls;
        if (gexec) { cudaGraphExecDestroy(gexec); cudaGraphDestroy(graph); }
        // Correctness pass: fresh data, one call, compare with the oracle.
        double bad = 0;
        if (a.check > 0) {
          for (int ck = 0; ck < a.check; ck++) {
            const uint64_t sd = seed + 100 + ck;
            initData(sd);
            NK(runColl(sp, rp, s, dt, op, a.root, rank, n, eb, c.comm, st));
            if (checksOnThisRank(rank, a.root)) {
              initExpected(expect, s, ti, oi, sd, rank, n, a.root, st);
              CK(cudaMemsetAsync(wrongDev, 0, 8, st));
              CK(b200::ver::verify(rp, expect, s.recvCount, (int)dt, reducing() ? oi : b200::ver::OP_NONE, n, wrongDev, st));
              unsigned long long w = 0;
              CK(cudaMemcpyAsync(&w, wrongDev, 8, cudaMemcpyDeviceToHost, st));
              CK(cudaStreamSynchronize(st));
              bad += (double)w;
            }
          }
        }
        double v[5] = {wallUs, bad, (double)ms * 1e3 / calls, 0, 0};
        crossRank(c, dbuf, v, st);
        // -a: 0 this (reporting) rank, 1 average, 2 minimum, 3 maximum over the ranks (common.cpp:1452-1455)
        timeUs[inplace] = a.average == 1 ? v[0] / n : a.average == 2 ? v[4] : a.average == 3 ? v[3] : wallUs;
        wrong[inplace] = a.check > 0 ? v[1] : -1;
        devUs[inplace] = v[2];
        c.wrongTotal += (long long)v[1];
        if (!inplace && a.delayUs > 0) usleep(a.delayUs);  // -q: pause between the out-of-place and the in-place run
      }
      if (c.report) {
        char line[512];
        int o = snprintf(line, sizeof(line), "%12zu  %12zu  %8s  %6s  %4d", ab, s.paramCount, kTypes[ti].name, reducing() ? kOps[oi] : "none", rooted() ? a.root : -1);
        for (int ip = 0; ip < 2; ip++) {
          if (timeUs[ip] < 0) { o += snprintf(line + o, sizeof(line) - o, "  %9s %7s %7s %6s %9s", "N/A", "N/A", "N/A", "N/A", "N/A"); continue; }
          const double alg = timeUs[ip] > 0 ? ab / timeUs[ip] / 1e3 : 0, bus = alg * busFactor(n);
          const double dbus = devUs[ip] > 0 ? ab / devUs[ip] / 1e3 * busFactor(n) : 0;
          o += snprintf(line + o, sizeof(line) - o, "  %9.2f %7.2f %7.2f %6s %9.2f", timeUs[ip], alg, bus,
                        wrong[ip] < 0 ? "N/A" : std::to_string((long long)wrong[ip]).c_str(), devUs[ip]);
          c.bwSum += dbus;
          c.bwCount++;
          if (c.out) {
            if (a.outFormat == "json")
              fprintf(c.out, "{\"collective\":\"%s\",\"impl\":\"%s\",\"ranks\":%d,\"size\":%zu,\"count\":%zu,\"type\":\"%s\",\"redop\":\"%s\",\"root\":%d,\"inplace\":%d,\"time_us\":%.3f,\"algbw\":%.3f,\"busbw\":%.3f,\"dev_time_us\":%.3f,\"dev_busbw\":%.3f,\"wrong\":%lld}\n",
                      PERF_NAME, PERF_IMPL, n, ab, s.paramCount, kTypes[ti].name, reducing() ? kOps[oi] : "none", rooted() ? a.root : -1, ip, timeUs[ip], alg, bus, devUs[ip], dbus, (long long)wrong[ip]);
            else
              fprintf(c.out, "%d,%s,%s,%d,%zu,%zu,%s,%s,%d,%d,%.3f,%.3f,%.3f,%.3f,%.3f,%lld\n", cyc, PERF_NAME, PERF_IMPL, n, ab, s.paramCount, kTypes[ti].name,
                      reducing() ? kOps[oi] : "none", rooted() ? a.root : -1, ip, timeUs[ip], alg, bus, devUs[ip], dbus, (long long)wrong[ip]);
          }
        }
        printf("%s\n", line);
        fflush(stdout);
      }
      if (a.stepFactor <= 1 && a.stepBytes == 0) break;
    }
    if (customOp) NK(ncclRedOpDestroy(op, c.comm));
  }
  CK(cudaStreamSynchronize(st));
  if (a.reg) {
    ncclCommDeregister(c.comm, hs);
    ncclCommDeregister(c.comm, hr);
  }
}

// ---- communicator splitting ---------------------------------------------------------------------------------------------
// NCCL_TESTS_SPLIT_MASK=<hex> or NCCL_TESTS_SPLIT=AND<n> | OR<n> | MOD<n> | DIV<n> (also & | % /) give every rank a colour;
// ranks of one colour form one communicator and the benchmark runs in all of them at once (common.cpp:1640-1672).
static int colorOf(int proc) {
  if (const char* m = getenv("NCCL_TESTS_SPLIT_MASK")) return proc & (int)strtoul(m, nullptr, 16);
  const char* e = getenv("NCCL_TESTS_SPLIT");
  if (!e) return 0;
  struct { const char* word; const char* sym; int op; } forms[] = {{"AND", "&", 0}, {"OR", "|", 1}, {"MOD", "%", 2}, {"DIV", "/", 3}};
  for (auto& f : forms) {
    const char* arg = nullptr;
    if (strncasecmp(e, f.word, strlen(f.word)) == 0) arg = e + strlen(f.word);
    else if (strncmp(e, f.sym, 1) == 0) arg = e + 1;
    if (!arg) continue;
    char* end = nullptr;
    const long v = strtol(arg, &end, 0);
    if (end == arg) continue;
    switch (f.op) {
      case 0: return proc & (int)v;
      case 1: return proc | (int)v;
      case 2: return v > 0 ? proc % (int)v : 0;
      default: return v > 0 ? proc / (int)v : 0;
    }
  }
  return 0;
}

// The ranks that share `proc`'s colour, in rank order.
static std::vector<int> groupOf(int proc, int nprocs) {
  std::vector<int> g;
  const int col = colorOf(proc);
  for (int p = 0; p < nprocs; p++)
    if (colorOf(p) == col) g.push_back(p);
  return g;
}

// ---- main ------------------------------------------------------------------------------------------------------------
static void usage() {
  printf("USAGE: %s_perf [-g ngpus] [-b minbytes] [-e maxbytes] [-i stepbytes] [-f stepfactor] [-n iters] [-w warmup_iters] [-m agg_iters]\n"
         "       [-N run_cycles] [-c check] [-o sum|prod|max|min|avg|mulsum|all] [-d type|all] [-r root] [-z blocking] [-G cudagraph]\n"
         "       [-C report_cputime] [-a average 0|1|2|3] [-R local_register] [-O out_of_place 0|1] [-T timeout_s] [-x output_file] [-Z csv|json]\n"
         "       [-p parallel_init] [-y stream_null] [-q delay_inout_place_us] [-E rotating_tensor] [-Y coarse|fine|host|managed]\n", PERF_NAME);
}

static bool idFromFile(ncclUniqueId* id, int rank, int color) {
  const char* over = getenv("B200_PERF_ID_FILE");
  std::string path = over ? over : std::string("/tmp/b200_perf_id.") + (getenv("MASTER_PORT") ? getenv("MASTER_PORT") : "0") + "." +
                                       (getenv("TORCHELASTIC_RUN_ID") ? getenv("TORCHELASTIC_RUN_ID") : "run") + "." PERF_IMPL "." PERF_NAME;
  path += ".c" + std::to_string(color);
  if (rank == 0) {
    NK(ncclGetUniqueId(id));
    std::string tmp = path + ".tmp";
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) return false;
    fwrite(id, sizeof(*id), 1, f);
    fclose(f);
    rename(tmp.c_str(), path.c_str());
    return true;
  }
  for (int i = 0; i < 6000; i++) {
    FILE* f = fopen(path.c_str(), "rb");
    if (f) {
      size_t got = fread(id, sizeof(*id), 1, f);
      fclose(f);
      if (got == 1) return true;
    }
    usleep(10000);
  }
  return false;
}

int main(int argc, char** argv) {
  Args a;
  for (int i = 1; i < argc; i++) {
    std::string f = argv[i];
    auto next = [&]() -> const char* { if (i + 1 >= argc) { usage(); exit(1); } return argv[++i]; };
    if (f == "-g" || f == "--ngpus") a.nGpus = atoi(next());
    else if (f == "-t" || f == "--nthreads") (void)next();  // one thread per GPU here; accepted for command-line compatibility
    else if (f == "-b" || f == "--minbytes") a.minBytes = parseSize(next());
    else if (f == "-e" || f == "--maxbytes") a.maxBytes = parseSize(next());
    else if (f == "-i" || f == "--stepbytes") a.stepBytes = parseSize(next());
    else if (f == "-f" || f == "--stepfactor") a.stepFactor = atof(next());
    else if (f == "-n" || f == "--iters") a.iters = atoi(next());
    else if (f == "-w" || f == "--warmup_iters") a.warmup = atoi(next());
    else if (f == "-m" || f == "--agg_iters") a.agg = std::max(1, atoi(next()));
    else if (f == "-N" || f == "--run_cycles") a.cycles = std::max(1, atoi(next()));
    else if (f == "-c" || f == "--check") a.check = atoi(next());
    else if (f == "-o" || f == "--op") a.op = next();
    else if (f == "-d" || f == "--datatype") a.dtype = next();
    else if (f == "-r" || f == "--root") a.root = atoi(next());
    else if (f == "-z" || f == "--blocking") a.blocking = atoi(next());
    else if (f == "-G" || f == "--cudagraph") a.graph = atoi(next());
    else if (f == "-C" || f == "--report_cputime") a.cputime = atoi(next());
    else if (f == "-a" || f == "--average") a.average = atoi(next());
    else if (f == "-R" || f == "--local_register") a.reg = atoi(next());
    else if (f == "-O" || f == "--out_of_place") a.outOfPlace = atoi(next());
    else if (f == "-T" || f == "--timeout") a.timeoutSec = atoi(next());
    else if (f == "-x" || f == "--output_file") a.outFile = next();
    else if (f == "-Z" || f == "--output_format") a.outFormat = next();
    else if (f == "-p" || f == "--parallel_init") a.parallelInit = atoi(next());
    else if (f == "-y" || f == "--stream_null") a.streamNull = atoi(next());
    else if (f == "-q" || f == "--delay_inout_place") a.delayUs = atoi(next());
    else if (f == "-E" || f == "--rotating_tensor") a.rotating = atoi(next());
    else if (f == "-Y" || f == "--memory_type") {
      a.memType = next();
      if (a.memType != "coarse" && a.memType != "fine" && a.memType != "host" && a.memType != "managed") { fprintf(stderr, "unknown -Y %s\n", a.memType.c_str()); return 1; }
    }
    else if (f == "-u" || f == "--cumask" || f == "-F" || f == "--cache_flush") (void)next();  // AMD-only knobs: accepted, no effect
    else if (f == "--print-split") {  // how NCCL_TESTS_SPLIT[_MASK] groups this many ranks; needs no GPU
      const int np = atoi(next());
      for (int pr = 0; pr < np; pr++) {
        const std::vector<int> g = groupOf(pr, np);
        int idx = 0;
        while (g[idx] != pr) idx++;
        printf("%d color %d rank %d of %zu\n", pr, colorOf(pr), idx, g.size());
      }
      return 0;
    }
    else if (f == "-h" || f == "--help") { usage(); return 0; }
    else { fprintf(stderr, "unknown flag %s\n", f.c_str()); usage(); return 1; }
  }
  if (a.maxBytes < a.minBytes) a.maxBytes = a.minBytes;
  if (a.iters < 1) a.iters = 1;
  const char* wsEnv = getenv("WORLD_SIZE");
  const int world = wsEnv ? atoi(wsEnv) : 1;
  const bool procMode = world > 1;
  const int nAll = procMode ? world : a.nGpus;
  const int myRank = procMode ? atoi(getenv("RANK") ? getenv("RANK") : "0") : 0;
  const std::vector<int> firstGroup = groupOf(0, nAll);
  const int n = (int)firstGroup.size();  // size of the communicator the reporting rank is in
  {
    size_t smallest = nAll;
    for (int pr = 0; pr < nAll; pr++) smallest = std::min(smallest, groupOf(pr, nAll).size());
    if (a.root < 0 || a.root >= (int)smallest) a.root = 0;
  }

  FILE* out = nullptr;
  if (myRank == 0) {
    printf("# %s_perf (%s): ranks %d %s%s, bytes %zu..%zu, warmup %d, iters %d, agg %d, check %d\n", PERF_NAME, PERF_IMPL, n,
           procMode ? "processes" : "threads", n != nAll ? " per communicator (split)" : "", a.minBytes, a.maxBytes, a.warmup, a.iters, a.agg, a.check);
    printf("#\n# %10s  %12s  %8s  %6s  %4s  %46s  %46s\n", "", "", "", "", "", "out-of-place", "in-place");
    printf("# %10s  %12s  %8s  %6s  %4s  %9s %7s %7s %6s %9s  %9s %7s %7s %6s %9s\n", "size", "count", "type", "redop", "root", "time", "algbw", "busbw",
           "#wrong", "dev_time", "time", "algbw", "busbw", "#wrong", "dev_time");
    printf("# %10s  %12s  %8s  %6s  %4s  %9s %7s %7s %6s %9s  %9s %7s %7s %6s %9s\n", "(B)", "(elements)", "", "", "", "(us)", "(GB/s)", "(GB/s)", "", "(us,max)",
           "(us)", "(GB/s)", "(GB/s)", "", "(us,max)");
    if (!a.outFile.empty()) {
      out = fopen(a.outFile.c_str(), "w");
      if (out && a.outFormat != "json") fprintf(out, "numCycle,collective,impl,ranks,size,count,type,redop,root,inplace,time,algbw,busbw,dev_time,dev_busbw,wrong\n");
    }
  }

  // NCCL_TESTS_DEVICE: the first GPU to use (common.cpp:1706); ranks take consecutive devices from there.
  const int devBase = getenv("NCCL_TESTS_DEVICE") ? atoi(getenv("NCCL_TESTS_DEVICE")) : 0;
  std::vector<RankCtx> ctx;
  if (procMode) {
    const int local = devBase + atoi(getenv("LOCAL_RANK") ? getenv("LOCAL_RANK") : "0");
    CK(cudaSetDevice(local));
    const std::vector<int> group = groupOf(myRank, nAll);
    int groupRank = 0;
    while (group[groupRank] != myRank) groupRank++;
    ncclUniqueId id;
    if (!idFromFile(&id, groupRank, colorOf(myRank))) { fprintf(stderr, "rank %d: no unique id\n", myRank); return 5; }
    ncclComm_t comm;
    NK(ncclCommInitRank(&comm, (int)group.size(), id, groupRank));
    ctx.push_back(RankCtx{groupRank, (int)group.size(), local, comm, &a, out, myRank == 0});
    runRank(ctx[0]);
    NK(ncclCommDestroy(comm));
  } else {
    std::vector<ncclComm_t> comms(nAll);
    std::vector<std::thread> th;
    std::vector<int> groupRankOf(nAll), groupSizeOf(nAll);
    std::vector<bool> seen(nAll, false);
    for (int lead = 0; lead < nAll; lead++) {  // one communicator per colour
      if (seen[lead]) continue;
      const std::vector<int> group = groupOf(lead, nAll);
      const int gn = (int)group.size();
      std::vector<ncclComm_t> gc(gn);
      if (a.parallelInit) {  // -p 1: every thread brings up its own rank from a shared id (common.cpp:1697-1700)
        ncclUniqueId id;
        NK(ncclGetUniqueId(&id));
        for (int r = 0; r < gn; r++) th.emplace_back([&, r]() { CK(cudaSetDevice(devBase + group[r])); NK(ncclCommInitRank(&gc[r], gn, id, r)); });
        for (auto& t : th) t.join();
        th.clear();
      } else {
        std::vector<int> devs(gn);
        for (int r = 0; r < gn; r++) devs[r] = devBase + group[r];
        NK(ncclCommInitAll(gc.data(), gn, devs.data()));
      }
      for (int r = 0; r < gn; r++) {
        comms[group[r]] = gc[r];
        groupRankOf[group[r]] = r;
        groupSizeOf[group[r]] = gn;
        seen[group[r]] = true;
      }
    }
    for (int r = 0; r < nAll; r++) ctx.push_back(RankCtx{groupRankOf[r], groupSizeOf[r], devBase + r, comms[r], &a, r == 0 ? out : nullptr, r == 0});
    for (int r = 0; r < nAll; r++) th.emplace_back(runRank, std::ref(ctx[r]));
    for (auto& t : th) t.join();
    for (int r = 0; r < nAll; r++) NK(ncclCommDestroy(comms[r]));
  }
  int rc = 0;
  if (myRank == 0) {
    const RankCtx& c = ctx[0];
    const double avgBw = c.bwCount ? c.bwSum / c.bwCount : 0;
    printf("# Out of bounds values : %lld %s\n", c.wrongTotal, c.wrongTotal ? "FAILED" : "OK");
    printf("# Avg bus bandwidth    : %g (device-timed, max over ranks)\n#\n", avgBw);
    // NCCL_TESTS_MIN_BW gate of the reference (common.cpp:1963-1986).
    const char* minBw = getenv("NCCL_TESTS_MIN_BW");
    if (c.wrongTotal) rc = 1;
    if (minBw && avgBw < 0.9 * atof(minBw)) rc = 1;
    if (out) fclose(out);
  }
  return rc;
}
