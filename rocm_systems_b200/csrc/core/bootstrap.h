// Out-of-band rendezvous between the ranks of a communicator.
//
// rccl-tests uses MPI for this (rccl-tests/src/common.cpp:1627-1686, 1759); the runtime under
// RCCL passes memory handles over an AF_UNIX socket with SCM_RIGHTS
// (rocr-runtime/runtime/hsa-runtime/core/runtime/runtime.cpp:1087-1197). Here both are one small
// service: the process that makes the ncclUniqueId runs a root thread; every rank keeps one
// TCP connection to it (all-gather / barrier rounds, failure notices) and one abstract-namespace
// datagram socket on which it receives file descriptors from its peers.
#pragma once

#include <stdint.h>

#include <map>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "common.h"

namespace b200 {

struct BootId {            // what lives inside ncclUniqueId::internal (128 bytes)
  uint64_t magic;          // kBootMagic
  uint64_t nonce;          // names the rendezvous; also seeds the unix-socket names
  uint32_t ip;             // IPv4 of the root, network order
  uint16_t port;           // TCP port of the root, host order
  uint16_t pad;
};
constexpr uint64_t kBootMagic = 0xb200c011ec7155ull;

ncclResult_t bootCreateRoot(ncclUniqueId* out);  // binds a listener and starts the root thread

class Bootstrap {
 public:
  Bootstrap() = default;
  ~Bootstrap();
  ncclResult_t init(const ncclUniqueId& id, int rank, int nranks);
  ncclResult_t allGather(const void* send, void* recv, size_t bytesPerRank);
  ncclResult_t barrier();
  ncclResult_t sendFd(int peer, int fd, uint32_t tag);
  ncclResult_t recvFd(int peer, uint32_t tag, int* fd);
  // Non-blocking: has the root reported that some rank's connection dropped?
  bool peerFailed(int* whichRank = nullptr);
  void close(bool graceful = true);
  int rank() const { return rank_; }
  int nranks() const { return nranks_; }
  uint64_t nonce() const { return nonce_; }

 private:
  ncclResult_t readReply(std::vector<char>& payload);
  std::string udsName(int rank) const;
  std::mutex mu_;
  int sock_ = -1, uds_ = -1;
  int rank_ = -1, nranks_ = 0;
  uint64_t nonce_ = 0;
  int failedRank_ = -1;
  uint64_t round_ = 0;
  std::map<std::pair<int, uint32_t>, int> stash_;  // fds that arrived before they were asked for
};

}  // namespace b200
