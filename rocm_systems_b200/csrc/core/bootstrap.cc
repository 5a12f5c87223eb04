#include "bootstrap.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stddef.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <random>
#include <thread>

namespace b200 {

namespace {

enum FrameType : uint32_t { FR_HELLO = 1, FR_ROUND = 2, FR_REPLY = 3, FR_NOTIFY = 4, FR_BYE = 5 };
struct Frame {
  uint32_t type;
  uint32_t arg;    // HELLO: rank; NOTIFY: dead rank; REPLY: 0 ok / 1 a rank was lost
  uint64_t bytes;  // payload that follows (HELLO: nranks, no payload)
};

bool writeAll(int fd, const void* p, size_t n) {
  const char* c = (const char*)p;
  while (n) {
    ssize_t w = ::send(fd, c, n, MSG_NOSIGNAL);
    if (w < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    c += w;
    n -= (size_t)w;
  }
  return true;
}

// 1 ok, 0 peer closed, -1 error, -2 timeout
int readAll(int fd, void* p, size_t n, int timeoutMs) {
  char* c = (char*)p;
  uint64_t deadline = nowNs() + (uint64_t)timeoutMs * 1000000ull;
  while (n) {
    pollfd pf{fd, POLLIN, 0};
    int64_t leftMs = ((int64_t)deadline - (int64_t)nowNs()) / 1000000;
    if (leftMs <= 0) return -2;
    int pr = ::poll(&pf, 1, (int)(leftMs > 1000 ? 1000 : leftMs));
    if (pr < 0) {
      if (errno == EINTR) continue;
      return -1;
    }
    if (pr == 0) continue;
    ssize_t r = ::recv(fd, c, n, 0);
    if (r == 0) return 0;
    if (r < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      return -1;
    }
    c += r;
    n -= (size_t)r;
  }
  return 1;
}

// The rendezvous root: accepts `nranks` HELLOs, then serves rounds until everyone has left.
void rootLoop(int lfd, uint64_t nonce, int timeoutMs) {
  std::vector<int> socks;
  int nranks = -1;
  uint64_t deadline = nowNs() + (uint64_t)timeoutMs * 1000000ull;
  int connected = 0;
  while (nranks < 0 || connected < nranks) {
    pollfd pf{lfd, POLLIN, 0};
    int pr = ::poll(&pf, 1, 500);
    if (pr <= 0) {
      if (nowNs() > deadline) {
        BWARN("bootstrap root: only %d of %d ranks arrived before the deadline", connected, nranks);
        for (int s : socks) if (s >= 0) ::close(s);
        ::close(lfd);
        return;
      }
      continue;
    }
    int fd = ::accept(lfd, nullptr, nullptr);
    if (fd < 0) continue;
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    Frame h;
    uint64_t n2 = 0;
    if (readAll(fd, &h, sizeof(h), 5000) != 1 || h.type != FR_HELLO ||
        readAll(fd, &n2, sizeof(n2), 5000) != 1 || n2 != nonce) {
      ::close(fd);  // a stray connection; not one of ours
      continue;
    }
    if (nranks < 0) {
      nranks = (int)h.bytes;
      socks.assign(nranks, -1);
    }
    if ((int)h.bytes != nranks || (int)h.arg >= nranks || socks[h.arg] >= 0) {
      BWARN("bootstrap root: inconsistent HELLO (rank %u of %lu, expected %d ranks)", h.arg,
            (unsigned long)h.bytes, nranks);
      ::close(fd);
      continue;
    }
    socks[h.arg] = fd;
    connected++;
  }
  ::close(lfd);
  // Everyone is here: release them with an empty reply.
  for (int r = 0; r < nranks; r++) {
    Frame f{FR_REPLY, 0, 0};
    writeAll(socks[r], &f, sizeof(f));
  }

  std::vector<char> state(nranks, 0);  // 0 idle, 1 contributed to the open round, 2 left, 3 dead
  std::vector<std::vector<char>> parts(nranks);
  int alive = nranks;
  bool lost = false;
  auto markDead = [&](int r) {
    if (state[r] == 2 || state[r] == 3) return;
    state[r] = 3;
    lost = true;
    ::close(socks[r]);
    socks[r] = -1;
    alive--;
    for (int q = 0; q < nranks; q++) {
      if (socks[q] < 0) continue;
      Frame f{FR_NOTIFY, (uint32_t)r, 0};
      writeAll(socks[q], &f, sizeof(f));
    }
  };
  while (alive > 0) {
    std::vector<pollfd> pfs;
    std::vector<int> who;
    for (int r = 0; r < nranks; r++)
      if (socks[r] >= 0 && state[r] != 1) {
        pfs.push_back({socks[r], POLLIN, 0});
        who.push_back(r);
      }
    if (pfs.empty()) break;
    int pr = ::poll(pfs.data(), pfs.size(), 1000);
    if (pr < 0 && errno != EINTR) break;
    if (pr <= 0) continue;
    for (size_t i = 0; i < pfs.size(); i++) {
      if (!(pfs[i].revents & (POLLIN | POLLHUP | POLLERR))) continue;
      int r = who[i];
      Frame f;
      int rc = readAll(socks[r], &f, sizeof(f), 5000);
      if (rc != 1) { markDead(r); continue; }
      if (f.type == FR_BYE) {
        state[r] = 2;
        ::close(socks[r]);
        socks[r] = -1;
        alive--;
        continue;
      }
      if (f.type != FR_ROUND || f.bytes > (64u << 20)) { markDead(r); continue; }
      parts[r].resize(f.bytes);
      if (f.bytes && readAll(socks[r], parts[r].data(), f.bytes, 30000) != 1) { markDead(r); continue; }
      state[r] = 1;
    }
    // Close the round once every rank still connected has contributed.
    bool all = true;
    int contributors = 0;
    for (int r = 0; r < nranks; r++) {
      if (socks[r] >= 0 && state[r] != 1) all = false;
      if (state[r] == 1) contributors++;
    }
    if (all && contributors > 0) {
      size_t per = 0;
      for (int r = 0; r < nranks; r++) if (state[r] == 1) per = parts[r].size();
      std::vector<char> cat((size_t)nranks * per, 0);
      for (int r = 0; r < nranks; r++)
        if (state[r] == 1 && parts[r].size() == per && per) memcpy(&cat[(size_t)r * per], parts[r].data(), per);
      for (int r = 0; r < nranks; r++) {
        if (state[r] != 1) continue;
        Frame f{FR_REPLY, lost ? 1u : 0u, cat.size()};
        if (!writeAll(socks[r], &f, sizeof(f)) || (cat.size() && !writeAll(socks[r], cat.data(), cat.size()))) {
          markDead(r);
          continue;
        }
        state[r] = 0;
      }
    }
  }
  for (int s : socks) if (s >= 0) ::close(s);
}

}  // namespace

ncclResult_t bootCreateRoot(ncclUniqueId* out) {
  const Flags& fl = Flags::get();
  memset(out, 0, sizeof(*out));
  std::string addr = fl.ifaddr;
  int wantPort = 0;
  if (!fl.commId.empty()) {
    size_t c = fl.commId.rfind(':');
    if (c == std::string::npos) BFAIL(ncclInvalidArgument, "COMM_ID must be ip:port, got '%s'", fl.commId.c_str());
    addr = fl.commId.substr(0, c);
    wantPort = atoi(fl.commId.c_str() + c + 1);
  }
  int lfd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (lfd < 0) BFAIL(ncclSystemError, "bootstrap: socket() failed: %s", strerror(errno));
  int one = 1;
  setsockopt(lfd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in sa{};
  sa.sin_family = AF_INET;
  sa.sin_port = htons((uint16_t)wantPort);
  if (inet_pton(AF_INET, addr.c_str(), &sa.sin_addr) != 1) {
    ::close(lfd);
    BFAIL(ncclInvalidArgument, "bootstrap: bad address '%s'", addr.c_str());
  }
  // With COMM_ID every rank calls this and has to end up with the same id and exactly one root:
  // the id is derived from the string alone, and the rank that gets the port serves the rendezvous
  // (the others find the address taken, which means the root is already up).
  const bool shared = !fl.commId.empty();
  bool haveRoot = true;
  if (::bind(lfd, (sockaddr*)&sa, sizeof(sa)) != 0 || ::listen(lfd, 64) != 0) {
    int e = errno;
    ::close(lfd);
    lfd = -1;
    if (!(shared && e == EADDRINUSE)) BFAIL(ncclSystemError, "bootstrap: bind/listen on %s:%d failed: %s", addr.c_str(), wantPort, strerror(e));
    haveRoot = false;
  }
  BootId id{};
  id.magic = kBootMagic;
  if (shared) {
    uint64_t h = 0xcbf29ce484222325ull;  // FNV-1a of the COMM_ID string: the same nonce on every rank
    for (char ch : fl.commId) h = (h ^ (unsigned char)ch) * 0x100000001b3ull;
    id.nonce = h ? h : 1;
    inet_pton(AF_INET, addr.c_str(), &id.ip);
    id.port = (uint16_t)wantPort;
  } else {
    socklen_t sl = sizeof(sa);
    getsockname(lfd, (sockaddr*)&sa, &sl);
    std::random_device rd;
    id.nonce = ((uint64_t)rd() << 32) ^ rd() ^ ((uint64_t)getpid() << 17) ^ nowNs();
    id.ip = sa.sin_addr.s_addr;
    id.port = ntohs(sa.sin_port);
  }
  static_assert(sizeof(BootId) <= NCCL_UNIQUE_ID_BYTES, "BootId must fit in ncclUniqueId");
  memcpy(out->internal, &id, sizeof(id));
  if (!haveRoot) {
    BINFO(SUB_BOOT, "bootstrap root for COMM_ID %s is served by another process", fl.commId.c_str());
    return ncclSuccess;
  }
  std::thread(rootLoop, lfd, id.nonce, fl.bootTimeoutMs).detach();
  BINFO(SUB_BOOT, "bootstrap root listening on %s:%d nonce %016lx", addr.c_str(), (int)id.port,
        (unsigned long)id.nonce);
  return ncclSuccess;
}

Bootstrap::~Bootstrap() { close(false); }

std::string Bootstrap::udsName(int rank) const {
  char buf[96];
  snprintf(buf, sizeof(buf), "b200coll.%016lx.%d", (unsigned long)nonce_, rank);
  return buf;
}

static socklen_t fillAbstract(sockaddr_un& un, const std::string& name) {
  memset(&un, 0, sizeof(un));
  un.sun_family = AF_UNIX;
  un.sun_path[0] = '\0';
  memcpy(un.sun_path + 1, name.data(), name.size());
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + name.size());
}

ncclResult_t Bootstrap::init(const ncclUniqueId& uid, int rank, int nranks) {
  BootId id;
  memcpy(&id, uid.internal, sizeof(id));
  if (id.magic != kBootMagic) BFAIL(ncclInvalidArgument, "ncclUniqueId was not made by ncclGetUniqueId");
  if (nranks < 1 || rank < 0 || rank >= nranks) BFAIL(ncclInvalidArgument, "bad rank %d / nranks %d", rank, nranks);
  rank_ = rank;
  nranks_ = nranks;
  nonce_ = id.nonce;
  const int timeoutMs = Flags::get().bootTimeoutMs;
  if (failPoint("boot_connect")) BFAIL(ncclSystemError, "bootstrap: connect failed (injected)");

  // Datagram socket on which peers hand us file descriptors.
  uds_ = ::socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (uds_ < 0) BFAIL(ncclSystemError, "bootstrap: unix socket failed: %s", strerror(errno));
  sockaddr_un un;
  socklen_t ul = fillAbstract(un, udsName(rank));
  if (::bind(uds_, (sockaddr*)&un, ul) != 0) BFAIL(ncclSystemError, "bootstrap: unix bind failed: %s", strerror(errno));

  sockaddr_in sa{};
  sa.sin_family = AF_INET;
  sa.sin_addr.s_addr = id.ip;
  sa.sin_port = htons(id.port);
  uint64_t deadline = nowNs() + (uint64_t)timeoutMs * 1000000ull;
  while (true) {
    sock_ = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (sock_ < 0) BFAIL(ncclSystemError, "bootstrap: socket() failed: %s", strerror(errno));
    if (::connect(sock_, (sockaddr*)&sa, sizeof(sa)) == 0) break;
    ::close(sock_);
    sock_ = -1;
    if (nowNs() > deadline) BFAIL(ncclSystemError, "bootstrap: rank %d could not reach the root: %s", rank, strerror(errno));
    usleep(20000);
  }
  int one = 1;
  setsockopt(sock_, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  Frame h{FR_HELLO, (uint32_t)rank, (uint64_t)nranks};
  if (!writeAll(sock_, &h, sizeof(h)) || !writeAll(sock_, &nonce_, sizeof(nonce_)))
    BFAIL(ncclSystemError, "bootstrap: HELLO failed: %s", strerror(errno));
  std::vector<char> none;
  std::lock_guard<std::mutex> lk(mu_);
  return readReply(none);
}

ncclResult_t Bootstrap::readReply(std::vector<char>& payload) {
  const int timeoutMs = Flags::get().bootTimeoutMs;
  while (true) {
    Frame f;
    int rc = readAll(sock_, &f, sizeof(f), timeoutMs);
    if (rc == -2) BFAIL(ncclSystemError, "bootstrap: rank %d timed out after %d ms waiting for its peers", rank_, timeoutMs);
    if (rc != 1) BFAIL(ncclRemoteError, "bootstrap: rank %d lost the rendezvous root", rank_);
    if (f.type == FR_NOTIFY) {
      failedRank_ = (int)f.arg;
      BFAIL(ncclRemoteError, "bootstrap: rank %d left the communicator unexpectedly", failedRank_);
    }
    if (f.type != FR_REPLY) BFAIL(ncclInternalError, "bootstrap: unexpected frame %u", f.type);
    payload.resize(f.bytes);
    if (f.bytes && readAll(sock_, payload.data(), f.bytes, timeoutMs) != 1)
      BFAIL(ncclRemoteError, "bootstrap: short reply");
    if (f.arg != 0) BFAIL(ncclRemoteError, "bootstrap: a rank was lost during the round");
    return ncclSuccess;
  }
}

ncclResult_t Bootstrap::allGather(const void* send, void* recv, size_t bytes) {
  std::lock_guard<std::mutex> lk(mu_);
  if (sock_ < 0) BFAIL(ncclInvalidUsage, "bootstrap: communicator is closed");
  if (failedRank_ >= 0) BFAIL(ncclRemoteError, "bootstrap: rank %d is gone", failedRank_);
  char key[64];
  snprintf(key, sizeof(key), "boot_skip_round_rank%d", rank_);
  if (failPoint(key)) {  // injected: this rank stays silent, its peers must time out cleanly
    usleep((useconds_t)Flags::get().bootTimeoutMs * 1000u + 200000u);
    BFAIL(ncclSystemError, "bootstrap: round skipped (injected)");
  }
  snprintf(key, sizeof(key), "boot_die_rank%d", rank_);
  if (failPoint(key)) {  // injected: drop the connection without saying goodbye
    ::close(sock_);
    sock_ = -1;
    BFAIL(ncclSystemError, "bootstrap: connection dropped (injected)");
  }
  Frame f{FR_ROUND, 0, bytes};
  if (!writeAll(sock_, &f, sizeof(f)) || (bytes && !writeAll(sock_, send, bytes)))
    BFAIL(ncclRemoteError, "bootstrap: send failed: %s", strerror(errno));
  std::vector<char> payload;
  BCHECK(readReply(payload));
  if (payload.size() != bytes * (size_t)nranks_) BFAIL(ncclInternalError, "bootstrap: reply of %zu bytes, expected %zu", payload.size(), bytes * nranks_);
  if (bytes) memcpy(recv, payload.data(), payload.size());
  round_++;
  return ncclSuccess;
}

ncclResult_t Bootstrap::barrier() { return allGather(nullptr, nullptr, 0); }

bool Bootstrap::peerFailed(int* which) {
  std::unique_lock<std::mutex> lk(mu_, std::try_to_lock);
  if (!lk.owns_lock()) return false;  // a round is in flight; it will see the notice itself
  if (failedRank_ >= 0) {
    if (which) *which = failedRank_;
    return true;
  }
  if (sock_ < 0) return false;
  pollfd pf{sock_, POLLIN, 0};
  if (::poll(&pf, 1, 0) <= 0) return false;
  Frame f;
  ssize_t r = ::recv(sock_, &f, sizeof(f), MSG_PEEK | MSG_DONTWAIT);
  if (r == 0) {  // the root itself is gone
    failedRank_ = 0;
  } else if (r == (ssize_t)sizeof(f) && f.type == FR_NOTIFY) {
    ::recv(sock_, &f, sizeof(f), 0);
    failedRank_ = (int)f.arg;
  }
  if (failedRank_ >= 0 && which) *which = failedRank_;
  return failedRank_ >= 0;
}

ncclResult_t Bootstrap::sendFd(int peer, int fd, uint32_t tag) {
  sockaddr_un un;
  socklen_t ul = fillAbstract(un, udsName(peer));
  struct { int32_t src; uint32_t tag; } hdr{rank_, tag};
  iovec iov{&hdr, sizeof(hdr)};
  char cbuf[CMSG_SPACE(sizeof(int))];
  memset(cbuf, 0, sizeof(cbuf));
  msghdr msg{};
  msg.msg_name = &un;
  msg.msg_namelen = ul;
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = cbuf;
  msg.msg_controllen = sizeof(cbuf);
  cmsghdr* cm = CMSG_FIRSTHDR(&msg);
  cm->cmsg_level = SOL_SOCKET;
  cm->cmsg_type = SCM_RIGHTS;
  cm->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(cm), &fd, sizeof(int));
  uint64_t deadline = nowNs() + (uint64_t)Flags::get().bootTimeoutMs * 1000000ull;
  while (::sendmsg(uds_, &msg, 0) < 0) {
    if ((errno == EINTR || errno == EAGAIN || errno == ECONNREFUSED || errno == ENOBUFS) && nowNs() < deadline) {
      usleep(1000);
      continue;
    }
    BFAIL(ncclSystemError, "bootstrap: passing a descriptor to rank %d failed: %s", peer, strerror(errno));
  }
  return ncclSuccess;
}

ncclResult_t Bootstrap::recvFd(int peer, uint32_t tag, int* fdOut) {
  auto key = std::make_pair(peer, tag);
  uint64_t deadline = nowNs() + (uint64_t)Flags::get().bootTimeoutMs * 1000000ull;
  while (true) {
    auto it = stash_.find(key);
    if (it != stash_.end()) {
      *fdOut = it->second;
      stash_.erase(it);
      return ncclSuccess;
    }
    pollfd pf{uds_, POLLIN, 0};
    int pr = ::poll(&pf, 1, 500);
    if (pr <= 0) {
      if (nowNs() > deadline) BFAIL(ncclSystemError, "bootstrap: rank %d never received a descriptor from rank %d", rank_, peer);
      if (peerFailed()) BFAIL(ncclRemoteError, "bootstrap: rank %d is gone", failedRank_);
      continue;
    }
    struct { int32_t src; uint32_t tag; } hdr{};
    iovec iov{&hdr, sizeof(hdr)};
    char cbuf[CMSG_SPACE(sizeof(int))];
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = cbuf;
    msg.msg_controllen = sizeof(cbuf);
    ssize_t r = ::recvmsg(uds_, &msg, MSG_CMSG_CLOEXEC);
    if (r < 0) {
      if (errno == EINTR) continue;
      BFAIL(ncclSystemError, "bootstrap: recvmsg failed: %s", strerror(errno));
    }
    cmsghdr* cm = CMSG_FIRSTHDR(&msg);
    if (r != (ssize_t)sizeof(hdr) || !cm || cm->cmsg_type != SCM_RIGHTS) continue;
    int fd;
    memcpy(&fd, CMSG_DATA(cm), sizeof(int));
    stash_[std::make_pair((int)hdr.src, hdr.tag)] = fd;
  }
}

void Bootstrap::close(bool graceful) {
  std::lock_guard<std::mutex> lk(mu_);
  if (sock_ >= 0) {
    if (graceful) {
      Frame f{FR_BYE, 0, 0};
      writeAll(sock_, &f, sizeof(f));
    }
    ::close(sock_);
    sock_ = -1;
  }
  if (uds_ >= 0) {
    ::close(uds_);
    uds_ = -1;
  }
  for (auto& kv : stash_) ::close(kv.second);
  stash_.clear();
}

}  // namespace b200
