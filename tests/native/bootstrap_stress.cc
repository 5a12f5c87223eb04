// Host-side stress of the rendezvous, built with -fsanitize=address,undefined or -fsanitize=thread
// by tests/test_sanitizers_cpu.py: several "ranks" as threads of one process run rounds of
// all-gather, barrier and descriptor passing with random start skew, twice over (two communicators
// back to back), and check every result.
#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <atomic>
#include <random>
#include <thread>
#include <vector>

#include "core/bootstrap.h"

using namespace b200;

static std::atomic<int> gErrors{0};

static void fail(const char* what, int rank) {
  fprintf(stderr, "rank %d: %s\n", rank, what);
  gErrors++;
}

static void rankMain(ncclUniqueId id, int rank, int n, int rounds, unsigned seed) {
  std::mt19937 rng(seed + rank);
  Bootstrap b;
  usleep(rng() % 20000);  // ranks do not arrive together
  if (b.init(id, rank, n) != ncclSuccess) return fail("init", rank);
  for (int r = 0; r < rounds; r++) {
    if (rng() % 3 == 0) usleep(rng() % 3000);
    const size_t per = 8 + 8 * (size_t)((r * 7 + 3) % 50);  // depends on the round only, so it is the same on every rank
    std::vector<unsigned char> mine(per), all(per * n);
    for (size_t i = 0; i < per; i++) mine[i] = (unsigned char)(rank * 31 + r * 7 + i);
    if (b.allGather(mine.data(), all.data(), per) != ncclSuccess) return fail("allGather", rank);
    for (int p = 0; p < n; p++)
      for (size_t i = 0; i < per; i++)
        if (all[p * per + i] != (unsigned char)(p * 31 + r * 7 + i)) return fail("allGather content", rank);
    if (r % 4 == 0 && b.barrier() != ncclSuccess) return fail("barrier", rank);
    if (r % 5 == 0 && n > 1) {
      // pass a pipe's write end to the right neighbour; the neighbour writes its rank, we read it back
      int fds[2];
      if (pipe(fds) != 0) return fail("pipe", rank);
      const int right = (rank + 1) % n, left = (rank + n - 1) % n;
      if (b.sendFd(right, fds[1], 100 + r) != ncclSuccess) return fail("sendFd", rank);
      int got = -1;
      if (b.recvFd(left, 100 + r, &got) != ncclSuccess || got < 0) return fail("recvFd", rank);
      unsigned char me = (unsigned char)rank;
      if (write(got, &me, 1) != 1) return fail("write", rank);
      ::close(got);
      ::close(fds[1]);
      unsigned char who = 255;
      if (read(fds[0], &who, 1) != 1 || who != (unsigned char)right) return fail("fd passing content", rank);
      ::close(fds[0]);
    }
  }
  int which = -1;
  if (b.peerFailed(&which)) fail("spurious peer failure", rank);
  b.close(true);
}

int main(int argc, char** argv) {
  const int n = argc > 1 ? atoi(argv[1]) : 4;
  const int rounds = argc > 2 ? atoi(argv[2]) : 40;
  for (int gen = 0; gen < 2; gen++) {
    ncclUniqueId id;
    if (bootCreateRoot(&id) != ncclSuccess) {
      fprintf(stderr, "bootCreateRoot failed\n");
      return 2;
    }
    std::vector<std::thread> th;
    for (int r = 0; r < n; r++) th.emplace_back(rankMain, id, r, n, rounds, 1234u + 100u * gen);
    for (auto& t : th) t.join();
  }
  if (gErrors.load()) {
    fprintf(stderr, "%d errors\n", gErrors.load());
    return 1;
  }
  printf("bootstrap stress OK: %d ranks x %d rounds x 2 communicators\n", n, rounds);
  return 0;
}
