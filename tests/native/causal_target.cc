// Target of the causal-profiling tests: every iteration runs cpu_slow_func and cpu_fast_func side by side and waits for
// both, so the iteration takes as long as the slow one. The fast one does `fast_percent` of the slow one's work: making
// the slow one up to (100 - fast_percent) % faster speeds the program up by as much, more than that gains nothing, and
// making the fast one faster gains nothing at all.
//   causal_target <iterations> <fast_percent> <work> [spawn|pool]
// "spawn" starts two threads per iteration and joins them; "pool" keeps two workers and hands work over with a mutex and
// condition variables.
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <initializer_list>
#include <mutex>
#include <thread>

#include "b200coll/causal.h"

static volatile double sink;
// Each function has its loop on a line of its own, so that a source-line scope can tell them apart.
extern "C" __attribute__((noinline)) void cpu_slow_func(long n) {
  double a = 1.0;
  for (long i = 1; i <= n; i++) a += 1.0 / (double)(i + (long)a % 3);  // SLOW_LINE
  sink = a;
}
extern "C" __attribute__((noinline)) void cpu_fast_func(long n) {
  double a = 1.0;
  for (long i = 1; i <= n; i++) a += 1.0 / (double)(i + (long)a % 3);  // FAST_LINE
  sink = a;
}

struct Worker {
  std::mutex m;
  std::condition_variable cv;
  long work = 0;
  bool has = false, done = false, quit = false;
  void (*fn)(long) = nullptr;
  std::thread th;
  void loop() {
    std::unique_lock<std::mutex> lk(m);
    for (;;) {
      cv.wait(lk, [&] { return has || quit; });
      if (quit) return;
      has = false;
      lk.unlock();
      fn(work);
      lk.lock();
      done = true;
      cv.notify_all();
    }
  }
  void give(long n) {
    std::lock_guard<std::mutex> lk(m);
    work = n;
    has = true;
    done = false;
    cv.notify_all();
  }
  void wait() {
    std::unique_lock<std::mutex> lk(m);
    cv.wait(lk, [&] { return done; });
  }
};

int main(int argc, char** argv) {
  const int iterations = argc > 1 ? atoi(argv[1]) : 50;
  const int fastPercent = argc > 2 ? atoi(argv[2]) : 80;
  const long work = argc > 3 ? atol(argv[3]) : 4000000;
  const bool pool = argc > 4 && !strcmp(argv[4], "pool");
  const long fastWork = work * fastPercent / 100;
  if (pool) {
    Worker slow, fast;
    slow.fn = cpu_slow_func;
    fast.fn = cpu_fast_func;
    slow.th = std::thread([&] { slow.loop(); });
    fast.th = std::thread([&] { fast.loop(); });
    for (int i = 0; i < iterations; i++) {
      slow.give(work);
      fast.give(fastWork);
      slow.wait();
      fast.wait();
      B200CAUSAL_PROGRESS_NAMED("iteration");
    }
    for (Worker* w : {&slow, &fast}) {
      { std::lock_guard<std::mutex> lk(w->m); w->quit = true; w->cv.notify_all(); }
      w->th.join();
    }
  } else {
    for (int i = 0; i < iterations; i++) {
      B200CAUSAL_BEGIN("item");
      std::thread a(cpu_slow_func, work), b(cpu_fast_func, fastWork);
      a.join();
      b.join();
      B200CAUSAL_END("item");
      B200CAUSAL_PROGRESS_NAMED("iteration");
    }
  }
  printf("done %d\n", iterations);
  return 0;
}
