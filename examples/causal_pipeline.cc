// Causal profiling of a three-stage pipeline: which stage is worth optimising?
//
//   decode (2 units of work per item) -> transform (5 units) -> write (1 unit), one thread per stage, bounded queues between
//   them. A flat profile says transform takes 5/8 of the CPU time; the causal profile says what that is worth: making
//   transform up to 60 % faster speeds the program up by as much (then decode becomes the bound), making decode or write
//   faster gains nothing.
//
//   g++ -O1 -g -std=c++17 -I../rocm_systems_b200/csrc/include causal_pipeline.cc -o causal_pipeline -lpthread -ldl
//   python -m rocm_systems_b200.tools.causal run -o pipeline.coz -s 0 20 40 60 80 --report -- ./causal_pipeline 4000
//
// "item" counts finished items (throughput); "in flight" brackets an item from the moment it is produced to the moment it
// is written (latency). The program runs unchanged without the profiler: the marks find no library and do nothing.
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <deque>
#include <mutex>
#include <thread>

#include "b200coll/causal.h"

static volatile double sink;
static inline __attribute__((always_inline)) double work(long units) {  // inlined: each stage's time is its own function's
  double a = 1.0;
  for (long i = 1; i <= units * 20000; i++) a += 1.0 / (double)(i + (long)a % 3);
  return a;
}
extern "C" __attribute__((noinline)) void decode(int) { sink = work(2); }
extern "C" __attribute__((noinline)) void transform(int) { sink = work(5); }
extern "C" __attribute__((noinline)) void write_out(int) { sink = work(1); }

class Queue {
 public:
  explicit Queue(size_t cap) : cap_(cap) {}
  void put(int v) {
    std::unique_lock<std::mutex> lk(m_);
    notFull_.wait(lk, [&] { return q_.size() < cap_; });
    q_.push_back(v);
    notEmpty_.notify_one();
  }
  int take() {
    std::unique_lock<std::mutex> lk(m_);
    notEmpty_.wait(lk, [&] { return !q_.empty(); });
    const int v = q_.front();
    q_.pop_front();
    notFull_.notify_one();
    return v;
  }

 private:
  size_t cap_;
  std::mutex m_;
  std::condition_variable notFull_, notEmpty_;
  std::deque<int> q_;
};

int main(int argc, char** argv) {
  const int items = argc > 1 ? atoi(argv[1]) : 2000;
  Queue a(8), b(8);
  std::thread first([&] {
    for (int i = 0; i < items; i++) {
      B200CAUSAL_BEGIN("in flight");
      decode(i);
      a.put(i);
    }
    a.put(-1);
  });
  std::thread second([&] {
    for (;;) {
      const int v = a.take();
      if (v < 0) break;
      transform(v);
      b.put(v);
    }
    b.put(-1);
  });
  long done = 0;
  for (;;) {
    const int v = b.take();
    if (v < 0) break;
    write_out(v);
    B200CAUSAL_END("in flight");
    B200CAUSAL_PROGRESS_NAMED("item");
    done++;
  }
  first.join();
  second.join();
  printf("causal_pipeline OK: %ld items\n", done);
  return 0;
}
