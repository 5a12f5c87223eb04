// Target of the host-sampler tests: one thread burns CPU in burn_cycles(), another sleeps in idle_wait(), for about a second.
#include <cmath>
#include <cstdio>
#include <thread>
#include <chrono>
extern "C" __attribute__((noinline)) double burn_cycles(long n) { double a = 0; for (long i = 0; i < n; i++) a += std::sqrt((double)i); return a; }
extern "C" __attribute__((noinline)) void idle_wait(int ms) { std::this_thread::sleep_for(std::chrono::milliseconds(ms)); }
int main() {
  std::thread t([] { idle_wait(1000); });
  double a = 0;
  auto t0 = std::chrono::steady_clock::now();
  while (std::chrono::steady_clock::now() - t0 < std::chrono::milliseconds(1000)) a += burn_cycles(2000000);
  t.join();
  printf("%g\n", a);
}
