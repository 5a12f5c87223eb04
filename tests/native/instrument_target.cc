// Target of the function-instrumentation test, built with -finstrument-functions: main calls outer() three times, outer
// calls inner() twice and sleeps 2 ms itself; never_called() stays cold; a second thread runs inner() once.
#include <chrono>
#include <cstdio>
#include <thread>
static volatile double sink;
__attribute__((noinline)) void inner(int n) { double a = 0; for (int i = 0; i < n; i++) a += i * 0.5; sink = a; std::this_thread::sleep_for(std::chrono::milliseconds(1)); }
__attribute__((noinline)) void outer() { inner(1000); inner(2000); std::this_thread::sleep_for(std::chrono::milliseconds(2)); }
__attribute__((noinline)) void never_called() { sink = 1; }
namespace app { struct Solver { __attribute__((noinline)) int run(int k) { outer(); return k + 1; } }; }
int main(int argc, char**) {
  app::Solver s;
  int k = 0;
  for (int i = 0; i < 3; i++) k = s.run(k);
  std::thread t([] { inner(10); });
  t.join();
  if (argc > 5) never_called();
  printf("instrument target done %d\n", k);
  return 0;
}
