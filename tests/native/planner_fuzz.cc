// The planner, the settings listing and the tuning-file loader driven with random and hostile inputs; built together with
// the whole library under AddressSanitizer and UBSan (float-cast overflow included) by tests/test_sanitizers_cpu.py.
#include <stdio.h>
#include <stdlib.h>
#include <string>
#include "b200coll/nccl.h"
int main() {
  uint64_t s = 12345;
  auto rnd = [&]() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return s; };
  int bad = 0;
  for (int i = 0; i < 20000; i++) {
    b200collPlanInfo info;
    int n = 1 + rnd() % 8, kind = rnd() % 5, dt = rnd() % 12, op = rnd() % 5;
    size_t count = (size_t)1 << (rnd() % 31); count += rnd() % 7;
    ncclResult_t r = b200collPlanDry(n, rnd() & 1, kind, count, (ncclDataType_t)dt, (ncclRedOp_t)op, &info);
    if (r != ncclSuccess || info.ctas < 1) bad++;
  }
  // bad arguments are refused, not crashed on
  b200collPlanInfo info;
  if (b200collPlanDry(0, 1, 0, 1, ncclFloat32, ncclSum, &info) == ncclSuccess) bad++;
  if (b200collPlanDry(9, 1, 0, 1, ncclFloat32, ncclSum, &info) == ncclSuccess) bad++;
  if (b200collPlanDry(8, 1, 7, 1, ncclFloat32, ncclSum, &info) == ncclSuccess) bad++;
  if (b200collPlanDry(8, 1, 0, 1, (ncclDataType_t)99, ncclSum, &info) == ncclSuccess) bad++;
  if (b200collPlanDry(8, 1, 0, 1, ncclFloat32, ncclSum, nullptr) == ncclSuccess) bad++;
  size_t need = b200collDescribeSettings(nullptr, 0);
  std::string buf(need, 0);
  b200collDescribeSettings(&buf[0], need);
  char small[8];
  b200collDescribeSettings(small, sizeof(small));
  ncclUniqueId id;
  (void)id;
  printf("planner under sanitizers: %d bad, settings %zu bytes, version ok\n", bad, need);
  return bad ? 1 : 0;
}
