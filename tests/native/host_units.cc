// Host-side units under sanitizers: the JSON reader of the tuning table against valid, truncated, mutated and
// deeply nested texts, and the range/marker recorder from many threads at once.
//   host_units json | markers
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <string>
#include <thread>
#include <vector>

#include "b200coll/markers.h"
#include "core/json.h"

using b200::JsonParser;
using b200::JsonValue;

static uint64_t rng(uint64_t& s) {
  s ^= s << 13;
  s ^= s >> 7;
  s ^= s << 17;
  return s;
}

static int fail(const char* what) {
  fprintf(stderr, "FAILED: %s\n", what);
  return 1;
}

static int testJson() {
  const std::string doc =
      "{ \"rows\": [ {\"coll\": \"all_reduce\", \"max_bytes\": 65536, \"algo\": \"ll\", \"ctas\": 8},\n"
      "  {\"coll\": \"all_gather\", \"max_bytes\": 1e9, \"algo\": \"p2p\", \"ctas\": 32, \"note\": \"a \\\"quoted\\\" word\\n\"} ],\n"
      "  \"enabled\": true, \"nothing\": null, \"neg\": -2.5, \"empty\": {}, \"none\": [] }";
  JsonValue v;
  if (!JsonParser(doc).parse(&v) || v.kind != JsonValue::Object) return fail("valid document refused");
  const JsonValue* rows = v.get("rows");
  if (!rows || rows->kind != JsonValue::Array || rows->arr.size() != 2) return fail("rows");
  if (rows->arr[0].stringOr("algo", "") != "ll" || rows->arr[0].numberOr("ctas", 0) != 8) return fail("row 0");
  if (rows->arr[1].numberOr("max_bytes", 0) != 1e9 || rows->arr[1].stringOr("note", "") != "a \"quoted\" word\n") return fail("row 1");
  if (!v.get("enabled")->b || v.get("nothing")->kind != JsonValue::Null || v.numberOr("neg", 0) != -2.5) return fail("scalars");
  if (v.numberOr("missing", 7) != 7 || v.stringOr("neg", "d") != "d") return fail("defaults");
  // Every prefix is either refused or (never, for this text) accepted; none may crash or read out of bounds.
  for (size_t n = 0; n < doc.size(); n++) {
    JsonValue x;
    const std::string cut = doc.substr(0, n);
    if (JsonParser(cut).parse(&x)) return fail("a truncated document was accepted");
  }
  // Random mutations: result does not matter, only that parsing ends without a sanitizer report.
  uint64_t s = 0x1234567;
  int accepted = 0;
  for (int it = 0; it < 20000; it++) {
    std::string m = doc;
    const int edits = 1 + (int)(rng(s) % 4);
    for (int e = 0; e < edits; e++) {
      const size_t pos = rng(s) % m.size();
      switch (rng(s) % 4) {
        case 0: m[pos] = (char)(rng(s) & 0xff); break;
        case 1: m.erase(pos, 1 + rng(s) % 5); break;
        case 2: m.insert(pos, 1, "{}[]\",:\\ 0e-"[rng(s) % 13]); break;
        default: m.insert(pos, m.substr(rng(s) % m.size(), rng(s) % 16)); break;
      }
      if (m.empty()) m = "x";
    }
    JsonValue x;
    accepted += JsonParser(m).parse(&x) ? 1 : 0;
  }
  // Nesting: 64 levels are read, 100000 are refused instead of overflowing the stack.
  {
    JsonValue x;
    if (!JsonParser(std::string(60, '[') + std::string(60, ']')).parse(&x)) return fail("60 levels refused");
    if (JsonParser(std::string(100000, '[') + std::string(100000, ']')).parse(&x)) return fail("100000 levels accepted");
    if (JsonParser(std::string(100000, '{')).parse(&x)) return fail("unterminated objects accepted");
  }
  printf("json OK (%d of 20000 mutated documents still parsed)\n", accepted);
  return 0;
}

static int testMarkers() {
  b200txEnable(1);
  b200txClear();
  constexpr int kThreads = 8, kIters = 2000;
  std::atomic<uint64_t> crossIds[kThreads];
  for (auto& c : crossIds) c.store(0);
  std::vector<std::thread> th;
  for (int t = 0; t < kThreads; t++)
    th.emplace_back([&, t]() {
      char name[64];
      for (int i = 0; i < kIters; i++) {
        snprintf(name, sizeof(name), "t%d.i%d", t, i);
        if (b200txRangePush(name) != 0) abort();
        if (b200txRangePush("inner") != 1) abort();
        b200txMark("tick");
        if (b200txRangePop() != 1) abort();
        if (b200txRangePop() != 0) abort();
        // A range started here is stopped by the next thread, as ranges that end on another thread do.
        const uint64_t mine = b200txRangeStart(name);
        const uint64_t other = crossIds[(t + 1) % kThreads].exchange(0);
        if (other) b200txRangeStop(other);
        const uint64_t prev = crossIds[t].exchange(mine);
        if (prev) b200txRangeStop(prev);
      }
    });
  for (auto& x : th) x.join();
  for (auto& c : crossIds)
    if (uint64_t id = c.exchange(0)) b200txRangeStop(id);
  if (b200txRangePop() != -1) return fail("pop on an empty stack");
  const uint64_t want = (uint64_t)kThreads * kIters * 4;  // outer + inner + mark + started range
  const uint64_t have = b200txGet(nullptr, 0);
  if (have != want) {
    fprintf(stderr, "records: have %llu want %llu\n", (unsigned long long)have, (unsigned long long)want);
    return 1;
  }
  std::vector<b200tx_record_t> recs(have);
  b200txGet(recs.data(), have);
  for (const auto& r : recs)
    if (r.endNs < r.beginNs || r.message[0] == 0) return fail("bad record");
  b200txClear();
  if (b200txGet(nullptr, 0) != 0) return fail("clear");
  printf("markers OK (%llu records from %d threads)\n", (unsigned long long)have, kThreads);
  return 0;
}

int main(int argc, char** argv) {
  const std::string what = argc > 1 ? argv[1] : "all";
  int rc = 0;
  if (what == "json" || what == "all") rc |= testJson();
  if (what == "markers" || what == "all") rc |= testMarkers();
  return rc;
}
