/*
 * b200causal — causal ("what if this function were faster") profiling of host code (csrc/prof/causal.cc).
 *
 * Preload libb200causal.so with B200CAUSAL_FILE set, mark progress in the program with the macros below, and read the
 * result with `python -m rocm_systems_b200.tools.causal report`. A program that includes this header needs no link
 * against the library: the calls look the entry points up at run time and do nothing when the library is not loaded.
 */
#ifndef B200COLL_CAUSAL_H_
#define B200COLL_CAUSAL_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  const char* file;          /* output, appended to (one block of lines per experiment) */
  const char* binaryScope;   /* regular expressions separated by ';' on the paths of loaded objects; "%MAIN%" = the executable */
  const char* functionScope; /* regular expressions on demangled function names; empty = every function in the binary scope */
  const char* functionExclude;
  const char* speedups;      /* "0,10,20,30": percentages to draw from */
  double freqHz;             /* SIGPROF rate on process CPU time */
  double experimentSeconds;  /* first length of an experiment; doubled while it sees too few visits of a progress point */
  double delaySeconds;       /* wait before the first experiment */
  double durationSeconds;    /* stop experimenting after this long; <= 0: until the program ends */
  int endToEnd;              /* one experiment over the whole run, its target and speed-up fixed when it starts */
  int resetFile;             /* truncate the file instead of appending */
  uint64_t seed;             /* 0: from the clock */
  int verbose;
  const char* backend;       /* "auto" (default: perf, else timer), "perf" (per-thread CPU-clock events), "timer" (ITIMER_PROF) */
  const char* sourceRanges;  /* source-line scope: file of "<name>\t<lo>-<hi>,..." (hex addresses of the executable's ELF file); replaces the function scope */
} b200causalConfig_t;

/* 0 on success; -1 already running, -2 bad argument, -3 nothing in scope, -4 signal or timer set-up failed. */
int b200causalStart(const b200causalConfig_t* cfg);
/* Ends the running experiment, writes what was measured and removes the timer. */
int b200causalStop(void);
int b200causalActive(void);
uint64_t b200causalExperiments(void); /* experiments finished so far */

/* Throughput point: one visit. Latency point: begin / end of one item in flight. Names are compared as strings. */
void b200causalProgress(const char* name);
void b200causalBegin(const char* name);
void b200causalEnd(const char* name);

#ifdef __cplusplus
}
#endif

/* ---- for instrumented programs: no link-time dependency ---- */
#if !defined(B200CAUSAL_NO_MACROS)
#include <dlfcn.h>
typedef void (*b200causalPointFn_)(const char*);
static inline void b200causalCall_(const char* symbol, const char* name, b200causalPointFn_* slot, int* looked) {
  if (!*looked) {
    *slot = (b200causalPointFn_)dlsym(RTLD_DEFAULT, symbol);
    *looked = 1;
  }
  if (*slot) (*slot)(name);
}
#define B200CAUSAL_STR2_(x) #x
#define B200CAUSAL_STR_(x) B200CAUSAL_STR2_(x)
#define B200CAUSAL_POINT_(symbol, name)                          \
  do {                                                           \
    static b200causalPointFn_ fn_ = 0;                           \
    static int looked_ = 0;                                      \
    b200causalCall_(symbol, name, &fn_, &looked_);               \
  } while (0)
#define B200CAUSAL_PROGRESS_NAMED(name) B200CAUSAL_POINT_("b200causalProgress", name)
#define B200CAUSAL_PROGRESS B200CAUSAL_PROGRESS_NAMED(__FILE__ ":" B200CAUSAL_STR_(__LINE__))
#define B200CAUSAL_BEGIN(name) B200CAUSAL_POINT_("b200causalBegin", name)
#define B200CAUSAL_END(name) B200CAUSAL_POINT_("b200causalEnd", name)
#endif

#endif /* B200COLL_CAUSAL_H_ */
