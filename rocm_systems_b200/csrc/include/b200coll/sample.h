/*
 * b200sample — call-stack sampling of host threads on CLOCK_MONOTONIC (csrc/prof/sampler.cc).
 * Preload libb200sample.so with B200SAMPLE_PREFIX set, or drive it from the program with the calls below.
 */
#ifndef B200COLL_SAMPLE_H_
#define B200COLL_SAMPLE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  B200SAMPLE_CPU = 0, /* ITIMER_PROF: samples go to threads in proportion to the CPU time they use */
  B200SAMPLE_WALL = 1 /* every thread is sampled every period, blocked ones included */
};

/* 0 on success; <0: already running (-1), bad argument (-2), no memory (-3), signal or timer set-up failed (-4, -5).
 * At most B200SAMPLE_MAX_SAMPLES samples (default 262144) are kept; later ones are counted as dropped. */
int b200sampleStart(double freqHz, int mode);
int b200sampleStartDelayed(double freqHz, int mode, double delaySeconds);
int b200sampleStop(void);
uint64_t b200sampleCount(void);
uint64_t b200sampleDropped(void);
void b200sampleClear(void); /* only while stopped */
/* Writes <prefix>.samples.csv (timestamp_ns,tid,depth,clock,"outer;...;leaf") and <prefix>.folded (one line per distinct
 * stack with its count, the input format of flame-graph tools). Returns the number of files written, <0 on error. */
int b200sampleWrite(const char* prefix);

#ifdef __cplusplus
}
#endif

#endif /* B200COLL_SAMPLE_H_ */
