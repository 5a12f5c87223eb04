/*
 * b200tx — user range / marker annotations that land in the same trace as the collectives (the
 * role roctx plays next to the tracers of the reference: roctracer/src/roctx/roctx.cpp,
 * rocprofiler-sdk/source/lib/rocprofiler-sdk-roctx). Ranges nest per thread.
 */
#ifndef B200COLL_MARKERS_H_
#define B200COLL_MARKERS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  uint64_t id;         /* range id; 0 for a point marker */
  uint64_t beginNs;    /* CLOCK_MONOTONIC */
  uint64_t endNs;      /* == beginNs for a point marker */
  uint32_t tid;
  uint32_t depth;      /* nesting depth at the time the range was pushed */
  char message[96];
} b200tx_record_t;

void b200txMark(const char* message);
int b200txRangePush(const char* message);        /* returns the new nesting depth (0-based), -1 when disabled */
int b200txRangePop(void);                        /* returns the depth popped, -1 when nothing was open */
uint64_t b200txRangeStart(const char* message);  /* ranges that may end on another thread */
void b200txRangeStop(uint64_t id);
/* A range that is already over, with its times on CLOCK_MONOTONIC (for tools that decide afterwards what is worth
 * recording). Returns the range id, 0 when recording is off. */
uint64_t b200txRangeAt(const char* message, uint64_t beginNs, uint64_t endNs);
/* Recording is off until enabled (or B200COLL_TRACE=1 is in the environment). */
void b200txEnable(int on);
/* Copies up to `max` finished records; returns how many exist. */
uint64_t b200txGet(b200tx_record_t* out, uint64_t max);
void b200txClear(void);

/* Library version and build description (cf. rocm-core's getROCmVersion / rocm_version.cpp). */
const char* b200collBuildInfo(void);
/* File this library was loaded from and the prefix it is installed under (the directory above its lib/); 0 on success.
 * (cf. rocm-core's getROCmInstallPath.) Either buffer may be NULL. */
int b200collGetInstallPath(char* library, size_t libraryLen, char* prefix, size_t prefixLen);

#ifdef __cplusplus
}
#endif

#endif /* B200COLL_MARKERS_H_ */
