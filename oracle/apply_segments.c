/*
 * CPU applier for the handoff oracle. TEST INFRASTRUCTURE ONLY: the product never links it.
 *
 * Performs the WRITE of a descriptor list the way the reference's transport
 * would on one host (vllm_rlt/pd/transport.py:187-199): for each (source
 * address, destination address, byte count) triple, copy the bytes. Triples are
 * dealt to worker threads round-robin in fixed-size pieces so that one very long
 * range does not serialise the copy. Used by the tests for large parity cases
 * and by the benchmark's CPU-baseline leg.
 */
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define PIECE (1 << 20)

typedef struct {
  const int64_t* seg; /* [count][3]: src address, dst address, bytes */
  int64_t count;
  int tid, threads;
} job_t;

static void* worker(void* arg) {
  job_t* j = (job_t*)arg;
  int64_t piece = 0;
  for (int64_t s = 0; s < j->count; ++s) {
    const char* src = (const char*)(uintptr_t)j->seg[3 * s];
    char* dst = (char*)(uintptr_t)j->seg[3 * s + 1];
    const int64_t n = j->seg[3 * s + 2];
    for (int64_t at = 0; at < n; at += PIECE, ++piece) {
      if (piece % j->threads != j->tid) continue;
      const int64_t m = n - at < PIECE ? n - at : PIECE;
      memcpy(dst + at, src + at, (size_t)m);
    }
  }
  return 0;
}

/* Returns bytes copied, or -1 on a bad argument. */
int64_t rlt_oracle_apply(const int64_t* seg, int64_t count, int threads) {
  if (seg == 0 || count < 0 || threads < 1 || threads > 1024) return -1;
  int64_t total = 0;
  for (int64_t s = 0; s < count; ++s) {
    if (seg[3 * s + 2] < 0) return -1;
    total += seg[3 * s + 2];
  }
  pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)threads);
  job_t* jobs = (job_t*)malloc(sizeof(job_t) * (size_t)threads);
  for (int t = 0; t < threads; ++t) {
    jobs[t].seg = seg;
    jobs[t].count = count;
    jobs[t].tid = t;
    jobs[t].threads = threads;
    if (t > 0) pthread_create(&th[t], 0, worker, &jobs[t]);
  }
  worker(&jobs[0]);
  for (int t = 1; t < threads; ++t) pthread_join(th[t], 0);
  free(th);
  free(jobs);
  return total;
}
