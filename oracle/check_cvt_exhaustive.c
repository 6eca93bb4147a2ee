/*
 * check_cvt_exhaustive.c -- pin of the oracle's integer fp8 encoders and decoders.
 *
 * TEST INFRASTRUCTURE ONLY.  Walks the fp32 bit patterns (all 2^32 by default; every `stride`-th one, from a few
 * offsets, when a stride is given as the first argument) and compares
 * orc_f32_to_f8e4m3 / orc_f32_to_f8e5m2 (both overflow flavours) with the reference's
 * skl_cvt_f32_f8e4m3 / skl_cvt_f32_f8e5m2 (ref/cvt/cvt_ofp8.c:97-172) taken from the
 * compiled reference library, and all 256 codes of both decoders.  Prints the mismatch
 * count; exit status 0 means none.
 *
 *   make -C oracle check-cvt                 all 2^32 inputs (about a minute per format on 8 cores)
 *   make -C oracle check-cvt CVT_STRIDE=4099  a coarse sample in a second (what the CPU test suite runs)
 */
#include "skl_oracle.h"
#include <pthread.h>
#include <stdbool.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

float skl_cvt_f8e4m3_f32(uint8_t in);
float skl_cvt_f8e5m2_f32(uint8_t in);
uint8_t skl_cvt_f32_f8e4m3(float in, bool is_sat);
uint8_t skl_cvt_f32_f8e5m2(float in, bool is_sat);

static unsigned long long g_stride = 1;
static int g_threads = 1;
typedef struct {
  int index;
  unsigned long long bad, tried;
} job_t;

/* thread t takes the high half-words t, t + threads, ... */
static void *worker(void *arg) {
  job_t *j = (job_t *)arg;
  unsigned long long bad = 0, tried = 0;
  /* with a stride the low half-word starts at an offset that moves with the high one, so that over the run every
   * residue of the stride is visited and rounding boundaries (low mantissa bits) are not skipped systematically */
  for (unsigned long long hi = (unsigned long long)j->index; hi < 65536; hi += (unsigned long long)g_threads) {
    for (unsigned long long lo = hi % g_stride; lo < 65536; lo += g_stride) {
      unsigned u = ((unsigned)hi << 16) | (unsigned)lo;
      float x;
      memcpy(&x, &u, 4);
      ++tried;
      for (int sat = 0; sat < 2; ++sat) {
        bad += skl_cvt_f32_f8e4m3(x, sat) != orc_f32_to_f8e4m3(x, sat);
        bad += skl_cvt_f32_f8e5m2(x, sat) != orc_f32_to_f8e5m2(x, sat);
      }
    }
  }
  j->bad = bad;
  j->tried = tried;
  return 0;
}

int main(int argc, char **argv) {
  unsigned long long bad = 0, tried = 0;
  g_stride = argc > 1 ? strtoull(argv[1], 0, 10) : 1ull;
  if (g_stride == 0 || g_stride > 65536) {
    fprintf(stderr, "stride must be in 1..65536\n");
    return 2;
  }
  for (unsigned c = 0; c < 256; ++c) {
    float r0 = skl_cvt_f8e4m3_f32((uint8_t)c), o0 = orc_f8e4m3_to_f32((uint8_t)c);
    float r1 = skl_cvt_f8e5m2_f32((uint8_t)c), o1 = orc_f8e5m2_to_f32((uint8_t)c);
    bad += memcmp(&r0, &o0, 4) != 0;
    bad += memcmp(&r1, &o1, 4) != 0;
  }
  printf("decode mismatches: %llu\n", bad);
  long cores = sysconf(_SC_NPROCESSORS_ONLN);
  g_threads = cores < 1 ? 1 : (cores > 64 ? 64 : (int)cores);
  pthread_t th[64];
  job_t jobs[64];
  for (int t = 0; t < g_threads; ++t) {
    jobs[t].index = t;
    jobs[t].bad = jobs[t].tried = 0;
    if (pthread_create(&th[t], 0, worker, &jobs[t]) != 0) {
      fprintf(stderr, "pthread_create failed\n");
      return 2;
    }
  }
  for (int t = 0; t < g_threads; ++t) {
    pthread_join(th[t], 0);
    bad += jobs[t].bad;
    tried += jobs[t].tried;
  }
  printf("total mismatches over %llu inputs x 2 formats x 2 flavours: %llu\n", tried, bad);
  return bad != 0;
}
