/*
 * check_cvt_exhaustive.c -- one-off pin of the oracle's integer fp8 encoders and decoders.
 *
 * TEST INFRASTRUCTURE ONLY.  Walks all 2^32 fp32 bit patterns and compares
 * orc_f32_to_f8e4m3 / orc_f32_to_f8e5m2 (both overflow flavours) with the reference's
 * skl_cvt_f32_f8e4m3 / skl_cvt_f32_f8e5m2 (ref/cvt/cvt_ofp8.c:97-172) taken from the
 * compiled reference library, and all 256 codes of both decoders.  Prints the mismatch
 * count; exit status 0 means none.
 *
 *   make -C oracle all
 *   gcc -O2 -fopenmp oracle/check_cvt_exhaustive.c -Ioracle -Loracle -Loracle/_ref \
 *       -loracle -lskl-ref -lm -Wl,-rpath,$PWD/oracle -Wl,-rpath,$PWD/oracle/_ref -o /tmp/check_cvt
 *   /tmp/check_cvt            (about a minute per format on 8 cores)
 */
#include "skl_oracle.h"
#include <stdbool.h>
#include <stdio.h>
#include <string.h>

float skl_cvt_f8e4m3_f32(uint8_t in);
float skl_cvt_f8e5m2_f32(uint8_t in);
uint8_t skl_cvt_f32_f8e4m3(float in, bool is_sat);
uint8_t skl_cvt_f32_f8e5m2(float in, bool is_sat);

int main(void) {
  unsigned long long bad = 0;
  for (unsigned c = 0; c < 256; ++c) {
    float r0 = skl_cvt_f8e4m3_f32((uint8_t)c), o0 = orc_f8e4m3_to_f32((uint8_t)c);
    float r1 = skl_cvt_f8e5m2_f32((uint8_t)c), o1 = orc_f8e5m2_to_f32((uint8_t)c);
    bad += memcmp(&r0, &o0, 4) != 0;
    bad += memcmp(&r1, &o1, 4) != 0;
  }
  printf("decode mismatches: %llu\n", bad);
#pragma omp parallel for reduction(+ : bad) schedule(static)
  for (long long hi = 0; hi < 65536; ++hi) {
    for (unsigned lo = 0; lo < 65536; ++lo) {
      unsigned u = ((unsigned)hi << 16) | lo;
      float x;
      memcpy(&x, &u, 4);
      for (int sat = 0; sat < 2; ++sat) {
        bad += skl_cvt_f32_f8e4m3(x, sat) != orc_f32_to_f8e4m3(x, sat);
        bad += skl_cvt_f32_f8e5m2(x, sat) != orc_f32_to_f8e5m2(x, sat);
      }
    }
  }
  printf("total mismatches over 2^32 inputs x 2 formats x 2 flavours: %llu\n", bad);
  return bad != 0;
}
