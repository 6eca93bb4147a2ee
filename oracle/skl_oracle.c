/*
 * skl_oracle.c -- CPU restatement of the SKL gemm / pack / cvt semantics.
 *
 * TEST INFRASTRUCTURE ONLY (see skl_oracle.h).  Plain C, single-threaded, written for clarity;
 * the callers thread it over disjoint row slabs when they need speed.
 *
 * The fp8 encoders are stated with integer arithmetic on the fp32 bit pattern (round to nearest
 * even on the discarded bits) instead of the reference's log2f / powf / nearbyintf formulation
 * (ref/cvt/cvt_ofp8.c:97-172); the two agree on every one of the 2^32 fp32 inputs for both formats
 * and both overflow flavours (checked exhaustively by oracle/check_cvt_exhaustive.c against the
 * compiled reference).
 */
#include "skl_oracle.h"

#include <math.h>
#include <string.h>

/* ------------------------------------------------------------------ bit casts */
static inline uint32_t f32_bits(float x) {
  uint32_t u;
  memcpy(&u, &x, sizeof u);
  return u;
}
static inline float bits_f32(uint32_t u) {
  float x;
  memcpy(&x, &u, sizeof x);
  return x;
}

/* Shift right by s >= 1 bits rounding to nearest, ties to even.  s may exceed 31. */
static inline uint32_t shr_rne(uint32_t v, int s) {
  if (s > 31) {
    return 0; /* v < 2^31 always here, so v / 2^s < 1/2 */
  }
  uint32_t q = v >> s;
  uint32_t rem = v & ((1u << s) - 1u);
  uint32_t half = 1u << (s - 1);
  if (rem > half || (rem == half && (q & 1u))) {
    q += 1u;
  }
  return q;
}

/* ------------------------------------------------------------------ fp8 -> fp32 */
/* ref/cvt/cvt_ofp8.c:18-52.  S.EEEE.MMM, bias 7, no infinity, one NaN magnitude (0x7F) which
 * the reference maps to the positive quiet NaN 0x7FC00000 whatever the sign bit says. */
float orc_f8e4m3_to_f32(uint8_t code) {
  uint32_t sign = (uint32_t)(code & 0x80u) << 24;
  uint32_t e = (code >> 3) & 0xFu;
  uint32_t m = code & 0x7u;
  if (e == 0xFu && m == 0x7u) {
    return bits_f32(0x7FC00000u);
  }
  if (e == 0) {
    /* m * 2^-9: exact in fp32; built as an integer-to-float conversion times a power of two */
    float mag = (float)m * bits_f32((uint32_t)(127 - 9) << 23);
    return bits_f32(f32_bits(mag) | sign);
  }
  return bits_f32(sign | ((e + 120u) << 23) | (m << 20));
}

/* ref/cvt/cvt_ofp8.c:54-95.  S.EEEEE.MM, bias 15, IEEE-style Inf (mantissa 0) and NaN; every NaN
 * code becomes +qNaN, infinities keep their sign. */
float orc_f8e5m2_to_f32(uint8_t code) {
  uint32_t sign = (uint32_t)(code & 0x80u) << 24;
  uint32_t e = (code >> 2) & 0x1Fu;
  uint32_t m = code & 0x3u;
  if (e == 0x1Fu) {
    return bits_f32(m == 0 ? (sign | 0x7F800000u) : 0x7FC00000u);
  }
  if (e == 0) {
    float mag = (float)m * bits_f32((uint32_t)(127 - 16) << 23); /* m * 2^-16 */
    return bits_f32(f32_bits(mag) | sign);
  }
  return bits_f32(sign | ((e + 112u) << 23) | (m << 21));
}

/* ------------------------------------------------------------------ fp32 -> fp8 */
/* Shared encoder.  mbits: mantissa bits (3 / 2); bias (7 / 15); max_code: largest finite magnitude
 * code (0x7E / 0x7B); over: code returned (sign already applied by the caller's choice) when the
 * rounded magnitude exceeds max_code or the input is infinite. */
static uint8_t encode_f8(float x, int mbits, int bias, uint32_t max_code, uint8_t over) {
  uint32_t u = f32_bits(x);
  uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
  uint32_t au = u & 0x7FFFFFFFu;
  if (au > 0x7F800000u) {
    return 0x7Fu; /* NaN in: the reference always answers 0x7F (cvt_ofp8.c:113-115,151-153) */
  }
  if (au == 0x7F800000u) {
    return over;
  }
  uint32_t be = au >> 23; /* biased fp32 exponent */
  if (be == 0) {
    return sign; /* zero and fp32 subnormals are far below half the smallest fp8 subnormal */
  }
  int e = (int)be - 127;
  uint32_t sig = (au & 0x7FFFFFu) | 0x800000u; /* 1.f as a 24-bit integer, value = sig * 2^(e-23) */
  int emin = 1 - bias;
  if (e < emin) {
    /* target subnormal: code = RNE(|x| * 2^(mbits - emin)); a carry to 2^mbits is the smallest normal */
    uint32_t q = shr_rne(sig, 23 - mbits + (emin - e));
    return (uint8_t)(sign | q);
  }
  uint32_t q = shr_rne(sig & 0x7FFFFFu, 23 - mbits); /* 0 .. 2^mbits, carry propagates into the exponent */
  uint32_t mag = ((uint32_t)(e + bias) << mbits) + q;
  if (e + bias > 0x7F >> mbits || mag > max_code) {
    return over;
  }
  return (uint8_t)(sign | mag);
}

/* ref/cvt/cvt_ofp8.c:97-134.  Overflow and +-Inf: saturating flavour gives sign|0x7E, the other one
 * gives the NaN code 0x7F with the sign dropped. */
uint8_t orc_f32_to_f8e4m3(float x, int saturate) {
  uint8_t sign = (uint8_t)((f32_bits(x) >> 24) & 0x80u);
  return encode_f8(x, 3, 7, 0x7Eu, saturate ? (uint8_t)(sign | 0x7Eu) : (uint8_t)0x7Fu);
}

/* ref/cvt/cvt_ofp8.c:136-172.  Overflow and +-Inf: saturating gives sign|0x7B, else sign|0x7C (Inf). */
uint8_t orc_f32_to_f8e5m2(float x, int saturate) {
  uint8_t sign = (uint8_t)((f32_bits(x) >> 24) & 0x80u);
  return encode_f8(x, 2, 15, 0x7Bu, (uint8_t)(sign | (saturate ? 0x7Bu : 0x7Cu)));
}

/* ------------------------------------------------------------------ 16-bit floats */
float orc_bf16_to_f32(uint16_t bits) { return bits_f32((uint32_t)bits << 16); }

/* Round to nearest even on the low 16 bits; NaN keeps sign and top payload bits and is quieted,
 * which is what gcc's (__bf16) cast does on x86-64. */
uint16_t orc_f32_to_bf16(float x) {
  uint32_t u = f32_bits(x);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) {
    return (uint16_t)((u >> 16) | 0x0040u);
  }
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

float orc_f16_to_f32(uint16_t bits) {
  uint32_t sign = (uint32_t)(bits & 0x8000u) << 16;
  uint32_t e = (bits >> 10) & 0x1Fu;
  uint32_t m = bits & 0x3FFu;
  if (e == 0x1Fu) {
    return bits_f32(sign | 0x7F800000u | (m << 13));
  }
  if (e == 0) {
    float mag = (float)m * bits_f32((uint32_t)(127 - 24) << 23); /* m * 2^-24, exact */
    return bits_f32(f32_bits(mag) | sign);
  }
  return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
}

uint16_t orc_f32_to_f16(float x) {
  uint32_t u = f32_bits(x);
  uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  uint32_t au = u & 0x7FFFFFFFu;
  if (au > 0x7F800000u) {
    return (uint16_t)(sign | 0x7E00u | ((au >> 13) & 0x3FFu));
  }
  if (au >= 0x47800000u) { /* >= 65536: Inf in, or overflow after rounding handled below */
    return (uint16_t)(sign | 0x7C00u);
  }
  int e = (int)(au >> 23) - 127;
  if (e < -25) {
    return sign;
  }
  uint32_t sig = (au & 0x7FFFFFu) | 0x800000u;
  if (e < -14) {
    return (uint16_t)(sign | shr_rne(sig, 13 + (-14 - e)));
  }
  uint32_t mag = ((uint32_t)(e + 15) << 10) + shr_rne(sig & 0x7FFFFFu, 13);
  return (uint16_t)(sign | (mag > 0x7C00u ? 0x7C00u : mag));
}

/* ref/cvt/cvt_ofp4.c:18-60: E2M1 nibble -> fp32 -> non-saturating E4M3 (every E2M1 value is exact). */
uint8_t orc_f4e2m1_to_f8e4m3(uint8_t nibble) {
  static const float mags[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  float v = mags[nibble & 7u];
  if (nibble & 8u) {
    v = -v;
  }
  return orc_f32_to_f8e4m3(v, 0);
}

/* ------------------------------------------------------------------ array conversions */
/* ref/cvt/cvt_ofp8.c:174-200: dst[i] = encode(src[i] * scale), the product rounded to fp32 first. */
void orc_cvt_f32_f8(uint8_t *dst, const float *src, float scale, size_t n, int fmt, int saturate) {
  for (size_t i = 0; i < n; ++i) {
    volatile float scaled = src[i] * scale; /* volatile: one fp32 rounding, never fused or widened */
    dst[i] = (fmt == ORC_F8E4M3) ? orc_f32_to_f8e4m3(scaled, saturate)
                                 : orc_f32_to_f8e5m2(scaled, saturate);
  }
}

/* ref/cvt/cvt_ofp8.c:202-228: the bf16 source is widened to fp32 before the multiply. */
void orc_cvt_bf16_f8(uint8_t *dst, const uint16_t *src, float scale, size_t n, int fmt,
                     int saturate) {
  for (size_t i = 0; i < n; ++i) {
    volatile float scaled = orc_bf16_to_f32(src[i]) * scale;
    dst[i] = (fmt == ORC_F8E4M3) ? orc_f32_to_f8e4m3(scaled, saturate)
                                 : orc_f32_to_f8e5m2(scaled, saturate);
  }
}

/* ref/cvt/cvt_ofp8.c:230-242: decode then narrow to bf16 (exact for every non-NaN code). */
void orc_cvt_f8_bf16(uint16_t *dst, const uint8_t *src, size_t n, int fmt) {
  for (size_t i = 0; i < n; ++i) {
    float v = (fmt == ORC_F8E4M3) ? orc_f8e4m3_to_f32(src[i]) : orc_f8e5m2_to_f32(src[i]);
    dst[i] = orc_f32_to_bf16(v);
  }
}

/* ref/cvt/cvt_ofp4.c:62-72: two nibbles per source byte, low nibble first; odd n uses the low
 * nibble of the last byte only. */
void orc_cvt_f4e2m1_f8e4m3(uint8_t *dst, const uint8_t *src, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    uint8_t byte = src[i / 2];
    dst[i] = orc_f4e2m1_to_f8e4m3((i & 1u) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0xFu));
  }
}

/* ------------------------------------------------------------------ operand decode */
static inline float load_fp(int t, const void *p, size_t idx) {
  switch (t) {
  case ORC_BF16:
    return orc_bf16_to_f32(((const uint16_t *)p)[idx]);
  case ORC_F16:
    return orc_f16_to_f32(((const uint16_t *)p)[idx]);
  case ORC_F8E4M3:
    return orc_f8e4m3_to_f32(((const uint8_t *)p)[idx]);
  case ORC_F8E5M2:
    return orc_f8e5m2_to_f32(((const uint8_t *)p)[idx]);
  default:
    return ((const float *)p)[idx];
  }
}

/* ------------------------------------------------------------------ GEMM, plain strides */
/* ref/gemm/gemm_i8rc_i8rc_i32rc.c:10-26.  Unsigned arithmetic gives the two's-complement
 * wrap-around the reference gets from its int32 expression on every supported target. */
void orc_gemm_i8_i32(size_t m, size_t n, size_t k, int32_t alpha, const int8_t *a, size_t rsa,
                     size_t csa, const int8_t *b, size_t rsb, size_t csb, int32_t beta, int32_t *c,
                     size_t rsc, size_t csc) {
  for (size_t i = 0; i < m; ++i) {
    for (size_t j = 0; j < n; ++j) {
      uint32_t acc = 0;
      const int8_t *ap = a + i * rsa;
      const int8_t *bp = b + j * csb;
      for (size_t p = 0; p < k; ++p) {
        acc += (uint32_t)((int32_t)ap[p * csa] * (int32_t)bp[p * rsb]);
      }
      int32_t *cp = c + i * rsc + j * csc;
      *cp = (int32_t)((uint32_t)beta * (uint32_t)*cp + (uint32_t)alpha * acc);
    }
  }
}

/* ref/gemm/gemm_bf16rc_bf16rc_f32rc.c:9-24 and siblings: fp32 product, one fp32 accumulator,
 * k ascending, then beta*c + alpha*acc with a rounding after each operation. */
void orc_gemm_fp_f32(size_t m, size_t n, size_t k, float alpha, int ta, const void *a, size_t rsa,
                     size_t csa, int tb, const void *b, size_t rsb, size_t csb, float beta, float *c,
                     size_t rsc, size_t csc) {
  for (size_t i = 0; i < m; ++i) {
    for (size_t j = 0; j < n; ++j) {
      float acc = 0.0f;
      for (size_t p = 0; p < k; ++p) {
        float prod = load_fp(ta, a, i * rsa + p * csa) * load_fp(tb, b, p * rsb + j * csb);
        acc = acc + prod;
      }
      float *cp = c + i * rsc + j * csc;
      float left = beta * *cp;
      float right = alpha * acc;
      *cp = left + right;
    }
  }
}

/* ------------------------------------------------------------------ GEMM, packed operands */
/* ref/gemm/gemm_i8rcprc_i8rcprc_i32rcprc.c:10-37: blocks (ii1, jj1) of m0 x n0 outputs; the
 * contraction walks k1 blocks of k0 elements, i.e. k ascending as in the plain routine. */
void orc_gemm_packed_i8_i32(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1,
                            int32_t alpha, const int8_t *a, size_t rsa0, size_t csa0, size_t rsa1,
                            size_t csa1, const int8_t *b, size_t rsb0, size_t csb0, size_t rsb1,
                            size_t csb1, int32_t beta, int32_t *c, size_t rsc0, size_t csc0,
                            size_t rsc1, size_t csc1) {
  for (size_t bi = 0; bi < m1; ++bi) {
    for (size_t bj = 0; bj < n1; ++bj) {
      for (size_t i = 0; i < m0; ++i) {
        for (size_t j = 0; j < n0; ++j) {
          uint32_t acc = 0;
          for (size_t bp = 0; bp < k1; ++bp) {
            const int8_t *ap = a + bi * rsa1 + bp * csa1 + i * rsa0;
            const int8_t *bq = b + bp * rsb1 + bj * csb1 + j * csb0;
            for (size_t p = 0; p < k0; ++p) {
              acc += (uint32_t)((int32_t)ap[p * csa0] * (int32_t)bq[p * rsb0]);
            }
          }
          int32_t *cp = c + bi * rsc1 + bj * csc1 + i * rsc0 + j * csc0;
          *cp = (int32_t)((uint32_t)beta * (uint32_t)*cp + (uint32_t)alpha * acc);
        }
      }
    }
  }
}

/* ref/gemm/gemm_bf16rcprc_bf16rcprc_f32rcprc.c:9-36 and the f16 / f8e4m3 / f8e5m2 siblings. */
void orc_gemm_packed_fp_f32(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1,
                            float alpha, int ta, const void *a, size_t rsa0, size_t csa0,
                            size_t rsa1, size_t csa1, int tb, const void *b, size_t rsb0,
                            size_t csb0, size_t rsb1, size_t csb1, float beta, float *c,
                            size_t rsc0, size_t csc0, size_t rsc1, size_t csc1) {
  for (size_t bi = 0; bi < m1; ++bi) {
    for (size_t bj = 0; bj < n1; ++bj) {
      for (size_t i = 0; i < m0; ++i) {
        for (size_t j = 0; j < n0; ++j) {
          float acc = 0.0f;
          for (size_t bp = 0; bp < k1; ++bp) {
            size_t abase = bi * rsa1 + bp * csa1 + i * rsa0;
            size_t bbase = bp * rsb1 + bj * csb1 + j * csb0;
            for (size_t p = 0; p < k0; ++p) {
              float prod = load_fp(ta, a, abase + p * csa0) * load_fp(tb, b, bbase + p * rsb0);
              acc = acc + prod;
            }
          }
          float *cp = c + bi * rsc1 + bj * csc1 + i * rsc0 + j * csc0;
          float left = beta * *cp;
          float right = alpha * acc;
          *cp = left + right;
        }
      }
    }
  }
}

/* ref/gemm/gemm_f64rcprc_f64rcprc_f64rcprc.c (and, with one block per dimension, gemm_f64rc_f64rc_f64rc.c:9-22) */
void orc_gemm_f64(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1, double alpha, const double *a,
                  size_t rsa0, size_t csa0, size_t rsa1, size_t csa1, const double *b, size_t rsb0, size_t csb0,
                  size_t rsb1, size_t csb1, double beta, double *c, size_t rsc0, size_t csc0, size_t rsc1,
                  size_t csc1) {
  for (size_t bi = 0; bi < m1; ++bi) {
    for (size_t bj = 0; bj < n1; ++bj) {
      for (size_t i = 0; i < m0; ++i) {
        for (size_t j = 0; j < n0; ++j) {
          double acc = 0.0;
          for (size_t bp = 0; bp < k1; ++bp) {
            size_t abase = bi * rsa1 + bp * csa1 + i * rsa0;
            size_t bbase = bp * rsb1 + bj * csb1 + j * csb0;
            for (size_t p = 0; p < k0; ++p) {
              double prod = a[abase + p * csa0] * b[bbase + p * rsb0];
              acc = acc + prod;
            }
          }
          double *cp = c + bi * rsc1 + bj * csc1 + i * rsc0 + j * csc0;
          double left = beta * *cp;
          double right = alpha * acc;
          *cp = left + right;
        }
      }
    }
  }
}

/* ref/gemm/gemm_f16rcprc_f16rcprc_f16rcprc.c (and, with one block per dimension, gemm_f16rc_f16rc_f16rc.c:9-22):
 * fp16 operands, accumulator, scalars and C.  Each statement of the reference -- `acc += a*b`,
 * `c = beta*c + alpha*acc` -- is evaluated in fp32 and rounded to fp16 once, which is what a compiler without native
 * half-precision arithmetic makes of the `_Float16` source (the product of two fp16 values is exact in fp32).
 * fp16 values travel as bit patterns; alpha and beta are floats holding fp16-representable values. */
void orc_gemm_f16acc(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1, float alpha,
                     const uint16_t *a, size_t rsa0, size_t csa0, size_t rsa1, size_t csa1, const uint16_t *b,
                     size_t rsb0, size_t csb0, size_t rsb1, size_t csb1, float beta, uint16_t *c, size_t rsc0,
                     size_t csc0, size_t rsc1, size_t csc1) {
  const float alpha_h = orc_f16_to_f32(orc_f32_to_f16(alpha)), beta_h = orc_f16_to_f32(orc_f32_to_f16(beta));
  for (size_t bi = 0; bi < m1; ++bi) {
    for (size_t bj = 0; bj < n1; ++bj) {
      for (size_t i = 0; i < m0; ++i) {
        for (size_t j = 0; j < n0; ++j) {
          float acc = 0.0f; /* always an fp16-representable value */
          for (size_t bp = 0; bp < k1; ++bp) {
            size_t abase = bi * rsa1 + bp * csa1 + i * rsa0;
            size_t bbase = bp * rsb1 + bj * csb1 + j * csb0;
            for (size_t p = 0; p < k0; ++p) {
              float prod = orc_f16_to_f32(a[abase + p * csa0]) * orc_f16_to_f32(b[bbase + p * rsb0]);
              float sum = acc + prod;
              acc = orc_f16_to_f32(orc_f32_to_f16(sum));
            }
          }
          uint16_t *cp = c + bi * rsc1 + bj * csc1 + i * rsc0 + j * csc0;
          float left = beta_h * orc_f16_to_f32(*cp);
          float right = alpha_h * acc;
          float sum = left + right;
          *cp = orc_f32_to_f16(sum);
        }
      }
    }
  }
}

/* ------------------------------------------------------------------ extended epilogue */
static inline float load_c(int tc, const void *c, size_t idx) {
  if (tc == ORC_I8) {
    return (float)((const int8_t *)c)[idx];
  }
  if (tc == ORC_F8E4M3) {
    return orc_f8e4m3_to_f32(((const uint8_t *)c)[idx]);
  }
  return load_fp(tc, c, idx);
}

static inline void store_c(int tc, void *c, size_t idx, float v) {
  switch (tc) {
  case ORC_BF16:
    ((uint16_t *)c)[idx] = orc_f32_to_bf16(v);
    break;
  case ORC_F16:
    ((uint16_t *)c)[idx] = orc_f32_to_f16(v);
    break;
  case ORC_F8E4M3:
    ((uint8_t *)c)[idx] = orc_f32_to_f8e4m3(v, 1);
    break;
  case ORC_I8: { /* requantised output: nearest even, saturating, NaN -> 0 (no reference routine) */
    float r = nearbyintf(v);
    int q = isnan(v) ? 0 : (r < -128.0f ? -128 : (r > 127.0f ? 127 : (int)r));
    ((int8_t *)c)[idx] = (int8_t)q;
    break;
  }
  default:
    ((float *)c)[idx] = v;
    break;
  }
}

/* ref/sigmoid/sigmoid_f32.c:10-28 (logistic in double, times the linear unit, times the gate, one final
 * rounding) and ref/gelu/gelu_f32.c:12-22 (relu plus a double-precision erfc offset), for one element. */
float orc_activation(int act, float p, float v, float up) {
  switch (act) {
  case ORC_ACT_LOGISTIC:
  case ORC_ACT_SWISH:
  case ORC_ACT_SWIGLU: {
    const float beta = (act == ORC_ACT_SWIGLU) ? 1.0f : p;
    const double x = v;
    double o = 1. / (1. + exp(-beta * x));
    if (act != ORC_ACT_LOGISTIC) {
      o *= v;
    }
    if (act == ORC_ACT_SWIGLU) {
      o *= (up + p);
    }
    return (float)o;
  }
  case ORC_ACT_GELU: {
    const double sqrt2 = 0x1.6a09e667f3bcdp0;
    float b = (v > 0) ? v : -0.f;
    float h = -0.5f * fabsf(v);
    double e = erfc(-sqrt2 * h);
    double g = fma(h, e, b);
    return (float)g;
  }
  default:
    return v;
  }
}

void orc_gemm_fused(size_t m, size_t n, size_t k, int ta, const void *a, size_t rsa, size_t csa, int tb,
                    const void *b, size_t rsb, size_t csb, float alpha, const float *row_scale,
                    const float *col_scale, const float *bias, float *global_max, float beta, int activation,
                    float act_param, int tc, void *c, size_t rsc, size_t csc) {
  for (size_t i = 0; i < m; ++i) {
    for (size_t j = 0; j < n; ++j) {
      float v;
      if (ta == ORC_I8) {
        uint32_t acc = 0;
        const int8_t *ap = (const int8_t *)a + i * rsa;
        const int8_t *bp = (const int8_t *)b + j * csb;
        for (size_t p = 0; p < k; ++p) {
          acc += (uint32_t)((int32_t)ap[p * csa] * (int32_t)bp[p * rsb]);
        }
        v = (float)(int32_t)acc;
      } else {
        float acc = 0.0f;
        for (size_t p = 0; p < k; ++p) {
          float prod = load_fp(ta, a, i * rsa + p * csa) * load_fp(tb, b, p * rsb + j * csb);
          acc = acc + prod;
        }
        v = acc;
      }
      v = alpha * v;
      if (row_scale) {
        v = v * row_scale[i];
      }
      if (col_scale) {
        v = v * col_scale[j];
      }
      if (bias) {
        v = v + bias[j];
      }
      size_t idx = i * rsc + j * csc;
      if (beta != 0.0f) {
        float left = beta * load_c(tc, c, idx);
        v = left + v;
      }
      if (activation != ORC_ACT_NONE) {
        v = orc_activation(activation, act_param, v, activation == ORC_ACT_SWIGLU ? load_c(tc, c, idx) : 0.0f);
      }
      if (global_max && v > *global_max) { /* false for NaN, as in the reference's example kernel */
        *global_max = v;
      }
      store_c(tc, c, idx, v);
    }
  }
}

void orc_gemm_ex(size_t m, size_t n, size_t k, int ta, const void *a, size_t rsa, size_t csa, int tb,
                 const void *b, size_t rsb, size_t csb, float alpha, const float *row_scale,
                 const float *col_scale, float beta, int tc, void *c, size_t rsc, size_t csc) {
  orc_gemm_fused(m, n, k, ta, a, rsa, csa, tb, b, rsb, csb, alpha, row_scale, col_scale, 0, 0, beta, ORC_ACT_NONE, 0.0f, tc, c,
                 rsc, csc);
}

/* ------------------------------------------------------------------ pack / unpack / transpose */
static inline void copy_elem(size_t esize, void *dst, size_t di, const void *src, size_t si) {
  switch (esize) {
  case 1:
    ((uint8_t *)dst)[di] = ((const uint8_t *)src)[si];
    break;
  case 2:
    ((uint16_t *)dst)[di] = ((const uint16_t *)src)[si];
    break;
  default:
    ((uint32_t *)dst)[di] = ((const uint32_t *)src)[si];
    break;
  }
}

static inline void set_elem(size_t esize, void *dst, size_t di, uint32_t v) {
  switch (esize) {
  case 1:
    ((uint8_t *)dst)[di] = (uint8_t)v;
    break;
  case 2:
    ((uint16_t *)dst)[di] = (uint16_t)v;
    break;
  default:
    ((uint32_t *)dst)[di] = v;
    break;
  }
}

/* ref/pack/pack_e8rc_e8rcprc.c:10-35: every element of every (m0 x n0) block of the
 * ceil(m/m0) x ceil(n/n0) grid is written: the source value when it exists, else `pad`. */
void orc_pack(size_t esize, size_t m, size_t n, const void *src, size_t rs, size_t cs, size_t m0,
              size_t n0, void *dst, size_t rs0, size_t cs0, size_t rs1, size_t cs1, uint32_t pad) {
  if (m0 == 0 || n0 == 0) {
    return; /* the reference would divide by zero; the product treats it as a no-op */
  }
  size_t m1 = (m + m0 - 1) / m0;
  size_t n1 = (n + n0 - 1) / n0;
  for (size_t bi = 0; bi < m1; ++bi) {
    for (size_t bj = 0; bj < n1; ++bj) {
      for (size_t i0 = 0; i0 < m0; ++i0) {
        for (size_t j0 = 0; j0 < n0; ++j0) {
          size_t i = bi * m0 + i0;
          size_t j = bj * n0 + j0;
          size_t di = bi * rs1 + bj * cs1 + i0 * rs0 + j0 * cs0;
          if (i < m && j < n) {
            copy_elem(esize, dst, di, src, i * rs + j * cs);
          } else {
            set_elem(esize, dst, di, pad);
          }
        }
      }
    }
  }
}

/* ref/pack/unpack_e8rcprc_e8rc.c:10-37: inverse of pack; padding elements are dropped. */
void orc_unpack(size_t esize, size_t m0, size_t n0, const void *src, size_t rs0, size_t cs0,
                size_t rs1, size_t cs1, size_t m, size_t n, void *dst, size_t rs, size_t cs) {
  if (m0 == 0 || n0 == 0) {
    return;
  }
  for (size_t i = 0; i < m; ++i) {
    for (size_t j = 0; j < n; ++j) {
      size_t si = (i / m0) * rs1 + (j / n0) * cs1 + (i % m0) * rs0 + (j % n0) * cs0;
      copy_elem(esize, dst, i * rs + j * cs, src, si);
    }
  }
}

/* ref/pack/transpose_e8.c:11-19: at[j*rsat + i] = a[i*rsa + j]. */
void orc_transpose(size_t esize, size_t m, size_t n, const void *a, size_t rsa, void *at,
                   size_t rsat) {
  for (size_t i = 0; i < m; ++i) {
    for (size_t j = 0; j < n; ++j) {
      copy_elem(esize, at, j * rsat + i, a, i * rsa + j);
    }
  }
}

/* ------------------------------------------------------------------ MX-FP4 GEMM (no reference routine)
 * Restates the published format (OCP Microscaling Formats v1.0: E2M1 elements, one E8M0 scale 2^(s - 127) per 32
 * consecutive k, s = 255 meaning NaN) on top of the reference's E2M1 value table (ref/cvt/cvt_ofp4.c:18-60) and the
 * reference's float GEMM loop (ref/gemm/gemm_bf16rc_bf16rc_f32rc.c:9-24): fp32 products of the scaled elements, one fp32
 * accumulator, k ascending, c = beta * c + alpha * acc.  Parity of the GEMM itself is unpinned (the reference has no
 * such routine); the element decode is pinned through orc_f4e2m1_to_f8e4m3 / orc_f8e4m3_to_f32. */
float orc_mxf4_element(uint8_t nibble, uint8_t scale) {
  volatile float v = orc_f8e4m3_to_f32(orc_f4e2m1_to_f8e4m3(nibble & 0xFu));
  volatile float f;
  if (scale == 255u) {
    union { uint32_t u; float f; } nan = {0x7FC00000u};
    f = nan.f;
  } else {
    union { uint32_t u; float f; } p2 = {scale == 0u ? 0x00400000u : (uint32_t)scale << 23};
    f = p2.f;
  }
  volatile float r = v * f;
  return r;
}

void orc_gemm_mxf4(size_t m, size_t n, size_t k, float alpha, const uint8_t *a, size_t rsa, const uint8_t *sa,
                   size_t rssa, const uint8_t *b, size_t csb, const uint8_t *sb, size_t cssb, float beta, float *c,
                   size_t rsc) {
  for (size_t i = 0; i < m; ++i) {
    for (size_t j = 0; j < n; ++j) {
      float acc = 0.0f;
      for (size_t kk = 0; kk < k; ++kk) {
        const uint8_t ab = a[i * rsa + kk / 2], bb = b[j * csb + kk / 2];
        const float av = orc_mxf4_element((kk & 1u) ? (uint8_t)(ab >> 4) : (uint8_t)(ab & 0xFu), sa[i * rssa + kk / 32]);
        const float bv = orc_mxf4_element((kk & 1u) ? (uint8_t)(bb >> 4) : (uint8_t)(bb & 0xFu), sb[j * cssb + kk / 32]);
        volatile float prod = av * bv;
        acc += prod;
      }
      volatile float scaled = alpha * acc;
      float *cp = c + i * rsc + j;
      if (beta == 0.0f) {
        *cp = scaled;
      } else {
        volatile float old = beta * *cp;
        *cp = old + scaled;
      }
    }
  }
}

