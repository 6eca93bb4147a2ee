// numerics.cuh -- device-side element conversions shared by the GEMM epilogues and the cvt kernels.
//
// Every routine reproduces, bit for bit, the scalar conversion SKL defines in ref/cvt/cvt_ofp8.c
// (decoders :18-95, encoders :97-172) or the C casts its reference GEMMs use for bf16 / fp16.
// They work on raw bit patterns so no translation unit depends on cuda_fp16/bf16/fp8 class types.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#include "../abi.h"

namespace sklb {

// Counts launches per host thread so callers can report how many kernels a call issued.
int &launch_counter_ref();
#define SKLB_COUNT_LAUNCH() (++::sklb::launch_counter_ref())

__device__ __forceinline__ uint32_t f2u(float x) { return __float_as_uint(x); }
__device__ __forceinline__ float u2f(uint32_t u) { return __uint_as_float(u); }

// ---------------------------------------------------------------- fp8 -> fp32 (exact)
// E4M3: bias 7, no Inf, code 0x7F/0xFF is NaN and decodes to +qNaN 0x7FC00000 (sign dropped).
__device__ __forceinline__ float dec_e4m3(uint32_t code) {
  uint32_t sign = (code & 0x80u) << 24;
  uint32_t mag = code & 0x7Fu;
  float sub = (float)(int)(mag & 7u) * 0.001953125f;  // m * 2^-9 (used when exponent field is 0)
  uint32_t nrm = (mag << 20) + 0x3C000000u;           // ((e + 120) << 23) | (m << 20)
  uint32_t bits = (mag < 8u) ? f2u(sub) : nrm;
  bits |= sign;
  return u2f(mag == 0x7Fu ? 0x7FC00000u : bits);
}

// E5M2: bias 15, Inf keeps its sign, every NaN code decodes to +qNaN.
__device__ __forceinline__ float dec_e5m2(uint32_t code) {
  uint32_t sign = (code & 0x80u) << 24;
  uint32_t mag = code & 0x7Fu;
  float sub = (float)(int)(mag & 3u) * 0.0000152587890625f;  // m * 2^-16
  uint32_t nrm = (mag << 21) + 0x38000000u;                  // ((e + 112) << 23) | (m << 21)
  uint32_t bits = (mag < 4u) ? f2u(sub) : nrm;
  bits = (mag == 0x7Cu) ? 0x7F800000u : bits;
  bits |= sign;
  return u2f(mag > 0x7Cu ? 0x7FC00000u : bits);
}

// ---------------------------------------------------------------- fp32 -> fp8, integer formulation
// Round-to-nearest-even right shift; s >= 1, may exceed 31.
__device__ __forceinline__ uint32_t shr_rne(uint32_t v, int s) {
  if (s > 31) return 0u;
  uint32_t q = v >> s;
  uint32_t rem = v & ((1u << s) - 1u);
  uint32_t half = 1u << (s - 1);
  return q + ((rem > half || (rem == half && (q & 1u))) ? 1u : 0u);
}

template <int MBITS, int BIAS, uint32_t MAXCODE>
__device__ __forceinline__ uint32_t enc_f8_soft(float x, uint32_t over_code) {
  uint32_t u = f2u(x);
  uint32_t sign = (u >> 24) & 0x80u;
  uint32_t au = u & 0x7FFFFFFFu;
  if (au > 0x7F800000u) return 0x7Fu;
  if (au == 0x7F800000u) return over_code;
  uint32_t be = au >> 23;
  if (be == 0u) return sign;
  int e = (int)be - 127;
  uint32_t sig = (au & 0x7FFFFFu) | 0x800000u;
  const int emin = 1 - BIAS;
  if (e < emin) return sign | shr_rne(sig, 23 - MBITS + (emin - e));
  uint32_t mag = ((uint32_t)(e + BIAS) << MBITS) + shr_rne(sig & 0x7FFFFFu, 23 - MBITS);
  if (e + BIAS > (0x7F >> MBITS) || mag > MAXCODE) return over_code;
  return sign | mag;
}

__device__ __forceinline__ uint32_t enc_e4m3_soft(float x, bool sat) {
  uint32_t sign = (f2u(x) >> 24) & 0x80u;
  return enc_f8_soft<3, 7, 0x7Eu>(x, sat ? (sign | 0x7Eu) : 0x7Fu);
}
__device__ __forceinline__ uint32_t enc_e5m2_soft(float x, bool sat) {
  uint32_t sign = (f2u(x) >> 24) & 0x80u;
  return enc_f8_soft<2, 15, 0x7Bu>(x, sign | (sat ? 0x7Bu : 0x7Cu));
}

// ---------------------------------------------------------------- fp32 -> fp8, hardware assisted
// cvt.rn.satfinite.{e4m3x2,e5m2x2}.f32 rounds to nearest even and clamps to the largest finite
// value.  It is used for in-range inputs only; overflow, infinities and NaN take SKL's conventions
// explicitly (E4M3 non-saturating: 0x7F with the sign dropped; E5M2 non-saturating: signed Inf).
__device__ __forceinline__ uint32_t hw_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t hw_e5m2x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

// Fix-up of one hardware-encoded byte.  E4M3: magnitudes above 464 round past the largest finite
// value 448 (464 itself ties to even = 448).
__device__ __forceinline__ uint32_t fix_e4m3(uint32_t hw, float x, bool sat) {
  uint32_t u = f2u(x);
  uint32_t au = u & 0x7FFFFFFFu;
  uint32_t sign = (u >> 24) & 0x80u;
  uint32_t over = sat ? (sign | 0x7Eu) : 0x7Fu;
  uint32_t r = (au > 0x43E80000u) ? over : hw;  // 464.0f = 0x43E80000
  return (au > 0x7F800000u) ? 0x7Fu : r;
}
// E5M2: magnitudes >= 61440 round to 65536 = overflow (61440 ties to even, which is the Inf slot).
__device__ __forceinline__ uint32_t fix_e5m2(uint32_t hw, float x, bool sat) {
  uint32_t u = f2u(x);
  uint32_t au = u & 0x7FFFFFFFu;
  uint32_t sign = (u >> 24) & 0x80u;
  uint32_t over = sign | (sat ? 0x7Bu : 0x7Cu);
  uint32_t r = (au >= 0x47700000u) ? over : hw;  // 61440.0f = 0x47700000
  return (au > 0x7F800000u) ? 0x7Fu : r;
}

__device__ __forceinline__ uint32_t enc_e4m3x2(float lo, float hi, bool sat) {
  uint32_t hw = hw_e4m3x2(lo, hi);
  return fix_e4m3(hw & 0xFFu, lo, sat) | (fix_e4m3(hw >> 8, hi, sat) << 8);
}
__device__ __forceinline__ uint32_t enc_e5m2x2(float lo, float hi, bool sat) {
  uint32_t hw = hw_e5m2x2(lo, hi);
  return fix_e5m2(hw & 0xFFu, lo, sat) | (fix_e5m2(hw >> 8, hi, sat) << 8);
}
__device__ __forceinline__ uint32_t enc_e4m3(float x, bool sat) {
  return fix_e4m3(hw_e4m3x2(x, 0.0f) & 0xFFu, x, sat);
}

// ---------------------------------------------------------------- 16-bit floats
__device__ __forceinline__ float dec_bf16(uint32_t bits) { return u2f(bits << 16); }

// RNE; NaN keeps sign and top payload and is quieted (what the host compiler's (__bf16) cast does).
__device__ __forceinline__ uint32_t enc_bf16(float x) {
  uint32_t u = f2u(x);
  uint32_t r = (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
  uint32_t nan = (u >> 16) | 0x40u;
  return ((u & 0x7FFFFFFFu) > 0x7F800000u) ? nan : r;
}

// Two finite-or-infinite values to packed bf16 / f16 with the hardware converter (lo in bits 0-15).  It rounds
// to nearest even exactly like enc_bf16 / enc_f16 but canonicalises NaN, so callers use it only on values they
// know are not NaN.
__device__ __forceinline__ uint32_t pack_bf16x2_no_nan(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ uint32_t pack_f16x2_no_nan(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

__device__ __forceinline__ float dec_f16(uint32_t bits) {
  float r;
  uint16_t h = (uint16_t)bits;
  asm("cvt.f32.f16 %0, %1;" : "=f"(r) : "h"(h));
  return r;
}
__device__ __forceinline__ uint32_t enc_f16(float x) {
  uint16_t h;
  asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(x));
  uint32_t u = f2u(x);
  uint32_t nan = ((u >> 16) & 0x8000u) | 0x7E00u | ((u >> 13) & 0x3FFu);
  return ((u & 0x7FFFFFFFu) > 0x7F800000u) ? nan : (uint32_t)h;
}

// ---------------------------------------------------------------- typed element access
template <int DT>
struct Elem;
template <>
struct Elem<SKL_DT_I8> {
  using store_t = int8_t;
};
template <>
struct Elem<SKL_DT_BF16> {
  using store_t = uint16_t;
};
template <>
struct Elem<SKL_DT_F16> {
  using store_t = uint16_t;
};
template <>
struct Elem<SKL_DT_F8E4M3> {
  using store_t = uint8_t;
};
template <>
struct Elem<SKL_DT_F8E5M2> {
  using store_t = uint8_t;
};
template <>
struct Elem<SKL_DT_F32> {
  using store_t = float;
};
template <>
struct Elem<SKL_DT_I32> {
  using store_t = int32_t;
};

__host__ __device__ __forceinline__ int dtype_size(int dt) {
  return (dt == SKL_DT_F32 || dt == SKL_DT_I32) ? 4 : ((dt == SKL_DT_BF16 || dt == SKL_DT_F16) ? 2 : 1);
}

// Load an operand element as fp32 (float pairs) -- dt is a runtime code, the switch is uniform.
__device__ __forceinline__ float load_as_f32(int dt, const void *p, int64_t idx) {
  switch (dt) {
    case SKL_DT_BF16:
      return dec_bf16(((const uint16_t *)p)[idx]);
    case SKL_DT_F16:
      return dec_f16(((const uint16_t *)p)[idx]);
    case SKL_DT_F8E4M3:
      return dec_e4m3(((const uint8_t *)p)[idx]);
    case SKL_DT_F8E5M2:
      return dec_e5m2(((const uint8_t *)p)[idx]);
    default:
      return ((const float *)p)[idx];
  }
}

// Read / write one C element of the float epilogue.
// Requantised int8 output: round to nearest even, saturate to [-128, 127], NaN -> 0.
__device__ __forceinline__ uint32_t enc_i8_sat(float v) {
  int32_t r;
  asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v));
  return (uint32_t)r & 0xFFu;
}
__device__ __forceinline__ float load_c_f32(int tc, const void *c, int64_t idx) {
  if (tc == SKL_DT_I32) return (float)((const int32_t *)c)[idx];
  if (tc == SKL_DT_I8) return (float)((const int8_t *)c)[idx];
  return load_as_f32(tc, c, idx);
}
__device__ __forceinline__ void store_c_f32(int tc, void *c, int64_t idx, float v) {
  switch (tc) {
    case SKL_DT_BF16:
      ((uint16_t *)c)[idx] = (uint16_t)enc_bf16(v);
      break;
    case SKL_DT_F16:
      ((uint16_t *)c)[idx] = (uint16_t)enc_f16(v);
      break;
    case SKL_DT_F8E4M3:
      ((uint8_t *)c)[idx] = (uint8_t)enc_e4m3(v, true);
      break;
    case SKL_DT_I8:
      ((uint8_t *)c)[idx] = (uint8_t)enc_i8_sat(v);
      break;
    default:
      ((float *)c)[idx] = v;
      break;
  }
}

// The float epilogue, one element: every step a separately rounded fp32 operation.
__device__ __forceinline__ float epilogue_value(float acc, float alpha, const float *row_scale,
                                                const float *col_scale, int64_t i, int64_t j) {
  float v = __fmul_rn(alpha, acc);
  if (row_scale) v = __fmul_rn(v, row_scale[i]);
  if (col_scale) v = __fmul_rn(v, col_scale[j]);
  return v;
}

// Activations of the float epilogue, after the reference's scalar definitions (ref/sigmoid/sigmoid_f32.c:10-28:
// logistic o = 1/(1+exp(-beta*x)), then o *= y for the linear unit, then o *= (up + delta) for the gate;
// ref/gelu/gelu_f32.c:12-22: relu(x) + (-|x|/2) * erfc(|x|/sqrt 2)).  The reference evaluates them in double and
// rounds once; here they are fp32 with the accurate expf / erfcf, the product -p*v carried as a rounded part
// plus its exact remainder so that a large exponent argument does not magnify the product's rounding.
__device__ __forceinline__ float logistic_f32(float p, float v) {
  const float hi = __fmul_rn(-p, v);
  const float lo = __fmaf_rn(-p, v, -hi);  // exact: -p*v = hi + lo
  if (hi > 20.0f) {
    // 1 + e^a = e^a to within 2^-28 here, so the result is e^-a: no overflow of e^a, and the tail runs
    // through the subnormals down to zero as the double-precision definition does
    const float t = expf(-hi);
    return __fmaf_rn(t, -lo, t);
  }
  float t = expf(hi);
  t = __fmaf_rn(t, lo, t);  // exp(hi + lo) ~ exp(hi) * (1 + lo)
  return __fdiv_rn(1.0f, __fadd_rn(1.0f, t));
}
__device__ __forceinline__ float gelu_f32(float v) {
  const float b = v > 0.0f ? v : -0.0f;
  const float h = __fmul_rn(-0.5f, fabsf(v));
  const float e = erfcf(__fmul_rn(-1.41421356237309504880f, h));
  return __fmaf_rn(h, e, b);
}
// `old` is C's previous value (read only for SKL_ACT_SWIGLU).
__device__ __forceinline__ float activation_value(int act, float p, float v, float old) {
  switch (act) {
    case SKL_ACT_LOGISTIC: return logistic_f32(p, v);
    case SKL_ACT_SWISH: return __fmul_rn(logistic_f32(p, v), v);
    case SKL_ACT_GELU: return gelu_f32(v);
    case SKL_ACT_SWIGLU: return __fmul_rn(__fmul_rn(logistic_f32(1.0f, v), v), __fadd_rn(old, p));
    default: return v;
  }
}

// *addr = max(*addr, v) for floats (NaN never wins): the IEEE ordering of non-negative floats equals the
// ordering of their bit patterns as signed integers, that of negative floats the reverse as unsigned.
// The branch is on the sign bit, not on v >= 0: -0.0 belongs with the negative patterns (it is the largest of
// them), so a maximum over values that are all <= -0.0 ends at -0.0 and +0.0 still wins over -0.0, which is
// the bit pattern a sequential `if (v > max) max = v` over the same values can end with.
__device__ __forceinline__ void atomic_max_f32(float *addr, float v) {
  if (!(v == v)) return;
  if ((__float_as_uint(v) >> 31) == 0u)
    atomicMax(reinterpret_cast<int *>(addr), __float_as_int(v));
  else
    atomicMin(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}

// Largest value across the warp (lanes without a value pass -INFINITY); every lane gets the result.
__device__ __forceinline__ float warp_max_f32(float v) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
  return v;
}

}  // namespace sklb
