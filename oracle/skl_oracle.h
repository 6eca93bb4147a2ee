/*
 * skl_oracle.h -- CPU restatement of the SKL gemm / pack / cvt semantics.
 *
 * TEST INFRASTRUCTURE ONLY.  This file and skl_oracle.c are the checker that the
 * parity tests, the smoke test and the benchmark's CPU-baseline leg compare the
 * CUDA library against.  Nothing in the product library includes, links or loads
 * them, and the product has no CPU fallback.
 *
 * Parity status: PINNED.  Every function here is checked, on seeded inputs and on
 * exhaustive code sweeps, against the reference's own scalar `_ref` routines
 * compiled from the reference tree (oracle/Makefile target `ref`), and against
 * golden vectors those routines produced (tests/golden/).
 *
 * Each function names the reference routine (path:line inside the SKL tree)
 * whose results it must reproduce bit for bit.
 *
 * Floating-point 16-bit and 8-bit values travel as raw bit patterns
 * (uint16_t / uint8_t) so the interface needs no compiler extension types.
 */
#ifndef SKL_ORACLE_H
#define SKL_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element type codes shared with the product's extension entry points. */
enum {
  ORC_I8 = 0,
  ORC_BF16 = 1,
  ORC_F16 = 2,
  ORC_F8E4M3 = 3,
  ORC_F8E5M2 = 4,
  ORC_F32 = 5,
  ORC_I32 = 6
};

/* ---- scalar conversions (ref/cvt/cvt_ofp8.c:18-172) ---- */
float orc_f8e4m3_to_f32(uint8_t code);            /* skl_cvt_f8e4m3_f32, cvt_ofp8.c:18-52  */
float orc_f8e5m2_to_f32(uint8_t code);            /* skl_cvt_f8e5m2_f32, cvt_ofp8.c:54-95  */
uint8_t orc_f32_to_f8e4m3(float x, int saturate); /* skl_cvt_f32_f8e4m3, cvt_ofp8.c:97-134 */
uint8_t orc_f32_to_f8e5m2(float x, int saturate); /* skl_cvt_f32_f8e5m2, cvt_ofp8.c:136-172 */
float orc_bf16_to_f32(uint16_t bits);             /* C cast (float)(__bf16)                */
uint16_t orc_f32_to_bf16(float x);                /* C cast (__bf16)(float), RNE           */
float orc_f16_to_f32(uint16_t bits);              /* C cast (float)(_Float16)              */
uint16_t orc_f32_to_f16(float x);                 /* C cast (_Float16)(float), RNE         */
uint8_t orc_f4e2m1_to_f8e4m3(uint8_t nibble);     /* ref/cvt/cvt_ofp4.c:18-60              */

/* ---- array conversions (ref/cvt/cvt_ofp8.c:174-242) ----
 * fmt is ORC_F8E4M3 or ORC_F8E5M2; saturate selects the skl_cvt_sat_* flavour. */
void orc_cvt_f32_f8(uint8_t *dst, const float *src, float scale, size_t n, int fmt, int saturate);
void orc_cvt_bf16_f8(uint8_t *dst, const uint16_t *src, float scale, size_t n, int fmt, int saturate);
void orc_cvt_f8_bf16(uint16_t *dst, const uint8_t *src, size_t n, int fmt);
void orc_cvt_f4e2m1_f8e4m3(uint8_t *dst, const uint8_t *src, size_t n); /* cvt_ofp4.c:62-72 */

/* ---- GEMM, general element strides ----
 * C[i,j] = beta*C[i,j] + alpha*sum_k A[i,k]*B[k,j], one accumulator per output, k ascending.
 * int8: ref/gemm/gemm_i8rc_i8rc_i32rc.c:10-26 (int32 wrap-around arithmetic). */
void orc_gemm_i8_i32(size_t m, size_t n, size_t k, int32_t alpha, const int8_t *a, size_t rsa,
                     size_t csa, const int8_t *b, size_t rsb, size_t csb, int32_t beta, int32_t *c,
                     size_t rsc, size_t csc);
/* float: ta/tb in {ORC_BF16, ORC_F16, ORC_F8E4M3, ORC_F8E5M2}; fp32 products and accumulator.
 * Same-type pairs restate ref/gemm/gemm_bf16rc_bf16rc_f32rc.c:9-24, gemm_f16rc_f16rc_f32rc.c:9-24,
 * gemm_f8e4m3rc_f8e4m3rc_f32rc.c:11-25, gemm_f8e5m2rc_f8e5m2rc_f32rc.c:11-25.  Mixed pairs use the
 * same loop with each operand decoded by its own type (no reference routine exists for them). */
void orc_gemm_fp_f32(size_t m, size_t n, size_t k, float alpha, int ta, const void *a, size_t rsa,
                     size_t csa, int tb, const void *b, size_t rsb, size_t csb, float beta, float *c,
                     size_t rsc, size_t csc);

/* fp64: ref/gemm/gemm_f64rc_f64rc_f64rc.c:9-22 and, packed, gemm_f64rcprc_f64rcprc_f64rcprc.c; fp32 operands
 * go through orc_gemm_fp_f32 with ta = tb = ORC_F32 (ref/gemm/gemm_f32rc_f32rc_f32rc.c:9-22). */
void orc_gemm_f64(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1, double alpha, const double *a,
                  size_t rsa0, size_t csa0, size_t rsa1, size_t csa1, const double *b, size_t rsb0, size_t csb0,
                  size_t rsb1, size_t csb1, double beta, double *c, size_t rsc0, size_t csc0, size_t rsc1,
                  size_t csc1);

/* fp16 accumulator: ref/gemm/gemm_f16rc_f16rc_f16rc.c:9-22 and gemm_f16rcprc_f16rcprc_f16rcprc.c, every statement
 * evaluated in fp32 and rounded to fp16 once (see the definition). */
void orc_gemm_f16acc(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1, float alpha,
                     const uint16_t *a, size_t rsa0, size_t csa0, size_t rsa1, size_t csa1, const uint16_t *b,
                     size_t rsb0, size_t csb0, size_t rsb1, size_t csb1, float beta, uint16_t *c, size_t rsc0,
                     size_t csc0, size_t rsc1, size_t csc1);

/* ---- GEMM, packed (blocked 4-D) operands ----
 * int8: ref/gemm/gemm_i8rcprc_i8rcprc_i32rcprc.c:10-37;
 * float: gemm_bf16rcprc_bf16rcprc_f32rcprc.c:9-36 and its f16 / f8 siblings. */
void orc_gemm_packed_i8_i32(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1,
                            int32_t alpha, const int8_t *a, size_t rsa0, size_t csa0, size_t rsa1,
                            size_t csa1, const int8_t *b, size_t rsb0, size_t csb0, size_t rsb1,
                            size_t csb1, int32_t beta, int32_t *c, size_t rsc0, size_t csc0,
                            size_t rsc1, size_t csc1);
void orc_gemm_packed_fp_f32(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1,
                            float alpha, int ta, const void *a, size_t rsa0, size_t csa0,
                            size_t rsa1, size_t csa1, int tb, const void *b, size_t rsb0,
                            size_t csb0, size_t rsb1, size_t csb1, float beta, float *c,
                            size_t rsc0, size_t csc0, size_t rsc1, size_t csc1);

/* ---- extended epilogue (no reference routine; composed from the pieces above) ----
 * acc as in the plain GEMM (int32 for int8 pairs, fp32 otherwise), then, all in fp32 with one
 * rounding per operation and no fused multiply-add:
 *     v = (float)acc;  v = alpha*v;  if row_scale: v = v*row_scale[i];  if col_scale: v = v*col_scale[j];
 *     if beta != 0:    v = beta*(float)C[i,j] + v;
 *     C[i,j] = narrow(v)   tc in {ORC_F32, ORC_BF16 (RNE), ORC_F16 (RNE), ORC_F8E4M3 (saturating),
 *                                 ORC_I8 (requantised: nearest even, saturating to [-128,127], NaN -> 0)}.
 * ta/tb may be ORC_I8 (both), or any float pair. */
void orc_gemm_ex(size_t m, size_t n, size_t k, int ta, const void *a, size_t rsa, size_t csa, int tb,
                 const void *b, size_t rsb, size_t csb, float alpha, const float *row_scale,
                 const float *col_scale, float beta, int tc, void *c, size_t rsc, size_t csc);

/* The same with the two epilogue kernels the reference documents as examples of its fused-kernel hook
 * (src/gemm/fused-kernel-API.md:170-217): a bias row vector added after the scales, and the running global
 * maximum of the results (NaN ignored), both optional:
 *     v = alpha*acc; *row_scale[i]; *col_scale[j]; v = v + bias[j]; v = beta*C + v; v = act(v);
 *     *gmax = max(*gmax, v); C = narrow(v)
 * act is one of the reference's element-wise routines (ref/sigmoid/sigmoid_f32.c:10-28,
 * ref/gelu/gelu_f32.c:12-22), evaluated in double and rounded once as they are there. */
enum { ORC_ACT_NONE = 0, ORC_ACT_LOGISTIC = 1, ORC_ACT_SWISH = 2, ORC_ACT_GELU = 3, ORC_ACT_SWIGLU = 4 };
/* LOGISTIC 1/(1+exp(-p*v)); SWISH that times v (p = 1: SiLU); GELU; SWIGLU silu(v)*(up + p). */
float orc_activation(int act, float p, float v, float up);
void orc_gemm_fused(size_t m, size_t n, size_t k, int ta, const void *a, size_t rsa, size_t csa, int tb,
                    const void *b, size_t rsb, size_t csb, float alpha, const float *row_scale,
                    const float *col_scale, const float *bias, float *global_max, float beta, int activation,
                    float act_param, int tc, void *c, size_t rsc, size_t csc);

/* ---- pack / unpack / transpose (ref/pack/pack_e8rc_e8rcprc.c:10-35, unpack_e8rcprc_e8rc.c:10-37,
 * transpose_e8.c:11-19 and the e16 / e32 siblings); esize is the element size in bytes (1, 2, 4). */
void orc_pack(size_t esize, size_t m, size_t n, const void *src, size_t rs, size_t cs, size_t m0,
              size_t n0, void *dst, size_t rs0, size_t cs0, size_t rs1, size_t cs1, uint32_t pad);
void orc_unpack(size_t esize, size_t m0, size_t n0, const void *src, size_t rs0, size_t cs0,
                size_t rs1, size_t cs1, size_t m, size_t n, void *dst, size_t rs, size_t cs);
void orc_transpose(size_t esize, size_t m, size_t n, const void *a, size_t rsa, void *at,
                   size_t rsat);

#ifdef __cplusplus
}
#endif
/* MX-FP4 (OCP Microscaling v1.0) on the reference's E2M1 table and float-GEMM loop; no reference routine exists */
float orc_mxf4_element(uint8_t nibble, uint8_t scale);
void orc_gemm_mxf4(size_t m, size_t n, size_t k, float alpha, const uint8_t *a, size_t rsa, const uint8_t *sa,
                   size_t rssa, const uint8_t *b, size_t csb, const uint8_t *sb, size_t cssb, float beta, float *c,
                   size_t rsc);

#endif /* SKL_ORACLE_H */
