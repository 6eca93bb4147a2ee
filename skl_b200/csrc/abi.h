/*
 * abi.h -- the thin C ABI between the C99 host layer and the CUDA translation units.
 *
 * Everything here takes DEVICE pointers, element counts, element strides and a cudaStream_t passed
 * as void*; no C++ or CUDA type appears, so the host layer compiles as plain C99.  Each launcher
 * enqueues its kernel(s) on `stream` and returns the cudaError_t of the launch as an int (0 = ok);
 * none of them synchronises, allocates or frees.
 */
#ifndef SKL_B200_ABI_H
#define SKL_B200_ABI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element type codes (same numbering as skl_b200_dtype_t) */
enum {
  SKL_DT_I8 = 0,
  SKL_DT_BF16 = 1,
  SKL_DT_F16 = 2,
  SKL_DT_F8E4M3 = 3,
  SKL_DT_F8E5M2 = 4,
  SKL_DT_F32 = 5,
  SKL_DT_I32 = 6,
  SKL_DT_F64 = 7
};

/* How the accumulator becomes C. */
enum {
  /* C = beta*C + alpha*acc in int32 two's-complement arithmetic (ref/gemm/gemm_i8rc_i8rc_i32rc.c:23) */
  SKL_EPI_INT = 0,
  /* v = alpha*(float)acc; *row_scale[i]; *col_scale[j]; (+ beta*C when beta != 0); narrow to tc */
  SKL_EPI_FLOAT = 1,
  /* C = beta*C + alpha*acc in double, one rounding per operation (ref/gemm/gemm_f64rc_f64rc_f64rc.c:9-22) */
  SKL_EPI_F64 = 2,
  /* fp16 operands, fp16 accumulator and fp16 C (ref/gemm/gemm_f16rc_f16rc_f16rc.c:9-22): each statement of the
   * reference evaluated in fp32 and rounded to fp16 once -- acc = h(acc + a*b) per k (the product of two fp16
   * values is exact in fp32), C = h(beta*C + alpha*acc); alpha_f / beta_f hold the fp16 scalars' values */
  SKL_EPI_F16ACC = 3
};

/* Activation applied to the float epilogue's value v (same numbering as skl_b200_activation_t); the
 * definitions are the reference's scalar routines ref/sigmoid/sigmoid_f32.c:10-28 and ref/gelu/gelu_f32.c:12-22. */
enum {
  SKL_ACT_NONE = 0,
  SKL_ACT_LOGISTIC = 1, /* 1 / (1 + exp(-p*v))                                  */
  SKL_ACT_SWISH = 2,    /* v / (1 + exp(-p*v));  p = 1 is SiLU                   */
  SKL_ACT_GELU = 3,     /* v * Phi(v), erf form                                  */
  SKL_ACT_SWIGLU = 4    /* v / (1 + exp(-v)) * (C_old[i,j] + p); beta must be 0  */
};

/* One GEMM problem.  Plain matrices use m1 = n1 = k1 = 1 and *1 strides of 0. */
typedef struct skl_b200_gemm_args {
  uint64_t m0, n0, k0; /* block extents (plain matrix: the matrix extents) */
  uint64_t m1, n1, k1; /* block counts                                      */
  int32_t ta, tb, tc;  /* SKL_DT_*                                          */
  int32_t epilogue;    /* SKL_EPI_*                                         */
  const void *a;
  const void *b;
  void *c;
  int64_t rsa0, csa0, rsa1, csa1;
  int64_t rsb0, csb0, rsb1, csb1;
  int64_t rsc0, csc0, rsc1, csc1;
  int32_t alpha_i, beta_i; /* SKL_EPI_INT   */
  float alpha_f, beta_f;   /* SKL_EPI_FLOAT */
  double alpha_d, beta_d;  /* SKL_EPI_F64   */
  const float *row_scale;  /* m entries or NULL (SKL_EPI_FLOAT) */
  const float *col_scale;  /* n entries or NULL (SKL_EPI_FLOAT) */
  int32_t col_scale_first; /* 0: v*row_scale then *col_scale (the defined order); 1: the reverse, used
                              when a problem is handed over transposed so the two vectors swap roles */
  const float *bias;       /* NULL, or a vector added after the scales (SKL_EPI_FLOAT): n entries indexed by
                              column, or m entries indexed by row when bias_per_row is set (transposed hand-over) */
  int32_t bias_per_row;
  float *global_max;       /* NULL, or one device float raised to the largest result value (NaN ignored) */
  int32_t activation;      /* SKL_ACT_*: applied after bias and beta*C, before the maximum and the narrowing */
  float act_param;         /* logistic / swish: beta; swiglu: delta */
  int32_t b_static;        /* the caller declared B (the weights) not written by earlier work on the stream: the
                              skinny kernel may then start streaming B before the preceding kernel has finished */
  uint32_t wait_limit_ms;  /* bound of every device-side wait of this launch; 0 = the default (2000 ms) */
  int32_t debug_skip_loads; /* testing aid: the kernel's producer announces its loads but does not issue them, so the
                               consumers' bounded waits must run out (exercises the give-up path without any fault) */
} skl_b200_gemm_args;

/* Device status word written by kernels whose bounded waits expire: 0 = ok, else a stage code. */
#define SKL_B200_DEVSTATUS_WORDS 4

/* Any-stride SIMT GEMM: every type pair, blocked operands, k == 0.  One accumulator per output,
 * k ascending, so float results reproduce the scalar reference's summation order. */
int skl_b200_launch_gemm_generic(const skl_b200_gemm_args *args, void *stream);

/* Tensor-core GEMM (TMA + tcgen05 + TMEM).  Plain (unblocked) operands only.
 * skl_b200_gemm_tc_supported returns 1 when the problem meets the kernel's layout rules:
 * each of A and B has one unit stride, 16-byte aligned base and leading stride, supported pair. */
int skl_b200_gemm_tc_supported(const skl_b200_gemm_args *args);
int skl_b200_launch_gemm_tc(const skl_b200_gemm_args *args, uint32_t *dev_status, void *stream);

/* Skinny int8 kernel: m <= 16, A rows and B columns contiguous in k (csa == 1, rsb == 1),
 * 16-byte aligned rows, k % 16 == 0, m*k bytes of A fit in shared memory. */
int skl_b200_gemv_i8_supported(const skl_b200_gemm_args *args);
int skl_b200_launch_gemv_i8(const skl_b200_gemm_args *args, uint32_t *dev_status, void *stream);

/* cvt: src_type in {F32, BF16}, dst_fmt in {F8E4M3, F8E5M2}. */
int skl_b200_launch_cvt_to_f8(void *dst, const void *src, int src_type, int dst_fmt, int saturate,
                              float scale, size_t n, void *stream);
int skl_b200_launch_cvt_f8_to_bf16(void *dst, const void *src, int src_fmt, size_t n, void *stream);
/* Strided widening used by the bf16 x fp8 GEMM: dst is a dense rows x cols bf16 matrix with the same
 * orientation as the source (unit stride kept), leading dimension ld_dst. */
int skl_b200_launch_cvt_f8_to_bf16_2d(void *dst, size_t ld_dst, const void *src, size_t ld_src,
                                      int src_fmt, size_t rows, size_t cols, void *stream);
int skl_b200_launch_cvt_f4_to_f8e4m3(void *dst, const void *src, size_t n, void *stream);
/* MX-FP4 rows (16 bytes + one E8M0 scale per block of 32 elements) -> bf16 rows; ld_* in elements of dst / bytes of src / scale bytes */
/* MX-FP4 GEMM on the block-scaled tensor-core instruction (device pointers; see gemm_tc.cu) */
int skl_b200_gemm_mxf4_supported(const void *a, int64_t rsa, const void *b, int64_t csb, int64_t m, int64_t n, int64_t k);
size_t skl_b200_gemm_mxf4_scale_bytes(int64_t rows, int64_t k); /* workspace for one operand's re-laid scales */
int skl_b200_launch_gemm_mxf4(const void *a, int64_t rsa, const void *sa, int64_t rssa, const void *b, int64_t csb,
                              const void *sb, int64_t cssb, float *c, int64_t rsc, int64_t m, int64_t n, int64_t k,
                              float alpha, float beta, void *ws_sa, void *ws_sb, uint32_t wait_limit_ms,
                              uint32_t *dev_status, void *stream);
int skl_b200_launch_cvt_mxf4_to_bf16(void *dst, size_t ld_dst, const void *src, size_t ld_src, const void *scales,
                                     size_t ld_scales, size_t rows, size_t kblocks, void *stream);
/* Device-side self check: counts inputs in [first, first+count) (fp32 bit patterns) for which the
 * hardware-assisted encoder and the integer encoder disagree; *mismatches is a device uint64. */
/* dst[c][r] = widen(src[r][c]): rows x cols fp8 (unit stride along cols) into cols x rows bf16 (unit stride along
 * rows).  Needs a 4-byte aligned src with ld_src % 4 == 0 and a 16-byte aligned dst with ld_dst % 8 == 0
 * (cudaErrorInvalidValue otherwise). */
int skl_b200_launch_cvt_f8_to_bf16_2d_transposed(void *dst, size_t ld_dst, const void *src, size_t ld_src,
                                                 int src_fmt, size_t rows, size_t cols, void *stream);
int skl_b200_launch_cvt_selfcheck(int dst_fmt, int saturate, uint64_t first, uint64_t count,
                                  unsigned long long *mismatches, void *stream);

/* pack / unpack / transpose; esize in {1, 2, 4}. */
int skl_b200_launch_pack(size_t esize, size_t m, size_t n, const void *src, size_t rs, size_t cs,
                         size_t m0, size_t n0, void *dst, size_t rs0, size_t cs0, size_t rs1,
                         size_t cs1, uint32_t pad, void *stream);
int skl_b200_launch_unpack(size_t esize, size_t m0, size_t n0, const void *src, size_t rs0,
                           size_t cs0, size_t rs1, size_t cs1, size_t m, size_t n, void *dst,
                           size_t rs, size_t cs, void *stream);
int skl_b200_launch_transpose(size_t esize, size_t m, size_t n, const void *a, size_t rsa, void *at,
                              size_t rsat, void *stream);

/* Number of kernel launches issued by this thread's launchers since the last reset. */
int skl_b200_launch_counter(int reset);

#ifdef __cplusplus
}
#endif
#endif /* SKL_B200_ABI_H */
