/*
 * skl-b200.h -- public C interface of the B200 (sm_100a) build of SKL's dense linear-algebra path:
 * the gemm family with its pack and cvt companions.
 *
 * Every function keeps the parameter list of the SKL routine it stands in for (cited per group as
 * path:line inside the SKL source tree); only the ISA field of the name changes to `sm100a`.
 * skl-b200-compat.h maps SKL's RISC-V names onto these so code written against skl.h compiles
 * unchanged.
 *
 * Conventions kept from SKL (include/skl-common.h:21-47, src/README.md:5-35, src/gemm/README.md:41-71):
 *   - plain C linkage, every function returns void, the caller owns every buffer;
 *   - strides are in ELEMENTS; fp8 travels as uint8_t, bf16 as __bf16, fp16 as _Float16;
 *   - C = alpha*A*B + beta*C; k == 0 gives C = beta*C; zero m or n is a no-op;
 *   - bytes of an output buffer that the (shape, stride) arguments do not address stay untouched.
 *
 * What is new on this target:
 *   - A pointer may be host memory or device memory (also managed); each argument is classified
 *     on its own.  Host operands are staged through device memory inside the call.
 *   - The work is issued on the calling thread's current library stream (default: the CUDA legacy
 *     default stream) and, unless asynchronous mode was selected, the call returns after it finished.
 *   - Errors cannot be returned through SKL's void signatures; skl_b200_last_status() reports the
 *     outcome of the calling thread's most recent library call.  There is no CPU fallback: when no
 *     usable device exists the call does nothing except record SKL_B200_ERR_CUDA.
 *   - beta == 0 means C is not read (SKL's scalar reference evaluates 0*C, which differs only when C
 *     holds NaN/Inf, or in the sign of a zero result).
 */
#ifndef SKL_B200_H
#define SKL_B200_H

#include <stddef.h>
#include <stdint.h>

#if !defined(SKL_FUNC)
#define SKL_FUNC /* same decorator hook as include/skl-common.h:21-34 */
#endif

#if !defined(SKL_RESTRICT)
#if defined(__cplusplus)
#define SKL_RESTRICT __restrict__
#else
#define SKL_RESTRICT restrict
#endif
#endif

/* 16-bit float storage types.  Only pointers to them cross the interface, so a build whose
 * compiler lacks the extension types may define these to uint16_t without changing the ABI. */
#if !defined(SKL_B200_BF16_T)
#if defined(__CUDACC__) || defined(SKL_B200_NO_EXT_FLOAT)
#define SKL_B200_BF16_T uint16_t
#define SKL_B200_F16_T uint16_t
#else
#define SKL_B200_BF16_T __bf16
#define SKL_B200_F16_T _Float16
#endif
#endif
typedef SKL_B200_BF16_T skl_bf16_t;
typedef SKL_B200_F16_T skl_f16_t;

#if defined(__cplusplus)
extern "C" {
#endif

/* ------------------------------------------------------------------ side channel (not in SKL) */

typedef enum skl_b200_status {
  SKL_B200_OK = 0,
  SKL_B200_ERR_INVALID_ARGUMENT = 1, /* null pointer with non-empty shape, overlapping restrict, bad enum */
  SKL_B200_ERR_CUDA = 2,             /* a CUDA runtime/driver call failed, or no sm_100 device        */
  SKL_B200_ERR_ALLOC = 3,            /* device workspace could not be allocated                       */
  SKL_B200_ERR_DEVICE_TIMEOUT = 4,   /* a bounded wait inside a kernel expired; output is undefined   */
  SKL_B200_ERR_UNSUPPORTED = 5       /* type combination not provided                                 */
} skl_b200_status_t;

/* Outcome of the calling thread's most recent library call. */
SKL_FUNC skl_b200_status_t skl_b200_last_status(void);
SKL_FUNC const char *skl_b200_status_string(skl_b200_status_t s);
/* Text of the last CUDA error seen by the calling thread ("" if none). */
SKL_FUNC const char *skl_b200_last_cuda_error(void);

/* Stream (a cudaStream_t passed as void*) used by the calling thread's later calls; NULL = legacy
 * default stream. */
SKL_FUNC void skl_b200_set_stream(void *cuda_stream);
SKL_FUNC void *skl_b200_get_stream(void);
/* 0 (default): each call returns after its device work completed.  1: calls whose arguments are
 * all device pointers only enqueue work; skl_b200_synchronize() waits.  Calls with host operands
 * always complete before returning. */
SKL_FUNC void skl_b200_set_async(int enabled);
SKL_FUNC void skl_b200_synchronize(void);
/* Releases the calling thread's cached device workspaces. */
SKL_FUNC void skl_b200_release_workspace(void);
/* Declares, for this thread's following calls, that the B operands (the weights) are static: nothing queued
 * earlier on the stream writes them.  The skinny int8 kernel (m <= 2) then launches as a programmatic
 * dependent of the preceding kernel: it starts streaming its weights while that kernel drains and waits for
 * it only before reading the activations, scales, bias or C.  A static fp8 B of a bf16 x fp8 GEMM is widened to
 * bf16 by the first call only; later calls with the same matrix reuse that copy.  Off by default; results are
 * identical. */
SKL_FUNC void skl_b200_set_static_weights(int enabled);

/* Which kernel family served the calling thread's last GEMM call (for tests and benchmarks). */
typedef enum skl_b200_path {
  SKL_B200_PATH_NONE = 0,
  SKL_B200_PATH_GENERIC = 1, /* any-stride SIMT kernel                         */
  SKL_B200_PATH_TCGEN05 = 2, /* TMA + tcgen05 tensor-core kernel               */
  SKL_B200_PATH_GEMV = 3     /* bandwidth-bound skinny kernel (m <= 16, int8)  */
} skl_b200_path_t;
SKL_FUNC skl_b200_path_t skl_b200_last_path(void);
/* Number of kernels the calling thread's last library call launched. */
SKL_FUNC int skl_b200_last_launch_count(void);
/* Kernel timing for benchmarks: after skl_b200_profile_begin(n) the next n GEMM calls of this thread
 * bracket their main kernel (not staging copies or the fp8-widening pre-pass) with CUDA events on the
 * launch stream; skl_b200_profile_end waits for the stream, stores the summed kernel time in
 * *total_ms and returns how many calls were recorded. */
SKL_FUNC void skl_b200_profile_begin(int max_calls);
SKL_FUNC int skl_b200_profile_end(double *total_ms);
/* Restricts GEMM dispatch (debug/testing): 0 = automatic, else force one skl_b200_path_t where legal. */
SKL_FUNC void skl_b200_force_path(int path);
/* Every wait inside the tensor-core and skinny kernels (on a shared-memory barrier that a copy or another warp
 * completes) is bounded: when it runs out the kernel records a stage code, all its warps leave through the normal
 * exit (tensor memory is released, nothing traps) and the call reports SKL_B200_ERR_DEVICE_TIMEOUT; the context
 * stays usable.  skl_b200_set_wait_limit sets that bound for the calling thread's later calls (milliseconds;
 * 0 restores the default of 2000).  skl_b200_debug_skip_loads(1) is a testing aid: the kernels' producers announce
 * their loads but do not issue them, so the consumers' waits must run out -- the give-up path is exercised
 * without any fault.  The output of such a call is undefined. */
SKL_FUNC void skl_b200_set_wait_limit(unsigned milliseconds);
SKL_FUNC void skl_b200_debug_skip_loads(int enabled);

/* Column range [*start, *start + *count) of an n-column matrix owned by shard `index` of `parts`
 * when B and C are partitioned by columns across devices (remainder spread over the first shards,
 * boundaries rounded to `align` columns where possible). */
SKL_FUNC void skl_b200_shard_columns(size_t n, size_t parts, size_t index, size_t align,
                                     size_t *start, size_t *count);
/* Companion of an all-gather of the column shards of C (no SKL counterpart: SKL has no multi-device code).
 * `gathered` holds the `parts` shards one after the other, `part_stride` elements apart: shard g is the row-major
 * m x count_g block (leading dimension count_g) that shard g of skl_b200_shard_columns(n, parts, g, align)
 * computed -- what ncclAllGather of equal shards produces.  Writes the row-major m x n matrix dst (row stride
 * rsd >= n elements of esize = 1, 2 or 4 bytes).  With equal shards the gathered buffer is an SKL packed matrix
 * with m0 = m, n0 = n / parts in block-column order (src/gemm/packed-gemm.md:63-77), and the routine is one
 * `unpack` (ref/pack/unpack_e8rcprc_e8rc.c:10-37); unequal shards take one strided copy per shard.  The
 * all-gather itself is the caller's (NCCL on the caller's communicator); pointers may be device or host. */
SKL_FUNC void skl_b200_unshard_columns_sm100a(size_t esize, size_t m, size_t n, size_t parts, size_t align,
                                              const void *gathered, size_t part_stride, void *dst, size_t rsd);

/* ------------------------------------------------------------------ GEMM, general element strides
 * Parameter lists of ref/gemm/gemm_i8rc_i8rc_i32rc.h:45-49, gemm_bf16rc_bf16rc_f32rc.h,
 * gemm_f16rc_f16rc_f32rc.h, gemm_f8e4m3rc_f8e4m3rc_f32rc.h, gemm_f8e5m2rc_f8e5m2rc_f32rc.h. */
SKL_FUNC void skl_gemm_i8rc_i8rc_i32rc_sm100a(size_t m, size_t n, size_t k, int32_t alpha,
                                              const int8_t *a, size_t rsa, size_t csa,
                                              const int8_t *b, size_t rsb, size_t csb, int32_t beta,
                                              int32_t *c, size_t rsc, size_t csc);
SKL_FUNC void skl_gemm_bf16rc_bf16rc_f32rc_sm100a(size_t m, size_t n, size_t k, float alpha,
                                                  const skl_bf16_t *a, size_t rsa, size_t csa,
                                                  const skl_bf16_t *b, size_t rsb, size_t csb,
                                                  float beta, float *c, size_t rsc, size_t csc);
SKL_FUNC void skl_gemm_f16rc_f16rc_f32rc_sm100a(size_t m, size_t n, size_t k, float alpha,
                                                const skl_f16_t *a, size_t rsa, size_t csa,
                                                const skl_f16_t *b, size_t rsb, size_t csb,
                                                float beta, float *c, size_t rsc, size_t csc);
SKL_FUNC void skl_gemm_f8e4m3rc_f8e4m3rc_f32rc_sm100a(size_t m, size_t n, size_t k, float alpha,
                                                      const uint8_t *a, size_t rsa, size_t csa,
                                                      const uint8_t *b, size_t rsb, size_t csb,
                                                      float beta, float *c, size_t rsc, size_t csc);
SKL_FUNC void skl_gemm_f8e5m2rc_f8e5m2rc_f32rc_sm100a(size_t m, size_t n, size_t k, float alpha,
                                                      const uint8_t *a, size_t rsa, size_t csa,
                                                      const uint8_t *b, size_t rsb, size_t csb,
                                                      float beta, float *c, size_t rsc, size_t csc);

/* ------------------------------------------------------------------ GEMM, row-major A, B, C
 * Parameter lists of src/gemm/gemm_i8_i8_i32_zve32x.h:50-53, gemm_bf16_bf16_f32_zvfbfwma.h:49-52,
 * gemm_f16_f16_f32_zvfh.h:49-51 (rsa/rsb/rsc are row strides; column strides are 1). */
SKL_FUNC void skl_gemm_i8_i8_i32_sm100a(size_t m, size_t n, size_t k, int32_t alpha,
                                        const int8_t *a, size_t rsa, const int8_t *b, size_t rsb,
                                        int32_t beta, int32_t *c, size_t rsc);
SKL_FUNC void skl_gemm_bf16_bf16_f32_sm100a(size_t m, size_t n, size_t k, float alpha,
                                            const skl_bf16_t *a, size_t rsa, const skl_bf16_t *b,
                                            size_t rsb, float beta, float *c, size_t rsc);
SKL_FUNC void skl_gemm_f16_f16_f32_sm100a(size_t m, size_t n, size_t k, float alpha,
                                          const skl_f16_t *a, size_t rsa, const skl_f16_t *b,
                                          size_t rsb, float beta, float *c, size_t rsc);

/* ------------------------------------------------------------------ GEMM, column-major A, row-major B, C
 * Parameter lists of src/gemm/gemm_i8c_i8_i32_xsfmm32a8i.h:57-60, gemm_bf16c_bf16_f32_xsfmm32a16f.h:56-60,
 * gemm_f16c_f16_f32_xsfmm32a16f.h:56-60, gemm_f8e4m3c_f8e4m3_f32_xsfmm32a8f.h:57-61,
 * gemm_f8e5m2c_f8e5m2_f32_xsfmm32a8f.h:57-61 (csa is the column stride of A; its row stride is 1). */
SKL_FUNC void skl_gemm_i8c_i8_i32_sm100a(size_t m, size_t n, size_t k, int32_t alpha,
                                         const int8_t *a, size_t csa, const int8_t *b, size_t rsb,
                                         int32_t beta, int32_t *c, size_t rsc);
SKL_FUNC void skl_gemm_bf16c_bf16_f32_sm100a(size_t m, size_t n, size_t k, float alpha,
                                             const skl_bf16_t *a, size_t csa, const skl_bf16_t *b,
                                             size_t rsb, float beta, float *c, size_t rsc);
SKL_FUNC void skl_gemm_f16c_f16_f32_sm100a(size_t m, size_t n, size_t k, float alpha,
                                           const skl_f16_t *a, size_t csa, const skl_f16_t *b,
                                           size_t rsb, float beta, float *c, size_t rsc);
SKL_FUNC void skl_gemm_f8e4m3c_f8e4m3_f32_sm100a(size_t m, size_t n, size_t k, float alpha,
                                                 const uint8_t *a, size_t csa, const uint8_t *b,
                                                 size_t rsb, float beta, float *c, size_t rsc);
SKL_FUNC void skl_gemm_f8e5m2c_f8e5m2_f32_sm100a(size_t m, size_t n, size_t k, float alpha,
                                                 const uint8_t *a, size_t csa, const uint8_t *b,
                                                 size_t rsb, float beta, float *c, size_t rsc);

/* ------------------------------------------------------------------ GEMM, packed (blocked 4-D) operands
 * Parameter lists of ref/gemm/gemm_i8rcprc_i8rcprc_i32rcprc.h:50-55 and the bf16 / f16 / f8e4m3 /
 * f8e5m2 siblings: m1 x k1 blocks of m0 x k0 for A, k1 x n1 blocks of k0 x n0 for B, m1 x n1 blocks
 * of m0 x n0 for C; *0 strides inside a block, *1 strides between blocks. */
SKL_FUNC void skl_gemm_i8rcprc_i8rcprc_i32rcprc_sm100a(
    size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1, int32_t alpha, const int8_t *a,
    size_t rsa0, size_t csa0, size_t rsa1, size_t csa1, const int8_t *b, size_t rsb0, size_t csb0,
    size_t rsb1, size_t csb1, int32_t beta, int32_t *c, size_t rsc0, size_t csc0, size_t rsc1,
    size_t csc1);
SKL_FUNC void skl_gemm_bf16rcprc_bf16rcprc_f32rcprc_sm100a(
    size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1, float alpha,
    const skl_bf16_t *a, size_t rsa0, size_t csa0, size_t rsa1, size_t csa1, const skl_bf16_t *b,
    size_t rsb0, size_t csb0, size_t rsb1, size_t csb1, float beta, float *c, size_t rsc0,
    size_t csc0, size_t rsc1, size_t csc1);
SKL_FUNC void skl_gemm_f16rcprc_f16rcprc_f32rcprc_sm100a(
    size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1, float alpha,
    const skl_f16_t *a, size_t rsa0, size_t csa0, size_t rsa1, size_t csa1, const skl_f16_t *b,
    size_t rsb0, size_t csb0, size_t rsb1, size_t csb1, float beta, float *c, size_t rsc0,
    size_t csc0, size_t rsc1, size_t csc1);
SKL_FUNC void skl_gemm_f8e4m3rcprc_f8e4m3rcprc_f32rcprc_sm100a(
    size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1, float alpha, const uint8_t *a,
    size_t rsa0, size_t csa0, size_t rsa1, size_t csa1, const uint8_t *b, size_t rsb0, size_t csb0,
    size_t rsb1, size_t csb1, float beta, float *c, size_t rsc0, size_t csc0, size_t rsc1,
    size_t csc1);
SKL_FUNC void skl_gemm_f8e5m2rcprc_f8e5m2rcprc_f32rcprc_sm100a(
    size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1, float alpha, const uint8_t *a,
    size_t rsa0, size_t csa0, size_t rsa1, size_t csa1, const uint8_t *b, size_t rsb0, size_t csb0,
    size_t rsb1, size_t csb1, float beta, float *c, size_t rsc0, size_t csc0, size_t rsc1,
    size_t csc1);

/* ------------------------------------------------------------------ GEMM, operands packed for the matrix engine
 * Parameter lists of skl_gemm_i8rcptex1c_i8rcp1xte_i32rcptexterc_xsfmm32a8i
 * (src/gemm/gemm_i8c_i8_i32_xsfmm32a8i.h:62-100) and the bf16 / f16 / f8e4m3 / f8e5m2 / f32 siblings
 * (gemm_bf16c_bf16_f32_xsfmm32a16f.h:97-100, gemm_f16c_f16_f32_xsfmm32a16f.h:97-100,
 * gemm_f8e4m3c_f8e4m3_f32_xsfmm32a8f.h:98-101, gemm_f8e5m2c_f8e5m2_f32_xsfmm32a8f.h:98-101,
 * gemm_f32c_f32_f32_xsfmm32a32f.h:96-99).  A is stored as TE x 1 blocks (element (i, kk) of block row i1 at
 * a + i1*rsa1 + kk*csa1 + i), B as 1 x TE blocks (element (kk, j) of block column j1 at b + kk*rsb1 + j1*csb1 + j),
 * C as TE x TE blocks with strides rsc0 / csc0 inside and rsc1 / csc1 between blocks; the matrices are
 * m1*TE x k, k x n1*TE and m1*TE x n1*TE.  Each call equals the general packed entry point with
 * m0 = n0 = TE, k0 = 1, (rsa0, csa0) = (1, 0), (rsb0, csb0) = (0, 1), as those headers state.
 *
 * In SKL the block edge TE is a property of the RISC-V matrix engine.  Here it is a property of the tensor-core
 * path: TE = SKL_B200_TE = 128 elements for every type, the row count of one tcgen05 accumulator tile.  That makes
 * a block row of A (and a block column of B) a run of whole 128-byte rows per k, which TMA loads straight into the
 * shared-memory layout the MMA reads: this is the pre-packed operand layout of this library -- no re-layout pass
 * runs before the GEMM -- and skl_pack_e{8,16,32}_e{8,16,32}rcptex1c_sm100a below produces it.  Index formula for
 * an M x K matrix packed with rs1 = TE*K, cs1 = TE (dense panels): element (i, kk) lives at
 * (i / TE)*TE*K + kk*TE + i % TE.  TMA needs 16-byte aligned bases and csa1 / rsa1 / rsb1 / csb1 that are multiples
 * of 16 bytes; other strides, or problems under 32768 multiply-adds, run on the any-stride kernel. */
#define SKL_B200_TE 128
SKL_FUNC size_t skl_b200_te(void);
SKL_FUNC void skl_gemm_i8rcptex1c_i8rcp1xte_i32rcptexterc_sm100a(
    size_t m1, size_t n1, size_t k, int32_t alpha, const int8_t *a, size_t rsa1, size_t csa1, const int8_t *b,
    size_t rsb1, size_t csb1, int32_t beta, int32_t *c, size_t rsc0, size_t csc0, size_t rsc1, size_t csc1);
SKL_FUNC void skl_gemm_bf16rcptex1c_bf16rcp1xte_f32rcptexterc_sm100a(
    size_t m1, size_t n1, size_t k, float alpha, const skl_bf16_t *a, size_t rsa1, size_t csa1, const skl_bf16_t *b,
    size_t rsb1, size_t csb1, float beta, float *c, size_t rsc0, size_t csc0, size_t rsc1, size_t csc1);
SKL_FUNC void skl_gemm_f16rcptex1c_f16rcp1xte_f32rcptexterc_sm100a(
    size_t m1, size_t n1, size_t k, float alpha, const skl_f16_t *a, size_t rsa1, size_t csa1, const skl_f16_t *b,
    size_t rsb1, size_t csb1, float beta, float *c, size_t rsc0, size_t csc0, size_t rsc1, size_t csc1);
SKL_FUNC void skl_gemm_f8e4m3rcptex1c_f8e4m3rcp1xte_f32rcptexterc_sm100a(
    size_t m1, size_t n1, size_t k, float alpha, const uint8_t *a, size_t rsa1, size_t csa1, const uint8_t *b,
    size_t rsb1, size_t csb1, float beta, float *c, size_t rsc0, size_t csc0, size_t rsc1, size_t csc1);
SKL_FUNC void skl_gemm_f8e5m2rcptex1c_f8e5m2rcp1xte_f32rcptexterc_sm100a(
    size_t m1, size_t n1, size_t k, float alpha, const uint8_t *a, size_t rsa1, size_t csa1, const uint8_t *b,
    size_t rsb1, size_t csb1, float beta, float *c, size_t rsc0, size_t csc0, size_t rsc1, size_t csc1);
SKL_FUNC void skl_gemm_f32rcptex1c_f32rcp1xte_f32rcptexterc_sm100a(
    size_t m1, size_t n1, size_t k, float alpha, const float *a, size_t rsa1, size_t csa1, const float *b,
    size_t rsb1, size_t csb1, float beta, float *c, size_t rsc0, size_t csc0, size_t rsc1, size_t csc1);

/* ------------------------------------------------------------------ GEMM, OCP MX-FP4 operands (no SKL counterpart)
 * SKL stops at the conversion of E2M1 to E4M3 (src/cvt/cvt_f4_f8_zvfofp4min.c:15-41, ref/cvt/cvt_ofp4.c:18-72); this
 * entry multiplies block-scaled E2M1 matrices.  Element (i, kk) of A is the E2M1 value of nibble kk of row i (two per
 * byte, low nibble first, as in SKL's cvt; row i starts at a + i*rsa bytes) times 2^(sa[i*rssa + kk/32] - 127): one
 * E8M0 scale byte per 32 consecutive k, 255 meaning NaN (OCP Microscaling Formats v1.0).  B is given one output column
 * per row of k ("[N][K]"): column j starts at b + j*csb bytes, its scales at sb + j*cssb.  k must be a multiple of 32.
 *     C[i, j] = beta * C[i, j] + alpha * sum_k A[i, k] * B[k, j]      (C row-major fp32, row stride rsc elements)
 * with SKL's float-GEMM conventions: products and sum in fp32 (ref/gemm/gemm_bf16rc_bf16rc_f32rc.c:9-24 with the
 * scaled elements as operands).  Device operands whose packed rows are 16-byte aligned (base and row strides) run on
 * the block-scaled tensor-core instruction; others are widened exactly to bf16 and run on the bf16 kernel.  Results
 * are within the forward bound of the reference's GEMM tests on either path. */
SKL_FUNC void skl_gemm_mxf4e2m1_mxf4e2m1_f32_sm100a(size_t m, size_t n, size_t k, float alpha, const uint8_t *a,
                                                    size_t rsa, const uint8_t *sa, size_t rssa, const uint8_t *b,
                                                    size_t csb, const uint8_t *sb, size_t cssb, float beta, float *c,
                                                    size_t rsc);

/* ------------------------------------------------------------------ GEMM, int8 with 4-deep k blocks
 * Same parameter list as skl_gemm_i8rcp1x4_i8p4x1c_i32_xsfvqdotq
 * (src/gemm/gemm_i8rcp1x4_i8p4x1c_i32_xsfvqdotq.h:70-75): A in 1 x 4 blocks (element (i, k) at
 * i*rsa1 + (k/4)*csa1 + k%4), B in 4 x 1 blocks, column blocks 4 elements apart (element (k, j) at
 * (k/4)*rsb1 + 4*j + k%4), C row-major; K = 4*k1.  Equivalent to the general packed entry with
 * m0 = n0 = 1, k0 = 4, as that header states. */
SKL_FUNC void skl_gemm_i8rcp1x4_i8p4x1c_i32_sm100a(size_t m, size_t n, size_t k1, int32_t alpha, const int8_t *a,
                                                   size_t rsa1, size_t csa1, const int8_t *b, size_t rsb1,
                                                   int32_t beta, int32_t *c, size_t rsc);

/* ------------------------------------------------------------------ GEMM, fp32 and fp64
 * Same parameter lists as skl_gemm_f32rc_f32rc_f32rc_ref / skl_gemm_f64rc_f64rc_f64rc_ref
 * (ref/gemm/gemm_f32rc_f32rc_f32rc.h, gemm_f64rc_f64rc_f64rc.h) and their packed forms
 * (gemm_f32rcprc_f32rcprc_f32rcprc.h, gemm_f64rcprc_f64rcprc_f64rcprc.h).  They run on the CUDA cores
 * (no TF32: that would change the results): one accumulator per output, k ascending, product and sum each
 * rounded once, which reproduces the reference compiled without floating-point contraction bit for bit. */
SKL_FUNC void skl_gemm_f32rc_f32rc_f32rc_sm100a(size_t m, size_t n, size_t k, float alpha, const float *a,
                                                size_t rsa, size_t csa, const float *b, size_t rsb, size_t csb,
                                                float beta, float *c, size_t rsc, size_t csc);
SKL_FUNC void skl_gemm_f32rcprc_f32rcprc_f32rcprc_sm100a(
    size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1, float alpha, const float *a, size_t rsa0,
    size_t csa0, size_t rsa1, size_t csa1, const float *b, size_t rsb0, size_t csb0, size_t rsb1, size_t csb1,
    float beta, float *c, size_t rsc0, size_t csc0, size_t rsc1, size_t csc1);
SKL_FUNC void skl_gemm_f64rc_f64rc_f64rc_sm100a(size_t m, size_t n, size_t k, double alpha, const double *a,
                                                size_t rsa, size_t csa, const double *b, size_t rsb, size_t csb,
                                                double beta, double *c, size_t rsc, size_t csc);
SKL_FUNC void skl_gemm_f64rcprc_f64rcprc_f64rcprc_sm100a(
    size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1, double alpha, const double *a, size_t rsa0,
    size_t csa0, size_t rsa1, size_t csa1, const double *b, size_t rsb0, size_t csb0, size_t rsb1, size_t csb1,
    double beta, double *c, size_t rsc0, size_t csc0, size_t rsc1, size_t csc1);

/* ------------------------------------------------------------------ GEMM, fp16 with an fp16 accumulator
 * Same parameter lists as skl_gemm_f16rc_f16rc_f16rc_ref (ref/gemm/gemm_f16rc_f16rc_f16rc.c:9-22) and its packed
 * form (ref/gemm/gemm_f16rcprc_f16rcprc_f16rcprc.c): fp16 operands, fp16 alpha / beta, an fp16 accumulator and an
 * fp16 C.  The reference's `_Float16` statements have no single defined rounding: a compiler without native
 * half-precision arithmetic evaluates each statement in fp32 and rounds it to fp16 once, a native one rounds after
 * every operation; SKL's own test accepts either within u = 2^-11 per step
 * (test/gemm/gemm_f16rcprc_f16rcprc_f16rcprc.c:155-163).  This library takes the first reading -- acc = h(acc + a*b)
 * for k ascending, C = h(beta*C + alpha*acc), fp32 inside h() -- which is bit-identical to the reference compiled by
 * gcc for x86-64.  Runs on the CUDA cores (the tensor cores accumulate in fp32, which is the other entry points).
 * The by-value fp16 scalars need a compiler with _Float16; the *_f32scalars forms take them as floats instead
 * (rounded to fp16 on entry) for bindings that cannot pass a 16-bit float. */
#if !defined(__CUDACC__) && !defined(SKL_B200_NO_EXT_FLOAT)
SKL_FUNC void skl_gemm_f16rc_f16rc_f16rc_sm100a(size_t m, size_t n, size_t k, skl_f16_t alpha, const skl_f16_t *a,
                                                size_t rsa, size_t csa, const skl_f16_t *b, size_t rsb, size_t csb,
                                                skl_f16_t beta, skl_f16_t *c, size_t rsc, size_t csc);
SKL_FUNC void skl_gemm_f16rcprc_f16rcprc_f16rcprc_sm100a(
    size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1, skl_f16_t alpha, const skl_f16_t *a, size_t rsa0,
    size_t csa0, size_t rsa1, size_t csa1, const skl_f16_t *b, size_t rsb0, size_t csb0, size_t rsb1, size_t csb1,
    skl_f16_t beta, skl_f16_t *c, size_t rsc0, size_t csc0, size_t rsc1, size_t csc1);
#endif
SKL_FUNC void skl_gemm_f16rc_f16rc_f16rc_f32scalars_sm100a(size_t m, size_t n, size_t k, float alpha,
                                                           const skl_f16_t *a, size_t rsa, size_t csa,
                                                           const skl_f16_t *b, size_t rsb, size_t csb, float beta,
                                                           skl_f16_t *c, size_t rsc, size_t csc);
SKL_FUNC void skl_gemm_f16rcprc_f16rcprc_f16rcprc_f32scalars_sm100a(
    size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1, float alpha, const skl_f16_t *a, size_t rsa0,
    size_t csa0, size_t rsa1, size_t csa1, const skl_f16_t *b, size_t rsb0, size_t csb0, size_t rsb1, size_t csb1,
    float beta, skl_f16_t *c, size_t rsc0, size_t csc0, size_t rsc1, size_t csc1);

/* ------------------------------------------------------------------ GEMM with the extended epilogue
 * No SKL counterpart: SKL's outputs are always int32 / fp32 with scalar alpha and beta
 * (src/gemm/README.md:41-47).  This entry adds per-row and per-column fp32 scale vectors, mixed
 * operand formats and a narrowed output, all fused into the accumulator read-out:
 *
 *     acc   = sum_k A[i,k]*B[k,j]      int32 when ta == tb == SKL_B200_I8, else fp32 accumulation
 *     v     = alpha * (float)acc
 *     v     = v * row_scale[i]          when row_scale != NULL   (m entries)
 *     v     = v * col_scale[j]          when col_scale != NULL   (n entries)
 *     v     = beta * (float)C[i,j] + v  when beta != 0
 *     C[i,j]= narrow(v)                 tc: F32 (none), BF16 / F16 (round to nearest even),
 *                                           F8E4M3 (SKL's saturating encoder, ref/cvt/cvt_ofp8.c:97-134),
 *                                           I8 (requantised: nearest even, saturating to [-128, 127], NaN -> 0)
 *
 * every step one fp32 operation with its own rounding, in that order.
 * Operand pairs: I8 x I8; any two of {F8E4M3, F8E5M2}; BF16 x BF16; F16 x F16; and BF16 x F8E4M3 /
 * BF16 x F8E5M2 (the fp8 operand is widened exactly to bf16 first, as skl_cvt_f8e4m3_bf16 does). */
typedef enum skl_b200_dtype {
  SKL_B200_I8 = 0,
  SKL_B200_BF16 = 1,
  SKL_B200_F16 = 2,
  SKL_B200_F8E4M3 = 3,
  SKL_B200_F8E5M2 = 4,
  SKL_B200_F32 = 5,
  SKL_B200_I32 = 6
} skl_b200_dtype_t;

SKL_FUNC void skl_gemm_ex_sm100a(size_t m, size_t n, size_t k, skl_b200_dtype_t ta, const void *a,
                                 size_t rsa, size_t csa, skl_b200_dtype_t tb, const void *b,
                                 size_t rsb, size_t csb, float alpha, const float *row_scale,
                                 const float *col_scale, float beta, skl_b200_dtype_t tc, void *c,
                                 size_t rsc, size_t csc);

/* ------------------------------------------------------------------ GEMM with fused epilogue kernels
 * SKL's matrix-engine GEMMs apply a "fused kernel" to every accumulator tile before it is stored
 * (src/gemm/fused-kernel-API.md:85-108); the one it ships is alpha/beta scaling, the two it documents as
 * examples are adding a bias row vector (:170-192) and tracking the global maximum of the product
 * (:194-217).  This entry provides those on top of the extended epilogue above:
 *
 *     v = alpha*(float)acc;  v *= row_scale[i];  v *= col_scale[j];     (each when its pointer != NULL)
 *     v = v + bias[j]                      when bias != NULL (n entries)
 *     v = beta*(float)C[i,j] + v           when beta != 0
 *     v = act(v)                           when activation != SKL_B200_ACT_NONE (below)
 *     *global_max = max(*global_max, v)    when global_max != NULL (NaN results are ignored; the caller
 *                                          initialises it, e.g. to -INFINITY; updated atomically)
 *     C[i,j] = narrow(v)
 *
 * Activations -- the step SKL names as the next candidate for fusion (src/gemm/README.md:46-47) -- follow the
 * definitions of SKL's element-wise routines (ref/sigmoid/sigmoid_f32.c:10-28, ref/gelu/gelu_f32.c:12-22),
 * evaluated in fp32; the tests hold them to ULP bounds taken from SKL's own activation tests
 * (test/sigmoid/sigmoid_f32_zve32f.c, test/gelu/skl_gelu_f32_zve32f.c):
 *     LOGISTIC  1 / (1 + exp(-act_param * v))                       skl_sigmoid_f32 with beta = act_param
 *     SWISH     v / (1 + exp(-act_param * v))                       skl_swish_f32; act_param = 1 is skl_silu_f32
 *     GELU      max(v, 0) - |v|/2 * erfc(|v| / sqrt 2)              skl_gelu_f32
 *     SWIGLU    v / (1 + exp(-v)) * (C[i,j] + act_param)            skl_swiglu_f32 with gate = v, up = the value
 *               already stored in C[i,j] (e.g. by the up-projection GEMM), delta = act_param; beta must be 0
 *
 * Pointers in the struct may be host or device memory, like every other argument. */
typedef enum skl_b200_activation {
  SKL_B200_ACT_NONE = 0,
  SKL_B200_ACT_LOGISTIC = 1,
  SKL_B200_ACT_SWISH = 2,
  SKL_B200_ACT_GELU = 3,
  SKL_B200_ACT_SWIGLU = 4
} skl_b200_activation_t;

typedef struct skl_b200_fused {
  float alpha;
  float beta;
  const float *row_scale; /* m entries or NULL */
  const float *col_scale; /* n entries or NULL */
  const float *bias;      /* n entries or NULL */
  float *global_max;      /* one float or NULL */
  int activation;         /* skl_b200_activation_t */
  float act_param;        /* see the table above */
} skl_b200_fused_t;

SKL_FUNC void skl_gemm_fused_sm100a(size_t m, size_t n, size_t k, skl_b200_dtype_t ta, const void *a,
                                    size_t rsa, size_t csa, skl_b200_dtype_t tb, const void *b,
                                    size_t rsb, size_t csb, const skl_b200_fused_t *f,
                                    skl_b200_dtype_t tc, void *c, size_t rsc, size_t csc);

/* ------------------------------------------------------------------ GEMM without device allocation
 * No counterpart in the reference: SKL's kernels never allocate because they never need scratch
 * memory, whereas the bf16 x fp8 case above widens B into a workspace obtained with cudaMalloc.
 * Callers that cannot tolerate that -- a latency-bound serving loop (cudaMalloc / cudaFree stall the
 * whole device), or a process whose free device memory is already owned by another allocator's pool,
 * where a cudaMalloc from this library would fail -- use this entry instead.  It computes exactly what
 *     skl_gemm_ex_sm100a(m, n, k, BF16, a, rsa, csa, F8E4M3, b, rsb, csb, alpha, NULL, col_scale, 0, BF16, c, rsc, csc)
 * computes, with the widened B held in a fixed 32 MiB array inside the library image, and it calls
 * no allocating routine.  Consequences of that one shared array:
 *   - every GPU that loads the library carries the 32 MiB until the process exits;
 *   - the widened B (k*n bf16 elements, rows padded to a multiple of 8) must fit in 32 MiB, otherwise
 *     the call is refused with return code 1 and a message naming both sizes;
 *   - the first call on each device resolves the array's device address; make it before any stream
 *     capture begins;
 *   - calls whose GPU work overlaps (other streams, other threads) race on the array: serialise them.
 *     A call returns only after its own work on cuda_stream has finished.
 * All pointers must be device memory (host pointers would need staging, hence an allocation).
 * Returns 0 or a skl_b200_status_t value; on failure a sentence saying why is copied to error_text
 * (error_text_len bytes including the terminator; may be NULL / 0). */
SKL_FUNC int skl_gemm_bf16_f8e4m3_bf16_noalloc_sm100a(size_t m, size_t n, size_t k, float alpha,
                                                      const void *a, size_t rsa, size_t csa,
                                                      const void *b, size_t rsb, size_t csb,
                                                      const float *col_scale, void *c, size_t rsc,
                                                      size_t csc, void *cuda_stream, char *error_text,
                                                      size_t error_text_len);

/* ------------------------------------------------------------------ cvt
 * Parameter lists of ref/cvt/cvt_ofp8.h:59-158 (src/cvt/cvt_f32_f8_zvfofp8min.h:61-112,
 * cvt_bf16_f8_zvfofp8min_zvfbfmin.h:67-122, cvt_f8_bf16_zvfofp8min.h:39-53) and
 * ref/cvt/cvt_ofp4.h (src/cvt/cvt_f4_f8_zvfofp4min.c:15-41): dst[i] = narrow(src[i] * scaling_factor). */
SKL_FUNC void skl_cvt_f32_f8e4m3_sm100a(uint8_t *pDst, const float *pSrc, float scaling_factor, size_t n);
SKL_FUNC void skl_cvt_sat_f32_f8e4m3_sm100a(uint8_t *pDst, const float *pSrc, float scaling_factor, size_t n);
SKL_FUNC void skl_cvt_f32_f8e5m2_sm100a(uint8_t *pDst, const float *pSrc, float scaling_factor, size_t n);
SKL_FUNC void skl_cvt_sat_f32_f8e5m2_sm100a(uint8_t *pDst, const float *pSrc, float scaling_factor, size_t n);
SKL_FUNC void skl_cvt_bf16_f8e4m3_sm100a(uint8_t *pDst, const skl_bf16_t *pSrc, float scaling_factor, size_t n);
SKL_FUNC void skl_cvt_sat_bf16_f8e4m3_sm100a(uint8_t *pDst, const skl_bf16_t *pSrc, float scaling_factor, size_t n);
SKL_FUNC void skl_cvt_bf16_f8e5m2_sm100a(uint8_t *pDst, const skl_bf16_t *pSrc, float scaling_factor, size_t n);
SKL_FUNC void skl_cvt_sat_bf16_f8e5m2_sm100a(uint8_t *pDst, const skl_bf16_t *pSrc, float scaling_factor, size_t n);
SKL_FUNC void skl_cvt_f8e4m3_bf16_sm100a(skl_bf16_t *pDst, const uint8_t *pSrc, size_t n);
SKL_FUNC void skl_cvt_f8e5m2_bf16_sm100a(skl_bf16_t *pDst, const uint8_t *pSrc, size_t n);
SKL_FUNC void skl_cvt_f4e2m1_f8e4m3_sm100a(uint8_t *pDst, const uint8_t *pSrc, size_t n);

/* ------------------------------------------------------------------ pack / unpack / transpose
 * Parameter lists of src/pack/pack_e8_zve32x.h:49-113 (ref/pack/pack_e8rc_e8rcprc.h,
 * unpack_e8rcprc_e8rc.h, transpose_e8.h) and the e16 / e32 siblings. */
SKL_FUNC void skl_pack_e8rc_e8rcprc_sm100a(size_t m, size_t n, const uint8_t *SKL_RESTRICT src,
                                           size_t rs, size_t cs, size_t m0, size_t n0,
                                           uint8_t *SKL_RESTRICT dst, size_t rs0, size_t cs0,
                                           size_t rs1, size_t cs1, uint8_t pad);
SKL_FUNC void skl_pack_e16rc_e16rcprc_sm100a(size_t m, size_t n, const uint16_t *SKL_RESTRICT src,
                                             size_t rs, size_t cs, size_t m0, size_t n0,
                                             uint16_t *SKL_RESTRICT dst, size_t rs0, size_t cs0,
                                             size_t rs1, size_t cs1, uint16_t pad);
SKL_FUNC void skl_pack_e32rc_e32rcprc_sm100a(size_t m, size_t n, const uint32_t *SKL_RESTRICT src,
                                             size_t rs, size_t cs, size_t m0, size_t n0,
                                             uint32_t *SKL_RESTRICT dst, size_t rs0, size_t cs0,
                                             size_t rs1, size_t cs1, uint32_t pad);
/* TE x 1 packing for the matrix-engine GEMMs above: parameter lists of skl_pack_e16_e16rcptex1c_xsfmmbase /
 * skl_pack_e32_e32rcptex1c_xsfmmbase (src/pack/pack_e16_xsfmmbase.h:20-51, pack_e32_xsfmmbase.h:20-51); the e8
 * form, which SKL does not have, serves int8 and fp8.  Each equals the general pack with (m0, n0) = (TE, 1),
 * (rs0, cs0) = (1, 0): row-major src (row stride rs) becomes ceil(m / TE) block rows of TE x 1 blocks, padded with
 * `pad`.  Packing B for the GEMM (1 x TE blocks) is the same call on B's transpose, as in SKL. */
SKL_FUNC void skl_pack_e8_e8rcptex1c_sm100a(size_t m, size_t n, const uint8_t *src, size_t rs, uint8_t *dst,
                                            size_t rs1, size_t cs1, uint8_t pad);
SKL_FUNC void skl_pack_e16_e16rcptex1c_sm100a(size_t m, size_t n, const uint16_t *src, size_t rs, uint16_t *dst,
                                              size_t rs1, size_t cs1, uint16_t pad);
SKL_FUNC void skl_pack_e32_e32rcptex1c_sm100a(size_t m, size_t n, const uint32_t *src, size_t rs, uint32_t *dst,
                                              size_t rs1, size_t cs1, uint32_t pad);
SKL_FUNC void skl_unpack_e8rcprc_e8rc_sm100a(size_t m0, size_t n0, const uint8_t *SKL_RESTRICT src,
                                             size_t rs0, size_t cs0, size_t rs1, size_t cs1,
                                             size_t m, size_t n, uint8_t *SKL_RESTRICT dst,
                                             size_t rs, size_t cs);
SKL_FUNC void skl_transpose_e8_sm100a(size_t m, size_t n, const uint8_t *SKL_RESTRICT a, size_t rsa,
                                      uint8_t *SKL_RESTRICT at, size_t rsat);
SKL_FUNC void skl_transpose_e16_sm100a(size_t m, size_t n, const uint16_t *SKL_RESTRICT a,
                                       size_t rsa, uint16_t *SKL_RESTRICT at, size_t rsat);
SKL_FUNC void skl_transpose_e32_sm100a(size_t m, size_t n, const uint32_t *SKL_RESTRICT a,
                                       size_t rsa, uint32_t *SKL_RESTRICT at, size_t rsat);

#if defined(__cplusplus)
} /* extern "C" */
#endif
#endif /* SKL_B200_H */
