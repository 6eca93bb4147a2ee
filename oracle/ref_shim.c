/*
 * ref_shim.c -- TEST INFRASTRUCTURE ONLY: entry points into the compiled reference for callers that cannot pass a
 * 16-bit float by value (Python's ctypes).  Linked into oracle/_ref/libskl-ref.so beside the reference's own objects;
 * contains no arithmetic of its own: it converts the two scalars and forwards to
 * skl_gemm_f16rcprc_f16rcprc_f16rcprc_ref (ref/gemm/gemm_f16rcprc_f16rcprc_f16rcprc.c).
 */
#include <stddef.h>

void skl_gemm_f16rcprc_f16rcprc_f16rcprc_ref(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1,
                                             _Float16 alpha, const _Float16 *a, size_t rsa0, size_t csa0, size_t rsa1,
                                             size_t csa1, const _Float16 *b, size_t rsb0, size_t csb0, size_t rsb1,
                                             size_t csb1, _Float16 beta, _Float16 *c, size_t rsc0, size_t csc0,
                                             size_t rsc1, size_t csc1);

void orc_ref_gemm_f16acc(size_t m0, size_t n0, size_t k0, size_t m1, size_t n1, size_t k1, float alpha, const void *a,
                         size_t rsa0, size_t csa0, size_t rsa1, size_t csa1, const void *b, size_t rsb0, size_t csb0,
                         size_t rsb1, size_t csb1, float beta, void *c, size_t rsc0, size_t csc0, size_t rsc1,
                         size_t csc1) {
  skl_gemm_f16rcprc_f16rcprc_f16rcprc_ref(m0, n0, k0, m1, n1, k1, (_Float16)alpha, (const _Float16 *)a, rsa0, csa0, rsa1,
                                          csa1, (const _Float16 *)b, rsb0, csb0, rsb1, csb1, (_Float16)beta,
                                          (_Float16 *)c, rsc0, csc0, rsc1, csc1);
}
