/*
 * skl-b200-compat.h -- optional source compatibility with code written against SKL's RISC-V names.
 *
 * SKL names each optimised kernel after the ISA extension it needs (src/README.md:5-22), e.g.
 * skl_gemm_i8_i8_i32_zve32x_x390.  Including this header after skl-b200.h maps those names onto the
 * sm100a entry points with the same parameter lists, so a caller's source compiles unchanged.
 * The packed matrix-engine entry points (…rcptex1c…) are mapped too; their block edge TE, a property of the
 * RISC-V matrix engine in SKL, is SKL_B200_TE here, so callers must pack with that value (SKL code reads it from
 * the hardware at run time; here it is skl_b200_te()).
 */
#ifndef SKL_B200_COMPAT_H
#define SKL_B200_COMPAT_H

#include "skl-b200.h"

/* row-major GEMMs: src/gemm/gemm_i8_i8_i32_zve32x.h:50-53 and siblings */
#define skl_gemm_i8_i8_i32_zve32x skl_gemm_i8_i8_i32_sm100a
#define skl_gemm_i8_i8_i32_zve32x_x390 skl_gemm_i8_i8_i32_sm100a
#define skl_gemm_bf16_bf16_f32_zvfbfwma skl_gemm_bf16_bf16_f32_sm100a
#define skl_gemm_bf16_bf16_f32_zvfbfwma_x390 skl_gemm_bf16_bf16_f32_sm100a
#define skl_gemm_f16_f16_f32_zvfh skl_gemm_f16_f16_f32_sm100a
#define skl_gemm_f16_f16_f32_zvfh_x390 skl_gemm_f16_f16_f32_sm100a

/* column-major-A GEMMs: src/gemm/gemm_i8c_i8_i32_xsfmm32a8i.h:57-60 and siblings */
#define skl_gemm_i8c_i8_i32_xsfmm32a8i skl_gemm_i8c_i8_i32_sm100a
#define skl_gemm_i8rcp1x4_i8p4x1c_i32_xsfvqdotq skl_gemm_i8rcp1x4_i8p4x1c_i32_sm100a
#define skl_gemm_bf16c_bf16_f32_xsfmm32a16f skl_gemm_bf16c_bf16_f32_sm100a
#define skl_gemm_f16c_f16_f32_xsfmm32a16f skl_gemm_f16c_f16_f32_sm100a
#define skl_gemm_f8e4m3c_f8e4m3_f32_xsfmm32a8f skl_gemm_f8e4m3c_f8e4m3_f32_sm100a
#define skl_gemm_f8e5m2c_f8e5m2_f32_xsfmm32a8f skl_gemm_f8e5m2c_f8e5m2_f32_sm100a

/* packed matrix-engine GEMMs: src/gemm/gemm_i8c_i8_i32_xsfmm32a8i.h:97-100 and siblings */
#define skl_gemm_i8rcptex1c_i8rcp1xte_i32rcptexterc_xsfmm32a8i skl_gemm_i8rcptex1c_i8rcp1xte_i32rcptexterc_sm100a
#define skl_gemm_bf16rcptex1c_bf16rcp1xte_f32rcptexterc_xsfmm32a16f skl_gemm_bf16rcptex1c_bf16rcp1xte_f32rcptexterc_sm100a
#define skl_gemm_f16rcptex1c_f16rcp1xte_f32rcptexterc_xsfmm32a16f skl_gemm_f16rcptex1c_f16rcp1xte_f32rcptexterc_sm100a
#define skl_gemm_f8e4m3rcptex1c_f8e4m3rcp1xte_f32rcptexterc_xsfmm32a8f skl_gemm_f8e4m3rcptex1c_f8e4m3rcp1xte_f32rcptexterc_sm100a
#define skl_gemm_f8e5m2rcptex1c_f8e5m2rcp1xte_f32rcptexterc_xsfmm32a8f skl_gemm_f8e5m2rcptex1c_f8e5m2rcp1xte_f32rcptexterc_sm100a
#define skl_gemm_f32rcptex1c_f32rcp1xte_f32rcptexterc_xsfmm32a32f skl_gemm_f32rcptex1c_f32rcp1xte_f32rcptexterc_sm100a

/* general-stride reference names: include/skl-ref.h */
#define skl_gemm_i8rc_i8rc_i32rc_ref skl_gemm_i8rc_i8rc_i32rc_sm100a
#define skl_gemm_bf16rc_bf16rc_f32rc_ref skl_gemm_bf16rc_bf16rc_f32rc_sm100a
#define skl_gemm_f16rc_f16rc_f32rc_ref skl_gemm_f16rc_f16rc_f32rc_sm100a
#define skl_gemm_f8e4m3rc_f8e4m3rc_f32rc_ref skl_gemm_f8e4m3rc_f8e4m3rc_f32rc_sm100a
#define skl_gemm_f8e5m2rc_f8e5m2rc_f32rc_ref skl_gemm_f8e5m2rc_f8e5m2rc_f32rc_sm100a

/* cvt: src/cvt/cvt_f32_f8_zvfofp8min.h:61-112, cvt_bf16_f8_zvfofp8min_zvfbfmin.h:67-122,
 * cvt_f8_bf16_zvfofp8min.h:39-53, cvt_f4_f8_zvfofp4min.c:15-41 */
#define skl_cvt_f32_f8e4m3_zvfofp8min skl_cvt_f32_f8e4m3_sm100a
#define skl_cvt_sat_f32_f8e4m3_zvfofp8min skl_cvt_sat_f32_f8e4m3_sm100a
#define skl_cvt_f32_f8e5m2_zvfofp8min skl_cvt_f32_f8e5m2_sm100a
#define skl_cvt_sat_f32_f8e5m2_zvfofp8min skl_cvt_sat_f32_f8e5m2_sm100a
#define skl_cvt_bf16_f8e4m3_zvfofp8min_zvfbfmin skl_cvt_bf16_f8e4m3_sm100a
#define skl_cvt_sat_bf16_f8e4m3_zvfofp8min_zvfbfmin skl_cvt_sat_bf16_f8e4m3_sm100a
#define skl_cvt_bf16_f8e5m2_zvfofp8min_zvfbfmin skl_cvt_bf16_f8e5m2_sm100a
#define skl_cvt_sat_bf16_f8e5m2_zvfofp8min_zvfbfmin skl_cvt_sat_bf16_f8e5m2_sm100a
#define skl_cvt_f8e4m3_bf16_zvfofp8min skl_cvt_f8e4m3_bf16_sm100a
#define skl_cvt_f8e5m2_bf16_zvfofp8min skl_cvt_f8e5m2_bf16_sm100a
#define skl_cvt_f4e2m1_f8e4m3_zvfofp4min skl_cvt_f4e2m1_f8e4m3_sm100a

/* pack / unpack / transpose: src/pack/pack_e8_zve32x.h:49-113 and e16 / e32 siblings,
 * src/pack/pack_e16_xsfmmbase.h:49-72, pack_e32_xsfmmbase.h:49-72 */
#define skl_pack_e8rc_e8rcprc_zve32x skl_pack_e8rc_e8rcprc_sm100a
#define skl_pack_e16rc_e16rcprc_zve32x skl_pack_e16rc_e16rcprc_sm100a
#define skl_pack_e32rc_e32rcprc_zve32x skl_pack_e32rc_e32rcprc_sm100a
#define skl_pack_e16_e16rcptex1c_xsfmmbase skl_pack_e16_e16rcptex1c_sm100a
#define skl_pack_e32_e32rcptex1c_xsfmmbase skl_pack_e32_e32rcptex1c_sm100a
#define skl_unpack_e8rcprc_e8rc_zve32x skl_unpack_e8rcprc_e8rc_sm100a
#define skl_transpose_e8_zve32x skl_transpose_e8_sm100a
#define skl_transpose_e16_zve32x skl_transpose_e16_sm100a
#define skl_transpose_e32_zve32x skl_transpose_e32_sm100a
#define skl_transpose_e8_xsfmmbase skl_transpose_e8_sm100a
#define skl_transpose_e16_xsfmmbase skl_transpose_e16_sm100a
#define skl_transpose_e32_xsfmmbase skl_transpose_e32_sm100a

#endif /* SKL_B200_COMPAT_H */
