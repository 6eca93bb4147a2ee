"""skl_b200 -- Python binding of libskl_b200.so (the sm_100a build of SKL's gemm / pack / cvt path).

The product is the C library declared in ``include/skl-b200.h``; this module only loads it through
ctypes and declares the argument types, so tests and benchmarks can call the very same entry points
a C caller links against.  There is no Python or CPU implementation behind these functions: if the
library has not been built, ``lib()`` raises.

Pointers: pass ``ptr(x)`` of a numpy array (host memory -- the library stages it) or of a CUDA torch
tensor (device memory -- used in place).  16-bit floats are raw ``uint16`` patterns on the numpy side.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libskl_b200.so")

# skl_b200_dtype_t
I8, BF16, F16, F8E4M3, F8E5M2, F32, I32 = range(7)
F64 = 7
# skl_b200_path_t
PATH_NONE, PATH_GENERIC, PATH_TCGEN05, PATH_GEMV = range(4)

_SZ, _VP, _F, _I, _I32 = C.c_size_t, C.c_void_p, C.c_float, C.c_int, C.c_int32

_GEMM_RC_I = [_SZ, _SZ, _SZ, _I32, _VP, _SZ, _SZ, _VP, _SZ, _SZ, _I32, _VP, _SZ, _SZ]
_GEMM_RC_F = [_SZ, _SZ, _SZ, _F, _VP, _SZ, _SZ, _VP, _SZ, _SZ, _F, _VP, _SZ, _SZ]
_GEMM_R_I = [_SZ, _SZ, _SZ, _I32, _VP, _SZ, _VP, _SZ, _I32, _VP, _SZ]
_GEMM_R_F = [_SZ, _SZ, _SZ, _F, _VP, _SZ, _VP, _SZ, _F, _VP, _SZ]
_GEMM_P_I = [_SZ] * 6 + [_I32, _VP] + [_SZ] * 4 + [_VP] + [_SZ] * 4 + [_I32, _VP] + [_SZ] * 4
_GEMM_P_F = [_SZ] * 6 + [_F, _VP] + [_SZ] * 4 + [_VP] + [_SZ] * 4 + [_F, _VP] + [_SZ] * 4

_GEMM_TE_I = [_SZ, _SZ, _SZ, _I32, _VP, _SZ, _SZ, _VP, _SZ, _SZ, _I32, _VP, _SZ, _SZ, _SZ, _SZ]
_GEMM_TE_F = [_SZ, _SZ, _SZ, _F, _VP, _SZ, _SZ, _VP, _SZ, _SZ, _F, _VP, _SZ, _SZ, _SZ, _SZ]

# every symbol include/skl-b200.h declares -> ctypes argument list (restype None unless noted)
SIGNATURES = {
    "skl_b200_last_status": ([], _I),
    "skl_b200_status_string": ([_I], C.c_char_p),
    "skl_b200_last_cuda_error": ([], C.c_char_p),
    "skl_b200_set_stream": ([_VP], None),
    "skl_b200_get_stream": ([], _VP),
    "skl_b200_set_async": ([_I], None),
    "skl_b200_synchronize": ([], None),
    "skl_b200_release_workspace": ([], None),
    "skl_b200_set_static_weights": ([_I], None),
    "skl_b200_last_path": ([], _I),
    "skl_b200_last_launch_count": ([], _I),
    "skl_b200_force_path": ([_I], None),
    "skl_b200_set_wait_limit": ([C.c_uint], None),
    "skl_b200_debug_skip_loads": ([_I], None),
    "skl_b200_profile_begin": ([_I], None),
    "skl_b200_profile_end": ([C.POINTER(C.c_double)], _I),
    "skl_b200_shard_columns": ([_SZ, _SZ, _SZ, _SZ, C.POINTER(_SZ), C.POINTER(_SZ)], None),
    "skl_b200_unshard_columns_sm100a": ([_SZ, _SZ, _SZ, _SZ, _SZ, _VP, _SZ, _VP, _SZ], None),
    "skl_gemm_i8rc_i8rc_i32rc_sm100a": (_GEMM_RC_I, None),
    "skl_gemm_bf16rc_bf16rc_f32rc_sm100a": (_GEMM_RC_F, None),
    "skl_gemm_f16rc_f16rc_f32rc_sm100a": (_GEMM_RC_F, None),
    "skl_gemm_f8e4m3rc_f8e4m3rc_f32rc_sm100a": (_GEMM_RC_F, None),
    "skl_gemm_f8e5m2rc_f8e5m2rc_f32rc_sm100a": (_GEMM_RC_F, None),
    "skl_gemm_i8_i8_i32_sm100a": (_GEMM_R_I, None),
    "skl_gemm_bf16_bf16_f32_sm100a": (_GEMM_R_F, None),
    "skl_gemm_f16_f16_f32_sm100a": (_GEMM_R_F, None),
    "skl_gemm_i8c_i8_i32_sm100a": (_GEMM_R_I, None),
    "skl_gemm_bf16c_bf16_f32_sm100a": (_GEMM_R_F, None),
    "skl_gemm_f16c_f16_f32_sm100a": (_GEMM_R_F, None),
    "skl_gemm_f8e4m3c_f8e4m3_f32_sm100a": (_GEMM_R_F, None),
    "skl_gemm_f8e5m2c_f8e5m2_f32_sm100a": (_GEMM_R_F, None),
    "skl_b200_te": ([], _SZ),
    "skl_gemm_mxf4e2m1_mxf4e2m1_f32_sm100a": ([_SZ, _SZ, _SZ, _F, _VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _F, _VP, _SZ], None),
    "skl_gemm_i8rcptex1c_i8rcp1xte_i32rcptexterc_sm100a": (_GEMM_TE_I, None),
    "skl_gemm_bf16rcptex1c_bf16rcp1xte_f32rcptexterc_sm100a": (_GEMM_TE_F, None),
    "skl_gemm_f16rcptex1c_f16rcp1xte_f32rcptexterc_sm100a": (_GEMM_TE_F, None),
    "skl_gemm_f8e4m3rcptex1c_f8e4m3rcp1xte_f32rcptexterc_sm100a": (_GEMM_TE_F, None),
    "skl_gemm_f8e5m2rcptex1c_f8e5m2rcp1xte_f32rcptexterc_sm100a": (_GEMM_TE_F, None),
    "skl_gemm_f32rcptex1c_f32rcp1xte_f32rcptexterc_sm100a": (_GEMM_TE_F, None),
    "skl_pack_e8_e8rcptex1c_sm100a": ([_SZ, _SZ, _VP, _SZ, _VP, _SZ, _SZ, C.c_uint8], None),
    "skl_pack_e16_e16rcptex1c_sm100a": ([_SZ, _SZ, _VP, _SZ, _VP, _SZ, _SZ, C.c_uint16], None),
    "skl_pack_e32_e32rcptex1c_sm100a": ([_SZ, _SZ, _VP, _SZ, _VP, _SZ, _SZ, C.c_uint32], None),
    "skl_gemm_i8rcp1x4_i8p4x1c_i32_sm100a": ([_SZ, _SZ, _SZ, _I32, _VP, _SZ, _SZ, _VP, _SZ, _I32, _VP, _SZ], None),
    # fp16 scalars by value cannot be passed through ctypes: declared and exported, called through the *_f32scalars forms
    "skl_gemm_f16rc_f16rc_f16rc_sm100a": None,
    "skl_gemm_f16rcprc_f16rcprc_f16rcprc_sm100a": None,
    "skl_gemm_f16rc_f16rc_f16rc_f32scalars_sm100a": (_GEMM_RC_F, None),
    "skl_gemm_f16rcprc_f16rcprc_f16rcprc_f32scalars_sm100a": (_GEMM_P_F, None),
    "skl_gemm_f32rc_f32rc_f32rc_sm100a": (_GEMM_RC_F, None),
    "skl_gemm_f64rc_f64rc_f64rc_sm100a": ([_SZ, _SZ, _SZ, C.c_double, _VP, _SZ, _SZ, _VP, _SZ, _SZ, C.c_double, _VP,
                                           _SZ, _SZ], None),
    "skl_gemm_f32rcprc_f32rcprc_f32rcprc_sm100a": (_GEMM_P_F, None),
    "skl_gemm_f64rcprc_f64rcprc_f64rcprc_sm100a": ([_SZ] * 6 + [C.c_double, _VP] + [_SZ] * 4 + [_VP] + [_SZ] * 4 +
                                                   [C.c_double, _VP] + [_SZ] * 4, None),
    "skl_gemm_i8rcprc_i8rcprc_i32rcprc_sm100a": (_GEMM_P_I, None),
    "skl_gemm_bf16rcprc_bf16rcprc_f32rcprc_sm100a": (_GEMM_P_F, None),
    "skl_gemm_f16rcprc_f16rcprc_f32rcprc_sm100a": (_GEMM_P_F, None),
    "skl_gemm_f8e4m3rcprc_f8e4m3rcprc_f32rcprc_sm100a": (_GEMM_P_F, None),
    "skl_gemm_f8e5m2rcprc_f8e5m2rcprc_f32rcprc_sm100a": (_GEMM_P_F, None),
    "skl_gemm_ex_sm100a": ([_SZ, _SZ, _SZ, _I, _VP, _SZ, _SZ, _I, _VP, _SZ, _SZ, _F, _VP, _VP, _F, _I,
                            _VP, _SZ, _SZ], None),
    "skl_gemm_fused_sm100a": ([_SZ, _SZ, _SZ, _I, _VP, _SZ, _SZ, _I, _VP, _SZ, _SZ, _VP, _I, _VP, _SZ, _SZ], None),
    "skl_gemm_bf16_f8e4m3_bf16_noalloc_sm100a": ([_SZ, _SZ, _SZ, _F, _VP, _SZ, _SZ, _VP, _SZ, _SZ, _VP, _VP, _SZ,
                                                  _SZ, _VP, C.c_char_p, _SZ], _I),
    "skl_cvt_f32_f8e4m3_sm100a": ([_VP, _VP, _F, _SZ], None),
    "skl_cvt_sat_f32_f8e4m3_sm100a": ([_VP, _VP, _F, _SZ], None),
    "skl_cvt_f32_f8e5m2_sm100a": ([_VP, _VP, _F, _SZ], None),
    "skl_cvt_sat_f32_f8e5m2_sm100a": ([_VP, _VP, _F, _SZ], None),
    "skl_cvt_bf16_f8e4m3_sm100a": ([_VP, _VP, _F, _SZ], None),
    "skl_cvt_sat_bf16_f8e4m3_sm100a": ([_VP, _VP, _F, _SZ], None),
    "skl_cvt_bf16_f8e5m2_sm100a": ([_VP, _VP, _F, _SZ], None),
    "skl_cvt_sat_bf16_f8e5m2_sm100a": ([_VP, _VP, _F, _SZ], None),
    "skl_cvt_f8e4m3_bf16_sm100a": ([_VP, _VP, _SZ], None),
    "skl_cvt_f8e5m2_bf16_sm100a": ([_VP, _VP, _SZ], None),
    "skl_cvt_f4e2m1_f8e4m3_sm100a": ([_VP, _VP, _SZ], None),
    "skl_pack_e8rc_e8rcprc_sm100a": ([_SZ, _SZ, _VP, _SZ, _SZ, _SZ, _SZ, _VP, _SZ, _SZ, _SZ, _SZ, C.c_uint8],
                                     None),
    "skl_pack_e16rc_e16rcprc_sm100a": ([_SZ, _SZ, _VP, _SZ, _SZ, _SZ, _SZ, _VP, _SZ, _SZ, _SZ, _SZ,
                                        C.c_uint16], None),
    "skl_pack_e32rc_e32rcprc_sm100a": ([_SZ, _SZ, _VP, _SZ, _SZ, _SZ, _SZ, _VP, _SZ, _SZ, _SZ, _SZ,
                                        C.c_uint32], None),
    "skl_unpack_e8rcprc_e8rc_sm100a": ([_SZ, _SZ, _VP, _SZ, _SZ, _SZ, _SZ, _SZ, _SZ, _VP, _SZ, _SZ], None),
    "skl_transpose_e8_sm100a": ([_SZ, _SZ, _VP, _SZ, _VP, _SZ], None),
    "skl_transpose_e16_sm100a": ([_SZ, _SZ, _VP, _SZ, _VP, _SZ], None),
    "skl_transpose_e32_sm100a": ([_SZ, _SZ, _VP, _SZ, _VP, _SZ], None),
}

# launch-ABI symbols tests reach directly (device-side self check)
_ABI_SIGNATURES = {
    "skl_b200_launch_cvt_selfcheck": ([_I, _I, C.c_uint64, C.c_uint64, _VP, _VP], _I),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library with argument types declared.  Raises if it was never built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m skl_b200._build` "
                "(there is no fallback implementation)")
        handle = C.CDLL(LIB_PATH)
        for table in (SIGNATURES, _ABI_SIGNATURES):
            for name, sig in table.items():
                fn = getattr(handle, name)
                if sig is None:  # exported, but its by-value arguments have no ctypes form
                    continue
                fn.argtypes, fn.restype = sig
        _lib = handle
    return _lib


def ptr(x) -> int:
    """Address of a numpy array's or torch tensor's first element (0 for None)."""
    if x is None:
        return 0
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    return int(x)


class Fused(C.Structure):
    """skl_b200_fused_t"""
    _fields_ = [("alpha", C.c_float), ("beta", C.c_float), ("row_scale", C.c_void_p), ("col_scale", C.c_void_p),
                ("bias", C.c_void_p), ("global_max", C.c_void_p), ("activation", C.c_int), ("act_param", C.c_float)]


ACT_NONE, ACT_LOGISTIC, ACT_SWISH, ACT_GELU, ACT_SWIGLU = range(5)


class SklB200Error(RuntimeError):
    pass


def check() -> None:
    """Raise if the calling thread's last library call recorded an error."""
    L = lib()
    st = L.skl_b200_last_status()
    if st != 0:
        raise SklB200Error(f"{L.skl_b200_status_string(st).decode()}: {L.skl_b200_last_cuda_error().decode()}")


def shard_columns(n: int, parts: int, index: int, align: int = 1) -> tuple[int, int]:
    s, c = _SZ(0), _SZ(0)
    lib().skl_b200_shard_columns(n, parts, index, align, C.byref(s), C.byref(c))
    return s.value, c.value
