"""ctypes front end for the two CPU checkers.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke test and by the benchmark's CPU-baseline
leg; never by the product package.

* ``port()``  -> this repository's C restatement (oracle/liboracle.so, built by ``make -C oracle port``)
* ``ref()``   -> the reference's own scalar ``_ref`` routines compiled in place
                 (oracle/_ref/libskl-ref.so, ``make -C oracle ref``); ``None`` when it was never built.

All matrices are numpy arrays (any shape, C-contiguous storage); strides are element strides as in
the SKL signatures.  16-bit floats travel as ``uint16`` bit patterns, fp8 as ``uint8``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import threading

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))

I8, BF16, F16, F8E4M3, F8E5M2, F32, I32 = range(7)
F64 = 7
_SZ = C.c_size_t
_VP = C.c_void_p
_F = C.c_float
_I = C.c_int

_port = None
_ref = None
_ref_tried = False


def build(quiet: bool = True) -> None:
    """Build liboracle.so and, where the reference tree is present, _ref/libskl-ref.so."""
    out = subprocess.run(["make", "-C", _DIR, "all"], capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + out.stdout + out.stderr)
    if not quiet:
        print(out.stdout)


def _p(a) -> int:
    if a is None:
        return 0
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    return int(a)


def port():
    global _port
    if _port is None:
        path = os.path.join(_DIR, "liboracle.so")
        if not os.path.exists(path):
            build()
        lib = C.CDLL(path)
        lib.orc_f8e4m3_to_f32.restype = _F
        lib.orc_f8e4m3_to_f32.argtypes = [C.c_uint8]
        lib.orc_f8e5m2_to_f32.restype = _F
        lib.orc_f8e5m2_to_f32.argtypes = [C.c_uint8]
        lib.orc_f32_to_f8e4m3.restype = C.c_uint8
        lib.orc_f32_to_f8e4m3.argtypes = [_F, _I]
        lib.orc_f32_to_f8e5m2.restype = C.c_uint8
        lib.orc_f32_to_f8e5m2.argtypes = [_F, _I]
        lib.orc_f32_to_bf16.restype = C.c_uint16
        lib.orc_f32_to_bf16.argtypes = [_F]
        lib.orc_f32_to_f16.restype = C.c_uint16
        lib.orc_f32_to_f16.argtypes = [_F]
        lib.orc_cvt_f32_f8.argtypes = [_VP, _VP, _F, _SZ, _I, _I]
        lib.orc_cvt_bf16_f8.argtypes = [_VP, _VP, _F, _SZ, _I, _I]
        lib.orc_cvt_f8_bf16.argtypes = [_VP, _VP, _SZ, _I]
        lib.orc_cvt_f4e2m1_f8e4m3.argtypes = [_VP, _VP, _SZ]
        lib.orc_mxf4_element.restype = _F
        lib.orc_mxf4_element.argtypes = [C.c_uint8, C.c_uint8]
        lib.orc_gemm_mxf4.argtypes = [_SZ, _SZ, _SZ, _F, _VP, _SZ, _VP, _SZ, _VP, _SZ, _VP, _SZ, _F, _VP, _SZ]
        lib.orc_gemm_i8_i32.argtypes = [_SZ, _SZ, _SZ, C.c_int32, _VP, _SZ, _SZ, _VP, _SZ, _SZ,
                                        C.c_int32, _VP, _SZ, _SZ]
        lib.orc_gemm_fp_f32.argtypes = [_SZ, _SZ, _SZ, _F, _I, _VP, _SZ, _SZ, _I, _VP, _SZ, _SZ, _F,
                                        _VP, _SZ, _SZ]
        lib.orc_gemm_packed_i8_i32.argtypes = [_SZ] * 6 + [C.c_int32, _VP] + [_SZ] * 4 + [_VP] + \
            [_SZ] * 4 + [C.c_int32, _VP] + [_SZ] * 4
        lib.orc_gemm_packed_fp_f32.argtypes = [_SZ] * 6 + [_F, _I, _VP] + [_SZ] * 4 + [_I, _VP] + \
            [_SZ] * 4 + [_F, _VP] + [_SZ] * 4
        lib.orc_gemm_ex.argtypes = [_SZ, _SZ, _SZ, _I, _VP, _SZ, _SZ, _I, _VP, _SZ, _SZ, _F, _VP, _VP,
                                    _F, _I, _VP, _SZ, _SZ]
        lib.orc_gemm_fused.argtypes = [_SZ, _SZ, _SZ, _I, _VP, _SZ, _SZ, _I, _VP, _SZ, _SZ, _F, _VP, _VP, _VP, _VP,
                                       _F, _I, _F, _I, _VP, _SZ, _SZ]
        lib.orc_gemm_f64.argtypes = [_SZ] * 6 + [C.c_double, _VP] + [_SZ] * 4 + [_VP] + [_SZ] * 4 + \
            [C.c_double, _VP] + [_SZ] * 4
        lib.orc_gemm_f16acc.argtypes = [_SZ] * 6 + [_F, _VP] + [_SZ] * 4 + [_VP] + [_SZ] * 4 + [_F, _VP] + [_SZ] * 4
        lib.orc_activation.argtypes = [_I, _F, _F, _F]
        lib.orc_activation.restype = _F
        lib.orc_pack.argtypes = [_SZ, _SZ, _SZ, _VP, _SZ, _SZ, _SZ, _SZ, _VP, _SZ, _SZ, _SZ, _SZ,
                                 C.c_uint32]
        lib.orc_unpack.argtypes = [_SZ, _SZ, _SZ, _VP, _SZ, _SZ, _SZ, _SZ, _SZ, _SZ, _VP, _SZ, _SZ]
        lib.orc_transpose.argtypes = [_SZ, _SZ, _SZ, _VP, _SZ, _VP, _SZ]
        _port = lib
    return _port


# name fragments of the reference routines per element type
_REF_T = {I8: "i8", BF16: "bf16", F16: "f16", F8E4M3: "f8e4m3", F8E5M2: "f8e5m2"}


def ref():
    """The compiled reference library, or None if oracle/_ref/libskl-ref.so does not exist."""
    global _ref, _ref_tried
    if _ref is None and not _ref_tried:
        _ref_tried = True
        path = os.path.join(_DIR, "_ref", "libskl-ref.so")
        if not os.path.exists(path):
            return None
        lib = C.CDLL(path)
        lib.skl_cvt_f8e4m3_f32.restype = _F
        lib.skl_cvt_f8e4m3_f32.argtypes = [C.c_uint8]
        lib.skl_cvt_f8e5m2_f32.restype = _F
        lib.skl_cvt_f8e5m2_f32.argtypes = [C.c_uint8]
        lib.skl_cvt_f32_f8e4m3.restype = C.c_uint8
        lib.skl_cvt_f32_f8e4m3.argtypes = [_F, C.c_bool]
        lib.skl_cvt_f32_f8e5m2.restype = C.c_uint8
        lib.skl_cvt_f32_f8e5m2.argtypes = [_F, C.c_bool]
        lib.skl_gemm_i8rc_i8rc_i32rc_ref.argtypes = [_SZ, _SZ, _SZ, C.c_int32, _VP, _SZ, _SZ, _VP, _SZ,
                                                     _SZ, C.c_int32, _VP, _SZ, _SZ]
        lib.skl_gemm_i8rcprc_i8rcprc_i32rcprc_ref.argtypes = [_SZ] * 6 + [C.c_int32, _VP] + [_SZ] * 4 + \
            [_VP] + [_SZ] * 4 + [C.c_int32, _VP] + [_SZ] * 4
        for t in ("bf16", "f16", "f8e4m3", "f8e5m2"):
            getattr(lib, f"skl_gemm_{t}rc_{t}rc_f32rc_ref").argtypes = [
                _SZ, _SZ, _SZ, _F, _VP, _SZ, _SZ, _VP, _SZ, _SZ, _F, _VP, _SZ, _SZ]
            getattr(lib, f"skl_gemm_{t}rcprc_{t}rcprc_f32rcprc_ref").argtypes = [_SZ] * 6 + [_F, _VP] + \
                [_SZ] * 4 + [_VP] + [_SZ] * 4 + [_F, _VP] + [_SZ] * 4
        for sat in ("", "sat_"):
            for src in ("f32", "bf16"):
                for f in ("f8e4m3", "f8e5m2"):
                    getattr(lib, f"skl_cvt_{sat}{src}_{f}_ref").argtypes = [_VP, _VP, _F, _SZ]
        for f in ("f8e4m3", "f8e5m2"):
            getattr(lib, f"skl_cvt_{f}_bf16_ref").argtypes = [_VP, _VP, _SZ]
        lib.skl_cvt_f4e2m1_f8e4m3_ref.argtypes = [_VP, _VP, _SZ]
        for e, padt in ((8, C.c_uint8), (16, C.c_uint16), (32, C.c_uint32)):
            getattr(lib, f"skl_pack_e{e}rc_e{e}rcprc_ref").argtypes = [_SZ, _SZ, _VP, _SZ, _SZ, _SZ, _SZ,
                                                                      _VP, _SZ, _SZ, _SZ, _SZ, padt]
            getattr(lib, f"skl_transpose_e{e}_ref").argtypes = [_SZ, _SZ, _VP, _SZ, _VP, _SZ]
        lib.skl_unpack_e8rcprc_e8rc_ref.argtypes = [_SZ, _SZ, _VP, _SZ, _SZ, _SZ, _SZ, _SZ, _SZ, _VP,
                                                    _SZ, _SZ]
        if hasattr(lib, "orc_ref_gemm_f16acc"):  # ref_shim.c: the fp16-accumulate reference with float scalars
            lib.orc_ref_gemm_f16acc.argtypes = [_SZ] * 6 + [_F, _VP] + [_SZ] * 4 + [_VP] + [_SZ] * 4 + [_F, _VP] + \
                [_SZ] * 4
        lib.skl_gemm_f32rc_f32rc_f32rc_ref.argtypes = [_SZ, _SZ, _SZ, _F, _VP, _SZ, _SZ, _VP, _SZ, _SZ, _F, _VP, _SZ,
                                                       _SZ]
        lib.skl_gemm_f64rc_f64rc_f64rc_ref.argtypes = [_SZ, _SZ, _SZ, C.c_double, _VP, _SZ, _SZ, _VP, _SZ, _SZ,
                                                       C.c_double, _VP, _SZ, _SZ]
        lib.skl_gemm_f32rcprc_f32rcprc_f32rcprc_ref.argtypes = [_SZ] * 6 + [_F, _VP] + [_SZ] * 4 + [_VP] + \
            [_SZ] * 4 + [_F, _VP] + [_SZ] * 4
        lib.skl_gemm_f64rcprc_f64rcprc_f64rcprc_ref.argtypes = [_SZ] * 6 + [C.c_double, _VP] + [_SZ] * 4 + [_VP] + \
            [_SZ] * 4 + [C.c_double, _VP] + [_SZ] * 4
        if hasattr(lib, "skl_sigmoid_f32_ref"):  # a library built before the activation files were added lacks them
            lib.skl_sigmoid_f32_ref.argtypes = [_VP, _F, _VP, _VP, _VP, _F, _SZ]
            lib.skl_gelu_f32_ref.argtypes = [_VP, _VP, _SZ]
        _ref = lib
    return _ref


# --------------------------------------------------------------------------- conveniences
def ref_gemm_rc(t: int, m, n, k, alpha, a, rsa, csa, b, rsb, csb, beta, c, rsc, csc) -> None:
    """Call the reference's plain-stride GEMM for a same-type operand pair (t = I8/BF16/F16/F8*)."""
    lib = ref()
    if t == I8:
        lib.skl_gemm_i8rc_i8rc_i32rc_ref(m, n, k, int(alpha), _p(a), rsa, csa, _p(b), rsb, csb,
                                         int(beta), _p(c), rsc, csc)
    else:
        name = _REF_T[t]
        getattr(lib, f"skl_gemm_{name}rc_{name}rc_f32rc_ref")(m, n, k, float(alpha), _p(a), rsa, csa,
                                                             _p(b), rsb, csb, float(beta), _p(c), rsc, csc)


def port_gemm_rc(ta: int, tb: int, m, n, k, alpha, a, rsa, csa, b, rsb, csb, beta, c, rsc, csc) -> None:
    lib = port()
    if ta == I8:
        lib.orc_gemm_i8_i32(m, n, k, int(alpha), _p(a), rsa, csa, _p(b), rsb, csb, int(beta), _p(c),
                            rsc, csc)
    else:
        lib.orc_gemm_fp_f32(m, n, k, float(alpha), ta, _p(a), rsa, csa, tb, _p(b), rsb, csb, float(beta),
                            _p(c), rsc, csc)


def port_gemm_ex(m, n, k, ta, a, rsa, csa, tb, b, rsb, csb, alpha, row_scale, col_scale, beta, tc, c,
                 rsc, csc) -> None:
    port().orc_gemm_ex(m, n, k, ta, _p(a), rsa, csa, tb, _p(b), rsb, csb, float(alpha), _p(row_scale),
                       _p(col_scale), float(beta), tc, _p(c), rsc, csc)


ACT_NONE, ACT_LOGISTIC, ACT_SWISH, ACT_GELU, ACT_SWIGLU = range(5)


def port_gemm_fused(m, n, k, ta, a, rsa, csa, tb, b, rsb, csb, alpha, row_scale, col_scale, bias, global_max, beta,
                    tc, c, rsc, csc, activation: int = ACT_NONE, act_param: float = 0.0) -> None:
    port().orc_gemm_fused(m, n, k, ta, _p(a), rsa, csa, tb, _p(b), rsb, csb, float(alpha), _p(row_scale),
                          _p(col_scale), _p(bias), _p(global_max), float(beta), int(activation), float(act_param),
                          tc, _p(c), rsc, csc)


_ESIZE = {I8: 1, BF16: 2, F16: 2, F8E4M3: 1, F8E5M2: 1, F32: 4, I32: 4}


def esize(t: int) -> int:
    return _ESIZE[t]


def rows_in_parallel(fn, m: int, threads: int) -> None:
    """Run ``fn(i0, rows)`` over disjoint row slabs of [0, m) on ``threads`` host threads.

    ctypes drops the GIL during the foreign call, so the slabs really run side by side; the
    arithmetic inside each output element is untouched (rows are independent in every GEMM here).
    """
    threads = max(1, min(threads, m))
    if threads == 1:
        fn(0, m)
        return
    bounds = [(m * t) // threads for t in range(threads + 1)]
    errs = []

    def work(i0, i1):
        try:
            if i1 > i0:
                fn(i0, i1 - i0)
        except Exception as e:  # pragma: no cover
            errs.append(e)

    ts = [threading.Thread(target=work, args=(bounds[t], bounds[t + 1])) for t in range(threads)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    if errs:
        raise errs[0]
