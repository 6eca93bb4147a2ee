"""The oracle port against the compiled reference library on fresh seeded inputs.
Skipped where oracle/_ref/libskl-ref.so was never built (the golden-vector test still runs)."""
import numpy as np
import pytest

import helpers as H
from oracle import pyoracle as orc

P = orc._p
pytestmark = pytest.mark.skipif(orc.ref() is None, reason="compiled reference library not present")

SHAPES = [(1, 1, 1), (7, 7, 7), (17, 17, 17), (1, 64, 64), (64, 1, 64), (4, 5, 0), (15, 17, 31), (33, 129, 20),
          (129, 33, 20), (63, 65, 64)]


@pytest.mark.parametrize("t", [H.I8, H.BF16, H.F16, H.F8E4M3, H.F8E5M2])
@pytest.mark.parametrize("shape", SHAPES)
def test_gemm_rc(t, shape):
    m, n, k = shape
    g = H.rng(hash((t, shape)) & 0xFFFF)
    for (rsa, csa), (rsb, csb), (rsc, csc) in [((max(k, 1), 1), (n, 1), (n, 1)), ((1, m), (1, max(k, 1)), (1, m)),
                                               ((max(k, 1) + 2, 1), (n + 3, 1), (2 * n, 2))]:
        A = H.Strided(t, m, k, rsa, csa, g, all_codes=True)
        B = H.Strided(t, k, n, rsb, csb, g, all_codes=True)
        C0 = H.Strided(H.I32 if t == H.I8 else H.F32, m, n, rsc, csc, g)
        C1 = C0.copy()
        orc.ref_gemm_rc(t, m, n, k, 2, A.view, rsa, csa, B.view, rsb, csb, 3, C0.view, rsc, csc)
        orc.port_gemm_rc(t, t, m, n, k, 2, A.view, rsa, csa, B.view, rsb, csb, 3, C1.view, rsc, csc)
        assert np.array_equal(C0.buf.view(np.uint8), C1.buf.view(np.uint8))


def test_gemm_ex_reduces_to_reference_when_plain():
    """With no scale vectors and fp32 output the extended epilogue is alpha*acc (+ beta*c)."""
    g = H.rng(77)
    m, n, k = 9, 11, 37
    for t in (H.BF16, H.F16, H.F8E4M3, H.F8E5M2):
        A = H.Strided(t, m, k, k, 1, g, all_codes=True)
        B = H.Strided(t, k, n, n, 1, g, all_codes=True)
        C0 = H.Strided(H.F32, m, n, n, 1, g)
        C1 = C0.copy()
        orc.ref_gemm_rc(t, m, n, k, 1.5, A.view, k, 1, B.view, n, 1, 0.5, C0.view, n, 1)
        orc.port_gemm_ex(m, n, k, t, A.view, k, 1, t, B.view, n, 1, 1.5, None, None, 0.5, H.F32, C1.view, n, 1)
        assert np.array_equal(C0.get(), C1.get())


def test_cvt_random_and_boundaries():
    g = H.rng(5)
    x = np.concatenate([g.uniform(-512, 512, 20000), g.normal(0, 1e-3, 5000), g.uniform(-1e5, 1e5, 5000)]).astype(np.float32)
    bits = g.integers(0, 2 ** 32, 50000, dtype=np.uint64).astype(np.uint32)
    x = np.concatenate([x, bits.view(np.float32)])
    xb = H.f32_to_bf16_bits(x)
    ref, port = orc.ref(), orc.port()
    for fmt, f in (("f8e4m3", H.F8E4M3), ("f8e5m2", H.F8E5M2)):
        for sat in ("", "sat_"):
            for scale in (1.0, 1.5, 0.37):
                a = np.zeros(x.size, np.uint8)
                b = np.zeros(x.size, np.uint8)
                getattr(ref, f"skl_cvt_{sat}f32_{fmt}_ref")(P(a), P(x), scale, x.size)
                port.orc_cvt_f32_f8(P(b), P(x), scale, x.size, f, int(sat != ""))
                assert np.array_equal(a, b)
                getattr(ref, f"skl_cvt_{sat}bf16_{fmt}_ref")(P(a), P(xb), scale, x.size)
                port.orc_cvt_bf16_f8(P(b), P(xb), scale, x.size, f, int(sat != ""))
                assert np.array_equal(a, b)


def test_bf16_narrowing_matches_compiler_cast():
    """orc_f32_to_bf16 against the reference's (__bf16) cast, reached through skl_cvt_f8*_bf16_ref for
    the exact cases and through a bf16 GEMM with k = 1 for rounding cases."""
    port = orc.port()
    g = H.rng(9)
    x = g.normal(0, 1, 4096).astype(np.float32)
    got = np.array([port.orc_f32_to_bf16(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(got, H.f32_to_bf16_bits(x))


@pytest.mark.parametrize("e", [8, 16, 32])
def test_pack_unpack_transpose(e):
    ref, port = orc.ref(), orc.port()
    dt = {8: np.uint8, 16: np.uint16, 32: np.uint32}[e]
    g = H.rng(100 + e)
    for (m, n, m0, n0) in [(128, 128, 8, 8), (13, 10, 4, 3), (1, 1, 1, 1), (65, 3, 64, 1), (7, 9, 16, 16)]:
        for src_cm in (0, 1):
            for blk_cm in (0, 1):
                src = g.integers(0, 255, size=m * n).astype(dt)
                rs, cs = (1, m) if src_cm else (n, 1)
                m1, n1 = -(-m // m0), -(-n // n0)
                rs0, cs0 = (1, m0) if blk_cm else (n0, 1)
                rs1, cs1 = n1 * m0 * n0, m0 * n0
                d0 = np.full(m1 * n1 * m0 * n0, 0x11, dtype=dt)
                d1 = d0.copy()
                getattr(ref, f"skl_pack_e{e}rc_e{e}rcprc_ref")(m, n, P(src), rs, cs, m0, n0, P(d0), rs0, cs0, rs1, cs1, 0xFF)
                port.orc_pack(e // 8, m, n, P(src), rs, cs, m0, n0, P(d1), rs0, cs0, rs1, cs1, 0xFF)
                assert np.array_equal(d0, d1)
                if e == 8:
                    b0 = np.zeros(m * n, dtype=dt)
                    b1 = np.zeros(m * n, dtype=dt)
                    ref.skl_unpack_e8rcprc_e8rc_ref(m0, n0, P(d0), rs0, cs0, rs1, cs1, m, n, P(b0), rs, cs)
                    port.orc_unpack(1, m0, n0, P(d0), rs0, cs0, rs1, cs1, m, n, P(b1), rs, cs)
                    assert np.array_equal(b0, b1) and np.array_equal(b0, src)
        a = g.integers(0, 255, size=m * (n + 1)).astype(dt)
        t0 = np.zeros(n * (m + 2), dtype=dt)
        t1 = t0.copy()
        getattr(ref, f"skl_transpose_e{e}_ref")(m, n, P(a), n + 1, P(t0), m + 2)
        port.orc_transpose(e // 8, m, n, P(a), n + 1, P(t1), m + 2)
        assert np.array_equal(t0, t1)


def test_fused_activation_equals_reference_elementwise_routine_on_the_gemm_result():
    """orc_gemm_fused with an activation = the reference GEMM into fp32, then the reference's own element-wise
    routine over the result (skl_sigmoid_f32_ref with its beta / y / up / delta arguments, skl_gelu_f32_ref)."""
    ref = orc.ref()
    if not hasattr(ref, "skl_sigmoid_f32_ref"):
        pytest.skip("reference library built without the activation files")
    g = H.rng(91)
    m, n, k = 13, 21, 48
    A = H.Strided(H.BF16, m, k, k, 1, g)
    B = H.Strided(H.BF16, k, n, n, 1, g)
    plain = np.zeros(m * n, np.float32)
    orc.ref_gemm_rc(H.BF16, m, n, k, 4.0, A.view, k, 1, B.view, n, 1, 0.0, plain, n, 1)
    up = g.normal(0, 2, m * n).astype(np.float32)
    for act, p in ((orc.ACT_LOGISTIC, 1.0), (orc.ACT_LOGISTIC, 0.7), (orc.ACT_SWISH, 1.0), (orc.ACT_SWISH, 2.0),
                   (orc.ACT_GELU, 0.0), (orc.ACT_SWIGLU, 0.5)):
        want = np.zeros(m * n, np.float32)
        if act == orc.ACT_LOGISTIC:
            ref.skl_sigmoid_f32_ref(P(want), p, P(plain), None, None, 0.0, m * n)
        elif act == orc.ACT_SWISH:
            ref.skl_sigmoid_f32_ref(P(want), p, P(plain), P(plain), None, 0.0, m * n)
        elif act == orc.ACT_SWIGLU:
            ref.skl_sigmoid_f32_ref(P(want), 1.0, P(plain), P(plain), P(up), p, m * n)
        else:
            ref.skl_gelu_f32_ref(P(want), P(plain), m * n)
        got = up.copy() if act == orc.ACT_SWIGLU else np.zeros(m * n, np.float32)
        orc.port_gemm_fused(m, n, k, H.BF16, A.view, k, 1, H.BF16, B.view, n, 1, 4.0, None, None, None, None, 0.0,
                            H.F32, got, n, 1, activation=act, act_param=p)
        assert np.array_equal(got, want, equal_nan=True), (act, p)


def test_f32_and_f64_gemm_port_equals_reference():
    """fp32 operands through orc_gemm_fp_f32 and fp64 through orc_gemm_f64 against skl_gemm_f32rc_f32rc_f32rc_ref /
    skl_gemm_f64rc_f64rc_f64rc_ref and the packed forms: bit for bit (same order, no contraction on either side)."""
    ref, port = orc.ref(), orc.port()
    g = H.rng(5)
    for (m, n, k) in [(1, 1, 1), (7, 5, 9), (33, 17, 40), (4, 6, 0)]:
        for dt in (np.float32, np.float64):
            a = g.normal(0, 1, (m, max(k, 1))).astype(dt)
            b = g.normal(0, 1, (max(k, 1), n)).astype(dt)
            c0 = g.normal(0, 1, (m, n)).astype(dt)
            c1 = c0.copy()
            ld = max(k, 1)
            if dt is np.float32:
                ref.skl_gemm_f32rc_f32rc_f32rc_ref(m, n, k, 1.5, P(a), ld, 1, P(b), n, 1, 0.5, P(c0), n, 1)
                port.orc_gemm_fp_f32(m, n, k, 1.5, H.F32, P(a), ld, 1, H.F32, P(b), n, 1, 0.5, P(c1), n, 1)
            else:
                ref.skl_gemm_f64rc_f64rc_f64rc_ref(m, n, k, 1.5, P(a), ld, 1, P(b), n, 1, 0.5, P(c0), n, 1)
                port.orc_gemm_f64(m, n, k, 1, 1, 1, 1.5, P(a), ld, 1, 0, 0, P(b), n, 1, 0, 0, 0.5, P(c1), n, 1, 0, 0)
            assert np.array_equal(c0, c1)
    # packed: blocks 4 x 3 x 2, counts 3 x 2 x 5, column-major inside C's blocks
    m0, n0, k0, m1, n1, k1 = 4, 3, 2, 3, 2, 5
    sa = (k0, 1, k1 * m0 * k0, m0 * k0)
    sb = (1, k0, n1 * k0 * n0, k0 * n0)
    sc = (1, m0, m0 * n0, m1 * m0 * n0)
    for dt in (np.float32, np.float64):
        a = g.normal(0, 1, m1 * k1 * m0 * k0).astype(dt)
        b = g.normal(0, 1, k1 * n1 * k0 * n0).astype(dt)
        c0 = g.normal(0, 1, m1 * n1 * m0 * n0).astype(dt)
        c1 = c0.copy()
        if dt is np.float32:
            ref.skl_gemm_f32rcprc_f32rcprc_f32rcprc_ref(m0, n0, k0, m1, n1, k1, 2.0, P(a), *sa, P(b), *sb, 3.0, P(c0), *sc)
            port.orc_gemm_packed_fp_f32(m0, n0, k0, m1, n1, k1, 2.0, H.F32, P(a), *sa, H.F32, P(b), *sb, 3.0, P(c1), *sc)
        else:
            ref.skl_gemm_f64rcprc_f64rcprc_f64rcprc_ref(m0, n0, k0, m1, n1, k1, 2.0, P(a), *sa, P(b), *sb, 3.0, P(c0), *sc)
            port.orc_gemm_f64(m0, n0, k0, m1, n1, k1, 2.0, P(a), *sa, P(b), *sb, 3.0, P(c1), *sc)
        assert np.array_equal(c0, c1)


def test_int8_wrap_around_equals_reference():
    """alpha and beta large enough that beta*C and alpha*acc wrap in int32: the port's unsigned arithmetic must
    give what the reference's signed expression gives on this target."""
    ref, port = orc.ref(), orc.port()
    g = H.rng(17)
    m, n, k = 9, 13, 96
    a = g.integers(-128, 128, size=(m, k), dtype=np.int8)
    b = g.integers(-128, 128, size=(k, n), dtype=np.int8)
    c0 = g.integers(-2**31, 2**31, size=(m, n), dtype=np.int64).astype(np.int32)
    c1 = c0.copy()
    alpha, beta = 0x01000001, -0x7FFFFFF
    ref.skl_gemm_i8rc_i8rc_i32rc_ref(m, n, k, alpha, P(a), k, 1, P(b), n, 1, beta, P(c0), n, 1)
    port.orc_gemm_i8_i32(m, n, k, alpha, P(a), k, 1, P(b), n, 1, beta, P(c1), n, 1)
    assert np.array_equal(c0, c1)


@pytest.mark.parametrize("shape", [(1, 1, 1), (7, 9, 33), (17, 5, 300), (4, 5, 0), (33, 20, 64)])
def test_f16_accumulate_gemm_port_equals_compiled_reference(shape):
    """ref/gemm/gemm_f16rc_f16rc_f16rc.c / gemm_f16rcprc_f16rcprc_f16rcprc.c: the port states each `_Float16` statement
    as one fp32 evaluation rounded to fp16; the reference compiled by this toolchain must agree bit for bit (plain
    and blocked operands)."""
    ref, port = orc.ref(), orc.port()
    if not hasattr(ref, "orc_ref_gemm_f16acc"):
        pytest.skip("reference library built without the fp16-scalar shim")
    m, n, k = shape
    g = H.rng(m * 100 + n * 10 + k)
    for blocked in (False, True):
        if blocked:
            m0, n0, k0, m1, n1, k1 = 2, 3, 2, m, n, (k + 1) // 2
            sa = (k0, 1, max(k1, 1) * m0 * k0, m0 * k0)
            sb = (1, k0, n1 * k0 * n0, k0 * n0)
            sc = (1, m0, m0 * n0, m1 * m0 * n0)
            na, nb, ncc = m1 * max(k1, 1) * m0 * k0, max(k1, 1) * n1 * k0 * n0, m1 * n1 * m0 * n0
        else:
            m0, n0, k0, m1, n1, k1 = m, n, k, 1, 1, 1
            sa, sb, sc = (max(k, 1), 1, 0, 0), (n, 1, 0, 0), (n, 1, 0, 0)
            na, nb, ncc = m * max(k, 1), max(k, 1) * n, m * n
        a = H.f32_to_f16_bits(g.uniform(-2, 2, na).astype(np.float32))
        b = H.f32_to_f16_bits(g.uniform(-2, 2, nb).astype(np.float32))
        c0 = H.f32_to_f16_bits(g.uniform(-8, 8, ncc).astype(np.float32))
        for alpha, beta in ((1.0, 0.0), (1.25, -0.75)):
            want, got = c0.copy(), c0.copy()
            ref.orc_ref_gemm_f16acc(m0, n0, k0, m1, n1, k1, alpha, P(a), *sa, P(b), *sb, beta, P(want), *sc)
            port.orc_gemm_f16acc(m0, n0, k0, m1, n1, k1, alpha, P(a), *sa, P(b), *sb, beta, P(got), *sc)
            assert np.array_equal(want, got)


def test_fp8_encoders_against_the_reference_on_a_sample_of_all_inputs():
    """`make -C oracle check-cvt CVT_STRIDE=n`: the port's encoders and decoders against the compiled reference on every
    n-th fp32 bit pattern (offsets rotating through all residues), both formats, both overflow flavours.  The full
    sweep (CVT_STRIDE=1, all 2^32 patterns, about half a minute) runs when SKL_B200_FULL_CVT_CHECK=1."""
    import os
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    stride = "1" if os.environ.get("SKL_B200_FULL_CVT_CHECK") == "1" else "257"
    out = subprocess.run(["make", "-C", os.path.join(root, "oracle"), "check-cvt", f"CVT_STRIDE={stride}"],
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "decode mismatches: 0" in out.stdout
    assert "flavours: 0" in out.stdout


def test_mxf4_element_decode_is_the_reference_f4_table_times_a_power_of_two():
    """The MX-FP4 GEMM has no reference routine; its element decode is pinned: E2M1 value = the reference's
    skl_cvt_f4e2m1_f8e4m3 followed by its E4M3 decode (ref/cvt/cvt_ofp4.c:18-72, cvt_ofp8.c:18-52), scale = 2^(s - 127)."""
    ref, port = orc.ref(), orc.port()
    src = np.array([lo | (hi << 4) for lo, hi in zip(range(0, 16, 2), range(1, 16, 2))], np.uint8)
    f8 = np.zeros(16, np.uint8)
    ref.skl_cvt_f4e2m1_f8e4m3_ref(P(f8), P(src), 16)
    for code in range(16):
        base = port.orc_f8e4m3_to_f32(int(f8[code]))
        for s in (0, 1, 100, 127, 128, 200, 254):
            want = np.float32(base) * np.float32(2.0) ** np.float32(s - 127) if s else np.float32(base) * np.float32(2.0 ** -127)
            got = np.float32(port.orc_mxf4_element(code, s))
            assert got.view(np.uint32) == np.float32(want).view(np.uint32), (code, s)
        assert np.isnan(port.orc_mxf4_element(code, 255))
