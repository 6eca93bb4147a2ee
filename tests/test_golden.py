"""The oracle port against golden vectors produced by the reference's own `_ref` routines
(tests/golden/make_golden.py).  CPU only; needs neither the reference tree nor a GPU."""
import os

import numpy as np
import pytest

import helpers as H
from oracle import pyoracle as orc

P = orc._p
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "skl_ref_golden.npz"))
NAMES = {H.I8: "i8", H.BF16: "bf16", H.F16: "f16", H.F8E4M3: "f8e4m3", H.F8E5M2: "f8e5m2"}


def bits_equal(a, b):
    return a.dtype == b.dtype and a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


@pytest.mark.parametrize("case", range(int(GOLD["gemm_rc_count"][0])))
def test_gemm_rc_port_matches_reference_vectors(case):
    key = f"gemm_rc_{case}"
    t, m, n, k, rsa, csa, rsb, csb, rsc, csc, alpha, beta, aoff, boff, coff = (int(v) for v in GOLD[key + "_meta"])
    a, b, c = GOLD[key + "_a"], GOLD[key + "_b"], GOLD[key + "_c0"].copy()
    orc.port_gemm_rc(t, t, m, n, k, alpha, a[aoff:], rsa, csa, b[boff:], rsb, csb, beta, c[coff:], rsc, csc)
    assert bits_equal(c, GOLD[key + "_c1"])


@pytest.mark.parametrize("case", range(int(GOLD["gemm_p_count"][0])))
def test_gemm_packed_port_matches_reference_vectors(case):
    key = f"gemm_p_{case}"
    meta = [int(v) for v in GOLD[key + "_meta"]]
    t, m0, n0, k0, m1, n1, k1 = meta[:7]
    sa, sb, sc = meta[7:11], meta[11:15], meta[15:19]
    alpha, beta = meta[19], meta[20]
    a, b, c = GOLD[key + "_a"], GOLD[key + "_b"], GOLD[key + "_c0"].copy()
    lib = orc.port()
    if t == H.I8:
        lib.orc_gemm_packed_i8_i32(m0, n0, k0, m1, n1, k1, alpha, P(a), *sa, P(b), *sb, beta, P(c), *sc)
    else:
        lib.orc_gemm_packed_fp_f32(m0, n0, k0, m1, n1, k1, float(alpha), t, P(a), *sa, t, P(b), *sb, float(beta),
                                   P(c), *sc)
    assert bits_equal(c, GOLD[key + "_c1"])


@pytest.mark.parametrize("fmt", ["f8e4m3", "f8e5m2"])
@pytest.mark.parametrize("sat", ["", "sat_"])
@pytest.mark.parametrize("si,scale", [(0, 1.0), (1, 1.5)])
def test_cvt_port_matches_reference_vectors(fmt, sat, si, scale):
    lib = orc.port()
    f = H.F8E4M3 if fmt == "f8e4m3" else H.F8E5M2
    src32, src16 = GOLD["cvt_src32"], GOLD["cvt_src16"]
    d = np.zeros(src32.size, dtype=np.uint8)
    lib.orc_cvt_f32_f8(P(d), P(src32), scale, src32.size, f, int(sat != ""))
    assert np.array_equal(d, GOLD[f"cvt_{sat}f32_{fmt}_{si}"])
    lib.orc_cvt_bf16_f8(P(d), P(src16), scale, src16.size, f, int(sat != ""))
    assert np.array_equal(d, GOLD[f"cvt_{sat}bf16_{fmt}_{si}"])


def test_cvt_widening_port_matches_reference_vectors():
    lib = orc.port()
    codes = np.arange(256, dtype=np.uint8)
    for fmt, f in (("f8e4m3", H.F8E4M3), ("f8e5m2", H.F8E5M2)):
        w = np.zeros(256, dtype=np.uint16)
        lib.orc_cvt_f8_bf16(P(w), P(codes), 256, f)
        assert np.array_equal(w, GOLD[f"cvt_{fmt}_bf16"])
    for n in (512, 511, 1):
        d = np.zeros(n, dtype=np.uint8)
        lib.orc_cvt_f4e2m1_f8e4m3(P(d), P(codes), n)
        assert np.array_equal(d, GOLD[f"cvt_f4_{n}"])


def test_known_answers_fp8():
    """The handful of conversions worth knowing by heart (observed from the compiled reference)."""
    lib = orc.port()
    e4, e5 = lib.orc_f32_to_f8e4m3, lib.orc_f32_to_f8e5m2
    assert e4(448.0, 0) == 0x7E and e4(464.0, 0) == 0x7E
    assert e4(465.0, 0) == 0x7F and e4(465.0, 1) == 0x7E
    assert e4(-1e9, 0) == 0x7F and e4(-1e9, 1) == 0xFE
    assert e4(0.0, 0) == 0x00 and e4(-0.0, 0) == 0x80
    assert e5(57344.0, 0) == 0x7B and e5(61440.0, 0) == 0x7C
    assert e5(float("-inf"), 0) == 0xFC and e5(float("-inf"), 1) == 0xFB
    assert e5(float("nan"), 0) == 0x7F and e4(float("nan"), 1) == 0x7F
    # round trip: identity except NaN canonicalisation
    for c in range(256):
        back4 = e4(lib.orc_f8e4m3_to_f32(c), 0)
        assert back4 == (0x7F if c == 0xFF else c)
        back5 = e5(lib.orc_f8e5m2_to_f32(c), 0)
        assert back5 == (0x7F if (c & 0x7F) > 0x7C else c)


@pytest.mark.parametrize("case", range(int(GOLD["pack_count"][0])))
def test_pack_port_matches_reference_vectors(case):
    lib = orc.port()
    key = f"pack_{case}"
    e, m, n, rs, cs, m0, n0, rs0, cs0, rs1, cs1 = (int(v) for v in GOLD[key + "_meta"])
    src, want = GOLD[key + "_src"], GOLD[key + "_dst"]
    dst = np.full(want.shape, 0xAB, dtype=want.dtype)
    lib.orc_pack(e // 8, m, n, P(src), rs, cs, m0, n0, P(dst), rs0, cs0, rs1, cs1, 0xFF)
    assert np.array_equal(dst, want)
    if e == 8:
        back = np.full(GOLD[key + "_back"].shape, 0xCD, dtype=want.dtype)
        lib.orc_unpack(1, m0, n0, P(want), rs0, cs0, rs1, cs1, m, n, P(back), rs, cs)
        assert np.array_equal(back, GOLD[key + "_back"])
    a, at_want = GOLD[key + "_ta"], GOLD[key + "_tat"]
    at = np.full(at_want.shape, 0xEE, dtype=at_want.dtype)
    lib.orc_transpose(e // 8, m, n, P(a), n + 2, P(at), m + 3)
    assert np.array_equal(at, at_want)


ACTS = {"logistic": (orc.ACT_LOGISTIC, 1.0), "silu": (orc.ACT_SWISH, 1.0), "swish2": (orc.ACT_SWISH, 2.0),
        "swiglu": (orc.ACT_SWIGLU, 0.5), "gelu": (orc.ACT_GELU, 0.0)}


@pytest.mark.parametrize("name", sorted(ACTS))
def test_activation_port_matches_reference_vectors(name):
    """orc_activation against skl_sigmoid_f32_ref / skl_gelu_f32_ref outputs (both evaluate in double and
    round once, so the results agree bit for bit)."""
    act, p = ACTS[name]
    fn = orc.port().orc_activation
    x, up, want = GOLD[f"act_{name}_x"], GOLD[f"act_{name}_up"], GOLD[f"act_{name}_out"]
    got = np.array([fn(act, p, float(v), float(u)) for v, u in zip(x, up)], dtype=np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)) or np.array_equal(got, want, equal_nan=True)


def test_f32_f64_gemm_port_matches_reference_vectors():
    port = orc.port()
    for name in ("f32", "f64"):
        a, b, c, want = (GOLD[f"gemm_{name}_{x}"] for x in ("a", "b", "c", "out"))
        m, k = a.shape
        n = b.shape[1]
        got = c.copy()
        if name == "f32":
            port.orc_gemm_fp_f32(m, n, k, 1.25, H.F32, P(a), k, 1, H.F32, P(b), n, 1, -0.5, P(got), n, 1)
        else:
            port.orc_gemm_f64(m, n, k, 1, 1, 1, 1.25, P(a), k, 1, 0, 0, P(b), n, 1, 0, 0, -0.5, P(got), n, 1, 0, 0)
        assert np.array_equal(got, want)
