"""The fp16-accumulate GEMM (ref/gemm/gemm_f16rc_f16rc_f16rc.c:9-22 and its packed form) through the C ABI.

The library evaluates every statement of the reference in fp32 and rounds it to fp16 once; the oracle port states
the same and is pinned bit for bit to the reference compiled here (tests/test_oracle_vs_ref.py).  So the GPU must
equal the port exactly, and both must sit inside the bound SKL's own test of this routine uses
(test/gemm/gemm_f16rcprc_f16rcprc_f16rcprc.c:155-163: u = 2^-11 per step) around the compiled reference."""
import numpy as np
import pytest

import helpers as H
import skl_b200 as S
from gpu_common import DeviceBuf
from oracle import pyoracle as orc

pytestmark = pytest.mark.gpu
P = orc._p


def f16(x):
    return H.f32_to_f16_bits(np.asarray(x, np.float32))


@pytest.mark.parametrize("where", ["device", "host"])
def test_plain_operands_equal_the_oracle(skl, where):
    g = H.rng(16)
    for (m, n, k, alpha, beta) in [(1, 1, 1, 1.0, 0.0), (7, 9, 33, 1.25, -0.75), (70, 130, 300, 1.0, 0.0), (4, 5, 0, 2.0, 0.5),
                                   (129, 65, 64, -1.5, 1.0)]:
        for (rsa, csa), (rsb, csb), (rsc, csc) in [((max(k, 1), 1), (n, 1), (n, 1)), ((1, m), (1, max(k, 1)), (1, m)),
                                                   ((max(k, 1) + 3, 1), (n + 5, 1), (2 * n + 1, 2))]:
            A = H.Strided(H.F16, m, k, rsa, csa, g)
            B = H.Strided(H.F16, k, n, rsb, csb, g)
            Cm = H.Strided(H.F16, m, n, rsc, csc, g)
            want = Cm.copy()
            orc.port().orc_gemm_f16acc(m, n, k, 1, 1, 1, alpha, P(A.view), rsa, csa, 0, 0, P(B.view), rsb, csb, 0, 0, beta,
                                       P(want.view), rsc, csc, 0, 0)
            before = Cm.copy()
            if where == "host":
                skl.skl_gemm_f16rc_f16rc_f16rc_f32scalars_sm100a(m, n, k, alpha, S.ptr(A.view), rsa, csa, S.ptr(B.view), rsb,
                                                                 csb, beta, S.ptr(Cm.view), rsc, csc)
                S.check()
                after = Cm.buf
            else:
                da, db, dc = DeviceBuf(A.buf), DeviceBuf(B.buf), DeviceBuf(Cm.buf)
                skl.skl_gemm_f16rc_f16rc_f16rc_f32scalars_sm100a(m, n, k, alpha, da.ptr(A.off), rsa, csa, db.ptr(B.off), rsb,
                                                                 csb, beta, dc.ptr(Cm.off), rsc, csc)
                S.check()
                after = dc.back()
            assert skl.skl_b200_last_path() == S.PATH_GENERIC
            H.assert_untouched_outside(before, after, "C")
            got = after[Cm.idx()]
            ref = want.get()
            if beta == 0.0:  # C is not read: only the sign of a zero result may differ from the reference's 0*C + ...
                assert np.all((got == ref) | (((got | ref) & 0x7FFF) == 0))
            else:
                assert np.array_equal(got, ref)


def test_packed_operands_and_the_reference_bound(skl):
    """Blocked operands; the result equals the port and lies within SKL's own bound around the compiled reference."""
    g = H.rng(17)
    m0, n0, k0, m1, n1, k1 = 4, 3, 2, 5, 7, 40
    sa = (k0, 1, k1 * m0 * k0, m0 * k0)
    sb = (1, k0, n1 * k0 * n0, k0 * n0)
    sc = (1, m0, m0 * n0, m1 * m0 * n0)
    a = f16(g.uniform(-2, 2, m1 * k1 * m0 * k0))
    b = f16(g.uniform(-2, 2, k1 * n1 * k0 * n0))
    c = f16(g.uniform(-8, 8, m1 * n1 * m0 * n0))
    want, got = c.copy(), c.copy()
    orc.port().orc_gemm_f16acc(m0, n0, k0, m1, n1, k1, 1.5, P(a), *sa, P(b), *sb, 0.5, P(want), *sc)
    skl.skl_gemm_f16rcprc_f16rcprc_f16rcprc_f32scalars_sm100a(m0, n0, k0, m1, n1, k1, 1.5, S.ptr(a), *sa, S.ptr(b), *sb, 0.5,
                                                              S.ptr(got), *sc)
    S.check()
    assert np.array_equal(got, want)
    ref = orc.ref()
    if ref is not None and hasattr(ref, "orc_ref_gemm_f16acc"):
        r = c.copy()
        ref.orc_ref_gemm_f16acc(m0, n0, k0, m1, n1, k1, 1.5, P(a), *sa, P(b), *sb, 0.5, P(r), *sc)
        af, bf, cf = (H.to_f32(H.F16, x).astype(np.float64) for x in (a, b, c))
        A = np.abs(af).reshape(m1, k1, m0, k0).transpose(0, 2, 1, 3).reshape(m0 * m1, k0 * k1)
        # B blocks are [k1][n1] of k0 x n0 with k unit stride inside: (k1, n1, n0, k0)
        B = np.abs(bf).reshape(k1, n1, n0, k0).transpose(0, 3, 1, 2).reshape(k0 * k1, n0 * n1)
        C0 = np.abs(cf).reshape(n1, m1, n0, m0).transpose(1, 3, 0, 2).reshape(m0 * m1, n0 * n1)
        u = 2.0 ** -11
        bound = 2 * np.expm1((k0 * k1 + 2) * np.log1p(u)) * (1.5 * (A @ B) + 0.5 * C0)
        G = H.to_f32(H.F16, got).astype(np.float64).reshape(n1, m1, n0, m0).transpose(1, 3, 0, 2).reshape(m0 * m1, n0 * n1)
        R = H.to_f32(H.F16, r).astype(np.float64).reshape(n1, m1, n0, m0).transpose(1, 3, 0, 2).reshape(m0 * m1, n0 * n1)
        assert np.all(np.abs(G - R) <= bound)
        assert np.array_equal(got, r), "compiled reference on this toolchain rounds once per statement, as the library does"
