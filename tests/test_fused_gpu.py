"""skl_gemm_fused_sm100a: bias row vector and global maximum fused into the accumulator read-out, the two
epilogue kernels the reference documents for its fused-kernel hook (src/gemm/fused-kernel-API.md:170-217).
int8 pairs have an exact accumulator, so outputs and the maximum must equal the oracle's bit for bit on
every kernel family; float pairs are held to the reference suite's forward bound."""
import ctypes as C

import numpy as np
import pytest

import helpers as H
import skl_b200 as S
from gpu_common import DeviceBuf, layout_strides
from oracle import pyoracle as orc

pytestmark = pytest.mark.gpu


def run_case(skl, m, n, k, ta, tb, tc, layout, beta, where, force, seed, alpha=1.25, act=0, act_param=0.0):
    g = H.rng(seed)
    (rsa, csa), (rsb, csb), (rsc, csc) = layout_strides(layout, m, n, k, 16)
    A = H.Strided(ta, m, k, rsa, csa, g, all_codes=False)
    B = H.Strided(tb, k, n, rsb, csb, g, all_codes=False)
    Cm = H.Strided(tc, m, n, rsc, csc, g)
    rs = g.uniform(0.5, 1.5, m).astype(np.float32)
    cs = (g.uniform(0.5, 1.5, n) * 1e-2).astype(np.float32)
    bias = g.uniform(-3, 3, n).astype(np.float32)
    want = Cm.copy()
    gmax_want = np.array([-np.inf], np.float32)
    orc.port_gemm_fused(m, n, k, ta, A.view, rsa, csa, tb, B.view, rsb, csb, alpha, rs, cs, bias, gmax_want, beta, tc,
                        want.view, rsc, csc, activation=act, act_param=act_param)
    before = Cm.copy()
    gmax = np.array([-np.inf], np.float32)
    skl.skl_b200_force_path(force)
    try:
        if where == "host":
            f = S.Fused(alpha, beta, S.ptr(rs), S.ptr(cs), S.ptr(bias), S.ptr(gmax), act, act_param)
            skl.skl_gemm_fused_sm100a(m, n, k, ta, S.ptr(A.view), rsa, csa, tb, S.ptr(B.view), rsb, csb, C.byref(f), tc,
                                      S.ptr(Cm.view), rsc, csc)
            S.check()
            after = Cm.buf
        else:
            import torch

            da, db, dc = DeviceBuf(A.buf), DeviceBuf(B.buf), DeviceBuf(Cm.buf)
            drs, dcs, dbias = (torch.from_numpy(x).cuda() for x in (rs, cs, bias))
            dg = torch.from_numpy(gmax).cuda()
            f = S.Fused(alpha, beta, drs.data_ptr(), dcs.data_ptr(), dbias.data_ptr(), dg.data_ptr(), act, act_param)
            skl.skl_gemm_fused_sm100a(m, n, k, ta, da.ptr(A.off), rsa, csa, tb, db.ptr(B.off), rsb, csb, C.byref(f), tc,
                                      dc.ptr(Cm.off), rsc, csc)
            S.check()
            torch.cuda.synchronize()
            after = dc.back()
            gmax = dg.cpu().numpy()
    finally:
        skl.skl_b200_force_path(0)
    H.assert_untouched_outside(before, after, "C")
    return A, B, before, want.get(), after[Cm.idx()], float(gmax_want[0]), float(gmax[0]), rs, cs


@pytest.mark.parametrize("m,n,k,expect", [(1, 257, 4096, S.PATH_GEMV), (2, 1000, 512, S.PATH_GEMV),
                                          (3, 1000, 512, S.PATH_TCGEN05), (16, 4099, 1024, S.PATH_TCGEN05),
                                          (130, 260, 192, S.PATH_TCGEN05), (33, 17, 48, S.PATH_GENERIC)])
@pytest.mark.parametrize("beta", [0.0, 0.5])
@pytest.mark.parametrize("where", ["device", "host"])
def test_int8_bias_and_global_max_are_exact(skl, m, n, k, expect, beta, where):
    layout = "rkr"
    _, _, _, want, got, gw, gg, _, _ = run_case(skl, m, n, k, H.I8, H.I8, H.F32, layout, beta, where, 0, m + n)
    assert skl.skl_b200_last_path() == expect
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert gg == gw
    # the any-stride kernel must agree as well
    _, _, _, want, got, gw, gg, _, _ = run_case(skl, m, n, k, H.I8, H.I8, H.F32, layout, beta, where, S.PATH_GENERIC,
                                               m + n)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)) and gg == gw


@pytest.mark.parametrize("m,n,k,expect", [(1, 600, 512, S.PATH_GEMV), (200, 300, 256, S.PATH_TCGEN05),
                                          (33, 17, 48, S.PATH_GENERIC)])
def test_global_max_of_results_that_are_all_zero_or_negative(skl, m, n, k, expect):
    """Non-negative operands and a negative alpha: every result is negative or -0.0 (rows of A that are all zero).
    The maximum must come out as a zero, as the sequential definition gives -- a float atomic maximum that files
    -0.0 with the non-negative bit patterns would leave the initial -inf in place."""
    import torch

    g = H.rng(m + n)
    a = g.integers(0, 100, size=(m, k), dtype=np.int8)
    a[0, :] = 0  # a whole row of exact zeros -> -0.0 after the negative alpha
    b = g.integers(1, 100, size=(n, k), dtype=np.int8)  # [N][K]
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    dc = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    dg = torch.full((1,), -np.inf, dtype=torch.float32, device="cuda")
    f = S.Fused(-0.5, 0.0, None, None, None, dg.data_ptr(), 0, 0.0)
    skl.skl_gemm_fused_sm100a(m, n, k, S.I8, da.data_ptr(), k, 1, S.I8, db.data_ptr(), 1, k, C.byref(f), S.F32,
                              dc.data_ptr(), n, 1)
    S.check()
    assert skl.skl_b200_last_path() == expect
    out = dc.cpu().numpy()
    assert np.all(out <= 0.0) and np.all(out[0] == 0.0) and np.all(np.signbit(out[0]))
    assert float(dg.cpu()[0]) == 0.0
    if m > 1:
        assert np.all(out[1:] < 0.0)


@pytest.mark.parametrize("pair", [(H.BF16, H.BF16), (H.F8E4M3, H.F8E5M2), (H.BF16, H.F8E4M3)])
@pytest.mark.parametrize("tc", [H.F32, H.BF16])
def test_float_pairs_with_bias_and_global_max(skl, pair, tc):
    ta, tb = pair
    for (m, n, k, layout, beta) in [(257, 300, 256, "rrr", 0.0), (130, 264, 192, "rkr", 0.5)]:
        A, B, before, want, got, gw, gg, rs, cs = run_case(skl, m, n, k, ta, tb, tc, layout, beta, "device", 0, m + k)
        assert skl.skl_b200_last_path() == S.PATH_TCGEN05
        ref = H.to_f32(tc, want).astype(np.float64)
        out = H.to_f32(tc, got).astype(np.float64)
        scale = np.abs(1.25 * rs[:, None].astype(np.float64) * cs[None, :].astype(np.float64))
        bound = H.skl_forward_bound(ta, A.get(), tb, B.get(), 1.0, 0.0, None, k) * scale * 2
        ulp = {H.F32: 2.0 ** -23, H.BF16: 2.0 ** -7}[tc]
        tol = bound + ulp * np.abs(ref) + 1e-30
        assert np.all(np.abs(out - ref) <= tol)
        assert abs(gg - gw) <= float(np.max(bound)) + 2.0 ** -20 * abs(gw)


# ---------------------------------------------------------------------------------------------- activations
def ulp_error_f32(x, r):
    """Distance between x and r in units of ulp(r): the measure of the reference's own activation tests
    (test/skl-test-driver.h:568-581)."""
    x, r = x.astype(np.float32), r.astype(np.float32)
    same = (x == r) | (np.isnan(x) & np.isnan(r))
    bad = np.isinf(r) | np.isnan(x) | np.isnan(r)
    with np.errstate(invalid="ignore", over="ignore"):
        d = np.abs(x - r).astype(np.float64)
    _, e = np.frexp(r)
    e = np.where((e < -125) | (r == 0), -125 - 24, e - 24)
    err = np.ldexp(d, -e)
    return np.where(same, 0.0, np.where(bad, np.inf, err))


# bounds from the reference's tests of its own kernels: test/sigmoid/sigmoid_f32_zve32f.c:66-76 (logistic 3 ulp,
# silu / swish / swiglu 52 ulp) and, for GELU by input class (v < -2, [-2,-1), [-1,0), >= 0), the bounds of its most
# accurate variant in test/gelu/skl_gelu_f32_zve32f.c:44
ACT_CASES = [("logistic", S.ACT_LOGISTIC, 1.0), ("silu", S.ACT_SWISH, 1.0), ("swish2", S.ACT_SWISH, 2.0),
             ("gelu", S.ACT_GELU, 0.0), ("swiglu", S.ACT_SWIGLU, 0.5)]
GELU_BOUNDS = [(-np.inf, -2.0, 1.7e7), (-2.0, -1.0, 62.0), (-1.0, 0.0, 5.0), (0.0, np.inf, 4.0)]


@pytest.mark.parametrize("name,act,p", ACT_CASES)
@pytest.mark.parametrize("m,n,k,expect", [(1, 1000, 512, S.PATH_GEMV), (16, 2000, 512, S.PATH_TCGEN05),
                                          (257, 520, 256, S.PATH_TCGEN05), (33, 17, 48, S.PATH_GENERIC)])
def test_activation_epilogue_within_reference_ulp_bounds(skl, name, act, p, m, n, k, expect):
    """int8 operands: the value entering the activation is exact, so the whole difference to the oracle is the
    activation's own fp32 evaluation.  alpha spreads the pre-activation values over about [-25, 25]."""
    alpha = 8.0 / (5476.0 * np.sqrt(k) * 1e-2)
    where = "host" if (act == S.ACT_SWIGLU and m == 257) else "device"
    _, _, before, want, got, gw, gg, _, _ = run_case(skl, m, n, k, H.I8, H.I8, H.F32, "rkr", 0.0, where, 0, 7 * m + n,
                                                     alpha=alpha, act=act, act_param=p)
    assert skl.skl_b200_last_path() == expect
    err = ulp_error_f32(got, want)
    if act == S.ACT_GELU:
        # recover the pre-activation value's class from the oracle without the activation
        _, _, _, pre, _, _, _, _, _ = run_case(skl, m, n, k, H.I8, H.I8, H.F32, "rkr", 0.0, "device", 0, 7 * m + n,
                                               alpha=alpha)
        for lo, hi, bound in GELU_BOUNDS:
            sel = (pre >= lo) & (pre < hi)
            assert sel.sum() == 0 or err[sel].max() <= bound, (name, lo, hi, float(err[sel].max()))
    else:
        bound = 3.0 if act == S.ACT_LOGISTIC else 52.0
        assert err.max() <= bound, (name, float(err.max()))
    # the maximum is taken after the activation
    assert ulp_error_f32(np.array([gg]), np.array([gw]))[0] <= 52.0


@pytest.mark.parametrize("name,act,p", ACT_CASES)
def test_activation_epilogue_bf16_output_and_float_operands(skl, name, act, p):
    """bf16 x bf16 -> bf16 with an activation: within one bf16 ulp of the oracle plus the reference suite's
    forward bound carried through the activation (all five have slope <= 1.13 in magnitude... times |up + delta|
    for the gate)."""
    m, n, k = 260, 384, 128
    A, B, before, want, got, gw, gg, rs, cs = run_case(skl, m, n, k, H.BF16, H.BF16, H.BF16, "rrr", 0.0, "device", 0,
                                                       31, alpha=40.0, act=act, act_param=p)
    assert skl.skl_b200_last_path() == S.PATH_TCGEN05
    ref = H.to_f32(H.BF16, want).astype(np.float64)
    out = H.to_f32(H.BF16, got).astype(np.float64)
    scale = np.abs(40.0 * rs[:, None].astype(np.float64) * cs[None, :].astype(np.float64))
    bound = H.skl_forward_bound(H.BF16, A.get(), H.BF16, B.get(), 1.0, 0.0, None, k) * scale * 2
    slope = 1.13 * (np.abs(H.to_f32(H.BF16, before.get()).astype(np.float64)).max() + 0.5 if act == S.ACT_SWIGLU else 1.0)
    tol = bound * slope * (2.0 if act == S.ACT_SWISH and p == 2.0 else 1.0) + 2.0 ** -7 * np.abs(ref) + 1e-30
    assert np.all(np.abs(out - ref) <= tol), float(np.max(np.abs(out - ref) - tol))


def test_swiglu_with_beta_is_rejected(skl):
    a = np.ones((4, 4), np.int8)
    c = np.zeros((4, 4), np.float32)
    f = S.Fused(1.0, 0.5, None, None, None, None, S.ACT_SWIGLU, 0.0)
    skl.skl_gemm_fused_sm100a(4, 4, 4, S.I8, S.ptr(a), 4, 1, S.I8, S.ptr(a), 4, 1, C.byref(f), S.F32, S.ptr(c), 4, 1)
    assert skl.skl_b200_last_status() == 1
    f = S.Fused(1.0, 0.0, None, None, None, None, 9, 0.0)
    skl.skl_gemm_fused_sm100a(4, 4, 4, S.I8, S.ptr(a), 4, 1, S.I8, S.ptr(a), 4, 1, C.byref(f), S.F32, S.ptr(c), 4, 1)
    assert skl.skl_b200_last_status() == 1
    assert np.all(c == 0)


# ---------------------------------------------------------------------------------------------- requantised output
@pytest.mark.parametrize("m,n,k,expect", [(1, 1000, 512, S.PATH_GEMV), (16, 2000, 512, S.PATH_TCGEN05),
                                          (257, 520, 256, S.PATH_TCGEN05), (33, 17, 48, S.PATH_GENERIC)])
@pytest.mark.parametrize("beta", [0.0, 0.5])
def test_int8_output_is_exact_for_int8_operands(skl, m, n, k, expect, beta):
    """Requantisation to int8 (nearest even, saturating): exact accumulator, so the codes must equal the oracle's.
    alpha spreads the values over about [-250, 250] so that both rounding and saturation occur."""
    alpha = 80.0 / (5476.0 * np.sqrt(k) * 1e-2)
    for where in ("device", "host"):
        _, _, _, want, got, gw, gg, _, _ = run_case(skl, m, n, k, H.I8, H.I8, H.I8, "rkr", beta, where, 0, 3 * m + n,
                                                    alpha=alpha)
        assert skl.skl_b200_last_path() == expect
        assert np.array_equal(got, want)
        assert (want == 127).any() and (want == -128).any() and (np.abs(want.astype(np.int32)) < 100).any()
        assert gg == gw  # the maximum is taken before the narrowing


def test_int8_output_from_float_operands(skl):
    """bf16 x bf16 -> int8: the accumulator differs from the oracle's by at most the reference suite's forward
    bound, which can move a value across a rounding boundary, so codes may differ by one step there."""
    m, n, k = 260, 384, 128
    A, B, _, want, got, _, _, rs, cs = run_case(skl, m, n, k, H.BF16, H.BF16, H.I8, "rrr", 0.0, "device", 0, 5, alpha=900.0)
    assert skl.skl_b200_last_path() == S.PATH_TCGEN05
    diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 0.01
    assert np.unique(want).size > 100


@pytest.mark.parametrize("tc", [H.BF16, H.F16, H.F32])
def test_non_finite_scales_give_non_finite_results_in_the_same_places(skl, tc):
    """A column scale of +inf / NaN: infinities must come out bit-exact, NaN wherever the oracle has NaN (the
    payload of a NaN produced by an fp32 multiply is the host's or the device's own, so only the class is held)."""
    m, n, k = 130, 260, 128
    g = H.rng(11)
    a = g.integers(-128, 128, size=(m, k), dtype=np.int8)
    b = g.integers(-128, 128, size=(n, k), dtype=np.int8)  # [N][K]
    cs = g.uniform(0.5, 1.5, n).astype(np.float32)
    cs[5], cs[77], cs[200] = np.inf, np.nan, -np.inf
    dt = H.NP_STORE[tc]
    want = np.zeros((m, n), dt)
    orc.port_gemm_fused(m, n, k, H.I8, a, k, 1, H.I8, b, 1, k, 1.0, None, cs, None, None, 0.0, tc, want, n, 1)
    import torch

    da, db, dcs = (torch.from_numpy(x).cuda() for x in (a, b, cs))
    dc = torch.zeros((m, n * dt().itemsize), dtype=torch.uint8, device="cuda")
    f = S.Fused(1.0, 0.0, None, dcs.data_ptr(), None, None, 0, 0.0)
    skl.skl_gemm_fused_sm100a(m, n, k, S.I8, da.data_ptr(), k, 1, S.I8, db.data_ptr(), 1, k, C.byref(f), tc, dc.data_ptr(), n, 1)
    S.check()
    assert skl.skl_b200_last_path() == S.PATH_TCGEN05
    got = dc.cpu().numpy().view(dt).reshape(m, n)
    wf, gf = H.to_f32(tc, want), H.to_f32(tc, got)
    assert np.array_equal(np.isnan(wf), np.isnan(gf)) and np.isnan(wf).sum() >= m
    ok = ~np.isnan(wf)
    assert np.array_equal(got[ok], want[ok])
    assert np.isinf(wf).sum() >= m
