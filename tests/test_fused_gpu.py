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


def run_case(skl, m, n, k, ta, tb, tc, layout, beta, where, force, seed):
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
    orc.port_gemm_fused(m, n, k, ta, A.view, rsa, csa, tb, B.view, rsb, csb, 1.25, rs, cs, bias, gmax_want, beta, tc,
                        want.view, rsc, csc)
    before = Cm.copy()
    gmax = np.array([-np.inf], np.float32)
    skl.skl_b200_force_path(force)
    try:
        if where == "host":
            f = S.Fused(1.25, beta, S.ptr(rs), S.ptr(cs), S.ptr(bias), S.ptr(gmax))
            skl.skl_gemm_fused_sm100a(m, n, k, ta, S.ptr(A.view), rsa, csa, tb, S.ptr(B.view), rsb, csb, C.byref(f), tc,
                                      S.ptr(Cm.view), rsc, csc)
            S.check()
            after = Cm.buf
        else:
            import torch

            da, db, dc = DeviceBuf(A.buf), DeviceBuf(B.buf), DeviceBuf(Cm.buf)
            drs, dcs, dbias = (torch.from_numpy(x).cuda() for x in (rs, cs, bias))
            dg = torch.from_numpy(gmax).cuda()
            f = S.Fused(1.25, beta, drs.data_ptr(), dcs.data_ptr(), dbias.data_ptr(), dg.data_ptr())
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
