"""Skinny int8 kernel and the extended epilogue on the GPU, through the C ABI."""
import numpy as np
import pytest

import helpers as H
import skl_b200 as S
from gpu_common import DeviceBuf, check_gemm_rc
from oracle import pyoracle as orc

pytestmark = pytest.mark.gpu
P = orc._p


@pytest.mark.parametrize("m", [1, 2, 3, 4, 7, 8, 13, 16])
def test_gemv_int32_bit_exact(skl, m):
    """Weights "[N][K]" (layout 'k'), activations row-major; int32 out with alpha/beta."""
    for (n, k, alpha, beta) in [(14336, 4096, 1, 0), (1000, 512, 2, 3), (5, 16, 1, 0), (257, 4096, 1, 1),
                                (4099, 1024, 1, 0),
                                # row counts whose 128-row tiles make a ragged last round of the grid: the
                                # tensor-core route cuts shorter tiles (68 and 91 rows here)
                                (5000, 512, 2, 3), (20000, 256, 1, 1), (40000, 128, 2, 0)]:
        # the dp4a streaming kernel, for every m it accepts
        used = check_gemm_rc(skl, H.I8, m, n, k, "rkr", alpha, beta, where="device", seed=m, path=S.PATH_GEMV)
        assert used == S.PATH_GEMV
        # automatic dispatch: dp4a up to m = 2, the transposed narrow tensor-core tile above
        used = check_gemm_rc(skl, H.I8, m, n, k, "rkr", alpha, beta, where="device", seed=m)
        assert used == (S.PATH_GEMV if m <= 2 else S.PATH_TCGEN05)


def ex_case(skl, m, n, k, ta, tb, tc, layout, alpha, beta, use_rs, use_cs, where, seed, force=0, amp=1.0):
    from gpu_common import layout_strides

    g = H.rng(seed)
    (rsa, csa), (rsb, csb), (rsc, csc) = layout_strides(layout, m, n, k, 16)
    A = H.Strided(ta, m, k, rsa, csa, g, all_codes=True)
    B = H.Strided(tb, k, n, rsb, csb, g, all_codes=True)
    cvals = None
    if tc == H.F8E4M3:
        cvals = H.random_operand(H.F8E4M3, (m, n), g)
    C = H.Strided(tc, m, n, rsc, csc, g, fill=cvals)
    rs = (g.uniform(0.5, 1.5, m) * amp).astype(np.float32) if use_rs else None
    cs = (g.uniform(0.5, 1.5, n) * 1e-2).astype(np.float32) if use_cs else None
    want = C.copy()
    orc.port_gemm_ex(m, n, k, ta, A.view, rsa, csa, tb, B.view, rsb, csb, alpha, rs, cs, beta, tc, want.view, rsc, csc)
    before = C.copy()
    skl.skl_b200_force_path(force)
    try:
        if where == "host":
            skl.skl_gemm_ex_sm100a(m, n, k, ta, S.ptr(A.view), rsa, csa, tb, S.ptr(B.view), rsb, csb, alpha, S.ptr(rs),
                                   S.ptr(cs), beta, tc, S.ptr(C.view), rsc, csc)
            S.check()
            after = C.buf
        else:
            import torch

            da, db, dc = DeviceBuf(A.buf), DeviceBuf(B.buf), DeviceBuf(C.buf)
            drs = torch.from_numpy(rs).cuda() if use_rs else None
            dcs = torch.from_numpy(cs).cuda() if use_cs else None
            skl.skl_gemm_ex_sm100a(m, n, k, ta, da.ptr(A.off), rsa, csa, tb, db.ptr(B.off), rsb, csb, alpha, S.ptr(drs),
                                   S.ptr(dcs), beta, tc, dc.ptr(C.off), rsc, csc)
            S.check()
            torch.cuda.synchronize()
            after = dc.back()
    finally:
        skl.skl_b200_force_path(0)
    H.assert_untouched_outside(before, after, "C")
    return A, B, before, want, after[C.idx()], rs, cs


@pytest.mark.parametrize("m", [1, 4, 16])
def test_config4_decode_gemv_dequantised(skl, m):
    """The decode-shape workload at full size: int8 weights 14336 x 4096 with per-row scales, int8 activations with
    per-row scale, fp32 out = ((float)acc * s_x[i]) * s_w[j].  The accumulator is exact, so the result
    must equal the oracle's bit for bit."""
    for where in ("device", "host"):
        for force in (0, S.PATH_GEMV):
            _, _, _, want, got, _, _ = ex_case(skl, m, 14336, 4096, H.I8, H.I8, H.F32, "rkr", 1.0, 0.0, True, True, where,
                                               40 + m, force)
            expect = S.PATH_GEMV if (m <= 2 or force) else S.PATH_TCGEN05
            assert skl.skl_b200_last_path() == expect
            assert np.array_equal(got.view(np.uint32), want.get().view(np.uint32))


@pytest.mark.parametrize("pair", [(H.I8, H.I8), (H.BF16, H.BF16), (H.F16, H.F16), (H.F8E4M3, H.F8E4M3),
                                  (H.F8E5M2, H.F8E4M3), (H.F8E4M3, H.F8E5M2), (H.BF16, H.F8E4M3), (H.BF16, H.F8E5M2)])
@pytest.mark.parametrize("tc", [H.F32, H.BF16, H.F16, H.F8E4M3])
def test_extended_epilogue_all_pairs_and_outputs(skl, pair, tc):
    ta, tb = pair
    for (m, n, k, layout, beta, force) in [(130, 260, 192, "rkr", 0.0, 0), (130, 260, 192, "rrr", 0.5, 0),
                                           (33, 17, 40, "rrp", 0.5, S.PATH_GENERIC), (64, 96, 128, "ckc", 0.0, 0)]:
        A, B, before, want, got, rs, cs = ex_case(skl, m, n, k, ta, tb, tc, layout, 1.5, beta, True, True, "device",
                                                  m + k, force, amp=(1.0 if ta == H.I8 else 100.0))
        ref = H.to_f32(tc, want.get()).astype(np.float64)
        out = H.to_f32(tc, got).astype(np.float64)
        if ta == H.I8:
            assert np.array_equal(got, want.get())  # integer accumulator: the whole chain is exact
            continue
        # float pairs: error of the accumulator (reference's bound) scaled through the epilogue, plus
        # one unit in the last place of the output type
        scale = np.abs(1.5 * rs[:, None].astype(np.float64) * cs[None, :].astype(np.float64))
        bound = H.skl_forward_bound(ta, A.get(), tb, B.get(), 1.0, 0.0, None, k) * scale * 2
        ulp = {H.F32: 2.0 ** -23, H.BF16: 2.0 ** -7, H.F16: 2.0 ** -10, H.F8E4M3: 2.0 ** -3}[tc]
        tol = bound + ulp * np.maximum(np.abs(ref), 2.0 ** -9 if tc == H.F8E4M3 else 0.0) + 1e-30
        err = np.where(out == ref, 0.0, np.abs(out - ref))  # equal infinities count as agreement
        tol = np.where(np.isfinite(tol), tol, np.inf)
        assert np.all(err <= tol), float(np.nanmax(err - tol))


@pytest.mark.parametrize("m", [1, 2, 4, 16])
def test_overlapped_launches_with_static_weights_keep_stream_order(skl, m):
    """With skl_b200_set_static_weights(1) each skinny launch (the dp4a kernel for m <= 2, the transposed tensor-core
    tile above) may start streaming weights before its predecessor has finished, but must still see everything the
    predecessor wrote.  A chain of launches accumulates into the same C
    (beta = 1), each from new activations written just before it on the same stream; the sum must be exact."""
    import torch

    n, k, steps = 3000, 2048, 24
    g = H.rng(500 + m)
    w = g.integers(-128, 128, size=(n, k), dtype=np.int8)
    xs = g.integers(-128, 128, size=(steps, m, k), dtype=np.int8)
    want = np.zeros((m, n), np.int64)
    for s_ in range(steps):
        want += xs[s_].astype(np.int64) @ w.astype(np.int64).T
    dw = torch.from_numpy(w).cuda()
    dxs = torch.from_numpy(xs).cuda()
    dx = torch.zeros((m, k), dtype=torch.int8, device="cuda")
    dc = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    stream = torch.cuda.Stream()
    skl.skl_b200_set_stream(stream.cuda_stream)
    skl.skl_b200_set_async(1)
    skl.skl_b200_set_static_weights(1)
    try:
        with torch.cuda.stream(stream):
            for s_ in range(steps):
                dx.copy_(dxs[s_])  # the activations change between launches, on the same stream
                skl.skl_gemm_i8rc_i8rc_i32rc_sm100a(m, n, k, 1, dx.data_ptr(), k, 1, dw.data_ptr(), 1, k, 1, dc.data_ptr(), n, 1)
                assert skl.skl_b200_last_path() == (S.PATH_GEMV if m <= 2 else S.PATH_TCGEN05)
        skl.skl_b200_synchronize()
        S.check()
    finally:
        skl.skl_b200_set_static_weights(0)
        skl.skl_b200_set_async(0)
        skl.skl_b200_set_stream(None)
        torch.cuda.synchronize()
    assert np.array_equal(dc.cpu().numpy().astype(np.int64), want)


def test_static_fp8_weights_are_widened_once(skl):
    """bf16 x fp8 with skl_b200_set_static_weights(1): the first call widens W (2 launches), repeats reuse the copy
    (1 launch), another W or switching the declaration off widens again; every result equals the plain call's."""
    import torch

    m, n, k = 256, 512, 256
    g = H.rng(321)
    x = torch.from_numpy(H.random_operand(H.BF16, (m, k), g).view(np.int16)).cuda()
    w1 = torch.from_numpy(H.random_operand(H.F8E4M3, (k, n), g)).cuda()
    w2 = torch.from_numpy(H.random_operand(H.F8E4M3, (k, n), g)).cuda()
    cs = torch.from_numpy(g.uniform(0.5, 1.5, n).astype(np.float32)).cuda()

    def run(w):
        c = torch.zeros((m, n), dtype=torch.int16, device="cuda")
        skl.skl_gemm_ex_sm100a(m, n, k, S.BF16, x.data_ptr(), k, 1, S.F8E4M3, w.data_ptr(), n, 1, 1.0, None, cs.data_ptr(),
                               0.0, S.BF16, c.data_ptr(), n, 1)
        S.check()
        return c, skl.skl_b200_last_launch_count()

    ref1, l0 = run(w1)
    ref2, _ = run(w2)
    assert l0 == 2
    skl.skl_b200_set_static_weights(1)
    try:
        a, la = run(w1)
        b, lb = run(w1)
        c2, lc = run(w2)
        d, ld = run(w2)
        e, le = run(w1)
    finally:
        skl.skl_b200_set_static_weights(0)
    assert (la, lb, lc, ld, le) == (2, 1, 2, 1, 2)
    for got, want in ((a, ref1), (b, ref1), (c2, ref2), (d, ref2), (e, ref1)):
        assert torch.equal(got, want)
    f, lf = run(w1)
    assert lf == 2 and torch.equal(f, ref1)


@pytest.mark.parametrize("tb", [H.F8E4M3, H.F8E5M2])
@pytest.mark.parametrize("where", ["device", "host"])
def test_bf16_x_fp8_with_reoriented_widening(skl, tb, where, monkeypatch):
    """m >= 512 and an n-contiguous fp8 B: the widened copy is written k-contiguous by the transposing kernel.
    Shapes ragged against its 128 x 64 tiles; the result must equal what the layout-keeping route gives, bit for
    bit (both feed exactly the same bf16 values to the same kernel family), and stay within the oracle's bound."""
    for (m, n, k) in [(520, 300, 200), (640, 257, 136), (512, 64, 128)]:
        outs = []
        for keep in ("", "1"):
            if keep:
                monkeypatch.setenv("SKL_B200_WIDEN_KEEP_LAYOUT", keep)
            else:
                monkeypatch.delenv("SKL_B200_WIDEN_KEEP_LAYOUT", raising=False)
            A, B, before, want, got, rs, cs = ex_case(skl, m, n, k, H.BF16, tb, H.F32, "rrr", 1.5, 0.0, False, True,
                                                      where, m + n, 0, amp=1.0)
            assert skl.skl_b200_last_path() == S.PATH_TCGEN05
            outs.append(got.copy())
        monkeypatch.delenv("SKL_B200_WIDEN_KEEP_LAYOUT", raising=False)
        ref = H.to_f32(H.F32, want.get()).astype(np.float64)
        scale = np.abs(1.5 * cs[None, :].astype(np.float64))
        bound = H.skl_forward_bound(H.BF16, A.get(), tb, B.get(), 1.0, 0.0, None, k) * scale * 2
        err = np.abs(outs[0].astype(np.float64) - ref)
        assert np.all(err <= bound + 2.0 ** -23 * np.abs(ref) + 1e-30)
        # k-order inside the MMA is the same for both orientations of B, so the two routes agree exactly
        assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
