"""The MX-FP4 (block-scaled E2M1) GEMM entry point on the GPU, through the C ABI.

SKL has no such routine (it stops at skl_cvt_f4e2m1_f8e4m3, ref/cvt/cvt_ofp4.c:18-72), so the checker is the oracle's
restatement of the published format on the reference's E2M1 table and float-GEMM loop.  The result is held to the
forward bound of the reference's float GEMM tests (test/gemm/gemm_bf16rc_bf16rc_f32rc.c), evaluated on the scaled
elements; with one k block of exactly representable sums it must be exact."""
import numpy as np
import pytest

import helpers as H
import skl_b200 as S
from gpu_common import DeviceBuf
from oracle import pyoracle as orc

pytestmark = pytest.mark.gpu
P = orc._p


def elements(codes, scales, k):
    """fp32 values of packed E2M1 rows `codes` [rows][k/2] with E8M0 scales [rows][k/32]."""
    table = np.array([orc.port().orc_mxf4_element(c, 127) for c in range(16)], np.float32)
    nib = np.empty((codes.shape[0], k), np.uint8)
    nib[:, 0::2] = codes[:, : k // 2] & 0xF
    nib[:, 1::2] = codes[:, : k // 2] >> 4
    f = np.exp2(scales[:, : k // 32].astype(np.float64) - 127.0).repeat(32, axis=1)
    return (table[nib].astype(np.float64) * f).astype(np.float32)


def case(skl, m, n, k, alpha, beta, where, seed, pad=0, lo=117, hi=137):
    g = H.rng(seed)
    rsa, csb = k // 2 + pad, k // 2 + 2 * pad
    rssa, cssb = k // 32 + pad, k // 32 + pad
    a = g.integers(0, 256, (m, rsa), dtype=np.uint8)
    b = g.integers(0, 256, (n, csb), dtype=np.uint8)
    sa = g.integers(lo, hi, (m, rssa), dtype=np.uint8)
    sb = g.integers(lo, hi, (n, cssb), dtype=np.uint8)
    rsc = n + pad
    c = g.standard_normal((m, rsc)).astype(np.float32)
    want = c.copy()
    orc.port().orc_gemm_mxf4(m, n, k, alpha, P(a), rsa, P(sa), rssa, P(b), csb, P(sb), cssb, beta, P(want), rsc)
    fn = skl.skl_gemm_mxf4e2m1_mxf4e2m1_f32_sm100a
    if where == "host":
        got = c.copy()
        fn(m, n, k, alpha, S.ptr(a), rsa, S.ptr(sa), rssa, S.ptr(b), csb, S.ptr(sb), cssb, beta, S.ptr(got), rsc)
        S.check()
    else:
        import torch

        da, dsa, db, dsb, dc = (DeviceBuf(x.reshape(-1).view(np.uint8)) for x in (a, sa, b, sb, c))
        fn(m, n, k, alpha, da.ptr(0), rsa, dsa.ptr(0), rssa, db.ptr(0), csb, dsb.ptr(0), cssb, beta, dc.ptr(0), rsc)
        S.check()
        torch.cuda.synchronize()
        got = dc.back().view(np.float32).reshape(m, rsc)
    assert np.array_equal(got[:, n:].view(np.uint32), c[:, n:].view(np.uint32)), "padding columns of C were written"
    A, B = elements(a, sa, k), elements(b, sb, k)
    bound = H.skl_forward_bound(H.F32, A, H.F32, B.T.copy(), alpha, beta, c[:, :n], k)
    err = np.abs(got[:, :n].astype(np.float64) - want[:, :n].astype(np.float64))
    assert np.all(err <= bound), f"worst excess {np.max(err - bound)}"
    return got[:, :n], want[:, :n]


@pytest.mark.parametrize("where,native", [("device", "1"), ("device", "0"), ("host", "1")])
def test_mxf4_gemm_within_the_forward_bound(skl, where, native, monkeypatch):
    """Device operands with TMA-compatible rows run on the block-scaled tensor-core instruction (native = 1); host C
    or SKL_B200_MXF4_NATIVE=0 take the exact widening to bf16 followed by the bf16 kernel."""
    monkeypatch.setenv("SKL_B200_MXF4_NATIVE", native)
    for i, (m, n, k, alpha, beta, pad) in enumerate([(256, 512, 1024, 1.0, 0.0, 0), (100, 300, 64, 0.5, 2.0, 3),
                                                      (1, 7, 32, 1.0, 1.0, 1), (130, 129, 4096, 2.0, 0.0, 0),
                                                      # k that ends inside a stage of 256 / inside an instruction of 64,
                                                      # ragged row and column counts, a single k block
                                                      (200, 260, 96, 1.0, 0.5, 0), (64, 40, 32, 1.0, 0.0, 0),
                                                      (300, 520, 352, -1.5, 1.0, 0), (129, 257, 288, 1.0, 0.0, 0)]):
        case(skl, m, n, k, alpha, beta, where, 10 * i + (where == "host"), pad)
        # pad = 0 keeps the packed rows 16-byte aligned: one launch that re-lays the scales + the block-scaled kernel;
        # otherwise two widening launches and the bf16 GEMM
        native_here = where == "device" and native == "1" and pad == 0
        assert skl.skl_b200_last_launch_count() == (2 if native_here else 3), (m, n, k, where, native)
    assert skl.skl_b200_last_path() in (S.PATH_TCGEN05, S.PATH_GENERIC)


def test_mxf4_gemm_runs_on_the_tensor_cores_and_is_exact_on_exact_sums(skl):
    """One block of k with equal scales: every product and partial sum is a small multiple of 2^-2 times a power of
    two, so any summation order gives the oracle's result bit for bit."""
    got, want = case(skl, 256, 256, 32, 1.0, 0.0, "device", 77, lo=127, hi=128)
    assert skl.skl_b200_last_path() == S.PATH_TCGEN05
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_mxf4_native_scale_placement(skl):
    """All elements 1.0; the scale of one (row, k block) of A and one (column, k block) of B set to 2^3 resp. 2^5: every
    output is then an exact small integer that names the row, column and block the hardware applied each scale to."""
    import torch

    m, n, k = 256, 384, 512
    fn = skl.skl_gemm_mxf4e2m1_mxf4e2m1_f32_sm100a
    for (ri, kbi, cj, kbj) in [(0, 0, 0, 0), (37, 5, 200, 5), (129, 15, 383, 2), (255, 9, 31, 9), (64, 3, 96, 12)]:
        a = np.full((m, k // 2), 0x22, np.uint8)
        b = np.full((n, k // 2), 0x22, np.uint8)
        sa = np.full((m, k // 32), 127, np.uint8)
        sb = np.full((n, k // 32), 127, np.uint8)
        sa[ri, kbi] = 130
        sb[cj, kbj] = 132
        want = np.full((m, n), float(k), np.float32)
        want[ri, :] += 32 * 7
        want[:, cj] += 32 * 31
        if kbi == kbj:
            want[ri, cj] += 32 * (8 * 32 - 8 - 32 + 1)
        da, dsa, db, dsb = (DeviceBuf(x.reshape(-1)) for x in (a, sa, b, sb))
        dc = torch.zeros((m, n), dtype=torch.float32, device="cuda")
        fn(m, n, k, 1.0, da.ptr(0), k // 2, dsa.ptr(0), k // 32, db.ptr(0), k // 2, dsb.ptr(0), k // 32, 0.0,
           dc.data_ptr(), n)
        S.check()
        assert skl.skl_b200_last_launch_count() == 2  # the block-scaled kernel, not the widening route
        got = dc.cpu().numpy()
        assert np.array_equal(got, want), (ri, kbi, cj, kbj, np.argwhere(got != want)[:4])


def test_mxf4_gemm_argument_checks_and_nan_scale(skl):
    a = np.zeros((4, 16), np.uint8)
    s = np.full((4, 1), 127, np.uint8)
    c = np.zeros((4, 4), np.float32)
    fn = skl.skl_gemm_mxf4e2m1_mxf4e2m1_f32_sm100a
    fn(4, 4, 48, 1.0, S.ptr(a), 24, S.ptr(s), 2, S.ptr(a), 24, S.ptr(s), 2, 0.0, S.ptr(c), 4)  # k not a multiple of 32
    assert skl.skl_b200_last_status() == 1  # SKL_B200_ERR_INVALID_ARGUMENT
    a[:] = 0x22  # all elements 1.0
    s[2, 0] = 255  # row 2 of A: NaN scale
    fn(4, 4, 32, 1.0, S.ptr(a), 16, S.ptr(s), 1, S.ptr(a), 16, S.ptr(np.full((4, 1), 127, np.uint8)), 1, 0.0, S.ptr(c), 4)
    S.check()
    assert np.all(np.isnan(c[2])) and np.all(c[[0, 1, 3]] == 32.0)
