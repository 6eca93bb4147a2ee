"""GEMM parity on the GPU through the C ABI, shape classes after the reference's own suites
(test/gemm/rvv/skl_gemm_i8_i8_i32_zve32x_x390.c:58-81, test/gemm/xsfmm/skl_gemm_i8c_i8_i32_xsfmm32a8i.c:61-89):
minimal, odd, skinny, k = 0 with and without beta, tile edge -1/0/+1 (re-centred on this library's
128 x 256 tile and 64 / 128-element k slabs), wide and tall, alpha = 2 / beta = 3."""
import numpy as np
import pytest

import helpers as H
import skl_b200 as S
from gpu_common import check_gemm_rc

pytestmark = pytest.mark.gpu
ALL_T = [H.I8, H.BF16, H.F16, H.F8E4M3, H.F8E5M2]

SMALL = [(1, 1, 0, 1, 0), (1, 1, 1, 1, 0), (7, 7, 7, 1, 0), (17, 17, 17, 1, 0), (1, 33, 31, 1, 0),
         (33, 1, 31, 1, 0), (33, 33, 0, 1, 0), (16, 16, 0, 1, 1), (16, 16, 16, 1, 0), (15, 17, 31, 1, 0),
         (33, 129, 32, 1, 0), (129, 33, 32, 1, 0), (32, 32, 32, 1, 1), (65, 65, 0, 2, 3), (65, 65, 33, 2, 3),
         (0, 5, 3, 1, 0), (5, 0, 3, 1, 0)]


@pytest.mark.parametrize("t", ALL_T)
@pytest.mark.parametrize("m,n,k,alpha,beta", SMALL)
def test_generic_path_small_shapes_device(skl, t, m, n, k, alpha, beta):
    for layout in ("rrr", "crr", "rkp"):
        check_gemm_rc(skl, t, m, n, k, layout, alpha, beta, where="device", path=S.PATH_GENERIC)


@pytest.mark.parametrize("t", ALL_T)
def test_host_pointers_are_staged(skl, t):
    for (m, n, k, layout, beta) in [(33, 29, 40, "rrr", 0), (33, 29, 40, "rrp", 3), (20, 31, 16, "crc", 1),
                                    (129, 260, 192, "rkr", 0)]:
        check_gemm_rc(skl, t, m, n, k, layout, 2, beta, where="host", align=16 if m > 100 else 1)


# tile-edge classes for the tensor-core kernel: (m, n, k)
TC_SHAPES = [(127, 255, 63), (128, 256, 64), (129, 257, 65), (128, 256, 128), (256, 512, 129), (1, 256, 64),
             (128, 16, 64), (130, 40, 1), (385, 300, 200), (64, 1000, 320), (300, 128, 1024), (255, 256, 448),
             (257, 513, 96), (1024, 768, 512)]


@pytest.mark.parametrize("t", ALL_T)
@pytest.mark.parametrize("layout", ["rkr", "rrr", "ckr", "crr", "rkc", "rrp"])
@pytest.mark.parametrize("pair", ["0", "2"])
def test_tensor_core_path(skl, t, layout, pair, monkeypatch):
    """Every operand-major combination (A k-major / m-major, B k-major / n-major) and C layouts, on
    the one-CTA kernel (pair = 0) and on the two-CTA cta_group::2 kernel (pair = 2: whenever legal)."""
    monkeypatch.setenv("SKL_B200_TC_PAIR", pair)
    for i, (m, n, k) in enumerate(TC_SHAPES):
        alpha, beta = ((2, 3) if i % 3 == 0 else (1, 0))
        check_gemm_rc(skl, t, m, n, k, layout, alpha, beta, where="device", path=S.PATH_TCGEN05, align=16,
                      expect_path=S.PATH_TCGEN05, seed=i)


@pytest.mark.parametrize("t", ALL_T)
def test_tensor_core_matches_generic_bits_for_int8_and_bound_for_float(skl, t):
    check_gemm_rc(skl, t, 512, 512, 1024, "rrr", 1, 0, where="device", path=0, expect_path=S.PATH_TCGEN05)


@pytest.mark.parametrize("pair", ["0", "2"])
def test_config1_int8_512x512x1024_bit_exact(skl, pair, monkeypatch):
    """The first configured workload (int8 512 x 512 x 1024): A row-major, B K x N row-major, int32 out, alpha 1, beta 0; both pointer domains."""
    monkeypatch.setenv("SKL_B200_TC_PAIR", pair)
    for where in ("device", "host"):
        check_gemm_rc(skl, H.I8, 512, 512, 1024, "rrr", 1, 0, where=where, seed=1, expect_path=S.PATH_TCGEN05)


@pytest.mark.parametrize("t", ALL_T)
def test_many_tiles_per_cta_and_raster_groups(skl, t, monkeypatch):
    """More tiles than SMs, so every CTA walks several tiles through both TMEM accumulators, with a
    small rasterisation group so group edges and the short last group are exercised."""
    monkeypatch.setenv("SKL_B200_RASTER_GM", "3")
    for pair in ("0", "2"):
        monkeypatch.setenv("SKL_B200_TC_PAIR", pair)
        check_gemm_rc(skl, t, 128 * 13 + 5, 256 * 14 + 9, 192, "rkr", 1, 0, where="device", path=S.PATH_TCGEN05, align=16,
                      expect_path=S.PATH_TCGEN05, seed=9, all_codes=False)


def test_unaligned_problem_falls_back_to_generic(skl):
    used = check_gemm_rc(skl, H.BF16, 130, 70, 77, "rrr", 1, 0, where="device")
    assert used == S.PATH_GENERIC


def test_specialised_entry_points(skl):
    """Row-major and column-major-A wrappers take SKL's shortened argument lists."""
    import torch
    from oracle import pyoracle as orc

    g = H.rng(3)
    m, n, k = 96, 80, 64
    a = H.random_operand(H.I8, (m, k), g)
    b = H.random_operand(H.I8, (k, n), g)
    want = np.zeros((m, n), np.int32)
    orc.port_gemm_rc(H.I8, H.I8, m, n, k, 1, a, k, 1, b, n, 1, 0, want, n, 1)
    c = np.zeros((m, n), np.int32)
    skl.skl_gemm_i8_i8_i32_sm100a(m, n, k, 1, S.ptr(a), k, S.ptr(b), n, 0, S.ptr(c), n)
    S.check()
    assert np.array_equal(c, want)
    at = np.ascontiguousarray(a.T)  # column-major A: element (i, p) at at[p, i]
    c2 = np.zeros((m, n), np.int32)
    skl.skl_gemm_i8c_i8_i32_sm100a(m, n, k, 1, S.ptr(at), m, S.ptr(b), n, 0, S.ptr(c2), n)
    S.check()
    assert np.array_equal(c2, want)
    for name, t in (("bf16", H.BF16), ("f16", H.F16)):
        af = H.random_operand(t, (m, k), g)
        bf = H.random_operand(t, (k, n), g)
        wantf = np.zeros((m, n), np.float32)
        orc.port_gemm_rc(t, t, m, n, k, 1.0, af, k, 1, bf, n, 1, 0.0, wantf, n, 1)
        cf = np.zeros((m, n), np.float32)
        getattr(skl, f"skl_gemm_{name}_{name}_f32_sm100a")(m, n, k, 1.0, S.ptr(af), k, S.ptr(bf), n, 0.0, S.ptr(cf), n)
        S.check()
        bound = H.skl_forward_bound(t, af, t, bf, 1.0, 0.0, None, k)
        assert np.all(np.abs(cf.astype(np.float64) - wantf) <= bound)
        cf2 = np.zeros((m, n), np.float32)
        aft = np.ascontiguousarray(af.T)
        getattr(skl, f"skl_gemm_{name}c_{name}_f32_sm100a")(m, n, k, 1.0, S.ptr(aft), m, S.ptr(bf), n, 0.0, S.ptr(cf2), n)
        S.check()
        assert np.all(np.abs(cf2.astype(np.float64) - wantf) <= bound)


@pytest.mark.parametrize("t", ALL_T)
def test_packed_operands(skl, t):
    """Blocked 4-D operands (all block counts up to 3 x 3, k1 0..3), block-column-major C."""
    from oracle import pyoracle as orc

    P = orc._p
    name = {H.I8: "i8", H.BF16: "bf16", H.F16: "f16", H.F8E4M3: "f8e4m3", H.F8E5M2: "f8e5m2"}[t]
    tc = H.I32 if t == H.I8 else H.F32
    fn = getattr(skl, f"skl_gemm_{name}rcprc_{name}rcprc_{'i32' if t == H.I8 else 'f32'}rcprc_sm100a")
    g = H.rng(11)
    for (m0, n0, k0) in [(4, 3, 2), (8, 8, 4)]:
        for m1 in (1, 3):
            for n1 in (1, 2):
                for k1 in (0, 1, 3):
                    a = H.random_operand(t, (max(1, m1 * k1 * m0 * k0),), g, True)
                    b = H.random_operand(t, (max(1, k1 * n1 * k0 * n0),), g, True)
                    c = H.random_operand(tc, (m1 * n1 * m0 * n0 + 9,), g)
                    sa = (k0, 1, max(k1, 1) * m0 * k0, m0 * k0)
                    sb = (1, k0, n1 * k0 * n0, k0 * n0)
                    sc = (1, m0, m0 * n0, m1 * m0 * n0)  # column-major inside and between blocks
                    want = c.copy()
                    if t == H.I8:
                        orc.port().orc_gemm_packed_i8_i32(m0, n0, k0, m1, n1, k1, 2, P(a), *sa, P(b), *sb, 3, P(want), *sc)
                    else:
                        orc.port().orc_gemm_packed_fp_f32(m0, n0, k0, m1, n1, k1, 2.0, t, P(a), *sa, t, P(b), *sb, 3.0,
                                                         P(want), *sc)
                    got = c.copy()
                    fn(m0, n0, k0, m1, n1, k1, 2, S.ptr(a), *sa, S.ptr(b), *sb, 3, S.ptr(got), *sc)
                    S.check()
                    if t == H.I8:
                        assert np.array_equal(got, want)
                    else:
                        assert np.allclose(got, want, rtol=1e-5, atol=1e-5)
                        assert np.array_equal(got[-9:], want[-9:])


@pytest.mark.parametrize("t", ALL_T)
@pytest.mark.parametrize("where", ["device", "host"])
def test_large_packed_operands_run_unblocked_on_the_tensor_cores(skl, t, where):
    """A blocked problem above 2^24 multiply-adds is unblocked into plain workspaces, run on the tensor-core
    kernel and blocked back (IREE mmt4d-like layout here: A [m1][k1][m0][k0], B [n1][k1][n0][k0], C [m1][n1][m0][n0]).
    int8 is exact; floats are held to the reference suite's forward bound; the guard elements must survive."""
    from oracle import pyoracle as orc
    from gpu_common import DeviceBuf

    P = orc._p
    name = {H.I8: "i8", H.BF16: "bf16", H.F16: "f16", H.F8E4M3: "f8e4m3", H.F8E5M2: "f8e5m2"}[t]
    tc = H.I32 if t == H.I8 else H.F32
    fn = getattr(skl, f"skl_gemm_{name}rcprc_{name}rcprc_{'i32' if t == H.I8 else 'f32'}rcprc_sm100a")
    g = H.rng(23)
    m0, n0, k0, m1, n1, k1 = 16, 8, 4, 20, 36, 72  # M = 320, N = 288, K = 288: 2.65e7 multiply-adds
    M, N, K = m0 * m1, n0 * n1, k0 * k1
    a = H.random_operand(t, (M * K,), g)
    b = H.random_operand(t, (K * N,), g)
    c = H.random_operand(tc, (M * N + 9,), g)
    sa = (k0, 1, k1 * m0 * k0, m0 * k0)              # rs0, cs0, rs1, cs1 of A[m][k]
    sb = (1, k0, n0 * k0, k1 * n0 * k0)              # B[k][n]: k within block unit stride, blocks [n1][k1]
    sc = (n0, 1, n1 * m0 * n0, m0 * n0)
    want = c.copy()
    if t == H.I8:
        orc.port().orc_gemm_packed_i8_i32(m0, n0, k0, m1, n1, k1, 2, P(a), *sa, P(b), *sb, 3, P(want), *sc)
    else:
        orc.port().orc_gemm_packed_fp_f32(m0, n0, k0, m1, n1, k1, 2.0, t, P(a), *sa, t, P(b), *sb, 3.0, P(want), *sc)
    if where == "host":
        got = c.copy()
        fn(m0, n0, k0, m1, n1, k1, 2, S.ptr(a), *sa, S.ptr(b), *sb, 3, S.ptr(got), *sc)
        S.check()
    else:
        da, db, dc = DeviceBuf(a), DeviceBuf(b), DeviceBuf(c)
        fn(m0, n0, k0, m1, n1, k1, 2, da.ptr(0), *sa, db.ptr(0), *sb, 3, dc.ptr(0), *sc)
        S.check()
        got = dc.back()
    assert skl.skl_b200_last_path() == S.PATH_TCGEN05
    assert np.array_equal(got[-9:], want[-9:])
    if t == H.I8:
        assert np.array_equal(got, want)
    else:
        # logical views for the bound
        A = H.to_f32(t, a).reshape(m1, k1, m0, k0).transpose(0, 2, 1, 3).reshape(M, K)
        B = H.to_f32(t, b).reshape(n1, k1, n0, k0).transpose(1, 3, 0, 2).reshape(K, N)
        Cold = c[:M * N].reshape(m1, n1, m0, n0).transpose(0, 2, 1, 3).reshape(M, N)
        u = 2.0 ** -24
        bound = 2 * ((1 + u) ** (K + 2) - 1) * (2.0 * np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64) + 3.0 * np.abs(Cold))
        diff = np.abs(got[:M * N].astype(np.float64) - want[:M * N].astype(np.float64))
        diff = diff.reshape(m1, n1, m0, n0).transpose(0, 2, 1, 3).reshape(M, N)
        assert np.all(diff <= bound + 1e-30)


@pytest.mark.parametrize("t", ALL_T)
@pytest.mark.parametrize("layout", ["rkr", "rrr"])
def test_tail_round_is_split_into_strips(skl, t, layout, monkeypatch):
    """Tile counts that leave a short last round on a 148-SM part (150 and 160 tiles of 128 x 256): the
    leftover tiles are cut into 4 or 2 column strips; results must not depend on the split."""
    for (m, n) in [(128 * 30, 256 * 5), (128 * 32 - 7, 256 * 5 - 9)]:
        for split in ("1", "0"):
            monkeypatch.setenv("SKL_B200_TC_TAIL_SPLIT", split)
            monkeypatch.setenv("SKL_B200_TC_PAIR", "0")
            check_gemm_rc(skl, t, m, n, 256, layout, 1, 0, where="device", path=S.PATH_TCGEN05, align=16,
                          expect_path=S.PATH_TCGEN05, seed=5, all_codes=False)


@pytest.mark.parametrize("beta", [0.0, 0.5])
def test_large_host_operands_take_the_row_chunk_pipeline(skl, beta, monkeypatch):
    """A and C in host memory and large enough for the chunked copy/compute/copy-back pipeline: the result
    must equal the unpipelined route bit for bit, and C's padding columns must survive."""
    import torch

    m, n, k, rsc = 4096 + 300, 2048 + 8, 1024, 2048 + 24
    g = H.rng(77)
    a = H.random_operand(H.BF16, (m, k), g)
    b = H.random_operand(H.BF16, (k, n), g)
    c0 = g.uniform(-1, 1, (m, rsc)).astype(np.float32)
    outs = []
    for mode in ("1", "0"):
        monkeypatch.setenv("SKL_B200_HOST_PIPELINE", mode)
        c = c0.copy()
        skl.skl_gemm_bf16rc_bf16rc_f32rc_sm100a(m, n, k, 1.5, S.ptr(a), k, 1, S.ptr(b), n, 1, beta, S.ptr(c), rsc, 1)
        S.check()
        assert skl.skl_b200_last_path() == S.PATH_TCGEN05
        assert np.array_equal(c[:, n:], c0[:, n:]), "columns outside the matrix were written"
        outs.append(c)
    assert np.array_equal(outs[0], outs[1])
    # and against the oracle on a few rows
    from oracle import pyoracle as orc
    rows = [0, 1, 2047, 2048, 2303, 2304, m - 1]
    for r in rows:
        want = c0[r:r + 1, :n].copy()
        orc.port_gemm_rc(H.BF16, H.BF16, 1, n, k, 1.5, a[r:], k, 1, b, n, 1, beta, want, n, 1)
        bound = H.skl_forward_bound(H.BF16, a[r:r + 1], H.BF16, b, 1.5, beta, c0[r:r + 1, :n], k)
        assert np.all(np.abs(outs[0][r:r + 1, :n].astype(np.float64) - want) <= bound)


@pytest.mark.parametrize("name,dt", [("f32", np.float32), ("f64", np.float64)])
@pytest.mark.parametrize("where", ["device", "host"])
def test_f32_and_f64_gemm_are_bit_exact(skl, name, dt, where):
    """ref/gemm/gemm_f32rc_f32rc_f32rc.c:9-22 and gemm_f64rc_f64rc_f64rc.c:9-22 (+ packed): one accumulator per
    output, k ascending, separately rounded product and sum -- the any-stride kernel reproduces the oracle exactly
    (beta != 0 so that C is read on both sides)."""
    from oracle import pyoracle as orc
    from gpu_common import DeviceBuf

    P = orc._p
    port = orc.port()
    g = H.rng(61)
    rc = getattr(skl, f"skl_gemm_{name}rc_{name}rc_{name}rc_sm100a")
    pk = getattr(skl, f"skl_gemm_{name}rcprc_{name}rcprc_{name}rcprc_sm100a")
    for (m, n, k, col_major_b) in [(1, 1, 1, 0), (17, 33, 65, 0), (130, 70, 257, 1), (5, 9, 0, 0)]:
        kk = max(k, 1)
        a = g.normal(0, 1, (m, kk)).astype(dt)
        b = g.normal(0, 1, (n, kk) if col_major_b else (kk, n)).astype(dt)
        rsb, csb = (1, kk) if col_major_b else (n, 1)
        c = g.normal(0, 1, m * (n + 3) + 5).astype(dt)  # padded rows and a tail the call must not touch
        want = c.copy()
        if name == "f32":
            port.orc_gemm_fp_f32(m, n, k, 1.5, H.F32, P(a), kk, 1, H.F32, P(b), rsb, csb, 0.75, P(want), n + 3, 1)
        else:
            port.orc_gemm_f64(m, n, k, 1, 1, 1, 1.5, P(a), kk, 1, 0, 0, P(b), rsb, csb, 0, 0, 0.75, P(want), n + 3, 1, 0, 0)
        if where == "host":
            got = c.copy()
            rc(m, n, k, 1.5, S.ptr(a), kk, 1, S.ptr(b), rsb, csb, 0.75, S.ptr(got), n + 3, 1)
            S.check()
        else:
            da, db, dc = DeviceBuf(a), DeviceBuf(b), DeviceBuf(c)
            rc(m, n, k, 1.5, da.ptr(0), kk, 1, db.ptr(0), rsb, csb, 0.75, dc.ptr(0), n + 3, 1)
            S.check()
            got = dc.back()
        assert skl.skl_b200_last_path() == S.PATH_GENERIC
        assert np.array_equal(got, want)
    m0, n0, k0, m1, n1, k1 = 4, 3, 2, 5, 7, 9
    sa = (k0, 1, k1 * m0 * k0, m0 * k0)
    sb = (1, k0, n1 * k0 * n0, k0 * n0)
    sc = (1, m0, m0 * n0, m1 * m0 * n0)
    a = g.normal(0, 1, m1 * k1 * m0 * k0).astype(dt)
    b = g.normal(0, 1, k1 * n1 * k0 * n0).astype(dt)
    c = g.normal(0, 1, m1 * n1 * m0 * n0 + 7).astype(dt)
    want = c.copy()
    if name == "f32":
        port.orc_gemm_packed_fp_f32(m0, n0, k0, m1, n1, k1, 2.0, H.F32, P(a), *sa, H.F32, P(b), *sb, 3.0, P(want), *sc)
    else:
        port.orc_gemm_f64(m0, n0, k0, m1, n1, k1, 2.0, P(a), *sa, P(b), *sb, 3.0, P(want), *sc)
    got = c.copy()
    pk(m0, n0, k0, m1, n1, k1, 2.0, S.ptr(a), *sa, S.ptr(b), *sb, 3.0, S.ptr(got), *sc)
    S.check()
    assert np.array_equal(got, want)


@pytest.mark.parametrize("m,n,k,expect", [(1, 300, 512, S.PATH_GEMV), (200, 300, 512, S.PATH_TCGEN05),
                                          (33, 17, 48, S.PATH_GENERIC)])
def test_int32_wrap_around_in_alpha_and_beta(skl, m, n, k, expect):
    """C = beta*C + alpha*acc in two's-complement int32 (ref/gemm/gemm_i8rc_i8rc_i32rc.c:23): factors large enough
    that both products wrap many times; every kernel family must reproduce the reference's wrapped values."""
    from oracle import pyoracle as orc
    from gpu_common import DeviceBuf

    P = orc._p
    g = H.rng(m + n)
    a = g.integers(-128, 128, size=(m, k), dtype=np.int8)
    b = g.integers(-128, 128, size=(n, k), dtype=np.int8)  # [N][K]
    c = g.integers(-2**31, 2**31, size=(m, n), dtype=np.int64).astype(np.int32)
    alpha, beta = 0x01000001, -0x7FFFFFF
    want = c.copy()
    orc.port().orc_gemm_i8_i32(m, n, k, alpha, P(a), k, 1, P(b), 1, k, beta, P(want), n, 1)
    da, db, dc = DeviceBuf(a), DeviceBuf(b), DeviceBuf(c)
    skl.skl_gemm_i8rc_i8rc_i32rc_sm100a(m, n, k, alpha, da.ptr(0), k, 1, db.ptr(0), 1, k, beta, dc.ptr(0), n, 1)
    S.check()
    assert skl.skl_b200_last_path() == expect
    assert np.array_equal(dc.back(), want)
    # the accumulator really wrapped in the reference arithmetic
    exact = beta * c.astype(object) + alpha * (a.astype(np.int64) @ b.astype(np.int64).T).astype(object)
    assert any(abs(int(v)) >= 2**31 for v in exact.ravel()[:64])


@pytest.mark.parametrize("m,n,k1,expect", [(5, 7, 3, S.PATH_GENERIC), (320, 288, 80, S.PATH_TCGEN05)])
def test_int8_1x4_4x1_blocked_entry_point(skl, m, n, k1, expect):
    """skl_gemm_i8rcp1x4_i8p4x1c_i32 (src/gemm/gemm_i8rcp1x4_i8p4x1c_i32_xsfvqdotq.h:43-75): A rows padded to a
    multiple of 4, B interleaved 4 deep; exact against the packed oracle called as that header prescribes."""
    from oracle import pyoracle as orc

    P = orc._p
    g = H.rng(m)
    k = 4 * k1
    rsa1 = k + 8  # padded rows, still a multiple of 4
    a = g.integers(-128, 128, size=m * rsa1, dtype=np.int8)
    rsb1 = 4 * n + 4
    b = g.integers(-128, 128, size=k1 * rsb1, dtype=np.int8)
    c = g.integers(-1000, 1000, size=m * (n + 2) + 3, dtype=np.int32)
    want = c.copy()
    orc.port().orc_gemm_packed_i8_i32(1, 1, 4, m, n, k1, 2, P(a), 0, 1, rsa1, 4, P(b), 1, 0, rsb1, 4, 3, P(want), 0, 0, n + 2, 1)
    got = c.copy()
    skl.skl_gemm_i8rcp1x4_i8p4x1c_i32_sm100a(m, n, k1, 2, S.ptr(a), rsa1, 4, S.ptr(b), rsb1, 3, S.ptr(got), n + 2)
    S.check()
    assert skl.skl_b200_last_path() == expect
    assert np.array_equal(got, want)
    # and against plain matrices rebuilt from the blocked ones
    A = a.reshape(m, rsa1)[:, :k].astype(np.int64)
    B = b.reshape(k1, rsb1)[:, :4 * n].reshape(k1, n, 4).transpose(0, 2, 1).reshape(k, n).astype(np.int64)
    C0 = c[:m * (n + 2)].reshape(m, n + 2)[:, :n].astype(np.int64)
    assert np.array_equal(got[:m * (n + 2)].reshape(m, n + 2)[:, :n], (3 * C0 + 2 * (A @ B)).astype(np.int32))
