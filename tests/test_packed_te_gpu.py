"""The matrix-engine packed GEMM entry points (skl_gemm_<t>rcptex1c_<t>rcp1xte_<out>rcptexterc_sm100a) and the TE x 1
packing routine, through the C ABI.

Each entry point is checked against the oracle's general packed GEMM called the way SKL's headers state the
equivalence (src/gemm/gemm_i8c_i8_i32_xsfmm32a8i.h:86-96: m0 = n0 = TE, k0 = 1, A strides (1, 0), B strides (0, 1)),
over the block-count sweep of SKL's own test of these kernels
(test/gemm/xsfmm/skl_gemm_i8rcptex1c_i8rcp1xte_i32rcptexterc_xsfmm32a8i.c:61-223): block counts 1..7, k = 0..15,
alpha / beta = 1 / 0 and 2 / 3, a strided C block (csc0 = 2) and a column-major one (rsc0 = 1, csc0 = TE).
int8 must be bit-exact; float types are held to the reference suite's forward bound.  Problems with TMA-compatible
strides run on the tensor cores straight from the packed panels; others fall to the any-stride kernel."""
import numpy as np
import pytest

import helpers as H
import skl_b200 as S
from gpu_common import DeviceBuf
from oracle import pyoracle as orc

pytestmark = pytest.mark.gpu
P = orc._p
NAMES = {H.I8: "i8", H.BF16: "bf16", H.F16: "f16", H.F8E4M3: "f8e4m3", H.F8E5M2: "f8e5m2"}


def te_fn(skl, t):
    n = NAMES[t]
    return getattr(skl, f"skl_gemm_{n}rcptex1c_{n}rcp1xte_{'i32' if t == H.I8 else 'f32'}rcptexterc_sm100a")


def run_case(skl, t, m1, n1, k, alpha, beta, cmode, where, kpad=0, seed=0):
    """cmode: 'r' row-major blocks, 's' csc0 = 2, 'c' column-major blocks.  kpad: extra elements in the k stride."""
    te = skl.skl_b200_te()
    g = H.rng(1000 * m1 + 100 * n1 + k + seed)
    tc = H.I32 if t == H.I8 else H.F32
    csa1 = te + kpad  # stride between consecutive k inside a block row of A
    rsa1 = csa1 * max(k, 1) + 16
    rsb1 = n1 * te + kpad  # B: all block columns of one k side by side
    csb1 = te
    a = H.random_operand(t, (m1 * rsa1 + 16,), g, False)
    b = H.random_operand(t, (max(k, 1) * rsb1 + 16,), g, False)
    if cmode == "r":
        rsc0, csc0, blk = te, 1, te * te
    elif cmode == "s":
        rsc0, csc0, blk = 2 * te, 2, 2 * te * te
    else:
        rsc0, csc0, blk = 1, te, te * te
    csc1, rsc1 = blk, n1 * blk
    c = H.random_operand(tc, (m1 * n1 * blk + 9,), g)
    want = c.copy()
    args_a = (1, 0, rsa1, csa1)
    args_b = (0, 1, rsb1, csb1)
    args_c = (rsc0, csc0, rsc1, csc1)
    if t == H.I8:
        orc.port().orc_gemm_packed_i8_i32(te, te, 1, m1, n1, k, alpha, P(a), *args_a, P(b), *args_b, beta, P(want), *args_c)
    else:
        orc.port().orc_gemm_packed_fp_f32(te, te, 1, m1, n1, k, float(alpha), t, P(a), *args_a, t, P(b), *args_b,
                                          float(beta), P(want), *args_c)
    fn = te_fn(skl, t)
    if where == "host":
        got = c.copy()
        fn(m1, n1, k, alpha, S.ptr(a), rsa1, csa1, S.ptr(b), rsb1, csb1, beta, S.ptr(got), *args_c)
        S.check()
    else:
        da, db, dc = DeviceBuf(a), DeviceBuf(b), DeviceBuf(c)
        fn(m1, n1, k, alpha, da.ptr(0), rsa1, csa1, db.ptr(0), rsb1, csb1, beta, dc.ptr(0), *args_c)
        S.check()
        got = dc.back()
    path = skl.skl_b200_last_path()
    if cmode == "s":  # the odd positions of a strided block belong to nobody
        untouched = np.ones(c.size, bool)
        for bi in range(m1 * n1):
            untouched[bi * blk:(bi + 1) * blk:2] = False
        assert np.array_equal(got[untouched], c[untouched]), "elements outside the blocks were written"
    assert np.array_equal(got[-9:], c[-9:])
    if t == H.I8:
        assert np.array_equal(got, want), f"{np.count_nonzero(got != want)} of {got.size} differ (path {path})"
    else:
        M, N = m1 * te, n1 * te
        A = np.zeros((M, max(k, 1)), np.float64)
        B = np.zeros((max(k, 1), N), np.float64)
        af, bf = H.to_f32(t, a).astype(np.float64), H.to_f32(t, b).astype(np.float64)
        for i1 in range(m1):
            for kk in range(k):
                A[i1 * te:(i1 + 1) * te, kk] = af[i1 * rsa1 + kk * csa1:i1 * rsa1 + kk * csa1 + te]
        for kk in range(k):
            for j1 in range(n1):
                B[kk, j1 * te:(j1 + 1) * te] = bf[kk * rsb1 + j1 * csb1:kk * rsb1 + j1 * csb1 + te]
        if k == 0:
            A[:], B[:] = 0, 0
        u = 2.0 ** -24
        acc = np.abs(A) @ np.abs(B)
        idx = np.zeros((M, N), np.int64)
        for i1 in range(m1):
            for j1 in range(n1):
                base = i1 * rsc1 + j1 * csc1
                idx[i1 * te:(i1 + 1) * te, j1 * te:(j1 + 1) * te] = (base + np.arange(te)[:, None] * rsc0 +
                                                                     np.arange(te)[None, :] * csc0)
        bound = 2 * ((1 + u) ** (k + 2) - 1) * (abs(alpha) * acc + abs(beta) * np.abs(c[idx].astype(np.float64)))
        diff = np.abs(got[idx].astype(np.float64) - want[idx].astype(np.float64))
        assert np.all(diff <= bound + 1e-30), f"outside the bound by {np.max(diff - bound):g} (path {path})"
    return path


@pytest.mark.parametrize("t", [H.I8, H.BF16, H.F16, H.F8E4M3, H.F8E5M2])
def test_block_count_sweep(skl, t):
    te = skl.skl_b200_te()
    assert te == 128
    for k in (0, 1, 2, 3, 7, 11):
        for n1 in (1, 2, 7):
            path = run_case(skl, t, 7, n1, k, 1, 0, "r", "device")
            big = 7 * n1 * te * te * k >= 32768
            assert path == (S.PATH_TCGEN05 if big else S.PATH_GENERIC)
    for m1 in (1, 2, 5):
        for n1 in (1, 3, 6):
            assert run_case(skl, t, m1, n1, 15, 1, 0, "r", "device") == S.PATH_TCGEN05
    for n1 in (1, 4, 7):
        assert run_case(skl, t, 7, n1, 15, 2, 3, "r", "device") == S.PATH_TCGEN05
    assert run_case(skl, t, 7, 7, 15, 2, 3, "s", "device") == S.PATH_TCGEN05
    assert run_case(skl, t, 7, 7, 15, 2, 3, "c", "device") == S.PATH_TCGEN05


@pytest.mark.parametrize("t", [H.I8, H.BF16, H.F8E4M3])
def test_deep_k_host_pointers_and_odd_strides(skl, t):
    # k spanning several 128-byte slabs with a ragged last one; host operands are staged and then read in place
    assert run_case(skl, t, 3, 2, 200, 2, 3, "r", "host") == S.PATH_TCGEN05
    assert run_case(skl, t, 2, 5, 333, 1, 0, "c", "device") == S.PATH_TCGEN05
    # k strides padded by 16 bytes stay on the tensor cores; a stride TMA cannot express goes to the any-stride kernel
    assert run_case(skl, t, 2, 2, 40, 2, 3, "r", "device", kpad=16) == S.PATH_TCGEN05
    assert run_case(skl, t, 2, 2, 40, 2, 3, "r", "device", kpad=1) == S.PATH_GENERIC


def test_f32_entry_point_is_bit_exact(skl):
    """The fp32 matrix-engine entry (gemm_f32c_f32_f32_xsfmm32a32f.h:96-99) runs on the any-stride kernel: one
    accumulator per output, k ascending, so it reproduces the oracle exactly."""
    te = skl.skl_b200_te()
    g = H.rng(5)
    m1, n1, k = 2, 3, 9
    a = g.uniform(-1, 1, m1 * te * k).astype(np.float32)
    b = g.uniform(-1, 1, k * n1 * te).astype(np.float32)
    c = g.uniform(-1, 1, m1 * n1 * te * te).astype(np.float32)
    want = c.copy()
    sa, sb, sc = (1, 0, te * k, te), (0, 1, n1 * te, te), (te, 1, n1 * te * te, te * te)
    orc.ref().skl_gemm_f32rcprc_f32rcprc_f32rcprc_ref(te, te, 1, m1, n1, k, 1.5, P(a), *sa, P(b), *sb, 0.5, P(want), *sc) \
        if orc.ref() is not None else None
    got = c.copy()
    skl.skl_gemm_f32rcptex1c_f32rcp1xte_f32rcptexterc_sm100a(m1, n1, k, 1.5, S.ptr(a), te * k, te, S.ptr(b), n1 * te, te,
                                                             0.5, S.ptr(got), *sc)
    S.check()
    if orc.ref() is not None:
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # and against the plain entry point on the unpacked matrices
    A = a.reshape(m1, k, te).transpose(0, 2, 1).reshape(m1 * te, k).copy()
    B = b.reshape(k, n1 * te)
    C0 = c.reshape(m1, n1, te, te).transpose(0, 2, 1, 3).reshape(m1 * te, n1 * te).copy()
    skl.skl_gemm_f32rc_f32rc_f32rc_sm100a(m1 * te, n1 * te, k, 1.5, S.ptr(A), k, 1, S.ptr(B), n1 * te, 1, 0.5, S.ptr(C0),
                                          n1 * te, 1)
    S.check()
    assert np.array_equal(got.reshape(m1, n1, te, te).transpose(0, 2, 1, 3).reshape(m1 * te, n1 * te), C0)


@pytest.mark.parametrize("bits,dt", [(8, np.uint8), (16, np.uint16), (32, np.uint32)])
@pytest.mark.parametrize("where", ["device", "host"])
def test_te_pack_matches_the_general_pack(skl, bits, dt, where):
    """skl_pack_e<bits>_e<bits>rcptex1c: the general pack with (m0, n0) = (TE, 1), (rs0, cs0) = (1, 0)
    (src/pack/pack_e16_xsfmmbase.h:30-51); ragged row counts are padded; bytes between block rows stay untouched."""
    te = skl.skl_b200_te()
    g = H.rng(bits)
    for (m, n, rs) in [(300, 70, 75), (128, 1, 1), (5, 33, 40), (1000, 260, 260)]:
        src = g.integers(0, 250, size=(m, rs)).astype(dt)
        m1 = -(-m // te)
        cs1, rs1 = te, te * n + 24
        dst = g.integers(0, 250, size=(m1 * rs1 + 5,)).astype(dt)
        want = dst.copy()
        orc.port().orc_pack(bits // 8, m, n, P(src), rs, 1, te, 1, P(want), 1, 0, rs1, cs1, 0xAB)
        fn = getattr(skl, f"skl_pack_e{bits}_e{bits}rcptex1c_sm100a")
        if where == "host":
            got = dst.copy()
            fn(m, n, S.ptr(src), rs, S.ptr(got), rs1, cs1, 0xAB)
            S.check()
        else:
            ds, dd = DeviceBuf(src), DeviceBuf(dst)
            fn(m, n, ds.ptr(0), rs, dd.ptr(0), rs1, cs1, 0xAB)
            S.check()
            got = dd.back()
        assert np.array_equal(got, want)


def test_pack_then_gemm_equals_the_plain_gemm(skl):
    """Round trip through the pre-packed layout: A (row-major) and B^T (row-major [N][K]) are packed into TE x 1 panels
    by the library, multiplied by the packed entry point, and the blocked C is compared with the plain int8 GEMM;
    unpacking the packed A with the general unpack gives A back."""
    import torch

    te = skl.skl_b200_te()
    m, n, k = 3 * te, 2 * te, 300
    g = H.rng(99)
    a = g.integers(-128, 128, size=(m, k), dtype=np.int8)
    bt = g.integers(-128, 128, size=(n, k), dtype=np.int8)  # B transposed: row j holds column j of B
    da, dbt = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    pa = torch.zeros(m * k, dtype=torch.int8, device="cuda")
    pb = torch.zeros(n * k, dtype=torch.int8, device="cuda")
    skl.skl_pack_e8_e8rcptex1c_sm100a(m, k, da.data_ptr(), k, pa.data_ptr(), te * k, te, 0)
    S.check()
    skl.skl_pack_e8_e8rcptex1c_sm100a(n, k, dbt.data_ptr(), k, pb.data_ptr(), te * k, te, 0)
    S.check()
    # packed B^T panels: element (kk, j) of block column j1 at j1*te*k + kk*te + j  ->  rsb1 = te, csb1 = te*k
    pc = torch.zeros(m * n, dtype=torch.int32, device="cuda")
    skl.skl_gemm_i8rcptex1c_i8rcp1xte_i32rcptexterc_sm100a(m // te, n // te, k, 1, pa.data_ptr(), te * k, te,
                                                           pb.data_ptr(), te, te * k, 0, pc.data_ptr(), te, 1,
                                                           (n // te) * te * te, te * te)
    S.check()
    assert skl.skl_b200_last_path() == S.PATH_TCGEN05
    plain = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    skl.skl_gemm_i8rc_i8rc_i32rc_sm100a(m, n, k, 1, da.data_ptr(), k, 1, dbt.data_ptr(), 1, k, 0, plain.data_ptr(), n, 1)
    S.check()
    blocked = pc.cpu().numpy().reshape(m // te, n // te, te, te).transpose(0, 2, 1, 3).reshape(m, n)
    assert np.array_equal(blocked, plain.cpu().numpy())
    assert np.array_equal(blocked, a.astype(np.int32) @ bt.astype(np.int32).T)
    back = torch.zeros((m, k), dtype=torch.int8, device="cuda")
    skl.skl_unpack_e8rcprc_e8rc_sm100a(te, 1, pa.data_ptr(), 1, 0, te * k, te, m, k, back.data_ptr(), k, 1)
    S.check()
    assert torch.equal(back, da)
