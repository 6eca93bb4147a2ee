"""Runs one GEMM through the C ABI (host or device pointers) and checks it against the oracle."""
from __future__ import annotations

import os

import numpy as np

import helpers as H
import skl_b200 as S
from oracle import pyoracle as orc

RC_FN = {H.I8: "skl_gemm_i8rc_i8rc_i32rc_sm100a", H.BF16: "skl_gemm_bf16rc_bf16rc_f32rc_sm100a",
         H.F16: "skl_gemm_f16rc_f16rc_f32rc_sm100a", H.F8E4M3: "skl_gemm_f8e4m3rc_f8e4m3rc_f32rc_sm100a",
         H.F8E5M2: "skl_gemm_f8e5m2rc_f8e5m2rc_f32rc_sm100a"}


def up(x, a):
    return (x + a - 1) // a * a


def layout_strides(layout: str, m: int, n: int, k: int, align: int = 1):
    """Element strides for A (m x k), B (k x n), C (m x n).  Letters: r row-major, c column-major;
    for B, 'k' is the "[N][K]" weight layout (k contiguous).  `align` pads leading strides."""
    kk, mm, nn = up(max(k, 1), align), up(m, align), up(n, align)
    sa = {"r": (kk, 1), "c": (1, mm)}[layout[0]]
    sb = {"r": (nn, 1), "c": (1, kk), "k": (1, kk)}[layout[1]]
    sc = {"r": (nn, 1), "c": (1, mm), "p": (2 * nn + 3, 2)}[layout[2]]
    return sa, sb, sc


class DeviceBuf:
    """A numpy buffer mirrored in device memory (torch), addressed by the same element offsets."""

    def __init__(self, arr: np.ndarray):
        import torch

        self.np = arr
        self.t = torch.from_numpy(arr.view(np.uint8).copy()).cuda()
        self.itemsize = arr.itemsize

    def ptr(self, off_elems: int) -> int:
        return self.t.data_ptr() + off_elems * self.itemsize

    def back(self) -> np.ndarray:
        return self.t.cpu().numpy().view(self.np.dtype).reshape(self.np.shape)


def call_rc(lib, t, m, n, k, alpha, A, B, beta, C, where: str):
    """A, B, C: helpers.Strided.  Returns the full C allocation after the call."""
    fn = getattr(lib, RC_FN[t])
    if where == "host":
        fn(m, n, k, alpha, S.ptr(A.view), A.rs, A.cs, S.ptr(B.view), B.rs, B.cs, beta, S.ptr(C.view), C.rs, C.cs)
        S.check()
        return C.buf
    import torch

    da, db, dc = DeviceBuf(A.buf), DeviceBuf(B.buf), DeviceBuf(C.buf)
    fn(m, n, k, alpha, da.ptr(A.off), A.rs, A.cs, db.ptr(B.off), B.rs, B.cs, beta, dc.ptr(C.off), C.rs, C.cs)
    S.check()
    torch.cuda.synchronize()
    return dc.back()


def check_gemm_rc(lib, t, m, n, k, layout="rrr", alpha=1, beta=0, where="device", path=0, align=1, seed=0,
                  all_codes=True, expect_path=None):
    g = H.rng(seed * 7919 + m * 31 + n * 17 + k)
    (rsa, csa), (rsb, csb), (rsc, csc) = layout_strides(layout, m, n, k, align)
    A = H.Strided(t, m, k, rsa, csa, g, all_codes=all_codes)
    B = H.Strided(t, k, n, rsb, csb, g, all_codes=all_codes)
    tc = H.I32 if t == H.I8 else H.F32
    C = H.Strided(tc, m, n, rsc, csc, g)
    want = C.copy()
    if m * n * max(k, 1) > (1 << 22):  # rows are independent: thread the oracle over row slabs
        orc.rows_in_parallel(lambda i0, cnt: orc.port_gemm_rc(t, t, cnt, n, k, alpha, A.view[i0 * rsa:], rsa, csa, B.view,
                                                              rsb, csb, beta, want.view[i0 * rsc:], rsc, csc),
                             m, min(16, os.cpu_count() or 1))
    else:
        orc.port_gemm_rc(t, t, m, n, k, alpha, A.view, rsa, csa, B.view, rsb, csb, beta, want.view, rsc, csc)
    before = C.copy()
    lib.skl_b200_force_path(path)
    try:
        after = call_rc(lib, t, m, n, k, alpha, A, B, beta, C, where)
    finally:
        lib.skl_b200_force_path(0)
    used = lib.skl_b200_last_path()
    if expect_path is not None and m and n:
        assert used == expect_path, f"expected kernel family {expect_path}, library used {used}"
    H.assert_untouched_outside(before, after, "C")
    got = after[C.idx()] if m and n else np.zeros((m, n), NP(tc))
    ref = want.get() if m and n else got
    if t == H.I8:
        assert np.array_equal(got, ref), f"int8 GEMM not bit-exact: {np.count_nonzero(got != ref)} of {got.size} differ"
    else:
        bound = H.skl_forward_bound(t, A.get() if k else np.zeros((m, 0), A.buf.dtype),
                                    t, B.get() if k else np.zeros((0, n), B.buf.dtype), alpha, beta,
                                    before.get() if m and n else None, k)
        err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
        worst = np.max(err - bound) if err.size else 0.0
        assert np.all(err <= bound + 1e-30), f"float GEMM outside the reference's bound by {worst:g} (path {used})"
    return used


def NP(t):
    return H.NP_STORE[t]
