"""Regenerates tests/golden/*.npz from the REFERENCE's own scalar routines.

Needs oracle/_ref/libskl-ref.so (``make -C oracle ref`` with the reference tree present).  The
fixtures freeze what skl_*_ref computed for seeded inputs; tests/test_golden.py then holds the
oracle port to them on machines where the reference tree and library are absent.

    python tests/golden/make_golden.py
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from oracle import pyoracle as orc  # noqa: E402
import helpers as H  # noqa: E402

P = orc._p
NAMES = {H.I8: "i8", H.BF16: "bf16", H.F16: "f16", H.F8E4M3: "f8e4m3", H.F8E5M2: "f8e5m2"}


def gemm_rc_cases():
    # (m, n, k, layout) ; layout: how A, B, C are strided
    shapes = [(1, 1, 1), (7, 17, 5), (4, 3, 0), (33, 9, 40), (2, 65, 31)]
    layouts = ["rrr", "crr", "rkr", "rrc", "pad"]
    out = []
    for si, (m, n, k) in enumerate(shapes):
        out.append((m, n, k, layouts[si % len(layouts)]))
    out.append((16, 16, 64, "rkr"))
    return out


def strides_for(layout, m, n, k):
    kk = max(k, 1)
    if layout == "rrr":
        return (kk, 1), (n, 1), (n, 1)
    if layout == "crr":
        return (1, m), (n, 1), (n, 1)
    if layout == "rkr":
        return (kk, 1), (1, kk), (n, 1)
    if layout == "rrc":
        return (kk, 1), (n, 1), (1, m)
    return (kk + 3, 1), (n + 5, 1), (2 * n + 1, 2)


def main():
    ref = orc.ref()
    if ref is None:
        raise SystemExit("oracle/_ref/libskl-ref.so missing: run `make -C oracle ref` first")
    store = {}

    # ---- plain-stride GEMM
    case = 0
    for t in (H.I8, H.BF16, H.F16, H.F8E4M3, H.F8E5M2):
        for (m, n, k, layout) in gemm_rc_cases():
            g = H.rng(1000 + case)
            (rsa, csa), (rsb, csb), (rsc, csc) = strides_for(layout, m, n, k)
            A = H.Strided(t, m, k, rsa, csa, g, all_codes=True)
            B = H.Strided(t, k, n, rsb, csb, g, all_codes=True)
            tc = H.I32 if t == H.I8 else H.F32
            Cm = H.Strided(tc, m, n, rsc, csc, g)
            c0 = Cm.buf.copy()
            alpha, beta = (2, 3) if case % 2 == 0 else (1, 0)
            orc.ref_gemm_rc(t, m, n, k, alpha, A.view, rsa, csa, B.view, rsb, csb, beta, Cm.view, rsc, csc)
            key = f"gemm_rc_{case}"
            store[key + "_meta"] = np.array([t, m, n, k, rsa, csa, rsb, csb, rsc, csc, alpha, beta, A.off, B.off,
                                             Cm.off], dtype=np.int64)
            store[key + "_a"], store[key + "_b"], store[key + "_c0"], store[key + "_c1"] = A.buf, B.buf, c0, Cm.buf
            case += 1
    store["gemm_rc_count"] = np.array([case])

    # ---- packed GEMM: blocks stored block-row-major, inside a block row-major (A, C) / column-major (B)
    case = 0
    for t in (H.I8, H.BF16, H.F16, H.F8E4M3, H.F8E5M2):
        for (m0, n0, k0, m1, n1, k1) in [(4, 3, 2, 2, 3, 5), (1, 4, 4, 3, 1, 2), (5, 5, 1, 1, 2, 7)]:
            g = H.rng(2000 + case)
            a = H.random_operand(t, (m1 * k1 * m0 * k0,), g, True)
            b = H.random_operand(t, (k1 * n1 * k0 * n0,), g, True)
            tc = H.I32 if t == H.I8 else H.F32
            c = H.random_operand(tc, (m1 * n1 * m0 * n0,), g)
            c0 = c.copy()
            sa = (k0, 1, k1 * m0 * k0, m0 * k0)      # rsa0, csa0, rsa1, csa1
            sb = (1, k0, n1 * k0 * n0, k0 * n0)      # rsb0, csb0, rsb1, csb1
            sc = (n0, 1, n1 * m0 * n0, m0 * n0)
            alpha, beta = (2, 3)
            name = NAMES[t]
            if t == H.I8:
                ref.skl_gemm_i8rcprc_i8rcprc_i32rcprc_ref(m0, n0, k0, m1, n1, k1, alpha, P(a), *sa, P(b), *sb, beta,
                                                          P(c), *sc)
            else:
                getattr(ref, f"skl_gemm_{name}rcprc_{name}rcprc_f32rcprc_ref")(
                    m0, n0, k0, m1, n1, k1, float(alpha), P(a), *sa, P(b), *sb, float(beta), P(c), *sc)
            key = f"gemm_p_{case}"
            store[key + "_meta"] = np.array([t, m0, n0, k0, m1, n1, k1, *sa, *sb, *sc, alpha, beta], dtype=np.int64)
            store[key + "_a"], store[key + "_b"], store[key + "_c0"], store[key + "_c1"] = a, b, c0, c
            case += 1
    store["gemm_p_count"] = np.array([case])

    # ---- cvt to fp8: specials, rounding boundaries of both formats, random values
    g = H.rng(3000)
    specials = np.array([np.nan, np.inf, -np.inf, 0.0, -0.0, 448, 464, 465, 480, -448, -464, -465, -1e9, 1e9,
                         57344, 61439.9, 61440, 65536, -57344, -61440, 2.0 ** -6, 2.0 ** -7, 2.0 ** -9, 2.0 ** -10,
                         1.5 * 2.0 ** -10, 2.0 ** -14, 2.0 ** -16, 2.0 ** -17, 3 * 2.0 ** -18, 1e-30, -1e-40,
                         0.9999999, 255.99998, 0.015624999], dtype=np.float32)
    codes = np.arange(256, dtype=np.uint8)
    mids = []
    for fmt in (H.F8E4M3, H.F8E5M2):
        v = H.f8_table(fmt)
        v = np.sort(np.unique(v[np.isfinite(v)]))
        mid = ((v[:-1].astype(np.float64) + v[1:].astype(np.float64)) / 2).astype(np.float32)
        mids += [mid, np.nextafter(mid, np.float32(np.inf)), np.nextafter(mid, np.float32(-np.inf)), v]
    rnd = np.concatenate([g.uniform(-512, 512, 1500), g.normal(0, 1, 1500), g.uniform(-7e4, 7e4, 500)]).astype(np.float32)
    src32 = np.concatenate([specials] + mids + [rnd]).astype(np.float32)
    src16 = H.f32_to_bf16_bits(src32)
    store["cvt_src32"], store["cvt_src16"] = src32, src16
    for fmt in ("f8e4m3", "f8e5m2"):
        for sat in ("", "sat_"):
            for si, scale in enumerate((1.0, 1.5)):
                d = np.zeros(src32.size, dtype=np.uint8)
                getattr(ref, f"skl_cvt_{sat}f32_{fmt}_ref")(P(d), P(src32), scale, src32.size)
                store[f"cvt_{sat}f32_{fmt}_{si}"] = d.copy()
                getattr(ref, f"skl_cvt_{sat}bf16_{fmt}_ref")(P(d), P(src16), scale, src16.size)
                store[f"cvt_{sat}bf16_{fmt}_{si}"] = d.copy()
        w = np.zeros(256, dtype=np.uint16)
        getattr(ref, f"skl_cvt_{fmt}_bf16_ref")(P(w), P(codes), 256)
        store[f"cvt_{fmt}_bf16"] = w
    for n in (512, 511, 1):
        d = np.zeros(n, dtype=np.uint8)
        ref.skl_cvt_f4e2m1_f8e4m3_ref(P(d), P(codes), n)
        store[f"cvt_f4_{n}"] = d

    # ---- pack / unpack / transpose
    case = 0
    for e, dt in ((8, np.uint8), (16, np.uint16), (32, np.uint32)):
        for (m, n, m0, n0, src_cm, blk_cm) in [(13, 10, 4, 3, 0, 0), (8, 8, 8, 8, 1, 1), (5, 7, 2, 4, 0, 1),
                                                (1, 9, 3, 3, 1, 0)]:
            g = H.rng(4000 + case)
            src = g.integers(0, 2 ** min(e, 31), size=m * n + 7).astype(dt)
            rs, cs = (1, m) if src_cm else (n, 1)
            m1, n1 = -(-m // m0), -(-n // n0)
            rs0, cs0 = (1, m0) if blk_cm else (n0, 1)
            rs1, cs1 = n1 * m0 * n0, m0 * n0
            dst = np.full(m1 * n1 * m0 * n0 + 5, 0xAB, dtype=dt)
            getattr(ref, f"skl_pack_e{e}rc_e{e}rcprc_ref")(m, n, P(src), rs, cs, m0, n0, P(dst), rs0, cs0, rs1, cs1, 0xFF)
            key = f"pack_{case}"
            store[key + "_meta"] = np.array([e, m, n, rs, cs, m0, n0, rs0, cs0, rs1, cs1], dtype=np.int64)
            store[key + "_src"], store[key + "_dst"] = src, dst.copy()
            if e == 8:
                back = np.full(m * n + 7, 0xCD, dtype=dt)
                ref.skl_unpack_e8rcprc_e8rc_ref(m0, n0, P(dst), rs0, cs0, rs1, cs1, m, n, P(back), rs, cs)
                store[key + "_back"] = back
            rsa, rsat = n + 2, m + 3
            a = g.integers(0, 2 ** min(e, 31), size=m * rsa).astype(dt)
            at = np.full(n * rsat, 0xEE, dtype=dt)
            getattr(ref, f"skl_transpose_e{e}_ref")(m, n, P(a), rsa, P(at), rsat)
            store[key + "_ta"], store[key + "_tat"] = a, at
            case += 1
    store["pack_count"] = np.array([case])

    # ---- activations the fused GEMM epilogue follows: skl_sigmoid_f32_ref (logistic / silu / swish / swiglu
    # through its beta, y, up, delta arguments) and skl_gelu_f32_ref, on the input ranges of the reference's
    # own tests (test/sigmoid/sigmoid_f32_zve32f.c:27-39, test/gelu/skl_gelu_f32_zve32f.c:23-24) plus specials
    g = H.rng(77)
    specials = np.array([0.0, -0.0, 1.0, -1.0, np.inf, -np.inf, np.nan, 1e-30, -1e-30, 88.0, -88.0, 104.0, -104.0],
                        dtype=np.float32)
    for name, lo, hi in (("logistic", -104.0, 18.0), ("silu", -110.0, 18.0), ("swish2", -110.0, 18.0),
                         ("swiglu", -55.0, 18.0), ("gelu", -14.356, 5.348)):
        x = np.concatenate([g.uniform(lo, hi, 4096).astype(np.float32), g.normal(0, 2, 2048).astype(np.float32),
                            specials])
        up = g.normal(0, 3, x.size).astype(np.float32)
        out = np.zeros_like(x)
        if name == "logistic":
            ref.skl_sigmoid_f32_ref(P(out), 1.0, P(x), None, None, 0.0, x.size)
        elif name == "silu":
            ref.skl_sigmoid_f32_ref(P(out), 1.0, P(x), P(x), None, 0.0, x.size)
        elif name == "swish2":
            ref.skl_sigmoid_f32_ref(P(out), 2.0, P(x), P(x), None, 0.0, x.size)
        elif name == "swiglu":
            ref.skl_sigmoid_f32_ref(P(out), 1.0, P(x), P(x), P(up), 0.5, x.size)
        else:
            ref.skl_gelu_f32_ref(P(out), P(x), x.size)
        store[f"act_{name}_x"], store[f"act_{name}_up"], store[f"act_{name}_out"] = x, up, out

    # ---- fp32 / fp64 GEMM (plain strides), skl_gemm_f32rc_f32rc_f32rc_ref / skl_gemm_f64rc_f64rc_f64rc_ref
    g = H.rng(88)
    for name, dt in (("f32", np.float32), ("f64", np.float64)):
        m, n, k = 9, 11, 23
        a = g.normal(0, 1, (m, k)).astype(dt)
        b = g.normal(0, 1, (k, n)).astype(dt)
        c = g.normal(0, 1, (m, n)).astype(dt)
        out = c.copy()
        getattr(ref, f"skl_gemm_{name}rc_{name}rc_{name}rc_ref")(m, n, k, 1.25, P(a), k, 1, P(b), n, 1, -0.5, P(out), n, 1)
        store[f"gemm_{name}_a"], store[f"gemm_{name}_b"], store[f"gemm_{name}_c"], store[f"gemm_{name}_out"] = a, b, c, out

    path = os.path.join(HERE, "skl_ref_golden.npz")
    np.savez_compressed(path, **store)
    print(path, os.path.getsize(path), "bytes,", len(store), "arrays")


if __name__ == "__main__":
    main()
