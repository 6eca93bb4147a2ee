"""cvt / pack / unpack / transpose parity on the GPU: byte-exact against the oracle, inputs after the
reference's suites (test/cvt/cvt_f32_f8.c:29-35 plants NaN, +Inf, -Inf in slots 0..2 of values in
[-512, 512]; test/cvt/cvt_f8_bf16.h:50-52 sweeps all 256 codes; test/pack/rvv/skl_pack_e8rc_e8rcprc_zve32x.c:57-159
covers row/column-major sources, every block orientation and pad = 0xFF)."""
import numpy as np
import pytest

import helpers as H
import skl_b200 as S
from gpu_common import DeviceBuf
from oracle import pyoracle as orc

pytestmark = pytest.mark.gpu
P = orc._p


def cvt_inputs(n, seed):
    g = H.rng(seed)
    x = g.uniform(-512, 512, n).astype(np.float32)
    x[:3] = np.array([np.nan, np.inf, -np.inf], np.float32)[:min(n, 3)]
    if n > 64:
        x[3:11] = [0.0, -0.0, 448, 464, 465, -465, 61440, 2.0 ** -10]
        x[11:40] = g.normal(0, 1e-2, 29)
        x[40:64] = g.uniform(-7e4, 7e4, 24)
    return x


@pytest.mark.parametrize("fmt", ["f8e4m3", "f8e5m2"])
@pytest.mark.parametrize("sat", ["", "sat_"])
@pytest.mark.parametrize("src", ["f32", "bf16"])
@pytest.mark.parametrize("n,scale", [(1024, 1.0), (1024, 1.5), (1, 1.0), (17, 1.5), (4099, 0.37), (1 << 20, 1.0)])
def test_cvt_to_fp8(skl, fmt, sat, src, n, scale):
    x = cvt_inputs(n, n + 3)
    f = H.F8E4M3 if fmt == "f8e4m3" else H.F8E5M2
    want = np.zeros(n, np.uint8)
    if src == "f32":
        xin = x
        orc.port().orc_cvt_f32_f8(P(want), P(xin), scale, n, f, int(sat != ""))
    else:
        xin = H.f32_to_bf16_bits(x)
        orc.port().orc_cvt_bf16_f8(P(want), P(xin), scale, n, f, int(sat != ""))
    fn = getattr(skl, f"skl_cvt_{sat}{src}_{fmt}_sm100a")
    # host pointers (staged), with canaries around dst
    dst = np.full(n + 32, 0x5A, np.uint8)
    fn(S.ptr(dst[16:]), S.ptr(xin), scale, n)
    S.check()
    assert np.array_equal(dst[16:16 + n], want)
    assert np.all(dst[:16] == 0x5A) and np.all(dst[16 + n:] == 0x5A)
    # device pointers, deliberately misaligned by one element to take the scalar path as well
    for shift in (0, 1):
        if n <= shift:
            continue
        dsrc, ddst = DeviceBuf(xin), DeviceBuf(np.full(n + 32, 0x5A, np.uint8))
        fn(ddst.ptr(16 + shift), dsrc.ptr(shift), scale, n - shift)
        S.check()
        out = ddst.back()
        assert np.array_equal(out[16 + shift:16 + n], want[shift:])
        assert np.all(out[:16 + shift] == 0x5A) and np.all(out[16 + n:] == 0x5A)


@pytest.mark.parametrize("fmt", ["f8e4m3", "f8e5m2"])
def test_cvt_fp8_to_bf16_all_codes(skl, fmt):
    f = H.F8E4M3 if fmt == "f8e4m3" else H.F8E5M2
    codes = np.tile(np.arange(256, dtype=np.uint8), 9)[:2301]
    want = np.zeros(codes.size, np.uint16)
    orc.port().orc_cvt_f8_bf16(P(want), P(codes), codes.size, f)
    got = np.zeros(codes.size, np.uint16)
    getattr(skl, f"skl_cvt_{fmt}_bf16_sm100a")(S.ptr(got), S.ptr(codes), codes.size)
    S.check()
    assert np.array_equal(got, want)
    d_in, d_out = DeviceBuf(codes), DeviceBuf(np.zeros(codes.size, np.uint16))
    getattr(skl, f"skl_cvt_{fmt}_bf16_sm100a")(d_out.ptr(0), d_in.ptr(0), codes.size)
    S.check()
    assert np.array_equal(d_out.back(), want)


def test_cvt_fp4_to_fp8(skl):
    codes = np.arange(256, dtype=np.uint8)
    for n in (512, 511, 1, 0):
        want = np.zeros(max(n, 1), np.uint8)
        orc.port().orc_cvt_f4e2m1_f8e4m3(P(want), P(codes), n)
        got = np.zeros(max(n, 1), np.uint8)
        skl.skl_cvt_f4e2m1_f8e4m3_sm100a(S.ptr(got), S.ptr(codes), n)
        S.check()
        assert np.array_equal(got, want)


def test_hardware_assisted_encoder_equals_integer_encoder_on_all_fp32(skl):
    """All 2^32 fp32 bit patterns, both formats, both overflow flavours, compared on the device."""
    import torch

    bad = torch.zeros(1, dtype=torch.int64, device="cuda")
    for fmt in (H.F8E4M3, H.F8E5M2):
        for sat in (0, 1):
            rc = skl.skl_b200_launch_cvt_selfcheck(fmt, sat, 0, 1 << 32, bad.data_ptr(), None)
            assert rc == 0
    torch.cuda.synchronize()
    assert int(bad.item()) == 0


def test_integer_encoder_on_device_equals_oracle_sample(skl):
    """2^22 fp32 patterns spread over the whole range through the public entry point vs the oracle."""
    g = H.rng(123)
    bits = (np.arange(1 << 22, dtype=np.uint64) * 1021 + g.integers(0, 1021, 1 << 22, dtype=np.uint64)).astype(np.uint32)
    x = bits.view(np.float32)
    for fmt, f in (("f8e4m3", H.F8E4M3), ("f8e5m2", H.F8E5M2)):
        for sat in ("", "sat_"):
            want = np.zeros(x.size, np.uint8)
            orc.port().orc_cvt_f32_f8(P(want), P(x), 1.0, x.size, f, int(sat != ""))
            got = np.zeros(x.size, np.uint8)
            getattr(skl, f"skl_cvt_{sat}f32_{fmt}_sm100a")(S.ptr(got), S.ptr(x), 1.0, x.size)
            S.check()
            assert np.array_equal(got, want)


PACK_CASES = [(128, 128, 8, 8), (13, 10, 4, 3), (1, 1, 1, 1), (65, 3, 64, 1), (7, 9, 16, 16), (200, 150, 32, 64),
              (64, 64, 64, 64), (3, 300, 1, 128), (0, 4, 2, 2), (256, 192, 128, 64), (250, 176, 32, 48), (96, 512, 96, 16)]


@pytest.mark.parametrize("e", [8, 16, 32])
@pytest.mark.parametrize("where", ["host", "device"])
def test_pack_unpack(skl, e, where):
    dt = {8: np.uint8, 16: np.uint16, 32: np.uint32}[e]
    g = H.rng(200 + e)
    fn = getattr(skl, f"skl_pack_e{e}rc_e{e}rcprc_sm100a")
    for (m, n, m0, n0) in PACK_CASES:
        for src_cm in (0, 1):
            for blk_cm in (0, 1):
                for gap in (0, 5):
                    src = g.integers(0, 255, size=max(1, m * n)).astype(dt)
                    rs, cs = (1, m) if src_cm else (n, 1)
                    m1, n1 = -(-m // m0), -(-n // n0)
                    rs0, cs0 = (1, m0) if blk_cm else (n0, 1)
                    cs1 = m0 * n0 + gap
                    rs1 = max(n1, 1) * cs1 + gap
                    size = max(1, m1 * rs1 + 8)
                    want = np.full(size, 0x11, dtype=dt)
                    orc.port().orc_pack(e // 8, m, n, P(src), rs, cs, m0, n0, P(want), rs0, cs0, rs1, cs1, 0xFF)
                    if where == "host":
                        got = np.full(size, 0x11, dtype=dt)
                        fn(m, n, S.ptr(src), rs, cs, m0, n0, S.ptr(got), rs0, cs0, rs1, cs1, 0xFF)
                        S.check()
                    else:
                        ds, dd = DeviceBuf(src), DeviceBuf(np.full(size, 0x11, dtype=dt))
                        fn(m, n, ds.ptr(0), rs, cs, m0, n0, dd.ptr(0), rs0, cs0, rs1, cs1, 0xFF)
                        S.check()
                        got = dd.back()
                    assert np.array_equal(got, want), (m, n, m0, n0, src_cm, blk_cm, gap)
                    if e == 8 and m:
                        back_want = np.full(m * n + 4, 0x22, dtype=dt)
                        orc.port().orc_unpack(1, m0, n0, P(want), rs0, cs0, rs1, cs1, m, n, P(back_want), rs, cs)
                        back = np.full(m * n + 4, 0x22, dtype=dt)
                        skl.skl_unpack_e8rcprc_e8rc_sm100a(m0, n0, S.ptr(want), rs0, cs0, rs1, cs1, m, n, S.ptr(back), rs, cs)
                        S.check()
                        assert np.array_equal(back, back_want)
                        assert np.array_equal(back[:m * n], src[:m * n])


@pytest.mark.parametrize("e", [8, 16, 32])
def test_transpose(skl, e):
    dt = {8: np.uint8, 16: np.uint16, 32: np.uint32}[e]
    g = H.rng(300 + e)
    fn = getattr(skl, f"skl_transpose_e{e}_sm100a")
    for (m, n) in [(0, 0), (1, 1), (63, 65), (64, 64), (65, 63), (127, 129), (257, 255), (1, 300), (300, 1), (1000, 513),
                   (256, 320), (130, 200), (16, 1024)]:
        for pad_a, pad_t in ((0, 0), (3, 5), ((-n) % 16, (-m) % 16)):  # the last keeps both pitches 16-byte multiples
            rsa, rsat = n + pad_a, m + pad_t
            a = g.integers(0, 255, size=max(1, m * rsa)).astype(dt)
            want = np.full(max(1, n * rsat), 0x33, dtype=dt)
            orc.port().orc_transpose(e // 8, m, n, P(a), rsa, P(want), rsat)
            got = np.full(max(1, n * rsat), 0x33, dtype=dt)
            fn(m, n, S.ptr(a), rsa, S.ptr(got), rsat)
            S.check()
            assert np.array_equal(got, want)
            da, dt_ = DeviceBuf(a), DeviceBuf(np.full(max(1, n * rsat), 0x33, dtype=dt))
            fn(m, n, da.ptr(0), rsa, dt_.ptr(0), rsat)
            S.check()
            assert np.array_equal(dt_.back(), want)
