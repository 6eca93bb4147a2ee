"""Shared test machinery: seeded inputs, comparison rules, guard bands.

Inputs come from numpy's counter-based Philox generator so a (seed, shape) pair names the same
matrix everywhere.  The comparison rules are the reference test suite's own:
  * int8 GEMM, cvt, pack: exact equality (test/gemm/gemm_i8rcprc_i8rcprc_i32rcprc.c:126-141,
    test/cvt/cvt_f32_f8.c:65-72, test/pack/pack_e8rc_e8rcprc.c:79-87);
  * float GEMM: |c - ref| <= 2*((1+u)^(K+2) - 1) * (|alpha| |A||B| + |beta| |C|), u = 2^-24
    (test/gemm/gemm_bf16rcprc_bf16rcprc_f32rcprc.c:130-191);
  * no byte outside the addressed elements of an output buffer may change
    (test/gemm/skl_test_gemm.h:58-169).
"""
from __future__ import annotations

import numpy as np

from oracle import pyoracle as orc

I8, BF16, F16, F8E4M3, F8E5M2, F32, I32 = range(7)
NP_STORE = {I8: np.int8, BF16: np.uint16, F16: np.uint16, F8E4M3: np.uint8, F8E5M2: np.uint8,
            F32: np.float32, I32: np.int32}


def rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(seed))


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    nan = (u >> 16) | 0x40
    return np.where((u & 0x7FFFFFFF) > 0x7F800000, nan, r).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def f16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(b, dtype=np.uint16).view(np.float16).astype(np.float32)


_DEC = {}


def f8_table(fmt: int) -> np.ndarray:
    """fp32 value of each of the 256 codes, from the oracle's decoder."""
    if fmt not in _DEC:
        lib = orc.port()
        fn = lib.orc_f8e4m3_to_f32 if fmt == F8E4M3 else lib.orc_f8e5m2_to_f32
        _DEC[fmt] = np.array([fn(c) for c in range(256)], dtype=np.float32)
    return _DEC[fmt]


def to_f32(t: int, a: np.ndarray) -> np.ndarray:
    if t == I8 or t == I32:
        return a.astype(np.float32)
    if t == BF16:
        return bf16_bits_to_f32(a)
    if t == F16:
        return f16_bits_to_f32(a)
    if t in (F8E4M3, F8E5M2):
        return f8_table(t)[a]
    return a.astype(np.float32)


def random_operand(t: int, shape, g: np.random.Generator, all_codes: bool = False) -> np.ndarray:
    """Values in the ranges the reference's harnesses use (test/gemm/*.h defaults); with all_codes the
    fp8 operands also take negative, subnormal and zero codes (never NaN/Inf)."""
    if t == I8:
        return g.integers(-128, 128, size=shape, dtype=np.int8)
    if t == BF16:
        return f32_to_bf16_bits(g.uniform(-1, 1, size=shape).astype(np.float32))
    if t == F16:
        return f32_to_f16_bits(g.uniform(-1, 1, size=shape).astype(np.float32))
    if t == F8E4M3:
        if all_codes:
            c = g.integers(0, 256, size=shape, dtype=np.uint16).astype(np.uint8)
            c[(c & 0x7F) == 0x7F] = 0x3A
            return c
        return g.integers(8, 127, size=shape, dtype=np.uint16).astype(np.uint8)
    if t == F8E5M2:
        if all_codes:
            c = g.integers(0, 256, size=shape, dtype=np.uint16).astype(np.uint8)
            c[(c & 0x7F) >= 0x7C] = 0x3A
            return c
        return g.integers(4, 124, size=shape, dtype=np.uint16).astype(np.uint8)
    if t == F32:
        return g.uniform(-1, 1, size=shape).astype(np.float32)
    if t == I32:
        return g.integers(-1000, 1000, size=shape, dtype=np.int32)
    raise ValueError(t)


class Strided:
    """A matrix laid out in a flat buffer with element strides and a canary-filled margin.

    ``buf`` is the whole allocation (guard bands included), ``off`` the offset of element (0, 0).
    """

    def __init__(self, t: int, rows: int, cols: int, rs: int, cs: int, g: np.random.Generator | None,
                 guard: int = 64, fill=None, all_codes=False):
        self.t, self.rows, self.cols, self.rs, self.cs = t, rows, cols, rs, cs
        span = (rows - 1) * rs + (cols - 1) * cs + 1 if rows and cols else 0
        self.off = guard
        self.span = span
        dt = NP_STORE[t]
        self.buf = np.empty(span + 2 * guard + 8, dtype=dt)
        canary = random_operand(t, self.buf.shape, rng(987654321))
        self.buf[:] = canary
        if rows and cols and g is not None:
            vals = random_operand(t, (rows, cols), g, all_codes) if fill is None else fill
            self.set(vals)

    def idx(self) -> np.ndarray:
        i = np.arange(self.rows)[:, None] * self.rs
        j = np.arange(self.cols)[None, :] * self.cs
        return self.off + i + j

    def set(self, vals: np.ndarray) -> None:
        self.buf[self.idx()] = vals

    def get(self) -> np.ndarray:
        return self.buf[self.idx()]

    @property
    def view(self) -> np.ndarray:
        """Array whose element 0 is matrix element (0, 0) (what the C call receives)."""
        return self.buf[self.off:]

    def copy(self) -> "Strided":
        o = Strided.__new__(Strided)
        o.__dict__.update(self.__dict__)
        o.buf = self.buf.copy()
        return o


def assert_untouched_outside(before: Strided, after_buf: np.ndarray, what: str = "output") -> None:
    """Every element of the allocation that the (shape, strides) do not address must be unchanged."""
    mask = np.ones(before.buf.shape, dtype=bool)
    if before.rows and before.cols:
        mask[before.idx().ravel()] = False
    a = before.buf.view(np.uint8).reshape(before.buf.shape[0], -1)
    b = after_buf.view(np.uint8).reshape(after_buf.shape[0], -1)
    bad = np.nonzero(mask & (a != b).any(axis=1))[0]
    assert bad.size == 0, f"{what}: {bad.size} unaddressed elements changed, first at flat index {bad[:5]}"


def skl_forward_bound(ta, a, tb, b, alpha, beta, c_old, k) -> np.ndarray:
    """The reference suite's forward error bound per element, evaluated in float64."""
    u = 2.0 ** -24
    gamma = 2.0 * ((1.0 + u) ** (k + 2) - 1.0)
    absab = np.abs(to_f32(ta, a).astype(np.float64)) @ np.abs(to_f32(tb, b).astype(np.float64))
    tail = abs(beta) * np.abs(c_old.astype(np.float64)) if c_old is not None else 0.0
    return gamma * (abs(alpha) * absab + tail)


def bf16_ulp(x: np.ndarray) -> np.ndarray:
    """Spacing of bf16 numbers at |x| (x given as fp32)."""
    ax = np.abs(x.astype(np.float32))
    e = np.floor(np.log2(np.maximum(ax, 2.0 ** -126)))
    return np.exp2(e - 7).astype(np.float64)
