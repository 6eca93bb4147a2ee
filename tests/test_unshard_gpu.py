"""skl_b200_unshard_columns_sm100a: the local re-layout that follows an all-gather of C's column shards.

The gathered buffer holds the shards one after the other ([G][M][N/G] for equal shards, what an all-gather of the ranks'
row-major shards produces); the routine must write the row-major M x N matrix.  Equal shards take one unpack launch
(the buffer is an SKL packed matrix with m0 = M, n0 = N/G in block-column order), unequal shards one strided copy per
shard; host and device pointers; bytes of dst beyond the N columns stay untouched."""
import numpy as np
import pytest

import helpers as H
import skl_b200 as S
from gpu_common import DeviceBuf

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("esize,dt", [(1, np.uint8), (2, np.uint16), (4, np.uint32)])
@pytest.mark.parametrize("where", ["device", "host"])
def test_unshard_equals_concatenation(skl, esize, dt, where):
    g = H.rng(esize)
    for (m, n, parts, align) in [(64, 1024, 4, 256), (33, 512, 2, 256), (40, 1000, 3, 16), (7, 14336, 8, 256), (5, 10, 4, 1)]:
        shards, full = [], np.zeros((m, n), dt)
        stride = 0
        for idx in range(parts):
            s, c = S.shard_columns(n, parts, idx, align)
            blk = g.integers(0, 250, size=(m, c)).astype(dt)
            full[:, s:s + c] = blk
            shards.append(blk)
            stride = max(stride, m * c)
        stride += 8  # shards need not be packed back to back
        gathered = np.full(parts * stride, 0xEE, dt)
        for idx, blk in enumerate(shards):
            gathered[idx * stride:idx * stride + blk.size] = blk.ravel()
        rsd = n + 6
        dst = np.full((m, rsd), 0x11, dt)
        if where == "host":
            skl.skl_b200_unshard_columns_sm100a(esize, m, n, parts, align, S.ptr(gathered), stride, S.ptr(dst), rsd)
            S.check()
            got = dst
        else:
            dg, dd = DeviceBuf(gathered), DeviceBuf(dst)
            skl.skl_b200_unshard_columns_sm100a(esize, m, n, parts, align, dg.ptr(0), stride, dd.ptr(0), rsd)
            S.check()
            got = dd.back()
        assert np.array_equal(got[:, :n], full)
        assert np.all(got[:, n:] == 0x11), "columns outside the matrix were written"


def test_bad_arguments_are_refused(skl):
    d = np.zeros(16, np.uint8)
    skl.skl_b200_unshard_columns_sm100a(3, 2, 4, 2, 1, S.ptr(d), 4, S.ptr(d), 4)
    assert skl.skl_b200_last_status() == 1
    skl.skl_b200_unshard_columns_sm100a(1, 2, 4, 2, 1, S.ptr(d), 4, S.ptr(d), 3)  # row stride shorter than a row
    assert skl.skl_b200_last_status() == 1
