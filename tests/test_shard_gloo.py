"""World-size-2 run of the column-sharded GEMM's host logic on CPU (gloo).

Each rank takes the column range skl_b200_shard_columns gives it, computes its slice of C from the
replicated A and its slice of B and of the per-column scale vector -- B addressed the way the GPU run
addresses it, `b + start` with the full matrix's row stride -- and the slices, gathered, must equal the
unsharded result bit for bit.  The arithmetic runs in the oracle here; on the GPU box the same
addressing feeds skl_gemm_ex_sm100a (bench.py --gpus N)."""
import os
import socket

import numpy as np
import pytest


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist

    import helpers as H
    import skl_b200 as S
    from oracle import pyoracle as orc

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, k, n = 24, 40, 100
        g = H.rng(5)  # same seed on every rank: replicated inputs
        a = H.random_operand(H.BF16, (m, k), g)
        b = H.random_operand(H.F8E4M3, (k, n), g, all_codes=True)
        cs = g.uniform(0.5, 1.5, n).astype(np.float32)
        start, count = S.shard_columns(n, world, rank, 16)
        mine = np.zeros((m, count), np.uint16)
        orc.port_gemm_ex(m, count, k, H.BF16, a, k, 1, H.F8E4M3, b.reshape(-1)[start:], n, 1, 1.0, None, cs[start:], 0.0,
                         H.BF16, mine, count, 1)
        sizes = [S.shard_columns(n, world, r, 16)[1] for r in range(world)]
        parts = [torch.zeros((m, c), dtype=torch.int32) for c in sizes]
        # gloo wants equal shapes: pad to the widest slice
        wmax = max(sizes)
        padded = torch.zeros((m, wmax), dtype=torch.int32)
        padded[:, :count] = torch.from_numpy(mine.astype(np.int32))
        bufs = [torch.zeros((m, wmax), dtype=torch.int32) for _ in range(world)]
        dist.all_gather(bufs, padded)
        full = np.concatenate([bufs[r][:, :sizes[r]].numpy() for r in range(world)], axis=1).astype(np.uint16)
        if rank == 0:
            want = np.zeros((m, n), np.uint16)
            orc.port_gemm_ex(m, n, k, H.BF16, a, k, 1, H.F8E4M3, b, n, 1, 1.0, None, cs, 0.0, H.BF16, want, n, 1)
            q.put(bool(np.array_equal(full, want)) and sum(sizes) == n)
        del parts
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_column_shards_stitch_to_the_unsharded_result():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(100)
        assert p.exitcode == 0
    assert q.get(timeout=5) is True


def _gather_worker(rank, world, port, q):
    """The optional final all-gather of C: equal column shards, gathered into [G][M][N/G] by the collective, then the
    re-layout skl_b200_unshard_columns_sm100a performs -- one `unpack` of an SKL packed matrix with m0 = M,
    n0 = N/G in block-column order -- done here by the oracle's unpack with the library's arguments."""
    import torch
    import torch.distributed as dist

    import helpers as H
    import skl_b200 as S
    from oracle import pyoracle as orc

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, k, n = 24, 40, 128
        g = H.rng(6)
        a = H.random_operand(H.BF16, (m, k), g)
        b = H.random_operand(H.F8E4M3, (k, n), g, all_codes=True)
        cs = g.uniform(0.5, 1.5, n).astype(np.float32)
        start, count = S.shard_columns(n, world, rank, 16)
        assert count * world == n
        mine = np.zeros((m, count), np.uint16)
        orc.port_gemm_ex(m, count, k, H.BF16, a, k, 1, H.F8E4M3, b.reshape(-1)[start:], n, 1, 1.0, None, cs[start:], 0.0,
                         H.BF16, mine, count, 1)
        gathered = torch.zeros((world * m, count), dtype=torch.int32)  # = [G][M][N/G]; gloo has no 16-bit integers
        dist.all_gather_into_tensor(gathered, torch.from_numpy(mine.astype(np.int32)))
        gbuf = np.ascontiguousarray(gathered.numpy().astype(np.uint16)).reshape(-1)
        full = np.zeros((m, n), np.uint16)
        # the library's call: unpack(esize, m0 = m, n0 = count, src, rs0 = count, cs0 = 1, rs1 = 0, cs1 = part_stride, ...)
        orc.port().orc_unpack(2, m, count, orc._p(gbuf), count, 1, 0, m * count, m, n, orc._p(full), n, 1)
        want = np.zeros((m, n), np.uint16)
        orc.port_gemm_ex(m, n, k, H.BF16, a, k, 1, H.F8E4M3, b, n, 1, 1.0, None, cs, 0.0, H.BF16, want, n, 1)
        q.put((rank, bool(np.array_equal(full, want))))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_gathered_shards_unshard_to_the_unsharded_result_on_every_rank():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gather_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(100)
        assert p.exitcode == 0
    got = dict(q.get(timeout=5) for _ in range(2))
    assert got == {0: True, 1: True}
