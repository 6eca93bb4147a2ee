"""The allocation-free bf16 x fp8 GEMM entry point against the regular one.

Some callers of this library cannot let it call cudaMalloc: a serving loop with a latency budget
(cudaMalloc and cudaFree stall the whole device), or a process in which another allocator's pool
already owns the free device memory, so that an allocation made by the library would fail.
skl_gemm_bf16_f8e4m3_bf16_noalloc_sm100a serves them from a fixed 32 MiB array inside the library.
The checks here: two calls in a row (a large problem, then a smaller one that reuses the front of the
same array while the rest still holds the first call's data) must each reproduce the regular entry
point's bf16 output bit for bit -- both run the same two kernels on the same data, so no tolerance is
needed -- and a problem whose widened B exceeds the array must be refused with a message, leaving C
untouched.  Further checks: sampled rows against the CPU oracle; an n-contiguous B with at least 512 rows of A
(both entry points then write the widened copy k-contiguous); free device memory does not move across a call on a
shape larger than any before (the defining property), while the regular entry point does allocate for it; k == 0,
a B without unit stride and an A layout the tensor-core kernel declines are refused with their codes.
The file sorts last so a run that stops at the first failure has already run everything else.
"""
import ctypes

import numpy as np
import pytest

import helpers as H
import skl_b200 as S

pytestmark = pytest.mark.gpu


def _device_problem(m, n, k, b_kmajor, seed):
    import torch

    g = H.rng(seed)
    a = torch.from_numpy(H.random_operand(H.BF16, (m, k), g).view(np.int16)).cuda()
    bshape = (n, k) if b_kmajor else (k, n)
    b = torch.from_numpy(H.random_operand(H.F8E4M3, bshape, g, all_codes=True)).cuda()
    cs = torch.from_numpy(g.uniform(0.5, 1.5, n).astype(np.float32)).cuda()
    return a, b, cs


def _run_both(skl, m, n, k, b_kmajor, seed):
    import torch

    a, b, cs = _device_problem(m, n, k, b_kmajor, seed)
    rsb, csb = (1, k) if b_kmajor else (n, 1)
    want = torch.full((m, n), 0x7FC0, dtype=torch.int16, device="cuda")
    got = torch.full((m, n), 0x7FC0, dtype=torch.int16, device="cuda")
    skl.skl_gemm_ex_sm100a(m, n, k, S.BF16, a.data_ptr(), k, 1, S.F8E4M3, b.data_ptr(), rsb, csb, 0.75, None,
                           cs.data_ptr(), 0.0, S.BF16, want.data_ptr(), n, 1)
    S.check()
    assert skl.skl_b200_last_path() == S.PATH_TCGEN05
    msg = ctypes.create_string_buffer(200)
    rc = skl.skl_gemm_bf16_f8e4m3_bf16_noalloc_sm100a(m, n, k, 0.75, a.data_ptr(), k, 1, b.data_ptr(), rsb, csb,
                                                      cs.data_ptr(), got.data_ptr(), n, 1, None, msg, len(msg))
    assert rc == 0, msg.value.decode()
    torch.cuda.synchronize()
    assert torch.equal(got, want), "allocation-free entry point differs from the regular one"


def test_two_calls_in_a_row_match_the_regular_entry_point(skl):
    _run_both(skl, 384, 1024, 2048, False, 1)  # fills 4 MiB of the fixed array
    _run_both(skl, 130, 264, 320, True, 2)     # smaller, other orientation, stale data behind it


def test_sampled_rows_against_the_oracle_and_the_reoriented_copy(skl):
    """m >= 512 with an n-contiguous B: the widened copy is written k-contiguous by both entry points; the output
    equals the regular entry point's and, on sampled rows, lies within the reference suite's bound of the oracle."""
    import torch
    from oracle import pyoracle as orc

    m, n, k = 640, 520, 264
    _run_both(skl, m, n, k, False, 3)
    a, b, cs = _device_problem(m, n, k, False, 3)
    got = torch.zeros((m, n), dtype=torch.int16, device="cuda")
    msg = ctypes.create_string_buffer(200)
    rc = skl.skl_gemm_bf16_f8e4m3_bf16_noalloc_sm100a(m, n, k, 0.75, a.data_ptr(), k, 1, b.data_ptr(), n, 1, cs.data_ptr(),
                                                      got.data_ptr(), n, 1, None, msg, len(msg))
    assert rc == 0, msg.value.decode()
    rows = [0, 1, 127, 128, 511, 512, m - 1]
    ah = a.cpu().numpy().view(np.uint16)[rows]
    bh, csh = b.cpu().numpy(), cs.cpu().numpy()
    want = np.zeros((len(rows), n), np.uint16)
    orc.port_gemm_ex(len(rows), n, k, H.BF16, ah, k, 1, H.F8E4M3, bh, n, 1, 0.75, None, csh, 0.0, H.BF16, want, n, 1)
    out = H.to_f32(H.BF16, got.cpu().numpy().view(np.uint16)[rows]).astype(np.float64)
    ref = H.to_f32(H.BF16, want).astype(np.float64)
    bound = H.skl_forward_bound(H.BF16, ah, H.F8E4M3, bh, 1.0, 0.0, None, k) * np.abs(0.75 * csh[None, :].astype(np.float64)) * 2
    assert np.all(np.abs(out - ref) <= bound + 2.0 ** -7 * np.abs(ref) + 1e-30)


def test_no_device_memory_is_allocated(skl):
    """Free device memory is the same before and after a call on a shape larger than any this process used with the
    entry point before (so nothing was cached for it); the regular entry point, given the same new shape, does take
    memory for its widened copy -- which shows the measurement can see an allocation."""
    import torch

    _run_both(skl, 130, 264, 320, True, 2)  # warm-up: module load, function attributes
    m, n, k = 256, 2048, 3968  # widened B: 15.5 MiB, more than any call above
    a, b, cs = _device_problem(m, n, k, True, 5)
    c = torch.zeros((m, n), dtype=torch.int16, device="cuda")
    msg = ctypes.create_string_buffer(200)
    skl.skl_b200_release_workspace()  # the regular path's cached workspaces go, so that it must allocate again below
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    rc = skl.skl_gemm_bf16_f8e4m3_bf16_noalloc_sm100a(m, n, k, 1.0, a.data_ptr(), k, 1, b.data_ptr(), 1, k, cs.data_ptr(),
                                                      c.data_ptr(), n, 1, None, msg, len(msg))
    assert rc == 0, msg.value.decode()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"the allocation-free entry point changed free device memory by {free0 - free1} bytes"
    skl.skl_gemm_ex_sm100a(m, n, k, S.BF16, a.data_ptr(), k, 1, S.F8E4M3, b.data_ptr(), 1, k, 1.0, None, cs.data_ptr(), 0.0,
                           S.BF16, c.data_ptr(), n, 1)
    S.check()
    free2, _ = torch.cuda.mem_get_info()
    assert free2 < free1, "the regular entry point was expected to allocate its widened copy"
    skl.skl_b200_release_workspace()


def test_refusals_carry_their_codes(skl):
    import torch

    a = torch.zeros((64, 64), dtype=torch.int16, device="cuda")
    b = torch.zeros((64, 64), dtype=torch.uint8, device="cuda")
    c = torch.full((64, 64), 7, dtype=torch.int16, device="cuda")
    msg = ctypes.create_string_buffer(200)

    def call(m, n, k, rsa, csa, rsb, csb):
        return skl.skl_gemm_bf16_f8e4m3_bf16_noalloc_sm100a(m, n, k, 1.0, a.data_ptr(), rsa, csa, b.data_ptr(), rsb, csb,
                                                            None, c.data_ptr(), 64, 1, None, msg, len(msg))

    assert call(8, 8, 0, 64, 1, 64, 1) == 1 and b"k == 0" in msg.value
    assert call(8, 8, 8, 64, 1, 2, 3) == 1 and b"unit stride" in msg.value          # B strided both ways
    assert call(8, 8, 8, 2, 3, 64, 1) == 5                                            # A without a unit stride
    assert call(8, 8, 8, 12, 1, 64, 1) == 5                                           # A rows not 16-byte aligned
    assert bool((c == 7).all())
    # a tiny problem is served (by the tensor-core kernel, unlike the regular entry point's any-stride kernel)
    assert call(2, 16, 8, 64, 1, 64, 1) == 0


def test_oversized_problem_is_refused_with_a_message(skl):
    import torch

    k, n = 4096, 4104  # k*n bf16 elements > 32 MiB
    a = torch.zeros((8, k), dtype=torch.int16, device="cuda")
    b = torch.zeros((k, n), dtype=torch.uint8, device="cuda")
    c = torch.full((8, n), 123, dtype=torch.int16, device="cuda")
    msg = ctypes.create_string_buffer(200)
    rc = skl.skl_gemm_bf16_f8e4m3_bf16_noalloc_sm100a(8, n, k, 1.0, a.data_ptr(), k, 1, b.data_ptr(), n, 1, None,
                                                      c.data_ptr(), n, 1, None, msg, len(msg))
    assert rc == 1
    text = msg.value.decode()
    assert "33554432" in text and str(k * n * 2) in text
    assert bool((c == 123).all())
    host = np.zeros((8, 16), np.uint16)
    rc = skl.skl_gemm_bf16_f8e4m3_bf16_noalloc_sm100a(8, 16, 16, 1.0, S.ptr(host), 16, 1, b.data_ptr(), 16, 1, None,
                                                      c.data_ptr(), 16, 1, None, msg, len(msg))
    assert rc == 1 and "device memory" in msg.value.decode()
