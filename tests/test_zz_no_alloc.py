"""The allocation-free bf16 x fp8 GEMM entry point against the regular one.

Some callers of this library cannot let it call cudaMalloc: a serving loop with a latency budget
(cudaMalloc and cudaFree stall the whole device), or a process in which another allocator's pool
already owns the free device memory, so that an allocation made by the library would fail.
skl_gemm_bf16_f8e4m3_bf16_noalloc_sm100a serves them from a fixed 32 MiB array inside the library.
The checks here: two calls in a row (a large problem, then a smaller one that reuses the front of the
same array while the rest still holds the first call's data) must each reproduce the regular entry
point's bf16 output bit for bit -- both run the same two kernels on the same data, so no tolerance is
needed -- and a problem whose widened B exceeds the array must be refused with a message, leaving C
untouched.  The file sorts last so a run that stops at the first failure has already run everything else.
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
