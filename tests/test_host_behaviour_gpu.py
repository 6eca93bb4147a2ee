"""Host-layer behaviour on a GPU box: argument errors are reported and leave memory alone, per-thread
contexts let several host threads call at once, and the asynchronous mode on a caller's stream orders
the library's kernels with the caller's own work."""
import threading

import numpy as np
import pytest

import helpers as H
import skl_b200 as S
from gpu_common import DeviceBuf

pytestmark = pytest.mark.gpu


def test_null_operands_are_rejected_and_c_is_untouched(skl):
    a = np.ones((8, 8), np.int8)
    c = np.full((8, 8), 7, np.int32)
    skl.skl_gemm_i8_i8_i32_sm100a(8, 8, 8, 1, None, 8, S.ptr(a), 8, 0, S.ptr(c), 8)
    assert skl.skl_b200_last_status() == 1
    with pytest.raises(S.SklB200Error):
        S.check()
    skl.skl_gemm_i8_i8_i32_sm100a(8, 8, 8, 1, S.ptr(a), 8, S.ptr(a), 8, 0, None, 8)
    assert skl.skl_b200_last_status() == 1
    assert np.all(c == 7)
    # k = 0 needs neither A nor B: C = beta * C
    skl.skl_gemm_i8_i8_i32_sm100a(8, 8, 0, 1, None, 8, None, 8, 3, S.ptr(c), 8)
    S.check()
    assert np.all(c == 21)
    # the status is per call: a good call after a bad one reads ok
    assert skl.skl_b200_last_status() == 0


def test_null_in_cvt_and_pack_is_rejected(skl):
    x = np.zeros(16, np.float32)
    skl.skl_cvt_f32_f8e4m3_sm100a(None, S.ptr(x), 1.0, 16)
    assert skl.skl_b200_last_status() == 1
    skl.skl_transpose_e8_sm100a(4, 4, None, 4, S.ptr(x), 4)
    assert skl.skl_b200_last_status() == 1
    skl.skl_pack_e8rc_e8rcprc_sm100a(4, 4, S.ptr(x), 4, 1, 2, 2, None, 2, 1, 8, 4, 0)
    assert skl.skl_b200_last_status() == 1
    # n = 0 is a no-op, not an error, even with null pointers
    skl.skl_cvt_f32_f8e4m3_sm100a(None, None, 1.0, 0)
    assert skl.skl_b200_last_status() == 0


def test_host_threads_have_their_own_context(skl):
    """Four host threads, each with its own shapes, call the int8 GEMM at the same time; every result is
    bit-exact and every thread reads its own status word."""
    errors = []

    def work(seed):
        try:
            g = H.rng(seed)
            for it in range(6):
                m, n, k = 128 + 16 * seed, 256 + 16 * it, 128 * (1 + (seed + it) % 3)
                a = g.integers(-128, 128, size=(m, k), dtype=np.int8)
                b = g.integers(-128, 128, size=(k, n), dtype=np.int8)
                c = np.zeros((m, n), np.int32)
                want = a.astype(np.int32) @ b.astype(np.int32)
                skl.skl_gemm_i8_i8_i32_sm100a(m, n, k, 1, S.ptr(a), k, S.ptr(b), n, 0, S.ptr(c), n)
                S.check()
                if not np.array_equal(c, want):
                    errors.append((seed, it, "mismatch"))
            # a bad call in this thread must not show in the others
            if seed == 0:
                skl.skl_gemm_i8_i8_i32_sm100a(8, 8, 8, 1, None, 8, None, 8, 0, None, 8)
                if skl.skl_b200_last_status() != 1:
                    errors.append((seed, "status"))
            else:
                if skl.skl_b200_last_status() != 0:
                    errors.append((seed, "foreign status", skl.skl_b200_last_status()))
            skl.skl_b200_release_workspace()
        except Exception as e:  # noqa: BLE001
            errors.append((seed, repr(e)))

    ts = [threading.Thread(target=work, args=(s,)) for s in range(4)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert not errors, errors


def test_thread_exit_releases_the_threads_workspaces(skl):
    """A thread that used the library with host operands owns device workspaces; when it ends without calling
    skl_b200_release_workspace() the library's thread-exit hook frees them: free device memory after the threads have
    gone is back where it was (short-lived worker threads must not leak device memory)."""
    import torch

    torch.cuda.synchronize()
    m, n, k = 2048, 2048, 2048  # 4 MiB A + 4 MiB B + 16 MiB C staged per thread
    a = np.ones((m, k), np.int8)
    b = np.ones((k, n), np.int8)
    errors = []

    def work():
        c = np.zeros((m, n), np.int32)
        skl.skl_gemm_i8_i8_i32_sm100a(m, n, k, 1, S.ptr(a), k, S.ptr(b), n, 0, S.ptr(c), n)
        if skl.skl_b200_last_status() != 0 or c[5, 7] != k:
            errors.append("bad result")

    # one throw-away thread first so that one-time costs (module load, streams) are not counted
    t = threading.Thread(target=work)
    t.start()
    t.join()
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        ts = [threading.Thread(target=work) for _ in range(4)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
    torch.cuda.synchronize()
    assert not errors, errors
    # join() returns when the thread's Python code has finished; the exit hook runs a moment later, as the OS thread
    # goes away: give it up to two seconds
    import time
    for _ in range(40):
        free1, _ = torch.cuda.mem_get_info()
        if free0 - free1 < (32 << 20):
            break
        time.sleep(0.05)
    # 12 threads x 24 MiB would be 288 MiB if nothing were released
    assert free0 - free1 < (32 << 20), f"device memory not returned: {(free0 - free1) >> 20} MiB still held"


def test_async_mode_on_a_caller_stream(skl):
    """With device operands, async mode and a caller's stream, the call only enqueues: work the caller puts
    on the same stream before and after it is ordered with the library's kernels."""
    import torch

    m, n, k = 256, 512, 256
    g = H.rng(77)
    a = g.integers(-128, 128, size=(m, k), dtype=np.int8)
    b = g.integers(-128, 128, size=(k, n), dtype=np.int8)
    want = a.astype(np.int32) @ b.astype(np.int32)
    stream = torch.cuda.Stream()
    skl.skl_b200_set_stream(stream.cuda_stream)
    skl.skl_b200_set_async(1)
    try:
        with torch.cuda.stream(stream):
            da = torch.empty((m, k), dtype=torch.int8, device="cuda")
            db = torch.from_numpy(b).cuda()
            dc = torch.full((m, n), 5, dtype=torch.int32, device="cuda")
            pinned = torch.from_numpy(a).pin_memory()
            da.copy_(pinned, non_blocking=True)  # producer on the same stream
            skl.skl_gemm_i8_i8_i32_sm100a(m, n, k, 1, da.data_ptr(), k, db.data_ptr(), n, 1, dc.data_ptr(), n)
            doubled = dc * 2  # consumer on the same stream
        skl.skl_b200_synchronize()
        S.check()
        assert np.array_equal(doubled.cpu().numpy(), 2 * (want + 5))
    finally:
        skl.skl_b200_set_async(0)
        skl.skl_b200_set_stream(None)
        torch.cuda.synchronize()


def test_profile_hook_reports_device_time(skl):
    """skl_b200_profile_begin / _end bracket calls with CUDA events on the library's stream."""
    m = n = k = 1024
    a = DeviceBuf(np.ones((m, k), np.int8))
    b = DeviceBuf(np.ones((k, n), np.int8))
    c = DeviceBuf(np.zeros((m, n), np.int32))
    skl.skl_gemm_i8_i8_i32_sm100a(m, n, k, 1, a.ptr(0), k, b.ptr(0), n, 0, c.ptr(0), n)  # warm
    S.check()
    import ctypes

    skl.skl_b200_profile_begin(4)
    for _ in range(6):  # only the first four are bracketed
        skl.skl_gemm_i8_i8_i32_sm100a(m, n, k, 1, a.ptr(0), k, b.ptr(0), n, 0, c.ptr(0), n)
    ms = ctypes.c_double(0.0)
    assert skl.skl_b200_profile_end(ctypes.byref(ms)) == 4
    S.check()
    assert 0.0 < ms.value < 50.0
    assert skl.skl_b200_last_launch_count() >= 1
    assert np.all(c.back() == k)
