"""The give-up path of the kernels' bounded waits.

Every wait inside the tensor-core kernels is bounded; when one runs out the kernel records a stage code, all its warps
leave through the normal exit (tensor memory released), and the call reports SKL_B200_ERR_DEVICE_TIMEOUT with the
context still usable.  Nothing here faults, traps or spins without limit: the testing aid
skl_b200_debug_skip_loads(1) makes the producer warp announce its loads without issuing them, so the consumers
wait for bytes that never come, for a wait limit shortened to a few milliseconds.  Each case is followed by a normal
call that must succeed and be exact."""
import time

import numpy as np
import pytest

import helpers as H
import skl_b200 as S
from gpu_common import check_gemm_rc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("pair", ["0", "2"])
def test_expired_wait_is_reported_and_the_context_survives(skl, pair, monkeypatch):
    import torch

    monkeypatch.setenv("SKL_B200_TC_PAIR", pair)  # 0: one CTA per tile; 2: the two-CTA kernel
    m, n, k = 512, 512, 512
    a = torch.randint(-128, 128, (m, k), dtype=torch.int8, device="cuda")
    b = torch.randint(-128, 128, (k, n), dtype=torch.int8, device="cuda")
    c = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    skl.skl_b200_set_wait_limit(5)
    skl.skl_b200_debug_skip_loads(1)
    try:
        t0 = time.perf_counter()
        skl.skl_gemm_i8_i8_i32_sm100a(m, n, k, 1, a.data_ptr(), k, b.data_ptr(), n, 0, c.data_ptr(), n)
        dt = time.perf_counter() - t0
        assert skl.skl_b200_last_path() == S.PATH_TCGEN05
        assert skl.skl_b200_last_status() == 4, "expected SKL_B200_ERR_DEVICE_TIMEOUT"
        assert b"stage code" in skl.skl_b200_last_cuda_error()
        assert dt < 1.0, "the give-up path must not take longer than a few wait limits"
    finally:
        skl.skl_b200_debug_skip_loads(0)
        skl.skl_b200_set_wait_limit(0)
    torch.cuda.synchronize()  # the context is intact: no sticky error
    skl.skl_gemm_i8_i8_i32_sm100a(m, n, k, 1, a.data_ptr(), k, b.data_ptr(), n, 0, c.data_ptr(), n)
    S.check()
    want = a.cpu().numpy().astype(np.int32) @ b.cpu().numpy().astype(np.int32)
    assert np.array_equal(c.cpu().numpy(), want)
    check_gemm_rc(skl, H.BF16, 300, 260, 192, "rkr", 1, 0, where="device", path=S.PATH_TCGEN05, align=16,
                  expect_path=S.PATH_TCGEN05, seed=3, all_codes=False)
