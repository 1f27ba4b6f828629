"""Failure detection on the device without faulting anything: a wait that cannot complete gives up after its
limit, the kernel reports through the status word and returns, and the same context keeps working."""
import ctypes
import time

import pytest

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_sets_the_status_word_and_the_context_survives(sp, orc, cuda):
    import torch

    L = sp.lib()
    sp.status()  # clean slate
    stream = torch.cuda.current_stream().cuda_stream
    t0 = time.perf_counter()
    assert L.spork_selftest_bounded_wait(20000, stream) == 0  # 20 ms limit; nothing ever arrives on the barrier
    detail = ctypes.c_uint32(0)
    rc = L.spork_gemm_sm100_status(stream, ctypes.byref(detail))
    elapsed = time.perf_counter() - t0
    assert rc == 10005  # SPORK_ERR_DEVICE_TIMEOUT
    assert detail.value >> 28 == 0xA
    assert 0.015 < elapsed < 2.0  # it waited for its limit, and no longer than that
    # the word was cleared by the read, and the device is healthy: a GEMM runs and is correct
    assert L.spork_gemm_sm100_status(stream, None) == 0
    with pytest.raises(sp.SporkError):
        assert L.spork_selftest_bounded_wait(1000, stream) == 0
        sp.status()
    M, N, K = 256, 256, 512
    a = torch.empty((M, K), dtype=torch.float16, device=cuda)
    b = torch.empty((N, K), dtype=torch.float16, device=cuda)
    sp.init_test_data(a, sp.DATA_UNIFORM_PM1, sp.SEED_A)
    sp.init_test_data(b, sp.DATA_UNIFORM_PM1, sp.SEED_B, transpose_rule=True)
    c = sp.matmul_sm100(a, b)
    sp.status()
    ref = orc.gemm_f16f32(a.cpu().numpy(), b.cpu().numpy())
    assert orc.normalised_error(c.cpu().numpy(), ref, 1.0, 1.0, K) <= 1.0


def test_selftest_rejects_unbounded_limits(sp, cuda):
    L = sp.lib()
    assert L.spork_selftest_bounded_wait(0, None) == 10001
    assert L.spork_selftest_bounded_wait(5000000, None) == 10001
