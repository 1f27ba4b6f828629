"""The allocation-free GEMM entry point, checked against the regular one through the C ABI.

Some users of the library cannot allocate device memory when they call it (their process has handed the
whole GPU to its own arena, or locked its allocator after start-up).  spork_gemm_sm100_f16f32_static keeps all
of its scratch - status word and split-K workspace - in a fixed array inside the library image.  This file
is collected last so that a failure here cannot hide the result of any other test; it passes on its own in a
fresh process as well as after the others.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1.0  # the normalised-error bound used by the other GEMM tests


def _operands(sp, cuda, M, N, K):
    import torch

    a = torch.empty((M, K), dtype=torch.float16, device=cuda)
    b = torch.empty((N, K), dtype=torch.float16, device=cuda)
    sp.init_test_data(a, sp.DATA_UNIFORM_PM1, sp.SEED_A)
    sp.init_test_data(b, sp.DATA_UNIFORM_PM1, sp.SEED_B, transpose_rule=True)
    return a, b


def _static(sp, a, b, c, split_k):
    import torch

    M, K = a.shape
    N = b.shape[0]
    stream = torch.cuda.current_stream().cuda_stream
    rc = sp.lib().spork_gemm_sm100_f16f32_static(M, N, K, a.data_ptr(), b.data_ptr(), c.data_ptr(), split_k, stream)
    assert rc == 0, f"static entry point returned {rc}"


def _query(sp):
    import torch

    return sp.lib().spork_gemm_sm100_f16f32_static(0, 0, 0, None, None, None, 1, torch.cuda.current_stream().cuda_stream)


def test_static_entry_point_matches_regular_entry_point_twice_in_a_row(sp, orc, cuda):
    import torch

    # two calls back to back with different shapes and split counts: the second reuses the workspace
    # that still holds the first call's partial sums
    for (M, N, K, split_k) in ((1024, 512, 2048, 4), (640, 200, 1032, 3)):
        a, b = _operands(sp, cuda, M, N, K)
        want = torch.empty((M, N), dtype=torch.float32, device=cuda)
        sp.matmul_sm100(a, b, want)
        sp.status()
        got = torch.empty((M, N), dtype=torch.float32, device=cuda)
        got.view(torch.uint8).fill_(0x7D)
        _static(sp, a, b, got, split_k)
        assert _query(sp) == 0
        err = orc.normalised_error(got.cpu().numpy(), want.cpu().numpy(), 1.0, 1.0, K)
        assert err <= TOL
        assert err < 1e-3  # only the fp32 summation order differs
        # and against the CPU oracle directly
        ref = orc.gemm_f16f32(a.cpu().numpy(), b.cpu().numpy())
        assert orc.normalised_error(got.cpu().numpy(), ref, 1.0, 1.0, K) <= TOL


def test_static_entry_point_is_bit_reproducible_and_unsplit_equals_regular(sp, cuda):
    import torch

    M, N, K = 512, 384, 1024
    a, b = _operands(sp, cuda, M, N, K)
    runs = []
    for _ in range(2):
        c = torch.empty((M, N), dtype=torch.float32, device=cuda)
        _static(sp, a, b, c, 4)
        runs.append(c)
    assert _query(sp) == 0
    assert torch.equal(runs[0], runs[1])
    c1 = torch.empty((M, N), dtype=torch.float32, device=cuda)
    _static(sp, a, b, c1, 1)
    want = sp.matmul_sm100(a, b)
    sp.status()
    assert _query(sp) == 0
    assert torch.equal(c1, want)  # one K range: the very same sequence of MMAs


def test_static_entry_point_rejects_what_does_not_fit(sp, cuda):
    import torch

    L = sp.lib()
    a = torch.zeros((128, 64), dtype=torch.float16, device=cuda)
    c = torch.zeros((128, 128), dtype=torch.float32, device=cuda)
    s = torch.cuda.current_stream().cuda_stream
    # 8192 x 8192 fp32 is 256 MiB of partial sums per split: beyond the 64 MiB workspace
    assert L.spork_gemm_sm100_f16f32_static(8192, 8192, 64, a.data_ptr(), a.data_ptr(), c.data_ptr(), 1, s) == 10006
    # fits unsplit (16 MiB), not with five splits
    assert L.spork_gemm_sm100_f16f32_static(4096, 1024, 4096, a.data_ptr(), a.data_ptr(), c.data_ptr(), 5, s) == 10006
    assert L.spork_gemm_sm100_f16f32_static(128, 128, 12, a.data_ptr(), a.data_ptr(), c.data_ptr(), 1, s) == 10002
    assert L.spork_gemm_sm100_f16f32_static(128, 128, 64, a.data_ptr(), a.data_ptr(), c.data_ptr(), 0, s) == 10001
    assert _query(sp) == 0
