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


@pytest.mark.parametrize("M,N,K,split_k", [(300, 201, 264, 1), (300, 201, 264, 3), (257, 131, 520, 1), (257, 131, 520, 3),
                                           (130, 67, 72, 2)])
def test_static_entry_point_with_rows_that_are_not_16_byte_multiples(sp, orc, cuda, M, N, K, split_k):
    """N % 4 != 0: the workspace rows are padded to a multiple of four floats (the TMA stores into it need
    16-byte row pitches) while C keeps its own pitch; both the padded workspace walk and the reduction's
    pitch arithmetic run."""
    import torch

    a, b = _operands(sp, cuda, M, N, K)
    got = torch.empty((M, N), dtype=torch.float32, device=cuda)
    got.view(torch.uint8).fill_(0x7D)
    _static(sp, a, b, got, split_k)
    assert _query(sp) == 0
    ref = orc.gemm_f16f32(a.cpu().numpy(), b.cpu().numpy())
    assert orc.normalised_error(got.cpu().numpy(), ref, 1.0, 1.0, K) < 1e-2
    want = sp.matmul_sm100(a, b)
    sp.status()
    assert orc.normalised_error(got.cpu().numpy(), want.cpu().numpy(), 1.0, 1.0, K) < 1e-3


def test_static_entry_point_allocates_nothing_and_runs_on_any_stream(sp, orc, cuda):
    """What the entry point's name promises: free device memory is the same before and after calls (the
    first call on the device was made by the tests above or is made here, before the measurement), also on a
    stream created as non-blocking and with a workspace use just under the 64 MiB capacity."""
    import torch

    L = sp.lib()
    M, N, K, split_k = 4096, 1020, 1280, 4          # 4 * 4096 * 1020 * 4 B = 63.75 MiB of partial sums; 20 K blocks
    a, b = _operands(sp, cuda, M, N, K)
    got = torch.empty((M, N), dtype=torch.float32, device=cuda)
    warm = torch.empty((128, 128), dtype=torch.float32, device=cuda)
    _static(sp, a[:128], b[:128], warm, 1)          # set-up of the device, if this file runs alone
    assert _query(sp) == 0
    s = torch.cuda.Stream()                          # torch streams are non-blocking streams
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        got.view(torch.uint8).fill_(0x7D)
        s.wait_stream(torch.cuda.current_stream())
        rc = L.spork_gemm_sm100_f16f32_static(M, N, K, a.data_ptr(), b.data_ptr(), got.data_ptr(), split_k, s.cuda_stream)
        assert rc == 0
        assert L.spork_gemm_sm100_f16f32_static(0, 0, 0, None, None, None, 1, s.cuda_stream) == 0   # status query
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
    A, B = a.cpu().numpy(), b.cpu().numpy()
    for m0 in (0, 2000, M - 16):
        ref = orc.gemm_f16f32_rows(A, B, m0, 16)
        assert orc.normalised_error(got[m0:m0 + 16].cpu().numpy(), ref, 1.0, 1.0, K) < 1e-2
    # one more split (five ranges of four K blocks) does not fit any more
    assert L.spork_gemm_sm100_f16f32_static(M, N, K, a.data_ptr(), b.data_ptr(), got.data_ptr(), 5, s.cuda_stream) == 10006
