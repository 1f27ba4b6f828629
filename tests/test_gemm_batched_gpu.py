"""The batched GEMM entry point (the batch dimension L of the reference's generated entry points,
xgemm_Sm90.py:45-48) against the single-product entry point and the CPU oracle, on a B200."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _batch(sp, orc, cuda, L, M, N, K):
    """L different fixtures: matrix l is the position hash with seed + l, uniform in [-1, 1)."""
    import torch

    a = torch.empty((L, M, K), dtype=torch.float16, device=cuda)
    b = torch.empty((L, N, K), dtype=torch.float16, device=cuda)
    for l in range(L):
        sp.init_test_data(a[l], sp.DATA_UNIFORM_PM1, orc.SEED_A + l)
        sp.init_test_data(b[l], sp.DATA_UNIFORM_PM1, orc.SEED_B + l, transpose_rule=True)
    return a, b


def _poisoned(cuda, shape):
    import torch

    c = torch.empty(shape, dtype=torch.float32, device=cuda)
    c.view(torch.uint8).fill_(0x7D)  # the reference poisons its outputs, gemm/gemm_test.cu:244-247
    return c


# ragged rows and columns, N not a multiple of 4 (guarded scalar stores), one tile per matrix, many tiles
SHAPES = [(3, 300, 200, 264), (5, 128, 64, 64), (2, 257, 130, 72), (4, 512, 768, 128), (7, 40, 24, 8), (1, 160, 480, 816)]


@pytest.mark.parametrize("L,M,N,K", SHAPES)
def test_batch_equals_the_single_products_bit_for_bit(sp, orc, cuda, L, M, N, K):
    a, b = _batch(sp, orc, cuda, L, M, N, K)
    c = _poisoned(cuda, (L, M, N))
    sp.matmul_sm100_batched(a, b, c)
    sp.status()
    got = c.cpu().numpy()
    for l in range(L):
        single = _poisoned(cuda, (M, N))
        sp.matmul_sm100(a[l], b[l], single)
        sp.status()
        assert (got[l].view(np.uint32) == single.cpu().numpy().view(np.uint32)).all(), l


@pytest.mark.parametrize("L,M,N,K", SHAPES[:3])
def test_batch_against_the_oracle(sp, orc, cuda, L, M, N, K):
    a, b = _batch(sp, orc, cuda, L, M, N, K)
    c = _poisoned(cuda, (L, M, N))
    sp.matmul_sm100_batched(a, b, c)
    sp.status()
    A, B, got = a.cpu().numpy(), b.cpu().numpy(), c.cpu().numpy()
    for l in range(L):
        ref = orc.gemm_f16f32(A[l], B[l])
        amax = float(np.abs(A[l].astype(np.float32)).max())
        bmax = float(np.abs(B[l].astype(np.float32)).max())
        assert orc.normalised_error(got[l], ref, amax, bmax, K) <= 1.0, l


@pytest.mark.parametrize("variant", [64, 128, 256])
def test_batch_tile_variants(sp, orc, cuda, variant):
    L, M, N, K = 3, 384, 320, 192
    a, b = _batch(sp, orc, cuda, L, M, N, K)
    c = _poisoned(cuda, (L, M, N))
    sp.matmul_sm100_batched(a, b, c, variant=variant)
    sp.status()
    got = c.cpu().numpy()
    for l in range(L):
        single = _poisoned(cuda, (M, N))
        sp.matmul_sm100(a[l], b[l], single, variant=variant)
        assert (got[l].view(np.uint32) == single.cpu().numpy().view(np.uint32)).all(), (variant, l)


def test_batch_with_split_k(sp, orc, cuda):
    """Partial products of each matrix are reduce-added into that matrix only."""
    L, M, N, K = 3, 200, 136, 1024
    a, b = _batch(sp, orc, cuda, L, M, N, K)
    c = _poisoned(cuda, (L, M, N))
    sp.matmul_sm100_batched(a, b, c, split_k=4)
    sp.status()
    A, B, got = a.cpu().numpy(), b.cpu().numpy(), c.cpu().numpy()
    for l in range(L):
        ref = orc.gemm_f16f32(A[l], B[l])
        amax = float(np.abs(A[l].astype(np.float32)).max())
        bmax = float(np.abs(B[l].astype(np.float32)).max())
        assert orc.normalised_error(got[l], ref, amax, bmax, K) <= 1.0, l


def test_empty_batch_and_k_zero(sp, orc, cuda):
    import torch

    a = torch.empty((0, 128, 64), dtype=torch.float16, device=cuda)
    b = torch.empty((0, 128, 64), dtype=torch.float16, device=cuda)
    c = torch.empty((0, 128, 128), dtype=torch.float32, device=cuda)
    L = sp.lib()
    assert L.spork_gemm_sm100_f16f32_batched(0, 128, 128, 64, None, None, None, 0, 1, None) == 0
    c = _poisoned(cuda, (2, 16, 8))
    assert L.spork_gemm_sm100_f16f32_batched(2, 16, 8, 0, None, None, int(c.data_ptr()), 0, 1, None) == 0
    torch.cuda.synchronize()
    assert (c.cpu().numpy() == 0).all()  # an empty sum
    del a, b
