"""The GEMM on the reference's own operand type: fp32 A and B read as tf32, fp32 accumulate/output."""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rand(M, K, seed, signed=True):
    import torch

    g = torch.Generator().manual_seed(seed)
    t = torch.rand((M, K), generator=g, dtype=torch.float32)
    return (t * 2 - 1) if signed else t


@pytest.mark.parametrize("M,N,K", [(256, 256, 512), (160, 480, 816), (1000, 264, 132), (384, 72, 2048), (130, 67, 64)])
def test_tf32_matches_cpu_oracle(sp, orc, cuda, M, N, K):
    """Against nyc25_gemm_cpu's loop on fp32 inputs (docs/nyc25.py:13-56).  Tolerance: tf32 keeps 10 mantissa
    bits, so each product is within 2^-10 relative (two truncations of 2^-11 each would be 2^-10):
    max|err| / (max|A| max|B| K 2^-10) <= 1; against the oracle fed tf32-truncated operands the error is
    only the fp32 summation order."""
    a, b = _rand(M, K, 1), _rand(N, K, 2)
    c = sp.matmul_sm100_tf32(a.to(cuda), b.to(cuda))
    sp.status()
    got = c.cpu().numpy()
    ref = orc.gemm_f32(a.numpy(), b.numpy(), 0)
    assert orc.normalised_error(got, ref, 1.0, 1.0, K) <= 1.0
    trunc = orc.gemm_f32(a.numpy(), b.numpy(), 1)
    rna = orc.gemm_f32(a.numpy(), b.numpy(), 2)
    e_trunc = orc.normalised_error(got, trunc, 1.0, 1.0, K)
    e_rna = orc.normalised_error(got, rna, 1.0, 1.0, K)
    # one of the two conversions is what the hardware does; it is matched far more tightly
    assert min(e_trunc, e_rna) < 2e-3, (e_trunc, e_rna)


def test_tf32_split_k_and_variants(sp, orc, cuda):
    M, N, K = 512, 384, 4096
    a, b = _rand(M, K, 3), _rand(N, K, 4)
    ref = orc.gemm_f32(a.numpy(), b.numpy(), 0)
    for variant, split_k in ((0, 1), (64, 1), (128, 1), (256, 4)):
        c = sp.matmul_sm100_tf32(a.to(cuda), b.to(cuda), variant=variant, split_k=split_k)
        sp.status()
        assert orc.normalised_error(c.cpu().numpy(), ref, 1.0, 1.0, K) <= 1.0


def test_tf32_exact_on_fp16_representable_inputs(sp, orc, cuda):
    """Values with at most 10 mantissa bits survive the tf32 conversion: identity x tiled numbers is exact."""
    import torch

    M, N, K = 384, 256, 512
    a16 = orc.fill_f16(M, K, orc.DATA_TILED_NUMBERS)
    b16 = orc.fill_f16(N, K, orc.DATA_IDENTITY, 0, True)
    a = torch.from_numpy(a16.astype(np.float32)).to(cuda)
    b = torch.from_numpy(b16.astype(np.float32)).to(cuda)
    c = sp.matmul_sm100_tf32(a, b)
    sp.status()
    assert (c.cpu().numpy() == orc.gemm_f16f32(a16, b16)).all()


def test_tf32_agrees_with_the_reference_kernels(sp, orc, cuda):
    """Same fp32 inputs through the reference's own matmul_baseline (fp32 FFMA) and matmul_sm80 (mma.sync
    tf32), compiled unmodified into oracle/_ref, checked with the reference's comparator on non-negative data
    (gemm/gemm_test.cu:131-154)."""
    import torch

    path = os.path.join(ROOT, "oracle", "_ref", "libspork_ref.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libspork_ref.so was not built (needs the reference tree at build time)")
    L = ctypes.CDLL(path)
    vp = ctypes.c_void_p
    for f in (L.spork_ref_matmul_baseline, L.spork_ref_matmul_sm80):
        f.argtypes = [ctypes.c_uint32] * 3 + [vp, vp, vp] + [ctypes.c_int] * 3 + [vp]
    M, N, K = 768, 1536, 1024
    a, b = _rand(M, K, 5, signed=False).to(cuda), _rand(N, K, 6, signed=False).to(cuda)
    ours = sp.matmul_sm100_tf32(a, b)
    sp.status()
    base = torch.full((M, N), float("nan"), device=cuda)
    assert L.spork_ref_matmul_baseline(M, N, K, a.data_ptr(), b.data_ptr(), base.data_ptr(), 0, 1, 0, None) == 0
    torch.cuda.synchronize()
    first, _ = sp.compare_f32(base, ours)
    assert first is None, f"reference comparator failed at {first}"
    assert L.spork_ref_matmul_sm80_supports(M, N, K)
    sm80 = torch.full((M, N), float("nan"), device=cuda)
    assert L.spork_ref_matmul_sm80(M, N, K, a.data_ptr(), b.data_ptr(), sm80.data_ptr(), 0, 1, 0, None) == 0
    torch.cuda.synchronize()
    first, max_diff = sp.compare_f32(sm80, ours)
    assert first is None
    # both read the operands as tf32: they agree far more closely than either does with fp32
    assert max_diff / (K * 2.0 ** -10) < 0.05


def test_tf32_argument_errors(sp, cuda):
    import torch

    L = sp.lib()
    a = torch.zeros((128, 68), dtype=torch.float32, device=cuda)
    c = torch.zeros((128, 128), dtype=torch.float32, device=cuda)
    assert L.spork_gemm_sm100_tf32f32(128, 128, 66, a.data_ptr(), a.data_ptr(), c.data_ptr(), 0, 1, None) == 10002
    assert L.spork_gemm_sm100_tf32f32(128, 128, 68, a.data_ptr(), a.data_ptr(), c.data_ptr(), 96, 1, None) == 10001
    assert L.spork_gemm_sm100_tf32f32(128, 128, 68, None, a.data_ptr(), c.data_ptr(), 0, 1, None) == 10001
    sp.status()


@pytest.mark.parametrize("seed", [21, 22])
def test_tf32_random_shapes_and_modes(sp, orc, cuda, seed):
    """A seeded sweep over ragged shapes (K a multiple of 4 only), tile variants and K modes of the tf32 path,
    including the automatic launch and stream-K on a problem with a thin last wave."""
    rng = np.random.RandomState(seed)
    cases = [(2560, 2560, 1024, dict(split_k=0))]   # 100 tiles: one wave of 74 + 26 cut in two (stream-K)
    for _ in range(7):
        M = int(rng.choice([rng.randint(1, 300), rng.randint(300, 1500)]))
        N = int(rng.choice([rng.randint(1, 200), rng.randint(200, 1300)]))
        K = 4 * int(rng.choice([rng.randint(1, 40), rng.randint(40, 500)]))
        kw = dict(variant=int(rng.choice([0, 64, 128, 256, 512])), split_k=int(rng.choice([1, 1, 2, 3, 0])))
        cases.append((M, N, K, kw))
    for (M, N, K, kw) in cases:
        a, b = _rand(M, K, seed * 100 + 1), _rand(N, K, seed * 100 + 2)
        c = sp.matmul_sm100_tf32(a.to(cuda), b.to(cuda), **kw)
        sp.status()
        if M * N * K <= 1 << 29:
            ref = orc.gemm_f32(a.numpy(), b.numpy(), 0)
        else:
            ref = (a.double() @ b.double().t()).float().numpy()
        assert orc.normalised_error(c.cpu().numpy(), ref, 1.0, 1.0, K) <= 1.0, (M, N, K, kw)
