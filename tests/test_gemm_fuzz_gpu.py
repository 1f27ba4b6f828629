"""Seeded sweep over ragged shapes and every launch mode of the sm_100a GEMM, on a B200.

The reference checks each algorithm on a fixed list of shapes (gemm/gemm_main.cpp:18-117); this sweep adds
shapes nobody chose by hand: odd row and column counts, K not a multiple of the 64-wide K block, tiles that
hang over every edge, with the tile width, the CTA group, the K mode and the grid bound drawn at random.
Every result is compared in full with the CUDA-core comparison kernel (itself pinned to the CPU oracle) and
on row blocks with the CPU oracle.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _cases(seed, count):
    rng = np.random.RandomState(seed)
    out = []
    for _ in range(count):
        M = int(rng.choice([rng.randint(1, 300), rng.randint(300, 1400), rng.randint(1400, 5000)]))
        N = int(rng.choice([rng.randint(1, 200), rng.randint(200, 1100), rng.randint(1100, 4200)]))
        K = 8 * int(rng.choice([rng.randint(1, 20), rng.randint(20, 200), rng.randint(200, 700)]))
        mode = rng.randint(0, 6)
        kw = {}
        if mode == 0:
            pass                                             # the default entry point
        elif mode == 1:
            kw = dict(split_k=0)                             # fully automatic
        elif mode == 2:
            kw = dict(variant=int(rng.choice([64, 128, 256, 512])))
        else:
            block_n = int(rng.choice([64, 128, 256, 512]))
            cta_group = 2 if block_n == 512 else int(rng.choice([1, 2]))
            split_k = int(rng.choice([1, 2, 3, 5, -1, -2, -3, 0]))
            if block_n == 512 and split_k == -1:
                split_k = 1
            kw = dict(block_n=block_n, cta_group=cta_group, split_k=split_k,
                      max_ctas=int(rng.choice([0, 0, 2 * cta_group, 20, 74, 111])))
        out.append((M, N, K, kw))
    return out


@pytest.mark.parametrize("seed", [1, 2, 3, 4])
def test_random_shapes_and_modes(sp, orc, cuda, seed):
    import torch

    for (M, N, K, kw) in _cases(seed, 12):
        a = torch.empty((M, K), dtype=torch.float16, device=cuda)
        b = torch.empty((N, K), dtype=torch.float16, device=cuda)
        sp.init_test_data(a, orc.DATA_UNIFORM_PM1, orc.SEED_A + seed)
        sp.init_test_data(b, orc.DATA_UNIFORM_PM1, orc.SEED_B + seed, transpose_rule=True)
        c = torch.empty((M, N), dtype=torch.float32, device=cuda)
        c.view(torch.uint8).fill_(0x7D)
        sp.matmul_sm100(a, b, c, **kw)
        sp.status()
        base = sp.gemm_baseline(a, b)
        _, max_diff = sp.compare_f32(base, c)
        assert max_diff / (K * 2.0 ** -10) < 1e-2, (M, N, K, kw, max_diff)
        A, B = a.cpu().numpy(), b.cpu().numpy()
        for m0 in sorted({0, max(0, M // 2 - 8), max(0, M - 16)}):
            rows = min(16, M - m0)
            ref = orc.gemm_f16f32_rows(A, B, m0, rows)
            assert orc.normalised_error(c[m0:m0 + rows].cpu().numpy(), ref, 1.0, 1.0, K) < 1e-2, (M, N, K, kw, m0)
