"""The 256 x 512 tile kernel (two 256-column accumulator halves per CTA pair, issued with a skew at both
ends of a tile) against the CPU oracle and against the 256 x 256 kernel, through the C ABI, on a B200.

The shapes walk through every form of the issue schedule: tiles of fewer K blocks than the skew (one
chunk), between one and two skews (two chunks), exactly two skews, many; several tiles per CTA pair (so the
accumulator hand-over between tiles runs); ragged M, N and K; a dead second half (N <= 256); N not a
multiple of 4 (guarded stores); split-K."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1.0


def _inputs(sp, orc, cuda, M, N, K):
    import torch

    a = torch.empty((M, K), dtype=torch.float16, device=cuda)
    b = torch.empty((N, K), dtype=torch.float16, device=cuda)
    sp.init_test_data(a, sp.DATA_UNIFORM_PM1, orc.SEED_A)
    sp.init_test_data(b, sp.DATA_UNIFORM_PM1, orc.SEED_B, transpose_rule=True)
    return a, b


def _poisoned(cuda, M, N):
    import torch

    c = torch.empty((M, N), dtype=torch.float32, device=cuda)
    c.view(torch.uint8).fill_(0x7D)
    return c


def _check(orc, a, b, c, K):
    ref = orc.gemm_f16f32(a.cpu().numpy(), b.cpu().numpy())
    err = orc.normalised_error(c.cpu().numpy(), ref, 1.0, 1.0, K)
    assert err <= TOL, f"normalised error {err}"
    assert err < 1e-2


SHAPES = [(256, 512, 64), (512, 1024, 256), (512, 1024, 320), (300, 700, 448), (768, 1536, 512),
          (512, 1024, 1032), (256, 200, 128), (130, 1031, 200), (1, 8, 8), (1000, 2050, 264)]


@pytest.mark.parametrize("shape", SHAPES)
def test_wide_tiles_against_the_oracle(sp, orc, cuda, shape):
    M, N, K = shape
    a, b = _inputs(sp, orc, cuda, M, N, K)
    c = _poisoned(cuda, M, N)
    sp.matmul_sm100(a, b, c, block_n=512, cta_group=2)
    sp.status()
    _check(orc, a, b, c, K)


@pytest.mark.parametrize("skew", [1, 2, 3, 4])
def test_every_skew_and_many_tiles_per_pair(sp, orc, cuda, skew):
    """Four CTAs (two pairs) walk sixteen tiles: the hand-over of both accumulator halves between tiles runs
    seven times per pair.  The result is the 256 x 256 kernel's bit for bit (same order of accumulation)."""
    import torch

    M, N, K = 1024, 2048, 1088  # 17 K blocks
    a, b = _inputs(sp, orc, cuda, M, N, K)
    narrow = _poisoned(cuda, M, N)
    sp.matmul_sm100(a, b, narrow, block_n=256, cta_group=2)
    try:
        sp.tune(wide_skew=skew, wide_group_m=3)
        c = _poisoned(cuda, M, N)
        sp.matmul_sm100(a, b, c, block_n=512, cta_group=2, max_ctas=4)
        sp.status()
    finally:
        sp.tune()
    assert torch.equal(c, narrow)
    _check(orc, a, b, c, K)


@pytest.mark.parametrize("split_k", [2, 3, 5])
def test_wide_tiles_split_k(sp, orc, cuda, split_k):
    M, N, K = 512, 1500, 2048
    a, b = _inputs(sp, orc, cuda, M, N, K)
    c = _poisoned(cuda, M, N)
    sp.matmul_sm100(a, b, c, block_n=512, cta_group=2, split_k=split_k)
    sp.status()
    _check(orc, a, b, c, K)


def test_library_choice_equals_the_narrow_kernel(sp, orc, cuda):
    """A problem large enough for the library to pick 256 x 512 tiles by itself; forced either way the
    result is the same bits."""
    import torch

    M, N, K = 9472, 8192, 4096  # 37 x 16 = 592 wide tiles: eight full waves of 74 pairs, and a long K
    a, b = _inputs(sp, orc, cuda, M, N, K)
    outs = []
    for wide in (0, 1, 2):
        try:
            sp.tune(wide=wide)
            assert sp.tuning()["wide"] == wide
            c = _poisoned(cuda, M, N)
            sp.matmul_sm100(a, b, c)
            sp.status()
        finally:
            sp.tune()
        outs.append(c)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])
    A, B = a.cpu().numpy(), b.cpu().numpy()
    for m0 in (0, 4800, M - 16):
        ref = orc.gemm_f16f32_rows(A, B, m0, 16)
        assert orc.normalised_error(outs[0][m0:m0 + 16].cpu().numpy(), ref, 1.0, 1.0, K) < 1e-2


def test_wide_tiles_tf32(sp, orc, cuda):
    import torch

    M, N, K = 512, 1100, 328
    g = torch.Generator(device="cpu").manual_seed(7)
    a = (torch.rand((M, K), generator=g) * 2 - 1).to(cuda)
    b = (torch.rand((N, K), generator=g) * 2 - 1).to(cuda)
    narrow = sp.matmul_sm100_tf32(a, b, variant=256)
    wide = sp.matmul_sm100_tf32(a, b, variant=512)
    sp.status()
    assert torch.equal(wide, narrow)


def test_tuning_round_trip(sp, cuda):
    """Every knob reaches the launch parameters, the "no hints" value of the L2 hint field included."""
    try:
        sp.tune(l2_hints=8)
        assert sp.tuning()["l2_hints"] == 0
        sp.tune(l2_hints=1)
        assert sp.tuning()["l2_hints"] == 1
        sp.tune(stages=4, group_m=6, backoff_ns=32, experiment=0, k_atoms=2, wide=1, wide_skew=3, wide_group_m=12)
        t = sp.tuning()
        assert (t["stages"], t["group_m"], t["backoff_ns"], t["k_atoms"], t["wide"], t["wide_skew"],
                t["wide_group_m"]) == (4, 6, 32, 2, 1, 3, 12)
    finally:
        sp.tune()
    assert sp.tuning()["l2_hints"] == 3  # the default: both operands evict-last
