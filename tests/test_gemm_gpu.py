"""Parity of the sm_100a GEMM with the CPU oracle, through the C ABI, on a B200.

Follows the reference's own test method (gemm/gemm_test.cu): seeded position-hashed
inputs, output poisoned with 0x7D bytes before each run, comparison of the whole
result; plus the headline tolerance max|err| / (max|A| max|B| K 2^-10) <= 1.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1.0  # normalised error bound of the headline configurations (fp32 accumulation)


def _inputs(sp, orc, cuda, M, N, K, code_a, code_b):
    """Fixtures made on the device, read back so the oracle sees the exact bits the kernel reads."""
    import torch

    a = torch.empty((M, K), dtype=torch.float16, device=cuda)
    b = torch.empty((N, K), dtype=torch.float16, device=cuda)
    sp.init_test_data(a, code_a, orc.SEED_A)
    # B is the logical K x N matrix stored transposed (the reference's d_bCol, gemm_test.cu:241)
    sp.init_test_data(b, code_b, orc.SEED_B, transpose_rule=True)
    return a, b


def _poisoned(cuda, M, N):
    import torch

    c = torch.empty((M, N), dtype=torch.float32, device=cuda)
    c.view(torch.uint8).fill_(0x7D)  # gemm_test.cu:244-247
    return c


def _check(sp, orc, a, b, c, K):
    A, B, got = a.cpu().numpy(), b.cpu().numpy(), c.cpu().numpy()
    ref = orc.gemm_f16f32(A, B)
    amax = float(np.abs(A.astype(np.float32)).max()) if A.size else 0.0
    bmax = float(np.abs(B.astype(np.float32)).max()) if B.size else 0.0
    if amax == 0 or bmax == 0 or K == 0:
        assert (got == 0).all()
        return 0.0
    err = orc.normalised_error(got, ref, amax, bmax, K)
    assert err <= TOL, f"normalised error {err}"
    return err


def test_device_fixtures_match_the_oracle_bit_for_bit(sp, orc, cuda):
    import torch

    for code in range(5):
        for transpose in (False, True):
            t = torch.empty((70, 136), dtype=torch.float16, device=cuda)
            sp.init_test_data(t, code, 101, transpose_rule=transpose)
            want = orc.fill_f16(70, 136, code, 101, transpose)
            assert (t.cpu().numpy().view(np.uint16) == want.view(np.uint16)).all(), (code, transpose)


def test_baseline_kernel_is_bit_exact_with_the_oracle(sp, orc, cuda):
    for M, N, K in ((256, 256, 512), (70, 130, 72)):
        a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
        c = sp.gemm_baseline(a, b, _poisoned(cuda, M, N))
        ref = orc.gemm_f16f32(a.cpu().numpy(), b.cpu().numpy())
        assert (c.cpu().numpy() == ref).all()


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("block_n", [64, 128, 256])
def test_config1_every_variant(sp, orc, cuda, cta_group, block_n):
    """M=256 N=256 K=512, uniform [-1,1], the reference-sized CPU-checkable configuration."""
    M, N, K = 256, 256, 512
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    c = _poisoned(cuda, M, N)
    sp.matmul_sm100(a, b, c, block_n=block_n, cta_group=cta_group)
    sp.status()
    err = _check(sp, orc, a, b, c, K)
    assert err < 1e-3  # fp32 accumulation: far inside the bound


@pytest.mark.parametrize("variant", [0, 64, 128, 256])
def test_default_entry_point_variants(sp, orc, cuda, variant):
    M, N, K = 384, 320, 264
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    c = _poisoned(cuda, M, N)
    sp.matmul_sm100(a, b, c, variant=variant)
    sp.status()
    _check(sp, orc, a, b, c, K)


# Ragged and extreme shapes from the reference's list (gemm/gemm_main.cpp:98-122), scaled so the
# CPU oracle finishes in seconds, plus shapes that straddle every tile edge.
RAGGED = [(160, 480, 816), (768, 768, 32), (1, 8, 8), (129, 257, 72), (255, 4, 64), (1000, 264, 136),
          (513, 1028, 200), (64, 2048, 1032), (2048, 64, 520), (300, 250, 64), (37, 53, 8), (128, 6, 4104)]


@pytest.mark.parametrize("shape", RAGGED)
@pytest.mark.parametrize("cta_group", [1, 2])
def test_ragged_shapes(sp, orc, cuda, shape, cta_group):
    M, N, K = shape
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    for block_n in (64, 256):
        c = _poisoned(cuda, M, N)
        sp.matmul_sm100(a, b, c, block_n=block_n, cta_group=cta_group)
        sp.status()
        _check(sp, orc, a, b, c, K)


@pytest.mark.parametrize("pair", ["tiled_x_identity", "identity_x_tiled", "random_x_random"])
def test_reference_fixture_pairings_and_comparator(sp, orc, cuda, pair):
    """The three data styles of gemm/gemm_main.cpp:81-95, checked with the reference's own comparator
    (gemm/gemm_test.cu:131-154) on the device and on the host."""
    M, N, K = 640, 384, 512
    codes = {"tiled_x_identity": (orc.DATA_TILED_NUMBERS, orc.DATA_IDENTITY),
             "identity_x_tiled": (orc.DATA_IDENTITY, orc.DATA_TILED_NUMBERS),
             "random_x_random": (orc.DATA_RANDOM, orc.DATA_RANDOM)}[pair]
    a, b = _inputs(sp, orc, cuda, M, N, K, *codes)
    c = _poisoned(cuda, M, N)
    sp.matmul_sm100(a, b, c)
    sp.status()
    base = sp.gemm_baseline(a, b, _poisoned(cuda, M, N))
    first, max_diff = sp.compare_f32(base, c)
    assert first is None, f"reference comparator failed first at {first}"
    ref = orc.gemm_f16f32(a.cpu().numpy(), b.cpu().numpy())
    assert orc.ratio_compare(ref, c.cpu().numpy()) is None
    if pair != "random_x_random":
        # exact small integers times one: the product must be exact, not merely close
        assert (c.cpu().numpy() == ref).all()
        assert max_diff == 0.0


def test_comparator_localises_a_planted_error(sp, orc, cuda):
    import torch

    x = torch.ones((300, 200), dtype=torch.float32, device=cuda)
    y = x.clone()
    y[123, 45] = 1.2
    y[200, 7] = -1.0
    first, max_diff = sp.compare_f32(x, y)
    assert first == (123, 45)
    assert max_diff == pytest.approx(2.0)


@pytest.mark.parametrize("split_k", [2, 3, 16, 1000])
def test_split_k_reduce_add(sp, orc, cuda, split_k):
    M, N, K = 384, 512, 2048
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    for cta_group in (1, 2):
        c = _poisoned(cuda, M, N)
        sp.matmul_sm100(a, b, c, block_n=128, cta_group=cta_group, split_k=split_k)
        sp.status()
        _check(sp, orc, a, b, c, K)


@pytest.mark.parametrize("split_k", [-2, -3, -7])
def test_split_k_with_k_fastest_in_the_schedule(sp, orc, cuda, split_k):
    """split_k <= -2: |split_k| K ranges whose work items are neighbours in the list, so that the ranges of
    one tile run at the same time on different CTA groups (gemm_sm90_k_mode::split_k_inner,
    gemm/gemm_sm90.cu:1096-1114); same sums as the K-slowest order."""
    M, N, K = 640, 1100, 2048
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    for block_n, cta_group, max_ctas in ((128, 2, 0), (256, 1, 6), (512, 2, 4)):
        c = _poisoned(cuda, M, N)
        sp.matmul_sm100(a, b, c, block_n=block_n, cta_group=cta_group, split_k=split_k, max_ctas=max_ctas)
        sp.status()
        _check(sp, orc, a, b, c, K)


@pytest.mark.parametrize("shape", [(1536, 2304, 8192), (512, 512, 4096), (16384, 64, 1024), (160, 480, 816),
                                   (2048, 6000, 264), (300, 131, 2056), (256, 256, 64), (2560, 2560, 1024),
                                   (2304, 2816, 2048), (1024, 4864, 512)])
def test_stream_k(sp, orc, cuda, shape):
    """split_k = -1: whole waves tile by tile, the tiles of a last wave that is at most half full cut into
    aligned K ranges that run at the same time and are reduce-added into tiles the kernel zeroes itself
    (the reference's stream-K modes, gemm/gemm_sm90.cu:1004-1094).  The shapes cover tails with and without
    whole waves before them, N % 4 != 0 (scalar zeroing and atomic adds) and tails that run whole."""
    M, N, K = shape
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    for cta_group, block_n, max_ctas in ((2, 256, 0), (1, 128, 0), (2, 64, 20)):
        c = _poisoned(cuda, M, N)
        sp.matmul_sm100(a, b, c, block_n=block_n, cta_group=cta_group, split_k=-1, max_ctas=max_ctas)
        sp.status()
        _check(sp, orc, a, b, c, K)


def test_stream_k_back_to_back(sp, orc, cuda):
    """Stream-K launches one after the other with nothing between them (each may set itself up while the
    previous one drains, and each meets at its own value of a device counter): every result is right, and
    the library's own choice (split_k = 0) takes this path for 2.35 waves of tiles."""
    import torch
    M, N, K = 2560, 2560, 1024
    assert sp.choice(M, N, 8 * K, split_k=0)["split_k"] == -1
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    cs = [_poisoned(cuda, M, N) for _ in range(20)]
    for c in cs:
        sp.matmul_sm100(a, b, c, block_n=256, cta_group=2, split_k=-1)
    sp.status()
    _check(sp, orc, a, b, cs[0], K)
    for c in cs[1:]:
        assert torch.equal(c, cs[0]) or float((c - cs[0]).abs().max()) < 1e-3  # reduce-add order may differ
    whole = _poisoned(cuda, M, N)
    sp.matmul_sm100(a, b, whole, block_n=256, cta_group=2, split_k=1)
    assert float((whole - cs[-1]).abs().max()) < 1e-2


def test_stream_k_counters_return_to_zero_and_launches_replay_from_a_graph(sp, orc, cuda):
    """The last CTA of a stream-K launch to leave resets the launch's counter pair, so the value a launch
    waits for depends on its grid only: after any number of launches every pair reads zero, and a launch
    recorded into a CUDA graph can be replayed (its parameters are fixed at capture)."""
    import torch

    M, N, K = 2560, 2560, 1024
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    ref = sp.gemm_baseline(a, b)
    for _ in range(40):   # more launches than there are counter pairs
        c = sp.matmul_sm100(a, b, block_n=256, cta_group=2, split_k=-1)
    sp.status()
    assert all(pair == (0, 0) for pair in sp.stream_k_counters())
    _, max_diff = sp.compare_f32(ref, c)
    assert max_diff / (K * 2.0 ** -10) < 1e-2
    # graph replay: capture one launch on a side stream, replay it into a poisoned result several times
    c = _poisoned(cuda, M, N)
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    try:
        with torch.cuda.stream(side):
            sp.matmul_sm100(a, b, c, block_n=256, cta_group=2, split_k=-1)   # warm: attributes, tensor maps
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                sp.matmul_sm100(a, b, c, block_n=256, cta_group=2, split_k=-1, stream=side)
    except (RuntimeError, sp.SporkError) as e:
        pytest.skip(f"this launch cannot be captured here: {e}")
    for _ in range(5):
        c.view(torch.uint8).fill_(0x7D)
        graph.replay()
        torch.cuda.synchronize()
        _, max_diff = sp.compare_f32(ref, c)
        assert max_diff / (K * 2.0 ** -10) < 1e-2
    sp.status()
    assert all(pair == (0, 0) for pair in sp.stream_k_counters())


def test_stream_k_launches_of_different_shapes_in_a_row(sp, orc, cuda):
    """Stream-K launches of different grids and partitions one after the other in one stream: the counters
    their CTAs meet at are handed out in rotation and never reset, so every launch must find its own count."""
    shapes = [(2560, 2560, 1024), (512, 512, 4096), (300, 131, 2056), (2304, 2816, 512)]
    data = []
    for (M, N, K) in shapes:
        a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
        data.append((a, b, sp.gemm_baseline(a, b), K))
    for _ in range(12):
        outs = []
        for (a, b, ref, K) in data:
            c = _poisoned(cuda, *ref.shape)
            sp.matmul_sm100(a, b, c, block_n=256, cta_group=2, split_k=-1)
            outs.append(c)
        sp.status()
        for (a, b, ref, K), c in zip(data, outs):
            _, max_diff = sp.compare_f32(ref, c)
            assert max_diff / (K * 2.0 ** -10) < 1e-2, (tuple(ref.shape), K, max_diff)


@pytest.mark.parametrize("shape", [(2560, 2560, 8192), (768, 3072, 3072), (1536, 2304, 8192), (8192, 4096, 4096),
                                   (300, 131, 2056)])
def test_fully_automatic_launch(sp, orc, cuda, shape):
    """split_k = 0 with no tile given: the library picks tile width and K mode (whole tiles, split-K or
    stream-K); whatever it picks, the product is right."""
    M, N, K = shape
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    c = _poisoned(cuda, M, N)
    sp.matmul_sm100(a, b, c, split_k=0)
    sp.status()
    _check(sp, orc, a, b, c, K)


@pytest.mark.parametrize("shape", [(16384, 64, 2048), (1000, 264, 136), (513, 128, 4104), (256, 256, 64), (300, 131, 200)])
def test_two_column_blocks_per_stage(sp, orc, cuda, shape):
    """The ring-stage variant chosen for skinny problems (256-byte row segments per TMA request), forced on
    shapes with ragged K so that the zero-filled tail spans a whole column block."""
    M, N, K = shape
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    try:
        sp.tune(l2_hints=0x200)
        for block_n, split_k in ((64, 1), (128, 2), (256, -1)):
            c = _poisoned(cuda, M, N)
            sp.matmul_sm100(a, b, c, block_n=block_n, cta_group=2, split_k=split_k)
            sp.status()
            _check(sp, orc, a, b, c, K)
    finally:
        sp.tune()


def test_n_not_multiple_of_four_uses_guarded_stores(sp, orc, cuda):
    for M, N, K in ((130, 67, 72), (256, 1, 64), (300, 131, 136)):
        a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
        for split_k in (1, 2):
            c = _poisoned(cuda, M, N)
            sp.matmul_sm100(a, b, c, block_n=128, cta_group=2, split_k=split_k)
            sp.status()
            _check(sp, orc, a, b, c, K)


def test_empty_and_degenerate_problems(sp, orc, cuda):
    import torch

    # K == 0: C is all zeros; M == 0 or N == 0: nothing to do
    a = torch.empty((64, 0), dtype=torch.float16, device=cuda)
    b = torch.empty((32, 0), dtype=torch.float16, device=cuda)
    c = _poisoned(cuda, 64, 32)
    sp.matmul_sm100(a, b, c)
    sp.status()
    assert (c == 0).all()
    a = torch.empty((0, 64), dtype=torch.float16, device=cuda)
    b = torch.empty((32, 64), dtype=torch.float16, device=cuda)
    sp.matmul_sm100(a, b, torch.empty((0, 32), dtype=torch.float32, device=cuda))
    sp.status()
    # all-zero operands
    a = torch.zeros((128, 64), dtype=torch.float16, device=cuda)
    b = torch.ones((128, 64), dtype=torch.float16, device=cuda)
    c = _poisoned(cuda, 128, 128)
    sp.matmul_sm100(a, b, c)
    sp.status()
    assert (c == 0).all()


def test_argument_errors_are_returned_not_trapped(sp, cuda):
    import torch

    L = sp.lib()
    a = torch.zeros((128, 72), dtype=torch.float16, device=cuda)
    b = torch.zeros((128, 72), dtype=torch.float16, device=cuda)
    c = torch.zeros((128, 128), dtype=torch.float32, device=cuda)
    assert L.spork_gemm_sm100_f16f32(128, 128, 12, a.data_ptr(), b.data_ptr(), c.data_ptr(), 0, None) == 10002
    assert L.spork_gemm_sm100_f16f32(128, 128, 72, a.data_ptr() + 2, b.data_ptr(), c.data_ptr(), 0, None) == 10001
    assert L.spork_gemm_sm100_f16f32(128, 128, 72, None, b.data_ptr(), c.data_ptr(), 0, None) == 10001
    assert L.spork_gemm_sm100_f16f32(128, 128, 72, a.data_ptr(), b.data_ptr(), c.data_ptr(), 100, None) == 10001
    assert L.spork_gemm_sm100_f16f32_ex(128, 128, 72, a.data_ptr(), b.data_ptr(), c.data_ptr(), 128, 3, 1, 0,
                                        None) == 10001
    assert L.spork_gemm_sm100_f16f32_ex(128, 128, 72, a.data_ptr(), b.data_ptr(), c.data_ptr(), 128, 2, 1, -1,
                                        None) == 10001  # max_ctas cannot be negative
    with pytest.raises(TypeError):
        sp.matmul_sm100(a.float(), b)
    with pytest.raises(ValueError):
        sp.matmul_sm100(a, b[:, :64].contiguous())
    sp.status()  # nothing was launched, nothing timed out


def test_host_buffer_entry_point(sp, orc, cuda):
    import torch

    M, N, K = 512, 384, 264
    A = orc.fill_f16(M, K, orc.DATA_UNIFORM_PM1, orc.SEED_A)
    B = orc.fill_f16(N, K, orc.DATA_UNIFORM_PM1, orc.SEED_B)
    c = sp.matmul_sm100_htod(torch.from_numpy(A), torch.from_numpy(B))
    ref = orc.gemm_f16f32(A, B)
    assert orc.normalised_error(c.numpy(), ref, 1.0, 1.0, K) <= TOL
    # a second, smaller call reuses the staging buffers
    c2 = sp.matmul_sm100_htod(torch.from_numpy(A[:128].copy()), torch.from_numpy(B))
    assert orc.normalised_error(c2.numpy(), ref[:128], 1.0, 1.0, K) <= TOL
    # shapes that make the chunk grid ragged in both directions, pinned and pageable host memory
    for (M2, N2, K2) in ((2300, 2050, 136), (257, 3, 64), (4096, 4100, 72)):
        A2 = orc.fill_f16(M2, K2, orc.DATA_UNIFORM_PM1, orc.SEED_A)
        B2 = orc.fill_f16(N2, K2, orc.DATA_UNIFORM_PM1, orc.SEED_B)
        want = orc.gemm_f16f32(A2, B2)
        for pin in (False, True):
            ta, tb = torch.from_numpy(A2), torch.from_numpy(B2)
            out = torch.full((M2, N2), float("nan"), dtype=torch.float32)
            if pin:
                ta, tb, out = ta.pin_memory(), tb.pin_memory(), out.pin_memory()
            sp.matmul_sm100_htod(ta, tb, out)
            assert orc.normalised_error(out.numpy(), want, 1.0, 1.0, K2) <= TOL


def test_non_default_stream_and_back_to_back_launches(sp, orc, cuda):
    import torch

    M, N, K = 512, 512, 1024
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    cs = [_poisoned(cuda, M, N) for _ in range(4)]
    torch.cuda.synchronize()
    for c in cs:
        sp.matmul_sm100(a, b, c, stream=s)
    sp.status(stream=s)
    for c in cs[1:]:
        assert torch.equal(c, cs[0])  # deterministic: same tiles, same order of accumulation
    _check(sp, orc, a, b, cs[0], K)


def test_in_kernel_clock_probe(sp, orc, cuda):
    M = N = K = 4096
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    sp.matmul_sm100(a, b)
    sp.status()
    mhz = sp.last_clock_mhz()
    assert 300.0 < mhz < 2500.0, mhz  # a B200 runs between its idle clock and 1965 MHz


def test_headline_size_properties(sp, orc, cuda):
    """8192^3 (the headline configuration): whole-matrix comparison against the CUDA-core comparison kernel,
    CPU-oracle check of sampled row blocks including both matrix edges, and linearity in A."""
    import torch

    M = N = K = 8192
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    c = _poisoned(cuda, M, N)
    sp.matmul_sm100(a, b, c)
    sp.status()
    base = sp.gemm_baseline(a, b, _poisoned(cuda, M, N))
    _, max_diff = sp.compare_f32(base, c)
    assert max_diff / (K * 2.0 ** -10) <= TOL
    assert max_diff / (K * 2.0 ** -10) < 1e-2
    A, B = a.cpu().numpy(), b.cpu().numpy()
    for m0 in (0, 4000, 8192 - 16):
        ref = orc.gemm_f16f32_rows(A, B, m0, 16)
        got = c[m0:m0 + 16].cpu().numpy()
        assert orc.normalised_error(got, ref, 1.0, 1.0, K) < 1e-2
    # linearity: (2A) B^T == 2 (A B^T) exactly (scaling by two is exact in fp16 and fp32)
    c2 = _poisoned(cuda, M, N)
    sp.matmul_sm100((a * 2).contiguous(), b, c2)
    sp.status()
    assert torch.equal(c2, c * 2)


def test_reference_oracle_kernel_agrees_with_cpu_oracle(orc, cuda):
    """Pins the CPU oracle: the reference's own matmul_baseline (gemm/gemm_baseline.cu, compiled unmodified
    into oracle/_ref) must reproduce it bit for bit on fp16-representable inputs; its Ampere-generation TF32
    kernel (gemm/gemm_sm80.cu) must agree within TF32 rounding."""
    import os

    import torch

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                        "libspork_ref.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libspork_ref.so was not built (needs the reference tree at build time)")
    L = ctypes.CDLL(path)
    vp = ctypes.c_void_p
    for f in (L.spork_ref_matmul_baseline, L.spork_ref_matmul_sm80):
        f.argtypes = [ctypes.c_uint32] * 3 + [vp, vp, vp] + [ctypes.c_int] * 3 + [vp]
    for M, N, K, code in ((256, 256, 512, orc.DATA_UNIFORM_PM1), (160, 480, 816, orc.DATA_UNIFORM_PM1),
                          (768, 768, 1024, orc.DATA_RANDOM)):
        A = orc.fill_f16(M, K, code, orc.SEED_A)
        B = orc.fill_f16(N, K, code, orc.SEED_B)
        ref = orc.gemm_f16f32(A, B)
        a = torch.from_numpy(A.astype(np.float32)).to(cuda)
        b = torch.from_numpy(B.astype(np.float32)).to(cuda)
        c = torch.full((M, N), float("nan"), device=cuda)
        assert L.spork_ref_matmul_baseline(M, N, K, a.data_ptr(), b.data_ptr(), c.data_ptr(), 0, 1, 0, None) == 0
        torch.cuda.synchronize()
        assert (c.cpu().numpy() == ref).all()
        if L.spork_ref_matmul_sm80_supports(M, N, K):
            c2 = torch.full((M, N), float("nan"), device=cuda)
            assert L.spork_ref_matmul_sm80(M, N, K, a.data_ptr(), b.data_ptr(), c2.data_ptr(), 0, 1, 0, None) == 0
            torch.cuda.synchronize()
            # TF32 keeps 10 mantissa bits, as many as fp16: the inputs are exact, only summation order differs
            assert orc.ratio_compare(ref, c2.cpu().numpy()) is None


@pytest.mark.parametrize("M,N,K", [(512, 512, 16384), (300, 520, 8192), (1536, 2304, 8192)])
def test_automatic_split_k(sp, orc, cuda, M, N, K):
    """split_k = 0: the library picks the number of K ranges (few output tiles, long K); the sum is the same
    product within the headline tolerance."""
    a, b = _inputs(sp, orc, cuda, M, N, K, sp.DATA_UNIFORM_PM1, sp.DATA_UNIFORM_PM1)
    c = _poisoned(cuda, M, N)
    sp.matmul_sm100(a, b, c, split_k=0)
    sp.status()
    _check(sp, orc, a, b, c, K)


@pytest.mark.parametrize("split_k", [1, 0])
@pytest.mark.parametrize("N", [64, 128, 256])
def test_skinny_configurations_at_their_own_size(sp, orc, cuda, N, split_k):
    """M = 16384, K = 8192, N = 64 / 128 / 256 through the default entry point (the path the benchmark
    times) and through the automatic launch: CPU-oracle check of row blocks at both edges and in the middle,
    and the whole result against the CUDA-core comparison kernel."""
    M, K = 16384, 8192
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    c = _poisoned(cuda, M, N)
    sp.matmul_sm100(a, b, c, split_k=split_k)
    sp.status()
    A, B = a.cpu().numpy(), b.cpu().numpy()
    for m0 in (0, 128, 8192 - 32, M - 64):
        ref = orc.gemm_f16f32_rows(A, B, m0, 64)
        assert orc.normalised_error(c[m0:m0 + 64].cpu().numpy(), ref, 1.0, 1.0, K) < 1e-2, (N, m0)
    base = sp.gemm_baseline(a, b, _poisoned(cuda, M, N))
    _, max_diff = sp.compare_f32(base, c)
    assert max_diff / (K * 2.0 ** -10) < 1e-2


@pytest.mark.parametrize("no_early_launch", [False, True])
def test_launches_that_depend_on_the_previous_kernel(sp, orc, cuda, no_early_launch):
    """A launch may set itself up while the previous kernel in the stream is still finishing, but must not
    touch memory before that kernel is complete.  A chain in which every product reads what the kernel
    before it wrote (and overwrites what the one before that read) shows any early access as wrong numbers:
    c1 = a b^T; a2 = half(c1 / K) by an elementwise kernel; c2 = a2 b^T; then c1 is overwritten by a third
    product while nothing else separates the launches."""
    import torch

    M, N, K = 1024, 1024, 1024
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    s = torch.cuda.Stream()
    torch.cuda.synchronize()
    try:
        sp.tune(no_early_launch=no_early_launch)
        with torch.cuda.stream(s):
            for _ in range(3):  # repeated so that launches really queue up behind one another
                c1 = _poisoned(cuda, M, N)
                c2 = _poisoned(cuda, M, N)
                sp.matmul_sm100(a, b, c1, stream=s)
                a2 = (c1 * (1.0 / K)).to(torch.float16)
                sp.matmul_sm100(a2, b, c2, stream=s)
                keep = c1.clone()
                sp.matmul_sm100(b, a, c1, stream=s)   # overwrites what the clone and the scaling read
        sp.status(stream=s)
    finally:
        sp.tune()
    A, B = a.cpu().numpy(), b.cpu().numpy()
    ref1 = orc.gemm_f16f32(A, B)
    assert orc.normalised_error(keep.cpu().numpy(), ref1, 1.0, 1.0, K) < 1e-2
    assert torch.equal(a2, (keep * (1.0 / K)).to(torch.float16))
    ref2 = orc.gemm_f16f32(a2.cpu().numpy(), B)
    assert orc.normalised_error(c2.cpu().numpy(), ref2, float(a2.abs().max()), 1.0, K) < 1e-2
    ref3 = orc.gemm_f16f32(B, A)
    assert orc.normalised_error(c1.cpu().numpy(), ref3, 1.0, 1.0, K) < 1e-2


def test_tensor_maps_are_encoded_once_per_operand(sp, orc, cuda):
    """A repeated launch on the same operands makes no driver call for its three TMA descriptors; the same
    memory viewed with another shape gets descriptors of its own (and the right answer)."""
    import torch

    M, N, K = 384, 256, 512
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    c = _poisoned(cuda, M, N)
    sp.matmul_sm100(a, b, c, block_n=128, cta_group=2)
    h0, m0 = sp.tmap_cache_stats()
    sp.matmul_sm100(a, b, c, block_n=128, cta_group=2)
    h1, m1 = sp.tmap_cache_stats()
    assert (h1 - h0, m1 - m0) == (3, 0)
    sp.status()
    _check(sp, orc, a, b, c, K)
    # the same allocations as a 192 x 1024 and a 128 x 1024 matrix
    a2, b2 = a.view(192, 1024), b.view(128, 1024)
    c2 = sp.matmul_sm100(a2, b2, block_n=128, cta_group=2)
    h2, m2 = sp.tmap_cache_stats()
    assert m2 - m1 == 3
    sp.status()
    _check(sp, orc, a2, b2, c2, 1024)


@pytest.mark.parametrize("shape", [(768, 3072, 3072), (1536, 768, 4096), (768, 2816, 4096)])
def test_default_entry_narrows_the_tile_to_fill_the_machine(sp, orc, cuda, shape):
    """Problems with fewer 256-wide tiles than CTA pairs run with 128- or 64-wide tiles through the default
    entry point; same result as the 256-wide tile taken literally (same order of accumulation per element)."""
    import torch

    M, N, K = shape
    assert sp.choice(M, N, K)["block_n"] in (64, 128)
    a, b = _inputs(sp, orc, cuda, M, N, K, orc.DATA_UNIFORM_PM1, orc.DATA_UNIFORM_PM1)
    c = _poisoned(cuda, M, N)
    sp.matmul_sm100(a, b, c)
    sp.status()
    _check(sp, orc, a, b, c, K)
    wide = _poisoned(cuda, M, N)
    sp.matmul_sm100(a, b, wide, variant=256)
    sp.status()
    assert torch.equal(c, wide)
