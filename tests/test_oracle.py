"""CPU tests of the oracle itself: it must be right before anything is compared to it."""
import glob
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def py_pcg3d(x, y, z):
    """Independent restatement of the PCG3D hash (Jarzynski & Olano, JCGT 9(3), 2020) with the
    64-bit fold of gemm/gemm_test.cu:52."""
    m = 0xFFFFFFFF
    x = (x * 1664525 + 1013904223) & m
    y = (y * 1664525 + 1013904223) & m
    z = (z * 1664525 + 1013904223) & m
    x = (x + y * z) & m
    y = (y + z * x) & m
    z = (z + x * y) & m
    x ^= x >> 16
    y ^= y >> 16
    z ^= z >> 16
    x = (x + y * z) & m
    y = (y + z * x) & m
    z = (z + x * y) & m
    return x ^ (y << 12) ^ (z << 24)


def test_half_conversion_matches_numpy(orc):
    L = orc.lib()
    bits = np.arange(0, 65536, 3, dtype=np.uint32).astype(np.uint16)
    ref = bits.view(np.float16).astype(np.float32)
    for h, f in zip(bits.tolist(), ref.tolist()):
        got = L.spork_oracle_half_to_float(h)
        assert (np.isnan(f) and np.isnan(got)) or got == f
    rng = np.random.default_rng(7)
    xs = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s
                         for s in (1.0, 1e-3, 1e-5, 6e-8, 3e-8, 100.0, 3e4, 7e4)] +
                        [np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 2.0 ** -24, 2.0 ** -25, 1.5 * 2.0 ** -25,
                                   np.inf, -np.inf], dtype=np.float32)])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    for x, w in zip(xs.tolist(), want.tolist()):
        assert L.spork_oracle_float_to_half(x) == w, x


def test_pcg3d_matches_independent_restatement(orc):
    rng = np.random.default_rng(1)
    cases = [(0, 0, 0), (1, 2, 3), (0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF), (8191, 8191, 20010106), (5, 7, 19980724)]
    cases += [tuple(int(v) for v in rng.integers(0, 2 ** 32, 3)) for _ in range(200)]
    for c in cases:
        assert orc.pcg3d(*c) == py_pcg3d(*c)


def test_reference_fixture_codes(orc):
    # identity and tiled_numbers follow gemm/gemm_test.cu:66-71
    eye = orc.fill_f16(70, 90, orc.DATA_IDENTITY).astype(np.float32)
    assert (eye == np.eye(70, 90, dtype=np.float32)).all()
    tiled = orc.fill_f16(130, 70, orc.DATA_TILED_NUMBERS).astype(np.float32)
    r, c = np.meshgrid(np.arange(130), np.arange(70), indexing="ij")
    want = ((c % 64) + 100 * (r % 64)).astype(np.float32).astype(np.float16).astype(np.float32)
    assert (tiled == want).all()
    # transpose_rule: the stored transpose holds the same logical values (gemm_test.cu:240-241)
    b_kn = orc.fill_f16(48, 80, orc.DATA_TILED_NUMBERS, 0, False)
    b_nk = orc.fill_f16(80, 48, orc.DATA_TILED_NUMBERS, 0, True)
    assert (b_kn.T == b_nk).all()
    # sparse random: 75% zeros, rest in [0,1] or the rare 1000
    rnd = orc.fill_f16(512, 512, orc.DATA_RANDOM).astype(np.float32)
    zero_frac = float((rnd == 0).mean())
    assert 0.72 < zero_frac < 0.80
    assert ((rnd <= 1.0) | (rnd == 1000.0)).all() and (rnd >= 0).all()
    x, y = 17, 33
    bits = py_pcg3d(x, y, 20010106)
    if bits % 100000 == 0:
        expect = np.float16(1000.0)
    elif bits % 4 != 0:
        expect = np.float16(0.0)
    else:
        v = np.float32(py_pcg3d(x, y, 19980724) % 1000000) * np.float32(1e-6)
        expect = np.float16((v * v) * (v * v))
    assert rnd[y, x] == np.float32(expect)


def test_seeded_distributions(orc):
    u = orc.fill_f16(256, 1024, orc.DATA_UNIFORM_PM1, orc.SEED_A).astype(np.float64)
    assert u.min() >= -1.0 and u.max() <= 1.0
    assert abs(u.mean()) < 0.01 and abs(u.std() - 1 / np.sqrt(3)) < 0.01
    x, y = 5, 9
    bits = py_pcg3d(x, y, orc.SEED_A) & 0xFFFFFF
    assert u[y, x] == float(np.float16(np.float32(bits) * np.float32(2.0 ** -23) - np.float32(1.0)))
    n = orc.fill_f16(256, 1024, orc.DATA_NORMAL, 101).astype(np.float64)
    assert abs(n.mean()) < 0.01 and abs(n.std() - 1.0) < 0.01
    # different seeds give different matrices; same seed reproduces
    assert (orc.fill_f16(8, 8, orc.DATA_NORMAL, 101) == orc.fill_f16(8, 8, orc.DATA_NORMAL, 101)).all()
    assert (orc.fill_f16(8, 8, orc.DATA_NORMAL, 101) != orc.fill_f16(8, 8, orc.DATA_NORMAL, 101 ^ 888)).any()


@pytest.mark.parametrize("M,N,K", [(256, 256, 512), (37, 53, 72), (1, 1, 8), (5, 70, 0), (130, 17, 816)])
def test_gemm_oracle_is_the_scalar_recurrence(orc, M, N, K):
    a = orc.fill_f16(M, K, orc.DATA_UNIFORM_PM1, orc.SEED_A)
    b = orc.fill_f16(N, K, orc.DATA_UNIFORM_PM1, orc.SEED_B)
    c = orc.gemm_f16f32(a, b)
    # docs/nyc25.py:34-55 / gemm/gemm_baseline.cu:74-83: accum = 0; for k: accum += a*b (fp32)
    rng = np.random.default_rng(0)
    for _ in range(12):
        m, n = int(rng.integers(0, M)), int(rng.integers(0, N))
        acc = np.float32(0)
        for k in range(K):
            acc = np.float32(acc + np.float32(a[m, k]) * np.float32(b[n, k]))
        assert c[m, n] == acc
    ref64 = a.astype(np.float64) @ b.astype(np.float64).T
    assert orc.normalised_error(c, ref64.astype(np.float32), 1.0, 1.0, max(K, 1)) < 1e-3
    assert np.abs(orc.gemm_f16f64(a, b) - ref64).max() < 1e-9
    if M >= 8:
        rows = orc.gemm_f16f32_rows(a, b, 3, 4)
        assert (rows == c[3:7]).all()


def test_gemm_known_answers(orc):
    # identity x tiled_numbers gives the tiled matrix back (the reference's pairing, gemm_main.cpp:81-90)
    M, N, K = 96, 160, 192
    tiled = orc.fill_f16(M, K, orc.DATA_TILED_NUMBERS)
    eye_nk = orc.fill_f16(N, K, orc.DATA_IDENTITY, 0, True)
    c = orc.gemm_f16f32(tiled, eye_nk)
    assert (c == tiled.astype(np.float32)[:, :N]).all()
    eye_mk = orc.fill_f16(M, K, orc.DATA_IDENTITY)
    tiled_nk = orc.fill_f16(N, K, orc.DATA_TILED_NUMBERS, 0, True)
    c = orc.gemm_f16f32(eye_mk, tiled_nk)
    assert (c == tiled_nk.astype(np.float32).T[:M, :]).all()


def test_gemm_oracle_matches_reference_kernel_output(orc):
    """Outputs of the reference's own oracle kernel (gemm/gemm_baseline.cu, run unmodified on a B200 on
    the same seeded inputs) are stored under tests/golden/; the CPU oracle must reproduce them bit for bit."""
    files = sorted(glob.glob(os.path.join(GOLDEN, "gemm_baseline_*.npz")))
    assert files, "golden GEMM vectors are missing"
    for f in files:
        g = np.load(f)
        M, N, K, code = (int(v) for v in g["shape_code"])
        a = orc.fill_f16(M, K, code, orc.SEED_A)
        b = orc.fill_f16(N, K, code, orc.SEED_B)
        c = orc.gemm_f16f32(a, b)
        assert c.shape == g["c"].shape
        assert (c.view(np.uint32) == g["c"].view(np.uint32)).all(), f


def test_ratio_comparator(orc):
    a = np.array([[1.0, 2.0, 0.0], [4.0, -1.0, 8.0]], dtype=np.float32)
    assert orc.ratio_compare(a, a.copy()) is None
    b = a.copy()
    b[0, 1] = 2.0 * (1 + 1 / 33.0)  # inside 1 + 1/32
    assert orc.ratio_compare(a, b) is None
    b[1, 2] = 8.0 * (1 + 1 / 31.0)  # outside
    assert orc.ratio_compare(a, b) == (1, 2)
    b[0, 2] = 1e-30  # zero vs non-zero fails, and comes first in row-major order
    assert orc.ratio_compare(a, b) == (0, 2)
    c = a.copy()
    c[1, 1] = 1.0  # sign flip
    assert orc.ratio_compare(a, c) == (1, 1)
    d = a.copy()
    d[0, 0] = np.nan
    assert orc.ratio_compare(a, d) == (0, 0)


def test_normalised_error(orc):
    ref = np.zeros((4, 4), dtype=np.float32)
    c = ref.copy()
    c[2, 1] = 0.5
    assert orc.normalised_error(c, ref, 1.0, 1.0, 1024) == pytest.approx(0.5)
    c[0, 0] = np.nan
    assert orc.normalised_error(c, ref, 1.0, 1.0, 1024) == float("inf")


@pytest.mark.parametrize("name", ["n256_d64", "n320_d128"])
def test_attention_oracle_matches_reference_math(orc, name):
    """Vectors produced by executing the reference's simple_attn (torch_attn.py:11-16); see make_attn_golden.py."""
    g = np.load(os.path.join(GOLDEN, f"attn_simple_{name}.npz"))
    q, k, v = (g[n][None] for n in ("q", "k", "v"))
    o16, o32 = orc.attn_f16(q, k, v)
    # fp32 math in a different summation order: agreement to a few fp32 ulps of the row scale
    assert np.abs(o32[0] - g["o"]).max() <= 2e-6 * max(1.0, float(np.abs(g["o"]).max()))
    assert (o16[0] == o32[0].astype(np.float16)).all()
    _, o32_s1 = orc.attn_f16(q, k, v, scale=1.0)
    assert np.abs(o32_s1[0] - g["o_scale1"]).max() <= 2e-6 * max(1.0, float(np.abs(g["o_scale1"]).max()))


def test_attention_oracle_bfloat16_matches_reference_math(orc):
    g = np.load(os.path.join(GOLDEN, "attn_simple_n256_d64_bf16.npz"))
    o16, o32 = orc.attn_bf16(g["q_bits"][None], g["k_bits"][None], g["v_bits"][None])
    assert np.abs(o32[0] - g["o"]).max() <= 2e-6 * max(1.0, float(np.abs(g["o"]).max()))
    # the rounded output is the nearest bfloat16 of the fp32 result
    assert np.abs(orc.bf16_bits_to_f32(o16[0]) - o32[0]).max() <= 2.0 ** -8 * float(np.abs(o32).max())


def test_attention_oracle_matches_torch_sdpa(orc):
    import torch

    BH, S, D = 3, 160, 128
    q = orc.fill_f16(BH * S, D, orc.DATA_NORMAL, 101).reshape(BH, S, D)
    k = orc.fill_f16(BH * S, D, orc.DATA_NORMAL, 101 ^ 888).reshape(BH, S, D)
    v = orc.fill_f16(BH * S, D, orc.DATA_NORMAL, 101 ^ 1776).reshape(BH, S, D)
    _, o32 = orc.attn_f16(q, k, v)
    tq, tk, tv = (torch.from_numpy(x.astype(np.float32)) for x in (q, k, v))
    ref = torch.nn.functional.scaled_dot_product_attention(tq, tk, tv).numpy()
    assert np.abs(o32 - ref).max() < 5e-6


def test_box_muller_fixture_is_a_unit_normal(orc):
    x = orc.fill_f16(512, 1024, orc.DATA_NORMAL_BM, 101).astype(np.float64)
    assert abs(x.mean()) < 0.01 and abs(x.std() - 1.0) < 0.01
    assert np.abs(x).max() > 4.0          # 5e5 samples of a true normal reach past four sigma
    y = orc.fill_f16(512, 1024, orc.DATA_NORMAL_BM, 101 ^ 888).astype(np.float64)
    assert abs(np.corrcoef(x.ravel(), y.ravel())[0, 1]) < 0.01   # another seed, another matrix
