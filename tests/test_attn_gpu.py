"""Parity of the sm_100a attention forward with the CPU oracle (the math of the reference's simple_attn,
torch_attn.py:11-16), through the C ABI, on a B200."""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# fp16 probabilities (P is rounded to fp16 before P.V, relative step 2^-11) and fp16 output:
# |o - o_ref| <= ATOL + RTOL * |o_ref| with o_ref the oracle's fp32 result.
ATOL = 2e-3
RTOL = 1e-2


def _close(got, ref):
    got = got.astype(np.float32)
    bad = np.abs(got - ref) > ATOL + RTOL * np.abs(ref)
    return not bad.any(), float(np.abs(got - ref).max())


def _qkv(sp, cuda, BH, S, D, seed=101, code=None):
    import torch

    ts = []
    # seeds s, s^888, s^1776 as in matrix_util.hpp:53-55
    for sd in (seed, seed ^ 888, seed ^ 1776):
        t = torch.empty((BH * S, D), dtype=torch.float16, device=cuda)
        sp.init_test_data(t, sp.DATA_NORMAL if code is None else code, sd)
        ts.append(t.view(BH, S, D))
    return ts


@pytest.mark.parametrize("BH,S,D", [(1, 256, 64), (2, 256, 128), (3, 512, 128), (2, 1024, 64), (1, 128, 128),
                                    (5, 384, 128)])
def test_attention_matches_oracle(sp, orc, cuda, BH, S, D):
    q, k, v = _qkv(sp, cuda, BH, S, D)
    o = sp.attn_fwd(q, k, v)
    sp.status()
    _, ref = orc.attn_f16(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy())
    ok, worst = _close(o.cpu().numpy(), ref)
    assert ok, f"max abs error {worst}"


@pytest.mark.parametrize("BH,S,D", [(2, 200, 128), (1, 1, 64), (3, 129, 64), (2, 257, 128), (1, 100, 128), (2, 2560, 64)])
def test_ragged_sequence_lengths(sp, orc, cuda, BH, S, D):
    """Sequence lengths that are not multiples of the 128-key block or the 256-row CTA (keys past the end are
    masked, rows past the end are not stored); 2560 x 64 is the size of the reference's script (torch_attn.py:26)."""
    import torch

    q, k, v = _qkv(sp, cuda, BH, S, D, seed=237)
    o = torch.full((BH, S, D), float("nan"), dtype=torch.float16, device=cuda)
    guard = torch.full((64,), 7.0, dtype=torch.float16, device=cuda)  # must survive: nothing is written past o
    sp.attn_fwd(q, k, v, o)
    sp.status()
    _, ref = orc.attn_f16(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy())
    ok, worst = _close(o.cpu().numpy(), ref)
    assert ok, f"max abs error {worst}"
    assert (guard == 7.0).all()


@pytest.mark.parametrize("name", ["n256_d64", "n320_d128"])
def test_golden_vectors_of_the_reference_math(sp, cuda, name):
    """Inputs and outputs produced by executing the reference's simple_attn (tests/golden/make_attn_golden.py)."""
    import torch

    g = np.load(os.path.join(GOLDEN, f"attn_simple_{name}.npz"))
    q, k, v = (torch.from_numpy(g[n]).to(cuda)[None].contiguous() for n in ("q", "k", "v"))
    o = sp.attn_fwd(q, k, v)
    sp.status()
    ok, worst = _close(o[0].cpu().numpy(), g["o"])
    assert ok, f"max abs error {worst}"
    o1 = sp.attn_fwd(q, k, v, scale=1.0)
    sp.status()
    ok, worst = _close(o1[0].cpu().numpy(), g["o_scale1"])
    assert ok, f"max abs error {worst} (scale = 1)"


# bfloat16 keeps 8 mantissa bits: P and O are rounded with a relative step of 2^-8
ATOL_BF16 = 8e-3
RTOL_BF16 = 2e-2


def _bits(t):
    import torch

    return t.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("BH,S,D", [(2, 256, 64), (2, 384, 128), (1, 200, 128), (3, 129, 64)])
def test_bfloat16_variant_matches_oracle(sp, orc, cuda, BH, S, D):
    """The reference interface's element type (HostAttnArgs holds __nv_bfloat16, matrix_util.hpp:40-45)."""
    import torch

    g = torch.Generator().manual_seed(7)
    q, k, v = (torch.randn((BH, S, D), generator=g).to(torch.bfloat16).to(cuda) for _ in range(3))
    o = sp.attn_fwd(q, k, v)
    sp.status()
    assert o.dtype == torch.bfloat16
    _, ref = orc.attn_bf16(_bits(q), _bits(k), _bits(v))
    got = o.float().cpu().numpy()
    assert not (np.abs(got - ref) > ATOL_BF16 + RTOL_BF16 * np.abs(ref)).any(), float(np.abs(got - ref).max())


def test_bfloat16_golden_vector_of_the_reference_math(sp, cuda):
    """bfloat16 inputs at the reference's testbed size (attn_main.hpp:2-3) through its simple_attn."""
    import torch

    g = np.load(os.path.join(GOLDEN, "attn_simple_n256_d64_bf16.npz"))
    q, k, v = (torch.from_numpy(g[n].view(np.int16)).view(torch.bfloat16).to(cuda)[None].contiguous()
               for n in ("q_bits", "k_bits", "v_bits"))
    o = sp.attn_fwd(q, k, v)
    sp.status()
    got = o[0].float().cpu().numpy()
    assert not (np.abs(got - g["o"]) > ATOL_BF16 + RTOL_BF16 * np.abs(g["o"])).any()


@pytest.mark.parametrize("BH,S,D", [(2, 256, 64), (2, 512, 128), (1, 200, 128), (3, 129, 64), (1, 1000, 128), (2, 1, 64)])
def test_causal_variant_matches_oracle(sp, orc, cuda, BH, S, D):
    """Causal masking (query i sees keys j <= i) is an addition to the reference's math; key blocks above the
    diagonal are skipped, the diagonal block is masked per element."""
    q, k, v = _qkv(sp, cuda, BH, S, D, seed=280)
    o = sp.attn_fwd(q, k, v, causal=True)
    sp.status()
    _, ref = orc.attn_causal_f16(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy())
    ok, worst = _close(o.cpu().numpy(), ref)
    assert ok, f"max abs error {worst}"
    # the first query row attends to the first key only: its output is v[0]
    assert np.abs(o[:, 0].float().cpu().numpy() - v[:, 0].float().cpu().numpy()).max() < 2e-3


def test_causal_large_against_torch(sp, cuda):
    import torch

    BH, S, D = 4, 4096, 128
    q, k, v = _qkv(sp, cuda, BH, S, D)
    o = sp.attn_fwd(q, k, v, causal=True)
    sp.status()
    ref = torch.nn.functional.scaled_dot_product_attention(q[:2].float(), k[:2].float(), v[:2].float(), is_causal=True)
    ok, worst = _close(o[:2].cpu().numpy(), ref.cpu().numpy())
    assert ok, f"max abs error {worst}"


def test_softmax_properties_at_larger_sizes(sp, orc, cuda):
    """Sizes the CPU oracle cannot cover in full: (i) V = ones gives O = 1 exactly up to fp16 rounding of P's
    row sums; (ii) attention is invariant to a permutation of the keys/values; (iii) sampled heads against
    the oracle."""
    import torch

    BH, S, D = 8, 4096, 128
    q, k, v = _qkv(sp, cuda, BH, S, D)
    ones = torch.ones_like(v)
    o = sp.attn_fwd(q, k, ones)
    sp.status()
    assert float((o.float() - 1.0).abs().max()) < 2e-3
    perm = torch.randperm(S, device=cuda, generator=torch.Generator(device=cuda).manual_seed(5))
    o_a = sp.attn_fwd(q, k, v)
    o_b = sp.attn_fwd(q, k[:, perm].contiguous(), v[:, perm].contiguous())
    sp.status()
    assert float((o_a.float() - o_b.float()).abs().max()) < 2e-3
    h = 5
    _, ref = orc.attn_f16(q[h:h + 1, :].cpu().numpy(), k[h:h + 1].cpu().numpy(), v[h:h + 1].cpu().numpy())
    ok, worst = _close(o_a[h:h + 1].cpu().numpy(), ref)
    assert ok, f"max abs error {worst}"


def test_large_scores_do_not_overflow(sp, orc, cuda):
    """Scores far outside exp's range: the running-max rescaling must keep everything finite."""
    BH, S, D = 1, 512, 64
    q, k, v = _qkv(sp, cuda, BH, S, D)
    o = sp.attn_fwd((q * 8).contiguous(), (k * 8).contiguous(), v, scale=1.0)
    sp.status()
    _, ref = orc.attn_f16((q * 8).cpu().numpy(), (k * 8).cpu().numpy(), v.cpu().numpy(), scale=1.0)
    assert np.isfinite(o.float().cpu().numpy()).all()
    ok, worst = _close(o.cpu().numpy(), ref)
    assert ok, f"max abs error {worst}"


def test_reference_shaped_host_entry_point(sp, orc, cuda):
    """htod_f32_attn_sm100_fwd has the signature of htod_f32_tk_4090_fwd (tk_4090_fwd.hpp:7) and is called the
    way torch_attn.py:40-57 calls it: host fp32 (N, d) arrays."""
    N, d = 256, 64
    g = np.load(os.path.join(GOLDEN, "attn_simple_n256_d64.npz"))
    q, k, v = (np.ascontiguousarray(g[n].astype(np.float32)) for n in ("q", "k", "v"))
    o = np.full((N, d), np.nan, dtype=np.float32)
    f32p = ctypes.POINTER(ctypes.c_float)
    sp.lib().htod_f32_attn_sm100_fwd(N, d, q.ctypes.data_as(f32p), k.ctypes.data_as(f32p), v.ctypes.data_as(f32p),
                                     o.ctypes.data_as(f32p))
    ok, worst = _close(o, g["o"])
    assert ok, f"max abs error {worst}"


def test_attention_argument_errors(sp, cuda):
    import torch

    L = sp.lib()
    q = torch.zeros((1, 128, 64), dtype=torch.float16, device=cuda)
    f = ctypes.c_float(0.125)
    assert L.spork_attn_sm100_fwd_f16(1, 128, 96, q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), f, None) == 10002
    assert L.spork_attn_sm100_fwd_f16(1, 128, 64, None, q.data_ptr(), q.data_ptr(), q.data_ptr(), f, None) == 10001
    assert L.spork_attn_sm100_fwd_f16(1, 128, 64, q.data_ptr() + 2, q.data_ptr(), q.data_ptr(), q.data_ptr(), f,
                                      None) == 10001
    assert L.spork_attn_sm100_fwd_f16(0, 128, 64, None, None, None, None, f, None) == 0
    assert sp.lib().spork_attn_sm100_supports(16, 4096, 128) == 1
    assert sp.lib().spork_attn_sm100_supports(16, 4096, 80) == 0
    sp.status()


def _ramp_inputs(cuda, BH, S, D, per_key, noise_seed):
    """Scores that move steadily along the keys: q_i = (a, noise...), k_j = (per_key * j, noise...), so that
    s_ij = a * per_key * j + noise.  The row maximum keeps moving from block to block, which drives the
    kernel through the rescaling of its accumulators (or, falling, lets every later block underflow)."""
    import torch

    g = torch.Generator(device="cpu").manual_seed(noise_seed)
    q = torch.randn((BH, S, D), generator=g) * 0.25
    k = torch.randn((BH, S, D), generator=g) * 0.25
    v = torch.randn((BH, S, D), generator=g)
    q[:, :, 0] = 4.0
    k[:, :, 0] = per_key * torch.arange(S, dtype=torch.float32)[None, :]
    return (t.to(torch.float16).to(cuda).contiguous() for t in (q, k, v))


# per-key steps of the score ramp: one 128-key block moves the scaled, log2 score by
# 4 * step * 128 * scale * log2(e); with scale = 1/sqrt(128) that is 65 * step: 0.05 -> 3 per block (below the
# lazy-rescale threshold of 8 most of the time), 0.25 -> 16 per block, 1.0 -> 65 per block (every block
# rescales), negative: scores fall away from the first block's maximum.
# At head dimension 64 (scale = 1/8: 92 * step per block) the kernel finds out from a block's row sums whether
# its scores stayed within 2^8 of the standing reference, and only then computes the row max: steps 0.02 and
# 0.05 (1.8 and 4.6 per block) cross that line every few blocks, in different rows at different blocks.
@pytest.mark.parametrize("per_key", [0.02, 0.05, 0.25, 1.0, 3.0, -0.25, -2.0])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D", [128, 64])
def test_moving_row_maximum(sp, orc, cuda, per_key, causal, D):
    BH, S = 2, 1024
    q, k, v = _ramp_inputs(cuda, BH, S, D, per_key, 7)
    o = sp.attn_fwd(q, k, v, causal=causal)
    sp.status()
    f = orc.attn_causal_f16 if causal else orc.attn_f16
    _, ref = f(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy())
    ok, worst = _close(o.cpu().numpy(), ref)
    assert ok, f"max abs error {worst}"


def test_moving_row_maximum_d64_ragged(sp, orc, cuda):
    BH, S, D = 3, 700, 64
    for per_key in (0.2, 0.7, -0.4):
        q, k, v = _ramp_inputs(cuda, BH, S, D, per_key, 11)
        o = sp.attn_fwd(q, k, v)
        sp.status()
        _, ref = orc.attn_f16(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy())
        ok, worst = _close(o.cpu().numpy(), ref)
        assert ok, f"per_key {per_key}: max abs error {worst}"


def test_the_reference_script_at_its_own_size(sp, cuda):
    """The flow of the reference's torch_attn.py at its own size and seeds (N = 2560, d = 64, inputs
    rand(seed)^3.6 with seeds 101 / 237 / 280, torch_attn.py:4-7,26-29): the math of simple_attn and torch's
    scaled_dot_product_attention on the CPU against the host-pointer entry point the script would load."""
    import math

    import torch

    N, d = 2560, 64

    def make(seed):
        g = torch.Generator().manual_seed(seed)
        return torch.pow(torch.rand((N, d), dtype=torch.float32, generator=g), 3.6)

    q, k, v = make(101), make(237), make(280)
    s = (q @ k.t()) * (1.0 / math.sqrt(d))
    simple_o = torch.softmax(s, dim=-1) @ v
    torch_o = torch.nn.functional.scaled_dot_product_attention(q, k, v)
    o = torch.empty((N, d), dtype=torch.float32)
    f32p = ctypes.POINTER(ctypes.c_float)
    as_ptr = lambda t: ctypes.cast(t.data_ptr(), f32p)  # noqa: E731
    sp.lib().htod_f32_attn_sm100_fwd(N, d, as_ptr(q), as_ptr(k), as_ptr(v), as_ptr(o))
    sp.status()
    # inputs are rounded to fp16 on the way in and the result on the way out: the same bound as elsewhere
    for ref in (simple_o, torch_o):
        ok, worst = _close(o.numpy(), ref.numpy())
        assert ok, f"max abs error {worst}"


def test_headline_size_and_long_sequences(sp, cuda):
    """The benchmark's own size (B*H = 256, S = 4096, D = 128: every CTA of 28 waves) and a sequence four times
    as long, through properties and a second implementation, since the CPU oracle would take minutes:
    V = ones gives O = 1, and sampled heads agree with torch's scaled_dot_product_attention on the GPU."""
    import torch

    for BH, S, D, heads in ((256, 4096, 128, (0, 100, 255)), (4, 16384, 128, (1, 3)), (8, 8192, 64, (2, 7))):
        q, k, v = _qkv(sp, cuda, BH, S, D, seed=280)
        o = sp.attn_fwd(q, k, torch.ones_like(v))
        sp.status()
        assert float((o.float() - 1.0).abs().max()) < 2e-3, (BH, S, D)
        o = sp.attn_fwd(q, k, v)
        sp.status()
        for h in heads:
            ref = torch.nn.functional.scaled_dot_product_attention(q[h:h + 1].float(), k[h:h + 1].float(),
                                                                   v[h:h + 1].float())
            ok, worst = _close(o[h:h + 1].cpu().numpy(), ref.cpu().numpy())
            assert ok, f"{(BH, S, D)} head {h}: max abs error {worst}"
        del q, k, v, o


def test_headline_size_heads_against_the_oracle(sp, orc, cuda):
    """B*H = 256, S = 4096, D = 128 with the configuration's seeds: three heads (first, middle, last) of the
    full launch against the CPU oracle (8.6 GFLOP per head)."""
    BH, S, D = 256, 4096, 128
    q, k, v = _qkv(sp, cuda, BH, S, D, seed=101, code=sp.DATA_NORMAL_BM)   # N(0,1), the configuration's distribution
    # a true normal: standard deviation one, and tails beyond what a sum of twelve uniforms can reach
    assert abs(float(q.float().std()) - 1.0) < 0.01 and abs(float(q.float().mean())) < 0.01
    assert float(q.float().abs().max()) > 4.5
    o = sp.attn_fwd(q, k, v)
    sp.status()
    for h in (0, 131, 255):
        _, ref = orc.attn_f16(q[h:h + 1].cpu().numpy(), k[h:h + 1].cpu().numpy(), v[h:h + 1].cpu().numpy())
        ok, worst = _close(o[h:h + 1].cpu().numpy(), ref)
        assert ok, f"head {h}: max abs error {worst}"
    # the causal form of the same launch, one head
    o = sp.attn_fwd(q, k, v, causal=True)
    sp.status()
    _, ref = orc.attn_causal_f16(q[77:78].cpu().numpy(), k[77:78].cpu().numpy(), v[77:78].cpu().numpy())
    ok, worst = _close(o[77:78].cpu().numpy(), ref)
    assert ok, f"causal head 77: max abs error {worst}"


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_sizes_masks_and_scales(sp, orc, cuda, seed):
    """A seeded sweep nobody chose by hand: ragged sequence lengths around the 128-key block and the 256-row
    CTA, both head dimensions, with and without the causal mask (each query tile then ends at its own
    diagonal block), the default and a random softmax scale."""
    import torch

    rng = np.random.RandomState(seed)
    for _ in range(8):
        BH = int(rng.randint(1, 5))
        S = int(rng.choice([rng.randint(1, 130), rng.randint(130, 520), rng.randint(520, 1300)]))
        D = int(rng.choice([64, 128]))
        causal = bool(rng.randint(0, 2))
        scale = None if rng.randint(0, 2) else float(rng.uniform(0.02, 0.3))
        q, k, v = _qkv(sp, cuda, BH, S, D, seed=int(rng.randint(1, 1 << 20)))
        o = torch.full((BH, S, D), float("nan"), dtype=torch.float16, device=cuda)
        sp.attn_fwd(q, k, v, o, causal=causal, **({} if scale is None else {"scale": scale}))
        sp.status()
        fn = orc.attn_causal_f16 if causal else orc.attn_f16
        args = (q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy())
        _, ref = fn(*args) if scale is None else fn(*args, scale=scale)
        ok, worst = _close(o.cpu().numpy(), ref)
        assert ok, f"BH={BH} S={S} D={D} causal={causal} scale={scale}: max abs error {worst}"
