"""The host-side model of the GEMM kernels' barrier protocol (spork_gemm_sm100_ring_model): the shared-memory
ring, the accumulator hand-over and the skewed chunk schedule of the 256 x 512 kernel, run as cooperative
agents over modelled mbarriers in seeded interleavings.  No GPU.  Stands where the reference's development
relies on compute-sanitizer's race checker."""
import pytest


def _ok(sp, *shape, **kw):
    rc, stats = sp.ring_model(*shape, **kw)
    assert rc == 0, (shape, kw, rc)
    return stats


@pytest.mark.parametrize("block_n,cta_group", [(64, 1), (128, 2), (256, 1), (256, 2)])
def test_ring_and_accumulator_protocol_of_the_256_wide_kernel(sp, block_n, cta_group):
    # few CTAs so that a group owns many work items (the accumulator buffers alternate and wrap)
    for seed in range(6):
        for stages in (2, 4, 6):
            st = _ok(sp, 1024, 768, 1024, block_n=block_n, cta_group=cta_group, max_ctas=2 * cta_group, stages=stages,
                     seed=seed, group=seed % 2)
            assert st["items"] >= 3 and st["mma_ops"] == st["items"] * 16
    # split-K and stream-K item lists
    _ok(sp, 512, 512, 4096, block_n=block_n, cta_group=cta_group, split_k=3, max_ctas=2 * cta_group, seed=11)
    _ok(sp, 1536, 2304, 2048, block_n=block_n, cta_group=cta_group, split_k=-1, sm_count=20, seed=12, group=3)
    # stream-K with whole waves in front of a thin last wave cut into aligned K ranges
    _ok(sp, 2560, 2560, 1024, block_n=block_n, cta_group=cta_group, split_k=-1, sm_count=64 * cta_group // 2 + 10, seed=13,
        group=2)


@pytest.mark.parametrize("skew", [1, 2, 3, 4])
def test_chunk_schedule_of_the_256x512_kernel(sp, skew):
    # K blocks per tile below the skew, between one and two skews, exactly two, many
    for K in (64, 192, 320, 448, 512, 1088, 2048):
        for seed in range(4):
            st = _ok(sp, 1024, 2048, K, block_n=512, max_ctas=4, skew=skew, seed=seed, group=seed % 2)
            assert st["items"] == 8 and st["mma_ops"] == 8 * 2 * (K // 64)
    _ok(sp, 512, 1500, 2048, block_n=512, split_k=3, max_ctas=2, skew=skew, seed=5)
    # a shallower ring bounds the skew
    _ok(sp, 1024, 1024, 1024, block_n=512, max_ctas=2, stages=2, skew=skew, seed=6)
    _ok(sp, 1024, 1024, 1024, block_n=512, max_ctas=2, stages=3, skew=skew, seed=7)


def test_the_headline_plan_one_group(sp):
    # 8192^3 as launched: 74 CTA pairs; group 73 owns 13 tiles of the 256 x 256 plan and 6 of the 256 x 512 plan
    st = _ok(sp, 8192, 8192, 8192, block_n=256, group=73, seed=1)
    assert st["groups"] == 74 and st["items"] == 13
    st = _ok(sp, 8192, 8192, 8192, block_n=512, group=73, seed=2)
    assert st["groups"] == 74 and st["items"] == 6


def test_planted_protocol_bugs_are_noticed(sp):
    """The checks bite: each planted bug is reported (in at least one of a few interleavings) with the code of
    the invariant it breaks, or as the deadlock it causes."""
    def codes(inject, K=1024, **kw):
        return {sp.ring_model(1024, 2048, K, max_ctas=4, seed=s, inject=inject, **kw)[0] for s in range(12)}

    assert codes(0, block_n=512) == {0}
    assert 3 in codes(1, block_n=512) or 2 in codes(1, block_n=512)    # a stage released before its second reader
    # (one K block per tile: the issuer is back at the accumulator before sixteen epilogue warps have read it)
    assert codes(2, K=64, block_n=512) & {4, 5}                       # the issuer overwrites an accumulator in use
    assert codes(2, K=64, block_n=256) & {4, 5}
    assert codes(3, block_n=256) & {2, 3}                             # the producer refills a stage in use
    assert sp.ring_model(1024, 1024, 1024, block_n=512, cta_group=1)[0] == 10001   # pairs only
