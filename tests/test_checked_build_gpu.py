"""The range-checked debug build (libspork_b200_checked.so, -DSPORK_CHECKED) on a B200: the same kernels with
every shared-memory and tensor-memory address and every TMA coordinate tested before use.  Runs in a child
process, because the library is chosen when the package first loads it."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECKED = os.path.join(ROOT, "spork_b200", "libspork_b200_checked.so")

CHILD = textwrap.dedent("""
    import sys
    sys.path.insert(0, %r)
    import numpy as np, torch
    import spork_b200 as sp
    from oracle import oracle as orc
    assert sp.library_path().endswith("libspork_b200_checked.so")
    dev = torch.device("cuda:0")
    L = sp.lib()
    # the checks refuse what is out of range, report through the status word, and access nothing
    for which in (0, 1, 2):
        assert L.spork_selftest_range_check(which, None) == 0
        try:
            sp.status()
            raise SystemExit("check %%d did not fire" %% which)
        except sp.SporkError as e:
            assert e.code == 10007 and ("0xc%%03x" %% (0x701 + which)) in str(e).lower(), str(e)
    assert L.spork_selftest_range_check(3, None) == 0
    sp.status()
    # every kernel family on small shapes: results as in the normal build, status word clear
    def inputs(M, N, K):
        a = torch.empty((M, K), dtype=torch.float16, device=dev); b = torch.empty((N, K), dtype=torch.float16, device=dev)
        sp.init_test_data(a, sp.DATA_UNIFORM_PM1, sp.SEED_A); sp.init_test_data(b, sp.DATA_UNIFORM_PM1, sp.SEED_B, transpose_rule=True)
        return a, b
    cases = [((300, 200, 264), dict(block_n=64, cta_group=1)), ((513, 1028, 200), dict(block_n=256, cta_group=2)),
             ((512, 512, 2048), dict(block_n=128, cta_group=2, split_k=3)), ((2560, 2560, 512), dict(block_n=256, cta_group=2, split_k=-1)),
             ((700, 1500, 1032), dict(block_n=512, cta_group=2)), ((130, 67, 72), dict(block_n=128, cta_group=2)),
             ((1000, 2050, 264), dict(block_n=512, cta_group=2, split_k=2))]
    for (M, N, K), kw in cases:
        a, b = inputs(M, N, K)
        c = sp.matmul_sm100(a, b, **kw)
        sp.status()
        ref = orc.gemm_f16f32(a.cpu().numpy(), b.cpu().numpy())
        assert orc.normalised_error(c.cpu().numpy(), ref, 1.0, 1.0, K) < 1e-2, (M, N, K, kw)
    a, b = inputs(16384, 64, 2048)
    c = sp.matmul_sm100(a, b)       # the two-column-block ring of the skinny shapes
    sp.status()
    a3 = torch.stack([inputs(256, 192, 136)[0]] * 3); b3 = torch.stack([inputs(256, 192, 136)[1]] * 3)
    c3 = sp.matmul_sm100_batched(a3, b3)
    sp.status()
    assert torch.equal(c3[0], c3[2])
    st = sp.matmul_sm100(a3[0], b3[0], None)
    assert torch.equal(st, c3[0])
    print("checked build ok")
""")


def test_checked_build_runs_clean_and_its_checks_fire(cuda):
    if not os.path.exists(CHECKED):
        pytest.skip("libspork_b200_checked.so was not built (python -m spork_b200.build --checked)")
    env = dict(os.environ, SPORK_B200_LIBRARY=CHECKED)
    r = subprocess.run([sys.executable, "-c", CHILD % ROOT], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and "checked build ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_normal_build_has_no_range_checks(sp):
    assert sp.lib().spork_selftest_range_check(0, None) == 10002
