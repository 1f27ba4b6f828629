"""Context columns: the reference's own GPU kernels that still build for sm_100a - matmul_baseline
(gemm/gemm_baseline.cu, fp32 FFMA, the reference's oracle) and matmul_sm80 (gemm/gemm_sm80.cu, mma.sync TF32,
Ampere generation) - timed on the B200 beside this library's tf32 and fp16 kernels at a headline-class
shape.  Different element types (the reference kernels take fp32 operands), so the numbers are context, not
a like-for-like comparison; they are printed (run with -s) and written to the file named by
SPORK_CONTEXT_OUT when that is set.  The reference's Hopper kernel (wgmma) and its CUTLASS build do not
compile for sm_100a and have no column."""
import ctypes
import json
import os

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libspork_ref.so")


def _time(torch, fn, n, warm=2):
    for _ in range(warm):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n


def test_reference_kernels_timed_beside_this_library(sp, orc, cuda):
    import torch

    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libspork_ref.so was not built (needs the reference tree at build time)")
    L = ctypes.CDLL(REF_LIB)
    vp = ctypes.c_void_p
    for f in (L.spork_ref_matmul_baseline, L.spork_ref_matmul_sm80):
        f.argtypes = [ctypes.c_uint32] * 3 + [vp, vp, vp] + [ctypes.c_int] * 3 + [vp]
    M, N, K = 7680, 7680, 8192   # the 8192-class shape matmul_sm80 accepts (M, N multiples of 768, K of 32)
    assert L.spork_ref_matmul_sm80_supports(M, N, K)
    a16 = torch.empty((M, K), dtype=torch.float16, device=cuda)
    b16 = torch.empty((N, K), dtype=torch.float16, device=cuda)
    sp.init_test_data(a16, sp.DATA_UNIFORM_PM1, sp.SEED_A)
    sp.init_test_data(b16, sp.DATA_UNIFORM_PM1, sp.SEED_B, transpose_rule=True)
    a32, b32 = a16.float(), b16.float()
    c = torch.empty((M, N), dtype=torch.float32, device=cuda)
    flops = 2.0 * M * N * K
    out = {"shape": [M, N, K], "unit": "TFLOP/s"}

    def ref_sm80():
        assert L.spork_ref_matmul_sm80(M, N, K, a32.data_ptr(), b32.data_ptr(), c.data_ptr(), 0, 1, 0, None) == 0

    def ref_baseline():
        assert L.spork_ref_matmul_baseline(M, N, K, a32.data_ptr(), b32.data_ptr(), c.data_ptr(), 0, 1, 0, None) == 0

    out["reference matmul_sm80 (fp32 in, mma.sync tf32)"] = flops / _time(torch, ref_sm80, 5) / 1e9
    c_sm80 = c.clone()
    out["reference matmul_baseline (fp32 FFMA, its oracle)"] = flops / _time(torch, ref_baseline, 1, warm=1) / 1e9
    c_base = c.clone()
    out["this library, tf32 (fp32 in)"] = flops / _time(torch, lambda: sp.matmul_sm100_tf32(a32, b32, c), 20) / 1e9
    c_tf32 = c.clone()
    out["this library, fp16 in"] = flops / _time(torch, lambda: sp.matmul_sm100(a16, b16, c), 20) / 1e9
    sp.status()
    out["cuBLAS tf32 (torch.mm, fp32 in)"] = None
    try:
        torch.backends.cuda.matmul.allow_tf32 = True
        bt = b32.t()
        out["cuBLAS tf32 (torch.mm, fp32 in)"] = flops / _time(torch, lambda: torch.mm(a32, bt), 20) / 1e9
    finally:
        torch.backends.cuda.matmul.allow_tf32 = False
    # all four agree: the operands are fp16-exact, so tf32 reads them exactly and only summation order differs
    bound = K * 2.0 ** -10
    for other in (c_sm80, c_tf32, c):
        assert float((other - c_base).abs().max()) / bound < 1e-2
    print("\ncontext columns:", json.dumps(out, indent=1))
    path = os.environ.get("SPORK_CONTEXT_OUT")
    if path:
        with open(path, "w") as f:
            json.dump(out, f, indent=1)
    # sanity only: the Blackwell kernel must be far ahead of the Ampere-generation one on this GPU
    assert out["this library, tf32 (fp32 in)"] > 2 * out["reference matmul_sm80 (fp32 in, mma.sync tf32)"]
