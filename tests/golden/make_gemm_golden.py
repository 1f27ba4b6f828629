"""Generates tests/golden/gemm_baseline_*.npz on a GPU box by running the
reference's own oracle kernel, matmul_baseline (gemm/gemm_baseline.cu), compiled
unmodified into oracle/_ref/libspork_ref.so by `make -C oracle ref`.

    python tests/golden/make_gemm_golden.py <output-dir>

Inputs are the seeded fp16 fixtures (widened to fp32, the type the reference
kernel takes; every value is exactly representable), operand layout
GPU_Tensors{M,N,K,a,bCol,c,0,1,0} as in gemm/gemm_test.cu:365.  Only the fp32
outputs and the shape/fixture code are stored.
"""
import ctypes
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402

CASES = [(256, 256, 512, orc.DATA_UNIFORM_PM1), (160, 480, 816, orc.DATA_RANDOM), (300, 200, 72, orc.DATA_TILED_NUMBERS),
         (96, 136, 1032, orc.DATA_UNIFORM_PM1)]


def main():
    out_dir = sys.argv[1]
    os.makedirs(out_dir, exist_ok=True)
    L = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libspork_ref.so"))
    vp = ctypes.c_void_p
    L.spork_ref_matmul_baseline.argtypes = [ctypes.c_uint32] * 3 + [vp, vp, vp] + [ctypes.c_int] * 3 + [vp]
    for M, N, K, code in CASES:
        a16 = orc.fill_f16(M, K, code, orc.SEED_A)
        b16 = orc.fill_f16(N, K, code, orc.SEED_B)
        a = torch.from_numpy(a16.astype(np.float32)).cuda()
        b = torch.from_numpy(b16.astype(np.float32)).cuda()
        c = torch.full((M, N), float("nan"), device="cuda")
        rc = L.spork_ref_matmul_baseline(M, N, K, a.data_ptr(), b.data_ptr(), c.data_ptr(), 0, 1, 0, None)
        torch.cuda.synchronize()
        assert rc == 0
        np.savez_compressed(os.path.join(out_dir, f"gemm_baseline_{M}x{N}x{K}_code{code}.npz"),
                            shape_code=np.array([M, N, K, code], dtype=np.int64), c=c.cpu().numpy())
        print("wrote", M, N, K, code)


if __name__ == "__main__":
    main()
