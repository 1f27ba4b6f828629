"""The C++ launch functions on the reference's own types: oracle/_ref/dropin_check is compiled against
the reference's gpu_tensor.h and matrix_util.hpp (make -C oracle dropin REF=...) and calls
matmul_sm100_tf32(GPU_Tensors, stream), matmul_sm100(GPU_TensorsF16 with a column-major C, stream) and
launch_attn_sm100_fwd_kernel(HostAttnArgs, o); this test writes its operands and checks what it wrote
against the CPU oracle."""
import os
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "oracle", "_ref", "dropin_check")


def _f32_to_bf16_bits(x):
    u = x.astype(np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)  # round to nearest even


def test_launch_functions_on_the_reference_types(orc, cuda, tmp_path):
    if not os.path.exists(EXE):
        pytest.skip("oracle/_ref/dropin_check was not built (needs the reference tree at build time)")
    M, N, K, S, D = 300, 520, 264, 384, 64
    A = orc.fill_f16(M, K, orc.DATA_UNIFORM_PM1, orc.SEED_A)
    B = orc.fill_f16(N, K, orc.DATA_UNIFORM_PM1, orc.SEED_B)
    A.astype(np.float32).tofile(tmp_path / "a.f32")   # fp16-exact values: tf32 reads them exactly
    B.astype(np.float32).tofile(tmp_path / "b.f32")
    rng = np.random.default_rng(101)
    qkv = [_f32_to_bf16_bits(rng.standard_normal((S, D)).astype(np.float32)) for _ in range(3)]
    for name, t in zip(("q", "k", "v"), qkv):
        t.tofile(tmp_path / f"{name}.bf16")
    r = subprocess.run([EXE, str(tmp_path), str(M), str(N), str(K), str(S), str(D)], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    ref = orc.gemm_f16f32(A, B)
    c_row = np.fromfile(tmp_path / "c_row.f32", dtype=np.float32).reshape(M, N)
    assert orc.normalised_error(c_row, ref, 1.0, 1.0, K) < 1e-2
    # column-major C: element (m, n) at n * M + m, i.e. the row-major N x M transpose
    for name in ("c_col.f32", "c16_col.f32"):
        c_col = np.fromfile(tmp_path / name, dtype=np.float32).reshape(N, M)
        assert orc.normalised_error(np.ascontiguousarray(c_col.T), ref, 1.0, 1.0, K) < 1e-2, name
    o_bits = np.fromfile(tmp_path / "o.bf16", dtype=np.uint16).reshape(1, S, D)
    _, o_ref = orc.attn_bf16(qkv[0].reshape(1, S, D), qkv[1].reshape(1, S, D), qkv[2].reshape(1, S, D))
    got = orc.bf16_bits_to_f32(o_bits)
    assert np.all(np.abs(got - o_ref) <= 8e-3 + 2e-2 * np.abs(o_ref)), float(np.abs(got - o_ref).max())
