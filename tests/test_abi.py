"""CPU tests of the drop-in boundary: the library loads and exports what the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not fn.endswith(".h"):
            continue
        text = open(os.path.join(ROOT, "include", fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        if 'extern "C"' not in text:
            continue  # C++-only convenience headers declare no ABI symbols
        for m in re.finditer(r"^\s*(?:const\s+)?[A-Za-z_][\w\s\*]*?\b(\w+)\s*\([^;{]*\)\s*;", text, flags=re.M):
            names.append(m.group(1))
    return names


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("spork_gemm_sm100_supports", "spork_gemm_sm100_f16f32", "spork_gemm_sm100_status",
                 "spork_attn_sm100_fwd_f16", "htod_f32_attn_sm100_fwd", "spork_gemm_baseline_f16f32"):
        assert must in names


def test_library_exports_every_declared_symbol(sp):
    L = ctypes.CDLL(sp.library_path())
    missing = [n for n in declared_functions() if not hasattr(L, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_supports_and_argument_errors_need_no_gpu(sp):
    assert sp.matmul_sm100_supports(8192, 8192, 8192)
    assert sp.matmul_sm100_supports(160, 480, 816)
    assert sp.matmul_sm100_supports(0, 0, 0)
    assert not sp.matmul_sm100_supports(128, 128, 12)  # K % 8 != 0: rows are not 16-byte multiples
    L = sp.lib()
    # unsupported shape and bad variant are rejected before any CUDA call
    assert L.spork_gemm_sm100_f16f32(128, 128, 12, None, None, None, 0, None) == 10002
    assert L.spork_gemm_sm100_f16f32(128, 128, 16, None, None, None, 96, None) == 10001
    # the batched form checks its arguments the same way
    assert L.spork_gemm_sm100_f16f32_batched(4, 128, 128, 12, None, None, None, 0, 1, None) == 10002
    assert L.spork_gemm_sm100_f16f32_batched(4, 128, 128, 16, None, None, None, 0, 0, None) == 10001
    assert L.spork_gemm_sm100_f16f32_batched(0, 128, 128, 16, None, None, None, 0, 1, None) == 0  # empty batch
    assert "sm_100a" in sp.version()


def test_attention_refuses_a_scale_that_is_not_positive(sp):
    """scale = 0 (the mean of V in the reference's simple_attn) cannot be computed by a kernel that folds the
    scale into the exponent; it is refused like a negative or NaN scale, before anything is launched."""
    import ctypes

    L = sp.lib()
    fake = ctypes.c_void_p(0x10000)  # aligned, never dereferenced: the argument check comes first
    for scale in (0.0, -1.0, float("nan")):
        assert L.spork_attn_sm100_fwd_f16(1, 128, 64, fake, fake, fake, fake, ctypes.c_float(scale), None) == 10001
    assert L.spork_attn_sm100_fwd_f16(1, 128, 96, fake, fake, fake, fake, ctypes.c_float(1.0), None) == 10002  # head dimension


def test_missing_library_fails_loudly(monkeypatch):
    import spork_b200.api as api

    monkeypatch.setattr(api, "_lib", None)
    monkeypatch.setattr(api, "_LIB_PATH", os.path.join(ROOT, "no_such_dir", "libspork_b200.so"))
    with pytest.raises(FileNotFoundError):
        api.lib()


def test_python_wrappers_reject_mismatched_shapes_before_any_launch(sp):
    """Tensor maps and stores are sized from the first operand: the wrappers refuse operands of another
    shape instead of letting a kernel run past an allocation.  CPU tensors do: the shape check comes first."""
    import torch

    q = torch.zeros((2, 256, 64), dtype=torch.float16)
    with pytest.raises(ValueError):
        sp.attn_fwd(q, q[:, :128].contiguous(), q)          # shorter k (a cross-attention call)
    with pytest.raises(ValueError):
        sp.attn_fwd(q, q, q[:, :, :32].contiguous())        # narrower v
    with pytest.raises(ValueError):
        sp.attn_fwd(q, q, q, o=torch.zeros((1, 256, 64), dtype=torch.float16))  # o too small
    with pytest.raises(ValueError):
        sp.attn_fwd(q[0], q[0], q[0])
    a = torch.zeros((128, 64))
    b = torch.zeros((96, 64))
    with pytest.raises(ValueError):
        sp.matmul_sm100_tf32(a, b, torch.zeros((128, 64)))   # c must be (128, 96)
    with pytest.raises(ValueError):
        sp.matmul_sm100(a.half(), b.half(), torch.zeros((64, 96)))


def test_tuning_knobs_round_trip_without_a_gpu(sp):
    try:
        sp.tune(l2_hints=8)                       # "no hints at all" must reach the launch as an empty mask
        assert sp.tuning()["l2_hints"] == 0
        sp.tune(l2_hints=4)
        assert sp.tuning()["l2_hints"] == 4
        sp.tune(stages=5, group_m=4, k_atoms=2, wide=2, wide_skew=2, wide_group_m=16, experiment=1)
        t = sp.tuning()
        assert (t["stages"], t["group_m"], t["k_atoms"], t["wide"], t["wide_skew"], t["wide_group_m"],
                t["experiment"]) == (5, 4, 2, 2, 2, 16, 1)
        assert sp.lib().spork_gemm_sm100_tune(0, 0, 3 << 10, 0) == 10001   # tile choice 3 does not exist
    finally:
        sp.tune()
    assert sp.tuning() == {"stages": 0, "group_m": 8, "l2_hints": 3, "backoff_ns": 0, "experiment": 0, "k_atoms": 0,
                           "wide": 0, "wide_skew": 0, "wide_group_m": 0, "no_early_launch": 0}
