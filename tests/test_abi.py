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


def test_missing_library_fails_loudly(monkeypatch):
    import spork_b200.api as api

    monkeypatch.setattr(api, "_lib", None)
    monkeypatch.setattr(api, "_LIB_PATH", os.path.join(ROOT, "no_such_dir", "libspork_b200.so"))
    with pytest.raises(FileNotFoundError):
        api.lib()
