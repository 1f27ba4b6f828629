"""Runs the C++ harness (spork_b200/bin/gemm), the counterpart of the reference's `gemm/gemm` binary, which is
the reference's own test suite (gemm/gemm_main.cpp, gemm/gemm_test.cu): every algorithm on every listed
shape is compared on the device against the comparison GEMM; the exit status is non-zero on any mismatch."""
import json
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_harness_quick_list(tmp_path, cuda):
    exe = os.path.join(ROOT, "spork_b200", "bin", "gemm")
    if not os.path.exists(exe):
        from spork_b200 import build

        exe = build.build_harness()
    out = tmp_path / "harness.jsonl"
    proc = subprocess.run([exe, "--quick", "--json", str(out)], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-2000:]
    rows = [json.loads(line) for line in out.read_text().splitlines()]
    assert rows and all(r["pass"] for r in rows)
    algos = {r["algorithm"] for r in rows}
    assert any("mine_sm_100" in a for a in algos) and any("cublas" in a for a in algos)
    # the headline shape ran with the new kernel
    assert any(r["M"] == 8192 and r["N"] == 8192 and r["K"] == 8192 and "mine_sm_100 (output" in r["algorithm"]
               for r in rows)
