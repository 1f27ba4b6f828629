"""The harness watch loop (the reference's gemm_loop.py) against a stand-in executable; no GPU."""
import io
import os
import stat
import threading
import time

from spork_b200 import gemm_loop


def test_runs_on_every_rebuild_and_stops_when_idle(tmp_path):
    log = tmp_path / "runs.log"
    exe = tmp_path / "fake_gemm"

    def build(tag):
        tmp = tmp_path / "fake_gemm.new"
        tmp.write_text(f"#!/bin/sh\necho {tag} \"$@\" >> {log}\nexit 3\n")
        tmp.chmod(tmp.stat().st_mode | stat.S_IXUSR)
        os.replace(tmp, exe)  # what a linker does: the new file appears in one step

    build("first")
    out = io.StringIO()
    result = {}
    t = threading.Thread(target=lambda: result.update(runs=gemm_loop.watch(str(exe), ["--quick"], 1.0, 0.02, out)))
    t.start()
    time.sleep(0.4)
    build("second")
    t.join(timeout=20)
    assert not t.is_alive()
    assert result["runs"] == 2
    assert log.read_text().split("\n")[:2] == ["first --quick", "second --quick"]
    assert out.getvalue().count("END (exit status 3)") == 2
