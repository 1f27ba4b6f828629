#!/usr/bin/env python3
"""Re-run the GEMM harness every time its binary is rebuilt.

The development loop of the reference's gemm_loop.py (gemm_loop.py:1-18): watch the harness executable,
run it whenever its modification time changes, give up after a stretch without a rebuild.  Here the
executable is ``spork_b200/bin/gemm`` (built by ``python -m spork_b200.build``), arguments after ``--`` are
passed through to it, and the exit status of every run is reported.

    python -m spork_b200.gemm_loop [--exe PATH] [--idle-timeout SECONDS] [--poll SECONDS] [-- harness args]
"""
import argparse
import os
import subprocess
import sys
import time

DEFAULT_EXE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "bin", "gemm")


def watch(exe: str, harness_args: list[str], idle_timeout: float, poll: float, out=sys.stderr) -> int:
    """Returns how many times the harness ran before `idle_timeout` seconds passed without a rebuild."""
    runs = 0
    seen_mtime = None
    last_activity = time.monotonic()
    while time.monotonic() - last_activity <= idle_timeout:
        try:
            mtime = os.stat(exe).st_mtime_ns
        except FileNotFoundError:
            mtime = None  # mid-rebuild: the linker has removed the old file
        if mtime is not None and mtime != seen_mtime:
            print(time.strftime("START %H:%M:%S"), file=out, flush=True)
            rc = subprocess.call([exe] + harness_args)
            print(f"END (exit status {rc})", file=out, flush=True)
            seen_mtime = mtime
            runs += 1
            last_activity = time.monotonic()
        time.sleep(poll)
    return runs


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    harness_args: list[str] = []
    if "--" in argv:
        i = argv.index("--")
        argv, harness_args = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--exe", default=DEFAULT_EXE)
    ap.add_argument("--idle-timeout", type=float, default=300.0, help="stop after this long without a rebuild")
    ap.add_argument("--poll", type=float, default=0.05, help="seconds between looks at the file")
    args = ap.parse_args(argv)
    runs = watch(args.exe, harness_args, args.idle_timeout, args.poll)
    print(f"no rebuild for {args.idle_timeout:g} s: stopping after {runs} run(s)", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
