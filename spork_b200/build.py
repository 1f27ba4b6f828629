"""Build step: compiles the CUDA sources under ``csrc/`` into ``libspork_b200.so``
(in-tree, next to this file) with nvcc for sm_100a.  Cross-compiles without a GPU."""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libspork_b200.so")
NVCC = os.environ.get("SPORK_NVCC", "nvcc")
FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--ptxas-options=-O3",
]


def sources() -> list[str]:
    found = glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp"))
    return sorted(p for p in found if not os.path.basename(p).startswith("main_"))


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


CHECKED_LIB = os.path.join(HERE, "libspork_b200_checked.so")


def build(force: bool = False, verbose: bool = False, checked: bool = False) -> str:
    """Compile each source to an object (only when stale) and link the shared library.

    ``checked=True`` builds the debug variant ``libspork_b200_checked.so`` (-DSPORK_CHECKED: the kernels
    range-check every shared-memory and tensor-memory address and every TMA coordinate and report through
    the device status word); select it at run time with the environment variable SPORK_B200_LIBRARY."""
    headers = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    objdir = os.path.join(HERE, "build_checked" if checked else "build")
    lib = CHECKED_LIB if checked else LIB
    flags = FLAGS + (["-DSPORK_CHECKED"] if checked else [])
    os.makedirs(objdir, exist_ok=True)
    objs = []
    procs = []
    for src in sources():
        obj = os.path.join(objdir, os.path.splitext(os.path.basename(src))[0] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [NVCC] + flags + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out)
        if p.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    if force or procs or _stale(lib, objs):
        cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", lib] + objs
        subprocess.run(cmd, check=True)
    return lib


CUTLASS_COLUMN = os.path.join(HERE, "bin", "libcutlass_column.so")


def find_cutlass() -> str | None:
    """A CUTLASS header tree for the harness's comparison column: $SPORK_CUTLASS_DIR, or the copy some
    Python packages ship in their data directory.  None if there is none (the column is then absent)."""
    import importlib.util

    cands = [os.environ.get("SPORK_CUTLASS_DIR")]
    for pkg, sub in (("flashinfer", os.path.join("data", "cutlass")),):
        spec = importlib.util.find_spec(pkg)
        if spec and spec.submodule_search_locations:
            cands.append(os.path.join(list(spec.submodule_search_locations)[0], sub))
    for c in cands:
        if c and os.path.exists(os.path.join(c, "include", "cutlass", "cutlass.h")):
            return c
    return None


def build_cutlass_column() -> str | None:
    """Compile csrc/main_cutlass_column.cu into bin/libcutlass_column.so (about a minute); the harness loads it
    at run time when it exists.  Returns None where no CUTLASS headers are installed."""
    root = find_cutlass()
    if root is None:
        return None
    src = os.path.join(CSRC, "main_cutlass_column.cu")
    if not os.path.exists(src):
        return None
    os.makedirs(os.path.dirname(CUTLASS_COLUMN), exist_ok=True)
    if _stale(CUTLASS_COLUMN, [src]):
        cmd = [NVCC, "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr",
               "-diag-suppress", "20012", "-I", os.path.join(root, "include"), "-I", os.path.join(root, "tools", "util", "include"),
               "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared", "-o", CUTLASS_COLUMN, src]
        subprocess.run(cmd, check=True)
    return CUTLASS_COLUMN


def build_harness() -> str:
    """Link the C++ benchmark/correctness harness (csrc/main_gemm.cpp) against the library and cuBLAS."""
    build()
    exe = os.path.join(HERE, "bin", "gemm")
    os.makedirs(os.path.dirname(exe), exist_ok=True)
    src = os.path.join(CSRC, "main_gemm.cpp")
    if _stale(exe, [src, LIB, os.path.join(HERE, "..", "include", "gemm_sm100.h")]):
        cmd = [NVCC, "-std=c++17", "-O2", "-x", "cu", src, "-o", exe, "-L", HERE, "-lspork_b200", "-lcublas", "-ldl",
               "-Xlinker", "-rpath=$ORIGIN/.."]
        subprocess.run(cmd, check=True)
    return exe


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, checked="--checked" in sys.argv))
    if "--harness" in sys.argv:
        print(build_harness())
    if "--cutlass" in sys.argv:
        print(build_cutlass_column() or "no CUTLASS headers found: the harness runs without that column")
