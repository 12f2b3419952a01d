"""Builds libspiral_b200.so (hand-written sm_100a CUDA behind a C ABI) in-tree.

    python spiral-s-ml-library_b200/build.py [--force] [--verbose]

nvcc cross-compiles for sm_100a without a GPU.  The library is one translation
unit (csrc/lib.cu) linked against the static CUDA runtime, so the resulting
.so has no dependency beyond libc and the driver present at run time.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "spiral_b200", "libspiral_b200.so")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-cudart", "static",
]


def sources():
    out = [os.path.join(HERE, "..", "include", "spiral_b200.h")]
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cu", ".cuh", ".h")):
            out.append(os.path.join(CSRC, name))
    return out


def is_stale():
    if not os.path.exists(OUT):
        return True
    built = os.path.getmtime(OUT)
    return any(os.path.getmtime(s) > built for s in sources())


def build(force=False, verbose=False):
    """Compiles the library when a source is newer than the .so; returns its path."""
    if not force and not is_stale():
        return OUT
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + [
        "-o", OUT, os.path.join(CSRC, "lib.cu")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libspiral_b200.so")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
