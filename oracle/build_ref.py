"""Builds the reference's own GEMM kernel for sm_100a into oracle/_ref/.  TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref.py [<reference checkout>]

The checkout is named by the argument, else by the environment variable SPIRAL_REFERENCE_ROOT, else a
directory called `reference` beside this repository is tried.

The reference has no CPU implementation of this path and no hand-written CUDA: its kernels are
Spiral-generated CUDA C++ embedded as a string in generated Python files, compiled at run time by
CuPy.  The grid-level TF32 WMMA GEMM of tests/matmul/test1_run.py (NT layout, alpha = beta = 1,
shape baked to 8192 x 8192 x 4096, 24 CTAs x 256 threads, 96 KB dynamic shared memory) compiles
unchanged with nvcc for sm_100a.  This script reads that string where it lies in the reference
checkout, compiles it with the reference's own options (corecuda/base.spi:56-81) and keeps only the
binary: oracle/_ref/ref_matmul_tf32.cubin (git-ignored; it travels to the GPU box).  No reference
source is copied into this repository -- the kernel text only passes through a temporary file.
"""
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
CUBIN = os.path.join(OUT_DIR, "ref_matmul_tf32.cubin")
GENERATED = os.path.join("tests", "matmul", "test1_run.py")
# launch facts baked into the generated file (tests/matmul/test1_run.py:1050-1053)
SHAPE = {"m": 8192, "n": 8192, "k": 4096, "blocks": 24, "threads": 256, "dyn_smem": 98304, "entry": "entry0"}
NVCC_OPTIONS = ["-std=c++20", "-DNDEBUG", "--restrict", "--maxrregcount=255", "-D__CUDA_NO_HALF_CONVERSIONS__",
                "--diag-suppress=550,20012,68,39,177"]


def default_ref_root():
    env = os.environ.get("SPIRAL_REFERENCE_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref_root=None, force=False):
    """Returns the cubin path, or None when the reference checkout is absent (the GPU box)."""
    if ref_root is None:
        ref_root = default_ref_root()
    src_py = os.path.join(ref_root, GENERATED)
    if not os.path.exists(src_py):
        return CUBIN if os.path.exists(CUBIN) else None
    if os.path.exists(CUBIN) and not force and os.path.getmtime(CUBIN) >= os.path.getmtime(src_py):
        return CUBIN
    text = open(src_py).read()
    kernel = text.split('kernel = r"""', 1)[1].split('\n"""', 1)[0]
    os.makedirs(OUT_DIR, exist_ok=True)
    tmp = tempfile.mkdtemp(prefix="sb_ref_")
    try:
        cu = os.path.join(tmp, "kernel.cu")
        with open(cu, "w") as f:
            f.write(kernel)
        cmd = [os.environ.get("NVCC", "nvcc"), "-gencode", "arch=compute_100a,code=sm_100a", "-cubin"] + \
            NVCC_OPTIONS + ["-o", CUBIN, cu]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("nvcc failed on the reference kernel")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    return CUBIN


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, force=True))
