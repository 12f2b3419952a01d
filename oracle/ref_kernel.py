"""Loads and launches the reference's own GEMM kernel (oracle/_ref/ref_matmul_tf32.cubin).
TEST INFRASTRUCTURE ONLY -- used by tests/ and by bench.py's reference-kernel timing row.

The cubin is built by oracle/build_ref.py from the reference checkout; this module never reads
the checkout.  The kernel computes C <- A * B^T + C in place for A [8192, 4096], B [8192, 4096],
C [8192, 8192], fp32 storage, TF32 WMMA multiply (tests/matmul/test1_run.py:1015-1053: arguments
in the order a, b, c; 24 CTAs x 256 threads; 98304 bytes of dynamic shared memory).
"""
import ctypes
import os

from .build_ref import CUBIN, SHAPE


def available():
    return os.path.exists(CUBIN)


class ReferenceMatmul:
    def __init__(self):
        from cuda.bindings import driver
        self.drv = driver
        err, = driver.cuInit(0)
        self._check(err, "cuInit")
        with open(CUBIN, "rb") as f:
            image = f.read()
        err, self.module = driver.cuModuleLoadData(image)
        self._check(err, "cuModuleLoadData")
        err, self.func = driver.cuModuleGetFunction(self.module, SHAPE["entry"].encode())
        self._check(err, "cuModuleGetFunction")
        err, = driver.cuFuncSetAttribute(
            self.func, driver.CUfunction_attribute.CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, SHAPE["dyn_smem"])
        self._check(err, "cuFuncSetAttribute")

    def _check(self, err, what):
        if int(err) != 0:
            raise RuntimeError("%s failed with CUresult %d" % (what, int(err)))

    def launch(self, a_ptr, b_ptr, c_ptr):
        """Asynchronous launch on the legacy default stream with the generated file's configuration."""
        args = (ctypes.c_void_p * 3)()
        holders = [ctypes.c_void_p(int(p)) for p in (a_ptr, b_ptr, c_ptr)]
        for i, h in enumerate(holders):
            args[i] = ctypes.addressof(h)
        err, = self.drv.cuLaunchKernel(self.func, SHAPE["blocks"], 1, 1, SHAPE["threads"], 1, 1, SHAPE["dyn_smem"], 0,
                                       ctypes.addressof(args), 0)
        self._check(err, "cuLaunchKernel")
        self._keep = (args, holders)
