"""Our TF32 GEMM against the reference's OWN kernel on the same inputs (GPU).

oracle/_ref/ref_matmul_tf32.cubin is the reference's generated TF32 WMMA GEMM
(tests/matmul/test1_run.py: NT, alpha = beta = 1, 8192 x 8192 x 4096) recompiled for sm_100a by
oracle/build_ref.py.  Both kernels multiply in TF32 and accumulate in fp32; with inputs that are
exactly representable in TF32 the only difference is the order of the fp32 additions, so the
relative Frobenius error is asserted at 2e-5 (the class tolerance is 2e-3).
"""
import numpy as np
import pytest

from oracle import ref_kernel
from oracle import spiral_oracle as so

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not ref_kernel.available(), reason="oracle/_ref/ref_matmul_tf32.cubin was not built")
def test_matmul_tf32_matches_reference_kernel(gpu):
    m, n, k = 8192, 8192, 4096
    g = so.rng(2024)
    a = so.round_tf32(g.standard_normal((m, k), dtype=np.float32))
    b = so.round_tf32(g.standard_normal((n, k), dtype=np.float32))
    c = g.standard_normal((m, n), dtype=np.float32)
    da, db = gpu.DeviceArray.from_numpy(a), gpu.DeviceArray.from_numpy(b)
    c_ref, c_ours = gpu.DeviceArray.from_numpy(c), gpu.DeviceArray.from_numpy(c)
    ref = ref_kernel.ReferenceMatmul()
    gpu.synchronize()
    ref.launch(da.ptr, db.ptr, c_ref.ptr)
    gpu.synchronize()
    gpu.matmul_tf32(False, True, 1.0, da, db, 1.0, c_ours)
    got, want = c_ours.numpy(), c_ref.numpy()
    assert so.rel_frobenius(got, want) <= 2e-5
    rows = so.rng(7).choice(m, size=16, replace=False)           # and both agree with the float64 definition
    exact = so.matmul(False, True, 1.0, a[rows], b, 1.0, c[rows])
    assert so.rel_frobenius(want[rows], exact) <= 2e-5
    assert so.rel_frobenius(got[rows], exact) <= 2e-5
