"""GPU parity of the fp32 (FFMA) GEMM against NumPy: relative Frobenius error <= 1e-5."""
import numpy as np
import pytest

from oracle import spiral_oracle as so

pytestmark = pytest.mark.gpu
TOL_F32 = 1e-5


def _operands(seed, at, bt, m, n, k, dist="uniform"):
    g = so.rng(seed)
    draw = (lambda s: g.uniform(-1, 1, size=s)) if dist == "uniform" else (lambda s: g.normal(size=s))
    a = draw((k, m) if at else (m, k)).astype(np.float32)
    b = draw((n, k) if bt else (k, n)).astype(np.float32)
    c = draw((m, n)).astype(np.float32)
    return a, b, c


def test_config_512_nt_fp32(gpu):
    """Benchmark configuration 1: C = A @ B.T, 512^3, uniform[-1,1), seed 1, NumPy float32 oracle."""
    a, b, c = _operands(1, False, True, 512, 512, 512)
    dc = gpu.DeviceArray((512, 512), "f32")
    gpu.matmul(False, True, 1.0, gpu.DeviceArray.from_numpy(a), gpu.DeviceArray.from_numpy(b), 0.0, dc,
               in_dtype="f32")
    got = dc.numpy()
    assert so.rel_frobenius(got, a @ b.T) <= TOL_F32
    assert so.rel_frobenius(got, so.matmul(False, True, 1.0, a, b, 0.0, None)) <= TOL_F32


@pytest.mark.parametrize("at,bt", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (65, 63, 17), (200, 130, 333)])
def test_layouts_and_ragged_shapes(gpu, at, bt, m, n, k):
    a, b, c = _operands(m * 7 + n + k, at, bt, m, n, k, "normal")
    dc = gpu.DeviceArray.from_numpy(c)
    gpu.matmul(at, bt, 1.5, gpu.DeviceArray.from_numpy(a), gpu.DeviceArray.from_numpy(b), -0.5, dc, in_dtype="f32")
    assert so.rel_frobenius(dc.numpy(), so.matmul(at, bt, 1.5, a, b, -0.5, c)) <= TOL_F32
