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


@pytest.mark.parametrize("at,bt", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(256, 192, 320), (512, 512, 512), (1000, 520, 260), (4, 4, 4)])
def test_fp32_class_on_tensor_cores_all_layouts(gpu, at, bt, m, n, k):
    """Shapes whose contiguous dimensions are multiples of 4 take the 3 x TF32 tensor-core path (operands split
    into TF32 head and tail, one GEMM over the K-concatenated parts): still within 1e-5 of the float64 product."""
    a, b, c = _operands(900 + m + n + k, at, bt, m, n, k, "normal")
    dc = gpu.DeviceArray.from_numpy(c)
    l0 = gpu.launch_count()
    gpu.matmul(at, bt, 1.5, gpu.DeviceArray.from_numpy(a), gpu.DeviceArray.from_numpy(b), -0.5, dc, in_dtype="f32")
    assert gpu.launch_count() - l0 == 2                      # the split and the GEMM
    assert so.rel_frobenius(dc.numpy(), so.matmul(at, bt, 1.5, a, b, -0.5, c)) <= TOL_F32


def test_fp32_class_bias_relu_and_4096_sampled_rows(gpu):
    g = so.rng(77)
    a = g.uniform(-1, 1, size=(300, 264)).astype(np.float32)
    b = g.uniform(-1, 1, size=(128, 264)).astype(np.float32)
    bias = g.normal(size=128).astype(np.float32)
    dc = gpu.DeviceArray((300, 128), "f32")
    gpu.matmul(False, True, 1.0, gpu.DeviceArray.from_numpy(a), gpu.DeviceArray.from_numpy(b), 0.0, dc, in_dtype="f32",
               epilogue=("bias", "relu"), bias=gpu.DeviceArray.from_numpy(bias))
    assert so.rel_frobenius(dc.numpy(), so.relu(so.matmul(False, True, 1.0, a, b, 0.0, None) + bias)) <= TOL_F32
    # a large case: 4096^3, oracle on 32 sampled rows; far tighter than single-pass TF32 (about 5e-4)
    a = g.standard_normal((4096, 4096), dtype=np.float32)
    b = g.standard_normal((4096, 4096), dtype=np.float32)
    dc = gpu.DeviceArray((4096, 4096), "f32")
    gpu.matmul(False, True, 1.0, gpu.DeviceArray.from_numpy(a), gpu.DeviceArray.from_numpy(b), 0.0, dc, in_dtype="f32")
    rows = g.choice(4096, size=32, replace=False)
    err = so.rel_frobenius(dc.numpy()[rows], so.matmul(False, True, 1.0, a[rows], b, 0.0, None))
    assert err <= TOL_F32
