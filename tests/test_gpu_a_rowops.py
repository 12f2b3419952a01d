"""GPU parity of the stand-alone row / elementwise kernels against the oracle and the
reference's golden outputs.  Tolerance: 2e-6 absolute against the six-decimal golden
prints, 1e-6 absolute against the fp32 oracle (probabilities in [0, 1])."""
import os

import numpy as np
import pytest

from oracle import spiral_oracle as so

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "primitives_golden.npz"))


def _dev(gpu, a, dtype=None):
    return gpu.DeviceArray.from_numpy(a, dtype)


@pytest.mark.parametrize("sub", ["a", "b"])
def test_golden_row_ops(gpu, sub):
    P = gpu.primitives
    x = GOLD["t2%s_input" % sub]
    dx = _dev(gpu, x)
    out = gpu.DeviceArray(x.shape, "f32")
    np.testing.assert_allclose(P.softmax(dx, out).numpy(), GOLD["t2%s_softmax" % sub], atol=2e-6, rtol=0)
    np.testing.assert_allclose(P.masked_softmax(4, dx, out).numpy(), GOLD["t2%s_masked_softmax4" % sub], atol=2e-6, rtol=0)
    np.testing.assert_allclose(P.masked_softmax(11, dx, out).numpy(), GOLD["t2%s_masked_softmax11" % sub], atol=2e-6, rtol=0)
    np.testing.assert_allclose(P.ln_l2(dx, out).numpy(), GOLD["t2%s_ln_l2" % sub], atol=2e-6, rtol=0)
    idx = gpu.DeviceArray((x.shape[0],), "i32")
    np.testing.assert_array_equal(P.argmax(dx, idx).numpy(), so.argmax(x))
    x3 = GOLD["t3%s_input" % sub]
    out3 = gpu.DeviceArray(x3.shape, "f32")
    np.testing.assert_allclose(P.masked_regret_matching(3, _dev(gpu, x3), out3).numpy(),
                               GOLD["t3%s_masked_regret3" % sub], atol=2e-6, rtol=0)


@pytest.mark.parametrize("rows,cols", [(1, 1), (7, 3), (33, 10), (256, 128), (5, 1000)])
def test_row_ops_against_oracle(gpu, rows, cols):
    P = gpu.primitives
    g = so.rng(rows * 1000 + cols)
    x = g.normal(size=(rows, cols)).astype(np.float32) * 3
    mask = (g.random((rows, cols)) < 0.6).astype(np.uint8)
    mask[:, 0] = 1
    dx, dm = _dev(gpu, x), _dev(gpu, mask)
    out = gpu.DeviceArray(x.shape, "f32")
    np.testing.assert_allclose(P.softmax(dx, out, mask=dm).numpy(), so.masked_softmax(x, mask), atol=1e-6)
    np.testing.assert_allclose(P.regret_matching(dx, out, mask=dm).numpy(), so.masked_regret_matching(x, mask), atol=1e-6)
    np.testing.assert_allclose(P.regret_matching(dx, out).numpy(), so.regret_matching(x), atol=1e-6)
    neg = -np.abs(x)
    np.testing.assert_allclose(P.regret_matching(_dev(gpu, neg), out, mask=dm).numpy(),
                               so.masked_regret_matching(neg, mask), atol=1e-6)
    np.testing.assert_array_equal(P.relu(dx, out).numpy(), so.relu(x))
    idx = gpu.DeviceArray((rows,), "i32")
    np.testing.assert_array_equal(P.argmax(dx, idx).numpy(), so.argmax(x))


def test_argmax_ties_take_lowest_index(gpu):
    x = np.zeros((4, 40), np.float32)
    x[1, [5, 37]] = 2.0
    x[2, [33, 34]] = 1.0
    idx = gpu.DeviceArray((4,), "i32")
    np.testing.assert_array_equal(gpu.primitives.argmax(_dev(gpu, x), idx).numpy(), [0, 5, 33, 0])


def test_in_place_and_empty(gpu):
    P = gpu.primitives
    x = so.rng(9).normal(size=(64, 10)).astype(np.float32)
    dx = _dev(gpu, x)
    np.testing.assert_allclose(P.softmax(dx).numpy(), so.softmax(x), atol=1e-6)
    empty = gpu.DeviceArray((0, 10), "f32")
    P.softmax(empty)
    P.relu(empty)


def test_convert_rounding_matches_host(gpu):
    from spiral_b200 import dtypes
    x = (so.rng(10).normal(size=4099) * 10).astype(np.float32)
    dx = _dev(gpu, x)
    for tag, rounder in (("bf16", dtypes.round_bf16), ("f16", dtypes.round_f16), ("tf32", dtypes.round_tf32)):
        out = gpu.DeviceArray(x.shape, tag)
        got = gpu.primitives.convert(dx, out).numpy()
        np.testing.assert_array_equal(got, rounder(x))


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
def test_encode_states_holdem_and_leduc_bit_exact(gpu, dtype):
    """The device encoder writes exactly the dense input the oracle builds from the same compact
    states: one-hot groups with "none" values, then the dense columns unchanged (bit-exact)."""
    P = gpu.primitives
    fields, dense, _ = so.holdem_states(7, 3001)            # ragged row count
    dense = so.round_input(dense, dtype) if dtype != "f32" else dense
    want = so.encode_states(fields, so.HOLDEM_WIDTHS, dense)
    out = gpu.DeviceArray((3001, 512), dtype)
    P.encode_states(_dev(gpu, fields), so.HOLDEM_WIDTHS, _dev(gpu, dense, dtype), out)
    np.testing.assert_array_equal(out.numpy(), want)
    assert np.array_equal(want, so.holdem_inputs(7, 3001)[0]) or dtype != "f32"
    fields, _ = so.leduc_states(8, 1000)
    out = gpu.DeviceArray((1000, 32), dtype)
    P.encode_states(_dev(gpu, fields), so.LEDUC_WIDTHS, None, out)
    np.testing.assert_array_equal(out.numpy(), so.leduc_inputs(8, 1000)[0])


def test_encode_states_edge_cases(gpu):
    P = gpu.primitives
    # a row width that is not a multiple of the 16-byte store (scalar path), values above the width
    fields = np.array([[0, 5], [2, 1], [3, 0], [255, 2]], dtype=np.uint8)
    dense = so.rng(3).random((4, 3), dtype=np.float32)
    out = gpu.DeviceArray((4, 3 + 3 + 3), "f32")
    P.encode_states(_dev(gpu, fields), (3, 3), _dev(gpu, dense), out)
    np.testing.assert_array_equal(out.numpy(), so.encode_states(fields, (3, 3), dense))
    # no rows: nothing is launched
    P.encode_states(gpu.DeviceArray((0, 2), "u8"), (3, 3), gpu.DeviceArray((0, 3), "f32"), gpu.DeviceArray((0, 9), "f32"))
    with pytest.raises(ValueError):
        P.encode_states(_dev(gpu, fields), (3, 3), _dev(gpu, dense), gpu.DeviceArray((4, 10), "f32"))
    with pytest.raises(gpu.SpiralError):
        P.encode_states(_dev(gpu, fields), (3, 300), None, gpu.DeviceArray((4, 303), "f32"))


def test_encode_states_wide_dense_rows_and_many_rows(gpu):
    """More than one CTA pass over the rows, a row count that is not a multiple of the 32-row group,
    fp32 dense rows wide enough to need the shared-memory opt-in, and a misaligned dense base."""
    P = gpu.primitives
    rows, n_dense = 148 * 16 * 32 + 45, 24
    g = so.rng(5)
    fields = g.integers(0, 5, size=(rows, 3)).astype(np.uint8)
    dense = g.random((rows, n_dense), dtype=np.float32)
    out = gpu.DeviceArray((rows, 4 + 4 + 4 + n_dense), "f32")
    P.encode_states(_dev(gpu, fields), (4, 4, 4), _dev(gpu, dense), out)
    np.testing.assert_array_equal(out.numpy(), so.encode_states(fields, (4, 4, 4), dense))
    rows, n_dense = 70, 500                                       # 32 x 500 x 4 B = 64000 B of shared memory
    fields = g.integers(0, 3, size=(rows, 1)).astype(np.uint8)
    dense = g.random((rows, n_dense), dtype=np.float32)
    out = gpu.DeviceArray((rows, 2 + n_dense), "f32")
    P.encode_states(_dev(gpu, fields), (2,), _dev(gpu, dense), out)
    np.testing.assert_array_equal(out.numpy(), so.encode_states(fields, (2,), dense))
    whole = gpu.DeviceArray.from_numpy(np.concatenate([np.zeros(1, np.float32), dense.ravel()]))
    shifted = whole.view((rows, n_dense), "f32", 4)               # dense base 4 bytes off a 16-byte boundary
    P.encode_states(_dev(gpu, fields), (2,), shifted, out)
    np.testing.assert_array_equal(out.numpy(), so.encode_states(fields, (2,), dense))


@pytest.mark.parametrize("rows,cols", [(1000, 3), (4097, 10), (64, 64)])
def test_discrete_sampling_matches_oracle(gpu, rows, cols):
    """sb_row_sample is a pure function of (row, u): bit-exact against the oracle, including masked
    (zero) entries, rows of zeros and u = 1."""
    g = so.rng(60 + cols)
    mask = g.random((rows, cols)) < 0.7
    mask[:, 0] |= ~mask.any(axis=1)
    probs = so.masked_softmax(g.normal(size=(rows, cols)).astype(np.float32), mask.astype(np.uint8))
    probs[5] = 0.0                                        # a row without a positive entry
    u = (1.0 - g.random(rows, dtype=np.float32)).astype(np.float32)     # (0, 1]
    u[7] = 1.0
    out = gpu.DeviceArray((rows,), "i32")
    gpu.primitives.sample(_dev(gpu, probs), _dev(gpu, u), out)
    got = out.numpy()
    np.testing.assert_array_equal(got, so.discrete_sampling(probs, u))
    assert got[5] == -1
    picked = got[got >= 0]
    assert np.all(probs[got >= 0, picked] > 0)            # never an illegal (zero-weight) action


@pytest.mark.parametrize("cols,modulo", [(8, 256), (20, 1000003), (32, 4294967295)])
def test_binarize_row_hash(gpu, cols, modulo):
    x = so.rng(70 + cols).normal(size=(777, cols)).astype(np.float32)
    x[3] = 0.0
    out = gpu.DeviceArray((777,), "i32")
    gpu.primitives.binarize(modulo, _dev(gpu, x), out)
    np.testing.assert_array_equal(out.numpy().view(np.uint32), so.binarize(x, modulo))
    with pytest.raises(gpu.SpiralError):
        gpu.primitives.binarize(7, gpu.DeviceArray((4, 33), "f32"), gpu.DeviceArray((4,), "i32"))
