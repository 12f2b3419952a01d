"""The NumPy oracle against the reference's own golden console outputs (CPU only).

Fixtures: tests/golden/primitives_golden.npz, extracted by tests/golden/make_golden.py
from the reference's test_text_outputs/primitives/{test2,test3}/{a,b}.  The
printed values carry six decimals, hence the 2e-6 absolute tolerance.
"""
import os

import numpy as np
import pytest

from oracle import spiral_oracle as so

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "primitives_golden.npz"))
ATOL = 2e-6


@pytest.mark.parametrize("sub", ["a", "b"])
def test_softmax_matches_reference_output(sub):
    x = GOLD["t2%s_input" % sub]
    np.testing.assert_allclose(so.softmax(x), GOLD["t2%s_softmax" % sub], atol=ATOL, rtol=0)


@pytest.mark.parametrize("sub", ["a", "b"])
@pytest.mark.parametrize("size", [4, 11])
def test_masked_softmax_matches_reference_output(sub, size):
    x = GOLD["t2%s_input" % sub]
    got = so.masked_softmax(x, so.prefix_mask(x.shape, size))
    np.testing.assert_allclose(got, GOLD["t2%s_masked_softmax%d" % (sub, size)], atol=ATOL, rtol=0)
    assert np.all(got[:, size:] == 0)


@pytest.mark.parametrize("sub", ["a", "b"])
def test_ln_l2_matches_reference_output(sub):
    x = GOLD["t2%s_input" % sub]
    np.testing.assert_allclose(so.ln_l2(x), GOLD["t2%s_ln_l2" % sub], atol=ATOL, rtol=0)


@pytest.mark.parametrize("sub", ["a", "b"])
def test_argmax_matches_reference_output(sub):
    x = GOLD["t2%s_input" % sub]
    want = GOLD["t2%s_argmax" % sub][: x.shape[0]]
    # the printed inputs are rounded to 6 decimals; only rows with a clear winner are decisive
    top2 = np.sort(x, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 2e-6
    assert clear.sum() >= x.shape[0] - 1
    np.testing.assert_array_equal(so.argmax(x)[clear], want[clear])


@pytest.mark.parametrize("sub", ["a", "b"])
def test_masked_regret_matching_matches_reference_output(sub):
    x = GOLD["t3%s_input" % sub]
    got = so.masked_regret_matching(x, so.prefix_mask(x.shape, 3))
    np.testing.assert_allclose(got, GOLD["t3%s_masked_regret3" % sub], atol=ATOL, rtol=0)


def test_regret_matching_uniform_when_nothing_positive():
    x = -np.abs(np.random.default_rng(0).normal(size=(5, 7))).astype(np.float32)
    mask = np.zeros((5, 7), bool)
    mask[:, [1, 4, 5]] = True
    got = so.masked_regret_matching(x, mask)
    np.testing.assert_allclose(got[:, [1, 4, 5]], 1 / 3, rtol=1e-6)
    assert np.all(got[:, [0, 2, 3, 6]] == 0)


def test_max_and_mean_subtraction_agree():
    x = np.random.default_rng(1).normal(size=(64, 10)).astype(np.float32)
    mask = np.random.default_rng(2).random((64, 10)) < 0.6
    mask[:, 0] = True
    ref = so.masked_softmax(x, mask)
    xm = np.where(mask, x, -np.inf)
    e = np.exp(xm - xm.max(axis=1, keepdims=True))
    alt = e / e.sum(axis=1, keepdims=True)
    np.testing.assert_allclose(ref, alt, atol=1e-6)


def test_matmul_layout_flags():
    g = np.random.default_rng(3)
    a = g.normal(size=(5, 7)).astype(np.float32)
    b = g.normal(size=(7, 3)).astype(np.float32)
    c = g.normal(size=(5, 3)).astype(np.float32)
    want = 2 * a.astype(np.float64) @ b.astype(np.float64) + 0.5 * c
    for at in (False, True):
        for bt in (False, True):
            aa = np.ascontiguousarray(a.T) if at else a
            bb = np.ascontiguousarray(b.T) if bt else b
            np.testing.assert_allclose(so.matmul(at, bt, 2.0, aa, bb, 0.5, c), want, rtol=1e-6)


def test_input_rounding_classes():
    x = np.float32([1.0 + 2 ** -9, 1.0 + 2 ** -12, 3.14159265])
    assert so.round_bf16(x)[0] in (np.float32(1.0), np.float32(1.0 + 2 ** -7))
    assert so.round_tf32(x)[1] == np.float32(1.0)
    assert abs(so.round_tf32(x)[2] - x[2]) <= 2 ** -10
    assert so.round_f16(x)[2] == np.float32(np.float16(x[2]))


def test_train_step_gradient_matches_finite_difference():
    sizes = [6, 8, 4]
    ws, bs = so.mlp_weights(5, sizes)
    g = so.rng(6)
    x = g.normal(size=(16, 6)).astype(np.float32)
    mask = np.ones((16, 4), np.uint8)
    mask[::2, 3] = 0
    tgt = so.random_target(7, mask)
    _, _, loss, grads = so.mlp_train_step(x, ws, bs, mask, tgt, 0.0)
    eps = 1e-3
    for (li, i, j) in [(0, 2, 3), (1, 1, 5), (1, 3, 0)]:
        wp = [w.copy() for w in ws]
        wp[li][i, j] += eps
        lp = so.cross_entropy_loss(so.mlp_forward(x, wp, bs, mask), tgt, mask)
        wm = [w.copy() for w in ws]
        wm[li][i, j] -= eps
        lm = so.cross_entropy_loss(so.mlp_forward(x, wm, bs, mask), tgt, mask)
        assert abs((lp - lm) / (2 * eps) - grads[li][0][i, j]) < 2e-3


def test_state_encoder_matches_the_dense_generators():
    """encode_states follows the bounded-int pickler (corebase/pickler.spi:20-37): one feature set per
    field, none for the out-of-range value; the dense generators are its image of the compact ones."""
    fields, dense, mask = so.holdem_states(11, 257)
    x, mask2 = so.holdem_inputs(11, 257)
    assert x.shape == (257, 512) and np.array_equal(mask, mask2)
    cards = x[:, :119].reshape(257, 7, 17)
    live = fields[:, 0::2] < 4
    assert np.array_equal(cards[:, :, :4].sum(axis=2) == 1, live)        # suit groups
    assert np.array_equal(cards[:, :, 4:].sum(axis=2) == 1, live)        # rank groups
    assert np.array_equal(np.argmax(cards[:, :, 4:], axis=2)[live], fields[:, 1::2][live])
    assert np.array_equal(x[:, 119:], dense)
    assert set(np.sum(live, axis=1)) <= {2, 5, 6, 7}
    f2, m2 = so.leduc_states(12, 100)
    x2, _ = so.leduc_inputs(12, 100)
    assert x2.shape == (100, 32) and np.all(x2[:, :24].reshape(100, -1).sum(axis=1) == 4)
    assert np.array_equal(x2[:, 24:], (f2[:, 4:] == 0).astype(np.float32))
    tiny = so.encode_states(np.array([[1, 2], [3, 0]], np.uint8), (3, 2), np.array([[0.5], [0.25]], np.float32))
    assert np.array_equal(tiny, np.array([[0, 1, 0, 0, 0, 0.5], [0, 0, 0, 1, 0, 0.25]], np.float32))


def test_discrete_sampling_oracle_follows_the_distribution():
    """The sampling oracle (ml/primitives.spi:782-800) draws index j with probability x[j] / sum(x) and
    never a zero-weight entry."""
    p = np.array([0.1, 0.0, 0.6, 0.3, 0.0], np.float32)
    g = so.rng(9)
    n = 200000
    u = (1.0 - g.random(n, dtype=np.float32)).astype(np.float32)
    idx = so.discrete_sampling(np.tile(p, (n, 1)), u)
    freq = np.bincount(idx, minlength=5) / n
    assert freq[1] == 0 and freq[4] == 0
    np.testing.assert_allclose(freq, p, atol=5e-3)
    assert so.discrete_sampling(np.zeros((1, 4), np.float32), np.ones(1, np.float32))[0] == -1
    assert so.discrete_sampling(p[None] * 3.0, np.array([1.0], np.float32))[0] == 3      # unnormalised weights, u = 1


def test_binarize_oracle():
    x = np.array([[1.0, -1.0, 0.0, 2.0], [0.0, 0.0, 0.0, 0.0], [5.0, 5.0, 5.0, 5.0]], np.float32)
    np.testing.assert_array_equal(so.binarize(x, 1 << 20), np.array([0b1001, 0, 0b1111], np.uint32))
    np.testing.assert_array_equal(so.binarize(x, 7), np.array([9 % 7, 0, 15 % 7], np.uint32))


def test_philox4x32_10_known_answers():
    """The oracle's Philox4x32-10 against the known-answer vectors published with the algorithm
    (Salmon et al., SC 2011: counter and key all zero, all ones, and the digits of pi)."""
    cases = [
        ([0, 0, 0, 0], [0, 0], [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]),
        ([0xffffffff] * 4, [0xffffffff] * 2, [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]),
        ([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0],
         [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]),
    ]
    for counter, key, want in cases:
        got = [int(w) for w in so.philox4x32_10(counter, key)]
        assert got == want


def test_philox_stream_layout_and_uniform_range():
    """Output n of a stream is word n % 4 of block n // 4; uniforms lie in (0, 1] (2^-33 for a zero draw,
    exactly 1 for the largest); the bounded draw is below its bound."""
    sub = np.arange(7, dtype=np.uint64) + np.uint64(2 ** 33)
    block1 = so.philox4x32_10([1, 0, sub & np.uint64(0xFFFFFFFF), sub >> np.uint64(32)], [99, 5])
    for w in range(4):
        np.testing.assert_array_equal(so.philox_u32(99 + (5 << 32), sub, 4 + w), block1[w])
    assert so.uniform_open_closed(np.uint32(0)) == np.float32(2.0 ** -33)
    assert so.uniform_open_closed(np.uint32(0xFFFFFFFF)) == np.float32(1.0)
    below = so.philox_below(1, np.arange(1000), 0, 7)
    assert below.min() >= 0 and below.max() < 7 and len(np.unique(below)) == 7


def test_discrete_sampling_picks_by_the_cumulative_distribution():
    p = np.array([[0.0, 0.25, 0.0, 0.5, 0.25, 0.0]], np.float32)
    for u, want in ((1e-6, 1), (0.25, 1), (0.2500001, 3), (0.75, 3), (0.76, 4), (1.0, 4)):
        assert so.discrete_sampling(p, np.array([u], np.float32))[0] == want
    assert so.discrete_sampling(np.zeros((1, 4), np.float32), np.array([0.5], np.float32))[0] == -1
