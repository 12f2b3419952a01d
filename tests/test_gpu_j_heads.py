"""Row heads fused into the GEMM at the reference's own widths, and the device random stream.

The reference's policy nets end in 64 (or `inner` = 128) columns of which the first few are legal
(game/leduc/model_cem.spi:37,52-60: `masked_regret_matching' 3` over 64 columns;
game/leduc/tests/train.spi:88-101: `masked_softmax_and_discrete_sample' 3` over 128 columns) and
put `ln_l2` between every matmul and relu (ml/layers.spi:562-568).  Checked here: the head
arithmetic against the oracle (ml/primitives.spi:748-800), the sampled index bit for bit against
the oracle's restatement of the same Philox4x32-10 stream, the sign hash bit for bit, and that each
case is ONE kernel launch with no mask matrix.
"""
import numpy as np
import pytest

from oracle import spiral_oracle as so

pytestmark = pytest.mark.gpu
TOL = 2e-3
TIGHT = 2e-5


def operands(seed, m, n, k):
    g = so.rng(seed)
    a = so.round_tf32(g.normal(size=(m, k)).astype(np.float32) * np.float32(0.2))
    b = so.round_tf32(g.normal(size=(n, k)).astype(np.float32))
    return a, b


def test_philox_uniform_matches_the_oracle_stream(gpu):
    out = gpu.DeviceArray((5000,), "f32")
    for seed, row_offset, position in ((0, 0, 0), (12344321, 7, 3), (2 ** 63 + 5, 2 ** 40, 2 ** 34 + 1)):
        gpu.primitives.philox_uniform(out, seed, row_offset, position)
        want = so.philox_uniform(seed, np.uint64(row_offset) + np.arange(5000, dtype=np.uint64), position)
        np.testing.assert_array_equal(out.numpy(), want)
    u = out.numpy()
    assert u.min() > 0.0 and u.max() <= 1.0


@pytest.mark.parametrize("n,prefix", [(48, -1), (64, -1), (64, 3), (128, 3), (128, 11), (256, 64), (40, 17), (300, 5), (300, -1)])
@pytest.mark.parametrize("heads", [("masked_softmax",), ("regret_matching",), ("masked_softmax", "regret_matching")])
def test_wide_and_prefix_heads_with_sampling(gpu, n, prefix, heads):
    m, k = 333, 128
    a, b = operands(300 + n + prefix, m, n, k)
    if prefix >= 0:
        mask_host, mask_dev = so.prefix_mask((m, n), prefix), None
    else:
        mask_host = (so.rng(23).random((m, n)) < 0.6)
        mask_host[:, 0] = True
        mask_dev = gpu.DeviceArray.from_numpy(mask_host.astype(np.uint8))
    idx, smp = gpu.DeviceArray((m,), "i32"), gpu.DeviceArray((m,), "i32")
    c = gpu.DeviceArray((m, n), "f32")
    spec = gpu.head_spec(heads + ("argmax", "sample"), prefix=prefix, mask=mask_dev, argmax_out=idx, sample_out=smp,
                         seed=99, row_offset=1000, position=2)
    l0 = gpu.launch_count()
    gpu.matmul_head(False, True, 1.0, gpu.DeviceArray.from_numpy(a), gpu.DeviceArray.from_numpy(b), 0.0, c, spec,
                    in_dtype="tf32")
    fused = n <= 64 or (n <= 256 and 0 <= prefix <= 64)
    assert (gpu.launch_count() - l0 == 1) == fused
    got = c.numpy()
    want = so.matmul(False, True, 1.0, a, b, 0.0, None)
    if "masked_softmax" in heads:
        want = so.masked_softmax(want, mask_host)
    if "regret_matching" in heads:
        want = so.masked_regret_matching(want, mask_host)
    np.testing.assert_allclose(got, want, atol=2e-5)
    assert np.all(got[~mask_host] == 0)
    np.testing.assert_array_equal(idx.numpy(), np.argmax(got, axis=1))
    u = so.philox_uniform(99, 1000 + np.arange(m), 2)
    picked = smp.numpy()
    np.testing.assert_array_equal(picked, so.discrete_sampling(got, u))       # bit-exact on the device's own row
    assert np.all(mask_host[np.arange(m), picked])                            # only legal actions are drawn


def test_sampling_frequencies_follow_the_probabilities(gpu):
    """Many rows with the same logits: the sampled indices follow the row's probabilities."""
    m, n, k = 65536, 64, 32
    g = so.rng(5)
    a = np.tile(so.round_tf32(g.normal(size=(1, k)).astype(np.float32)), (m, 1))
    b = so.round_tf32(g.normal(size=(n, k)).astype(np.float32) * np.float32(0.3))
    smp = gpu.DeviceArray((m,), "i32")
    c = gpu.DeviceArray((m, n), "f32")
    spec = gpu.head_spec(("masked_softmax", "sample"), prefix=5, sample_out=smp, seed=2024)
    gpu.matmul_head(False, True, 1.0, gpu.DeviceArray.from_numpy(a), gpu.DeviceArray.from_numpy(b), 0.0, c, spec, in_dtype="tf32")
    probs = c.numpy()[0]
    freq = np.bincount(smp.numpy(), minlength=n) / m
    np.testing.assert_allclose(freq, probs, atol=4 * np.sqrt(0.25 / m) + 1e-6)
    assert freq[5:].sum() == 0


@pytest.mark.parametrize("n", [8, 24, 32])
def test_sign_hash_head(gpu, n):
    m, k = 300, 64
    a, b = operands(400 + n, m, n, k)
    hashes = gpu.DeviceArray((m,), "i32")
    c = gpu.DeviceArray((m, n), "f32")
    spec = gpu.head_spec(("binarize",), hash_out=hashes, modulo=1000003)
    l0 = gpu.launch_count()
    gpu.matmul_head(False, True, 1.0, gpu.DeviceArray.from_numpy(a), gpu.DeviceArray.from_numpy(b), 0.0, c, spec, in_dtype="tf32")
    assert gpu.launch_count() - l0 == 1
    logits = c.numpy()
    assert so.rel_frobenius(logits, so.matmul(False, True, 1.0, a, b, 0.0, None)) <= TIGHT
    np.testing.assert_array_equal(hashes.numpy().view(np.uint32), so.binarize(logits, 1000003))


@pytest.mark.parametrize("n,out_dtype,in_dtype", [(64, "f32", "tf32"), (128, "f32", "tf32"), (256, "tf32", "tf32"),
                                                  (128, "bf16", "bf16"), (64, "f16", "f16")])
def test_row_normalisation_epilogue(gpu, n, out_dtype, in_dtype):
    """matmul -> ln_l2 -> relu in one launch (x / sum(x^2) over the row, ml/primitives.spi:701-703)."""
    m, k = 1000, 128
    g = so.rng(500 + n)
    a = so.round_input(g.normal(size=(m, k)).astype(np.float32) * np.float32(0.2), in_dtype)
    b = so.round_input(g.normal(size=(n, k)).astype(np.float32), in_dtype)
    st = "f32" if in_dtype == "tf32" else in_dtype
    c = gpu.DeviceArray((m, n), out_dtype)
    l0 = gpu.launch_count()
    gpu.matmul(False, True, 1.0, gpu.DeviceArray.from_numpy(a, st), gpu.DeviceArray.from_numpy(b, st), 0.0, c,
               in_dtype=in_dtype, epilogue=("ln_l2", "relu"))
    assert gpu.launch_count() - l0 == 1
    want = so.relu(so.ln_l2(so.matmul(False, True, 1.0, a, b, 0.0, None)))
    if out_dtype == "f32":
        assert so.rel_frobenius(c.numpy(), want) <= TIGHT
    else:
        assert so.rel_frobenius(c.numpy(), so.round_input(want, out_dtype)) <= 3e-3
    with pytest.raises(gpu.SpiralError):            # the tile must span the row
        gpu.matmul(False, True, 1.0, gpu.DeviceArray((8, 64), st), gpu.DeviceArray((512, 64), st), 0.0,
                   gpu.DeviceArray((8, 512), out_dtype), in_dtype=in_dtype, epilogue=("ln_l2",))


def test_reference_test_net_runs_in_three_launches(gpu):
    """The reference's test net (ml/layers.spi:594-608; game/leduc/tests/train.spi:88-101): three dense layers
    with ln_l2 + relu between them and a prefix-masked softmax + sampling head, every member of an ensemble:
    one launch per layer, nothing allocated, output against the oracle."""
    L = gpu.layers
    members, width, rows, size = 4, 128, 512, 3
    g = L.masked_softmax_and_discrete_sample(size, L.matmul_ensemble((members, width, width), L.relu(L.ln_l2(
        L.matmul_ensemble((members, width, width), L.relu(L.ln_l2(L.matmul_ensemble((members, width, width),
                          L.input("input", (2, rows // 2, width))))))))))
    model = L.pass_init(L.create_model(g))
    x = so.round_tf32(so.rng(48).normal(size=(rows, width)).astype(np.float32))
    L.key_extract(model, "input").upload(x)
    gpu.synchronize()
    free_before = gpu.mem_info()[0]
    for e in range(members):
        l0 = gpu.launch_count()
        idx = L.graph_run_host(model, ensemble=e, seed=11, row_offset=5000)
        assert gpu.launch_count() - l0 == 3
        gpu.synchronize()
        assert gpu.mem_info()[0] == free_before                  # no allocation per call
        idx = idx.numpy().copy()
        probs = model.tensor(model.nodes[-2]).numpy()
        ws = [so.round_tf32(w) for w in L.get_weights(model, e)]
        h = x
        for w in ws[:-1]:
            h = so.relu(so.ln_l2(so.matmul(False, True, 1.0, h, w, 0.0, None, in_dtype="tf32")))
        want = so.masked_softmax(so.matmul(False, True, 1.0, h, ws[-1], 0.0, None, in_dtype="tf32"),
                                 so.prefix_mask((rows, width), size))
        assert so.rel_frobenius(probs, want) <= TOL
        assert np.all(probs[:, size:] == 0)
        u = so.philox_uniform(11, 5000 + np.arange(rows), e)
        np.testing.assert_array_equal(idx, so.discrete_sampling(probs, u))
        assert idx.min() >= 0 and idx.max() < size
