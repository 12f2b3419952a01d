"""GPU parity at the sizes the benchmark runs, not at reduced ones.

The reference checks its GEMM against cp.matmul at its full size on every run
(ml/matmul/run.spi:41,54-58).  Here the oracle is a float64 product on the host, which is
affordable at these sizes only on a sample: every test below compares SAMPLED output rows (chosen
to include the first and last row and rows beyond 2^17) with the oracle on the same seeded inputs,
and adds size-independent properties over the whole output (rows of probabilities sum to one,
illegal actions are exactly zero, sign words agree with the stored activations).

Tolerances: TIGHT = 2e-5 where the inputs are exactly representable in the input class (the only
difference from the float64 oracle is fp32 accumulation order), 3e-3 where the output was rounded
once to a 16-bit storage type, TOL = 2e-3 (the benchmark's class tolerance) on probabilities and
gradients that went through several rounded layers.
"""
import numpy as np
import pytest

from oracle import spiral_oracle as so

pytestmark = pytest.mark.gpu
TOL = 2e-3
TIGHT = 2e-5
WGRAD_TOL = 1e-4      # exact inputs, but an fp32 sum of 262144 products per element (9 partial sums, then their sum)
HOLDEM = [512, 1024, 1024, 1024, 1024, 10]
LEDUC = [32, 256, 256, 256, 3]
FULL_BATCH = 262144


def sample_rows(n, count, seed):
    """`count` distinct row indices of range(n): the two ends, rows on both sides of every power of two
    from 2^16 up (tile and index-width boundaries) and random ones."""
    fixed = {0, n - 1}
    p = 1 << 16
    while p < n:
        fixed.update((p - 1, p))
        p <<= 1
    g = so.rng(seed)
    rows = set(int(r) for r in fixed if 0 <= r < n)
    while len(rows) < min(count, n):
        rows.add(int(g.integers(0, n)))
    return np.array(sorted(rows), dtype=np.int64)


def storage(in_dtype):
    return "f32" if in_dtype == "tf32" else in_dtype


def gemm_operands(seed, at, bt, m, n, k, in_dtype):
    g = so.rng(seed)
    a = so.round_input(g.standard_normal((k, m) if at else (m, k), dtype=np.float32), in_dtype)
    b = so.round_input(g.standard_normal((n, k) if bt else (k, n), dtype=np.float32), in_dtype)
    return a, b


def run_gemm(gpu, at, bt, a, b, m, n, in_dtype):
    c = gpu.DeviceArray((m, n), "f32")
    gpu.matmul(at, bt, 1.0, gpu.DeviceArray.from_numpy(a, storage(in_dtype)),
               gpu.DeviceArray.from_numpy(b, storage(in_dtype)), 0.0, c, in_dtype=in_dtype)
    return c.numpy()


LAYOUTS = {"NT": (False, True), "NN": (False, False), "TN": (True, False)}
CELLS = [(dt, name) for dt in ("bf16", "f16", "tf32") for name in ("NN", "NT", "TN")]


@pytest.mark.parametrize("in_dtype,layout", CELLS)
def test_4096_cubed_every_layout_and_class(gpu, in_dtype, layout):
    """Benchmark configuration 2: M = N = K = 4096, layouts NN / NT / TN, bf16 / fp16 / tf32 inputs, fp32
    accumulate and output; the oracle on 48 sampled output rows."""
    at, bt = LAYOUTS[layout]
    m = n = k = 4096
    a, b = gemm_operands(160 + len(in_dtype) + 3 * len(layout) + at + 2 * bt, at, bt, m, n, k, in_dtype)
    got = run_gemm(gpu, at, bt, a, b, m, n, in_dtype)
    rows = sample_rows(m, 48, 17)
    a_rows = a[:, rows] if at else a[rows]
    want = so.matmul(at, bt, 1.0, a_rows, b, 0.0, None)
    assert so.rel_frobenius(got[rows], want) <= TIGHT
    assert np.isfinite(got).all()


@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
def test_ragged_4000x3000x1000_fp16(gpu, layout):
    """Configuration 2's ragged shape in the fp16 class (bf16 and tf32 are covered by the layout sweep)."""
    at, bt = LAYOUTS[layout]
    a, b = gemm_operands(170 + at + 2 * bt, at, bt, 4000, 3000, 1000, "f16")
    got = run_gemm(gpu, at, bt, a, b, 4000, 3000, "f16")
    assert so.rel_frobenius(got, so.matmul(at, bt, 1.0, a, b, 0.0, None)) <= TIGHT


def holdem_net(gpu, batch, training, head, seed=5):
    ws, bs = so.mlp_weights(seed, HOLDEM)
    g = so.rng(seed + 100)
    bs = [(g.normal(size=b.shape) * 0.05).astype(np.float32) for b in bs]
    net = gpu.PolicyMLP(HOLDEM, batch, in_dtype="bf16", head=head, training=training)
    net.load_weights(ws, bs)
    return net, ws, bs


def test_holdem_forward_full_batch_sampled_rows(gpu):
    """Benchmark configuration 5, inference: 512-1024x4-10 at B = 262144 in bf16; the oracle on 256 sampled
    rows, head properties on all rows."""
    batch = FULL_BATCH
    net, ws, bs = holdem_net(gpu, batch, False, ("masked_softmax", "argmax"))
    x, mask = so.holdem_inputs(5, batch)
    probs = net.forward(gpu.to_storage(x, "bf16"), gpu.DeviceArray.from_numpy(mask)).numpy()
    rows = sample_rows(batch, 256, 51)
    want = so.mlp_forward(x[rows], ws, bs, mask[rows], in_dtype="bf16", act_dtype="bf16")
    assert so.rel_frobenius(probs[rows], want) <= TOL
    np.testing.assert_allclose(probs.sum(axis=1), 1.0, atol=1e-5)
    assert np.all(probs[mask == 0] == 0)
    actions = net.actions.numpy()
    np.testing.assert_array_equal(actions, np.argmax(probs, axis=1))
    top2 = np.sort(want, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 5e-3
    np.testing.assert_array_equal(actions[rows][clear], so.argmax(want)[clear])


def bits_to_bool(words, m, n):
    by_row = np.ascontiguousarray(words.view(np.uint32).reshape(n // 32, m).T)
    return np.unpackbits(by_row.view(np.uint8).reshape(m, -1), axis=1, bitorder="little").reshape(m, n).astype(bool)


def test_holdem_training_full_batch_layer_by_layer(gpu):
    """Benchmark configuration 5, training, at the batch the headline number is taken on (262144 rows:
    wgrad inner dimension 262144 with its 9-way split-K, row indices beyond 2^17).

    The backward pass is run one layer at a time so that every layer's dY can be read back; each
    GEMM of the step is then checked against the oracle's arithmetic on the device's own (already
    checked) inputs: forward activations on sampled batch rows, d logits from the probabilities,
    dgrad with its sign-bit gate on sampled batch rows, wgrad (a sum over all 262144 rows) on 16
    sampled output rows per layer, bias gradients as column sums over all rows.
    """
    batch, n_layers = FULL_BATCH, len(HOLDEM) - 1
    net, ws, bs = holdem_net(gpu, batch, True, ("masked_softmax",), seed=7)
    wr = [so.round_bf16(w) for w in ws]
    x, mask = so.holdem_inputs(7, batch)
    x = so.round_bf16(x)
    target = so.random_target(77, mask)
    dx, dm, dt = gpu.to_storage(x, "bf16"), gpu.DeviceArray.from_numpy(mask), gpu.DeviceArray.from_numpy(target)
    net.loss.fill_zero()
    net.forward(dx, dm, head_flags=8)
    rows = sample_rows(batch, 192, 71)

    # ---- forward: every layer on the sampled rows, from the device's own input of that layer ----
    acts_rows = [x[rows]]
    for i in range(n_layers - 1):
        h = net.activations[i].numpy()
        want = so.round_bf16(so.relu(so.matmul(False, True, 1.0, acts_rows[i], wr[i], 0.0, None) + bs[i]))
        assert so.rel_frobenius(h[rows], want) <= 3e-3, "activations of layer %d" % i
        bits = bits_to_bool(net.relu_bits[i].numpy(), batch, HOLDEM[i + 1])
        np.testing.assert_array_equal(bits, h > 0)          # sign words == the stored activations, all rows
        acts_rows.append(h[rows])
        del h, bits
    probs = net.probs.numpy()
    logits = so.matmul(False, True, 1.0, acts_rows[-1], wr[-1], 0.0, None) + bs[-1]
    assert so.rel_frobenius(probs[rows], so.masked_softmax(logits, mask[rows])) <= TOL
    np.testing.assert_allclose(probs.sum(axis=1), 1.0, atol=1e-5)

    # ---- backward, one layer per call ----
    dy_prev_rows = None          # the oracle's dY of the layer in hand, on the sampled rows
    out_rows = sample_rows(1024, 16, 72)
    for layer in range(n_layers - 1, -1, -1):
        net.backward_layers(dx, dm, dt, layer, layer)
        dy = net.layer_dy(layer).numpy()                       # [batch, width padded to 8], bf16 values
        width = HOLDEM[layer + 1]
        if layer == n_layers - 1:
            m = mask.astype(bool)
            tsum = np.sum(np.where(m, target, 0), axis=1, keepdims=True, dtype=np.float32)
            want_dy = np.where(m, probs * tsum - target, 0).astype(np.float32) / np.float32(batch)
            assert so.rel_frobenius(dy[:, :width], so.round_bf16(want_dy)) <= 3e-3
            assert not dy[:, width:].any()
            loss = so.cross_entropy_loss(probs, np.where(m, target, 0), m)
            assert abs(float(net.loss.numpy()[0]) - loss) <= 2e-3 * abs(loss)
        else:
            assert so.rel_frobenius(dy[rows], dy_prev_rows) <= 3e-3, "dgrad into layer %d" % layer
        grads = net.split_flat(net.grads.numpy())
        # bias gradient = column sums over all rows (taken on the device before the bf16 rounding of dY)
        db_want = dy[:, :width].sum(axis=0, dtype=np.float64)
        assert so.rel_frobenius(grads[layer][1], db_want) <= 5e-3, "db of layer %d" % layer
        # wgrad on sampled output rows: dW[r, :] = sum over the batch of dY[:, r] * H_in
        h_in_dev = dx if layer == 0 else net.activations[layer - 1]
        h_in = h_in_dev.numpy()
        r_out = np.arange(width) if width < 1024 else out_rows
        want_dw = np.zeros((len(r_out), HOLDEM[layer]), np.float64)
        for b0 in range(0, batch, 32768):
            want_dw += dy[b0:b0 + 32768][:, r_out].T.astype(np.float64) @ h_in[b0:b0 + 32768].astype(np.float64)
        assert so.rel_frobenius(grads[layer][0][r_out], want_dw) <= WGRAD_TOL, "dW of layer %d" % layer
        if layer > 0:
            gate = h_in[rows] > 0
            dy_prev_rows = so.round_bf16(np.where(gate, so.matmul(False, False, 1.0, dy[rows][:, :width], wr[layer], 0.0, None), 0))
        del dy, h_in
    assert gpu.device_status() == (0, 0)


def test_leduc_training_full_batch(gpu):
    """Benchmark configuration 4: the 32-256-256-256-3 net at B = 65536, every gradient against the oracle
    on the whole batch."""
    batch = 65536
    ws, bs = so.mlp_weights(4, LEDUC)
    g = so.rng(104)
    bs = [(g.normal(size=b.shape) * 0.05).astype(np.float32) for b in bs]
    net = gpu.PolicyMLP(LEDUC, batch, in_dtype="bf16", training=True)
    net.load_weights(ws, bs)
    x, mask = so.leduc_inputs(4, batch)
    target = so.random_target(44, mask)
    dx, dm, dt = gpu.to_storage(x, "bf16"), gpu.DeviceArray.from_numpy(mask), gpu.DeviceArray.from_numpy(target)
    net.loss.fill_zero()
    net.forward(dx, dm, head_flags=8)
    net.backward(dx, dm, dt)
    got = net.split_flat(net.grads.numpy())
    _, _, loss, want = so.mlp_train_step(x, [so.round_bf16(w) for w in ws], bs, mask, target, 0.0,
                                         in_dtype="bf16", act_dtype="bf16")
    assert abs(float(net.loss.numpy()[0]) - loss) <= 2e-3 * abs(loss)
    for i, ((gw, gb), (ww, wb)) in enumerate(zip(got, want)):
        assert so.rel_frobenius(gw, ww) <= TOL, "dW of layer %d" % i
        assert so.rel_frobenius(gb, wb) <= 5e-3, "db of layer %d" % i
