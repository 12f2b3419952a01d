"""GPU parity of the dense policy network (forward, backward, SGD) against the oracle.

The oracle rounds weights, inputs and hidden activations at the same points as the
CUDA path (storage type of the arithmetic class), so forward probabilities agree
to accumulation order; the benchmark's tolerance for the tf32 / bf16 / fp16 classes
(2e-3 relative Frobenius error) is asserted on probabilities and on every gradient.
"""
import numpy as np
import pytest

from oracle import spiral_oracle as so

pytestmark = pytest.mark.gpu
TOL = 2e-3


def build(gpu, sizes, batch, in_dtype, seed, head=("masked_softmax",), training=False, bias_scale=0.0):
    ws, bs = so.mlp_weights(seed, sizes)
    if bias_scale:
        g = so.rng(seed + 100)
        bs = [(g.normal(size=b.shape) * bias_scale).astype(np.float32) for b in bs]
    net = gpu.PolicyMLP(sizes, batch, in_dtype=in_dtype, head=head, training=training)
    net.load_weights(ws, bs)
    return net, ws, bs


@pytest.mark.parametrize("in_dtype", ["tf32", "f16", "bf16"])
def test_leduc_forward(gpu, in_dtype):
    """Benchmark configuration 3 shape (32-256-256-256-3, masked softmax then regret matching) at B=2048."""
    sizes, batch = [32, 256, 256, 256, 3], 2048
    net, ws, bs = build(gpu, sizes, batch, in_dtype, 3, head=("masked_softmax", "regret_matching", "argmax"))
    x, mask = so.leduc_inputs(3, batch)
    probs = net.forward(gpu.to_storage(x, in_dtype), gpu.DeviceArray.from_numpy(mask)).numpy()
    want = so.mlp_forward(x, ws, bs, mask, in_dtype=in_dtype, act_dtype=in_dtype,
                          head=("masked_softmax", "regret_matching"))
    assert so.rel_frobenius(probs, want) <= TOL
    assert np.all(probs[mask == 0] == 0)
    np.testing.assert_allclose(probs.sum(1), 1.0, atol=1e-5)
    actions = net.actions.numpy()
    np.testing.assert_array_equal(actions, np.argmax(probs, axis=1))
    top2 = np.sort(want, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 5e-3
    np.testing.assert_array_equal(actions[clear], so.argmax(want)[clear])
    # against the un-rounded fp32 network the class tolerance still holds for fp16 / tf32
    if in_dtype != "bf16":
        full = so.mlp_forward(x, ws, bs, mask, head=("masked_softmax", "regret_matching"))
        assert so.rel_frobenius(probs, full) <= TOL


def test_holdem_forward_bf16(gpu):
    """Benchmark configuration 5 shape (512-1024x4-10, 10-way masked softmax) at B=1024."""
    sizes, batch = [512, 1024, 1024, 1024, 1024, 10], 1024
    net, ws, bs = build(gpu, sizes, batch, "bf16", 5)
    x, mask = so.holdem_inputs(5, batch)
    probs = net.forward(gpu.to_storage(x, "bf16"), gpu.DeviceArray.from_numpy(mask)).numpy()
    want = so.mlp_forward(x, ws, bs, mask, in_dtype="bf16", act_dtype="bf16")
    assert so.rel_frobenius(probs, want) <= TOL


@pytest.mark.parametrize("in_dtype,sizes,batch", [
    ("tf32", [32, 256, 256, 256, 3], 1536),
    ("bf16", [32, 256, 256, 256, 3], 1536),
    ("bf16", [512, 1024, 1024, 10], 2048),
])
def test_backward_gradients(gpu, in_dtype, sizes, batch):
    net, ws, bs = build(gpu, sizes, batch, in_dtype, 4, training=True, bias_scale=0.05)
    if sizes[0] == 32:
        x, mask = so.leduc_inputs(4, batch)
    else:
        x, mask = so.holdem_inputs(4, batch, features=sizes[0], actions=sizes[-1])
    target = so.random_target(44, mask)
    dx, dm, dt = gpu.to_storage(x, in_dtype), gpu.DeviceArray.from_numpy(mask), gpu.DeviceArray.from_numpy(target)
    net.forward(dx, dm, head_flags=8)
    net.backward(dx, dm, dt)
    got = net.split_flat(net.grads.numpy())
    _, _, loss, want = so.mlp_train_step(x, [so.round_input(w, in_dtype) for w in ws], bs, mask, target, 0.0,
                                         in_dtype=in_dtype, act_dtype=in_dtype)
    assert abs(float(net.loss.numpy()[0]) - loss) <= 2e-3 * abs(loss)
    for i, ((gw, gb), (ww, wb)) in enumerate(zip(got, want)):
        assert so.rel_frobenius(gw, ww) <= TOL, "dW of layer %d" % i
        assert so.rel_frobenius(gb, wb) <= 5e-3, "db of layer %d" % i      # column sums of 16-bit dY
    # padding of the flat gradient vector stays zero
    flat = net.grads.numpy().copy()
    for i in range(net.n_layers):
        o, ob = net.offsets[2 * i], net.offsets[2 * i + 1]
        flat[o:o + sizes[i + 1] * sizes[i]] = 0
        flat[ob:ob + sizes[i + 1]] = 0
    assert not flat.any()


@pytest.mark.parametrize("in_dtype,sizes,batch", [
    ("bf16", [64, 1088, 7], 1001),       # 1088 columns: two passes of the head dgrad; odd batch: unaligned sign words
    ("f16", [64, 96, 12], 777),          # 12 outputs, a row of three warps' worth of 16-byte groups
    ("bf16", [32, 160, 16], 520),        # 16 outputs: the widest head the CUDA-core dgrad takes
    ("bf16", [32, 128, 8], 4096),
])
def test_backward_gradients_head_widths(gpu, in_dtype, sizes, batch):
    """The dgrad of a head with at most 16 outputs runs on the CUDA cores (one instance per width class,
    sign words read 8 rows at a time, column sums per block): gradients against the oracle for the
    widths, row lengths and batch sizes that take its different paths."""
    net, ws, bs = build(gpu, sizes, batch, in_dtype, 14, training=True, bias_scale=0.05)
    g = so.rng(15)
    x = g.random((batch, sizes[0]), dtype=np.float32)
    mask = (g.random((batch, sizes[-1])) < 0.7).astype(np.uint8)
    mask[:, 0] = 1
    target = so.random_target(16, mask)
    dx, dm, dt = gpu.to_storage(x, in_dtype), gpu.DeviceArray.from_numpy(mask), gpu.DeviceArray.from_numpy(target)
    net.forward(dx, dm, head_flags=8)
    net.backward(dx, dm, dt)
    got = net.split_flat(net.grads.numpy())
    _, _, loss, want = so.mlp_train_step(x, [so.round_input(w, in_dtype) for w in ws], bs, mask, target, 0.0,
                                         in_dtype=in_dtype, act_dtype=in_dtype)
    assert abs(float(net.loss.numpy()[0]) - loss) <= 2e-3 * abs(loss)
    for i, ((gw, gb), (ww, wb)) in enumerate(zip(got, want)):
        assert so.rel_frobenius(gw, ww) <= TOL, "dW of layer %d" % i
        assert so.rel_frobenius(gb, wb) <= 5e-3, "db of layer %d" % i


def test_train_step_updates_master_and_compute_weights(gpu):
    sizes, batch, lr = [32, 256, 256, 256, 3], 4096, 1e-3
    net, ws, bs = build(gpu, sizes, batch, "bf16", 6, training=True)
    x, mask = so.leduc_inputs(6, batch)
    target = so.random_target(66, mask)
    net.train_step(gpu.to_storage(x, "bf16"), gpu.DeviceArray.from_numpy(mask), gpu.DeviceArray.from_numpy(target), lr)
    new_w, new_b = net.get_weights()
    w_ref, b_ref, _, grads = so.mlp_train_step(x, [so.round_bf16(w) for w in ws], bs, mask, target, lr,
                                               in_dtype="bf16", act_dtype="bf16")
    for i in range(len(ws)):
        step_got = ws[i] - new_w[i]          # lr * dW, master weights are fp32
        step_want = lr * grads[i][0]
        assert so.rel_frobenius(step_got, step_want) <= 1e-2      # fp32 cancellation in w - w'
    from spiral_b200 import dtypes
    flat = net.params.numpy()
    np.testing.assert_array_equal(net.w_compute.numpy(), dtypes.round_bf16(flat))
    # a second step still runs on the updated weights and lowers the loss on the same batch
    l0 = float(net.loss.numpy()[0])
    net.loss.fill_zero()
    for _ in range(20):
        net.loss.fill_zero()
        net.train_step(gpu.to_storage(x, "bf16"), gpu.DeviceArray.from_numpy(mask), gpu.DeviceArray.from_numpy(target), 0.05)
    assert float(net.loss.numpy()[0]) < l0


def test_empty_batch_is_a_no_op(gpu):
    net = gpu.PolicyMLP([32, 64, 3], 0, in_dtype="bf16")
    net.forward(gpu.DeviceArray((0, 32), "bf16"))


def test_layer_graph_runs_fused_and_matches_oracle(gpu):
    """The reference's builder names (ml/layers.spi:347-420) on the fused path: a 3-layer net with
    ReLU and a prefix-masked softmax head, weights N(0, 0.1) from pass_init."""
    L = gpu.layers
    g = L.masked_softmax(3, L.matmul((64, 8), L.relu(L.matmul((64, 64), L.relu(L.matmul((32, 64),
                         L.input("input", (2, 256, 32))))))))
    model = L.pass_init(L.create_model(g))
    x = so.round_tf32(so.rng(8).normal(size=(512, 32)).astype(np.float32))
    L.key_extract(model, "input").upload(x)
    out = L.graph_run_host(model).numpy()
    ws = [so.round_tf32(w) for w in L.get_weights(model)]
    h = x
    for w in ws[:-1]:
        h = so.relu(so.matmul(False, True, 1.0, h, w, 0.0, None, in_dtype="tf32"))
    want = so.masked_softmax(so.matmul(False, True, 1.0, h, ws[-1], 0.0, None, in_dtype="tf32"),
                             so.prefix_mask((512, 8), 3))
    assert so.rel_frobenius(out, want) <= TOL
    assert np.all(out[:, 3:] == 0)
    # unfused nodes: ln_l2 and argmax after a plain matmul
    g2 = L.argmax(L.ln_l2(L.matmul((32, 16), L.input("input", (1, 128, 32)))))
    m2 = L.pass_init(L.create_model(g2))
    L.key_extract(m2, "input").upload(x[:128])
    idx = L.graph_run_host(m2).numpy()
    w2 = so.round_tf32(L.get_weights(m2)[0])
    ref = so.ln_l2(so.matmul(False, True, 1.0, x[:128], w2, 0.0, None, in_dtype="tf32"))
    top2 = np.sort(ref, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 1e-4 * np.abs(top2[:, 1])
    np.testing.assert_array_equal(idx[clear], so.argmax(ref)[clear])


@pytest.mark.parametrize("in_dtype,batch", [("f16", 1000), ("bf16", 16384), ("f16", 25600)])
def test_fused_persistent_forward_matches_layerwise_and_oracle(gpu, in_dtype, batch):
    """One persistent kernel for the Leduc-sized net: ragged last tile (1000), the benchmark batch
    (16384 = 128 tiles) and more tiles than SMs (25600 = 200 tiles)."""
    sizes = [32, 256, 256, 256, 3]
    net, ws, bs = build(gpu, sizes, batch, in_dtype, 3, head=("masked_softmax", "regret_matching", "argmax"),
                        bias_scale=0.1)
    x, mask = so.leduc_inputs(9, batch)
    dx, dm = gpu.to_storage(x, in_dtype), gpu.DeviceArray.from_numpy(mask)
    layerwise = net.forward(dx, dm).numpy().copy()
    actions_layerwise = net.actions.numpy().copy()
    net.probs.fill_zero()
    net.actions.fill_zero()
    fused = net.forward_fused(dx, dm).numpy()
    assert so.rel_frobenius(fused, layerwise) <= 1e-5        # same rounding points, same arithmetic
    want = so.mlp_forward(x, ws, bs, mask, in_dtype=in_dtype, act_dtype=in_dtype,
                          head=("masked_softmax", "regret_matching"))
    assert so.rel_frobenius(fused, want) <= TOL
    actions = net.actions.numpy()
    np.testing.assert_array_equal(actions, np.argmax(fused, axis=1))
    agree = actions == actions_layerwise
    assert agree.mean() > 0.999


def test_fused_forward_other_shapes_and_limits(gpu):
    from spiral_b200 import SpiralError
    sizes, batch = [64, 128, 64, 10], 777
    net, ws, bs = build(gpu, sizes, batch, "bf16", 12)
    g = so.rng(12)
    x = g.random((batch, 64), dtype=np.float32)
    mask = (g.random((batch, 10)) < 0.6).astype(np.uint8)
    mask[:, 0] = 1
    got = net.forward_fused(gpu.to_storage(x, "bf16"), gpu.DeviceArray.from_numpy(mask)).numpy()
    want = so.mlp_forward(x, ws, bs, mask, in_dtype="bf16", act_dtype="bf16")
    assert so.rel_frobenius(got, want) <= TOL
    wide = gpu.PolicyMLP([512, 1024, 10], 128, in_dtype="bf16")
    with pytest.raises(SpiralError) as err:
        wide.forward_fused(gpu.DeviceArray((128, 512), "bf16"))
    assert err.value.code == -3


def test_backward_split_by_layer_equals_whole_pass(gpu):
    """sb_mlp_backward_range over layers 3, 2, 1, 0 in four calls gives the gradients of one call (both
    weight and bias gradients are sums whose order is not fixed -- split-K tiles are added by the memory
    system, bias columns by atomics -- so they agree to fp32 rounding, not bit for bit)."""
    sizes, batch = [32, 256, 256, 256, 3], 2048
    net, ws, bs = build(gpu, sizes, batch, "bf16", 21, training=True, bias_scale=0.05)
    x, mask = so.leduc_inputs(21, batch)
    target = so.random_target(22, mask)
    dx, dm, dt = gpu.to_storage(x, "bf16"), gpu.DeviceArray.from_numpy(mask), gpu.DeviceArray.from_numpy(target)
    net.forward(dx, dm, head_flags=8)
    whole = net.backward(dx, dm, dt).numpy().copy()
    loss_whole = float(net.loss.numpy()[0])
    net.loss.fill_zero()
    net.grads.fill_zero()
    for layer in (3, 2, 1, 0):
        net.backward_layers(dx, dm, dt, layer, layer)
    split = net.grads.numpy()
    for i, ((gw, gb), (ww, wb)) in enumerate(zip(net.split_flat(split), net.split_flat(whole))):
        np.testing.assert_allclose(gw, ww, rtol=1e-4, atol=1e-6 * float(np.abs(ww).max()))
        np.testing.assert_allclose(gb, wb, rtol=1e-4, atol=1e-7)
    assert abs(float(net.loss.numpy()[0]) - loss_whole) <= 1e-5 * abs(loss_whole)
    assert net.layer_segment(0)[0] == 0 and net.layer_segment(3)[1] == net.n_params


@pytest.mark.parametrize("members,batch,in_dtype", [(4, 1000, "f16"), (16, 6144, "bf16"), (3, 128, "f16")])
def test_ensemble_forward_in_one_launch_equals_the_members_one_by_one(gpu, members, batch, in_dtype):
    """All members of an ensemble on one input batch in a single fused launch: every member's
    probabilities and actions equal the single-net fused forward with that member's weights
    bit for bit, and the oracle within the class tolerance."""
    sizes = [32, 64, 64, 3]
    head = ("masked_softmax", "regret_matching", "argmax")
    x, mask = so.leduc_inputs(31, batch)
    dx, dm = gpu.to_storage(x, in_dtype), gpu.DeviceArray.from_numpy(mask)
    sets = [so.mlp_weights(100 + e, sizes) for e in range(members)]
    biases = [[so.rng(200 + e).normal(size=b.shape).astype(np.float32) * 0.1 for b in bs] for e, (_, bs) in enumerate(sets)]
    ens = gpu.EnsemblePolicyMLP(sizes, batch, members, in_dtype=in_dtype, head=head)
    ens.load_weights([ws for ws, _ in sets], biases)
    l0 = gpu.launch_count()
    probs = ens.forward(dx, dm).numpy()
    assert gpu.launch_count() - l0 == 1
    actions = ens.actions.numpy()
    single = gpu.PolicyMLP(sizes, batch, in_dtype=in_dtype, head=head)
    for e in range(members):
        single.load_weights(sets[e][0], biases[e])
        want_probs = single.forward_fused(dx, dm).numpy()
        np.testing.assert_array_equal(probs[e], want_probs)
        np.testing.assert_array_equal(actions[e], single.actions.numpy())
    oracle = so.mlp_forward(x, sets[members - 1][0], biases[members - 1], mask, in_dtype=in_dtype, act_dtype=in_dtype,
                            head=("masked_softmax", "regret_matching"))
    assert so.rel_frobenius(probs[members - 1], oracle) <= TOL
    with pytest.raises(gpu.SpiralError):
        gpu.EnsemblePolicyMLP([32, 96, 3], batch, 2).forward(dx, dm)        # hidden width not a multiple of 64


def test_layer_graph_with_ensemble_layers(gpu):
    """layers.matmul_ensemble (ml/layers.spi:468-471): one weight matrix per member, the graph run with
    an ensemble index; every member's output follows the oracle with that member's weights."""
    L = gpu.layers
    members = 3
    g = L.softmax(L.matmul_ensemble((members, 64, 8), L.relu(L.matmul_ensemble((members, 32, 64),
                  L.input("input", (1, 256, 32))))))
    model = L.pass_init(L.create_model(g))
    x = so.round_tf32(so.rng(18).normal(size=(256, 32)).astype(np.float32))
    L.key_extract(model, "input").upload(x)
    outs = []
    for e in range(members):
        out = L.graph_run_host(model, ensemble=e).numpy().copy()
        w0, w1 = [so.round_tf32(w) for w in L.get_weights(model, e)]
        h = so.relu(so.matmul(False, True, 1.0, x, w0, 0.0, None, in_dtype="tf32"))
        want = so.softmax(so.matmul(False, True, 1.0, h, w1, 0.0, None, in_dtype="tf32"))
        assert so.rel_frobenius(out, want) <= TOL
        outs.append(out)
    assert so.rel_frobenius(outs[0], outs[1]) > 1e-2          # the members really differ
    with pytest.raises(IndexError):
        L.graph_run_host(model, ensemble=members)


def test_checkpoint_round_trip(gpu, tmp_path):
    sizes, batch = [32, 64, 3], 256
    net, ws, bs = build(gpu, sizes, batch, "bf16", 77, bias_scale=0.1)
    x, mask = so.leduc_inputs(78, batch)
    dx, dm = gpu.to_storage(x, "bf16"), gpu.DeviceArray.from_numpy(mask)
    want = net.forward(dx, dm).numpy().copy()
    path = str(tmp_path / "policy.npz")
    net.save(path)
    other = gpu.PolicyMLP(sizes, batch, in_dtype="bf16")
    other.load(path)
    np.testing.assert_array_equal(other.forward(dx, dm).numpy(), want)
    for a, b in zip(other.get_weights()[0], net.get_weights()[0]):
        np.testing.assert_array_equal(a, b)
    with pytest.raises(ValueError):
        gpu.PolicyMLP([32, 128, 3], batch, in_dtype="bf16").load(path)


def test_layer_graph_sampling_head(gpu):
    """masked_softmax_and_discrete_sample (ml/layers.spi:422-431): indices are legal (below the prefix
    size), follow the oracle for the uniforms in use, and change with the seed."""
    L = gpu.layers
    g = L.masked_softmax_and_discrete_sample(5, L.matmul((32, 8), L.input("input", (1, 512, 32))))
    model = L.pass_init(L.create_model(g))
    x = so.round_tf32(so.rng(28).normal(size=(512, 32)).astype(np.float32))
    L.key_extract(model, "input").upload(x)
    l0 = gpu.launch_count()
    idx = L.graph_run_host(model, seed=7).numpy().copy()
    assert gpu.launch_count() - l0 == 1                     # matmul + masked softmax + sampling: one launch
    probs = model.tensor(model.nodes[-2]).numpy()
    u = so.philox_uniform(7, np.arange(512), 0)             # the draw the head made: stream (seed, row), output 0
    np.testing.assert_array_equal(idx, so.discrete_sampling(probs, u))
    assert idx.min() >= 0 and idx.max() < 5
    w = so.round_tf32(L.get_weights(model)[0])
    want = so.masked_softmax(so.matmul(False, True, 1.0, x, w, 0.0, None, in_dtype="tf32"), so.prefix_mask((512, 8), 5))
    assert so.rel_frobenius(probs, want) <= TOL
    assert (L.graph_run_host(model, seed=8).numpy() != idx).any()
    u2 = np.full(512, 1.0, np.float32)
    model.uniforms(model.nodes[-1]).upload(u2)                      # caller-provided uniforms: u = 1 picks the last legal action
    np.testing.assert_array_equal(L.graph_run_host(model).numpy(), np.full(512, 4, np.int32))


def test_layer_graph_binarize_head(gpu):
    L = gpu.layers
    g = L.binarize(1000003, L.matmul((32, 24), L.input("input", (1, 300, 32))))
    model = L.pass_init(L.create_model(g))
    x = so.round_tf32(so.rng(38).normal(size=(300, 32)).astype(np.float32))
    L.key_extract(model, "input").upload(x)
    got = L.graph_run_host(model).numpy().view(np.uint32)
    logits = model.tensor(model.nodes[-2]).numpy()
    np.testing.assert_array_equal(got, so.binarize(logits, 1000003))
    w = so.round_tf32(L.get_weights(model)[0])
    ref = so.matmul(False, True, 1.0, x, w, 0.0, None, in_dtype="tf32")
    decided = np.all(np.abs(ref) > 5e-3, axis=1)              # rows whose signs do not hinge on TF32 rounding
    np.testing.assert_array_equal(got[decided], so.binarize(ref, 1000003)[decided])


@pytest.mark.parametrize("in_dtype,batch,sizes", [("bf16", 3000, [32, 256, 256, 256, 3]), ("f16", 65536, [32, 256, 256, 256, 3]),
                                                  ("bf16", 1000, [64, 128, 64, 10])])
def test_fused_training_forward_leaves_what_backward_needs(gpu, in_dtype, batch, sizes):
    """The training forward of a narrow net as ONE launch (sb_mlp_forward_fused_train): hidden activations and
    ReLU sign words land in global memory as the layer-wise forward leaves them, and the backward pass that
    follows gives the oracle's gradients."""
    net, ws, bs = build(gpu, sizes, batch, in_dtype, 31, training=True, bias_scale=0.05)
    if sizes[0] == 32:
        x, mask = so.leduc_inputs(31, batch)
    else:
        g = so.rng(31)
        x = g.random((batch, sizes[0]), dtype=np.float32)
        mask = (g.random((batch, sizes[-1])) < 0.6).astype(np.uint8)
        mask[:, 0] = 1
    target = so.random_target(32, mask)
    dx, dm, dt = gpu.to_storage(x, in_dtype), gpu.DeviceArray.from_numpy(mask), gpu.DeviceArray.from_numpy(target)
    net.forward(dx, dm, head_flags=8, fused=False)
    acts_ref = [a.numpy().copy() for a in net.activations]
    bits_ref = [b.numpy().copy() for b in net.relu_bits]
    probs_ref = net.probs.numpy().copy()
    for buf in net.activations + net.relu_bits + [net.probs]:
        buf.fill_zero()
    l0 = gpu.launch_count()
    net.forward(dx, dm, head_flags=8)              # a training net of this shape takes the fused path by itself
    assert gpu.launch_count() - l0 == 1
    for i, a in enumerate(net.activations):
        got = a.numpy()
        assert so.rel_frobenius(got, acts_ref[i]) <= 1e-5, "activations of layer %d" % i
        words = net.relu_bits[i].numpy().view(np.uint32).reshape(sizes[i + 1] // 32, batch)
        by_row = np.ascontiguousarray(words.T)
        bits = np.unpackbits(by_row.view(np.uint8).reshape(batch, -1), axis=1, bitorder="little").astype(bool)
        # The sign is taken from the fp32 value before it is rounded to the storage type, as the
        # layer-wise kernel does: a positive value below the smallest fp16 subnormal is stored as 0
        # with its bit set, nothing else may differ.
        stored = got.astype(np.float32) > 0
        assert not (stored & ~bits).any()
        assert np.mean(bits & ~stored) < 1e-6
        assert np.mean(words != bits_ref[i].view(np.uint32).reshape(words.shape)) < 1e-3
    assert so.rel_frobenius(net.probs.numpy(), probs_ref) <= 1e-5
    net.loss.fill_zero()
    net.backward(dx, dm, dt)
    got = net.split_flat(net.grads.numpy())
    _, _, loss, want = so.mlp_train_step(x, [so.round_input(w, in_dtype) for w in ws], bs, mask, target, 0.0,
                                         in_dtype=in_dtype, act_dtype=in_dtype)
    assert abs(float(net.loss.numpy()[0]) - loss) <= 2e-3 * abs(loss)
    for i, ((gw, gb), (ww, wb)) in enumerate(zip(got, want)):
        assert so.rel_frobenius(gw, ww) <= TOL, "dW of layer %d" % i
        assert so.rel_frobenius(gb, wb) <= 5e-3, "db of layer %d" % i
