"""The fused ensemble forward at the reference's own net shapes and the per-decision call.

Reference: the games build ensembles of small nets that end in 64 columns with a prefix-masked head
(game/leduc/model_cem.spi:37,52-60), the test nets put ln_l2 between matmul and relu and end in a
prefix-masked softmax + sampling head over `inner` = 128 columns (game/leduc/tests/train.spi:88-101),
and models.noinline_run (ml/models.spi:9-76) serialises the state, runs every member, draws a member
and returns its action with the probabilities all members gave that action.

Probabilities are compared with the oracle within the class tolerance (2e-3); everything downstream
of the probabilities (sampled indices, the drawn member, the reported probabilities) is a pure
function of them and of the Philox stream and is compared bit for bit.
"""
import numpy as np
import pytest

from oracle import spiral_oracle as so

pytestmark = pytest.mark.gpu
TOL = 2e-3


def member_weights(seed, sizes, members, std=None):
    sets = []
    for e in range(members):
        if std is None:
            sets.append(so.mlp_weights(seed + e, sizes)[0])
        else:
            g = so.rng(seed + e)
            sets.append([g.normal(0.0, std, size=(sizes[i + 1], sizes[i])).astype(np.float32) for i in range(len(sizes) - 1)])
    return sets


def test_leduc_cem_shape_64_columns_three_legal(gpu):
    """128 -> 64 -> 64 with `masked_regret_matching' 3`, 32 members (game/leduc/model_cem.spi:33-60): one
    launch, equal to member-by-member runs bit for bit, the oracle within tolerance, zeros beyond the prefix."""
    sizes, members, batch = [128, 64, 64], 32, 1536
    ws = member_weights(700, sizes, members)
    x = (so.rng(70).random((batch, 128)) < 0.15).astype(np.float32)
    dx = gpu.to_storage(x, "bf16")
    ens = gpu.EnsemblePolicyMLP(sizes, batch, members, in_dtype="bf16", with_bias=False)
    ens.load_weights(ws)
    l0 = gpu.launch_count()
    probs = ens.forward_head(dx, head=("regret_matching", "argmax"), prefix=3).numpy()
    assert gpu.launch_count() - l0 == 1
    want = so.ensemble_forward(x, ws, None, so.prefix_mask((batch, 64), 3), in_dtype="bf16", head=("regret_matching",))
    assert so.rel_frobenius(probs, want) <= TOL
    assert np.all(probs[:, :, 3:] == 0)
    np.testing.assert_allclose(probs.sum(axis=2), 1.0, atol=1e-5)
    np.testing.assert_array_equal(ens.actions.numpy(), np.argmax(probs, axis=2))
    single = gpu.EnsemblePolicyMLP(sizes, batch, 1, in_dtype="bf16", with_bias=False)
    for e in (0, 13, 31):
        single.load_weights([ws[e]])
        np.testing.assert_array_equal(single.forward_head(dx, head=("regret_matching",), prefix=3).numpy()[0], probs[e])


def test_row_normalised_net_with_sampling_head_over_128_columns(gpu):
    """128 -> 128 -> 128 -> 128, ln_l2 + relu between the layers, `masked_softmax_and_discrete_sample' 3`
    (game/leduc/tests/train.spi:88-101), weights N(0, 0.1) as the reference initialises them."""
    sizes, members, batch = [128, 128, 128, 128], 4, 1000
    ws = member_weights(710, sizes, members, std=0.1)
    x = so.round_bf16(so.rng(71).normal(size=(batch, 128)).astype(np.float32))
    ens = gpu.EnsemblePolicyMLP(sizes, batch, members, in_dtype="bf16", hidden_norm=True)
    ens.load_weights(ws)
    l0 = gpu.launch_count()
    probs = ens.forward_head(gpu.to_storage(x, "bf16"), head=("masked_softmax", "sample"), prefix=3, seed=31,
                             row_offset=10 ** 6, position=4).numpy()
    assert gpu.launch_count() - l0 == 1
    want = so.ensemble_forward(x, ws, None, so.prefix_mask((batch, 128), 3), in_dtype="bf16", hidden_norm=True)
    assert so.rel_frobenius(probs, want) <= TOL
    idx = ens.indices.numpy()
    for e in range(members):
        u = so.philox_uniform(31, 10 ** 6 + np.arange(batch), 4 + e)
        np.testing.assert_array_equal(idx[e], so.discrete_sampling(probs[e], u))
    assert idx.min() >= 0 and idx.max() < 3


@pytest.mark.parametrize("members", [4, 16])
def test_policy_decide_matches_the_oracle(gpu, members):
    """The per-decision call on compact Leduc states: encoder + ONE fused launch; members' probabilities
    within tolerance, the tail (indices, drawn member, action, both probability outputs) bit for bit."""
    sizes, batch = [32, 64, 64], 3000              # 64 output columns, 3 legal (prefix), ragged last tile
    ws = member_weights(720, sizes, members)
    fields, _ = so.leduc_states(72, batch)
    x = so.encode_states(fields, so.LEDUC_WIDTHS)
    ens = gpu.EnsemblePolicyMLP(sizes, batch, members, in_dtype="f16", with_bias=False)
    ens.load_weights(ws)
    dfields = gpu.DeviceArray.from_numpy(fields)
    for call, seed in enumerate((2024, 2025)):       # the second call finds the tile counters zero again
        l0 = gpu.launch_count()
        out = ens.decide(seed, fields=dfields, widths=so.LEDUC_WIDTHS, head=("masked_softmax",), prefix=3, row_offset=77)
        assert gpu.launch_count() - l0 == 2
        probs = out["output_probs"].numpy()
        want = so.ensemble_forward(x, ws, None, so.prefix_mask((batch, 64), 3), in_dtype="f16")
        assert so.rel_frobenius(probs, want) <= TOL
        action, member, selected, by_member, indices = so.policy_decide(probs, seed, row_offset=77)
        np.testing.assert_array_equal(out["output_indices"].numpy(), indices)
        np.testing.assert_array_equal(out["ensemble_id"].numpy(), member)
        np.testing.assert_array_equal(out["action"].numpy(), action)
        np.testing.assert_array_equal(out["sampling_prob_selected"].numpy(), selected)
        np.testing.assert_array_equal(out["sampling_prob_ensemble"].numpy(), by_member)
        assert action.min() >= 0 and action.max() < 3
        assert not ens._decide["tile_counters"].numpy().any()
    assert len(np.unique(member)) == members           # every member gets drawn somewhere in 3000 states


def test_policy_decide_with_a_legal_action_mask_and_ready_input(gpu):
    """The benchmark's Leduc net (32-256-256-256-3, biases, byte mask of legal actions) as an ensemble of 3,
    the input already encoded: one launch."""
    sizes, members, batch = [32, 256, 256, 256, 3], 3, 2048
    ws = member_weights(730, sizes, members)
    bs = [[so.rng(740 + e + 10 * i).normal(size=sizes[i + 1]).astype(np.float32) * 0.1 for i in range(4)] for e in range(members)]
    x, mask = so.leduc_inputs(73, batch)
    ens = gpu.EnsemblePolicyMLP(sizes, batch, members, in_dtype="bf16")
    ens.load_weights(ws, bs)
    l0 = gpu.launch_count()
    out = ens.decide(5, x=gpu.to_storage(x, "bf16"), head=("masked_softmax", "regret_matching"),
                     mask=gpu.DeviceArray.from_numpy(mask))
    assert gpu.launch_count() - l0 == 1
    probs = out["output_probs"].numpy()
    want = so.ensemble_forward(x, ws, bs, mask, in_dtype="bf16", head=("masked_softmax", "regret_matching"))
    assert so.rel_frobenius(probs, want) <= TOL
    action, member, selected, by_member, indices = so.policy_decide(probs, 5)
    np.testing.assert_array_equal(out["action"].numpy(), action)
    np.testing.assert_array_equal(out["ensemble_id"].numpy(), member)
    np.testing.assert_array_equal(out["sampling_prob_ensemble"].numpy(), by_member)
    assert np.all(mask[np.arange(batch), action] == 1)


def test_holdem_cem_shape_512_to_64(gpu):
    """The reference's Hold'em policy net (game/nl_hu_holdem/model_cem.spi:62-98): one dense layer from the
    512-wide pickled state to 64 columns, `masked_regret_matching'` over the first 3, an ensemble of 4.  The
    pickled state is bits and one-hot groups, so the input here is {0,1}."""
    sizes, members, batch = [512, 64], 4, 5000
    ws = member_weights(750, sizes, members)
    x = (so.rng(75).random((batch, 512)) < 0.1).astype(np.float32)
    ens = gpu.EnsemblePolicyMLP(sizes, batch, members, in_dtype="bf16", with_bias=False)
    ens.load_weights(ws)
    l0 = gpu.launch_count()
    out = ens.decide(9, x=gpu.to_storage(x, "bf16"), head=("regret_matching",), prefix=3)
    assert gpu.launch_count() - l0 == 1
    probs = out["output_probs"].numpy()
    want = so.ensemble_forward(x, ws, None, so.prefix_mask((batch, 64), 3), in_dtype="bf16", head=("regret_matching",))
    assert so.rel_frobenius(probs, want) <= TOL
    action, member, selected, by_member, indices = so.policy_decide(probs, 9)
    np.testing.assert_array_equal(out["action"].numpy(), action)
    np.testing.assert_array_equal(out["sampling_prob_ensemble"].numpy(), by_member)
    # a wide input with wide hidden layers does not fit the kernel's shared memory and says so
    with pytest.raises(gpu.SpiralError) as err:
        gpu.EnsemblePolicyMLP([512, 256, 64], 128, 2, in_dtype="bf16").forward_head(gpu.DeviceArray((128, 512), "bf16"), prefix=3)
    assert err.value.code == -3
