"""The allocation-free forward pass (sb_mlp_forward_static) against the ordinary one.

Some hosts cannot give the library a workspace: they own no device allocator, run where
allocation is forbidden, or are inside a stream capture.  For them the hidden activations live in
a fixed 32 MiB array inside the library.  This file is collected last on purpose: if it fails,
a run that stops at the first failure has already run every other test.  The check is the
tolerance the other MLP tests use (2e-3 relative Frobenius error); both paths run the same
kernels, so the results are normally identical.
"""
import ctypes

import numpy as np
import pytest

from oracle import spiral_oracle as so

pytestmark = pytest.mark.gpu
TOL = 2e-3


def test_no_alloc_forward_matches_workspace_forward_twice(gpu):
    sizes, batch = [32, 256, 256, 256, 3], 4096
    ws, bs = so.mlp_weights(3, sizes)
    net = gpu.PolicyMLP(sizes, batch, in_dtype="f16", head=("masked_softmax", "regret_matching", "argmax"))
    net.load_weights(ws, bs)
    out = gpu.DeviceArray((batch, 3), "f32")
    actions = gpu.DeviceArray((batch,), "i32")
    for seed in (3, 4):                      # two calls in a row share the built-in workspace
        x, mask = so.leduc_inputs(seed, batch)
        dx, dm = gpu.to_storage(x, "f16"), gpu.DeviceArray.from_numpy(mask)
        want = net.forward(dx, dm).numpy()
        want_actions = net.actions.numpy()
        out.fill_zero()
        gpu.synchronize()
        free_before = gpu.mem_info()[0]
        net.forward_no_alloc(dx, out, dm, actions=actions)
        gpu.synchronize()
        # The call took no device memory: the free-memory reading is the same before and after
        # (the first call's one-time set-up -- symbol address, kernel attributes -- allocates nothing either).
        assert gpu.mem_info()[0] == free_before
        got = out.numpy()
        assert so.rel_frobenius(got, want) <= TOL
        np.testing.assert_array_equal(actions.numpy(), want_actions)
        oracle = so.mlp_forward(x, ws, bs, mask, in_dtype="f16", act_dtype="f16",
                                head=("masked_softmax", "regret_matching"))
        assert so.rel_frobenius(got, oracle) <= TOL


def test_no_alloc_forward_rejects_what_does_not_fit(gpu):
    from spiral_b200 import SpiralError, _lib
    sizes = (ctypes.c_int * 3)(512, 1024, 10)
    with pytest.raises(SpiralError) as err:          # 65536 x 1024 bf16 = 128 MiB of hidden activations
        _lib.call("sb_mlp_forward_static", 2, sizes, 65536, _lib.BF16, 16, 16, None, 8, None, 16, None, None)
    assert err.value.code == -6          # SB_ERR_TOO_LARGE
    assert "workspace" in str(err.value)
