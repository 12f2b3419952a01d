"""GPU tests of the data-parallel update over peer memory (csrc/dp.cu), on one GPU.

Several ranks are emulated inside one process: every "rank" has its own gradient, parameter,
compute-copy and flag buffers, and the ranks' updates run one after the other with the flag
barriers switched off (no kernel ever waits for another one on the same GPU).  The real
multi-process path (IPC handles, barriers) is exercised by ``bench.py`` under torchrun.
The result must equal the oracle's update with the summed gradients: bit-exact in fp32 when the
sum has one rounding order (rank order), and the compute copy must be its rounding.
"""
import ctypes

import numpy as np
import pytest

from oracle import spiral_oracle as so

pytestmark = pytest.mark.gpu


def _tables(arrays_per_rank):
    world = len(arrays_per_rank)
    return [(ctypes.c_void_p * world)(*[(a[k].ptr if a[k] is not None else None) for a in arrays_per_rank]) for k in range(4)]


def _rank_buffers(gpu, n, seed, storage, params0):
    g = so.rng(seed).normal(size=n).astype(np.float32)
    grads = gpu.DeviceArray.from_numpy(g)
    params = gpu.DeviceArray.from_numpy(params0.copy())
    compute = gpu.DeviceArray.zeros((n,), storage)
    flags = gpu.DeviceArray.zeros((32,), "i32")
    return g, (grads, params, compute, flags)


@pytest.mark.parametrize("world,n,storage", [(1, 4096, "bf16"), (2, 4100 * 4, "bf16"), (3, 1000 * 4, "f16"), (8, 64 * 4, "f32"),
                                             (4, 8, "bf16")])
def test_emulated_ranks_reduce_update_and_redistribute(gpu, world, n, storage):
    from spiral_b200 import _lib
    params0 = so.rng(1).normal(size=n).astype(np.float32)
    host_grads, bufs = [], []
    for r in range(world):
        g, b = _rank_buffers(gpu, n, 10 + r, storage, params0)
        host_grads.append(g)
        bufs.append(b)
    g_t, p_t, w_t, f_t = _tables(bufs)
    lr = 0.05
    for r in range(world):       # one rank after the other, barriers off
        _lib.call("sb_dp_sgd_update", world, r, g_t, p_t, w_t, f_t, ctypes.c_uint(1), ctypes.c_longlong(0), ctypes.c_longlong(n),
                  ctypes.c_float(lr), _lib.DTYPE_CODES[storage], 0, None, 0, 0, 100, 0, None)
    gpu.synchronize()
    total = np.zeros(n, np.float32)
    for g in host_grads:         # the kernel adds in rank order, in fp32
        total = (total + g).astype(np.float32)
    want = (params0 - np.float32(lr) * total).astype(np.float32)
    for r in range(world):
        got = bufs[r][1].numpy()
        np.testing.assert_allclose(got, want, rtol=0, atol=1e-6)      # fused multiply-add vs two roundings
        np.testing.assert_array_equal(got, bufs[0][1].numpy())        # identical on every rank
        comp = bufs[r][2].numpy()
        np.testing.assert_array_equal(comp, so.round_input(got, storage) if storage != "f32" else got)
    # the slices partition the vector
    cover = np.zeros(n, np.int32)
    for r in range(world):
        b, e = gpu.update_slice(n, world, r)
        cover[b:e] += 1
    assert np.all(cover == 1)


def test_sharded_master_keeps_biases_everywhere_and_gather_completes_it(gpu):
    """SB_DP_SHARDED_MASTER: after a step a rank's master vector is current in its own slice and in the
    replicated (bias) ranges, the compute copy everywhere; SB_DP_GATHER_MASTER completes the master."""
    from spiral_b200 import _lib
    world, n, lr = 3, 3000 * 4, 0.1
    params0 = so.rng(21).normal(size=n).astype(np.float32)
    host_grads, bufs = [], []
    for r in range(world):
        g, b = _rank_buffers(gpu, n, 30 + r, "bf16", params0)
        host_grads.append(g)
        bufs.append(b)
    g_t, p_t, w_t, f_t = _tables(bufs)
    ranges = (ctypes.c_longlong * 4)(400, 800, 11000, 11200)       # two replicated ranges, in different slices
    for r in range(world):
        _lib.call("sb_dp_sgd_update", world, r, g_t, p_t, w_t, f_t, ctypes.c_uint(1), ctypes.c_longlong(0), ctypes.c_longlong(n),
                  ctypes.c_float(lr), _lib.DTYPE_CODES["bf16"], 1, ranges, 2, 0, 100, 0, None)
    gpu.synchronize()
    total = np.zeros(n, np.float32)
    for g in host_grads:
        total = (total + g).astype(np.float32)
    want = (params0 - np.float32(lr) * total).astype(np.float32)
    current = np.zeros(n, bool)
    current[400:800] = True
    current[11000:11200] = True
    for r in range(world):
        mine = current.copy()
        b, e = gpu.update_slice(n, world, r)
        mine[b:e] = True
        got = bufs[r][1].numpy()
        np.testing.assert_allclose(got[mine], want[mine], rtol=0, atol=1e-6)
        np.testing.assert_array_equal(got[~mine], params0[~mine])             # untouched elsewhere
        np.testing.assert_allclose(bufs[r][2].numpy(), so.round_bf16(want), rtol=0, atol=2e-2 * np.abs(want).max())
        np.testing.assert_array_equal(bufs[r][2].numpy(), bufs[0][2].numpy())
    for r in range(world):
        _lib.call("sb_dp_sgd_update", world, r, None, p_t, w_t, f_t, ctypes.c_uint(3), ctypes.c_longlong(0), ctypes.c_longlong(n),
                  ctypes.c_float(0.0), _lib.DTYPE_CODES["bf16"], 2, None, 0, 0, 100, 0, None)
    gpu.synchronize()
    for r in range(world):
        np.testing.assert_allclose(bufs[r][1].numpy(), want, rtol=0, atol=1e-6)
        np.testing.assert_array_equal(bufs[r][1].numpy(), bufs[0][1].numpy())


def test_a_sub_range_leaves_the_rest_untouched(gpu):
    from spiral_b200 import _lib
    world, n, lr = 2, 4096, 0.25
    params0 = so.rng(41).normal(size=n).astype(np.float32)
    host_grads, bufs = [], []
    for r in range(world):
        g, b = _rank_buffers(gpu, n, 42 + r, "f32", params0)
        host_grads.append(g)
        bufs.append(b)
    g_t, p_t, w_t, f_t = _tables(bufs)
    begin, end = 1024, 3000
    for r in range(world):
        _lib.call("sb_dp_sgd_update", world, r, g_t, p_t, w_t, f_t, ctypes.c_uint(1), ctypes.c_longlong(begin),
                  ctypes.c_longlong(end), ctypes.c_float(lr), _lib.DTYPE_CODES["f32"], 0, None, 0, 3, 100, 0, None)
    gpu.synchronize()
    want = params0.copy()
    want[begin:end] = (params0 - np.float32(lr) * (host_grads[0] + host_grads[1]))[begin:end]
    for r in range(world):
        np.testing.assert_allclose(bufs[r][1].numpy(), want, rtol=0, atol=1e-6)
    cover = np.zeros(n, np.int32)
    for r in range(world):
        b, e = gpu.update_slice(end, world, r, begin=begin)
        cover[b:e] += 1
    assert np.all(cover[begin:end] == 1) and cover.sum() == end - begin


def test_single_rank_equals_the_plain_sgd_update(gpu):
    from spiral_b200 import _lib
    n = 10240
    params0 = so.rng(2).normal(size=n).astype(np.float32)
    g, (grads, params, compute, flags) = _rank_buffers(gpu, n, 3, "bf16", params0)
    g_t, p_t, w_t, f_t = _tables([(grads, params, compute, flags)])
    _lib.call("sb_dp_sgd_update", 1, 0, g_t, p_t, w_t, f_t, ctypes.c_uint(1), ctypes.c_longlong(0), ctypes.c_longlong(n),
              ctypes.c_float(0.01), _lib.DTYPE_CODES["bf16"], 0, None, 0, 0, 100, 1, None)      # barriers on: a rank always meets itself
    ref_p = gpu.DeviceArray.from_numpy(params0.copy())
    ref_c = gpu.DeviceArray.zeros((n,), "bf16")
    _lib.call("sb_sgd_update", ref_p.ptr, grads.ptr, ref_c.ptr, ctypes.c_longlong(n), ctypes.c_float(0.01),
              _lib.DTYPE_CODES["bf16"], None)
    np.testing.assert_array_equal(params.numpy(), ref_p.numpy())
    np.testing.assert_array_equal(compute.numpy(), ref_c.numpy())
    status = ctypes.c_int(-1)
    _lib.call("sb_dp_status", flags.ptr, ctypes.byref(status))
    assert status.value == 0


def test_a_peer_that_never_arrives_ends_the_wait_with_a_status(gpu):
    """Rank 0 of 2 waits for a rank 1 that does not exist: the bounded wait (50 ms here) expires, the
    update is skipped, the flag block reports 0x100 + 1, and the device stays healthy."""
    from spiral_b200 import _lib
    n = 1024
    params0 = so.rng(4).normal(size=n).astype(np.float32)
    _, b0 = _rank_buffers(gpu, n, 5, "bf16", params0)
    _, b1 = _rank_buffers(gpu, n, 6, "bf16", params0)
    g_t, p_t, w_t, f_t = _tables([b0, b1])
    _lib.call("sb_dp_sgd_update", 2, 0, g_t, p_t, w_t, f_t, ctypes.c_uint(1), ctypes.c_longlong(0), ctypes.c_longlong(n),
              ctypes.c_float(0.5), _lib.DTYPE_CODES["bf16"], 0, None, 0, 0, 50, 1, None)
    gpu.synchronize()
    status = ctypes.c_int(0)
    _lib.call("sb_dp_status", b0[3].ptr, ctypes.byref(status))
    assert status.value == 0x100 + 1
    np.testing.assert_array_equal(b0[1].numpy(), params0)      # nothing was updated
    assert gpu.device_status() == (0, 0)


def test_argument_checks(gpu):
    from spiral_b200 import _lib
    n = 64
    _, b0 = _rank_buffers(gpu, n, 7, "bf16", np.zeros(n, np.float32))
    g_t, p_t, w_t, f_t = _tables([b0])
    for bad in [dict(world=0), dict(rank=1), dict(n=6), dict(timeout=0), dict(dtype=99), dict(mode=7)]:
        with pytest.raises(gpu.SpiralError):
            _lib.call("sb_dp_sgd_update", bad.get("world", 1), bad.get("rank", 0), g_t, p_t, w_t, f_t, ctypes.c_uint(1),
                      ctypes.c_longlong(0), ctypes.c_longlong(bad.get("n", n)), ctypes.c_float(0.1),
                      bad.get("dtype", _lib.DTYPE_CODES["bf16"]), bad.get("mode", 0), None, 0, 0, bad.get("timeout", 100), 0, None)


@pytest.mark.parametrize("world,sizes", [(2, [32, 256, 256, 3]), (4, [64, 512, 512, 10])])
def test_emulated_ranks_backward_adds_tiles_to_the_owners_and_update_reads_only_its_own(gpu, world, sizes):
    """The data-parallel backward pass whose weight-gradient GEMMs add their tiles into the owner's buffer
    (sb_mlp_backward_dp), with the ranks emulated one after the other on one GPU: every rank has its own net
    buffers and batch shard, all gradient buffers sit in one table.  After all ranks' passes, rank r's buffer
    holds the batch-wide sum of the rows it owns for the wide layers (rows of the other ranks stay zero);
    the update over per-layer ranges (reduced = 1 for those layers, barriers off) then gives every rank the
    oracle's SGD step on the whole batch and leaves the owned rows zero again."""
    from spiral_b200 import _lib
    shard, lr = 1024, 0.05
    gbatch = shard * world
    ws, bs = so.mlp_weights(61, sizes)
    bs = [(so.rng(62 + i).normal(size=b.shape) * 0.05).astype(np.float32) for i, b in enumerate(bs)]
    if sizes[0] == 32:
        x, mask = so.leduc_inputs(63, gbatch)
    else:
        x = so.round_bf16(so.rng(63).random((gbatch, sizes[0]), dtype=np.float32))
        mask = (so.rng(64).random((gbatch, sizes[-1])) < 0.6).astype(np.uint8)
        mask[:, :2] = 1
    target = so.random_target(65, mask)
    nets = []
    for r in range(world):
        net = gpu.PolicyMLP(sizes, shard, in_dtype="bf16", training=True)
        net.load_weights(ws, bs)
        net.grads.fill_zero()
        nets.append(net)
    n_layers = len(sizes) - 1
    fused = (ctypes.c_int * n_layers)()
    _lib.call("sb_mlp_dp_fused_layers", n_layers, nets[0]._sizes_c, world, fused)
    assert list(fused) == [1, 1, 0]
    table = (ctypes.c_void_p * world)(*[n.grads.ptr for n in nets])
    for r, net in enumerate(nets):
        rows = slice(r * shard, (r + 1) * shard)
        dx, dm, dt = gpu.to_storage(x[rows], "bf16"), gpu.DeviceArray.from_numpy(mask[rows]), gpu.DeviceArray.from_numpy(target[rows])
        net.loss.fill_zero()
        net.forward(dx, dm, head_flags=8)
        net.backward_dp(dx, dm, dt, table, world, r, global_batch=gbatch)
    gpu.synchronize()
    new_w, new_b, loss, want = so.mlp_train_step(x, [so.round_bf16(w) for w in ws], bs, mask, target, lr,
                                                 in_dtype="bf16", act_dtype="bf16")
    got = [n.split_flat(n.grads.numpy()) for n in nets]
    for layer in range(n_layers):
        out = sizes[layer + 1]
        if fused[layer]:
            per = out // world
            for r in range(world):
                mine = got[r][layer][0]
                assert so.rel_frobenius(mine[r * per:(r + 1) * per], want[layer][0][r * per:(r + 1) * per]) <= 2e-3
                other = np.delete(mine, np.s_[r * per:(r + 1) * per], axis=0)
                assert not other.any()                      # nobody adds into rows this rank does not own
        else:
            total = sum(got[r][layer][0] for r in range(world))
            assert so.rel_frobenius(total, want[layer][0]) <= 2e-3
        assert so.rel_frobenius(sum(got[r][layer][1] for r in range(world)), want[layer][1]) <= 5e-3
    assert abs(sum(float(n.loss.numpy()[0]) for n in nets) - loss) <= 2e-3 * abs(loss)

    # the update: one launch per rank over the per-layer ranges, reading only its own buffer where reduced
    seg, red = [], []
    net0 = nets[0]
    for layer in range(n_layers):
        end = net0.offsets[2 * layer + 2] if layer + 1 < n_layers else net0.n_params
        seg += [net0.offsets[2 * layer], net0.offsets[2 * layer + 1], net0.offsets[2 * layer + 1], end]
        red += [int(fused[layer]), 0]
    seg_c, red_c = (ctypes.c_longlong * len(seg))(*seg), (ctypes.c_int * len(red))(*red)
    flags = [gpu.DeviceArray.zeros((32,), "i32") for _ in range(world)]
    p_t = (ctypes.c_void_p * world)(*[n.params.ptr for n in nets])
    w_t = (ctypes.c_void_p * world)(*[n.w_compute.ptr for n in nets])
    f_t = (ctypes.c_void_p * world)(*[f.ptr for f in flags])
    for r in range(world):
        _lib.call("sb_dp_sgd_update_segments", world, r, table, p_t, w_t, f_t, ctypes.c_uint(1), len(red), seg_c, red_c,
                  ctypes.c_float(lr), _lib.DTYPE_CODES["bf16"], 0, None, 0, 0, 100, 0, None)
    gpu.synchronize()
    for r, net in enumerate(nets):
        gw, gb = net.get_weights()
        for layer in range(n_layers):
            step_got, step_want = ws[layer] - gw[layer], lr * want[layer][0]      # the master weights are fp32
            assert so.rel_frobenius(step_got, step_want) <= 1e-2          # fp32 cancellation in w - w'
        np.testing.assert_array_equal(net.params.numpy(), nets[0].params.numpy())
        np.testing.assert_array_equal(net.w_compute.numpy(), so.round_bf16(net.params.numpy()))
        left = net.split_flat(net.grads.numpy())
        for layer in range(n_layers):
            if fused[layer]:
                assert not left[layer][0].any()                          # consumed and zeroed by its owner
