"""Host-side logic that needs no GPU: row sharding, gradient buckets, the layer-graph planner and a
two-rank gloo run of the data-parallel exchange (CPU only)."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest


def test_shard_rows_cover_the_batch_exactly(sb):
    for total, world in ((262144, 8), (65536, 4), (10, 3), (5, 8), (0, 2)):
        spans = [sb.shard_rows(total, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sb.shard_rows(8, 2, 2)


def test_bucket_ranges(sb):
    assert sb.bucket_ranges(10, 4) == [(0, 4), (4, 8), (8, 10)]
    assert sb.bucket_ranges(0, 4) == []
    n = sb.param_offsets([512, 1024, 1024, 1024, 1024, 10])[-1]
    spans = sb.bucket_ranges(n, 1 << 20)
    assert spans[0][0] == 0 and spans[-1][1] == n and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))


def test_param_offsets_layout(sb):
    off = sb.param_offsets([32, 256, 256, 256, 3])
    assert off[0] == 0 and all(o % 64 == 0 for o in off)
    assert off[1] - off[0] >= 256 * 32 and off[2] - off[1] >= 256
    assert off[7] - off[6] >= 8 * 256          # the 3-row head is padded to 8 rows
    assert off[-1] > 140032                    # parameters of the Leduc net plus padding


def test_layer_graph_planner_mirrors_reference_shapes(sb):
    L = sb.layers
    g = L.masked_softmax(3, L.matmul((64, 3), L.relu(L.matmul((32, 64), L.input("input", (4, 256, 32))))))
    model = L.create_model(g, allocate=False)
    assert [n.op for n in model.nodes] == ["input", "matmul", "relu", "matmul", "softmax"]
    assert model.nodes[-1].dims == (4, 256, 3) and model.nodes[1].dims == (4, 256, 64)
    weights, workspace, adjoint = model.partition_bytes
    assert weights >= (32 * 64 + 64 * 3) * 4 and workspace >= 4 * 256 * (32 + 64 + 64 + 3 + 3) * 4 and adjoint == 0
    offsets = [n.offset for n in model.nodes]
    assert offsets == sorted(offsets) and all(o % 16 == 0 for o in offsets)
    with pytest.raises(ValueError):
        L.matmul((31, 8), L.input("input", (1, 8, 32)))


RANK_SCRIPT = textwrap.dedent('''
    import os, sys
    sys.path.insert(0, os.environ["SB_ROOT"]); sys.path.insert(0, os.path.join(os.environ["SB_ROOT"], "spiral-s-ml-library_b200"))
    import numpy as np, torch, torch.distributed as dist
    from spiral_b200.parallel import DataParallel, shard_rows
    from oracle import spiral_oracle as so
    dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
    rank, world = dist.get_rank(), dist.get_world_size()
    sizes, gbatch, lr = [6, 8, 4], 32, 0.5
    ws, bs = so.mlp_weights(1, sizes)
    x = so.rng(2).normal(size=(gbatch, 6)).astype(np.float32)
    mask = np.ones((gbatch, 4), np.uint8); target = so.random_target(3, mask)
    b, e = shard_rows(gbatch, world, rank)

    class HostNet:                                   # stands in for PolicyMLP: same calls, NumPy arithmetic
        def __init__(self):
            self.loss = type("L", (), {"fill_zero": lambda self, s=None: None})()
            self.w = [w.copy() for w in ws]; self.b = [v.copy() for v in bs]
        def forward(self, x, mask, stream=None): pass
        def backward(self, x, mask, target, global_batch=None, stream=None):
            _, _, _, g = so.mlp_train_step(x, self.w, self.b, mask, target, 0.0, global_batch=global_batch)
            self.grads = torch.from_numpy(np.concatenate([np.concatenate([gw.ravel(), gb]) for gw, gb in g]))
        def sgd(self, lr, stream=None):
            flat = self.grads.numpy(); o = 0
            for i in range(len(self.w)):
                n = self.w[i].size; self.w[i] -= lr * flat[o:o + n].reshape(self.w[i].shape); o += n
                n = self.b[i].size; self.b[i] -= lr * flat[o:o + n]; o += n

    net = HostNet()
    dp = DataParallel(net, gbatch, all_reduce=lambda g: dist.all_reduce(g), world_size=world, rank=rank)
    dp.train_step(x[b:e], mask[b:e], target[b:e], lr)
    want_w, want_b, _, _ = so.mlp_train_step(x, ws, bs, mask, target, lr)
    for got, want in zip(net.w + net.b, want_w + want_b):
        assert np.allclose(got, want, atol=1e-5), "rank %d disagrees with the single-process step" % rank
    flat = torch.from_numpy(np.concatenate([w.ravel() for w in net.w]))
    gathered = [torch.zeros_like(flat) for _ in range(world)]
    dist.all_gather(gathered, flat)
    assert all(torch.equal(gathered[0], t) for t in gathered), "replicas diverged"

    # The peer-update protocol on the host: every rank reduces only its slice of the flat gradient vector
    # (all ranks' gradients summed in rank order), updates that slice and hands it to every rank.
    from spiral_b200.parallel import update_slice

    class HostPeerUpdate:
        overlap_layer = 0
        def __init__(self, net): self.net = net
        def step(self, lr, stream=None):
            mine = self.net.grads.clone()
            everyone = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(everyone, mine)
            n = mine.numel()
            n4 = (n + 3) // 4 * 4
            b4, e4 = update_slice(n4, world, rank)
            b4, e4 = min(b4, n), min(e4, n)
            total = torch.zeros(e4 - b4)
            for g in everyone:
                total += g[b4:e4]
            flat = np.concatenate([np.concatenate([w.ravel(), v]) for w, v in zip(self.net.w, self.net.b)])
            new_slice = torch.from_numpy(flat[b4:e4] - lr * total.numpy())
            sizes_ = [None] * world
            dist.all_gather_object(sizes_, (b4, e4, new_slice))
            for bb, ee, sl in sizes_:
                flat[bb:ee] = sl.numpy()
            o = 0
            for i in range(len(self.net.w)):
                k = self.net.w[i].size; self.net.w[i] = flat[o:o + k].reshape(self.net.w[i].shape).copy(); o += k
                k = self.net.b[i].size; self.net.b[i] = flat[o:o + k].copy(); o += k

    net2 = HostNet()
    dp2 = DataParallel(net2, gbatch, world_size=world, rank=rank, peer_update=HostPeerUpdate(net2))
    dp2.train_step(x[b:e], mask[b:e], target[b:e], lr)
    for got, want in zip(net2.w + net2.b, want_w + want_b):
        assert np.allclose(got, want, atol=1e-5), "rank %d: the sliced update disagrees with the single-process step" % rank
    for got, ref in zip(net2.w + net2.b, net.w + net.b):
        assert np.allclose(got, ref, atol=1e-6)
    dist.destroy_process_group()
    print("rank", rank, "ok")
''')


def test_two_rank_gloo_data_parallel_step(tmp_path):
    """Sharded backward + all-reduce + SGD on 2 gloo ranks equals the single-process step, and the
    replicas end bit-identical; the sliced reduce-update-redistribute protocol of the peer update
    (every rank owns one slice, update_slice) gives the same weights."""
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29731",
                   SB_ROOT=root, OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=180)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)


@pytest.mark.parametrize("n,world", [(3681856, 8), (3681856, 3), (64, 8), (8, 16), (0, 2), (4, 1)])
def test_peer_update_slices_partition_the_parameter_vector(n, world):
    """Every element is reduced and updated by exactly one rank; slices are whole 4-element vectors."""
    import spiral_b200 as sb
    cover = np.zeros(n, np.int32)
    for r in range(world):
        b, e = sb.update_slice(n, world, r)
        assert 0 <= b <= e <= n and b % 4 == 0 and e % 4 == 0
        cover[b:e] += 1
    assert np.all(cover == 1)
    with pytest.raises(sb.SpiralError):
        sb.update_slice(6, 2, 0)
    with pytest.raises(sb.SpiralError):
        sb.update_slice(64, 2, 2)
