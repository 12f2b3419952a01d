"""Data-parallel policy training: batch rows sharded over ranks, weights replicated, one
gradient all-reduce per step.

The reference is single-GPU; the unit sharded here is its own batch decomposition (every CTA owns
a slab of rows, ml/layers.spi:182,231).  The exchange is pluggable: ``all_reduce(buffer)`` must sum
the flat fp32 gradient buffer in place across ranks (``torch.distributed.all_reduce`` over NCCL on
GPUs; any callable on CPU tests).  Inference needs no exchange at all.
"""


def shard_rows(total_rows, world_size, rank):
    """Contiguous [begin, end) of the rows rank ``rank`` owns; the first ``total % world`` ranks get one more."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError("rank %d of world size %d" % (rank, world_size))
    base, extra = divmod(int(total_rows), world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def bucket_ranges(n_elements, bucket_elements):
    """[(begin, end), ...] covering a flat buffer in buckets of at most ``bucket_elements``."""
    if bucket_elements < 1:
        raise ValueError("bucket size must be positive")
    return [(b, min(n_elements, b + bucket_elements)) for b in range(0, int(n_elements), int(bucket_elements))]


class DataParallel:
    """Wraps a ``PolicyMLP`` built for this rank's shard."""

    def __init__(self, net, global_batch, all_reduce=None, world_size=1, rank=0, all_reduce_segment=None):
        """``all_reduce(buffer)`` sums the whole flat gradient buffer in place.  Optional
        ``all_reduce_segment(buffer, begin, end)`` starts an asynchronous sum of elements
        [begin, end) and returns a handle with ``wait()`` (or None when it completed in order)."""
        self.net, self.global_batch = net, int(global_batch)
        self.all_reduce, self.world_size, self.rank = all_reduce, int(world_size), int(rank)
        self.all_reduce_segment = all_reduce_segment
        if self.world_size > 1 and all_reduce is None and all_reduce_segment is None:
            raise ValueError("more than one rank needs an all_reduce callable")

    def train_step(self, x, mask, target, lr, stream=None):
        """forward + backward on the local shard (gradients already scaled by 1/global_batch),
        all-reduce of the flat gradient buffer, then the same SGD update on every rank.

        With ``all_reduce_segment`` the exchange is issued layer by layer, top layer first, as soon as
        that layer's gradients are enqueued, so it overlaps the backward of the layers below."""
        net = self.net
        net.loss.fill_zero(stream)
        net.forward(x, mask, stream=stream)
        if self.world_size > 1 and self.all_reduce_segment is not None:
            pending = []
            for layer in range(net.n_layers - 1, -1, -1):
                net.backward_layers(x, mask, target, layer, layer, global_batch=self.global_batch, stream=stream)
                begin, end = net.layer_segment(layer)
                pending.append(self.all_reduce_segment(net.grads, begin, end))
            for handle in pending:
                if handle is not None:
                    handle.wait()
        else:
            net.backward(x, mask, target, global_batch=self.global_batch, stream=stream)
            if self.world_size > 1:
                self.all_reduce(net.grads)
        net.sgd(lr, stream=stream)

    def infer(self, x, mask=None, stream=None):
        return self.net.forward(x, mask, stream=stream)
