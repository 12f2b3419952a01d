"""Data-parallel policy training: batch rows sharded over ranks, weights replicated, one
gradient all-reduce per step.

The reference is single-GPU; the unit sharded here is its own batch decomposition (every CTA owns
a slab of rows, ml/layers.spi:182,231).  The exchange is pluggable: ``all_reduce(buffer)`` must sum
the flat fp32 gradient buffer in place across ranks (``torch.distributed.all_reduce`` over NCCL on
GPUs; any callable on CPU tests).  Inference needs no exchange at all.

``PeerUpdate`` replaces all-reduce + SGD by the library's own kernel over peer memory: every rank
reduces one slice of the gradient vector straight out of its peers' buffers, updates that slice
and stores the new weights into every rank's buffers (csrc/dp.cu).
"""
import ctypes

from . import _lib
from .device import DeviceArray, stream_ptr


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


def update_slice(n_params, world_size, rank, begin=0):
    """The part of [begin, n_params) of the flat parameter vector that ``rank`` reduces and updates
    when a peer update covers that range in one call."""
    out = (ctypes.c_longlong * 2)()
    _lib.call("sb_dp_slice", ctypes.c_longlong(int(begin)), ctypes.c_longlong(int(n_params)), int(world_size),
              int(rank), out)
    return int(out[0]), int(out[1])


class PeerUpdate:
    """Gradient reduction + SGD + weight redistribution in one kernel over peer memory.

    ``exchange(payload)`` is the only host-side communication: an all-gather of a small picklable
    object (``torch.distributed.all_gather_object`` or any equivalent), called once at set-up with
    this rank's four 64-byte memory handles; it returns the payloads of all ranks in rank order.
    """

    REPLICATED, SHARDED_MASTER, GATHER_MASTER = 0, 1, 2

    def __init__(self, net, world_size, rank, exchange, timeout_ms=2000, shard_master=True):
        """``shard_master``: a rank's fp32 master parameters are kept current only in the slice it owns
        (plus all biases, which the forward pass reads in fp32): a third of the bytes leave the GPU per
        step.  Call ``gather_master()`` before reading the whole master vector on a rank
        (``net.get_weights()``, a checkpoint)."""
        if net.grads is None or not isinstance(net.grads, DeviceArray):
            raise ValueError("a peer update needs a network built for training with its own gradient buffer")
        self.net, self.world_size, self.rank = net, int(world_size), int(rank)
        self.timeout_ms, self.epoch = int(timeout_ms), 1
        self.shard_master = bool(shard_master)
        bias_ranges = []
        for layer in range(net.n_layers):
            bias_ranges += [net.offsets[2 * layer + 1], net.offsets[2 * layer + 2]]
        self._ranges = (ctypes.c_longlong * len(bias_ranges))(*bias_ranges)
        self._n_ranges = len(bias_ranges) // 2
        words = _lib.load().sb_dp_flag_bytes() // 4
        self.flags = DeviceArray.zeros((words,), "i32")
        mine = [net.grads.ptr, net.params.ptr, net.w_compute.ptr, self.flags.ptr]
        handles = []
        for ptr in mine:
            h = (ctypes.c_ubyte * 64)()
            _lib.call("sb_ipc_export", ptr, h)
            handles.append(bytes(h))
        everyone = exchange(handles)
        if len(everyone) != self.world_size:
            raise ValueError("exchange returned %d payloads for %d ranks" % (len(everyone), self.world_size))
        self._opened = []
        tables = [[None] * self.world_size for _ in mine]
        for r, payload in enumerate(everyone):
            for k in range(len(mine)):
                if r == self.rank:
                    tables[k][r] = mine[k]
                else:
                    out = ctypes.c_void_p()
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(payload[k])
                    _lib.call("sb_ipc_open", buf, ctypes.byref(out))
                    self._opened.append(out.value)
                    tables[k][r] = out.value
        self._tables = [(ctypes.c_void_p * self.world_size)(*t) for t in tables]

    def step(self, lr, stream=None):
        """All ranks call this after their backward pass; returns once the launch is enqueued."""
        self._call(self.SHARDED_MASTER if self.shard_master else self.REPLICATED, lr, stream)

    def gather_master(self, stream=None):
        """Every owner's slice of the master parameters is copied to all ranks (all ranks call this)."""
        self._call(self.GATHER_MASTER, 0.0, stream)

    def _call(self, mode, lr, stream):
        net = self.net
        g, p, w, f = self._tables
        _lib.call("sb_dp_sgd_update", self.world_size, self.rank, g, p, w, f, ctypes.c_uint(self.epoch),
                  ctypes.c_longlong(0), ctypes.c_longlong(net.n_params), ctypes.c_float(lr),
                  _lib.DTYPE_CODES[net.storage], mode, self._ranges, self._n_ranges, 0, self.timeout_ms, 1,
                  stream_ptr(stream))
        self.epoch += 2

    def status(self):
        """0, or 0x100 + the rank whose arrival a bounded wait gave up on (synchronises the device)."""
        out = ctypes.c_int(0)
        _lib.call("sb_dp_status", self.flags.ptr, ctypes.byref(out))
        return out.value

    def check(self):
        """Raises SpiralError (SB_ERR_DEVICE_TIMEOUT) when a flag wait of this rank's update kernel gave
        up.  The update of that step may then be partial (some CTAs may have seen the late flag and
        stored their part): restore the weights from a checkpoint and zero the flag block before the
        next step.  Synchronises the device."""
        code = self.status()
        if code != 0:
            raise _lib.SpiralError(-5, "the peer update gave up waiting for rank %d (status 0x%x); the weights of "
                                   "this step may be partly updated" % (code - 0x100, code))

    def close(self):
        for ptr in self._opened:
            _lib.call("sb_ipc_close", ptr)
        self._opened = []


class DataParallel:
    """Wraps a ``PolicyMLP`` built for this rank's shard."""

    def __init__(self, net, global_batch, all_reduce=None, world_size=1, rank=0, all_reduce_segment=None,
                 peer_update=None):
        """``all_reduce(buffer)`` sums the whole flat gradient buffer in place.  Optional
        ``all_reduce_segment(buffer, begin, end)`` starts an asynchronous sum of elements
        [begin, end) and returns a handle with ``wait()`` (or None when it completed in order)."""
        self.net, self.global_batch = net, int(global_batch)
        self.all_reduce, self.world_size, self.rank = all_reduce, int(world_size), int(rank)
        self.all_reduce_segment = all_reduce_segment
        self.peer_update = peer_update
        if self.world_size > 1 and all_reduce is None and all_reduce_segment is None and peer_update is None:
            raise ValueError("more than one rank needs an all_reduce callable or a PeerUpdate")

    def train_step(self, x, mask, target, lr, stream=None):
        """forward + backward on the local shard (gradients already scaled by 1/global_batch),
        all-reduce of the flat gradient buffer, then the same SGD update on every rank.

        With ``all_reduce_segment`` the exchange is issued layer by layer, top layer first, as soon as
        that layer's gradients are enqueued, so it overlaps the backward of the layers below."""
        net = self.net
        net.loss.fill_zero(stream)
        net.forward(x, mask, stream=stream)
        if self.world_size > 1 and self.peer_update is not None:
            net.backward(x, mask, target, global_batch=self.global_batch, stream=stream)
            self.peer_update.step(lr, stream=stream)
            return
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
