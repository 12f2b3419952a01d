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
from .device import DeviceArray, Event, Stream, stream_ptr


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

    def __init__(self, net, world_size, rank, exchange, timeout_ms=2000, shard_master=True, fused_reduce=False):
        """``shard_master``: a rank's fp32 master parameters are kept current only in the slice it owns
        (plus all biases, which the forward pass reads in fp32): a third of the bytes leave the GPU per
        step.  Call ``gather_master()`` before reading the whole master vector on a rank
        (``net.get_weights()``, a checkpoint)."""
        if net.grads is None or not isinstance(net.grads, DeviceArray):
            raise ValueError("a peer update needs a network built for training with its own gradient buffer")
        self.net, self.world_size, self.rank = net, int(world_size), int(rank)
        self.timeout_ms = int(timeout_ms)
        self.shard_master = bool(shard_master)
        # The parameter vector is handled as one range per layer's weights and one per layer's bias; rank r
        # owns slice r of every range.  fused_reduce: the backward pass (net.backward_dp) adds every
        # weight-gradient tile of the wide layers straight into the owning rank's gradient buffer over peer
        # memory, so the update reads no remote gradients for those layers.  Off by default: with split-K
        # every split's tile crosses NVLink (4 x the gradient bytes at 32768 rows per rank) in a burst at
        # the end of each GEMM, which measured 12 us per weight-gradient GEMM against the 10 us the update
        # kernel saves (2 x B200).
        fused = (ctypes.c_int * net.n_layers)()
        if fused_reduce and self.world_size > 1:
            _lib.call("sb_mlp_dp_fused_layers", net.n_layers, net._sizes_c, self.world_size, fused)
        self.fused_layers = [bool(v) for v in fused]
        seg, red = [], []
        for layer in range(net.n_layers):
            end = net.offsets[2 * layer + 2] if layer + 1 < net.n_layers else net.n_params
            seg += [net.offsets[2 * layer], net.offsets[2 * layer + 1], net.offsets[2 * layer + 1], end]
            red += [int(self.fused_layers[layer]), 0]
        self._segments = (ctypes.c_longlong * len(seg))(*seg)
        self._reduced = (ctypes.c_int * len(red))(*red)
        self._n_segments = len(red)
        bias_ranges = []
        for layer in range(net.n_layers):
            bias_ranges += [net.offsets[2 * layer + 1], net.offsets[2 * layer + 2]]
        self._ranges = (ctypes.c_longlong * len(bias_ranges))(*bias_ranges)
        self._n_ranges = len(bias_ranges) // 2
        # One flag block for the whole-vector update and one per layer: updates of different layers may
        # be in flight at the same time (train_step(overlap=True)), and each needs a block of its own.
        self._flag_words = _lib.load().sb_dp_flag_bytes() // 4
        self._n_blocks = net.n_layers + 1
        self.flags = DeviceArray.zeros((self._flag_words * self._n_blocks,), "i32")
        self._epochs = [1] * self._n_blocks
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
        flag_bases = tables[3]
        self._flag_tables = [(ctypes.c_void_p * self.world_size)(*[b + 4 * self._flag_words * k for b in flag_bases])
                             for k in range(self._n_blocks)]

    def step(self, lr, stream=None, reduced=False):
        """All ranks call this after their backward pass; returns once the launch is enqueued.
        ``reduced``: the pass was ``net.backward_dp`` (the wide layers' gradients are already summed in
        their owners' buffers); False after a plain ``net.backward``, whose gradients are all local."""
        self._call(self.SHARDED_MASTER if self.shard_master else self.REPLICATED, lr, stream, reduced=reduced)

    def gather_master(self, stream=None):
        """Every owner's slices of the master parameters are copied to all ranks (all ranks call this)."""
        self._call(self.GATHER_MASTER, 0.0, stream)

    def grads_table(self):
        """HOST array of every rank's gradient buffer (device pointers), for ``net.backward_dp``."""
        return self._tables[0]

    def zero_gradients(self, stream=None):
        """Zeroes this rank's whole gradient buffer.  The ranges that peers add into must be zero before the
        first ``backward_dp`` pass and whenever a plain ``backward`` has written them in between; the
        caller puts a barrier across the ranks after it."""
        self.net.grads.fill_zero(stream)

    def step_layer(self, layer, lr, stream=None, max_blocks=0):
        """The same for the parameters of one layer only (its weight and bias segments), with that layer's
        own flag block: all ranks call it for the same layers in the same order.  Updates of different
        layers may overlap each other and the backward pass of the layers below."""
        self._call(self.SHARDED_MASTER if self.shard_master else self.REPLICATED, lr, stream, block=layer + 1,
                   layer=layer, max_blocks=max_blocks, reduced=False)

    def _call(self, mode, lr, stream, block=0, layer=None, max_blocks=0, reduced=False):
        net = self.net
        g, p, w, _ = self._tables
        if layer is None:
            n_seg, seg, red = self._n_segments, self._segments, self._reduced
        else:                                   # the weight and the bias range of one layer
            n_seg = 2
            seg = (ctypes.c_longlong * 4)(*self._segments[4 * layer:4 * layer + 4])
            red = (ctypes.c_int * 2)(*self._reduced[2 * layer:2 * layer + 2])
        _lib.call("sb_dp_sgd_update_segments", self.world_size, self.rank, g, p, w, self._flag_tables[block],
                  ctypes.c_uint(self._epochs[block]), n_seg, seg, red if (reduced and mode != self.GATHER_MASTER) else None,
                  ctypes.c_float(lr), _lib.DTYPE_CODES[net.storage], mode, self._ranges, self._n_ranges,
                  int(max_blocks), self.timeout_ms, 1, stream_ptr(stream))
        self._epochs[block] += 2

    @property
    def epoch(self):
        return self._epochs[0]

    @epoch.setter
    def epoch(self, value):
        self._epochs[0] = int(value)

    def status(self):
        """0, or 0x100 + the rank whose arrival a bounded wait gave up on, of the first flag block that
        recorded one (synchronises the device)."""
        out = ctypes.c_int(0)
        for k in range(self._n_blocks):
            _lib.call("sb_dp_status", self.flags.ptr + 4 * self._flag_words * k, ctypes.byref(out))
            if out.value != 0:
                return out.value
        return 0

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
                 peer_update=None, overlap_update=False, reserve_smem=4096):
        """``all_reduce(buffer)`` sums the whole flat gradient buffer in place.  Optional
        ``all_reduce_segment(buffer, begin, end)`` starts an asynchronous sum of elements
        [begin, end) and returns a handle with ``wait()`` (or None when it completed in order)."""
        self.net, self.global_batch = net, int(global_batch)
        self.all_reduce, self.world_size, self.rank = all_reduce, int(world_size), int(rank)
        self.all_reduce_segment = all_reduce_segment
        self.peer_update = peer_update
        # overlap_update: with a PeerUpdate, every layer's parameters are exchanged and updated on a second
        # stream as soon as that layer's gradients are complete, beside the backward pass of the layers
        # below.  The update CTAs must be resident next to the GEMM CTAs, which fill an SM's shared memory:
        # during the backward pass the GEMM is told to leave `reserve_smem` bytes free.
        self.overlap_update = bool(overlap_update) and peer_update is not None
        self.reserve_smem = int(reserve_smem)
        self._side = None
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
        if self.world_size > 1 and self.peer_update is not None and self.overlap_update:
            if self._side is None:
                self._side = Stream()
                self._ready = [Event() for _ in range(net.n_layers)]
                self._done = Event()
            side = self._side
            _lib.call("sb_gemm_reserve_smem", self.reserve_smem)
            try:
                for layer in range(net.n_layers - 1, -1, -1):
                    net.backward_layers(x, mask, target, layer, layer, global_batch=self.global_batch, stream=stream)
                    self._ready[layer].record(stream)
                    side.wait_event(self._ready[layer])
                    self.peer_update.step_layer(layer, lr, stream=side.ptr)
            finally:
                _lib.call("sb_gemm_reserve_smem", 0)
            self._done.record(side.ptr)
            _lib.call("sb_stream_wait_event", stream_ptr(stream), self._done.ptr)
            return
        if self.world_size > 1 and self.peer_update is not None:
            peer = self.peer_update
            if any(getattr(peer, "fused_layers", ())):
                # the weight-gradient GEMMs of the wide layers add their tiles into the owners' buffers
                net.backward_dp(x, mask, target, peer.grads_table(), self.world_size, self.rank,
                                global_batch=self.global_batch, stream=stream)
                peer.step(lr, stream=stream, reduced=True)
            else:
                net.backward(x, mask, target, global_batch=self.global_batch, stream=stream)
                peer.step(lr, stream=stream)
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
