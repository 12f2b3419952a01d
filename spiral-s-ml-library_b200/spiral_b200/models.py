"""Dense policy network on the GPU: the caller of the GEMM path.

Reference: ml/models.spi:9-76 (run a layer graph per decision) and the model
graphs game/leduc/model_cem.spi:41-66, game/nl_hu_holdem/model_cem.spi:71-103
(input -> matmul -> relu ... -> masked head).  ``PolicyMLP`` owns the buffers the
reference keeps in its weight / workspace / adjoint arenas and drives
sb_mlp_forward / sb_mlp_backward / sb_sgd_update.
"""
import ctypes

import numpy as np

from . import _lib
from .device import DeviceArray, device_ptr, stream_ptr
from . import dtypes

HEAD_FLAGS = {"masked_softmax": _lib.EPI_MASKED_SOFTMAX, "regret_matching": _lib.EPI_REGRET_MATCHING,
              "argmax": _lib.EPI_ARGMAX}


def param_offsets(sizes):
    """Element offsets [W0, b0, W1, b1, ..., total] of the flat parameter vector."""
    n = len(sizes) - 1
    arr = (ctypes.c_int * len(sizes))(*sizes)
    out = (ctypes.c_longlong * (2 * n + 1))()
    _lib.call("sb_mlp_param_offsets", n, arr, out)
    return list(out)


class PolicyMLP:
    """ReLU MLP with a masked row head; weights W_i stored [out, in] like layers.weight."""

    def __init__(self, sizes, batch, in_dtype="bf16", head=("masked_softmax",), with_bias=True,
                 training=False, grads=None):
        if in_dtype not in ("tf32", "bf16", "f16"):
            raise ValueError("in_dtype must be 'tf32', 'bf16' or 'f16'")
        self.sizes = [int(s) for s in sizes]
        self.n_layers = len(self.sizes) - 1
        self.batch = int(batch)
        self.in_dtype = in_dtype
        self.storage = in_dtype          # 'tf32' = fp32 storage holding TF32-rounded values
        self.head = tuple(head)
        self.head_flags = 0
        for h in self.head:
            self.head_flags |= HEAD_FLAGS[h]
        self.with_bias = bool(with_bias)
        self.offsets = param_offsets(self.sizes)
        self.n_params = self.offsets[-1]
        self._sizes_c = (ctypes.c_int * len(self.sizes))(*self.sizes)
        self.params = DeviceArray.zeros((self.n_params,), "f32")
        self.w_compute = DeviceArray.zeros((self.n_params,), self.storage)
        self.activations = [DeviceArray((self.batch, self.sizes[i + 1]), self.storage)
                            for i in range(self.n_layers - 1)]
        self._acts_c = (ctypes.c_void_p * max(1, self.n_layers - 1))(*[a.ptr for a in self.activations])
        self.probs = DeviceArray((self.batch, self.sizes[-1]), "f32")
        self.actions = DeviceArray((self.batch,), "i32") if "argmax" in self.head else None
        self.training = bool(training)
        # ReLU sign bits of every hidden layer (uint32 [width / 32, batch], column-block-major): recorded by the
        # forward pass when training so that backward gates by bits instead of re-reading H.
        self.relu_bits = []
        self._bits_c = None
        if self.training and all(w % 32 == 0 for w in self.sizes[1:-1]) and self.n_layers > 1:
            self.relu_bits = [DeviceArray((self.sizes[i + 1] // 32, self.batch), "i32")
                              for i in range(self.n_layers - 1)]
            self._bits_c = (ctypes.c_void_p * (self.n_layers - 1))(*[b.ptr for b in self.relu_bits])
        self.grads = None
        self.scratch = None
        self.loss = None
        if self.training:
            self.grads = grads if grads is not None else DeviceArray.zeros((self.n_params,), "f32")
            nbytes = ctypes.c_size_t(0)
            _lib.call("sb_mlp_backward_scratch_bytes", self.n_layers, self._sizes_c, self.batch,
                      _lib.DTYPE_CODES[in_dtype], ctypes.byref(nbytes))
            self.scratch = DeviceArray((nbytes.value,), "u8")
            self.loss = DeviceArray.zeros((1,), "f32")

    # -- parameters ----------------------------------------------------------
    def load_weights(self, weights, biases=None):
        """Uploads per-layer [out, in] fp32 weights (and biases) into the flat buffers."""
        flat = np.zeros(self.n_params, np.float32)
        for i, w in enumerate(weights):
            w = np.asarray(w, np.float32)
            if w.shape != (self.sizes[i + 1], self.sizes[i]):
                raise ValueError("layer %d weight shape %s" % (i, w.shape))
            o = self.offsets[2 * i]
            flat[o:o + w.size] = w.ravel()
            if biases is not None:
                b = np.asarray(biases[i], np.float32)
                ob = self.offsets[2 * i + 1]
                flat[ob:ob + b.size] = b
        self.params.upload(flat)
        self.w_compute.upload(flat)       # the upload rounds to the storage type
        return self

    def get_weights(self):
        flat = self.params.numpy()
        ws, bs = [], []
        for i in range(self.n_layers):
            o, ob = self.offsets[2 * i], self.offsets[2 * i + 1]
            n = self.sizes[i + 1] * self.sizes[i]
            ws.append(flat[o:o + n].reshape(self.sizes[i + 1], self.sizes[i]).copy())
            bs.append(flat[ob:ob + self.sizes[i + 1]].copy())
        return ws, bs

    def save(self, path):
        """Checkpoint: the flat fp32 master parameter vector with the layer sizes (NumPy .npz)."""
        np.savez(path, params=self.params.numpy(), sizes=np.asarray(self.sizes, np.int64))

    def load(self, path):
        """Restores a checkpoint written by ``save`` (same architecture) into the master parameters
        and the compute copy."""
        with np.load(path) as ck:
            if [int(v) for v in ck["sizes"]] != self.sizes:
                raise ValueError("checkpoint is for layer sizes %s, the model has %s" % (list(ck["sizes"]), self.sizes))
            flat = np.asarray(ck["params"], np.float32)
        if flat.shape != (self.n_params,):
            raise ValueError("checkpoint holds %d parameters, the model %d" % (flat.size, self.n_params))
        self.params.upload(flat)
        self.w_compute.upload(flat)
        return self

    def split_flat(self, flat):
        """Views of a flat host vector as [(W_i, b_i), ...]."""
        out = []
        for i in range(self.n_layers):
            o, ob = self.offsets[2 * i], self.offsets[2 * i + 1]
            n = self.sizes[i + 1] * self.sizes[i]
            out.append((flat[o:o + n].reshape(self.sizes[i + 1], self.sizes[i]), flat[ob:ob + self.sizes[i + 1]]))
        return out

    # -- execution -----------------------------------------------------------
    def forward(self, x, mask=None, head_flags=None, stream=None, fused=None):
        """probs <- head(MLP(x)); returns the probs DeviceArray (and fills actions for argmax heads).
        A net built for training whose shape the fused kernel takes runs the whole pass as one launch that
        also writes the activations and sign words backward needs (``fused=False``: one GEMM per layer)."""
        flags = self.head_flags if head_flags is None else head_flags
        if fused is None:
            fused = self.training and self.batch > 0 and self._fused_ok()
        if fused:
            _lib.call("sb_mlp_forward_fused_train", self.n_layers, self._sizes_c, self.batch,
                      _lib.DTYPE_CODES[self.in_dtype], device_ptr(x), self.w_compute.ptr,
                      self.params.ptr if self.with_bias else None, self._acts_c, self._bits_c, flags, device_ptr(mask),
                      self.probs.ptr, device_ptr(self.actions) if flags & _lib.EPI_ARGMAX else None, stream_ptr(stream))
            return self.probs
        _lib.call("sb_mlp_forward", self.n_layers, self._sizes_c, self.batch, _lib.DTYPE_CODES[self.in_dtype],
                  device_ptr(x), self.w_compute.ptr, self.params.ptr if self.with_bias else None, self._acts_c,
                  self._bits_c, flags, device_ptr(mask), self.probs.ptr, device_ptr(self.actions) if flags & _lib.EPI_ARGMAX else None,
                  stream_ptr(stream))
        return self.probs

    def _fused_ok(self):
        if self.in_dtype not in ("bf16", "f16"):
            return False
        return bool(_lib.load().sb_mlp_fused_supported(self.n_layers, self._sizes_c, _lib.DTYPE_CODES[self.in_dtype]))

    def forward_fused(self, x, mask=None, head_flags=None, stream=None):
        """Forward pass as one persistent kernel (narrow nets: 16-bit class, hidden widths multiples of
        64 up to 256, at most 32 outputs); hidden activations never reach global memory.  Raises
        SpiralError (SB_ERR_UNSUPPORTED) for shapes outside those limits."""
        flags = self.head_flags if head_flags is None else head_flags
        _lib.call("sb_mlp_forward_fused", self.n_layers, self._sizes_c, self.batch,
                  _lib.DTYPE_CODES[self.in_dtype], device_ptr(x), self.w_compute.ptr,
                  self.params.ptr if self.with_bias else None, flags, device_ptr(mask), self.probs.ptr,
                  device_ptr(self.actions) if flags & _lib.EPI_ARGMAX else None, stream_ptr(stream))
        return self.probs

    def forward_no_alloc(self, x, out, mask=None, actions=None, head_flags=None, stream=None):
        """Forward pass whose hidden activations use the library's built-in 32 MiB workspace.

        For callers that may not allocate device memory (no allocator of their own, a context where
        allocation is forbidden, inside a stream capture).  `out` (fp32 [batch, actions]) and
        `actions` (int32 [batch], for argmax heads) are caller buffers.  Raises SpiralError
        (SB_ERR_TOO_LARGE) when batch x hidden widths does not fit.  Calls share the one workspace:
        do not overlap two of them on the GPU.
        """
        flags = self.head_flags if head_flags is None else head_flags
        _lib.call("sb_mlp_forward_static", self.n_layers, self._sizes_c, self.batch,
                  _lib.DTYPE_CODES[self.in_dtype], device_ptr(x), self.w_compute.ptr,
                  self.params.ptr if self.with_bias else None, flags, device_ptr(mask), device_ptr(out),
                  device_ptr(actions) if flags & _lib.EPI_ARGMAX else None, stream_ptr(stream))
        return out

    def backward(self, x, mask, target, global_batch=None, stream=None):
        """grads <- d(mean cross-entropy)/d(params) for this shard (after a masked-softmax forward)."""
        gb = self.batch if global_batch is None else int(global_batch)
        _lib.call("sb_mlp_backward", self.n_layers, self._sizes_c, self.batch, ctypes.c_float(1.0 / gb),
                  _lib.DTYPE_CODES[self.in_dtype], device_ptr(x), self.w_compute.ptr, self._acts_c, self._bits_c,
                  self.probs.ptr,
                  device_ptr(mask), device_ptr(target), device_ptr(self.grads), int(self.with_bias),
                  self.scratch.ptr, self.scratch.nbytes, self.loss.ptr, stream_ptr(stream))
        return self.grads

    def backward_dp(self, x, mask, target, grads_table, world_size, rank, global_batch=None, stream=None):
        """The backward pass of a data-parallel step: like ``backward``, but the weight-gradient GEMMs of
        the wide layers add their tiles straight into the gradient buffer of the rank that owns those rows
        (``grads_table``: HOST array of every rank's buffer, ``PeerUpdate.grads_table()``), over peer
        memory -- the reduce-scatter half of the gradient all-reduce done by the GEMM itself."""
        gb = self.batch * int(world_size) if global_batch is None else int(global_batch)
        _lib.call("sb_mlp_backward_dp", self.n_layers, self._sizes_c, self.batch, ctypes.c_float(1.0 / gb),
                  _lib.DTYPE_CODES[self.in_dtype], device_ptr(x), self.w_compute.ptr, self._acts_c, self._bits_c,
                  self.probs.ptr, device_ptr(mask), device_ptr(target), grads_table, int(world_size), int(rank),
                  int(self.with_bias), self.scratch.ptr, self.scratch.nbytes, self.loss.ptr, stream_ptr(stream))
        return self.grads

    def backward_layers(self, x, mask, target, first_layer, last_layer, global_batch=None, stream=None):
        """The backward pass of layers first_layer .. last_layer (descending); successive calls covering
        n_layers-1 .. 0 equal one ``backward``."""
        gb = self.batch if global_batch is None else int(global_batch)
        _lib.call("sb_mlp_backward_range", self.n_layers, self._sizes_c, self.batch, ctypes.c_float(1.0 / gb),
                  _lib.DTYPE_CODES[self.in_dtype], device_ptr(x), self.w_compute.ptr, self._acts_c, self._bits_c,
                  self.probs.ptr, device_ptr(mask), device_ptr(target), device_ptr(self.grads), int(self.with_bias),
                  self.scratch.ptr, self.scratch.nbytes, self.loss.ptr, int(first_layer), int(last_layer),
                  stream_ptr(stream))
        return self.grads

    def layer_dy(self, layer):
        """View of d(loss)/d(output of layer ``layer``) inside the backward scratch: [batch, width padded
        to 8] in the storage type.  Valid after ``backward_layers`` has processed ``layer`` and until it
        processes ``layer - 2`` (the two dY buffers alternate)."""
        off = ctypes.c_size_t(0)
        _lib.call("sb_mlp_backward_dy_offset", self.n_layers, self._sizes_c, self.batch,
                  _lib.DTYPE_CODES[self.in_dtype], int(layer), ctypes.byref(off))
        width = (self.sizes[layer + 1] + 7) // 8 * 8
        return self.scratch.view((self.batch, width), self.storage, off.value)

    def layer_segment(self, layer):
        """[begin, end) of layer `layer`'s weights and bias inside the flat parameter / gradient vectors."""
        end = self.offsets[2 * layer + 2] if layer + 1 < self.n_layers else self.n_params
        return self.offsets[2 * layer], end

    def sgd(self, lr, stream=None):
        _lib.call("sb_sgd_update", self.params.ptr, device_ptr(self.grads), self.w_compute.ptr,
                  ctypes.c_longlong(self.n_params), ctypes.c_float(lr), _lib.DTYPE_CODES[self.storage],
                  stream_ptr(stream))

    def train_step(self, x, mask, target, lr, stream=None):
        """Forward + backward + SGD on one GPU (no gradient exchange)."""
        _lib.call("sb_mlp_train_step", self.n_layers, self._sizes_c, self.batch, _lib.DTYPE_CODES[self.in_dtype],
                  device_ptr(x), self.params.ptr, self.w_compute.ptr, self._acts_c, self._bits_c, device_ptr(mask),
                  device_ptr(target), self.probs.ptr, device_ptr(self.grads), int(self.with_bias),
                  ctypes.c_float(lr), self.scratch.ptr, self.scratch.nbytes, self.loss.ptr, stream_ptr(stream))

    def flops_per_sample(self, training=False):
        f = sum(2 * self.sizes[i] * self.sizes[i + 1] for i in range(self.n_layers))
        if training:
            f = 3 * f - 2 * self.sizes[0] * self.sizes[1]     # no dgrad into the input
        return f


def to_storage(x, in_dtype):
    """Host fp32 array -> DeviceArray in the storage type of an arithmetic class."""
    return DeviceArray.from_numpy(np.asarray(x, np.float32), in_dtype)


class EnsemblePolicyMLP:
    """An ensemble of ``members`` policy nets of one architecture evaluated on ONE input batch in a
    single launch of the fused kernel (the reference builds such nets with ``layers.matmul_ensemble``,
    ml/layers.spi:468-471, and runs the graph once per member, ml/models.spi:47-49).

    16-bit arithmetic classes and the fused kernel's width limits only (input <= 512, hidden layers
    multiples of 64 up to 256, at most 64 outputs -- or 256 under a prefix mask of at most 64 columns).
    Outputs: ``probs`` fp32 [members, batch, n_out] and, with an argmax head, ``actions`` int32
    [members, batch].

    ``hidden_norm``: ln_l2 before every ReLU, as in the reference's nets (ml/layers.spi:594-603; no bias
    then).  ``decide`` (below) is the reference's per-decision call ml/models.spi:9-76.
    """

    def __init__(self, sizes, batch, members, in_dtype="f16", head=("masked_softmax",), with_bias=True,
                 hidden_norm=False):
        if in_dtype not in ("bf16", "f16"):
            raise ValueError("the fused ensemble forward runs in 'bf16' or 'f16'")
        self.sizes = [int(s) for s in sizes]
        self.n_layers = len(self.sizes) - 1
        self.batch, self.members = int(batch), int(members)
        self.in_dtype = self.storage = in_dtype
        self.head = tuple(head)
        self.head_flags = 0
        for h in self.head:
            self.head_flags |= HEAD_FLAGS[h]
        self.hidden_norm = bool(hidden_norm)
        self.with_bias = bool(with_bias) and not self.hidden_norm
        self.offsets = param_offsets(self.sizes)
        self.n_params = self.offsets[-1]
        self._sizes_c = (ctypes.c_int * len(self.sizes))(*self.sizes)
        self._decide = None
        self.params = DeviceArray.zeros((self.members, self.n_params), "f32")
        self.w_compute = DeviceArray.zeros((self.members, self.n_params), self.storage)
        self.probs = DeviceArray((self.members, self.batch, self.sizes[-1]), "f32")
        self.actions = DeviceArray((self.members, self.batch), "i32") if "argmax" in self.head else None

    def load_weights(self, member_weights, member_biases=None):
        """``member_weights[e][i]`` = layer i's [out, in] fp32 weights of member e (biases alike)."""
        if len(member_weights) != self.members:
            raise ValueError("%d weight sets for %d members" % (len(member_weights), self.members))
        flat = np.zeros((self.members, self.n_params), np.float32)
        for e, weights in enumerate(member_weights):
            for i, w in enumerate(weights):
                w = np.asarray(w, np.float32)
                if w.shape != (self.sizes[i + 1], self.sizes[i]):
                    raise ValueError("member %d layer %d weight shape %s" % (e, i, w.shape))
                o = self.offsets[2 * i]
                flat[e, o:o + w.size] = w.ravel()
                if member_biases is not None:
                    b = np.asarray(member_biases[e][i], np.float32)
                    ob = self.offsets[2 * i + 1]
                    flat[e, ob:ob + b.size] = b
        self.params.upload(flat)
        self.w_compute.upload(flat)       # the upload rounds to the storage type
        return self

    def forward(self, x, mask=None, stream=None):
        """All members on the batch ``x`` [batch, features] (storage type); returns ``probs``."""
        _lib.call("sb_mlp_forward_fused_ensemble", self.n_layers, self._sizes_c, self.batch, self.members,
                  _lib.DTYPE_CODES[self.in_dtype], device_ptr(x), self.w_compute.ptr,
                  self.params.ptr if self.with_bias else None, self.head_flags, device_ptr(mask), self.probs.ptr,
                  self.actions.ptr if self.actions is not None else None, stream_ptr(stream))
        return self.probs

    def forward_head(self, x, head=("masked_softmax",), prefix=-1, mask=None, seed=0, row_offset=0, position=0,
                     stream=None):
        """All members with the head given in full: ``head`` names from ``matmul.HEAD_FLAGS`` (softmax,
        regret matching, argmax, sample), legal columns ``j < prefix`` (or ``mask``), sampling from the
        Philox stream (seed, row_offset + row), member e using output ``position + e``.  Fills ``probs``,
        ``actions`` (argmax) and ``indices`` (sample)."""
        from .matmul import head_spec
        if "sample" in head and getattr(self, "indices", None) is None:
            self.indices = DeviceArray((self.members, self.batch), "i32")
        if "argmax" in head and self.actions is None:
            self.actions = DeviceArray((self.members, self.batch), "i32")
        spec = head_spec(tuple(head), prefix=prefix, mask=mask, argmax_out=self.actions if "argmax" in head else None,
                         sample_out=self.indices if "sample" in head else None, seed=seed, row_offset=row_offset,
                         position=position)
        _lib.call("sb_mlp_forward_fused_head", self.n_layers, self._sizes_c, self.batch, self.members,
                  _lib.DTYPE_CODES[self.in_dtype], device_ptr(x), self.w_compute.ptr,
                  self.params.ptr if self.with_bias else None, int(self.hidden_norm), ctypes.byref(spec),
                  self.probs.ptr, stream_ptr(stream))
        return self.probs

    def decide(self, seed, fields=None, widths=None, dense=None, x=None, head=("masked_softmax",), prefix=-1,
               mask=None, row_offset=0, stream=None):
        """One decision per game state: the reference's ``models.run`` (ml/models.spi:9-76).

        The states come either as compact records (``fields`` uint8 [batch, len(widths)] and optional
        ``dense`` values, serialised into the network input on the device) or as a ready input ``x``.
        Every member samples an action per state from its head, a member is drawn per state, and the
        result is a dict of device arrays: ``action`` int32 [batch], ``ensemble_id`` int32 [batch],
        ``sampling_prob_selected`` fp32 [batch], ``sampling_prob_ensemble`` fp32 [batch, members],
        plus the reference's tensors ``output_probs`` [members, batch, n_out] and ``output_indices``
        [members, batch].  Two kernel launches (one when ``x`` is given).  Buffers are created on the
        first call and reused."""
        if self._decide is None:
            b, e = self.batch, self.members
            self._decide = dict(
                x=DeviceArray((b, self.sizes[0]), self.storage), output_indices=DeviceArray((e, b), "i32"),
                ensemble_id=DeviceArray((b,), "i32"), action=DeviceArray((b,), "i32"),
                sampling_prob_selected=DeviceArray((b,), "f32"), sampling_prob_ensemble=DeviceArray((b, e), "f32"),
                tile_counters=DeviceArray.zeros(((b + 127) // 128,), "i32"))
        d = self._decide
        flags = 0
        for name in head:
            flags |= HEAD_FLAGS[name]
        a = _lib.DecideArgs()
        a.n_layers, a.sizes, a.members = self.n_layers, self._sizes_c, self.members
        a.in_dtype = _lib.DTYPE_CODES[self.in_dtype]
        a.w_compute, a.params = self.w_compute.ptr, (self.params.ptr if self.with_bias else None)
        a.hidden_norm, a.rows = int(self.hidden_norm), self.batch
        if fields is not None:
            widths = [int(w) for w in widths]
            self._widths_c = (ctypes.c_int * len(widths))(*widths)
            a.fields, a.n_fields, a.widths = device_ptr(fields), len(widths), self._widths_c
            a.dense, a.n_dense = device_ptr(dense), (0 if dense is None else int(dense.shape[1]))
            a.x = d["x"].ptr
        else:
            a.fields, a.n_fields, a.dense, a.n_dense = None, 0, None, 0
            a.x = device_ptr(x)
        a.head_flags, a.prefix, a.mask = flags, int(prefix), device_ptr(mask)
        a.seed, a.row_offset = int(seed), int(row_offset)
        a.output_probs, a.output_indices = self.probs.ptr, d["output_indices"].ptr
        a.ensemble_id, a.action = d["ensemble_id"].ptr, d["action"].ptr
        a.sampling_prob_selected, a.sampling_prob_ensemble = d["sampling_prob_selected"].ptr, d["sampling_prob_ensemble"].ptr
        a.tile_counters = d["tile_counters"].ptr
        _lib.call("sb_policy_decide", ctypes.byref(a), stream_ptr(stream))
        out = {k: d[k] for k in ("action", "ensemble_id", "sampling_prob_selected", "sampling_prob_ensemble",
                                 "output_indices")}
        out["output_probs"] = self.probs
        return out
