"""Layer-graph builder with the reference's names, run on the fused GEMM path.

Mirrors the dense subset of ml/layers.spi: graph builders ``input``, ``matmul``,
``relu``, ``softmax``, ``masked_softmax``, ``regret_matching``,
``masked_regret_matching``, ``argmax``, ``ln_l2``, ``matmul_ensemble``,
``masked_softmax_and_discrete_sample``, ``binarize`` (:347-436, 467-471, 482-484), the
arena planner ``create_model`` (:127-172, 486-490), ``pass_init`` (:307, weights
N(0, 0.1) as weight_init :460-463), ``key_extract`` (:321-325) and
``graph_run_host`` (:339-344).

Differences by design: the reference emits one device function per node and a
global-memory pass for every activation and head; here ``graph_run_host`` fuses
``matmul -> relu`` and ``matmul -> head`` chains into one GEMM launch each, and
only nodes that cannot be fused run as stand-alone kernels.  Tensors are 3-D in
the reference (blocks, rows, features); the leading dimensions are the batch.
"""
import numpy as np

from . import primitives
from .device import DeviceArray
from .matmul import matmul as _matmul

WEIGHT_ID, WORKSPACE_ID, WEIGHT_ADJOINT_ID = 0, 1, 2     # ml/layers.spi:6-12
CONSTANT_SEED = 12344321                                 # corecuda/cupy.spi:6
_ALIGN = 256                                             # bytes; the reference aligns to 16 (partitionm.spi:3-4)


class Node:
    """One graph node; ``dims`` is the shape of its output tensor."""

    def __init__(self, op, src=None, dims=None, **attrs):
        self.op, self.src, self.dims, self.attrs = op, src, tuple(dims), attrs
        self.offset = None        # byte offset of the output in the workspace arena
        self.weight_offset = None

    @property
    def rows(self):
        return int(np.prod(self.dims[:-1]))

    @property
    def cols(self):
        return int(self.dims[-1])


def input(key, dims):
    """A keyed workspace tensor the caller fills (layers.input, ml/layers.spi:482-484)."""
    return Node("input", None, dims, key=key)


def matmul(in_out, x):
    """Dense layer y = x W^T with W stored [out, in]; ``in_out`` = (in, out) as in ``matmul (b,a) x``
    (ml/layers.spi:467: BlockMatmul(x, weight (a,b)))."""
    fan_in, fan_out = int(in_out[0]), int(in_out[1])
    if x.cols != fan_in:
        raise ValueError("matmul: input has %d features, the layer expects %d" % (x.cols, fan_in))
    return Node("matmul", x, x.dims[:-1] + (fan_out,), fan_in=fan_in, fan_out=fan_out)


def matmul_ensemble(ens_in_out, x):
    """Dense layer with one weight matrix per ensemble member: ``ens_in_out`` = (members, in, out) as in
    ``matmul_ensemble (c,b,a) x`` (ml/layers.spi:468-471: weights (c,a,b), the member picked by the
    ``ensemble`` index the graph is run with)."""
    members, fan_in, fan_out = (int(v) for v in ens_in_out)
    if members < 1:
        raise ValueError("matmul_ensemble: at least one member")
    if x.cols != fan_in:
        raise ValueError("matmul_ensemble: input has %d features, the layer expects %d" % (x.cols, fan_in))
    return Node("matmul", x, x.dims[:-1] + (fan_out,), fan_in=fan_in, fan_out=fan_out, members=members)


def relu(x):
    return Node("relu", x, x.dims)


def softmax(x):
    return Node("softmax", x, x.dims, size=-1)


def masked_softmax(size, x):
    """Legal iff column index < size (ml/layers.spi:408-414)."""
    return Node("softmax", x, x.dims, size=int(size))


def regret_matching(x):
    return Node("regret_matching", x, x.dims, size=-1)


def masked_regret_matching(size, x):
    return Node("regret_matching", x, x.dims, size=int(size))


def ln_l2(x):
    return Node("ln_l2", x, x.dims)


def argmax(x):
    """Index of the row maximum; the output keeps a trailing dimension of 1 (one int32 per row)."""
    return Node("argmax", x, x.dims[:-1] + (1,))


def binarize(modulo, x):
    """Row hash of the signs, modulo ``modulo`` (ml/layers.spi:433-436); the output keeps a trailing
    dimension of 1 (one unsigned value per row, stored as int32)."""
    if x.cols > 32:
        raise ValueError("binarize: rows of at most 32 values")
    return Node("binarize", x, x.dims[:-1] + (1,), modulo=int(modulo))


def masked_softmax_and_discrete_sample(size, x):
    """Prefix-masked softmax followed by one sampled index per row (ml/layers.spi:422-431).  The node's
    output is the int32 index tensor [..., 1]; its source node holds the probabilities.  The uniform
    numbers come from the caller (``Model.uniforms(node).upload(u)``, one in (0, 1] per row) or, when
    ``graph_run_host`` is given a seed, are drawn on the device inside the head from a Philox4x32-10
    stream per row, as the reference draws them from its per-thread generator."""
    probs = Node("softmax", x, x.dims, size=int(size))
    return Node("sample", probs, x.dims[:-1] + (1,))


class Model:
    """Planned graph + its three arenas (weights, workspace, weight adjoint), ml/layers.spi:486-502."""

    def __init__(self, graph, in_dtype):
        self.graph, self.in_dtype = graph, in_dtype
        self.nodes = []
        n = graph
        while n is not None:
            self.nodes.append(n)
            n = n.src
        self.nodes.reverse()
        if self.nodes[0].op != "input":
            raise ValueError("a graph must start at an input node")
        sizes = [0, 0, 0]
        for n in self.nodes:                      # pass_calculate_partitions, ml/layers.spi:127-172
            if n.op == "matmul":
                n.weight_offset = sizes[WEIGHT_ID]
                member_bytes = _round_up(n.attrs["fan_in"] * n.attrs["fan_out"] * 4, _ALIGN)
                n.attrs["member_bytes"] = member_bytes
                sizes[WEIGHT_ID] += member_bytes * n.attrs.get("members", 1)
            n.offset = sizes[WORKSPACE_ID]
            sizes[WORKSPACE_ID] += _round_up(n.rows * (n.cols if n.op not in ("argmax", "sample", "binarize") else 1) * 4, _ALIGN)
            if n.op == "sample":
                n.attrs["uniform_offset"] = sizes[WORKSPACE_ID]
                sizes[WORKSPACE_ID] += _round_up(n.rows * 4, _ALIGN)
        self.partition_bytes = tuple(sizes)
        self.arenas = None

    def allocate(self):
        if self.arenas is None:
            self.arenas = [DeviceArray.zeros((max(b, 16),), "u8") for b in self.partition_bytes]
        return self

    def tensor(self, node, rounded=False):
        """Typed view of a node's output inside the workspace arena.  ``rounded``: tagged 'tf32' so that the
        GEMM that writes it rounds the values to TF32 (the input of the next tensor-core layer)."""
        if node.op in ("argmax", "sample", "binarize"):
            return self.arenas[WORKSPACE_ID].view((node.rows,), "i32", node.offset)
        return self.arenas[WORKSPACE_ID].view((node.rows, node.cols),
                                              "tf32" if rounded and self.in_dtype == "tf32" else "f32", node.offset)

    def uniforms(self, node):
        """The fp32 [rows] tensor of uniform numbers a sample node consumes."""
        return self.arenas[WORKSPACE_ID].view((node.rows,), "f32", node.attrs["uniform_offset"])

    def weight(self, node, ensemble=0):
        """The [out, in] weight matrix of a matmul node (of member ``ensemble`` for an ensemble layer)."""
        members = node.attrs.get("members", 1)
        if not 0 <= ensemble < members:
            if members == 1:
                ensemble = 0            # plain layers are shared by all members
            else:
                raise IndexError("ensemble member %d of %d" % (ensemble, members))
        # In the TF32 class the view is tagged 'tf32': an upload rounds the weights to TF32 (nearest even)
        # once, as the reference rounds every operand element when it loads a fragment
        # (ml/matmul/kernel.spi:197,212); the tensor core itself would truncate unrounded fp32.
        return self.arenas[WEIGHT_ID].view((node.attrs["fan_out"], node.attrs["fan_in"]),
                                           "tf32" if self.in_dtype == "tf32" else "f32",
                                           node.weight_offset + ensemble * node.attrs["member_bytes"])


def _round_up(x, a):
    return (x + a - 1) // a * a


def create_model(graph, in_dtype="tf32", allocate=True):
    """Plans the arenas of ``graph`` (and allocates them).  ``in_dtype``: 'tf32' (the reference's
    arithmetic, default) or 'f32' (FFMA)."""
    if in_dtype not in ("tf32", "f32"):
        raise ValueError("layer graphs store fp32; in_dtype must be 'tf32' or 'f32'")
    model = Model(graph, in_dtype)
    return model.allocate() if allocate else model


def model_to_model_ptrs(model):
    """(weights, workspace, weight_adjoint) device pointers, the kernel arguments of ml/layers.py:4500."""
    return tuple(a.ptr for a in model.arenas)


def pass_init(model, seed=CONSTANT_SEED, std=0.1):
    """Initialises every weight tensor N(0, std^2) (weight_init, ml/layers.spi:460-463)."""
    gen = np.random.Generator(np.random.Philox(seed))
    for n in model.nodes:
        if n.op == "matmul":
            for e in range(n.attrs.get("members", 1)):
                w = gen.normal(0.0, std, size=(n.attrs["fan_out"], n.attrs["fan_in"])).astype(np.float32)
                model.weight(n, e).upload(w)
    return model


def get_weights(model, ensemble=0):
    return [model.weight(n, ensemble).numpy() for n in model.nodes if n.op == "matmul"]


def key_extract(model, key):
    """The workspace tensor registered under ``key`` (ml/layers.spi:321-325)."""
    for n in model.nodes:
        if n.op == "input" and n.attrs["key"] == key:
            return model.tensor(n)
    raise KeyError(key)


def graph_run_host(model, stream=None, ensemble=0, seed=None, row_offset=0):
    """Runs the graph (ml/layers.spi:339-344) and returns the output tensor of the last node.
    ``ensemble`` picks the member whose weights the ``matmul_ensemble`` layers use, as the reference's
    ``graph_run_host model {ensemble}`` does (ml/layers.spi:623); plain layers are the same for all.
    ``seed``: sample nodes draw on the device, row r from output ``ensemble`` of the Philox stream
    (seed, row_offset + r) -- one draw per member and row, like the reference's per-thread generator
    that every member's run advances (ml/models.spi:47-49); without a seed they use the uniform numbers
    the caller uploaded into ``model.uniforms(node)``.

    Fusion: ``matmul [-> ln_l2] -> relu`` is one GEMM launch, and so is ``matmul -> softmax /
    regret_matching [-> sample] | argmax | binarize`` (a prefix mask is an argument of the head: no mask
    matrix, no allocation, no synchronisation); everything else runs as a stand-alone kernel."""
    nodes = model.nodes
    tc = model.in_dtype == "tf32"
    i = 1
    while i < len(nodes):
        n = nodes[i]
        src = model.tensor(n.src)
        if n.op == "matmul":
            j = i + 1
            w = model.weight(n, ensemble)
            # hidden layer: [ln_l2 ->] relu
            k, epilogue = j, []
            if tc and k + 1 < len(nodes) and nodes[k].op == "ln_l2" and nodes[k + 1].op == "relu" \
                    and n.cols % 32 == 0 and n.cols <= 256:
                epilogue, k = ["ln_l2", "relu"], k + 2
            elif k < len(nodes) and nodes[k].op == "relu":
                epilogue, k = ["relu"], k + 1
            if epilogue:
                feeds_matmul = k < len(nodes) and nodes[k].op == "matmul"
                _matmul(False, True, 1.0, src, w, 0.0, model.tensor(nodes[k - 1], rounded=feeds_matmul),
                        in_dtype=model.in_dtype, epilogue=tuple(epilogue), stream=stream)
                i = k
                continue
            # row head: softmax and regret matching fuse (in that order) when they share one prefix,
            # then one of sample / argmax; or the sign hash by itself
            head, size, last, k = [], None, n, j
            while k < len(nodes) and nodes[k].op in ("softmax", "regret_matching"):
                want = "masked_softmax" if nodes[k].op == "softmax" else "regret_matching"
                if want in head or (want == "masked_softmax" and "regret_matching" in head):
                    break
                if size is not None and nodes[k].attrs["size"] != size:
                    break
                size = nodes[k].attrs["size"]
                head.append(want)
                last, k = nodes[k], k + 1
            kw = {}
            if head and k < len(nodes) and nodes[k].op == "sample" and seed is not None:
                head.append("sample")
                kw = dict(sample_out=model.tensor(nodes[k]), seed=int(seed), row_offset=int(row_offset), position=int(ensemble))
                k += 1
            elif head and k < len(nodes) and nodes[k].op == "argmax":
                head.append("argmax")
                kw = dict(argmax_out=model.tensor(nodes[k]))
                k += 1
            elif not head and k < len(nodes) and nodes[k].op == "binarize" and n.cols <= 32:
                head.append("binarize")
                kw = dict(hash_out=model.tensor(nodes[k]), modulo=nodes[k].attrs["modulo"])
                k += 1
            if head:
                from .matmul import head_spec, matmul_head
                spec = head_spec(tuple(head), prefix=-1 if size is None else size, **kw)
                matmul_head(False, True, 1.0, src, w, 0.0, model.tensor(last), spec, in_dtype=model.in_dtype, stream=stream)
                i = k
                continue
            _matmul(False, True, 1.0, src, w, 0.0, model.tensor(n), in_dtype=model.in_dtype, stream=stream)
            i = j
            continue
        out = model.tensor(n)
        if n.op == "relu":
            primitives.relu(src, out, stream=stream)
        elif n.op == "softmax":
            primitives.softmax(src, out, prefix=n.attrs["size"], stream=stream)
        elif n.op == "regret_matching":
            primitives.regret_matching(src, out, prefix=n.attrs["size"], stream=stream)
        elif n.op == "ln_l2":
            primitives.ln_l2(src, out, stream=stream)
        elif n.op == "argmax":
            primitives.argmax(src, out, stream=stream)
        elif n.op == "binarize":
            primitives.binarize(n.attrs["modulo"], src, out, stream=stream)
        elif n.op == "sample":
            if seed is not None:
                primitives.sample_seeded(src, out, seed, row_offset=row_offset, position=ensemble, stream=stream)
            else:
                primitives.sample(src, model.uniforms(n), out, stream=stream)
        else:
            raise ValueError("unknown node %r" % n.op)
        i += 1
    return model.tensor(nodes[-1])
