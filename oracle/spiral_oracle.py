"""NumPy restatement of the reference's dense-matmul path.  TEST INFRASTRUCTURE ONLY.

Each function cites the reference file:line (paths inside
mrakgr/Spiral-s-ml-library) whose arithmetic it restates.  The product never
imports this module; it is the checker used by tests/, the smoke check and the
CPU-baseline timing of bench.py.

Pinning.  The row operations (softmax, masked softmax, masked regret matching,
L2 row normalisation, argmax) are pinned against the reference's own golden
console outputs (tests/golden/primitives_golden.npz, extracted from
test_text_outputs/primitives/ by tests/golden/make_golden.py).  The GEMM has no
stored vectors in the reference (its self-test compares against cp.matmul on
unsaved random inputs, ml/matmul/run.spi:41,54-58); it is pinned instead against
the reference's own kernel, recompiled for sm_100a by oracle/build_ref.py and run
on the same inputs (tests/test_gpu_e_reference_kernel.py), at the one shape that
kernel is generated for.  Elsewhere the oracle is the definition
C = alpha*op(A)*op(B) + beta*C evaluated in float64.  Cross-entropy, dgrad, wgrad and SGD have no reference
implementation at all; they are defined here.
"""
import numpy as np

FLT_MAX = np.float32(3.402823466e38)


# ----------------------------------------------------------------------------
# input rounding of the tensor-core input classes
# ----------------------------------------------------------------------------
def round_bf16(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    r = np.where((u & np.uint32(0x7F800000)) == np.uint32(0x7F800000), u & np.uint32(0xFFFF0000), r)
    return r.view(np.float32).reshape(np.shape(x))


def round_f16(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def round_tf32(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (u + np.uint32(0x0FFF) + ((u >> np.uint32(13)) & np.uint32(1))) & np.uint32(0xFFFFE000)
    r = np.where((u & np.uint32(0x7F800000)) == np.uint32(0x7F800000), u, r)
    return r.view(np.float32).reshape(np.shape(x))


def round_input(x, in_dtype):
    """Value the arithmetic class `in_dtype` actually multiplies (kept as fp32)."""
    if in_dtype == "bf16":
        return round_bf16(x)
    if in_dtype == "f16":
        return round_f16(x)
    if in_dtype == "tf32":
        return round_tf32(x)
    return np.asarray(x, dtype=np.float32)


# ----------------------------------------------------------------------------
# GEMM   (ml/matmul/run.spi:21-26, ml/matmul/kernel.spi:25-240)
# ----------------------------------------------------------------------------
def matmul(a_trans, b_trans, alpha, a, b, beta, c, in_dtype="f32", exact=True):
    """Returns alpha * op(a) @ op(b) + beta * c as float32.

    a is stored [M,K] ([K,M] when a_trans); b is stored [K,N] ([N,K] when
    b_trans); c is [M,N] (ml/matmul/run.spi:22-23, kernel.spi:51-76).  The
    reference multiplies TF32-rounded inputs and accumulates in fp32
    (corecuda/wmma.spi:78-82,99-105).  With exact=True the products are summed
    in float64 (the tolerance classes absorb accumulation-order differences);
    exact=False uses NumPy's float32 matmul, the oracle the first benchmark
    configuration names.
    """
    a = round_input(a, in_dtype)
    b = round_input(b, in_dtype)
    opa = a.T if a_trans else a
    opb = b.T if b_trans else b
    if exact:
        prod = opa.astype(np.float64) @ opb.astype(np.float64)
        out = alpha * prod
        if beta != 0:
            out = out + beta * np.asarray(c, dtype=np.float64)
        return out.astype(np.float32)
    out = np.float32(alpha) * (opa @ opb)
    if beta != 0:
        out = out + np.float32(beta) * np.asarray(c, dtype=np.float32)
    return out.astype(np.float32)


def rel_frobenius(got, want):
    """||got - want||_F / ||want||_F (0 when both are all zero)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    den = np.linalg.norm(want)
    num = np.linalg.norm(got - want)
    return float(num / den) if den > 0 else float(num)


# ----------------------------------------------------------------------------
# elementwise and row operations
# ----------------------------------------------------------------------------
def relu(x):
    """layers.relu: BlockMap (max 0)  (ml/layers.spi:355)."""
    return np.maximum(np.asarray(x, dtype=np.float32), np.float32(0))


def ln_l2(x):
    """local_ln_l2: x / sum(x^2) per row, 0 where the sum is 0  (ml/primitives.spi:701-703)."""
    x = np.asarray(x, dtype=np.float32)
    s = np.sum(x * x, axis=-1, keepdims=True, dtype=np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        return np.where(s != 0, x / s, np.float32(0)).astype(np.float32)


def argmax(x):
    """local_argmax  (ml/primitives.spi:705-708).  The reference's tie order is
    unspecified (butterfly reduce); this oracle and the CUDA path both take the
    lowest index."""
    return np.argmax(np.asarray(x), axis=-1).astype(np.int32)


def discrete_sampling(x, u):
    """local_discrete_sampling (ml/primitives.spi:782-800) with the uniform numbers u in (0, 1] given:
    per row the first j with x[j] > 0 and cdf[j] >= u * (cdf at the last positive entry); -1 when the
    row has no positive entry.  Sums in index order, float32."""
    x = np.asarray(x, dtype=np.float32)
    u = np.asarray(u, dtype=np.float32)
    cdf = np.cumsum(x, axis=-1, dtype=np.float32)
    pos = x > 0
    top = np.max(np.where(pos, cdf, np.float32(0)), axis=-1).astype(np.float32)
    ok = pos & ((cdf - (u * top)[..., None].astype(np.float32)) >= 0)
    first = np.argmax(ok, axis=-1)
    return np.where(ok.any(axis=-1), first, -1).astype(np.int32)


# Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC 2011), the
# generator behind the reference's per-thread cuRAND state (curandStatePhilox4_32_10_t,
# corecuda/random.spi:9-24).  Pinned by the paper's known-answer vectors in tests/test_oracle_golden.py.
_PHILOX_M0, _PHILOX_M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85
_U32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(counter, key):
    """One block per element: `counter` = four arrays (or ints) of 32-bit words, `key` = two ints.
    Returns four uint32 arrays."""
    c = [np.asarray(x, dtype=np.uint64) & _U32 for x in counter]
    k0, k1 = int(key[0]) & 0xFFFFFFFF, int(key[1]) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = _PHILOX_M0 * c[0], _PHILOX_M1 * c[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & _U32
        hi1, lo1 = p1 >> np.uint64(32), p1 & _U32
        c = [hi1 ^ c[1] ^ np.uint64(k0), lo1, hi0 ^ c[3] ^ np.uint64(k1), lo0]
        k0, k1 = (k0 + _PHILOX_W0) & 0xFFFFFFFF, (k1 + _PHILOX_W1) & 0xFFFFFFFF
    return [x.astype(np.uint32) for x in c]


def philox_u32(seed, subsequence, position):
    """32-bit output number `position` of the stream (seed, subsequence): key = the 64-bit seed, counter =
    (position // 4 as 64 bits, subsequence as 64 bits), word position % 4 of the block -- the layout of
    curand_init(seed, subsequence, offset) followed by `position - offset` draws.  `subsequence` may be
    an array (one stream per row)."""
    sub = np.asarray(subsequence, dtype=np.uint64)
    pos = np.broadcast_to(np.asarray(position, dtype=np.uint64), sub.shape)
    block = pos >> np.uint64(2)
    words = philox4x32_10([block & _U32, block >> np.uint64(32), sub & _U32, sub >> np.uint64(32)],
                          [int(seed) & 0xFFFFFFFF, (int(seed) >> 32) & 0xFFFFFFFF])
    which = (pos & np.uint64(3)).astype(np.int64)
    return np.choose(which, words).astype(np.uint32)


def uniform_open_closed(x):
    """A 32-bit draw as a float32 in (0, 1]: x * 2^-32 + 2^-33 rounded once, the mapping of
    curand_uniform (corecuda/random.spi:84: "an uniform value in the (0,1] range")."""
    xf = np.asarray(x, dtype=np.uint32).astype(np.float32).astype(np.float64)
    return (xf * 2.0 ** -32 + 2.0 ** -33).astype(np.float32)


def philox_uniform(seed, subsequence, position):
    return uniform_open_closed(philox_u32(seed, subsequence, position))


def philox_below(seed, subsequence, position, bound):
    """Unbiased integers in [0, bound) by rejection (corecuda/random.spi:53-59: draw r, x = r mod bound,
    accept when r - x <= 2^32 - bound), draws taken at position, position + 1, ...; at most 8 tries."""
    sub = np.asarray(subsequence, dtype=np.uint64)
    out = np.zeros(sub.shape, dtype=np.uint32)
    done = np.zeros(sub.shape, dtype=bool)
    for attempt in range(8):
        r = philox_u32(seed, sub, np.uint64(position + attempt)).astype(np.uint64)
        x = r % np.uint64(bound)
        ok = (r - x) <= np.uint64(2 ** 32 - bound)
        out = np.where(done, out, x.astype(np.uint32))
        done = done | ok
        if done.all():
            break
    return out.astype(np.int32)


def binarize(x, modulo):
    """local_binarize (ml/primitives.spi:816-821): per row the word with bit j = (x[j] > 0), modulo
    `modulo`; rows of at most 32 values."""
    x = np.asarray(x)
    bits = (x > 0).astype(np.uint64) << np.arange(x.shape[-1], dtype=np.uint64)
    return (np.sum(bits, axis=-1, dtype=np.uint64) % np.uint64(modulo)).astype(np.uint32)


def softmax(x):
    """local_softmax: exp(x - mean(x)) normalised  (ml/primitives.spi:711-716)."""
    x = np.asarray(x, dtype=np.float32)
    e = np.exp(x - np.mean(x, axis=-1, keepdims=True, dtype=np.float32))
    return (e / np.sum(e, axis=-1, keepdims=True, dtype=np.float32)).astype(np.float32)


def prefix_mask(shape, size):
    """The mask layers.masked_softmax / masked_regret_matching instantiate: j < size
    (ml/layers.spi:409,416)."""
    m = np.zeros(shape, dtype=bool)
    m[..., :size] = True
    return m


def masked_softmax(x, mask):
    """local_masked_softmax  (ml/primitives.spi:748-759): subtract the mean of
    the legal entries, masked entries enter exp as -FLT_MAX (so contribute 0)."""
    x = np.asarray(x, dtype=np.float32)
    mask = np.asarray(mask, dtype=bool)
    count = np.sum(mask, axis=-1, keepdims=True).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        avg = np.sum(np.where(mask, x, np.float32(0)), axis=-1, keepdims=True, dtype=np.float32) / count
        e = np.exp(np.where(mask, x, -FLT_MAX) - avg)
        e = np.where(mask, e, np.float32(0))
        s = np.sum(e, axis=-1, keepdims=True, dtype=np.float32)
        out = e / s
    return np.where(np.isfinite(out), out, np.float32(0)).astype(np.float32)


def regret_matching(x):
    """local_regret_matching  (ml/primitives.spi:718-722)."""
    return masked_regret_matching(x, np.ones(np.shape(x), dtype=bool))


def masked_regret_matching(x, mask):
    """local_masked_regret_matching  (ml/primitives.spi:761-780): p = max(0,x) on
    legal entries; p / sum(p) if the sum is non-zero, else uniform over the
    legal entries; illegal entries are 0."""
    x = np.asarray(x, dtype=np.float32)
    mask = np.asarray(mask, dtype=bool)
    p = np.where(mask, np.maximum(x, np.float32(0)), np.float32(0))
    s = np.sum(p, axis=-1, keepdims=True, dtype=np.float32)
    count = np.sum(mask, axis=-1, keepdims=True).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        out = np.where(s != 0, p / s, np.float32(1) / count)
    out = np.where(mask, out, np.float32(0))
    return np.where(np.isfinite(out), out, np.float32(0)).astype(np.float32)


# ----------------------------------------------------------------------------
# dense layers and the policy MLP  (ml/layers.spi:227-240, 353-355, 408-420)
# ----------------------------------------------------------------------------
def dense(x, w, bias=None, in_dtype="f32", exact=True):
    """BlockMatmul: y = x @ w.T with w stored [out, in] (NT, alpha=1, beta=0;
    ml/layers.spi:229-235,467).  The reference has no bias; `bias` is the
    benchmark configurations' addition."""
    y = matmul(False, True, 1.0, x, w, 0.0, None, in_dtype=in_dtype, exact=exact)
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float32)
    return y.astype(np.float32)


def mlp_forward(x, weights, biases=None, mask=None, in_dtype="f32", head=("masked_softmax",),
                act_dtype=None, return_activations=False, exact=True):
    """Hidden layers dense+ReLU, last layer dense + row head.

    `act_dtype` rounds every hidden activation to the storage type the CUDA path
    keeps between layers (None = fp32).  Heads apply in the order
    masked_softmax, regret_matching; mask=None means every action is legal.
    Returns probabilities (and optionally the list [x, h1, ..., logits]).
    exact=False multiplies in float32 BLAS instead of float64 (CPU-baseline timing).
    """
    acts = [np.asarray(x, dtype=np.float32)]
    h = acts[0]
    n_layers = len(weights)
    for i, w in enumerate(weights):
        b = None if biases is None else biases[i]
        h = dense(h, w, b, in_dtype=in_dtype, exact=exact)
        if i < n_layers - 1:
            h = relu(h)
            if act_dtype is not None:
                h = round_input(h, act_dtype)
        acts.append(h)
    logits = h
    m = np.ones(logits.shape, dtype=bool) if mask is None else np.asarray(mask, dtype=bool)
    out = logits
    if "masked_softmax" in head:
        out = masked_softmax(out, m)
    if "regret_matching" in head:
        out = masked_regret_matching(out, m)
    if return_activations:
        return out, acts
    return out


def ensemble_forward(x, member_weights, member_biases=None, mask=None, in_dtype="f32", head=("masked_softmax",),
                     hidden_norm=False):
    """Every ensemble member's net on the same input (layers.matmul_ensemble, ml/layers.spi:468-471, run once
    per member, ml/models.spi:47-49): hidden layers dense [+ ln_l2] + ReLU rounded to the storage type, the
    last layer dense + row head.  Returns probabilities [members, rows, n_out]."""
    outs = []
    for e, ws in enumerate(member_weights):
        bs = None if member_biases is None else member_biases[e]
        h = np.asarray(x, dtype=np.float32)
        for i, w in enumerate(ws):
            h = dense(h, w, None if bs is None else bs[i], in_dtype=in_dtype)
            if i < len(ws) - 1:
                if hidden_norm:
                    h = ln_l2(h)
                h = round_input(relu(h), in_dtype)
        m = np.ones(h.shape, dtype=bool) if mask is None else np.asarray(mask, dtype=bool)
        if "masked_softmax" in head:
            h = masked_softmax(h, m)
        if "regret_matching" in head:
            h = masked_regret_matching(h, m)
        outs.append(h)
    return np.stack(outs)


def policy_decide(output_probs, seed, row_offset=0):
    """The per-decision tail of models.noinline_run (ml/models.spi:51-76) on the members' probabilities
    [members, rows, n_out]: member e samples an index per row with output e of the row's Philox stream
    (seed, row_offset + row) (local_discrete_sampling, ml/primitives.spi:782-800), a member is drawn per
    row with the outputs from `members` on (random.int_range, corecuda/random.spi:53-71), and the result is
    (action, ensemble_id, sampling_prob_selected, sampling_prob_ensemble [rows, members], output_indices)."""
    probs = np.asarray(output_probs, dtype=np.float32)
    members, rows, _ = probs.shape
    streams = np.uint64(row_offset) + np.arange(rows, dtype=np.uint64)
    indices = np.stack([discrete_sampling(probs[e], philox_uniform(seed, streams, e)) for e in range(members)])
    ensemble_id = philox_below(seed, streams, members, members)
    r = np.arange(rows)
    action = indices[ensemble_id, r]
    safe = np.maximum(action, 0)
    by_member = np.where(action[None, :] >= 0, probs[:, r, safe], np.float32(0))       # [members, rows]
    return action, ensemble_id, by_member[ensemble_id, r], np.ascontiguousarray(by_member.T), indices


def cross_entropy_loss(probs, target, mask=None):
    """Mean over rows of -sum_j target_j * log(probs_j) over legal j.  Not in the
    reference (it has no loss); defined by the benchmark's training configurations."""
    probs = np.asarray(probs, dtype=np.float64)
    target = np.asarray(target, dtype=np.float64)
    m = np.ones(probs.shape, dtype=bool) if mask is None else np.asarray(mask, dtype=bool)
    with np.errstate(divide="ignore"):
        lp = np.where(m, np.log(np.maximum(probs, 1e-38)), 0.0)
    return float(-np.sum(np.where(m, target * lp, 0.0)) / probs.shape[0])


def mlp_train_step(x, weights, biases, mask, target, lr, in_dtype="f32", act_dtype=None, global_batch=None,
                   exact=True):
    """One SGD step on cross-entropy(masked_softmax(logits), target).  Not in the
    reference (no backward pass exists there, ml/layers.spi:10 is CEM scratch).

    d logits = (softmax - target * legal) / global_batch on legal entries (the
    target is renormalised over legal entries by the caller); dgrad is NN
    (dX = dY @ W), wgrad is TN (dW = dY.T @ X), db = column sums; hidden
    gradients pass through ReLU'(h) = [h > 0].  Returns (new_weights,
    new_biases, loss, grads) with grads = [(dW, db), ...] already divided by
    the global batch.
    """
    probs, acts = mlp_forward(x, weights, biases, mask, in_dtype=in_dtype, head=("masked_softmax",),
                              act_dtype=act_dtype, return_activations=True, exact=exact)
    bsz = x.shape[0] if global_batch is None else global_batch
    m = np.ones(probs.shape, dtype=bool) if mask is None else np.asarray(mask, dtype=bool)
    tgt = np.where(m, np.asarray(target, dtype=np.float32), np.float32(0))
    loss = cross_entropy_loss(probs, tgt, m)
    tsum = np.sum(tgt, axis=-1, keepdims=True, dtype=np.float32)
    dy = np.where(m, probs * tsum - tgt, np.float32(0)).astype(np.float32) / np.float32(bsz)
    grads = [None] * len(weights)
    for i in range(len(weights) - 1, -1, -1):
        h_in = acts[i]
        dy_r = round_input(dy, in_dtype) if in_dtype != "f32" else dy
        dw = matmul(True, False, 1.0, dy_r, h_in, 0.0, None, in_dtype=in_dtype, exact=exact)   # [out,in] = dY.T @ X
        db = np.sum(dy, axis=0, dtype=np.float64).astype(np.float32)
        grads[i] = (dw, db)
        if i > 0:
            dx = matmul(False, False, 1.0, dy_r, weights[i], 0.0, None, in_dtype=in_dtype, exact=exact)  # dY @ W
            dy = np.where(acts[i] > 0, dx, np.float32(0)).astype(np.float32)
            if act_dtype is not None:
                dy = round_input(dy, act_dtype)
    new_w = [np.asarray(w, np.float32) - np.float32(lr) * g[0] for w, g in zip(weights, grads)]
    new_b = None
    if biases is not None:
        new_b = [np.asarray(b, np.float32) - np.float32(lr) * g[1] for b, g in zip(biases, grads)]
    return new_w, new_b, loss, grads


# ----------------------------------------------------------------------------
# seeded synthetic inputs of the benchmark configurations
# ----------------------------------------------------------------------------
def rng(seed):
    return np.random.Generator(np.random.Philox(seed))


def kaiming_uniform(gen, fan_out, fan_in):
    """U(-sqrt(6/fan_in), +sqrt(6/fan_in)), stored [out, in] like layers.weight
    (ml/layers.spi:467; the reference itself initialises N(0, 0.1), :460-463)."""
    bound = np.sqrt(6.0 / fan_in)
    return gen.uniform(-bound, bound, size=(fan_out, fan_in)).astype(np.float32)


def mlp_weights(seed, sizes):
    gen = rng(seed)
    ws = [kaiming_uniform(gen, sizes[i + 1], sizes[i]) for i in range(len(sizes) - 1)]
    bs = [np.zeros(sizes[i + 1], dtype=np.float32) for i in range(len(sizes) - 1)]
    return ws, bs


def encode_states(fields, widths, dense=None):
    """Dense network input from compact game states: field j (an integer in [0, widths[j]]) becomes
    a one-hot group of widths[j] features, the value widths[j] (or anything above) meaning "none"
    (all zeros), the way corebase/pickler.spi:20-37 serialises a bounded int into the input tensor
    that ml/models.spi:30-41 zeroes first; `dense` [rows, n] values follow unchanged."""
    fields = np.asarray(fields)
    rows = fields.shape[0]
    total = int(np.sum(widths))
    n_dense = 0 if dense is None else dense.shape[1]
    x = np.zeros((rows, total + n_dense), dtype=np.float32)
    col = 0
    r = np.arange(rows)
    for j, w in enumerate(widths):
        idx = fields[:, j].astype(np.int64)
        ok = idx < w
        x[r[ok], col + idx[ok]] = 1.0
        col += w
    if n_dense:
        x[:, total:] = dense
    return x


LEDUC_WIDTHS = (3, 4, 14, 3) + (1,) * 8
HOLDEM_WIDTHS = (4, 13) * 7


def leduc_states(seed, batch):
    """Compact Leduc states: uint8 [batch, 12] = card(3) | community(4) | pot(14) | raises left(3) |
    8 history bits (width-1 fields: 0 = set, 1 = clear); plus a mask with 2 or 3 legal actions of 3."""
    gen = rng(seed)
    cols = [gen.integers(0, w, size=batch) for w in LEDUC_WIDTHS[:4]]
    bits = gen.random((batch, 8)) < 0.5
    fields = np.concatenate([np.stack(cols, axis=1), np.where(bits, 0, 1)], axis=1).astype(np.uint8)
    mask = np.ones((batch, 3), dtype=np.uint8)
    drop = gen.integers(0, 4, size=batch)          # 3 = keep all three legal
    rows = np.arange(batch)[drop < 3]
    mask[rows, drop[drop < 3]] = 0
    return fields, mask


def leduc_inputs(seed, batch):
    """[batch, 32] {0,1} states (the encoding of leduc_states) and the legal-action mask."""
    fields, mask = leduc_states(seed, batch)
    return encode_states(fields, LEDUC_WIDTHS), mask


def holdem_states(seed, batch, features=512, actions=10):
    """Compact Hold'em states: uint8 [batch, 14] = 7 card slots x (suit in [0,4], rank in [0,13]),
    the top value meaning an empty slot (game/nl_hu_holdem/model_cem.spi:13-15,26-27; trailing
    board slots are empty according to a random street); float32 [batch, features - 119]
    continuous U[0,1) stack/pot values; and a mask with 2..actions legal actions."""
    gen = rng(seed)
    fields = np.zeros((batch, 14), dtype=np.uint8)
    street_cards = np.array([2, 5, 6, 7])[gen.integers(0, 4, size=batch)]
    for slot in range(7):
        live = street_cards > slot
        suit = gen.integers(0, 4, size=batch)
        rank = gen.integers(0, 13, size=batch)
        fields[:, 2 * slot] = np.where(live, suit, 4)
        fields[:, 2 * slot + 1] = np.where(live, rank, 13)
    dense = gen.random((batch, features - 119), dtype=np.float32)
    mask = (gen.random((batch, actions)) < 0.6).astype(np.uint8)
    mask[:, 0] = 1
    mask[:, 1] = 1
    return fields, dense, mask


def holdem_inputs(seed, batch, features=512, actions=10):
    """[batch, 512]: 119 {0,1} card features then the continuous values (the encoding of
    holdem_states) and the legal-action mask."""
    fields, dense, mask = holdem_states(seed, batch, features, actions)
    return encode_states(fields, HOLDEM_WIDTHS, dense), mask


def random_target(seed, mask):
    """Random fp32 target distribution over the legal actions of each row."""
    gen = rng(seed)
    t = gen.random(mask.shape, dtype=np.float32) * (np.asarray(mask) != 0)
    return (t / np.sum(t, axis=-1, keepdims=True)).astype(np.float32)
