"""GEMM call surface: the reference's ``matmul_tf32 a_trans b_trans alpha a b beta c``.

Reference: ml/matmul/run.spi:21-26 -- M and N come from ``c``'s shape, K from
``a``'s (swapped when ``a_trans``), every tensor is row-major and ``c`` is
updated in place: ``c <- alpha * op(a) @ op(b) + beta * c``.
"""
import ctypes

from . import _lib
from .device import device_ptr, dtype_tag, stream_ptr

EPILOGUE_FLAGS = {
    "bias": _lib.EPI_BIAS, "relu": _lib.EPI_RELU, "relu_grad": _lib.EPI_RELU_GRAD,
    "masked_softmax": _lib.EPI_MASKED_SOFTMAX, "regret_matching": _lib.EPI_REGRET_MATCHING,
    "argmax": _lib.EPI_ARGMAX, "relu_mask_out": _lib.EPI_RELU_MASK_OUT, "relu_grad_mask": _lib.EPI_RELU_GRAD_MASK,
    "colsum_out": _lib.EPI_COLSUM_OUT, "ln_l2": _lib.EPI_LN_L2,
}


def _shape2(x, what):
    shape = tuple(getattr(x, "shape", ()))
    if len(shape) != 2:
        raise ValueError("%s must be a 2-D array, got shape %s" % (what, shape))
    return int(shape[0]), int(shape[1])


def _dims(a_trans, b_trans, a, b, c):
    m, n = _shape2(c, "c")
    ar, ac = _shape2(a, "a")
    br, bc = _shape2(b, "b")
    am, k = (ac, ar) if a_trans else (ar, ac)
    bk, bn = (bc, br) if b_trans else (br, bc)
    if am != m or bn != n or bk != k:
        raise ValueError("shape mismatch: op(a) is %dx%d, op(b) is %dx%d, c is %dx%d" % (am, k, bk, bn, m, n))
    return m, n, k


_F32X3_WORKSPACES = {}


def _f32x3_aligned(a_trans, b_trans, m, n, k):
    """Contiguous dimensions are multiples of 4 elements (16-byte row pitches for the split operands)."""
    return n % 4 == 0 and (m % 4 == 0 if a_trans else k % 4 == 0) and (k % 4 == 0 if b_trans else n % 4 == 0)


def _f32x3_workspace(m, n, k, stream):
    from .device import DeviceArray
    need = ctypes.c_size_t(0)
    _lib.call("sb_matmul_f32_workspace_bytes", m, n, k, ctypes.byref(need))
    key = stream_ptr(stream) or 0
    ws = _F32X3_WORKSPACES.get(key)
    if ws is None or ws.nbytes < need.value:
        if ws is not None:
            _lib.call("sb_stream_sync", stream_ptr(stream))      # the old buffer may still be in use
        ws = DeviceArray((need.value,), "u8")
        _F32X3_WORKSPACES[key] = ws
    return ws


def matmul(a_trans, b_trans, alpha, a, b, beta, c, in_dtype=None, epilogue=(), bias=None, mask=None,
           aux_in=None, aux_out=None, stream=None):
    """``c <- alpha * op(a) @ op(b) + beta * c`` with an optional fused epilogue.

    ``in_dtype``: 'f32' (FFMA, 1e-5 class), 'tf32' (fp32 storage, TF32 multiply),
    'bf16', 'f16'; by default fp32 storage runs as 'tf32', the reference's own
    arithmetic.  ``epilogue``: iterable of names from EPILOGUE_FLAGS.
    """
    m, n, k = _dims(bool(a_trans), bool(b_trans), a, b, c)
    storage = dtype_tag(a)
    fp32_storage = ("f32", "tf32")                 # 'tf32' tags fp32 storage whose values are TF32-rounded
    if storage != dtype_tag(b) and not (storage in fp32_storage and dtype_tag(b) in fp32_storage):
        raise TypeError("a and b must share a storage dtype (%s vs %s)" % (storage, dtype_tag(b)))
    if in_dtype is None:
        in_dtype = "tf32" if storage in ("f32", "tf32") else storage
    if (in_dtype in ("f32", "tf32")) != (storage in ("f32", "tf32")) or \
            (in_dtype in ("bf16", "f16") and in_dtype != storage):
        raise TypeError("in_dtype %s does not match the storage dtype %s" % (in_dtype, storage))
    out_dtype = dtype_tag(c)   # a 'tf32'-tagged output is fp32 storage rounded to TF32
    epi = 0
    for name in epilogue:
        epi |= EPILOGUE_FLAGS[name]
    if in_dtype == "f32" and out_dtype == "f32" and not (epi & ~(_lib.EPI_BIAS | _lib.EPI_RELU)) and k > 0 \
            and _f32x3_aligned(bool(a_trans), bool(b_trans), m, n, k) and device_ptr(c) % 16 == 0:
        # fp32 class on the tensor cores (3 x TF32); the split operands live in a workspace this host
        # keeps per stream and grows on demand (the C ABI itself allocates nothing).
        ws = _f32x3_workspace(m, n, k, stream)
        _lib.call("sb_matmul_f32x3", int(bool(a_trans)), int(bool(b_trans)), ctypes.c_float(alpha), device_ptr(a),
                  device_ptr(b), ctypes.c_float(beta), device_ptr(c), m, n, k, epi, device_ptr(bias), ws.ptr,
                  ws.nbytes, stream_ptr(stream))
        return c
    _lib.call("sb_matmul_ex", int(bool(a_trans)), int(bool(b_trans)), ctypes.c_float(alpha),
              device_ptr(a), device_ptr(b), ctypes.c_float(beta), device_ptr(c), m, n, k,
              _lib.DTYPE_CODES[in_dtype], _lib.DTYPE_CODES[out_dtype], epi, device_ptr(bias),
              device_ptr(mask), device_ptr(aux_in), device_ptr(aux_out), stream_ptr(stream))
    return c


HEAD_FLAGS = {"masked_softmax": _lib.EPI_MASKED_SOFTMAX, "softmax": _lib.EPI_MASKED_SOFTMAX,
              "regret_matching": _lib.EPI_REGRET_MATCHING, "argmax": _lib.EPI_ARGMAX, "sample": _lib.EPI_SAMPLE,
              "binarize": _lib.EPI_BINARIZE}


def head_spec(head=(), prefix=-1, mask=None, argmax_out=None, sample_out=None, hash_out=None, modulo=0,
              seed=0, row_offset=0, position=0):
    """The ctypes ``sb_head_spec`` of a row head: ``head`` names from HEAD_FLAGS; legal columns are
    ``j < prefix`` when ``prefix >= 0`` (the reference's ``masked_softmax size`` etc.), else ``mask``,
    else all; a sampling head draws output ``position`` of the Philox stream (seed, row_offset + row)."""
    flags = 0
    for name in head:
        flags |= HEAD_FLAGS[name]
    return _lib.HeadSpec(flags, int(prefix), device_ptr(mask), device_ptr(argmax_out), device_ptr(sample_out),
                         device_ptr(hash_out), int(modulo), int(seed), int(row_offset), int(position))


def matmul_head(a_trans, b_trans, alpha, a, b, beta, c, spec, in_dtype=None, epilogue=(), bias=None, stream=None):
    """``c <- head(alpha * op(a) @ op(b) + beta * c (+ bias) (relu))`` with the row head ``spec``
    (``head_spec(...)``); fp32 output.  One launch for rows of up to 64 columns, or up to 256 under a
    prefix mask of at most 64 columns; nothing is allocated."""
    m, n, k = _dims(bool(a_trans), bool(b_trans), a, b, c)
    storage = dtype_tag(a)
    if in_dtype is None:
        in_dtype = "tf32" if storage in ("f32", "tf32") else storage
    epi = 0
    for name in epilogue:
        epi |= EPILOGUE_FLAGS[name]
    _lib.call("sb_matmul_head", int(bool(a_trans)), int(bool(b_trans)), ctypes.c_float(alpha), device_ptr(a),
              device_ptr(b), ctypes.c_float(beta), device_ptr(c), m, n, k, _lib.DTYPE_CODES[in_dtype], epi,
              device_ptr(bias), ctypes.byref(spec), stream_ptr(stream))
    return c


def matmul_tf32(a_trans, b_trans, alpha, a, b, beta, c, stream=None):
    """Drop-in for the reference's ``matmul_tf32`` (fp32 storage, TF32 multiply, fp32 accumulate)."""
    m, n, k = _dims(bool(a_trans), bool(b_trans), a, b, c)
    for x, what in ((a, "a"), (b, "b"), (c, "c")):
        if dtype_tag(x) not in ("f32", "tf32"):
            raise TypeError("matmul_tf32: %s must be fp32" % what)
    _lib.call("sb_matmul_tf32", int(bool(a_trans)), int(bool(b_trans)), ctypes.c_float(alpha),
              device_ptr(a), device_ptr(b), ctypes.c_float(beta), device_ptr(c), m, n, k,
              stream_ptr(stream))
    return c


def matmul_plan(a_trans, b_trans, m, n, k, in_dtype="tf32"):
    """Tile plan of the tensor-core path: dict(block_m, block_n, block_k, stages, grid).

    Counterpart of matmul_config_tf32 (ml/matmul/run.spi:8-19); unlike it, no
    divisibility of m, n, k by the tile is demanded (ragged edges are zero-filled).
    """
    plan = (ctypes.c_int * 5)()
    _lib.call("sb_matmul_plan", int(bool(a_trans)), int(bool(b_trans)), int(m), int(n), int(k),
              _lib.DTYPE_CODES[in_dtype], 0, plan)
    return dict(zip(("block_m", "block_n", "block_k", "stages", "grid"), list(plan)))
