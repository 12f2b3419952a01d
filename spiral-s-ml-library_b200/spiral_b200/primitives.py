"""Stand-alone row / elementwise operations (reference: ml/primitives.spi:701-780, ml/layers.spi:353-420)."""
from . import _lib
from .device import device_ptr, stream_ptr


def _rows_cols(x):
    shape = tuple(x.shape)
    if len(shape) < 1:
        raise ValueError("row operation on a 0-d array")
    cols = int(shape[-1])
    rows = 1
    for s in shape[:-1]:
        rows *= int(s)
    return rows, cols


def relu(x, out=None, stream=None):
    out = x if out is None else out
    _lib.call("sb_relu", device_ptr(x), device_ptr(out), int(x.size), stream_ptr(stream))
    return out


def softmax(x, out=None, mask=None, prefix=-1, stream=None):
    """Row softmax; `mask` (uint8, same shape) or `prefix` (legal iff j < prefix) restricts it."""
    out = x if out is None else out
    rows, cols = _rows_cols(x)
    _lib.call("sb_row_softmax", device_ptr(x), device_ptr(out), rows, cols, device_ptr(mask), int(prefix),
              stream_ptr(stream))
    return out


def masked_softmax(size, x, out=None, stream=None):
    """layers.masked_softmax size (ml/layers.spi:408-414): legal iff column index < size."""
    return softmax(x, out=out, prefix=size, stream=stream)


def regret_matching(x, out=None, mask=None, prefix=-1, stream=None):
    out = x if out is None else out
    rows, cols = _rows_cols(x)
    _lib.call("sb_row_regret_matching", device_ptr(x), device_ptr(out), rows, cols, device_ptr(mask),
              int(prefix), stream_ptr(stream))
    return out


def masked_regret_matching(size, x, out=None, stream=None):
    """layers.masked_regret_matching size (ml/layers.spi:415-420)."""
    return regret_matching(x, out=out, prefix=size, stream=stream)


def argmax(x, out, stream=None):
    rows, cols = _rows_cols(x)
    _lib.call("sb_row_argmax", device_ptr(x), device_ptr(out), rows, cols, stream_ptr(stream))
    return out


def sample(probs, uniforms, out, stream=None):
    """One index per row drawn from the row's non-negative weights with the caller's uniform numbers
    in (0, 1] (one per row): the reference's discrete sampling head (ml/primitives.spi:782-800)."""
    rows, cols = _rows_cols(probs)
    _lib.call("sb_row_sample", device_ptr(probs), device_ptr(uniforms), device_ptr(out), rows, cols,
              stream_ptr(stream))
    return out


def sample_seeded(probs, out, seed, row_offset=0, position=0, stream=None):
    """The same with the uniform numbers drawn on the device as the reference does: row r uses output
    ``position`` of the Philox4x32-10 stream (seed, row_offset + r)."""
    import ctypes
    rows, cols = _rows_cols(probs)
    _lib.call("sb_row_sample_seeded", device_ptr(probs), device_ptr(out), rows, cols, ctypes.c_ulonglong(int(seed)),
              ctypes.c_ulonglong(int(row_offset)), ctypes.c_ulonglong(int(position)), stream_ptr(stream))
    return out


def philox_uniform(out, seed, row_offset=0, position=0, stream=None):
    """Fills the fp32 device array ``out`` with the uniform numbers in (0, 1] a sampling head draws:
    element i = output ``position`` of the stream (seed, row_offset + i)."""
    import ctypes
    _lib.call("sb_philox_uniform", device_ptr(out), ctypes.c_longlong(int(out.size)), ctypes.c_ulonglong(int(seed)),
              ctypes.c_ulonglong(int(row_offset)), ctypes.c_ulonglong(int(position)), stream_ptr(stream))
    return out


def binarize(modulo, x, out, stream=None):
    """Row hash: bit j = (x[r, j] > 0), modulo ``modulo`` (ml/primitives.spi:816-821); ``out`` is an int32
    device array [rows] holding the unsigned values."""
    import ctypes
    rows, cols = _rows_cols(x)
    _lib.call("sb_row_binarize", device_ptr(x), device_ptr(out), rows, cols, ctypes.c_uint(int(modulo)),
              stream_ptr(stream))
    return out


def ln_l2(x, out=None, stream=None):
    out = x if out is None else out
    rows, cols = _rows_cols(x)
    _lib.call("sb_row_ln_l2", device_ptr(x), device_ptr(out), rows, cols, stream_ptr(stream))
    return out


def encode_states(fields, widths, dense, out, stream=None):
    """Compact game states -> the dense network input ``out`` [rows, sum(widths) + n_dense].

    ``fields``: uint8 device array [rows, len(widths)], value v < widths[j] sets feature v of the
    j-th one-hot group, any other value leaves the group zero (the bounded-int pickler of
    corebase/pickler.spi:20-37, run on the device as ml/models.spi:30-41 does); ``dense``: device
    array [rows, n_dense] in the dtype of ``out`` (or None), copied behind the one-hot groups.
    """
    import ctypes
    rows = int(out.shape[0])
    widths = [int(w) for w in widths]
    n_dense = 0 if dense is None else int(dense.shape[1])
    if int(out.shape[1]) != sum(widths) + n_dense:
        raise ValueError("encode_states: out has %d features, the layout describes %d"
                         % (out.shape[1], sum(widths) + n_dense))
    if tuple(fields.shape) != (rows, len(widths)):
        raise ValueError("encode_states: fields must be [%d, %d], got %s" % (rows, len(widths), tuple(fields.shape)))
    if dense is not None and (int(dense.shape[0]) != rows or dense.dtype != out.dtype):
        raise ValueError("encode_states: dense must be [%d, n] in the dtype of out" % rows)
    w_c = (ctypes.c_int * max(1, len(widths)))(*widths)
    _lib.call("sb_encode_states", device_ptr(fields), len(widths), w_c, device_ptr(dense), n_dense,
              device_ptr(out), rows, _lib.DTYPE_CODES[out.dtype], stream_ptr(stream))
    return out


def convert(x, out, stream=None):
    """fp32 device array -> `out` (bf16 / f16 / tf32-rounded fp32 / fp32)."""
    _lib.call("sb_convert", device_ptr(x), device_ptr(out), int(x.size), _lib.DTYPE_CODES[out.dtype],
              stream_ptr(stream))
    return out
