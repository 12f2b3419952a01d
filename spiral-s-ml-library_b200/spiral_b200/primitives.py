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


def ln_l2(x, out=None, stream=None):
    out = x if out is None else out
    rows, cols = _rows_cols(x)
    _lib.call("sb_row_ln_l2", device_ptr(x), device_ptr(out), rows, cols, stream_ptr(stream))
    return out


def convert(x, out, stream=None):
    """fp32 device array -> `out` (bf16 / f16 / tf32-rounded fp32 / fp32)."""
    _lib.call("sb_convert", device_ptr(x), device_ptr(out), int(x.size), _lib.DTYPE_CODES[out.dtype],
              stream_ptr(stream))
    return out
