"""Device memory for hosts that bring no allocator of their own.

The reference passes CuPy arrays to its kernels (corecuda/base.spi:100-108).
This package accepts anything that can name a device address -- a
``DeviceArray``, a CuPy array (``.data.ptr``), a torch tensor
(``.data_ptr()``), an object with ``__cuda_array_interface__`` or a plain
integer -- and passes the raw pointer through the C ABI.
"""
import ctypes

import numpy as np

from . import _lib
from . import dtypes

_ITEMSIZE = {"f32": 4, "tf32": 4, "bf16": 2, "f16": 2, "i32": 4, "u8": 1}
_NP_STORAGE = {"f32": np.float32, "tf32": np.float32, "bf16": np.uint16, "f16": np.float16,
               "i32": np.int32, "u8": np.uint8}


def device_count():
    n = ctypes.c_int(0)
    rc = _lib.load().sb_device_count(ctypes.byref(n))
    return n.value if rc == 0 else 0


def set_device(index):
    _lib.call("sb_set_device", int(index))


def sm_count():
    """Streaming multiprocessors of the current device (the tile planner's worker count)."""
    n = ctypes.c_int(0)
    _lib.call("sb_device_sm_count", ctypes.byref(n))
    return n.value


def synchronize():
    """Waits for all device work (corecuda/base.spi:45 device_sync)."""
    _lib.call("sb_device_sync")


def mem_info():
    """(free, total) bytes of device memory on the current device."""
    free, total = ctypes.c_size_t(0), ctypes.c_size_t(0)
    _lib.call("sb_mem_info", ctypes.byref(free), ctypes.byref(total))
    return free.value, total.value


def check_device(stream=None):
    """Synchronises ``stream`` and raises SpiralError (SB_ERR_DEVICE_TIMEOUT) if a bounded device-side
    wait expired since the status word was last cleared."""
    _lib.call("sb_check_device", stream_ptr(stream))


def device_status(clear=True):
    """(first expired wait site, number of expired waits); (0, 0) when healthy."""
    st = (ctypes.c_int * 2)()
    _lib.call("sb_device_status", st, 1 if clear else 0)
    return st[0], st[1]


class DeviceArray:
    """A contiguous row-major device buffer with a shape and a storage dtype tag."""

    def __init__(self, shape, dtype="f32", ptr=None, owner=None):
        if dtype not in _ITEMSIZE:
            raise ValueError("unknown dtype %r" % (dtype,))
        self.shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        self.dtype = dtype
        self.size = int(np.prod(self.shape)) if self.shape else 1
        self.nbytes = self.size * _ITEMSIZE[dtype]
        self._owner = owner
        self._owned = ptr is None
        if ptr is None:
            p = ctypes.c_void_p()
            _lib.call("sb_malloc", ctypes.byref(p), self.nbytes)
            ptr = p.value
        self.ptr = int(ptr)

    # -- construction ------------------------------------------------------
    @classmethod
    def from_numpy(cls, array, dtype=None, stream=None):
        """Uploads a host array; fp32 data is rounded to `dtype` on the host first."""
        array = np.asarray(array)
        if dtype is None:
            dtype = {np.dtype(np.float32): "f32", np.dtype(np.float16): "f16", np.dtype(np.int32): "i32",
                     np.dtype(np.uint8): "u8", np.dtype(np.bool_): "u8",
                     np.dtype(np.float64): "f32"}.get(array.dtype)
            if dtype is None:
                raise TypeError("cannot infer a device dtype for %s" % array.dtype)
        out = cls(array.shape, dtype)
        out.upload(array, stream)
        return out

    @classmethod
    def zeros(cls, shape, dtype="f32"):
        out = cls(shape, dtype)
        out.fill_zero()
        return out

    def _host_storage(self, array):
        if self.dtype == "bf16":
            return np.ascontiguousarray(dtypes.f32_to_bf16_bits(np.asarray(array, np.float32)))
        if self.dtype == "tf32":
            return np.ascontiguousarray(dtypes.round_tf32(np.asarray(array, np.float32)))
        return np.ascontiguousarray(np.asarray(array).astype(_NP_STORAGE[self.dtype], copy=False))

    def upload(self, array, stream=None):
        host = self._host_storage(array)
        if host.size != self.size:
            raise ValueError("upload of %d elements into a buffer of %d" % (host.size, self.size))
        _lib.call("sb_memcpy_h2d", self.ptr, host.ctypes.data, host.nbytes, stream_ptr(stream))
        _lib.call("sb_stream_sync", stream_ptr(stream))
        return self

    def fill_zero(self, stream=None):
        _lib.call("sb_memset", self.ptr, 0, self.nbytes, stream_ptr(stream))
        return self

    # -- readback ----------------------------------------------------------
    def numpy(self, stream=None):
        """Downloads; 16-bit float storage comes back widened to fp32."""
        host = np.empty(self.shape, dtype=_NP_STORAGE[self.dtype])
        _lib.call("sb_memcpy_d2h", host.ctypes.data, self.ptr, host.nbytes, stream_ptr(stream))
        # Synchronises, and raises SpiralError(SB_ERR_DEVICE_TIMEOUT) when a kernel gave up a bounded
        # wait: what was just read may then be incomplete.
        _lib.call("sb_check_device", stream_ptr(stream))
        if self.dtype == "bf16":
            return dtypes.bf16_bits_to_f32(host).reshape(self.shape)
        if self.dtype == "f16":
            return host.astype(np.float32)
        return host

    def view(self, shape, dtype=None, offset_bytes=0):
        """A non-owning typed view into this buffer (arena-style layouts)."""
        v = DeviceArray(shape, dtype or self.dtype, ptr=self.ptr + int(offset_bytes), owner=self)
        if offset_bytes + v.nbytes > self.nbytes:
            raise ValueError("view exceeds the underlying buffer")
        return v

    def free(self):
        if self._owned and self.ptr:
            _lib.call("sb_free", self.ptr)
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def __repr__(self):
        return "DeviceArray(shape=%s, dtype=%s, ptr=0x%x)" % (self.shape, self.dtype, self.ptr)


def device_ptr(obj):
    """Raw device address of `obj` (None -> NULL)."""
    if obj is None:
        return None
    if isinstance(obj, DeviceArray):
        return obj.ptr
    if isinstance(obj, int):
        return obj
    if hasattr(obj, "data_ptr"):
        return int(obj.data_ptr())
    cai = getattr(obj, "__cuda_array_interface__", None)
    if cai is not None:
        return int(cai["data"][0])
    data = getattr(obj, "data", None)
    if data is not None and hasattr(data, "ptr"):
        return int(data.ptr)
    raise TypeError("cannot take a device pointer from %r" % type(obj))


def dtype_tag(obj):
    """Storage dtype tag of a device array-like ('f32', 'bf16', 'f16', ...)."""
    if isinstance(obj, DeviceArray):
        return obj.dtype
    name = str(getattr(obj, "dtype", "")).replace("torch.", "")
    return {"float32": "f32", "bfloat16": "bf16", "float16": "f16", "int32": "i32", "uint8": "u8",
            "bool": "u8"}.get(name, None)


def stream_ptr(stream):
    """Accepts None, an int handle, a torch/cupy stream object."""
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream
    for attr in ("cuda_stream", "ptr"):
        if hasattr(stream, attr):
            return int(getattr(stream, attr))
    raise TypeError("cannot take a stream handle from %r" % type(stream))


class Stream:
    """A non-blocking CUDA stream (does not synchronise with the legacy default stream)."""

    def __init__(self):
        p = ctypes.c_void_p()
        _lib.call("sb_stream_create", ctypes.byref(p))
        self.ptr = p.value

    def wait_event(self, event):
        _lib.call("sb_stream_wait_event", self.ptr, event.ptr)

    def synchronize(self):
        _lib.call("sb_stream_sync", self.ptr)

    def __del__(self):
        try:
            if self.ptr:
                _lib.load().sb_stream_destroy(self.ptr)
                self.ptr = None
        except Exception:
            pass


def wait_event(stream, event):
    """Work submitted to `stream` (None = default stream) after this call waits for `event`."""
    _lib.call("sb_stream_wait_event", stream_ptr(stream), event.ptr)


class Event:
    """CUDA event for device-side timing on the launching stream."""

    def __init__(self):
        p = ctypes.c_void_p()
        _lib.call("sb_event_create", ctypes.byref(p))
        self.ptr = p.value

    def record(self, stream=None):
        _lib.call("sb_event_record", self.ptr, stream_ptr(stream))
        return self

    def elapsed_ms(self, stop):
        ms = ctypes.c_float(0)
        _lib.call("sb_event_elapsed_ms", self.ptr, stop.ptr, ctypes.byref(ms))
        return ms.value

    def __del__(self):
        try:
            if self.ptr:
                _lib.load().sb_event_destroy(self.ptr)
                self.ptr = None
        except Exception:
            pass


def launch_count():
    """Kernels launched by the library in this process so far."""
    return int(_lib.load().sb_launch_count())


class GemmProfile:
    """Context manager: CUDA-event timing of every tensor-core GEMM launch inside the block."""

    def __enter__(self):
        _lib.call("sb_gemm_profile_begin")
        self.launches, self.ms, self.flops = 0, 0.0, 0.0
        return self

    def __exit__(self, *exc):
        n = ctypes.c_int(0)
        ms = ctypes.c_double(0)
        fl = ctypes.c_double(0)
        _lib.call("sb_gemm_profile_end", ctypes.byref(n), ctypes.byref(ms), ctypes.byref(fl))
        self.launches, self.ms, self.flops = n.value, ms.value, fl.value
        self.entries = []
        for i in range(n.value):
            _lib.call("sb_gemm_profile_entry", i, ctypes.byref(ms), ctypes.byref(fl))
            self.entries.append((ms.value, fl.value))
        return False
