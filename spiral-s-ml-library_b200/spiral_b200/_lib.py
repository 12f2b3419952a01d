"""ctypes binding of libspiral_b200.so: the only way the Python host reaches the GPU.

There is no CPU fallback: if the shared library is missing, or a call fails,
an exception is raised.
"""
import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_size_t, c_void_p, POINTER

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libspiral_b200.so")

SB_OK = 0
STATUS_NAMES = {
    0: "SB_OK", -1: "SB_ERR_BAD_ARG", -2: "SB_ERR_MISALIGNED", -3: "SB_ERR_UNSUPPORTED",
    -4: "SB_ERR_CUDA", -5: "SB_ERR_DEVICE_TIMEOUT", -6: "SB_ERR_TOO_LARGE", -7: "SB_ERR_NO_DEVICE",
}

# sb_dtype
F32, TF32, BF16, F16, I32, U8 = 0, 1, 2, 3, 4, 5
DTYPE_CODES = {"f32": F32, "tf32": TF32, "bf16": BF16, "f16": F16, "i32": I32, "u8": U8}

# epilogue flags
EPI_NONE, EPI_BIAS, EPI_RELU, EPI_RELU_GRAD = 0, 1, 2, 4
EPI_MASKED_SOFTMAX, EPI_REGRET_MATCHING, EPI_ARGMAX = 8, 16, 32
EPI_RELU_MASK_OUT, EPI_RELU_GRAD_MASK, EPI_COLSUM_OUT = 64, 128, 256
EPI_SAMPLE, EPI_BINARIZE, EPI_LN_L2 = 512, 1024, 2048


class HeadSpec(ctypes.Structure):
    """sb_head_spec of include/spiral_b200.h."""
    _fields_ = [("flags", c_int), ("prefix", c_int), ("mask", c_void_p), ("argmax_out", c_void_p),
                ("sample_out", c_void_p), ("hash_out", c_void_p), ("modulo", ctypes.c_uint32),
                ("seed", ctypes.c_ulonglong), ("row_offset", ctypes.c_ulonglong), ("position", ctypes.c_ulonglong)]


class SpiralError(RuntimeError):
    """A libspiral_b200 call returned a negative status."""

    def __init__(self, code, text):
        self.code = code
        super().__init__("%s (%d): %s" % (STATUS_NAMES.get(code, "?"), code, text))


_P = c_void_p
_I = c_int
_F = c_float
_Z = c_size_t
_PP = POINTER(c_void_p)
_IP = POINTER(c_int)

class DecideArgs(ctypes.Structure):
    """sb_decide_args of include/spiral_b200.h."""
    _fields_ = [("n_layers", c_int), ("sizes", POINTER(c_int)), ("members", c_int), ("in_dtype", c_int),
                ("w_compute", c_void_p), ("params", c_void_p), ("hidden_norm", c_int), ("rows", ctypes.c_longlong),
                ("fields", c_void_p), ("n_fields", c_int), ("widths", POINTER(c_int)), ("dense", c_void_p),
                ("n_dense", c_int), ("x", c_void_p), ("head_flags", c_int), ("prefix", c_int), ("mask", c_void_p),
                ("seed", ctypes.c_ulonglong), ("row_offset", ctypes.c_ulonglong), ("output_probs", c_void_p),
                ("output_indices", c_void_p), ("ensemble_id", c_void_p), ("action", c_void_p),
                ("sampling_prob_selected", c_void_p), ("sampling_prob_ensemble", c_void_p),
                ("tile_counters", c_void_p)]


# name -> (restype, argtypes); every symbol include/spiral_b200.h declares.
SIGNATURES = {
    "sb_last_error_string": (c_char_p, []),
    "sb_version": (_I, []),
    "sb_device_count": (_I, [_IP]),
    "sb_set_device": (_I, [_I]),
    "sb_device_sm_count": (_I, [_IP]),
    "sb_malloc": (_I, [_PP, _Z]),
    "sb_free": (_I, [_P]),
    "sb_malloc_host": (_I, [_PP, _Z]),
    "sb_free_host": (_I, [_P]),
    "sb_memcpy_h2d": (_I, [_P, _P, _Z, _P]),
    "sb_memcpy_d2h": (_I, [_P, _P, _Z, _P]),
    "sb_memcpy_d2d": (_I, [_P, _P, _Z, _P]),
    "sb_memset": (_I, [_P, _I, _Z, _P]),
    "sb_stream_create": (_I, [_PP]),
    "sb_stream_destroy": (_I, [_P]),
    "sb_stream_sync": (_I, [_P]),
    "sb_device_sync": (_I, []),
    "sb_event_create": (_I, [_PP]),
    "sb_event_destroy": (_I, [_P]),
    "sb_event_record": (_I, [_P, _P]),
    "sb_stream_wait_event": (_I, [_P, _P]),
    "sb_event_elapsed_ms": (_I, [_P, _P, POINTER(c_float)]),
    "sb_device_status": (_I, [_IP, _I]),
    "sb_check_device": (_I, [_P]),
    "sb_mem_info": (_I, [POINTER(c_size_t), POINTER(c_size_t)]),
    "sb_selftest_bounded_wait": (_I, [_IP]),
    "sb_launch_count": (ctypes.c_ulonglong, []),
    "sb_gemm_profile_begin": (_I, []),
    "sb_gemm_profile_end": (_I, [_IP, POINTER(ctypes.c_double), POINTER(ctypes.c_double)]),
    "sb_gemm_profile_entry": (_I, [_I, POINTER(ctypes.c_double), POINTER(ctypes.c_double)]),
    "sb_matmul_tf32": (_I, [_I, _I, _F, _P, _P, _F, _P, _I, _I, _I, _P]),
    "sb_matmul_ex": (_I, [_I, _I, _F, _P, _P, _F, _P, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    "sb_matmul_f32_workspace_bytes": (_I, [_I, _I, _I, POINTER(c_size_t)]),
    "sb_matmul_f32x3": (_I, [_I, _I, _F, _P, _P, _F, _P, _I, _I, _I, _I, _P, _P, _Z, _P]),
    "sb_matmul_head": (_I, [_I, _I, _F, _P, _P, _F, _P, _I, _I, _I, _I, _I, _P, POINTER(HeadSpec), _P]),
    "sb_gemm_reserve_smem": (_I, [_I]),
    "sb_matmul_plan": (_I, [_I, _I, _I, _I, _I, _I, _I, _IP]),
    "sb_relu": (_I, [_P, _P, _Z, _P]),
    "sb_row_softmax": (_I, [_P, _P, _I, _I, _P, _I, _P]),
    "sb_row_regret_matching": (_I, [_P, _P, _I, _I, _P, _I, _P]),
    "sb_row_argmax": (_I, [_P, _P, _I, _I, _P]),
    "sb_row_sample": (_I, [_P, _P, _P, _I, _I, _P]),
    "sb_row_sample_seeded": (_I, [_P, _P, _I, _I, ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_ulonglong, _P]),
    "sb_philox_uniform": (_I, [_P, ctypes.c_longlong, ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_ulonglong, _P]),
    "sb_row_binarize": (_I, [_P, _P, _I, _I, ctypes.c_uint, _P]),
    "sb_row_ln_l2": (_I, [_P, _P, _I, _I, _P]),
    "sb_convert": (_I, [_P, _P, _Z, _I, _P]),
    "sb_ipc_export": (_I, [_P, _P]),
    "sb_ipc_open": (_I, [_P, _PP]),
    "sb_ipc_close": (_I, [_P]),
    "sb_dp_flag_bytes": (_I, []),
    "sb_dp_slice": (_I, [ctypes.c_longlong, ctypes.c_longlong, _I, _I, POINTER(ctypes.c_longlong)]),
    "sb_dp_sgd_update": (_I, [_I, _I, _PP, _PP, _PP, _PP, ctypes.c_uint, ctypes.c_longlong, ctypes.c_longlong,
                              ctypes.c_float, _I, _I, POINTER(ctypes.c_longlong), _I, _I, _I, _I, _P]),
    "sb_dp_sgd_update_segments": (_I, [_I, _I, _PP, _PP, _PP, _PP, ctypes.c_uint, _I, POINTER(ctypes.c_longlong), _IP,
                                       ctypes.c_float, _I, _I, POINTER(ctypes.c_longlong), _I, _I, _I, _I, _P]),
    "sb_dp_status": (_I, [_P, _IP]),
    "sb_mlp_dp_fused_layers": (_I, [_I, _IP, _I, _IP]),
    "sb_mlp_backward_dp": (_I, [_I, _IP, _I, _F, _I, _P, _P, _PP, _PP, _P, _P, _P, _PP, _I, _I, _I, _P, _Z, _P, _P]),
    "sb_encode_states": (_I, [_P, _I, _IP, _P, _I, _P, ctypes.c_longlong, _I, _P]),
    "sb_mlp_param_offsets": (_I, [_I, _IP, POINTER(ctypes.c_longlong)]),
    "sb_mlp_forward": (_I, [_I, _IP, _I, _I, _P, _P, _P, _PP, _PP, _I, _P, _P, _P, _P]),
    "sb_mlp_forward_fused": (_I, [_I, _IP, _I, _I, _P, _P, _P, _I, _P, _P, _P, _P]),
    "sb_mlp_forward_fused_ensemble": (_I, [_I, _IP, _I, _I, _I, _P, _P, _P, _I, _P, _P, _P, _P]),
    "sb_mlp_fused_supported": (_I, [_I, _IP, _I]),
    "sb_mlp_forward_fused_train": (_I, [_I, _IP, _I, _I, _P, _P, _P, _PP, _PP, _I, _P, _P, _P, _P]),
    "sb_mlp_forward_fused_head": (_I, [_I, _IP, _I, _I, _I, _P, _P, _P, _I, POINTER(HeadSpec), _P, _P]),
    "sb_policy_decide": (_I, [POINTER(DecideArgs), _P]),
    "sb_mlp_forward_static": (_I, [_I, _IP, _I, _I, _P, _P, _P, _I, _P, _P, _P, _P]),
    "sb_mlp_backward_scratch_bytes": (_I, [_I, _IP, _I, _I, POINTER(c_size_t)]),
    "sb_mlp_backward": (_I, [_I, _IP, _I, _F, _I, _P, _P, _PP, _PP, _P, _P, _P, _P, _I, _P, _Z, _P, _P]),
    "sb_mlp_backward_dy_offset": (_I, [_I, _IP, _I, _I, _I, POINTER(c_size_t)]),
    "sb_mlp_backward_range": (_I, [_I, _IP, _I, _F, _I, _P, _P, _PP, _PP, _P, _P, _P, _P, _I, _P, _Z, _P, _I, _I, _P]),
    "sb_sgd_update": (_I, [_P, _P, _P, ctypes.c_longlong, _F, _I, _P]),
    "sb_mlp_train_step": (_I, [_I, _IP, _I, _I, _P, _P, _P, _PP, _PP, _P, _P, _P, _P, _I, _F, _P, _Z, _P, _P]),
}

_lib = None


def load():
    """Loads the shared library once and attaches the signatures."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libspiral_b200.so is not built (%s); run spiral-s-ml-library_b200/build.py -- "
            "there is no CPU fallback" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc):
    if rc != SB_OK:
        text = load().sb_last_error_string()
        raise SpiralError(rc, text.decode("utf-8", "replace") if text else "")
    return rc


def call(name, *args):
    """Calls an int-returning entry point and raises SpiralError on failure."""
    return check(getattr(load(), name)(*args))
