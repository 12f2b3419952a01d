"""Host-side conversions between fp32 and the storage types of the tensor-core input classes."""
import numpy as np


def f32_to_bf16_bits(x):
    """Round-to-nearest-even fp32 -> bf16, returned as uint16 bit patterns."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    out = np.where((u & np.uint32(0x7F800000)) == np.uint32(0x7F800000), u, rounded)
    return (out >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(bits):
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_bf16(x):
    """fp32 values rounded to the nearest bf16, kept as fp32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(np.shape(x))


def round_f16(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def round_tf32(x):
    """fp32 values rounded (nearest-even) to 10 explicit mantissa bits, kept as fp32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (u + np.uint32(0x0FFF) + ((u >> np.uint32(13)) & np.uint32(1))) & np.uint32(0xFFFFE000)
    out = np.where((u & np.uint32(0x7F800000)) == np.uint32(0x7F800000), u, rounded)
    return out.view(np.float32).reshape(np.shape(x))


def trunc_tf32(x):
    """fp32 values with the low 13 mantissa bits cleared (what the tensor core reads)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) & np.uint32(0xFFFFE000)
    return u.view(np.float32).reshape(np.shape(x))


ROUNDERS = {"f32": lambda x: np.asarray(x, np.float32), "tf32": round_tf32, "bf16": round_bf16,
            "f16": round_f16}
