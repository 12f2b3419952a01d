"""The C-ABI library loads without a GPU and exports every symbol the header declares (CPU only)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "spiral_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "sb_matmul_tf32" in names and "sb_matmul_ex" in names
    assert len(names) >= 25


def test_library_exports_every_declared_symbol(sb):
    lib = ctypes.CDLL(sb.LIB_PATH)
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, "declared in include/spiral_b200.h but not exported: %s" % missing


def test_binding_table_covers_header(sb):
    from spiral_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_plan_needs_no_device(sb):
    plan = sb.matmul_plan(False, True, 4096, 4096, 4096, "bf16")
    assert plan["block_m"] in (128, 256) and plan["block_n"] % 16 == 0 and plan["grid"] <= 148
    assert plan["block_k"] in (64, 128) and plan["stages"] >= 2      # one or two 128-byte sub-blocks per stage
    if plan["block_m"] == 256:          # CTA pairs: an even grid, each CTA stages half of the B columns
        assert plan["grid"] % 2 == 0 and plan["block_n"] % 32 == 0
    plan = sb.matmul_plan(False, False, 4000, 3000, 1000, "tf32")
    assert plan["block_k"] in (32, 64) and plan["block_n"] % 32 == 0
    small = sb.matmul_plan(False, True, 16384, 3, 256, "tf32")
    assert small["block_n"] == 16 and small["grid"] == 128 and small["block_m"] == 128


def test_bad_arguments_are_rejected_before_any_launch(sb):
    from spiral_b200 import _lib
    with pytest.raises(sb.SpiralError) as e:
        _lib.call("sb_matmul_tf32", 0, 1, ctypes.c_float(1), None, None, ctypes.c_float(0), None, 4, 4, 4, None)
    assert e.value.code == -1
    with pytest.raises(sb.SpiralError):
        _lib.call("sb_matmul_tf32", 0, 1, ctypes.c_float(1), 16, 16, ctypes.c_float(0), 16, -1, 4, 4, None)
    # zero-sized outputs are a no-op, not an error
    _lib.call("sb_matmul_tf32", 0, 1, ctypes.c_float(1), None, None, ctypes.c_float(0), None, 0, 4, 4, None)


def test_shape_inference_follows_the_reference(sb):
    class Fake:
        def __init__(self, shape):
            self.shape, self.dtype = shape, "float32"
    from spiral_b200.matmul import _dims
    assert _dims(False, True, Fake((8, 5)), Fake((3, 5)), Fake((8, 3))) == (8, 3, 5)
    assert _dims(True, False, Fake((5, 8)), Fake((5, 3)), Fake((8, 3))) == (8, 3, 5)
    with pytest.raises(ValueError):
        _dims(False, False, Fake((8, 5)), Fake((3, 5)), Fake((8, 3)))
