"""The bounded device-side wait, made to run out on purpose (GPU).

A kernel waits on a barrier that nothing signals.  It must come back by itself after the library's
wait limit, report the wait site through the device status word, release the other waiter of the
CTA through the abort flag, and leave the context fully usable -- no trap, no hang.
"""
import ctypes

import numpy as np
import pytest

from oracle import spiral_oracle as so

pytestmark = pytest.mark.gpu


def test_expired_wait_reports_and_context_survives(gpu):
    from spiral_b200 import _lib
    assert gpu.device_status() == (0, 0)
    res = (ctypes.c_int * 5)()
    _lib.call("sb_selftest_bounded_wait", res)
    ok0, ok1, ms0, ms1, flag = list(res)
    assert (ok0, ok1, flag) == (0, 0, 1)                 # both waits gave up, the abort flag was raised
    assert 300 <= max(ms0, ms1) <= 2000                  # after the 0.4 s limit, not forever
    site, count = gpu.device_status(clear=True)
    assert site == 8 and count >= 1                      # SB_SITE_DRAIN recorded
    assert gpu.device_status() == (0, 0)                 # cleared
    # the context is still healthy: a GEMM right after gives the right answer
    g = so.rng(5)
    a = so.round_bf16(g.normal(size=(256, 128)).astype(np.float32))
    b = so.round_bf16(g.normal(size=(192, 128)).astype(np.float32))
    c = gpu.DeviceArray((256, 192), "f32")
    gpu.matmul(False, True, 1.0, gpu.DeviceArray.from_numpy(a, "bf16"), gpu.DeviceArray.from_numpy(b, "bf16"), 0.0, c)
    assert so.rel_frobenius(c.numpy(), so.matmul(False, True, 1.0, a, b, 0.0, None)) <= 2e-5
