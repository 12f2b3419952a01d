"""spiral_b200: B200 (sm_100a) dense-matmul / policy-MLP path behind the reference's call surface.

A thin ctypes host over libspiral_b200.so (hand-written CUDA: tcgen05 MMAs with
TMEM accumulators fed by TMA).  No CPU fallback exists: without the built
library every operation raises.
"""
from ._lib import SpiralError, LIB_PATH  # noqa: F401
from .device import (DeviceArray, Event, Stream, wait_event, GemmProfile, launch_count, device_count, device_ptr, device_status, check_device, mem_info, set_device, sm_count,  # noqa: F401
                     synchronize)
from .matmul import head_spec, matmul, matmul_head, matmul_plan, matmul_tf32  # noqa: F401
from . import primitives  # noqa: F401
from .models import EnsemblePolicyMLP, PolicyMLP, param_offsets, to_storage  # noqa: F401
from . import layers  # noqa: F401
from .parallel import DataParallel, PeerUpdate, shard_rows, bucket_ranges, update_slice  # noqa: F401
